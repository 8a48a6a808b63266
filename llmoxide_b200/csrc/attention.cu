// Attention over the paged cache, general form: any number of heads and
// groups, any head size that is a multiple of 16 up to 256, a window or none,
// whole prompts and single tokens alike.  It is the float32 path's kernel and
// the bfloat16 path's fallback for the sizes the tiled kernels refuse.
//
// For the query at position p of head hq (crates/model/src/qwen35/cpu.rs:325-355):
// kv head g = hq / (H/G); keys first..p are visible, first = 0 or p-(w-1) under
// a window (crates/model/src/cache.rs:31-37); s_j = (q . k_j) * scale; softmax
// with the maximum subtracted; out = sum_j w_j v_j.  All of it in float32.
// With `keep_first` > 0 the keys 0..keep_first-1 stay visible under the window
// as well (they are taken first, then the window's keys).  Values may have a
// size Dv of their own; a query row may sit in a wider row (q_stride elements
// from token to token), e.g. the q|k|v row of a fused product.  With `sink` > 0
// the softmax's denominator has that much added: w_j = exp(s_j) / (sink + sum exp(s_j)).
// With `chunk` > 0 positions are cut into chunks of that many, counted from the sequence's position 0, and a
// query sees only the keys of its own chunk: first = p - p % chunk (beside a window, the later of the two).
//
// With `pool` > 0 every block of `pool` positions that lies wholly before the window (block b = positions
// b*pool .. b*pool+pool-1, seen from p when b*pool+pool-1 <= p - window) is seen as one key and one value: row b of
// a second store (pool_k, pool_v, with a block table of its own), taken first, in the same softmax.
// With `gate` a head's output is multiplied by sigmoid(gate[t * gate_stride + hq]).
//
// One warp per (token, head).  Keys are taken 32 at a time starting at the
// range's first key: lane j scores key lo + c*32 + j with a sequential dot over
// D, the chunk's maximum and sum update a running softmax, and the lanes then
// own dims (lane, lane+32, ...) of the output and add the chunk's values key
// by key.  Chunk boundaries depend on (keep_first, first, p) only, so a
// position's result does not depend on how tokens were cut into steps or batched.
#include "common.cuh"

#define ATT_WARPS 4
#define ATT_MAX_D 256

template <typename TA, typename TC>
__global__ void attention_paged_kernel(const TA* __restrict__ q, TA* __restrict__ out,
                                       const TC* __restrict__ k_cache_w, const TC* __restrict__ v_cache_w,
                                       const int* __restrict__ block_table, int table_width,
                                       const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                       int H, int G, int D, int Dv, size_t q_stride, int window, int keep_first,
                                       float scale, float sink, int chunk, int pool,
                                       const TC* __restrict__ pool_k, const TC* __restrict__ pool_v,
                                       const int* __restrict__ pool_table, const float* __restrict__ gate,
                                       size_t gate_stride) {
  extern __shared__ float q_buf[];  // [ATT_WARPS][D]
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;                        // tokens on x: a step may bring more than 65535
  const int hq = blockIdx.y * ATT_WARPS + warp;
  if (hq >= H) return;
  const int g = hq / (H / G);
  const int p = token_pos[t];
  int first = (window > 0 && p - (window - 1) > 0) ? p - (window - 1) : 0;
  if (chunk > 0) first = max(first, p - p % chunk);
  const int* pages = block_table + (size_t)token_seq[t] * table_width;     // (re-pointed per range below)

  float* qs = q_buf + warp * D;
  const TA* qrow = q + (size_t)t * q_stride + (size_t)hq * D;
  for (int i = lane; i < D; i += 32) qs[i] = to_f32(qrow[i]);
  __syncwarp();

  constexpr int MAX_OWN = ATT_MAX_D / 32;
  float acc[MAX_OWN];
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) acc[i] = 0.f;
  float m = -INFINITY, l = 0.f;

  // two ranges of keys: the kept first ones that lie before the window (or the pooled blocks that do, out of their
  // own store), then the window up to p
  int n_kept = keep_first < first ? keep_first : first;
  if (pool > 0) n_kept = p - window + 1 >= pool ? (p - window + 1) / pool : 0;
  const int* pages_w = pages;
  const int* pages_0 = pool > 0 ? pool_table + (size_t)token_seq[t] * table_width : pages;
  const TC* kc0 = pool > 0 ? pool_k : k_cache_w;
  const TC* vc0 = pool > 0 ? pool_v : v_cache_w;
  for (int range = n_kept > 0 ? 0 : 1; range < 2; ++range) {
  const int lo = range ? first : 0, last = range ? p : n_kept - 1;
  const TC* k_cache = range ? k_cache_w : kc0;
  const TC* v_cache = range ? v_cache_w : vc0;
  pages = range ? pages_w : pages_0;
  for (int base = lo; base <= last; base += 32) {
    const int j = base + lane;
    const bool live = j <= last;
    float s = -INFINITY;
    if (live) {
      const TC* krow = k_cache + cache_row_offset(pages[j / LLMX_PAGE], g, j % LLMX_PAGE, G, D);
      float dot = 0.f;
      for (int i = 0; i < D; ++i) dot += qs[i] * to_f32(krow[i]);
      s = dot * scale;
    }
    const float m_new = fmaxf(m, warp_max(s));
    const float corr = expf(m - m_new);  // exp(-inf) = 0 on the first chunk; lane 0 of a chunk is always live
    const float e = live ? expf(s - m_new) : 0.f;
    l = l * corr + warp_sum(e);
#pragma unroll
    for (int i = 0; i < MAX_OWN; ++i) acc[i] *= corr;
    const int n_live = (last - base + 1) < 32 ? (last - base + 1) : 32;
    for (int jj = 0; jj < n_live; ++jj) {
      const float w = __shfl_sync(0xffffffffu, e, jj);
      const int key = base + jj;
      const TC* vrow = v_cache + cache_row_offset(pages[key / LLMX_PAGE], g, key % LLMX_PAGE, G, Dv);
#pragma unroll
      for (int i = 0; i < MAX_OWN; ++i) {
        const int dim = lane + 32 * i;
        if (dim < Dv) acc[i] += w * to_f32(vrow[dim]);
      }
    }
    m = m_new;
  }
  }
  // a sink: `sink` keys of score 0 that have no value; they only add to the denominator
  float inv = 1.0f / (sink > 0.f ? l + sink * expf(-m) : l);
  if (gate) inv *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_stride + hq]));
  TA* orow = out + ((size_t)t * H + hq) * Dv;
#pragma unroll
  for (int i = 0; i < MAX_OWN; ++i) {
    const int dim = lane + 32 * i;
    if (dim < Dv) orow[dim] = from_f32<TA>(acc[i] * inv);
  }
}

// pool > 0: pool_k / pool_v hold one row per block of `pool` positions, paged like the cache, with the block table
// pool_table (as wide as block_table); needs a window and no kept first keys.  gate: null, or float32 with
// gate[t * gate_stride + head] the logit of head's output gate.
LLMX_API int llmx_attention_paged_pooled(const void* q, void* out, int act_dtype, const void* k_cache,
                                  const void* v_cache, int cache_dtype, const int* block_table, int table_width,
                                  const int* token_seq, const int* token_pos, int n_tokens, int H, int G, int D,
                                  int Dv, long long q_stride, int window, int keep_first, float scale, float sink,
                                  int chunk, int pool, const void* pool_k, const void* pool_v, const int* pool_table,
                                  const float* gate, long long gate_stride, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (chunk < 0 || (chunk > 0 && keep_first > 0)) return LLMX_REFUSED(1);
  if (pool < 0 || (pool > 0 && (window <= 0 || keep_first > 0 || chunk > 0 || !pool_k || !pool_v || !pool_table)))
    return LLMX_REFUSED(1);
  if (gate && gate_stride < H) return LLMX_REFUSED(1);
  if (H <= 0 || G <= 0 || H % G != 0 || D <= 0 || D > ATT_MAX_D || window < 0) return LLMX_REFUSED(1);
  if (Dv <= 0 || Dv > ATT_MAX_D || keep_first < 0 || q_stride < (long long)H * D) return LLMX_REFUSED(1);
  dim3 grid(n_tokens, (H + ATT_WARPS - 1) / ATT_WARPS);
  const size_t smem = (size_t)ATT_WARPS * D * sizeof(float);
#define CASE(TA, TC)                                                                                      \
  launch_pdl(attention_paged_kernel<TA, TC>, grid, dim3(ATT_WARPS * 32), smem, stream,                    \
      (const TA*)q, (TA*)out, (const TC*)k_cache, (const TC*)v_cache, block_table, table_width, token_seq, \
      token_pos, H, G, D, Dv, (size_t)q_stride, window, keep_first, scale, sink, chunk, pool, (const TC*)pool_k,  \
      (const TC*)pool_v, pool_table, gate, (size_t)gate_stride)
  if (act_dtype == LLMX_F32 && cache_dtype == LLMX_F32) CASE(float, float);
  else if (act_dtype == LLMX_BF16 && cache_dtype == LLMX_BF16) CASE(bf16, bf16);
  else if (act_dtype == LLMX_F32 && cache_dtype == LLMX_BF16) CASE(float, bf16);
  else if (act_dtype == LLMX_BF16 && cache_dtype == LLMX_F32) CASE(bf16, float);
  else return LLMX_REFUSED(2);
#undef CASE
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_attention_paged_chunked(const void* q, void* out, int act_dtype, const void* k_cache,
                                  const void* v_cache, int cache_dtype, const int* block_table, int table_width,
                                  const int* token_seq, const int* token_pos, int n_tokens, int H, int G, int D,
                                  int Dv, long long q_stride, int window, int keep_first, float scale, float sink,
                                  int chunk, cudaStream_t stream) {
  return llmx_attention_paged_pooled(q, out, act_dtype, k_cache, v_cache, cache_dtype, block_table, table_width,
                                     token_seq, token_pos, n_tokens, H, G, D, Dv, q_stride, window, keep_first, scale,
                                     sink, chunk, 0, nullptr, nullptr, nullptr, nullptr, 0, stream);
}

LLMX_API int llmx_attention_paged(const void* q, void* out, int act_dtype, const void* k_cache,
                                  const void* v_cache, int cache_dtype, const int* block_table, int table_width,
                                  const int* token_seq, const int* token_pos, int n_tokens, int H, int G, int D,
                                  int Dv, long long q_stride, int window, int keep_first, float scale, float sink,
                                  cudaStream_t stream) {
  return llmx_attention_paged_chunked(q, out, act_dtype, k_cache, v_cache, cache_dtype, block_table, table_width,
                                      token_seq, token_pos, n_tokens, H, G, D, Dv, q_stride, window, keep_first, scale,
                                      sink, 0, stream);
}

// ---------------------------------------------------------------------------
// The store of one row per block of `pool` positions: when a step writes the last position of block b
// (position b*pool + pool - 1), that block's key is the mean of its `pool` keys as the cache holds them, its value
// the mean of the values, summed in float32 in an order that `pool` alone decides, times 1 / pool, and stored as
// row b of the second store.
// The cache must still hold the block's positions: its window is at least `pool`.
// ---------------------------------------------------------------------------
// A lane owns V consecutive dims (16 bytes of the cache where the sizes allow it) and walks positions in order
// with several loads in flight.
template <int V>
__device__ __forceinline__ void pb_load(const float* p, float* o) {
  if (V == 1) {
    o[0] = p[0];
  } else {
    const float4 x = *reinterpret_cast<const float4*>(p);
    o[0] = x.x, o[1] = x.y, o[2] = x.z, o[3] = x.w;
  }
}
template <int V>
__device__ __forceinline__ void pb_load(const bf16* p, float* o) {
  if (V == 1) {
    o[0] = to_f32(p[0]);
  } else {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      const float2 f = __bfloat1622float2(h2[e]);
      o[2 * e] = f.x, o[2 * e + 1] = f.y;
    }
  }
}

#define PB_WARPS 8

// One CTA per (block that ends in the step, kv head, keys or values).  A block's positions are cut into PB_WARPS runs of equal length; warp w
// sums its run in position order (a lane owns V consecutive dims), and the runs' sums are added in the order of the
// runs: an order that depends on `pool` alone.
template <typename TC, int V>
__global__ void pool_blocks_kernel(const TC* __restrict__ k_cache, const TC* __restrict__ v_cache,
                                   const int* __restrict__ block_table, TC* __restrict__ pool_k,
                                   TC* __restrict__ pool_v, const int* __restrict__ pool_table, int table_width,
                                   const int* __restrict__ seq_start, const int* __restrict__ seq_past, int n_seqs,
                                   int G, int D, int Dv, int pool, int n_pages, int n_pool_pages) {
  extern __shared__ float pb_part[];                    // [PB_WARPS][width]
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int unit = blockIdx.y;                          // unit: kv head g's keys (2g) or values (2g+1)
  // The grid's x axis counts the blocks that end in this step, sequence after sequence: sequence s, which held
  // `past` positions and brings n, ends the blocks past / pool .. (past + n) / pool - 1.  CTAs beyond the step's
  // count leave at once (the grid is sized from the step's shape alone: tokens / pool + sequences).
  int left = blockIdx.x, seq = -1, p = 0;
  for (int s2 = 0; s2 < n_seqs; ++s2) {
    const int past = seq_past[s2], n = seq_start[s2 + 1] - seq_start[s2];
    const int first = past / pool, count = (past + n) / pool - first;
    if (left < count) {
      seq = s2;
      p = (first + left) * pool + pool - 1;               // the block's last position
      break;
    }
    left -= count;
  }
  if (seq < 0) return;                                    // uniform over the CTA
  const int g = unit >> 1, is_v = unit & 1;
  const int b = p / pool;
  const int* pages = block_table + (size_t)seq * table_width;
  const int dst_page = pool_table[(size_t)seq * table_width + b / LLMX_PAGE];
  if (dst_page < 0 || dst_page >= n_pool_pages) {
    if (threadIdx.x == 0) llmx_report(1);
    return;
  }
  const int width = is_v ? Dv : D;
  const TC* src = is_v ? v_cache : k_cache;
  TC* dst = (is_v ? pool_v : pool_k) + cache_row_offset(dst_page, g, b % LLMX_PAGE, G, width);
  pdl_wait();
  const int run = (pool + PB_WARPS - 1) / PB_WARPS;
  const int j_lo = p - pool + 1 + warp * run, j_hi = min(j_lo + run, p + 1);     // this warp's positions
  bool bad = false;
  for (int d0 = lane * V; d0 < width; d0 += 32 * V) {
    float sum[V];
#pragma unroll
    for (int e = 0; e < V; ++e) sum[e] = 0.f;
    for (int jb = j_lo; jb < j_hi; jb += 8) {              // eight positions' loads go out together
      float x[8][V];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int j = jb + u;
        if (j < j_hi) {
          int page = pages[j / LLMX_PAGE];
          if (page < 0 || page >= n_pages) bad = true, page = 0;
          pb_load<V>(src + cache_row_offset(page, g, j % LLMX_PAGE, G, width) + d0, x[u]);
        }
      }
#pragma unroll
      for (int u = 0; u < 8; ++u)
        if (jb + u < j_hi) {
#pragma unroll
          for (int e = 0; e < V; ++e) sum[e] += x[u][e];
        }
    }
#pragma unroll
    for (int e = 0; e < V; ++e) pb_part[warp * width + d0 + e] = sum[e];
  }
  if (bad) llmx_report(2);
  __syncthreads();
  const float inv = 1.0f / (float)pool;
  for (int d = threadIdx.x; d < width; d += PB_WARPS * 32) {
    float sum = pb_part[d];
#pragma unroll
    for (int w = 1; w < PB_WARPS; ++w) sum += pb_part[w * width + d];
    dst[d] = from_f32<TC>(sum * inv);
  }
}

// seq_start [n_seqs + 1], seq_past [n_seqs]: where each sequence's tokens start in the step and how many positions it
// held before; n_tokens: the step's tokens.
LLMX_API int llmx_pool_blocks(const void* k_cache, const void* v_cache, int cache_dtype, const int* block_table,
                              void* pool_k, void* pool_v, const int* pool_table, int table_width, const int* seq_start,
                              const int* seq_past, int n_seqs, int n_tokens, int G, int D, int Dv, int pool,
                              long long n_pages, long long n_pool_pages, cudaStream_t stream) {
  if (n_tokens <= 0 || n_seqs <= 0) return 0;
  if (G <= 0 || D <= 0 || Dv <= 0 || pool < 1 || n_pages < 1 || n_pool_pages < 1) return LLMX_REFUSED(1);
  if (2 * G > 65535) return LLMX_REFUSED(3);
  dim3 grid(n_tokens / pool + n_seqs, 2 * G);             // at least as many as blocks can end in such a step
  const size_t smem = (size_t)PB_WARPS * (D > Dv ? D : Dv) * sizeof(float);
  if (smem > 48 * 1024) return LLMX_REFUSED(3);
  const int v = cache_dtype == LLMX_BF16 ? 8 : 4;
  const bool vec = D % v == 0 && Dv % v == 0 && !(((uintptr_t)k_cache | (uintptr_t)v_cache) & 15);
#define CASE(TC, V)                                                                                           \
  launch_pdl(pool_blocks_kernel<TC, V>, grid, dim3(PB_WARPS * 32), smem, stream, (const TC*)k_cache,           \
             (const TC*)v_cache, block_table, (TC*)pool_k, (TC*)pool_v, pool_table, table_width, seq_start,    \
             seq_past, n_seqs, G, D, Dv, pool, (int)n_pages, (int)n_pool_pages)
  if (cache_dtype == LLMX_F32) {
    if (vec) CASE(float, 4); else CASE(float, 1);
  } else if (cache_dtype == LLMX_BF16) {
    if (vec) CASE(bf16, 8); else CASE(bf16, 1);
  } else {
    return LLMX_REFUSED(2);
  }
#undef CASE
  return LLMX_LAUNCH_STATUS();
}
