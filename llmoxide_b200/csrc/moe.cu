// Routed experts (a mixture of small gated feed-forward layers of which each token uses a few).
//
//   route      per token: scores from the router's float32 logits, the groups of experts a token may choose
//              from, its `top` experts and their weights
//   sort       the step's (token, choice) pairs ordered by expert, and the list of row tiles per expert
//   grouped products on the sorted rows: gate|up with the gated activation, then down times the pair's weight
//
// Everything a token gets depends on that token alone: routing is per token, and every output element of the
// products is accumulated by one thread in the order k = 0..K-1 whatever tile the row falls into, so results
// do not depend on what else is in the batch or on how a prompt was cut.  The order of rows inside an
// expert's segment is whatever the sort's atomics gave; no value depends on it.
#include "common.cuh"

#define MOE_TILE 64          // rows (and columns) per tile of the grouped products
#define MOE_BK 16
#define MOE_MAX_TOP 16
#define MOE_MAX_EXPERTS 1024

// SOFTMAX_TOP: the choice goes by the logits themselves, and the weights are the softmax over the chosen logits only.
enum { MOE_SCORE_SIGMOID = 0, MOE_SCORE_SOFTMAX = 1, MOE_SCORE_SOFTMAX_TOP = 2 };

// ---------------------------------------------------------------------------
// Routing.  One warp per token.  s = sigmoid(z) (or softmax(z)).  The expert indices are cut into n_groups
// contiguous blocks of E / n_groups; a block ranks by the sum of its group_top highest s, and only the
// keep_groups top-ranked blocks stay eligible.  Among the eligible experts the `top` highest s win (ties: the
// lower index); a winner's weight is its s, over (the winners' sum + norm_eps) when `normalize`, times `scale`.
// With a correction (`bias`, one number per expert) the groups are ranked and the experts chosen by s + bias,
// while the weights stay the chosen experts' s.
// ---------------------------------------------------------------------------
__device__ __forceinline__ void warp_argmax(float& v, int& i) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float v2 = __shfl_xor_sync(0xffffffffu, v, o);
    const int i2 = __shfl_xor_sync(0xffffffffu, i, o);
    if (v2 > v || (v2 == v && i2 < i)) v = v2, i = i2;
  }
}

// One token, by one warp: z its E logits (global or shared memory), s, c and gs scratch of E, E and n_groups
// floats (c: the scores the choice goes by), ids and wts its `top` outputs.
__device__ __forceinline__ void moe_route_token(const float* z, float* s, float* c, float* gs, int* __restrict__ ids,
                                                float* __restrict__ wts, int lane, int E, int top, int n_groups,
                                                int keep_groups, int group_top, int score_kind, int normalize,
                                                float norm_eps, float scale, const float* __restrict__ bias) {
  if (score_kind == MOE_SCORE_SOFTMAX) {
    float m = -INFINITY;
    for (int e = lane; e < E; e += 32) m = fmaxf(m, z[e]);
    m = warp_max(m);
    float sum = 0.f;
    for (int e = lane; e < E; e += 32) sum += expf(z[e] - m);
    sum = warp_sum(sum);
    for (int e = lane; e < E; e += 32) s[e] = expf(z[e] - m) / sum;
  } else if (score_kind == MOE_SCORE_SOFTMAX_TOP) {
    for (int e = lane; e < E; e += 32) s[e] = z[e];
  } else {
    for (int e = lane; e < E; e += 32) s[e] = 1.0f / (1.0f + expf(-z[e]));
  }
  __syncwarp();
  for (int e = lane; e < E; e += 32) c[e] = bias ? s[e] + bias[e] : s[e];
  __syncwarp();
  const int per = E / n_groups;
  if (n_groups > 1 && keep_groups < n_groups) {
    // a group's score: the sum of its group_top largest (picked one by one; an index picked is left out)
    for (int g = lane; g < n_groups; g += 32) {
      int picked[8];
      float sum = 0.f;
      const int n_pick = group_top < per ? group_top : per;
      for (int k = 0; k < n_pick; ++k) {
        float best = -INFINITY;
        int bi = -1;
        for (int e = g * per; e < (g + 1) * per; ++e) {
          bool used = false;
          for (int j = 0; j < k; ++j) used = used || picked[j] == e;
          if (!used && c[e] > best) best = c[e], bi = e;
        }
        picked[k] = bi;
        sum += best;
      }
      gs[g] = sum;
    }
    __syncwarp();
    // the keep_groups best groups stay; the others' experts get a score no expert can have
    for (int k = 0; k < keep_groups; ++k) {
      float best = -INFINITY;
      int bi = 0x7fffffff;
      for (int g = lane; g < n_groups; g += 32)
        if (gs[g] > best) best = gs[g], bi = g;     // ascending g: the lower index wins a tie
      warp_argmax(best, bi);
      if (lane == 0) gs[bi] = -INFINITY;            // kept: marked
      __syncwarp();
    }
    for (int e = lane; e < E; e += 32)
      if (gs[e / per] != -INFINITY) c[e] = -INFINITY;   // not kept
    __syncwarp();
  }
  float sum = 0.f, mine = 0.f;
  int my_id = 0;
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
    for (int e = lane; e < E; e += 32)
      if (c[e] > best) best = c[e], bi = e;
    warp_argmax(best, bi);
    if (bi >= E) {
      // No score compares greater than -inf: the token's row holds a NaN (or every score is -inf).  That is
      // reported (code 1); the lowest expert not chosen yet stands in, so that no index leaves its array.
      bi = 0x7fffffff;
      for (int e = lane; e < E; e += 32)
        if (!(c[e] == -INFINITY) && e < bi) bi = e;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) bi = min(bi, __shfl_xor_sync(0xffffffffu, bi, o));
      if (bi >= E) bi = k % E;
      if (lane == 0) llmx_report(1);
    }
    if (lane == 0) c[bi] = -INFINITY;               // chosen: out of the running
    __syncwarp();
    const float sb = s[bi];
    if (lane == k) mine = sb, my_id = bi;
    sum += sb;
  }
  if (score_kind == MOE_SCORE_SOFTMAX_TOP) {
    // lane k holds the k-th chosen logit: softmax over those (all lanes take part in the butterflies)
    const float zk = lane < top ? mine : -INFINITY;
    const float z_max = warp_max(zk);
    const float ek = lane < top ? expf(zk - z_max) : 0.f;
    const float total = warp_sum(ek);
    if (lane < top) {
      ids[lane] = my_id;
      wts[lane] = (ek / total) * scale;
    }
    return;
  }
  if (lane < top) {
    const float w = normalize ? mine / (sum + norm_eps) : mine;
    ids[lane] = my_id;
    wts[lane] = w * scale;
  }
}

__global__ void moe_route_kernel(const float* __restrict__ logits, int* __restrict__ ids, float* __restrict__ wts,
                                 int n_tokens, int E, int top, int n_groups, int keep_groups, int group_top,
                                 int score_kind, int normalize, float norm_eps, float scale,
                                 const float* __restrict__ bias) {
  extern __shared__ float route_smem[];            // per warp: E scores, E choice scores, n_groups group scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x * 4 + warp;
  if (t >= n_tokens) return;
  float* s = route_smem + warp * (2 * E + n_groups);
  moe_route_token(logits + (size_t)t * E, s, s + E, s + 2 * E, ids + (size_t)t * top, wts + (size_t)t * top, lane, E, top,
                  n_groups, keep_groups, group_top, score_kind, normalize, norm_eps, scale, bias);
}

// The router's product and the routing in one kernel: a CTA of 8 warps takes TOK tokens (4 in a prompt step, so
// that a row of the router's matrix is fetched once for four tokens; 1 in a step of few tokens, so that more SMs
// take part); warp w computes the float32 logits of experts w, w + 8, ... (a lane adds its share of k in
// ascending order, eight consecutive k at a time, then the lanes are added by a butterfly: the order depends on
// nothing but K), then warp j routes token j.  The matrix may hold n_extra rows behind the experts' (a gate
// that reads the same input): their logits are written to extra_out [T, n_extra] as they are.
__device__ __forceinline__ void moe_load8(const float* p, float* v) {
  const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
  v[0] = a.x, v[1] = a.y, v[2] = a.z, v[3] = a.w, v[4] = b.x, v[5] = b.y, v[6] = b.z, v[7] = b.w;
}
__device__ __forceinline__ void moe_load8(const bf16* p, float* v) {
  const uint4 raw = *reinterpret_cast<const uint4*>(p);
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const float2 f = __bfloat1622float2(h[i]);
    v[2 * i] = f.x, v[2 * i + 1] = f.y;
  }
}

template <typename TX, int TOK>
__global__ void __launch_bounds__(256)
moe_router_kernel(const TX* __restrict__ x, long long ldx, const float* __restrict__ w, int* __restrict__ ids,
                  float* __restrict__ wts, int n_tokens, int K, int E, int top, int n_groups, int keep_groups,
                  int group_top, int score_kind, int normalize, float norm_eps, float scale, int vec,
                  const float* __restrict__ bias, int n_extra, float* __restrict__ extra_out,
                  const float* __restrict__ logit_bias) {
  extern __shared__ float route_smem[];            // per token: E + n_extra logits, E scores, n_groups group scores
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t0 = blockIdx.x * TOK;
  const int per_tok = 2 * E + n_extra + n_groups;
  const int n_rows = E + n_extra;
  const TX* xr[TOK];
#pragma unroll
  for (int j = 0; j < TOK; ++j) xr[j] = x + (size_t)min(t0 + j, n_tokens - 1) * ldx;
  for (int e = warp; e < n_rows; e += 8) {
    const float* wr = w + (size_t)e * K;
    float acc[TOK];
#pragma unroll
    for (int j = 0; j < TOK; ++j) acc[j] = 0.f;
    if (vec) {           // K a multiple of 8 and rows 16-byte aligned: 8 consecutive k per lane and step
#pragma unroll 2
      for (int k = lane * 8; k < K; k += 256) {
        float wv[8], xv[TOK][8];
        moe_load8(wr + k, wv);
#pragma unroll
        for (int j = 0; j < TOK; ++j) moe_load8(xr[j] + k, xv[j]);
#pragma unroll
        for (int j = 0; j < TOK; ++j)
#pragma unroll
          for (int i = 0; i < 8; ++i) acc[j] = fmaf(xv[j][i], wv[i], acc[j]);
      }
    } else {
      for (int k0 = lane * 8; k0 < K; k0 += 256)
        for (int k = k0; k < k0 + 8 && k < K; ++k) {
          const float wv = wr[k];
#pragma unroll
          for (int j = 0; j < TOK; ++j) acc[j] = fmaf(to_f32(xr[j][k]), wv, acc[j]);
        }
    }
#pragma unroll
    for (int j = 0; j < TOK; ++j) {
      const float v = warp_sum(acc[j]);
      if (lane == 0) route_smem[j * per_tok + e] = (logit_bias && e < E) ? v + logit_bias[e] : v;
    }
  }
  __syncthreads();
  const int t = t0 + warp;
  if (warp >= TOK || t >= n_tokens) return;
  float* z = route_smem + warp * per_tok;
  if (lane < n_extra) extra_out[(size_t)t * n_extra + lane] = z[E + lane];
  // (the logits are not needed once the scores exist: their place holds the choice scores)
  moe_route_token(z, z + n_rows, z, z + n_rows + E, ids + (size_t)t * top, wts + (size_t)t * top, lane, E, top, n_groups,
                  keep_groups, group_top, score_kind, normalize, norm_eps, scale, bias);
}

// x [T, K] (float32 or bfloat16, row stride ldx), w float32 [E, K] -> ids int32 [T, top], wts float32 [T, top].
// logit_bias: null, or float32 [E] added to the experts' logits before anything is made of them.
LLMX_API int llmx_moe_router_biased(const void* x, int x_dtype, long long ldx, const float* w, int* ids, float* wts,
                             int n_tokens, int K, int E, int top, int n_groups, int keep_groups, int group_top,
                             int score_kind, int normalize, float norm_eps, float scale, const float* bias,
                             int n_extra, float* extra_out, const float* logit_bias, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (score_kind < MOE_SCORE_SIGMOID || score_kind > MOE_SCORE_SOFTMAX_TOP || top > 32) return LLMX_REFUSED(1);
  if (n_extra < 0 || n_extra > 32 || (n_extra > 0 && !extra_out)) return LLMX_REFUSED(1);
  if (K <= 0 || ldx < K || E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP || n_groups <= 0 || E % n_groups ||
      keep_groups <= 0 || keep_groups > n_groups || group_top <= 0 || group_top > 8 ||
      top > E / n_groups * keep_groups)
    return LLMX_REFUSED(1);
  const int tok = n_tokens <= 64 ? 1 : 4;
  const size_t smem = (size_t)tok * (2 * E + n_extra + n_groups) * sizeof(float);
  const dim3 grid((n_tokens + tok - 1) / tok);
  const int esz = x_dtype == LLMX_F32 ? 4 : 2;
  const int vec = (K % 8 == 0) && ((ldx * esz) % 16 == 0) && !((uintptr_t)x & 15) && !((uintptr_t)w & 15);
#define GO(TX, TOK)                                                                                                    \
  launch_pdl(moe_router_kernel<TX, TOK>, grid, dim3(256), smem, stream, (const TX*)x, ldx, w, ids, wts, n_tokens, K, E, \
             top, n_groups, keep_groups, group_top, score_kind, normalize, norm_eps, scale, vec, bias, n_extra, extra_out, \
             logit_bias)
  if (x_dtype == LLMX_F32) {
    if (tok == 1) GO(float, 1); else GO(float, 4);
  } else if (x_dtype == LLMX_BF16) {
    if (tok == 1) GO(bf16, 1); else GO(bf16, 4);
  } else {
    return LLMX_REFUSED(2);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_moe_router(const void* x, int x_dtype, long long ldx, const float* w, int* ids, float* wts,
                             int n_tokens, int K, int E, int top, int n_groups, int keep_groups, int group_top,
                             int score_kind, int normalize, float norm_eps, float scale, const float* bias,
                             int n_extra, float* extra_out, cudaStream_t stream) {
  return llmx_moe_router_biased(x, x_dtype, ldx, w, ids, wts, n_tokens, K, E, top, n_groups, keep_groups, group_top,
                                score_kind, normalize, norm_eps, scale, bias, n_extra, extra_out, nullptr, stream);
}

LLMX_API int llmx_moe_route(const float* logits, int* ids, float* wts, int n_tokens, int E, int top, int n_groups,
                            int keep_groups, int group_top, int score_kind, int normalize, float norm_eps,
                            float scale, const float* bias, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (E <= 0 || E > MOE_MAX_EXPERTS || top <= 0 || top > MOE_MAX_TOP || top > 32 || n_groups <= 0 || E % n_groups ||
      keep_groups <= 0 || keep_groups > n_groups || group_top <= 0 || group_top > 8 ||
      top > E / n_groups * keep_groups)
    return LLMX_REFUSED(1);
  const size_t smem = 4 * (size_t)(2 * E + n_groups) * sizeof(float);
  launch_pdl(moe_route_kernel, dim3((n_tokens + 3) / 4), dim3(128), smem, stream, logits, ids, wts, n_tokens, E, top,
             n_groups, keep_groups, group_top, score_kind, normalize, norm_eps, scale, bias);
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Sort.  One CTA.  P = n_tokens * top pairs, pair r = t * top + choice.  Out: perm[P] (sorted place -> pair),
// tiles: for every row tile of tile_rows sorted rows that lie in one expert's segment, (expert, first row,
// number of rows); the used tiles come first, unused ones have expert -1.  max_tiles >= P / tile_rows + E.
// Experts n_tiled..E-1 have no products (identity experts): their pairs are placed but get no tiles.
// ---------------------------------------------------------------------------
__global__ void __launch_bounds__(1024)
moe_sort_kernel(const int* __restrict__ ids, const float* __restrict__ pair_weight, int P, int E, int top,
                int n_tokens, int* __restrict__ perm, int* __restrict__ dest, float* __restrict__ sorted_weight,
                int* __restrict__ tiles, int max_tiles, int tile_rows, int n_tiled) {
  __shared__ int count[MOE_MAX_EXPERTS];
  __shared__ int start[MOE_MAX_EXPERTS + 1];
  __shared__ int tile0[MOE_MAX_EXPERTS + 1];
  pdl_launch_dependents();
  pdl_wait();
  const int tid = threadIdx.x;
  for (int e = tid; e < E; e += blockDim.x) count[e] = 0;
  __syncthreads();
  // (an expert id outside 0..E-1 cannot come from this library's routing; it is reported, code 2, and counted as the
  // last expert, so that no index leaves its array)
  for (int r = tid; r < P; r += blockDim.x) {
    int e = ids[r];
    if ((unsigned)e >= (unsigned)E) {
      llmx_report(2);
      e = E - 1;
    }
    atomicAdd(&count[e], 1);
  }
  __syncthreads();
  if (tid == 0) {
    int at = 0, tl = 0;
    for (int e = 0; e < E; ++e) {
      start[e] = at;
      tile0[e] = tl;
      at += count[e];
      if (e < n_tiled) tl += (count[e] + tile_rows - 1) / tile_rows;
    }
    start[E] = at;
    tile0[E] = tl;
  }
  __syncthreads();
  for (int e = tid; e < E; e += blockDim.x) {
    const int n = count[e];
    for (int k = 0, tl = tile0[e]; k < n && e < n_tiled; k += tile_rows, ++tl) {
      tiles[3 * tl] = e;
      tiles[3 * tl + 1] = start[e] + k;
      tiles[3 * tl + 2] = (n - k) < tile_rows ? (n - k) : tile_rows;
    }
    count[e] = 0;          // reused as the segment's fill counter
  }
  for (int tl = tile0[E] + tid; tl < max_tiles; tl += blockDim.x) tiles[3 * tl] = -1;
  __syncthreads();
  for (int r = tid; r < P; r += blockDim.x) {
    int e = ids[r];
    if ((unsigned)e >= (unsigned)E) e = E - 1;
    const int place = start[e] + atomicAdd(&count[e], 1);
    perm[place] = r;
    if (dest) {             // where the pair's result goes in [top, n_tokens, ...], and its weight, in sorted order
      const int t = r / top;
      dest[place] = (r - t * top) * n_tokens + t;
      sorted_weight[place] = pair_weight[r];
    }
  }
}

// dest, sorted_weight (both [P]) may be null; with them pair_weight [P], top and n_tokens are needed.
LLMX_API int llmx_moe_sort(const int* ids, const float* pair_weight, int P, int E, int top, int n_tokens, int* perm,
                           int* dest, float* sorted_weight, int* tiles, int max_tiles, int tile_rows, int n_tiled,
                           cudaStream_t stream) {
  if (P <= 0) return 0;
  if (n_tiled < 0 || n_tiled > E) return LLMX_REFUSED(1);
  if (E <= 0 || E > MOE_MAX_EXPERTS || tile_rows <= 0 || max_tiles < (P + tile_rows - 1) / tile_rows + E)
    return LLMX_REFUSED(1);
  if (dest && (!sorted_weight || !pair_weight || top <= 0 || n_tokens <= 0)) return LLMX_REFUSED(4);
  launch_pdl(moe_sort_kernel, dim3(1), dim3(P >= 4096 ? 1024 : 256), 0, stream, ids, pair_weight, P, E, top, n_tokens,
             perm, dest, sorted_weight, tiles, max_tiles, tile_rows, n_tiled);
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Grouped products on the FMA units (float32 accumulation, k = 0..K-1 per output element).
//
// GATED: rows are tokens' rows of x gathered through perm (token = pair / top); W = [E][2F][K], gate rows then
//   up rows; out act[place][f] = gated_act(gate, up) (common.cuh), in sorted order.
// else:  rows are act[place]; W = [E][N][K]; out y[choice][token][n] = weight[pair] * sum, float32: one partial
//   per choice, which whoever adds them to the residual stream sums in the order of the choices.
// ---------------------------------------------------------------------------
template <typename TX, typename TW, typename TY, bool GATED>
__global__ void __launch_bounds__(256)
moe_grouped_fma_kernel(const TX* __restrict__ X, long long ldx, const TW* __restrict__ W, TY* __restrict__ Y,
                       const int* __restrict__ perm, const int* __restrict__ tiles,
                       const float* __restrict__ pair_weight, int top, int n_tokens, int N, int K, const GateAct act) {
  __shared__ float Xs[MOE_BK][MOE_TILE + 4];
  __shared__ float Ws[MOE_BK][MOE_TILE + 4];
  __shared__ float Us[GATED ? MOE_BK : 1][MOE_TILE + 4];
  __shared__ int row_src[MOE_TILE];
  pdl_launch_dependents();
  pdl_wait();
  const int tl = blockIdx.y;
  const int e = tiles[3 * tl];
  if (e < 0) return;
  const int row0 = tiles[3 * tl + 1], n_rows = tiles[3 * tl + 2];
  const int tid = threadIdx.x;
  const int tx = tid & 15, ty = tid >> 4;
  const int n0 = blockIdx.x * MOE_TILE;
  const int lrow = tid >> 2, lk = (tid & 3) * 4;
  if (tid < MOE_TILE) row_src[tid] = tid < n_rows ? perm[row0 + tid] : -1;
  __syncthreads();
  const int pair = row_src[lrow];
  const TX* xrow = nullptr;
  if (pair >= 0) xrow = GATED ? X + (size_t)(pair / top) * ldx : X + (size_t)(row0 + lrow) * ldx;
  const size_t w_rows = GATED ? 2 * (size_t)N : (size_t)N;
  const TW* We = W + (size_t)e * w_rows * K;
  const int n_load = n0 + lrow;
  const TW* wrow = n_load < N ? We + (size_t)n_load * K : nullptr;
  const TW* urow = (GATED && n_load < N) ? We + ((size_t)N + n_load) * K : nullptr;

  float acc[4][4], acu[GATED ? 4 : 1][4];
#pragma unroll
  for (int i = 0; i < 4; ++i)
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      acc[i][j] = 0.f;
      if constexpr (GATED) acu[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += MOE_BK) {
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const int k = k0 + lk + c;
      Xs[lk + c][lrow] = (xrow && k < K) ? to_f32(xrow[k]) : 0.f;
      Ws[lk + c][lrow] = (wrow && k < K) ? to_f32(wrow[k]) : 0.f;
      if constexpr (GATED) Us[lk + c][lrow] = (urow && k < K) ? to_f32(urow[k]) : 0.f;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < MOE_BK; ++kk) {
      float a[4], b[4], u[4];
#pragma unroll
      for (int i = 0; i < 4; ++i) a[i] = Xs[kk][ty * 4 + i];
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        b[j] = Ws[kk][tx * 4 + j];
        if constexpr (GATED) u[j] = Us[kk][tx * 4 + j];
      }
#pragma unroll
      for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
          acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
          if constexpr (GATED) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const int lr = ty * 4 + i;
    const int pr = row_src[lr];
    if (pr < 0) continue;
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int n = n0 + tx * 4 + j;
      if (n >= N) continue;
      if constexpr (GATED) {
        Y[(size_t)(row0 + lr) * N + n] = from_f32<TY>(gated_act(act, acc[i][j], acu[i][j]));
      } else {
        const int t = pr / top, choice = pr - t * top;
        Y[((size_t)choice * n_tokens + t) * N + n] = from_f32<TY>(pair_weight[pr] * acc[i][j]);
      }
    }
  }
}

// gated != 0: X = x [n_tokens, K] (row stride ldx), W [E, 2N, K], Y = act [P, N].
// else:       X = act [P, K], W [E, N, K], Y = float32 [top, n_tokens, N].
// The tile list must have been made with MOE_TILE rows per tile.
LLMX_API int llmx_moe_grouped_fma(const void* X, int x_dtype, long long ldx, const void* W, int w_dtype, void* Y,
                                  int y_dtype, const int* perm, const int* tiles, int max_tiles,
                                  const float* pair_weight, int top, int n_tokens, int N, int K, int gated,
                                  int act_kind, float slope, float limit, float shift, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (act_kind < LLMX_ACT_SILU || act_kind > LLMX_ACT_LAST) return LLMX_REFUSED(1);
  const GateAct act = {act_kind, slope, limit, shift};
  if (N <= 0 || K <= 0 || top <= 0 || max_tiles <= 0 || max_tiles > 65535 || ldx < K) return LLMX_REFUSED(1);
  if (x_dtype != w_dtype) return LLMX_REFUSED(2);
  dim3 grid((N + MOE_TILE - 1) / MOE_TILE, max_tiles);
#define GO(TX, TY, G)                                                                                          \
  launch_pdl(moe_grouped_fma_kernel<TX, TX, TY, G>, grid, dim3(256), 0, stream, (const TX*)X, ldx, (const TX*)W, \
             (TY*)Y, perm, tiles, pair_weight, top, n_tokens, N, K, act)
  if (gated) {
    if (x_dtype == LLMX_F32 && y_dtype == LLMX_F32) GO(float, float, true);
    else if (x_dtype == LLMX_BF16 && y_dtype == LLMX_BF16) GO(bf16, bf16, true);
    else return LLMX_REFUSED(2);
  } else {
    if (y_dtype != LLMX_F32) return LLMX_REFUSED(2);
    if (x_dtype == LLMX_F32) GO(float, float, false);
    else if (x_dtype == LLMX_BF16) GO(bf16, float, false);
    else return LLMX_REFUSED(2);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Identity experts and a gated shared expert, both written as further partials of the feed-forward's result, in
// one launch.
//
// CTAs 0 .. T*top-1, one per pair (t, choice): if the pair's expert id is >= n_real (an identity expert, whose
//   output is its input), y[choice][t][:] = weight * x[t][:]; pairs of real experts are left alone.
// CTAs T*top .. T*top+T-1 (with a shared expert), one per token: y[top][t][:] = sigmoid(z[t * ldz]) * sum_p
//   shared[p][t][:], the shared expert's result times one number per token.
// ---------------------------------------------------------------------------
template <typename TX, typename TS, int VEC>
__global__ void __launch_bounds__(256)
moe_extras_kernel(const TX* __restrict__ x, long long ldx, const int* __restrict__ ids, const float* __restrict__ wts,
                  float* __restrict__ y, int n_tokens, int top, int d, int n_real, const TS* __restrict__ shared,
                  int n_split, size_t split_stride, const float* __restrict__ z, int ldz) {
  pdl_launch_dependents();
  pdl_wait();
  const int n_pairs = n_tokens * top;
  if ((int)blockIdx.x < n_pairs) {
    const int pair = blockIdx.x;
    if (ids[pair] < n_real) return;
    const int t = pair / top, choice = pair - t * top;
    const float w = wts[pair];
    const TX* xr = x + (size_t)t * ldx;
    float* yr = y + ((size_t)choice * n_tokens + t) * d;
    for (int i = threadIdx.x * VEC; i < d; i += blockDim.x * VEC) {
      if (VEC == 8) {
        float v[8];
        moe_load8(xr + i, v);
        *reinterpret_cast<float4*>(yr + i) = make_float4(w * v[0], w * v[1], w * v[2], w * v[3]);
        *reinterpret_cast<float4*>(yr + i + 4) = make_float4(w * v[4], w * v[5], w * v[6], w * v[7]);
      } else {
        yr[i] = w * to_f32(xr[i]);
      }
    }
    return;
  }
  const int t = blockIdx.x - n_pairs;
  const float gate = z ? 1.0f / (1.0f + expf(-z[(size_t)t * ldz])) : 1.0f;      // no logit: the result joins as it is
  float* yr = y + ((size_t)top * n_tokens + t) * d;
  for (int i = threadIdx.x * VEC; i < d; i += blockDim.x * VEC) {
    if (VEC == 8) {
      float v[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
      for (int p = 0; p < n_split; ++p) {
        float a[8];
        moe_load8(shared + (size_t)p * split_stride + (size_t)t * d + i, a);
#pragma unroll
        for (int e = 0; e < 8; ++e) v[e] += a[e];
      }
      *reinterpret_cast<float4*>(yr + i) = make_float4(gate * v[0], gate * v[1], gate * v[2], gate * v[3]);
      *reinterpret_cast<float4*>(yr + i + 4) = make_float4(gate * v[4], gate * v[5], gate * v[6], gate * v[7]);
    } else {
      float v = 0.f;
      for (int p = 0; p < n_split; ++p) v += to_f32(shared[(size_t)p * split_stride + (size_t)t * d + i]);
      yr[i] = gate * v;
    }
  }
}

// x [T, d] (row stride ldx); ids, wts [T, top]; y float32 [top (+1), T, d]; identity experts are ids >= n_real
// (n_real >= all ids: none).  shared: null, or the shared expert's result [T, d] as n_split partials, with z (one
// float per token, ldz apart) the logit of its gate, or null for no gate.
LLMX_API int llmx_moe_extras(const void* x, int x_dtype, long long ldx, const int* ids, const float* wts, float* y,
                             int n_tokens, int top, int d, int n_real, const void* shared, int shared_dtype, int n_split,
                             long long split_stride, const float* z, int ldz, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (top <= 0 || d <= 0 || ldx < d || (shared && ((z && ldz < 1) || n_split < 1))) return LLMX_REFUSED(1);
  const dim3 grid((unsigned)n_tokens * top + (shared ? (unsigned)n_tokens : 0u));
  // eight columns per thread and load where every row starts on a 32-byte boundary
  const bool vec = d % 8 == 0 && ldx % 8 == 0 && split_stride % 8 == 0 &&
                   !(((uintptr_t)x | (uintptr_t)y | (uintptr_t)shared) & 31);
  const int threads = d >= 2048 ? 256 : 128;
#define GO(TX, TS)                                                                                                      \
  do {                                                                                                                  \
    if (vec)                                                                                                            \
      launch_pdl(moe_extras_kernel<TX, TS, 8>, grid, dim3(threads), 0, stream, (const TX*)x, ldx, ids, wts, y, n_tokens, \
                 top, d, n_real, (const TS*)shared, n_split, (size_t)split_stride, z, ldz);                             \
    else                                                                                                                \
      launch_pdl(moe_extras_kernel<TX, TS, 1>, grid, dim3(threads), 0, stream, (const TX*)x, ldx, ids, wts, y, n_tokens, \
                 top, d, n_real, (const TS*)shared, n_split, (size_t)split_stride, z, ldz);                             \
  } while (0)
  const int key = x_dtype * 2 + (shared ? shared_dtype : LLMX_F32);
  switch (key) {
    case 0: GO(float, float); break;
    case 1: GO(float, bf16); break;
    case 2: GO(bf16, float); break;
    case 3: GO(bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// Routing by a table: a token's experts are row `token id` of an integer table [vocab, top], each with the same
// weight.  An id outside the vocabulary or an expert outside [0, E) is reported (code 3) and expert 0 stands in,
// so that nothing later indexes with it.
// ---------------------------------------------------------------------------
__global__ void moe_table_route_kernel(const int* __restrict__ tokens, const int* __restrict__ table, int vocab,
                                       int E, int top, float weight, int* __restrict__ ids, float* __restrict__ wts,
                                       int n_tokens) {
  pdl_launch_dependents();
  pdl_wait();
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= n_tokens * top) return;
  const int t = i / top, k = i % top;
  const int tok = tokens[t];
  int e = 0;
  if (tok < 0 || tok >= vocab) {
    llmx_report(3);
  } else {
    e = table[(size_t)tok * top + k];
    if (e < 0 || e >= E) {
      llmx_report(3);
      e = 0;
    }
  }
  ids[i] = e;
  wts[i] = weight;
}

LLMX_API int llmx_moe_table_route(const int* tokens, const int* table, int vocab, int E, int top, float weight, int* ids,
                                  float* wts, int n_tokens, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (vocab <= 0 || E <= 0 || top <= 0 || top > E) return LLMX_REFUSED(1);
  const int n = n_tokens * top;
  launch_pdl(moe_table_route_kernel, dim3((n + 127) / 128), dim3(128), 0, stream, tokens, table, vocab, E, top, weight,
             ids, wts, n_tokens);
  return LLMX_LAUNCH_STATUS();
}
