// A short causal convolution over time on every channel of a fused q|k|v projection, followed by what the
// attention mixer does to its heads before it attends: rotation of q and k, mixing of the values with those
// of an earlier layer, the cache write of k and v.
//
//   y_p[c] = sum_j w[j][c] * u_(p - taps + 1 + j)[c],   j = 0..taps-1,   u = 0 before the sequence's start
// (the weights come tap-major, [taps][C], so that a warp's lanes read neighbouring channels of one tap)
//
// u of the positions before the step's first token comes from the sequence's state: the last taps-1 projected
// rows, float32 [slot][taps-1][C], oldest first (zero-filled when the slot gets its owner, which is also what
// positions before the start must read).  conv_state_update moves the state on by the step's tokens; it is a
// second kernel because the first one's CTAs still read the old state.  In a step in which every sequence brings
// one token (`inline_state`) the first kernel moves the state on itself.
//
// Row layout of the projection: q heads (H of D), k heads (G of D), v heads (G of Dv); C = (H+G) D + G Dv.
// One warp per (token, head).  The convolved head is staged in shared memory so that a dim can read its
// rotation partner (i, i + n_rot/2).  Values: v_mix_mode 1 writes the head to v_first (float32 [T, G Dv]) as
// well; 2 replaces it by (1 - lambda) v + lambda v_first before the cache write.  All arithmetic is float32
// in a fixed order (taps oldest first, partials in order).
#include "common.cuh"

#define SC_WARPS 4
#define SC_MAX_TAPS 16

template <typename TIN>
__device__ __forceinline__ float sc_value(const TIN* p, int n_split, size_t split_stride) {
  float v = to_f32(p[0]);
  for (int s = 1; s < n_split; ++s) v += to_f32(p[(size_t)s * split_stride]);
  return v;
}

// Four consecutive channels at a time (the vector path of the kernel below).
__device__ __forceinline__ void sc_load4(const float* p, float* o) {
  const float4 x = *reinterpret_cast<const float4*>(p);
  o[0] = x.x, o[1] = x.y, o[2] = x.z, o[3] = x.w;
}
__device__ __forceinline__ void sc_load4(const bf16* p, float* o) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  o[0] = a.x, o[1] = a.y, o[2] = b.x, o[3] = b.y;
}
__device__ __forceinline__ void sc_store4(float* p, const float* v) {
  *reinterpret_cast<float4*>(p) = make_float4(v[0], v[1], v[2], v[3]);
}
__device__ __forceinline__ void sc_store4(bf16* p, const float* v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}
template <typename TIN>
__device__ __forceinline__ void sc_value4(const TIN* p, int n_split, size_t split_stride, float* o) {
  sc_load4(p, o);
  for (int s = 1; s < n_split; ++s) {
    float t[4];
    sc_load4(p + (size_t)s * split_stride, t);
#pragma unroll
    for (int e = 0; e < 4; ++e) o[e] += t[e];
  }
}

// VEC: a lane takes four consecutive dims per load and store (head sizes, the rotation's half and every row
// offset are multiples of four, all pointers 16-byte aligned); the sums run in the same order as one by one.
// SPW: heads per warp, one after another: a prompt step's warp takes four, so that the token's indices are
// fetched once for all of them; a step of few tokens gives every head a warp of its own.
template <typename TIN, typename TA, typename TC, bool VEC, int SPW>
__global__ void conv_rope_cache_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride,
                                       float* state, int inline_state, const float* __restrict__ conv_w, int taps,
                                       TA* __restrict__ q_out, TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                       const int* __restrict__ block_table, int table_width,
                                       const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                       const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                                       const int* __restrict__ seq_slot, const float* __restrict__ cos_t,
                                       const float* __restrict__ sin_t, int n_rot, float* __restrict__ v_first,
                                       const float* __restrict__ v_lambda, int v_mix_mode, int H, int G, int D, int Dv,
                                       int n_tokens, int n_seqs, int n_slots, int n_pages) {
  extern __shared__ float head_buf[];
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x;
  const int slot0 = (blockIdx.y * SC_WARPS + warp) * SPW;    // the warp's first head of the fused row
  if (slot0 >= H + 2 * G) return;
  const size_t C = (size_t)(H + G) * D + (size_t)G * Dv;
  const int b = token_seq[t], pos = token_pos[t];
  // Every index that comes out of the step's arrays is checked before it addresses anything: a step buffer that
  // does not fit the launch is reported (code 1) and the warp does nothing.
  if (b < 0 || b >= n_seqs || pos < 0 || pos / LLMX_PAGE >= table_width) {
    if (lane == 0) llmx_report(1);
    return;
  }
  const int p0 = seq_past[b], row0 = seq_start[b], slot = seq_slot[b];
  const int page = slot0 + SPW <= H ? 0 : block_table[(size_t)b * table_width + pos / LLMX_PAGE];
  if (p0 < 0 || p0 > pos || row0 < 0 || row0 + (pos - p0) >= n_tokens || slot < 0 || slot >= n_slots || page < 0 ||
      page >= n_pages) {
    if (lane == 0) llmx_report(1);
    return;
  }
  float* st = taps > 1 ? state + (size_t)slot * (taps - 1) * C : nullptr;
  // A step in which this sequence brings one token: the warp that convolves a head is the only reader of that
  // head's channels of the state, so it moves them on itself (row j of the old state becomes row j - 1, the token's
  // own projected row the last) and the second kernel is not launched.  A thread writes a row only after it has
  // read it and the one behind it.
  float* st_new = (inline_state && st && pos == p0 && seq_start[b + 1] - row0 == 1) ? st : nullptr;
  const float lam = v_mix_mode == 2 ? v_lambda[0] : 0.f;
  float* buf = head_buf + warp * max(D, Dv);
  pdl_wait();
  for (int hs = 0; hs < SPW; ++hs) {
  const int slot_h = slot0 + hs;                             // which head of the fused row
  if (slot_h >= H + 2 * G) break;
  const bool is_q = slot_h < H, is_k = !is_q && slot_h < H + G;
  const int hd = (is_q || is_k) ? D : Dv;
  const size_t c0 = (is_q || is_k) ? (size_t)slot_h * D : (size_t)(H + G) * D + (size_t)(slot_h - H - G) * Dv;
  if (VEC) {
    for (int i = lane * 4; i < hd; i += 128) {
      const size_t c = c0 + i;
      float y[4];
      if (taps > 0) {
        const float* wp = conv_w + c;                 // tap j of these four channels: wp + j * C
        y[0] = y[1] = y[2] = y[3] = 0.f;
        // four taps' rows are asked for together (their addresses do not depend on one another), then added in
        // the order of the taps
        for (int j0 = 0; j0 < taps; j0 += 4) {
          float u[4][4];
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            const int pp = pos - taps + 1 + j0 + jj;
            u[jj][0] = u[jj][1] = u[jj][2] = u[jj][3] = 0.f;
            if (j0 + jj < taps) {
              if (pp >= p0) sc_value4(proj + (size_t)(row0 + pp - p0) * C + c, n_split, split_stride, u[jj]);
              else if (pp >= 0) sc_load4(st + (size_t)(pp - (p0 - (taps - 1))) * C + c, u[jj]);
            }
          }
#pragma unroll
          for (int jj = 0; jj < 4; ++jj) {
            if (j0 + jj < taps) {
              if (st_new && j0 + jj >= 1) sc_store4(st_new + (size_t)(j0 + jj - 1) * C + c, u[jj]);
              float w[4];
              sc_load4(wp + (size_t)(j0 + jj) * C, w);
#pragma unroll
              for (int e = 0; e < 4; ++e) y[e] = fmaf(w[e], u[jj][e], y[e]);
            }
          }
        }
      } else {
        sc_value4(proj + (size_t)t * C + c, n_split, split_stride, y);
      }
      sc_store4(buf + i, y);
    }
    __syncwarp();
    if (is_q || is_k) {
      const int half = n_rot >> 1;
      const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
      const float* sv = sin_t ? sin_t + (size_t)pos * half : nullptr;
      TA* qrow = is_q ? q_out + (size_t)t * H * D + (size_t)slot_h * D : nullptr;
      TC* krow = is_k ? k_cache + cache_row_offset(page, slot_h - H, pos % LLMX_PAGE, G, D) : nullptr;
      for (int i = lane * 4; i < D; i += 128) {
        float v[4], o[4], cs[4], sn[4];
        sc_load4(buf + i, v);
        if (i < n_rot) {         // (i and the rotation's borders are multiples of four)
          const bool low = i < half;
          sc_load4(low ? buf + i + half : buf + i - half, o);
          sc_load4(c + (low ? i : i - half), cs);
          sc_load4(sv + (low ? i : i - half), sn);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = low ? v[e] * cs[e] - o[e] * sn[e] : v[e] * cs[e] + o[e] * sn[e];
        }
        if (is_q) sc_store4(qrow + i, v);
        else sc_store4(krow + i, v);
      }
    } else {
      const int g = slot_h - H - G;
      TC* vrow = v_cache + cache_row_offset(page, g, pos % LLMX_PAGE, G, Dv);
      float* first = v_mix_mode ? v_first + (size_t)t * G * Dv + (size_t)g * Dv : nullptr;
      for (int i = lane * 4; i < Dv; i += 128) {
        float v[4], f[4];
        sc_load4(buf + i, v);
        if (v_mix_mode == 1) {
          sc_store4(first + i, v);
        } else if (v_mix_mode == 2) {
          sc_load4(first + i, f);
#pragma unroll
          for (int e = 0; e < 4; ++e) v[e] = (1.0f - lam) * v[e] + lam * f[e];
        }
        sc_store4(vrow + i, v);
      }
    }
    __syncwarp();      // buf is filled again for the warp's next head
    continue;
  }
  for (int i = lane; i < hd; i += 32) {
    const size_t c = c0 + i;
    float y;
    if (taps > 0) {
      y = 0.f;
      for (int j = 0; j < taps; ++j) {
        const int pp = pos - taps + 1 + j;
        float u = 0.f;
        if (pp >= p0) u = sc_value(proj + (size_t)(row0 + pp - p0) * C + c, n_split, split_stride);
        else if (pp >= 0) u = st[(size_t)(pp - (p0 - (taps - 1))) * C + c];
        if (st_new && j >= 1) st_new[(size_t)(j - 1) * C + c] = u;
        y = fmaf(conv_w[(size_t)j * C + c], u, y);
      }
    } else {
      y = sc_value(proj + (size_t)t * C + c, n_split, split_stride);
    }
    buf[i] = y;
  }
  __syncwarp();
  if (is_q || is_k) {
    const int half = n_rot >> 1;
    const float* c = cos_t ? cos_t + (size_t)pos * half : nullptr;
    const float* sv = sin_t ? sin_t + (size_t)pos * half : nullptr;
    TA* qrow = is_q ? q_out + (size_t)t * H * D + (size_t)slot_h * D : nullptr;
    TC* krow = is_k ? k_cache + cache_row_offset(page, slot_h - H, pos % LLMX_PAGE, G, D) : nullptr;
    for (int i = lane; i < D; i += 32) {
      float v = buf[i];
      if (i < half) v = buf[i] * c[i] - buf[i + half] * sv[i];
      else if (i < n_rot) v = buf[i] * c[i - half] + buf[i - half] * sv[i - half];
      if (is_q) qrow[i] = from_f32<TA>(v);
      else krow[i] = from_f32<TC>(v);
    }
  } else {
    const int g = slot_h - H - G;
    TC* vrow = v_cache + cache_row_offset(page, g, pos % LLMX_PAGE, G, Dv);
    float* first = v_mix_mode ? v_first + (size_t)t * G * Dv + (size_t)g * Dv : nullptr;
    for (int i = lane; i < Dv; i += 32) {
      float v = buf[i];
      if (v_mix_mode == 1) first[i] = v;
      else if (v_mix_mode == 2) v = (1.0f - lam) * v + lam * first[i];
      vrow[i] = from_f32<TC>(v);
    }
  }
  __syncwarp();        // buf is filled again for the warp's next head
  }
}

// One thread per (sequence, channel): the state's rows become the projected rows of the last taps-1 positions
// after the step (old rows where the step brought fewer tokens than that).
template <typename TIN>
__global__ void conv_state_update_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride,
                                         float* __restrict__ state, int taps, const int* __restrict__ seq_start,
                                         const int* __restrict__ seq_slot, int n_seqs, size_t C, int n_tokens,
                                         int n_slots) {
  pdl_launch_dependents();
  pdl_wait();
  const int b = blockIdx.y;
  const size_t c = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= C || b >= n_seqs) return;
  const int row0 = seq_start[b], n_new = seq_start[b + 1] - row0, slot = seq_slot[b];
  if (row0 < 0 || n_new < 0 || row0 + n_new > n_tokens || slot < 0 || slot >= n_slots) {
    if (c == 0) llmx_report(2);
    return;
  }
  const int keep = taps - 1;
  float* st = state + (size_t)slot * keep * C + c;
  float nv[SC_MAX_TAPS];
#pragma unroll
  for (int i = 0; i < SC_MAX_TAPS; ++i) {
    if (i >= keep) break;
    const int j = n_new - keep + i;          // place among the step's tokens; negative: still an old row
    nv[i] = j >= 0 ? sc_value(proj + (size_t)(row0 + j) * C + c, n_split, split_stride) : st[(size_t)(i + n_new) * C];
  }
#pragma unroll
  for (int i = 0; i < SC_MAX_TAPS; ++i) {
    if (i >= keep) break;
    st[(size_t)i * C] = nv[i];
  }
}

// proj [T, C] or n_split float32 partials; conv_w float32 [taps, C] (taps 0: no convolution); state float32
// [slots, taps-1, C]; q_out [T, H*D]; cos/sin float32 [positions, n_rot/2]; v_first float32 [T, G*Dv] (v_mix_mode
// 1: written, 2: read with the weight *v_lambda).  inline_state: sequences that bring exactly one token have their
// state moved on by this kernel (the caller then leaves llmx_conv_state_update out; every sequence must bring one).
LLMX_API int llmx_conv_rope_cache(const void* proj, int in_dtype, int n_split, long long split_stride, float* state,
                                  int inline_state, const float* conv_w, int taps, void* q_out, int act_dtype, void* k_cache, void* v_cache,
                                  int cache_dtype, const int* block_table, int table_width, const int* token_seq,
                                  const int* token_pos, const int* seq_start, const int* seq_past, const int* seq_slot,
                                  const float* cos_t, const float* sin_t, int n_rot, float* v_first, const float* v_lambda,
                                  int v_mix_mode, int n_tokens, int H, int G, int D, int Dv, int n_seqs, int n_slots,
                                  long long n_pages, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || G <= 0 || D <= 0 || Dv <= 0 || n_rot < 0 || n_rot > D || (n_rot & 1) || n_split < 1 || taps < 0 ||
      taps > SC_MAX_TAPS || v_mix_mode < 0 || v_mix_mode > 2)
    return LLMX_REFUSED(1);
  if ((n_rot > 0 && (!cos_t || !sin_t)) || (taps > 0 && !conv_w) || (taps > 1 && !state) || (v_mix_mode && !v_first) ||
      (v_mix_mode == 2 && !v_lambda))
    return LLMX_REFUSED(4);
  const int hd = D > Dv ? D : Dv;
  const size_t smem = (size_t)SC_WARPS * hd * sizeof(float);
  if (smem > 48 * 1024) return LLMX_REFUSED(3);
  const int spw = n_tokens > 64 ? 4 : 1;
  dim3 grid(n_tokens, (H + 2 * G + SC_WARPS * spw - 1) / (SC_WARPS * spw));
  const bool vec = D % 4 == 0 && Dv % 4 == 0 && n_rot % 8 == 0 && split_stride % 4 == 0 &&
                   !(((uintptr_t)proj | (uintptr_t)state | (uintptr_t)conv_w | (uintptr_t)q_out | (uintptr_t)k_cache |
                      (uintptr_t)v_cache | (uintptr_t)cos_t | (uintptr_t)sin_t | (uintptr_t)v_first) & 15);
#define GO(TIN, TA, TC, VEC)              \
  do {                                    \
    if (spw == 4) GO2(TIN, TA, TC, VEC, 4); \
    else GO2(TIN, TA, TC, VEC, 1);        \
  } while (0)
#define GO2(TIN, TA, TC, VEC, SPW)                                                                                      \
  launch_pdl(conv_rope_cache_kernel<TIN, TA, TC, VEC, SPW>, grid, dim3(SC_WARPS * 32), smem, stream, (const TIN*)proj, n_split, \
             (size_t)split_stride, state, inline_state, conv_w, taps, (TA*)q_out, (TC*)k_cache, (TC*)v_cache, block_table,           \
             table_width, token_seq, token_pos, seq_start, seq_past, seq_slot, cos_t, sin_t, n_rot, v_first, v_lambda, \
             v_mix_mode, H, G, D, Dv, n_tokens, n_seqs, n_slots, (int)n_pages)
#define CASE(TIN, TA, TC)              \
  do {                                 \
    if (vec) GO(TIN, TA, TC, true);    \
    else GO(TIN, TA, TC, false);       \
  } while (0)
  const int key = in_dtype * 4 + act_dtype * 2 + cache_dtype;
  switch (key) {
    case 0: CASE(float, float, float); break;
    case 1: CASE(float, float, bf16); break;
    case 2: CASE(float, bf16, float); break;
    case 3: CASE(float, bf16, bf16); break;
    case 6: CASE(bf16, bf16, float); break;
    case 7: CASE(bf16, bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef CASE
#undef GO
#undef GO2
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_conv_state_update(const void* proj, int in_dtype, int n_split, long long split_stride, float* state,
                                    int taps, const int* seq_start, const int* seq_slot, int n_seqs, long long C,
                                    int n_tokens, int n_slots, cudaStream_t stream) {
  if (n_seqs <= 0 || taps <= 1) return 0;
  if (taps > SC_MAX_TAPS || C <= 0 || n_split < 1 || n_seqs > 65535) return LLMX_REFUSED(1);
  dim3 grid((unsigned)((C + 127) / 128), n_seqs);
  if (in_dtype == LLMX_F32)
    launch_pdl(conv_state_update_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, n_split,
               (size_t)split_stride, state, taps, seq_start, seq_slot, n_seqs, (size_t)C, n_tokens, n_slots);
  else if (in_dtype == LLMX_BF16)
    launch_pdl(conv_state_update_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)proj, n_split,
               (size_t)split_stride, state, taps, seq_start, seq_slot, n_seqs, (size_t)C, n_tokens, n_slots);
  else
    return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// A sublayer's input with its own short convolution added: out_p = x_p + sum_j w[j] * x_(p - taps + 1 + j), per
// channel, zeros before the sequence's start (tap-major weights [taps][C] as above; the last tap meets x_p itself).
// Rows before the step's first token come from the sequence's state (the last taps-1 rows of x, float32
// [slot][taps-1][C], oldest first).  One thread per (token, channel); taps oldest first, then x_p.  With
// `inline_state` (every sequence brings one token) the thread, the only reader of its channel's state, moves the
// state on itself; otherwise llmx_conv_state_update does so afterwards.
// ---------------------------------------------------------------------------
// V consecutive channels per thread (one 16-byte load of x for V = 8 bfloat16 or V = 4 float32; V = 1 where the
// width or an address does not allow it); the sums run per channel in the same order whatever V is.
template <int V>
__device__ __forceinline__ void rc_load(const float* p, float* o) {
  if (V == 4) sc_load4(p, o);
  else o[0] = p[0];
}
template <int V>
__device__ __forceinline__ void rc_load(const bf16* p, float* o) {
  if (V == 8) {
    sc_load4(p, o);
    sc_load4(p + 4, o + 4);
  } else {
    o[0] = to_f32(p[0]);
  }
}
template <int V>
__device__ __forceinline__ void rc_load_f32(const float* p, float* o) {
  if (V == 1) {
    o[0] = p[0];
  } else {
#pragma unroll
    for (int e = 0; e < V; e += 4) sc_load4(p + e, o + e);
  }
}
template <int V>
__device__ __forceinline__ void rc_store(float* p, const float* v) {
  if (V == 4) sc_store4(p, v);
  else p[0] = v[0];
}
template <int V>
__device__ __forceinline__ void rc_store(bf16* p, const float* v) {
  if (V == 8) {
    __nv_bfloat162 a = __floats2bfloat162_rn(v[0], v[1]), b = __floats2bfloat162_rn(v[2], v[3]);
    __nv_bfloat162 c = __floats2bfloat162_rn(v[4], v[5]), d = __floats2bfloat162_rn(v[6], v[7]);
    uint4 raw;
    raw.x = *reinterpret_cast<uint32_t*>(&a), raw.y = *reinterpret_cast<uint32_t*>(&b);
    raw.z = *reinterpret_cast<uint32_t*>(&c), raw.w = *reinterpret_cast<uint32_t*>(&d);
    *reinterpret_cast<uint4*>(p) = raw;
  } else {
    p[0] = from_f32<bf16>(v[0]);
  }
}

template <typename TX, int V>
__global__ void residual_conv_kernel(const TX* __restrict__ x, float* state, int inline_state,
                                     const float* __restrict__ conv_w, int taps, TX* __restrict__ out,
                                     const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                     const int* __restrict__ seq_start, const int* __restrict__ seq_past,
                                     const int* __restrict__ seq_slot, size_t C, int n_tokens, int n_seqs,
                                     int n_slots) {
  pdl_launch_dependents();
  const int t = blockIdx.x;
  const int b = token_seq[t], pos = token_pos[t];
  if (b < 0 || b >= n_seqs || pos < 0) {
    if (threadIdx.x == 0) llmx_report(1);
    return;
  }
  const int p0 = seq_past[b], row0 = seq_start[b], slot = seq_slot[b];
  const int keep = taps - 1;
  if (p0 < 0 || p0 > pos || row0 < 0 || row0 + (pos - p0) >= n_tokens || (keep > 0 && (slot < 0 || slot >= n_slots))) {
    if (threadIdx.x == 0) llmx_report(1);
    return;
  }
  float* st = keep > 0 ? state + (size_t)slot * keep * C : nullptr;
  const bool move = inline_state && st && pos == p0 && seq_start[b + 1] - row0 == 1;
  pdl_wait();
  for (size_t c = ((size_t)blockIdx.y * blockDim.x + threadIdx.x) * V; c < C; c += (size_t)gridDim.y * blockDim.x * V) {
    float y[V];
#pragma unroll
    for (int e = 0; e < V; ++e) y[e] = 0.f;
    for (int j = 0; j < taps; ++j) {
      const int q = pos - keep + j;                       // the position this tap reads
      float u[V], w[V];
      if (q >= p0) rc_load<V>(x + (size_t)(row0 + q - p0) * C + c, u);
      else rc_load_f32<V>(st + (size_t)(keep - (p0 - q)) * C + c, u);     // row i of the state is position p0 - keep + i
      rc_load_f32<V>(conv_w + (size_t)j * C + c, w);
#pragma unroll
      for (int e = 0; e < V; ++e) y[e] += w[e] * u[e];
    }
    float own[V];
    rc_load<V>(x + (size_t)t * C + c, own);
#pragma unroll
    for (int e = 0; e < V; ++e) y[e] = own[e] + y[e];
    rc_store<V>(out + (size_t)t * C + c, y);
    if (move) {
      for (int i = 0; i + 1 < keep; ++i) {
        float r[V];
        rc_load_f32<V>(st + (size_t)(i + 1) * C + c, r);
#pragma unroll
        for (int e = 0; e < V; ++e) st[(size_t)i * C + c + e] = r[e];
      }
#pragma unroll
      for (int e = 0; e < V; ++e) st[(size_t)(keep - 1) * C + c + e] = own[e];
    }
  }
}

// x, out [T, C] (float32 or bfloat16, the same); conv_w float32 [taps, C]; state float32 [slots, taps-1, C].
LLMX_API int llmx_residual_conv(const void* x, int dtype, float* state, int inline_state, const float* conv_w,
                                int taps, void* out, const int* token_seq, const int* token_pos,
                                const int* seq_start, const int* seq_past, const int* seq_slot, int n_tokens,
                                long long C, int n_seqs, int n_slots, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (C <= 0 || taps < 1 || taps > SC_MAX_TAPS || !conv_w || (taps > 1 && !state)) return LLMX_REFUSED(1);
  const int v = dtype == LLMX_BF16 ? 8 : 4;
  const bool vec = C % v == 0 && !(((uintptr_t)x | (uintptr_t)out | (uintptr_t)state | (uintptr_t)conv_w) & 15);
  const long long units = vec ? C / v : C;              // a thread's share: v channels, or one
  const int threads = units >= 256 ? 256 : units >= 128 ? 128 : 64;
  const long long per_row = (units + threads - 1) / threads;
  dim3 grid(n_tokens, (unsigned)(per_row < 64 ? per_row : 64));
#define GO(TX, V)                                                                                                       \
  launch_pdl(residual_conv_kernel<TX, V>, grid, dim3(threads), 0, stream, (const TX*)x, state, inline_state, conv_w,    \
             taps, (TX*)out, token_seq, token_pos, seq_start, seq_past, seq_slot, (size_t)C, n_tokens, n_seqs, n_slots)
  if (dtype == LLMX_F32) {
    if (vec) GO(float, 4); else GO(float, 1);
  } else if (dtype == LLMX_BF16) {
    if (vec) GO(bf16, 8); else GO(bf16, 1);
  } else {
    return LLMX_REFUSED(2);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}
