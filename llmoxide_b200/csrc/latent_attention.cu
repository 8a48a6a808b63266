// Attention whose queries, keys and values come through low-rank latents: the two small kernels between its
// matrix products.
//
// The first product of the mixer is fused: row t of `down` holds [ dq (Rq) | dkv latent (Rkv) | shared rotated key
// part (R) | head gates (H) ], float32 or split float32 partials.
//
// latent_norms: cq = rms(down[:Rq]) * gq and c = rms(down[Rq : Rq+Rkv]) * gkv, x / sqrt(mean(x^2) + eps), float32
// statistics, written in the compute dtype as the operands of the two up-projections.  One CTA of 128 threads per
// token; sums in an order fixed by the width alone.
//
// latent_rope_cache: per (token, head), from q [T, H, R + D] (up-projected queries, every head [rotated part |
// unrotated part]), kv [T, H*D + H*Dv] (up-projected unrotated keys, then values) and the shared rotated key part
// of `down`:
//   q_out[t, h]          = [ rot(q_rot) | q_plain ]
//   k_cache[pos, h]      = [ rot(k_rot shared) | k_plain[h] ]        (one cached key per head, size R + D)
//   v_cache[pos, h]      = v[h]
// rot turns the pairs (i, i + R/2) by the position's angles (tables [positions, R/2] that already carry the
// rotation's amplitude).  One warp per (token, head).  Everything is float32 until it is stored.
#include "common.cuh"

#define LA_WARPS 4

template <typename TIN>
__device__ __forceinline__ float la_value(const TIN* p, int n_split, size_t split_stride) {
  float v = to_f32(p[0]);
  for (int s = 1; s < n_split; ++s) v += to_f32(p[(size_t)s * split_stride]);
  return v;
}

template <typename TIN, typename TA>
__global__ void latent_norms_kernel(const TIN* __restrict__ down, int n_split, size_t split_stride, size_t row_stride,
                                    const float* __restrict__ q_gain, const float* __restrict__ kv_gain, float eps,
                                    TA* __restrict__ cq, TA* __restrict__ c, int Rq, int Rkv) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int t = blockIdx.x, which = blockIdx.y;          // which: 0 the query latent, 1 the key/value latent
  const int n = which ? Rkv : Rq;
  const TIN* src = down + (size_t)t * row_stride + (which ? Rq : 0);
  const float* gain = which ? kv_gain : q_gain;
  TA* dst = (which ? c : cq) + (size_t)t * n;
  pdl_wait();
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    const float v = la_value(src + i, n_split, split_stride);
    ss += v * v;
  }
  const float rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
  for (int i = threadIdx.x; i < n; i += blockDim.x)
    dst[i] = from_f32<TA>((la_value(src + i, n_split, split_stride) * rstd) * gain[i]);
}

template <typename TIN, typename TQ, typename TA, typename TC>
__global__ void latent_rope_cache_kernel(const TQ* __restrict__ q, const TQ* __restrict__ kv,
                                         const TIN* __restrict__ down, int n_split, size_t split_stride,
                                         size_t row_stride, int k_rot_off, TA* __restrict__ q_out,
                                         TC* __restrict__ k_cache, TC* __restrict__ v_cache,
                                         const int* __restrict__ block_table, int table_width,
                                         const int* __restrict__ token_seq, const int* __restrict__ token_pos,
                                         const float* __restrict__ cos_t, const float* __restrict__ sin_t, int H,
                                         int D, int R, int Dv, int n_seqs, int n_pages) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x, h = blockIdx.y * LA_WARPS + warp;
  if (h >= H) return;
  const int b = token_seq[t], pos = token_pos[t];
  if (b < 0 || b >= n_seqs || pos < 0 || pos / LLMX_PAGE >= table_width) {
    if (lane == 0) llmx_report(1);
    return;
  }
  const int page = block_table[(size_t)b * table_width + pos / LLMX_PAGE];
  if (page < 0 || page >= n_pages) {
    if (lane == 0) llmx_report(1);
    return;
  }
  const int half = R >> 1, E = R + D;
  const float* cs = cos_t + (size_t)pos * half;
  const float* sn = sin_t + (size_t)pos * half;
  pdl_wait();
  const TQ* qh = q + ((size_t)t * H + h) * E;
  TA* qo = q_out + ((size_t)t * H + h) * E;
  TC* krow = k_cache + cache_row_offset(page, h, pos % LLMX_PAGE, H, E);
  TC* vrow = v_cache + cache_row_offset(page, h, pos % LLMX_PAGE, H, Dv);
  const TIN* kr = down + (size_t)t * row_stride + k_rot_off;
  for (int i = lane; i < half; i += 32) {
    const float c = cs[i], s = sn[i];
    const float a = to_f32(qh[i]), bq = to_f32(qh[i + half]);
    qo[i] = from_f32<TA>(a * c - bq * s);
    qo[i + half] = from_f32<TA>(bq * c + a * s);
    const float ka = la_value(kr + i, n_split, split_stride), kb = la_value(kr + i + half, n_split, split_stride);
    krow[i] = from_f32<TC>(ka * c - kb * s);
    krow[i + half] = from_f32<TC>(kb * c + ka * s);
  }
  const TQ* kp = kv + (size_t)t * ((size_t)H * (D + Dv)) + (size_t)h * D;
  for (int i = lane; i < D; i += 32) {
    qo[R + i] = from_f32<TA>(to_f32(qh[R + i]));
    krow[R + i] = from_f32<TC>(to_f32(kp[i]));
  }
  const TQ* vp = kv + (size_t)t * ((size_t)H * (D + Dv)) + (size_t)H * D + (size_t)h * Dv;
  for (int i = lane; i < Dv; i += 32) vrow[i] = from_f32<TC>(to_f32(vp[i]));
}

// out[t, h, :] *= sigmoid(gate[t * gate_stride + h]): the heads' output gate behind an attention kernel that has none.
// A thread takes V consecutive values of one head (16 bytes where Dv and the address allow it).
template <typename TA, int V>
__global__ void head_gate_kernel(TA* __restrict__ out, const float* __restrict__ gate, size_t gate_stride, int H, int Dv,
                                 size_t n_units) {
  pdl_launch_dependents();
  pdl_wait();
  const int per_head = Dv / V;
  for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n_units; i += (size_t)gridDim.x * blockDim.x) {
    const size_t th = i / per_head;                       // token * H + head
    const float z = gate[(th / H) * gate_stride + th % H];
    const float g = 1.0f / (1.0f + expf(-z));
    TA* p = out + i * V;
    if (V == 1) {
      p[0] = from_f32<TA>(to_f32(p[0]) * g);
    } else {
      uint4 raw = *reinterpret_cast<const uint4*>(p);
      if (sizeof(TA) == 2) {
        __nv_bfloat162* h2 = reinterpret_cast<__nv_bfloat162*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          const float2 f = __bfloat1622float2(h2[e]);
          h2[e] = __floats2bfloat162_rn(f.x * g, f.y * g);
        }
      } else {
        float* f = reinterpret_cast<float*>(&raw);
#pragma unroll
        for (int e = 0; e < 4; ++e) f[e] *= g;
      }
      *reinterpret_cast<uint4*>(p) = raw;
    }
  }
}

LLMX_API int llmx_head_gate(void* out, int dtype, const float* gate, long long gate_stride, int n_tokens, int H, int Dv,
                            cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || Dv <= 0 || gate_stride < H || !gate || (dtype != LLMX_F32 && dtype != LLMX_BF16)) return LLMX_REFUSED(1);
  const int v = dtype == LLMX_BF16 ? 8 : 4;
  const bool vec = Dv % v == 0 && !((uintptr_t)out & 15);
  const size_t n = (size_t)n_tokens * H * Dv / (vec ? v : 1);
  const size_t want = (n + 255) / 256;
  dim3 grid((unsigned)(want < 148 * 16 ? want : 148 * 16));
#define GO(TA, V) \
  launch_pdl(head_gate_kernel<TA, V>, grid, dim3(256), 0, stream, (TA*)out, gate, (size_t)gate_stride, H, Dv, n)
  if (dtype == LLMX_F32) {
    if (vec) GO(float, 4); else GO(float, 1);
  } else {
    if (vec) GO(bf16, 8); else GO(bf16, 1);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}

// down: [T, row_stride] float32 or bfloat16, or n_split float32 partials split_stride elements apart.
LLMX_API int llmx_latent_norms(const void* down, int in_dtype, int n_split, long long split_stride,
                               long long row_stride, const float* q_gain, const float* kv_gain, float eps, void* cq,
                               void* c, int act_dtype, int n_tokens, int Rq, int Rkv, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (Rq <= 0 || Rkv <= 0 || n_split < 1 || row_stride < Rq + Rkv || !q_gain || !kv_gain) return LLMX_REFUSED(1);
  dim3 grid(n_tokens, 2);
#define CASE(TIN, TA)                                                                                          \
  launch_pdl(latent_norms_kernel<TIN, TA>, grid, dim3(128), 0, stream, (const TIN*)down, n_split,               \
             (size_t)split_stride, (size_t)row_stride, q_gain, kv_gain, eps, (TA*)cq, (TA*)c, Rq, Rkv)
  if (in_dtype == LLMX_F32 && act_dtype == LLMX_F32) CASE(float, float);
  else if (in_dtype == LLMX_F32 && act_dtype == LLMX_BF16) CASE(float, bf16);
  else if (in_dtype == LLMX_BF16 && act_dtype == LLMX_BF16) CASE(bf16, bf16);
  else return LLMX_REFUSED(2);
#undef CASE
  return LLMX_LAUNCH_STATUS();
}

// q [T, H*(R+D)] and kv [T, H*D + H*Dv] in the compute dtype (or float32); the caches [pages, H, PAGE, R+D] and
// [pages, H, PAGE, Dv].
LLMX_API int llmx_latent_rope_cache(const void* q, const void* kv, int q_dtype, const void* down, int in_dtype,
                                    int n_split, long long split_stride, long long row_stride, int k_rot_off,
                                    void* q_out, int act_dtype, void* k_cache, void* v_cache, int cache_dtype,
                                    const int* block_table, int table_width, const int* token_seq,
                                    const int* token_pos, const float* cos_t, const float* sin_t, int n_tokens, int H,
                                    int D, int R, int Dv, int n_seqs, long long n_pages, cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || D < 0 || R <= 0 || (R & 1) || Dv <= 0 || n_split < 1 || k_rot_off < 0 || row_stride < k_rot_off + R)
    return LLMX_REFUSED(1);
  if (!cos_t || !sin_t) return LLMX_REFUSED(4);
  dim3 grid(n_tokens, (H + LA_WARPS - 1) / LA_WARPS);
#define CASE(TIN, TQ, TA, TC)                                                                                    \
  launch_pdl(latent_rope_cache_kernel<TIN, TQ, TA, TC>, grid, dim3(LA_WARPS * 32), 0, stream, (const TQ*)q,      \
             (const TQ*)kv, (const TIN*)down, n_split, (size_t)split_stride, (size_t)row_stride, k_rot_off,       \
             (TA*)q_out, (TC*)k_cache, (TC*)v_cache, block_table, table_width, token_seq, token_pos, cos_t, sin_t, \
             H, D, R, Dv, n_seqs, (int)n_pages)
  const int key = in_dtype * 8 + q_dtype * 4 + act_dtype * 2 + cache_dtype;
  switch (key) {
    case 0: CASE(float, float, float, float); break;      // everything float32
    case 3: CASE(float, float, bf16, bf16); break;
    case 7: CASE(float, bf16, bf16, bf16); break;
    case 15: CASE(bf16, bf16, bf16, bf16); break;
    default: return LLMX_REFUSED(2);
  }
#undef CASE
  return LLMX_LAUNCH_STATUS();
}
