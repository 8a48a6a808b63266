// A sublayer's result normed before it joins the residual stream, the residual add, and the norm that the next
// sublayer reads, in one pass over a row ("sandwich" blocks: x <- x + norm_b(f(norm_a(x)))).
//
// For output row r (source row t = rows ? rows[r] : r):
//   y = w0 * sum_s delta0[s][t,:] (+ w1 * sum_s delta1[s][t,:]) (+ bias)
//                                                     partials added in the order s = 0..S-1; a second group of
//                                                     partials is what a second mixer beside the first returned
//   y = y * sigmoid(z[t,:] + zb)                      when a gate z is given (z: partials added in order like a group's)
//   y = norm(y) * post_gain                           when post_gain is given (else y joins as it is)
//   v = h[t,:] + y;  h[t,:] = v when write_h
//   out[r,:] = norm(v) * gain                         when out is given
// Either norm is a layer norm without bias, (x - mean) / sqrt(mean((x - mean)^2) + eps), or an RMS norm,
// x / sqrt(mean(x^2) + eps); the two norms choose independently (`post_center`, `center`).  Everything is float32;
// mean and variance are taken in two passes over the row, which is held in registers (rows of up to 8192 aligned
// floats) or staged in shared memory.  The thread count and each thread's elements depend on d (and the pointers'
// alignment) alone, so a row's sums do not depend on the batch.
#include "common.cuh"

__device__ __forceinline__ float4 pn_load4(const float* p) { return *reinterpret_cast<const float4*>(p); }
__device__ __forceinline__ float4 pn_load4(const bf16* p) {
  const uint2 raw = *reinterpret_cast<const uint2*>(p);
  const float2 a = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
  const float2 b = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
  return make_float4(a.x, a.y, b.x, b.y);
}
__device__ __forceinline__ void pn_store4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void pn_store4(bf16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  uint2 raw;
  raw.x = *reinterpret_cast<uint32_t*>(&a);
  raw.y = *reinterpret_cast<uint32_t*>(&b);
  *reinterpret_cast<uint2*>(p) = raw;
}

// 1 / sqrt(variance + eps) and the mean of the staged row (mean 0 for an RMS norm)
__device__ __forceinline__ void pn_stats(const float* row, int d, bool center, float eps, float* red, float& mean,
                                         float& rstd) {
  mean = 0.f;
  if (center) {
    float s = 0.f;
    for (int i = threadIdx.x; i < d; i += blockDim.x) s += row[i];
    mean = block_sum(s, red) / (float)d;
  }
  float ss = 0.f;
  for (int i = threadIdx.x; i < d; i += blockDim.x) {
    const float c = row[i] - mean;
    ss += c * c;
  }
  rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
}

// One group of partials: n_split tensors [T, d] of float32 or bfloat16, `stride` elements apart, times `weight`.
struct PnGroup {
  const void* p;
  int n_split, is_bf16;
  size_t stride;
  float weight;
};
__device__ __forceinline__ float4 pn_group4(const PnGroup& g, size_t at) {
  float4 y = g.is_bf16 ? pn_load4((const bf16*)g.p + at) : pn_load4((const float*)g.p + at);
  for (int s = 1; s < g.n_split; ++s) {
    const size_t o = at + (size_t)s * g.stride;
    const float4 q = g.is_bf16 ? pn_load4((const bf16*)g.p + o) : pn_load4((const float*)g.p + o);
    y.x += q.x, y.y += q.y, y.z += q.z, y.w += q.w;
  }
  return make_float4(y.x * g.weight, y.y * g.weight, y.z * g.weight, y.w * g.weight);
}
__device__ __forceinline__ float pn_group1(const PnGroup& g, size_t at) {
  float y = g.is_bf16 ? to_f32(((const bf16*)g.p)[at]) : ((const float*)g.p)[at];
  for (int s = 1; s < g.n_split; ++s) {
    const size_t o = at + (size_t)s * g.stride;
    y += g.is_bf16 ? to_f32(((const bf16*)g.p)[o]) : ((const float*)g.p)[o];
  }
  return y * g.weight;
}

// The gate on a result: y * sigmoid(z + zb), z a group of partials with weight 1, zb float32 [d] or null.
__device__ __forceinline__ float pn_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float4 pn_gated4(float4 y, const PnGroup& gz, const float* zb, size_t at, int col) {
  float4 z = pn_group4(gz, at);
  if (zb) {
    const float4 b = pn_load4(zb + col);
    z.x += b.x, z.y += b.y, z.z += b.z, z.w += b.w;
  }
  return make_float4(y.x * pn_sigmoid(z.x), y.y * pn_sigmoid(z.y), y.z * pn_sigmoid(z.z), y.w * pn_sigmoid(z.w));
}
__device__ __forceinline__ float pn_gated1(float y, const PnGroup& gz, const float* zb, size_t at, int col) {
  float z = pn_group1(gz, at);
  if (zb) z += zb[col];
  return y * pn_sigmoid(z);
}

template <typename TO, bool VEC>
__global__ void __launch_bounds__(512)
post_norm_add_norm_kernel(float* __restrict__ h, const PnGroup g0, const PnGroup g1, const PnGroup gz,
                          const float* __restrict__ zb, const float* __restrict__ bias, const float* __restrict__ post_gain, int post_center,
                          float post_eps, const int* __restrict__ rows, const float* __restrict__ gain, int center,
                          float eps, TO* __restrict__ out, int d, int write_h) {
  extern __shared__ __align__(16) float pn_row[];       // [d]
  __shared__ float red[32];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;                     // a step input, not a result of the kernel before
  float* hrow = h + (size_t)t * d;
  pdl_wait();
  if (g0.p) {
    const size_t at0 = (size_t)t * d;
    if (VEC) {
      for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        float4 y = pn_group4(g0, at0 + i);
        if (g1.p) {
          const float4 z = pn_group4(g1, at0 + i);
          y.x += z.x, y.y += z.y, y.z += z.z, y.w += z.w;
        }
        if (bias) {
          const float4 b = pn_load4(bias + i);
          y.x += b.x, y.y += b.y, y.z += b.z, y.w += b.w;
        }
        if (gz.p) y = pn_gated4(y, gz, zb, at0 + i, i);
        pn_store4(pn_row + i, y);
      }
    } else {
      for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float y = pn_group1(g0, at0 + i);
        if (g1.p) y += pn_group1(g1, at0 + i);
        if (bias) y += bias[i];
        if (gz.p) y = pn_gated1(y, gz, zb, at0 + i, i);
        pn_row[i] = y;
      }
    }
    __syncthreads();
    float mean = 0.f, rstd = 1.f;
    if (post_gain) pn_stats(pn_row, d, post_center != 0, post_eps, red, mean, rstd);
    // every thread takes the columns it staged itself: no barrier between the two uses of the row
    if (VEC) {
      for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
        float4 y = pn_load4(pn_row + i);
        if (post_gain) {
          const float4 g = pn_load4(post_gain + i);
          y.x = ((y.x - mean) * rstd) * g.x, y.y = ((y.y - mean) * rstd) * g.y;
          y.z = ((y.z - mean) * rstd) * g.z, y.w = ((y.w - mean) * rstd) * g.w;
        }
        const float4 x = pn_load4(hrow + i);
        const float4 v = make_float4(x.x + y.x, x.y + y.y, x.z + y.z, x.w + y.w);
        if (write_h) pn_store4(hrow + i, v);
        pn_store4(pn_row + i, v);
      }
    } else {
      for (int i = threadIdx.x; i < d; i += blockDim.x) {
        float y = pn_row[i];
        if (post_gain) y = ((y - mean) * rstd) * post_gain[i];
        const float v = hrow[i] + y;
        if (write_h) hrow[i] = v;
        pn_row[i] = v;
      }
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) pn_row[i] = hrow[i];
  }
  if (!out) return;
  __syncthreads();
  float mean, rstd;
  pn_stats(pn_row, d, center != 0, eps, red, mean, rstd);
  TO* orow = out + (size_t)r * d;
  if (VEC) {
    for (int i = threadIdx.x * 4; i < d; i += blockDim.x * 4) {
      const float4 v = pn_load4(pn_row + i), g = pn_load4(gain + i);
      pn_store4(orow + i, make_float4(((v.x - mean) * rstd) * g.x, ((v.y - mean) * rstd) * g.y,
                                      ((v.z - mean) * rstd) * g.z, ((v.w - mean) * rstd) * g.w));
    }
  } else {
    for (int i = threadIdx.x; i < d; i += blockDim.x) orow[i] = from_f32<TO>(((pn_row[i] - mean) * rstd) * gain[i]);
  }
}

// The same for rows of up to 16 floats a thread (d <= 8192, everything 16-byte aligned): the row stays in registers.
// Thread j owns the float4s j, j + T, .., j + (NV - 1) T of the row; NV and T depend on d alone (8 floats a thread
// up to d = 4096: more of them make the block-wide sums cheaper for a prompt's rows but a decode step's few rows
// slower).  Mean and variance are still two passes (over registers).
template <int NV>
__device__ __forceinline__ void pn_stats_reg(const float4 (&v)[NV], const bool (&live)[NV], int d, bool center,
                                             float eps, float* red, float& mean, float& rstd) {
  mean = 0.f;
  if (center) {
    float s = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k)
      if (live[k]) s += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    mean = block_sum(s, red) / (float)d;
  }
  float ss = 0.f;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (live[k]) {
      const float a = v[k].x - mean, b = v[k].y - mean, c = v[k].z - mean, e = v[k].w - mean;
      ss += (a * a + b * b) + (c * c + e * e);
    }
  rstd = 1.0f / sqrtf(block_sum(ss, red) / (float)d + eps);
}

template <typename TO, int NV>
__global__ void __launch_bounds__(512)
post_norm_add_norm_reg_kernel(float* __restrict__ h, const PnGroup g0, const PnGroup g1, const PnGroup gz,
                              const float* __restrict__ zb, const float* __restrict__ bias, const float* __restrict__ post_gain, int post_center,
                              float post_eps, const int* __restrict__ rows, const float* __restrict__ gain, int center,
                              float eps, TO* __restrict__ out, int d, int write_h) {
  __shared__ float red[32];
  pdl_launch_dependents();
  const int r = blockIdx.x;
  const int t = rows ? rows[r] : r;                     // a step input, not a result of the kernel before
  float* hrow = h + (size_t)t * d;
  const int n4 = d >> 2;
  float4 v[NV];
  bool live[NV];
  int col[NV];
#pragma unroll
  for (int k = 0; k < NV; ++k) {
    const int j = threadIdx.x + k * blockDim.x;
    live[k] = j < n4;
    col[k] = j * 4;
  }
  pdl_wait();
  if (g0.p) {
    const size_t at0 = (size_t)t * d;
    float4 x[NV];
#pragma unroll
    for (int k = 0; k < NV; ++k) x[k] = live[k] ? pn_load4(hrow + col[k]) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      float4 y = make_float4(0.f, 0.f, 0.f, 0.f);
      if (live[k]) {
        y = pn_group4(g0, at0 + col[k]);
        if (g1.p) {
          const float4 z = pn_group4(g1, at0 + col[k]);
          y.x += z.x, y.y += z.y, y.z += z.z, y.w += z.w;
        }
        if (bias) {
          const float4 b = pn_load4(bias + col[k]);
          y.x += b.x, y.y += b.y, y.z += b.z, y.w += b.w;
        }
        if (gz.p) y = pn_gated4(y, gz, zb, at0 + col[k], col[k]);
      }
      v[k] = y;
    }
    if (post_gain) {
      float mean, rstd;
      pn_stats_reg<NV>(v, live, d, post_center != 0, post_eps, red, mean, rstd);
#pragma unroll
      for (int k = 0; k < NV; ++k)
        if (live[k]) {
          const float4 g = pn_load4(post_gain + col[k]);
          v[k].x = ((v[k].x - mean) * rstd) * g.x, v[k].y = ((v[k].y - mean) * rstd) * g.y;
          v[k].z = ((v[k].z - mean) * rstd) * g.z, v[k].w = ((v[k].w - mean) * rstd) * g.w;
        }
    }
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      v[k] = make_float4(x[k].x + v[k].x, x[k].y + v[k].y, x[k].z + v[k].z, x[k].w + v[k].w);
      if (write_h && live[k]) pn_store4(hrow + col[k], v[k]);
    }
  } else {
#pragma unroll
    for (int k = 0; k < NV; ++k) v[k] = live[k] ? pn_load4(hrow + col[k]) : make_float4(0.f, 0.f, 0.f, 0.f);
  }
  if (!out) return;
  float mean, rstd;
  pn_stats_reg<NV>(v, live, d, center != 0, eps, red, mean, rstd);
  TO* orow = out + (size_t)r * d;
#pragma unroll
  for (int k = 0; k < NV; ++k)
    if (live[k]) {
      const float4 g = pn_load4(gain + col[k]);
      pn_store4(orow + col[k], make_float4(((v[k].x - mean) * rstd) * g.x, ((v[k].y - mean) * rstd) * g.y,
                                           ((v[k].z - mean) * rstd) * g.z, ((v[k].w - mean) * rstd) * g.w));
    }
}

// h float32 [T, d]; delta0 / delta1: null, or n_split partials [T, d] split_stride elements apart, each group
// times its weight (delta1 only beside delta0); bias, post_gain, gain: float32 [d] or null; rows: int32 [n_rows]
// or null (every row of h); out: [n_rows, d] or null.
// gate: null, or n_split partials [T, d] whose sum (+ gate_bias, float32 [d] or null) is the logit of the gate on y.
LLMX_API int llmx_post_norm_add_norm_gated(float* h, const void* delta0, int dtype0, int n_split0, long long stride0,
                                     float weight0, const void* delta1, int dtype1, int n_split1, long long stride1,
                                     float weight1, const float* bias, const float* post_gain, int post_center,
                                     float post_eps, const int* rows, int n_rows, const float* gain, int center,
                                     float eps, void* out, int out_dtype, int d, int write_h, const void* gate,
                                     int gate_dtype, int gate_split, long long gate_stride, const float* gate_bias,
                                     cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (gate && (!delta0 || gate_split < 1 || (gate_dtype != LLMX_F32 && gate_dtype != LLMX_BF16))) return LLMX_REFUSED(1);
  const PnGroup gz = {gate, gate_split, gate_dtype == LLMX_BF16, (size_t)gate_stride, 1.0f};
  const float* zb = gate ? gate_bias : nullptr;
  if (d <= 0 || (delta0 && n_split0 < 1) || (delta1 && (n_split1 < 1 || !delta0)) || (out && !gain))
    return LLMX_REFUSED(1);
  if ((delta0 && dtype0 != LLMX_F32 && dtype0 != LLMX_BF16) || (delta1 && dtype1 != LLMX_F32 && dtype1 != LLMX_BF16))
    return LLMX_REFUSED(2);
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return LLMX_REFUSED(3);
  const PnGroup g0 = {delta0, n_split0, dtype0 == LLMX_BF16, (size_t)stride0, weight0};
  const PnGroup g1 = {delta1, n_split1, dtype1 == LLMX_BF16, (size_t)stride1, weight1};
  auto aligned = [](const PnGroup& g) {
    const int esz = g.is_bf16 ? 2 : 4;
    return !g.p || (!((uintptr_t)g.p & (4 * esz - 1)) && g.stride % 4 == 0);
  };
  const int osz = out_dtype == LLMX_F32 ? 4 : 2;
  const bool vec = d % 4 == 0 && !((uintptr_t)h & 15) && aligned(g0) && aligned(g1) && aligned(gz) &&
                   !((uintptr_t)zb & 15) && !((uintptr_t)bias & 15) &&
                   !((uintptr_t)post_gain & 15) && !((uintptr_t)gain & 15) && !((uintptr_t)out & (4 * osz - 1));
  int threads = ((d + 3) / 4 + 31) / 32 * 32;
  threads = threads < 64 ? 64 : threads > 512 ? 512 : threads;
#define GO(TO, VEC)                                                                                                      \
  do {                                                                                                                   \
    if (smem > 48 * 1024) {                                                                                              \
      cudaError_t e = cudaFuncSetAttribute(post_norm_add_norm_kernel<TO, VEC>,                                           \
                                           cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);                      \
      if (e != cudaSuccess) return (int)e;                                                                               \
    }                                                                                                                    \
    launch_pdl(post_norm_add_norm_kernel<TO, VEC>, dim3(n_rows), dim3(threads), smem, stream, h, g0, g1, gz, zb, bias,   \
               post_gain, post_center, post_eps, rows, gain, center, eps, (TO*)out, d, write_h);                         \
  } while (0)
  if (out && out_dtype != LLMX_BF16 && out_dtype != LLMX_F32) return LLMX_REFUSED(2);
  const bool out_bf16 = out && out_dtype == LLMX_BF16;
  const int n4 = d / 4;
  if (vec && n4 <= 2048) {                              // the row in registers
    const int nv = n4 > 1024 ? 4 : n4 > 128 ? 2 : 1;
    const int reg_threads = ((n4 + nv - 1) / nv + 31) / 32 * 32;
#define GO_REG(TO, NV)                                                                                                   \
    launch_pdl(post_norm_add_norm_reg_kernel<TO, NV>, dim3(n_rows), dim3(reg_threads), 0, stream, h, g0, g1, gz, zb, bias, \
               post_gain, post_center, post_eps, rows, gain, center, eps, (TO*)out, d, write_h)
    if (out_bf16) {
      if (nv == 4) GO_REG(bf16, 4); else if (nv == 2) GO_REG(bf16, 2); else GO_REG(bf16, 1);
    } else {
      if (nv == 4) GO_REG(float, 4); else if (nv == 2) GO_REG(float, 2); else GO_REG(float, 1);
    }
#undef GO_REG
    return LLMX_LAUNCH_STATUS();
  }
  if (out_bf16) {
    if (vec) GO(bf16, true); else GO(bf16, false);
  } else {
    if (vec) GO(float, true); else GO(float, false);
  }
#undef GO
  return LLMX_LAUNCH_STATUS();
}

LLMX_API int llmx_post_norm_add_norm(float* h, const void* delta0, int dtype0, int n_split0, long long stride0,
                                     float weight0, const void* delta1, int dtype1, int n_split1, long long stride1,
                                     float weight1, const float* bias, const float* post_gain, int post_center,
                                     float post_eps, const int* rows, int n_rows, const float* gain, int center,
                                     float eps, void* out, int out_dtype, int d, int write_h, cudaStream_t stream) {
  return llmx_post_norm_add_norm_gated(h, delta0, dtype0, n_split0, stride0, weight0, delta1, dtype1, n_split1, stride1,
                                       weight1, bias, post_gain, post_center, post_eps, rows, n_rows, gain, center, eps,
                                       out, out_dtype, d, write_h, nullptr, LLMX_F32, 1, 0, nullptr, stream);
}

// y[t, :] += bias for a product's output that no later kernel of this file reads (y: [n_rows, d], float32 or
// bfloat16; the sum is float32).
template <typename TY>
__global__ void add_bias_kernel(TY* __restrict__ y, const float* __restrict__ bias, size_t n, int d) {
  pdl_launch_dependents();
  pdl_wait();
  for (size_t i = blockIdx.x * (size_t)blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x)
    y[i] = from_f32<TY>(to_f32(y[i]) + bias[i % d]);
}

LLMX_API int llmx_add_bias(void* y, int dtype, int n_rows, int d, const float* bias, cudaStream_t stream) {
  if (n_rows <= 0) return 0;
  if (d <= 0 || !bias) return LLMX_REFUSED(1);
  const size_t n = (size_t)n_rows * d;
  const int blocks = (int)((n + 255) / 256 < 148 * 16 ? (n + 255) / 256 : 148 * 16);
  if (dtype == LLMX_F32) launch_pdl(add_bias_kernel<float>, dim3(blocks), dim3(256), 0, stream, (float*)y, bias, n, d);
  else if (dtype == LLMX_BF16) launch_pdl(add_bias_kernel<bf16>, dim3(blocks), dim3(256), 0, stream, (bf16*)y, bias, n, d);
  else return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}
