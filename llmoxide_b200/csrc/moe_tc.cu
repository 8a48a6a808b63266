// The grouped products of the routed experts on the Blackwell tensor cores (tcgen05), bfloat16.
//
// The step's (token, choice) pairs are sorted by expert (moe.cu); `tiles` lists, for every run of up to BN
// sorted rows that lie in one expert's segment, (expert, first row, rows).  A work unit is (tile of 128 rows
// of that expert's matrix, one such tile of rows); as in the plain product the weights are the MMA's M operand
// and the rows of activations its N operand, so a decode step streams every touched expert's weights once and
// a prompt step uses wide row tiles.  Operands come by TMA with the 128-byte swizzle into a ring in shared
// memory: the weights from one map over all experts' rows [E * rows, K], the activations from one map over the
// sorted rows [P, K].  A row tile that ends before BN rows brings rows of the next expert's segment along;
// their columns of the accumulator are never stored.  Accumulators live in tensor memory, two sets where they
// fit, so a unit's epilogue overlaps the next unit's MMAs.  Roles per CTA: one thread issues the copies, one the
// MMAs, four warps read the accumulators back (tcgen05.ld) and finish the unit:
//
//   MODE 1 (gate|up): two accumulators, rows n and n + F of the expert's [2F, K]; act[row, n] = gated_act(gate, up) (common.cuh)
//   MODE 0 (down):    y[dest[row]][n] = weight[row] * acc, float32 (dest = choice * tokens + token, from the sort)
//
// Which expert a unit reads is decided on the device by the kernel before, so every thread waits for that
// kernel first.  Every wait on an mbarrier is bounded; when one runs out the CTA records it in the library's
// status word, stops issuing work, frees its tensor memory and returns.
#include "tc_ptx.cuh"

#define MT_BM 128
#define MT_BK 64
#define MT_UMMA_K 16
#define MT_THREADS 192

__device__ __forceinline__ void mt_report(int code) { llmx_report(code); }

__host__ __device__ constexpr uint32_t mt_idesc(int n) {     // bf16 x bf16 -> f32, both K-major, M = 128
  return (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n >> 3) << 17) | ((uint32_t)(MT_BM >> 4) << 24);
}

template <int BN, int MODE, typename TY>
__global__ void __launch_bounds__(MT_THREADS)
moe_grouped_tc_kernel(const __grid_constant__ CUtensorMap map_w, const __grid_constant__ CUtensorMap map_x,
                      TY* __restrict__ Y, const int* __restrict__ tiles, int max_tiles, const int* __restrict__ dest,
                      const float* __restrict__ sorted_weight, int N, int K, int w_rows, int n_stages, int row_tiles,
                      const GateAct act) {
  extern __shared__ uint8_t smem_raw[];
  constexpr int N_ACC = MODE == 1 ? 2 : 1;
  constexpr uint32_t A_BYTES = MT_BM * MT_BK * 2;
  constexpr uint32_t B_BYTES = BN * MT_BK * 2;
  constexpr uint32_t STAGE_BYTES = N_ACC * A_BYTES + B_BYTES;
  constexpr uint32_t ACC_COLS = N_ACC * BN;
  constexpr int ACC_BUFS = (2 * ACC_COLS <= 512) ? 2 : 1;
  constexpr uint32_t TMEM_COLS = (ACC_BUFS * ACC_COLS) < 32 ? 32 : (ACC_BUFS * ACC_COLS);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n_kb = (K + MT_BK - 1) / MT_BK;
  const uint32_t base = (smem_u32(smem_raw) + 1023u) & ~1023u;
  uint8_t* base_ptr = smem_raw + (base - smem_u32(smem_raw));
  uint64_t* bars = reinterpret_cast<uint64_t*>(base_ptr + (size_t)n_stages * STAGE_BYTES);
  const uint32_t full0 = smem_u32(bars), empty0 = full0 + 8u * n_stages;
  const uint32_t acc_full0 = empty0 + 8u * n_stages, acc_empty0 = acc_full0 + 16u;
  uint32_t* tmem_holder = reinterpret_cast<uint32_t*>(bars + 2 * n_stages + 4);
  int* tile_dest = reinterpret_cast<int*>(bars + 2 * n_stages + 6);          // [BN] MODE 0: the unit's output rows
  float* tile_weight = reinterpret_cast<float*>(tile_dest + BN);            // [BN] and their weights
  volatile int* gave_up = reinterpret_cast<volatile int*>(tile_weight + BN); // an epilogue warp's wait ran out: all four leave

  pdl_launch_dependents();
  if (threadIdx.x == 0) {
    *gave_up = 0;
    for (int s = 0; s < n_stages; ++s) {
      mbar_init(full0 + 8u * s, 1);
      mbar_init(empty0 + 8u * s, 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(acc_full0 + 8u * i, 1);
      mbar_init(acc_empty0 + 8u * i, 4);      // one arrival per epilogue warp
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_w) : "memory");
    asm volatile("prefetch.tensormap [%0];" ::"l"(&map_x) : "memory");
  }
  if (warp == 1) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_holder)),
                 "r"(TMEM_COLS)
                 : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_holder;
  pdl_wait();                    // the tile list, the sorted rows and the weights of the pairs come from the kernels before

  // Unit u = tile (u / row_tiles) x row tile (u % row_tiles).  The used tiles come first in the list, so a CTA
  // is done at the first unused one; every role walks the same units.
  const int n_units = max_tiles * row_tiles;
  auto unit = [&](int u, int& e, int& row0, int& n_rows, int& n0) {
    const int tl = u / row_tiles;
    e = __ldcg(tiles + 3 * tl);
    row0 = __ldcg(tiles + 3 * tl + 1);
    n_rows = __ldcg(tiles + 3 * tl + 2);
    n0 = (u - tl * row_tiles) * MT_BM;
    return e >= 0;
  };

  if (warp == 0) {
    // ---------------- producer ----------------
    if (lane == 0) {
      RingPos pos{0, 0};
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x) {
        int e, row0, n_rows, n0;
        if (!unit(u, e, row0, n_rows, n0)) break;
        const int wrow = e * w_rows + n0;
        for (int i = 0; i < n_kb; ++i, pos.next(n_stages)) {
          const int s = pos.s;
          if (!mbar_wait(empty0 + 8u * s, pos.phase ^ 1u)) { mt_report(1); ok = false; break; }
          const uint32_t stage = base + (uint32_t)s * STAGE_BYTES, bar = full0 + 8u * s;
          mbar_expect_tx(bar, STAGE_BYTES);
          const int k = i * MT_BK;
          tma_load_2d(stage, &map_w, k, wrow, bar);
          if (MODE == 1) tma_load_2d(stage + A_BYTES, &map_w, k, wrow + N, bar);     // the up rows: N = F
          tma_load_2d(stage + N_ACC * A_BYTES, &map_x, k, row0, bar);
        }
      }
    }
  } else if (warp == 1) {
    // ---------------- MMA issuer ----------------
    if (lane == 0) {
      constexpr uint32_t idesc = mt_idesc(BN);
      int j = 0;
      RingPos pos{0, 0};
      const uint32_t desc0 = umma_desc_lo(base);
      bool ok = true;
      for (int u = blockIdx.x; u < n_units && ok; u += gridDim.x, ++j) {
        int e, row0, n_rows, n0;
        if (!unit(u, e, row0, n_rows, n0)) break;
        const int buf = j % ACC_BUFS, use = j / ACC_BUFS;
        const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS;
        if (!mbar_wait(acc_empty0 + 8u * buf, (use & 1) ^ 1)) { mt_report(4); ok = false; break; }
        tc_fence_after();
        for (int i = 0; i < n_kb; ++i, pos.next(n_stages)) {
          const int s = pos.s;
          if (!mbar_wait(full0 + 8u * s, pos.phase)) { mt_report(2); ok = false; break; }
          tc_fence_after();
          const uint32_t da = desc0 + (uint32_t)s * (STAGE_BYTES >> 4);
#pragma unroll
          for (int kk = 0; kk < MT_BK / MT_UMMA_K; ++kk) {
            const uint32_t db = da + ((N_ACC * A_BYTES) >> 4) + kk * ((MT_UMMA_K * 2) >> 4);
            const uint32_t acc = (i > 0 || kk > 0) ? 1u : 0u;
            umma_bf16_lo(acc_addr, da + kk * ((MT_UMMA_K * 2) >> 4), db, idesc, acc);
            if (MODE == 1)
              umma_bf16_lo(acc_addr + BN, da + (A_BYTES >> 4) + kk * ((MT_UMMA_K * 2) >> 4), db, idesc, acc);
          }
          umma_commit(empty0 + 8u * s);
        }
        if (!(j == 0 && llmx_withhold)) umma_commit(acc_full0 + 8u * buf);
      }
    }
  } else {
    // ---------------- epilogue ----------------
    const int quad = warp & 3;
    bool failed = false;
    int j = 0;
    for (int u = blockIdx.x; u < n_units; u += gridDim.x, ++j) {
      int e, row0, n_rows, n0;
      if (!unit(u, e, row0, n_rows, n0)) break;
      const int buf = j % ACC_BUFS, use = j / ACC_BUFS;
      if (MODE == 0) {
        // where the unit's rows go and what they weigh: one coalesced load, shared by the four warps
        asm volatile("bar.sync 1, 128;" ::: "memory");     // (the unit before has been stored)
        const int r = (int)threadIdx.x - 64;
        if (r < BN && r < n_rows) {
          tile_dest[r] = __ldcg(dest + row0 + r);
          tile_weight[r] = __ldcg(sorted_weight + row0 + r);
        }
      }
      bool ok = mbar_wait(acc_full0 + 8u * buf, use & 1);
      if (!ok && lane == 0) {
        mt_report(3);
        *gave_up = 1;
      }
      if (MODE == 0) {
        asm volatile("bar.sync 1, 128;" ::: "memory");     // the rows' list is in place, and so is any warp's failure
        failed = *gave_up != 0;
      } else {
        failed = __shfl_sync(0xffffffffu, ok ? 0 : 1, 0) != 0;
      }
      if (failed) break;
      tc_fence_after();
      const uint32_t acc_addr = tmem_base + (uint32_t)buf * ACC_COLS + ((uint32_t)(quad * 32) << 16);
      const int n = n0 + quad * 32 + lane;                 // this lane's row of the expert's matrix = output feature
#pragma unroll 1
      for (int c = 0; c < BN; c += 16) {
        if (c >= n_rows) break;
        float v[16], g[16];
        tmem_ld16(acc_addr + (uint32_t)c, v);
        if (MODE == 1) tmem_ld16(acc_addr + (uint32_t)(BN + c), g);
        if (n < N) {
#pragma unroll
          for (int i = 0; i < 16; ++i) {
            const int r = c + i;
            if (r >= n_rows) break;
            if (MODE == 1) {
              Y[(size_t)(row0 + r) * N + n] = from_f32<TY>(gated_act_fast(act, v[i], g[i]));
            } else {
              Y[(size_t)tile_dest[r] * N + n] = from_f32<TY>(tile_weight[r] * v[i]);
            }
          }
        }
      }
      tc_fence_before();
      __syncwarp();
      if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(acc_empty0 + 8u * buf) : "memory");
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(TMEM_COLS) : "memory");
  }
}

static int mt_sm_count() {
  static int n = 0;
  if (!n) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
      n = 148;
  }
  return n;
}

template <int BN, int MODE, typename TY>
static int mt_launch(const CUtensorMap& mw, const CUtensorMap& mx, void* Y, const int* tiles, int max_tiles, const int* dest,
                     const float* sorted_weight, int N, int K, int w_rows, const GateAct act, cudaStream_t stream) {
  constexpr int N_ACC = MODE == 1 ? 2 : 1;
  constexpr size_t STAGE = (size_t)N_ACC * MT_BM * MT_BK * 2 + (size_t)BN * MT_BK * 2;
  const int row_tiles = (N + MT_BM - 1) / MT_BM;
  const long long n_units = (long long)row_tiles * max_tiles;
  if (n_units > 0x7fffffff) return LLMX_REFUSED(3);
  // narrow row tiles stream weights: two CTAs per SM keep more loads in flight; wide ones take the whole SM
  const int ctas_per_sm = BN <= 64 ? 2 : 1;
  const size_t budget = ctas_per_sm == 2 ? 108 * 1024 : 200 * 1024;
  int stages = (int)(budget / STAGE);
  if (stages > 12) stages = 12;
  if (stages < 2) stages = 2;
  const size_t smem = 1024 + (size_t)stages * STAGE + (2 * stages + 6) * 8 + (size_t)BN * 8 + 16;
  auto kernel = moe_grouped_tc_kernel<BN, MODE, TY>;
  static bool attr_set = false;
  if (!attr_set) {
    cudaError_t e = cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 227 * 1024);
    if (e != cudaSuccess) return (int)e;
    attr_set = true;
  }
  const int max_ctas = mt_sm_count() * ctas_per_sm;
  const int grid = n_units < max_ctas ? (int)n_units : max_ctas;
  launch_pdl(kernel, dim3(grid), dim3(MT_THREADS), smem, stream, mw, mx, (TY*)Y, tiles, max_tiles, dest, sorted_weight, N, K,
             w_rows, stages, row_tiles, act);
  return LLMX_LAUNCH_STATUS();
}

// X: bf16 sorted rows [P, K] (row stride ldx); W: bf16 [E, w_rows, K] contiguous, w_rows = 2N when gated (gate rows,
// then up rows) else N; tiles: int32 [max_tiles, 3] made with tile_rows rows per tile (16, 64 or 128).
// gated: Y = act bf16 [P, N].  else: Y = float32 rows of N, row dest[place] = sorted_weight[place] * product
// (dest and sorted_weight [P] in sorted order, from the sort).
LLMX_API int llmx_moe_grouped_tc(const void* X, long long ldx, long long P, const void* W, int n_experts, void* Y,
                                 const int* tiles, int max_tiles, int tile_rows, const int* dest,
                                 const float* sorted_weight, int N, int K, int gated, int act_kind, float slope, float limit,
                                 float shift, cudaStream_t stream) {
  if (P <= 0) return 0;
  if (act_kind < LLMX_ACT_SILU || act_kind > LLMX_ACT_LAST) return LLMX_REFUSED(1);
  const GateAct act = {act_kind, slope, limit, shift};
  if (N <= 0 || K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)X & 15) || ((uintptr_t)W & 15) || max_tiles <= 0 ||
      n_experts <= 0 || (!gated && (!dest || !sorted_weight)))
    return LLMX_REFUSED(1);
  const int w_rows = gated ? 2 * N : N;
  CUtensorMap mw, mx;
  if (make_map(&mw, W, (uint64_t)n_experts * w_rows, (uint64_t)K, (uint64_t)K, MT_BM, true)) return LLMX_REFUSED(4);
  if (make_map(&mx, X, (uint64_t)P, (uint64_t)K, (uint64_t)ldx, (uint32_t)tile_rows, false)) return LLMX_REFUSED(4);
#define GO(BN)                                                                                                      \
  return gated ? mt_launch<BN, 1, bf16>(mw, mx, Y, tiles, max_tiles, dest, sorted_weight, N, K, w_rows, act, stream) \
               : mt_launch<BN, 0, float>(mw, mx, Y, tiles, max_tiles, dest, sorted_weight, N, K, w_rows, act, stream)
  switch (tile_rows) {
    case 16: GO(16);
    case 64: GO(64);
    case 128: GO(128);
    default: return LLMX_REFUSED(1);
  }
#undef GO
}

// Sorted rows of x: xs[place] = x[perm[place] / top] (bfloat16, 16 bytes per thread and step).
__global__ void moe_gather_rows_kernel(const bf16* __restrict__ x, long long ldx, const int* __restrict__ perm, int top,
                                       bf16* __restrict__ xs, int K) {
  pdl_launch_dependents();
  pdl_wait();
  const int place = blockIdx.x;
  const bf16* src = x + (size_t)(perm[place] / top) * ldx;
  bf16* dst = xs + (size_t)place * K;
  for (int i = threadIdx.x * 8; i < K; i += blockDim.x * 8)
    *reinterpret_cast<uint4*>(dst + i) = *reinterpret_cast<const uint4*>(src + i);
}

LLMX_API int llmx_moe_gather_rows(const void* x, long long ldx, const int* perm, int top, void* xs, int P, int K,
                                  cudaStream_t stream) {
  if (P <= 0) return 0;
  if (K <= 0 || (K % 8) || (ldx % 8) || ((uintptr_t)x & 15) || ((uintptr_t)xs & 15)) return LLMX_REFUSED(1);
  int threads = 32;
  while (threads < 256 && threads * 8 < K) threads <<= 1;
  launch_pdl(moe_gather_rows_kernel, dim3(P), dim3(threads), 0, stream, (const bf16*)x, ldx, perm, top, (bf16*)xs, K);
  return LLMX_LAUNCH_STATUS();
}
