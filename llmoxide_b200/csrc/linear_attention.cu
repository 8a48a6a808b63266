// Linear attention with a fixed decay per head (no softmax, no denominator), as a recurrence over a
// per-sequence state, and the normalisation and gate that follow it.
//
//   S_t = decay_h * S_{t-1} + k_t v_t^T        S: [D, Dv] per (sequence, head), float32, kept from step to step
//   o_t = S_t^T q_t
//
// q, k and v come out of one fused projection (a row holds q heads, k heads, v heads and the gate's columns).
// What the design does to them before the recurrence is done by a kernel of its own, once per (token, head):
// an activation (none or SiLU), the rotation of q and k (pairs (i, i + n_rot/2) of a head's first n_rot dims,
// angle from float32 tables), a scale on k.  All of it, the state and the sums are float32.
//
// The recurrence is independent for every column of v, so a CTA owns `cols` columns of one (sequence, head)
// and walks that sequence's tokens of the step in order.  Within a CTA a warp owns 4 columns; the 8 lanes of
// a column split D among them in blocks of 4 dims (lane r owns dims 4 (r + 8 i) + 0..3), update their part of
// S and add up q . S with three shuffles.  The order of every addition is fixed by (d, column) alone, and a
// token's update is the same arithmetic whether it arrives in a prompt, in a later portion of one or alone, so
// a position's result does not depend on how tokens were cut into steps or batched, to the last bit.
//
// The same kernels run a recurrence whose decay and input weight change from token to token (the matrix memory
// of an mLSTM layer, GATED below):
//
//   m_t = max(f_t + m_{t-1}, i_t)                            f, i: log forget and log input gate; m starts at 0
//   S_t = a_t S_{t-1} + b_t k_t v_t^T,  a_t = exp(f_t + m_{t-1} - m_t),  b_t = exp(i_t - m_t)
//   n_t = a_t n_{t-1} + b_t k_t
//   o_t = S_t^T q_t / (max(|n_t . q_t|, exp(-m_t)) + den_eps)
//
// n is carried as one more column of S whose "value" is 1 for every token, so n_t . q_t comes out as one more
// output column; a small kernel of its own walks the gates of a (sequence, head) in order, keeps m, and leaves
// (a_t, b_t, exp(-m_t), the product of a over the token's segment so far) for every token.
//
// Work per token and head is 3 D Dv float32 operations (a multiply for k v, one fused multiply-add for the
// state, one for the output), which is what the FMA units are for; the state is read and written once per
// step, which is what bounds a decode step.
#include "common.cuh"

#define LA_CHUNK 8           // tokens per staged chunk
#define LA_STAGES 3          // chunks in flight or in use
#define LA_SEG 128           // tokens per segment of a long prompt
#define LA_MAX_D 256

enum { LA_ACT_NONE = 0, LA_ACT_SILU = 1, LA_ACT_SIGMOID = 2 };

__device__ __forceinline__ float la_act(float x, int act) {
  if (act == LA_ACT_SILU) return x / (1.0f + expf(-x));
  if (act == LA_ACT_SIGMOID) return 1.0f / (1.0f + expf(-x));
  return x;
}

// value of column c of token row t: one tensor, or split partials added in order
template <typename TIN>
__device__ __forceinline__ float la_value(const TIN* row, int c, int n_split, size_t split_stride) {
  float v = to_f32(row[c]);
  for (int s = 1; s < n_split; ++s) v += to_f32(row[s * split_stride + c]);
  return v;
}

// Before the recurrence: what the design does to q, k and v, once per (token, head), into float32 rows
// prep[t][h] = (q[Dp], k[Dp], v[Dvp]) with Dp, Dvp the sizes rounded up to 4 (the padding is zero).
template <typename TIN>
__global__ void __launch_bounds__(128)
decay_prep_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride, size_t row_stride, int q_off,
                  int k_off, int v_off, float* __restrict__ prep, const int* __restrict__ token_pos,
                  const float* __restrict__ cos_t, const float* __restrict__ sin_t, int n_rot, int act, float k_scale,
                  float q_scale, int v_ones, int H, int D, int Dv) {
  pdl_launch_dependents();
  const int t = blockIdx.x, h = blockIdx.y;
  const int Dp = (D + 3) & ~3, Dvp = (Dv + v_ones + 3) & ~3;   // v_ones: one more column of v that is 1
  const int pos = token_pos[t], half = n_rot >> 1;
  pdl_wait();
  const TIN* row = proj + (size_t)t * row_stride;
  const TIN* qrow = row + q_off + h * D;
  const TIN* krow = row + k_off + h * D;
  const TIN* vrow = row + v_off + h * Dv;
  float* out = prep + ((size_t)t * H + h) * (size_t)(2 * Dp + Dvp);
  for (int d = threadIdx.x; d < Dp; d += blockDim.x) {
    float qv = 0.f, kv = 0.f;
    if (d < D) {
      qv = la_act(la_value(qrow, d, n_split, split_stride), act);
      kv = la_act(la_value(krow, d, n_split, split_stride), act);
      if (d < n_rot) {
        const int i = d < half ? d : d - half;
        const float c = cos_t[(size_t)pos * half + i], s = sin_t[(size_t)pos * half + i];
        const int partner = d < half ? d + half : d - half;
        const float qp = la_act(la_value(qrow, partner, n_split, split_stride), act);
        const float kp = la_act(la_value(krow, partner, n_split, split_stride), act);
        // (u, v) -> (u cos - v sin, v cos + u sin) for the pair (i, i + half)
        qv = d < half ? qv * c - qp * s : qv * c + qp * s;
        kv = d < half ? kv * c - kp * s : kv * c + kp * s;
      }
      kv *= k_scale;
      qv *= q_scale;
    }
    out[d] = qv;
    out[Dp + d] = kv;
  }
  for (int c = threadIdx.x; c < Dvp; c += blockDim.x)
    out[2 * Dp + c] = c < Dv ? la_act(la_value(vrow, c, n_split, split_stride), act) : (c == Dv && v_ones) ? 1.f : 0.f;
}

__device__ __forceinline__ void la_cp_async16(float* dst, const float* src) {
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(dst)), "l"(src)
               : "memory");
}
__device__ __forceinline__ void la_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N>
__device__ __forceinline__ void la_cp_async_wait() {
  asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory");
}

// The recurrence over the prepared rows.  Chunks of LA_CHUNK tokens come into a ring of LA_STAGES buffers by
// 16-byte asynchronous copies, two chunks ahead of the one being walked.
//
// A long prompt is cut into segments of seg_len tokens that run side by side (a sequence alone would keep only
// H * Dv / cols CTAs busy).  PASS 1: every segment runs the recurrence, the first from the stored state, the
// others from zero, and leaves its last state in `partial` (a sequence of one segment writes the state itself).
// PASS 2, for the segments after the first: the state the segment should have started from, E, is put together
// from the segments before it (E_0 = partial_0, E_s = decay^seg_len E_(s-1) + partial_s); a token i of the
// segment then lacks decay^(i+1) E^T q_i, which is added to its output; the last segment also writes the
// sequence's new state.  Segments are counted from the step's first token of a sequence, so a sum may be
// rounded differently when a prompt is cut differently; a step of up to seg_len tokens per sequence (every
// decode step) is the plain recurrence.
// DPT: dims of D per thread (a multiple of 4; 8 threads share a column, so D <= 8 DPT).
// GATED: decay and input weight per token from `gates` [T, H, 4] = (a, b, exp(-m), product of a over the segment
// up to and including the token) instead of the head's fixed decay.  head_stride: floats from one head's state to
// the next (a design may keep more than S there).
template <int DPT, int PASS, bool GATED>
__global__ void __launch_bounds__(256)
decay_scan_kernel(const float* __restrict__ prep, float* __restrict__ out, float* __restrict__ state,
                  float* __restrict__ partial, const int* __restrict__ seq_start, const int* __restrict__ seq_slot,
                  const float* __restrict__ decay, const float* __restrict__ gates, size_t head_stride, int H, int D,
                  int Dv, int cols, int col_blocks, int seg_len, int n_seg_max) {
  extern __shared__ __align__(16) float la_smem[];
  const int Dp = (D + 3) & ~3, Dvp = (Dv + 3) & ~3;
  const int row_len = 2 * Dp + Dvp;               // floats per (token, head) of prep
  const int tok_len = 2 * Dp + cols + (GATED ? 4 : 0);   // floats per staged token: q, k, this CTA's columns of v, gates
  pdl_launch_dependents();
  const int b = blockIdx.z, h = blockIdx.y;
  const int seg = blockIdx.x / col_blocks, c0 = (blockIdx.x - seg * col_blocks) * cols;
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int col = c0 + warp * 4 + (lane >> 3);    // this thread's column of v
  const int r = lane & 7;                         // its share of D
  const bool col_live = col < Dv;
  const int seq_t0 = seq_start[b], seq_new = seq_start[b + 1] - seq_t0;
  const int n_seg = (seq_new + seg_len - 1) / seg_len;        // this sequence's segments
  const float g = GATED ? 1.f : decay[h];
  float* S = state + ((size_t)seq_slot[b] * H + h) * head_stride;
  if (seg >= n_seg || (PASS == 2 && (n_seg == 1 || seg == 0))) return;       // (uniform over the CTA)
  const int t0 = seq_t0 + seg * seg_len;                                      // the segment's first token
  const int n_new = min(seg_len, seq_new - seg * seg_len);
  float* part_seq = partial ? partial + ((size_t)b * H + h) * (size_t)n_seg_max * D * Dv : nullptr;
  pdl_wait();

  auto own = [&](int i) { return 4 * (r + 8 * (i >> 2)) + (i & 3); };        // dim of this thread's i-th state value
  float s_reg[DPT];
  if (PASS == 1) {
#pragma unroll
    for (int i = 0; i < DPT; ++i) s_reg[i] = (seg == 0 && col_live && own(i) < D) ? S[(size_t)own(i) * Dv + col] : 0.f;
  } else {
    // E_(seg-1): what the segments before left, each decayed over the segments after it
    float g_seg = 1.f;
    if (!GATED)
      for (int i = 0; i < seg_len; ++i) g_seg *= g;
#pragma unroll
    for (int i = 0; i < DPT; ++i) s_reg[i] = 0.f;
    for (int sp = 0; sp < seg; ++sp) {
      const float* ps = part_seq + (size_t)sp * D * Dv;
      if (GATED) g_seg = __ldcg(gates + ((size_t)(seq_t0 + (sp + 1) * seg_len - 1) * H + h) * 4 + 3);   // over all of segment sp
#pragma unroll
      for (int i = 0; i < DPT; ++i)
        if (col_live && own(i) < D) s_reg[i] = fmaf(g_seg, s_reg[i], __ldcg(ps + (size_t)own(i) * Dv + col));
    }
  }

  const int n_chunks = (n_new + LA_CHUNK - 1) / LA_CHUNK;
  const int qk_pieces = (PASS == 1 ? 2 : 1) * Dp / 4, v_pieces = PASS == 1 ? cols / 4 : 0;
  const int pieces = qk_pieces + v_pieces + (GATED ? 1 : 0);
  const int tid_tok = tid / pieces, tid_pc = tid - tid_tok * pieces;              // where this thread's first piece lies
  const int step_tok = (int)blockDim.x / pieces, step_pc = (int)blockDim.x - step_tok * pieces;   // and its stride
  auto load_chunk = [&](int chunk) {
    float* buf = la_smem + (size_t)(chunk % LA_STAGES) * LA_CHUNK * tok_len;
    const int base = chunk * LA_CHUNK;
    const int n_tok = (n_new - base) < LA_CHUNK ? (n_new - base) : LA_CHUNK;
    // piece e of the chunk is piece (e % pieces) of token (e / pieces); a thread walks its pieces without dividing
    const float* src0 = prep + ((size_t)(t0 + base) * H + h) * row_len;
    const size_t tok_stride = (size_t)H * row_len;
    const float* gsrc0 = GATED ? gates + ((size_t)(t0 + base) * H + h) * 4 : nullptr;
    int tt = tid_tok, pc = tid_pc;
    for (int e = tid; e < n_tok * pieces; e += blockDim.x) {
      const float* src = src0 + tt * tok_stride;
      float* dst = buf + tt * tok_len;
      if (pc < qk_pieces) la_cp_async16(dst + 4 * pc, src + 4 * pc);
      else if (GATED && pc == pieces - 1) la_cp_async16(dst + 2 * Dp + cols, gsrc0 + (size_t)tt * H * 4);
      else if (c0 + 4 * (pc - qk_pieces) < Dvp) la_cp_async16(dst + 2 * Dp + 4 * (pc - qk_pieces), src + 2 * Dp + c0 + 4 * (pc - qk_pieces));
      tt += step_tok;
      pc += step_pc;
      if (pc >= pieces) pc -= pieces, ++tt;
    }
  };
  for (int c = 0; c < LA_STAGES - 1; ++c) {
    if (c < n_chunks) load_chunk(c);
    la_cp_async_commit();
  }
  float g_pow = g;                                 // PASS 2: decay^(i+1) for the token at hand
  const size_t out_stride = (size_t)H * Dv;
  float* out_col = out + (size_t)t0 * out_stride + (size_t)h * Dv + col;        // this thread's column of the segment's first token
  for (int chunk = 0; chunk < n_chunks; ++chunk) {
    if (chunk + LA_STAGES - 1 < n_chunks) load_chunk(chunk + LA_STAGES - 1);     // into the buffer walked last round
    la_cp_async_commit();
    la_cp_async_wait<LA_STAGES - 1>();            // this chunk's copies have landed
    __syncthreads();
    const float* buf = la_smem + (size_t)(chunk % LA_STAGES) * LA_CHUNK * tok_len;
    const int base = chunk * LA_CHUNK;
    const int n_tok = (n_new - base) < LA_CHUNK ? (n_new - base) : LA_CHUNK;
    // one token.  PASS 1: S = g S + k v, then this thread's share of q . S.  PASS 2: its share of q . E.  The
    // shares are added and stored afterwards, so that in a full chunk (the loop below unrolls) one token's
    // shuffles overlap the next token's arithmetic.
    auto one_token = [&](int tt) {
      const float* qrow = buf + tt * tok_len;
      const float* krow = qrow + Dp;
      float v = (PASS == 1 && col_live) ? qrow[2 * Dp + warp * 4 + (lane >> 3)] : 0.f;
      float gt = g;
      if (GATED && PASS == 1) gt = qrow[2 * Dp + cols], v *= qrow[2 * Dp + cols + 1];      // a_t; b_t rides on v
      float acc0 = 0.f, acc1 = 0.f, acc2 = 0.f, acc3 = 0.f;
#pragma unroll
      for (int i4 = 0; i4 < DPT / 4; ++i4) {
        const int d = 4 * (r + 8 * i4);
        if (d < Dp) {
          const float4 q4 = *reinterpret_cast<const float4*>(qrow + d);
          float* s4 = s_reg + 4 * i4;
          if (PASS == 1) {
            const float4 k4 = *reinterpret_cast<const float4*>(krow + d);
            s4[0] = fmaf(gt, s4[0], k4.x * v);
            s4[1] = fmaf(gt, s4[1], k4.y * v);
            s4[2] = fmaf(gt, s4[2], k4.z * v);
            s4[3] = fmaf(gt, s4[3], k4.w * v);
          }
          acc0 = fmaf(s4[0], q4.x, acc0);
          acc1 = fmaf(s4[1], q4.y, acc1);
          acc2 = fmaf(s4[2], q4.z, acc2);
          acc3 = fmaf(s4[3], q4.w, acc3);
        }
      }
      return (acc0 + acc1) + (acc2 + acc3);
    };
    const bool writer = r == 0 && col_live;
    float* out_chunk = out_col + (size_t)base * out_stride;
    auto out_at = [&](int tt) { return out_chunk + (size_t)tt * out_stride; };
    auto finish = [&](int tt, float acc, float before) {       // before: PASS 2, what the first pass left there
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (PASS == 1) {
        if (writer) *out_at(tt) = acc;
      } else if (GATED) {
        if (writer) *out_at(tt) = before + buf[tt * tok_len + 2 * Dp + cols + 3] * acc;
      } else {
        if (writer) *out_at(tt) = before + g_pow * acc;
        g_pow *= g;
      }
    };
    if (n_tok == LA_CHUNK) {
      float part[LA_CHUNK], before[LA_CHUNK];
      if (PASS == 2) {                       // the chunk's outputs of the first pass, fetched together
#pragma unroll
        for (int tt = 0; tt < LA_CHUNK; ++tt) before[tt] = writer ? __ldcg(out_at(tt)) : 0.f;
      }
#pragma unroll
      for (int tt = 0; tt < LA_CHUNK; ++tt) part[tt] = one_token(tt);
#pragma unroll
      for (int tt = 0; tt < LA_CHUNK; ++tt) finish(tt, part[tt], PASS == 2 ? before[tt] : 0.f);
    } else {
      for (int tt = 0; tt < n_tok; ++tt) {
        const float before = (PASS == 2 && writer) ? __ldcg(out_at(tt)) : 0.f;
        finish(tt, one_token(tt), before);
      }
    }
    __syncthreads();                              // the buffer is refilled by the next round's copies
  }
  if (PASS == 1) {
    float* dst = n_seg == 1 ? S : part_seq + (size_t)seg * D * Dv;
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (col_live && own(i) < D) dst[(size_t)own(i) * Dv + col] = s_reg[i];
  } else if (seg == n_seg - 1) {
    // the sequence's new state: E_(n_seg-1) = decay^(its length) E_(n_seg-2) + partial_(n_seg-1)
    float g_len = 1.f;
    if (GATED) g_len = __ldcg(gates + ((size_t)(t0 + n_new - 1) * H + h) * 4 + 3);
    else
      for (int i = 0; i < n_new; ++i) g_len *= g;
    const float* ps = part_seq + (size_t)seg * D * Dv;
#pragma unroll
    for (int i = 0; i < DPT; ++i)
      if (col_live && own(i) < D)
        S[(size_t)own(i) * Dv + col] = fmaf(g_len, s_reg[i], __ldcg(ps + (size_t)own(i) * Dv + col));
  }
}

// One warp per (sequence, head) walks the step's tokens of the sequence in order: the gates' pre-activations are
// columns i_off + h and f_off + h of the projected row (plus a bias), i = cap tanh(z_i / cap), f =
// logsigmoid(cap tanh(z_f / cap)); m is read from and written back to the sequence's state (m_off floats into the
// head's state).  Thirty-two tokens at a time: every lane prepares one token's (i, f), all lanes then run the chain
// m_t = max(f_t + m_(t-1), i_t) over the 32 values (two dependent operations a token), and lane j keeps what
// token j needs.  The sum of f over a segment (which the segments' second pass wants as a product of a) restarts
// wherever a segment of seg_len tokens starts, counted from the sequence's first token of the step.
template <typename TIN>
__global__ void __launch_bounds__(128)
gate_scan_kernel(const TIN* __restrict__ proj, int n_split, size_t split_stride, size_t row_stride, int i_off, int f_off,
                 const float* __restrict__ bias_i, const float* __restrict__ bias_f, float cap,
                 float* __restrict__ gates, float* __restrict__ state, size_t head_stride, int m_off,
                 const int* __restrict__ seq_start, const int* __restrict__ seq_slot, int H, int seg_len) {
  pdl_launch_dependents();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int h = blockIdx.x * 4 + warp, b = blockIdx.y;
  if (h >= H) return;
  const int t0 = seq_start[b], n_new = seq_start[b + 1] - t0;
  float* m_ptr = state + ((size_t)seq_slot[b] * H + h) * head_stride + m_off;
  const float bi = bias_i ? bias_i[h] : 0.f, bf = bias_f ? bias_f[h] : 0.f;
  pdl_wait();
  float m = *m_ptr, cum = 0.f, m_base = m;
  int in_seg = 0;                                    // (base + j) % seg_len, kept by counting
  for (int base = 0; base < n_new; base += 32) {
    const int n = min(32, n_new - base);
    float il = 0.f, fl = 0.f;
    if (lane < n) {
      const TIN* row = proj + (size_t)(t0 + base + lane) * row_stride;
      float zi = la_value(row, i_off + h, n_split, split_stride) + bi;
      float zf = la_value(row, f_off + h, n_split, split_stride) + bf;
      if (cap > 0.f) zi = cap * tanhf(zi / cap), zf = cap * tanhf(zf / cap);
      il = zi;
      fl = fminf(zf, 0.f) - log1pf(expf(-fabsf(zf)));           // log sigmoid(zf)
    }
    float my_prev = 0.f, my_m = 0.f, my_sum = 0.f;
    // every lane walks the chain m -> max(f + m, i); a whole block of 32 tokens is unrolled, so that the broadcasts
    // run ahead of the chain
    auto token = [&](int j) {
      const float f = __shfl_sync(0xffffffffu, fl, j), i = __shfl_sync(0xffffffffu, il, j);
      if (in_seg == 0) cum = 0.f, m_base = m;
      if (++in_seg == seg_len) in_seg = 0;
      const float m_new = fmaxf(f + m, i);
      cum += f;
      if (lane == j) my_prev = m, my_m = m_new, my_sum = cum + m_base;
      m = m_new;
    };
    if (n == 32) {
#pragma unroll
      for (int j = 0; j < 32; ++j) token(j);
    } else {
      for (int j = 0; j < n; ++j) token(j);
    }
    if (lane < n)
      *reinterpret_cast<float4*>(gates + ((size_t)(t0 + base + lane) * H + h) * 4) =
          make_float4(expf(fl + my_prev - my_m), expf(il - my_m), expf(-my_m), expf(my_sum - my_m));
  }
  if (lane == 0) *m_ptr = m;
}

// proj: [T, row_stride] (or split partials of it); gates: float32 [T, H, 4], 16-byte aligned; state: float32
// [slots, H, head_stride] with a head's m at m_off; bias_i, bias_f: float32 [H] or null; cap <= 0: no cap.
LLMX_API int llmx_gate_scan(const void* proj, int in_dtype, int n_split, long long split_stride, long long row_stride,
                            int i_off, int f_off, const float* bias_i, const float* bias_f, float cap, float* gates,
                            float* state, long long head_stride, int m_off, const int* seq_start, const int* seq_slot,
                            int n_seqs, int H, int seg_len, cudaStream_t stream) {
  if (n_seqs <= 0) return 0;
  if (H <= 0 || n_split < 1 || head_stride <= m_off || m_off < 0 || n_seqs > 65535 || ((uintptr_t)gates & 15))
    return LLMX_REFUSED(1);
  if (seg_len <= 0) seg_len = LA_SEG;
  const dim3 grid((H + 3) / 4, n_seqs);
  if (in_dtype == LLMX_F32)
    launch_pdl(gate_scan_kernel<float>, grid, dim3(128), 0, stream, (const float*)proj, n_split, (size_t)split_stride,
               (size_t)row_stride, i_off, f_off, bias_i, bias_f, cap, gates, state, (size_t)head_stride, m_off,
               seq_start, seq_slot, H, seg_len);
  else if (in_dtype == LLMX_BF16)
    launch_pdl(gate_scan_kernel<bf16>, grid, dim3(128), 0, stream, (const bf16*)proj, n_split, (size_t)split_stride,
               (size_t)row_stride, i_off, f_off, bias_i, bias_f, cap, gates, state, (size_t)head_stride, m_off,
               seq_start, seq_slot, H, seg_len);
  else
    return LLMX_REFUSED(2);
  return LLMX_LAUNCH_STATUS();
}

// proj: [T, row_stride] (or split partials of it); prep: float32 scratch of T * H * (2 Dp + Dvp) elements, 16-byte
// aligned; out: float32 [T, H*Dva]; state: float32 [slots, H, head_stride >= D*Dva], Dva = Dv + v_ones (v_ones:
// the values get one more column that is 1 for every token).  max_new: most tokens of one sequence; seg_len:
// tokens per segment (0: LA_SEG); partial: float32 scratch [n_seqs, H, ceil(max_new / seg_len), D, Dva], needed
// when max_new > seg_len.  gates: null (the heads' fixed `decay`), or float32 [T, H, 4] as gate_scan leaves them
// (made with the same seg_len).
LLMX_API int llmx_decay_scan(const void* proj, int in_dtype, int n_split, long long split_stride, long long row_stride,
                             int q_off, int k_off, int v_off, float* prep, float* out, float* state, float* partial,
                             const int* seq_start, const int* token_pos, const int* seq_slot, const float* decay,
                             const float* cos_t, const float* sin_t, int n_rot, int act, float k_scale, int n_tokens,
                             int n_seqs, int max_new, int seg_len, int H, int D, int Dv, int n_sm, const float* gates,
                             long long head_stride, float q_scale, int v_ones, cudaStream_t stream) {
  if (n_seqs <= 0 || n_tokens <= 0) return 0;
  if (H <= 0 || D <= 0 || D > LA_MAX_D || Dv <= 0 || n_split < 1 || n_rot < 0 || n_rot > D || (n_rot & 1))
    return LLMX_REFUSED(1);
  v_ones = v_ones ? 1 : 0;
  const int Dva = Dv + v_ones;
  if (head_stride <= 0) head_stride = (long long)D * Dva;
  if (head_stride < (long long)D * Dva || (!gates && !decay) || ((uintptr_t)gates & 15)) return LLMX_REFUSED(1);
  if (n_rot > 0 && (!cos_t || !sin_t)) return LLMX_REFUSED(4);
  if (act != LA_ACT_NONE && act != LA_ACT_SILU) return LLMX_REFUSED(1);
  if (n_seqs > 65535 || H > 65535 || ((uintptr_t)prep & 15)) return LLMX_REFUSED(3);
  if (seg_len <= 0) seg_len = LA_SEG;
  if (max_new <= 0 || max_new > n_tokens) max_new = n_tokens;
  const int n_seg = (max_new + seg_len - 1) / seg_len;
  if (n_seg > 1 && !partial) return LLMX_REFUSED(4);
  const dim3 pgrid(n_tokens, H);
  if (in_dtype == LLMX_F32)
    launch_pdl(decay_prep_kernel<float>, pgrid, dim3(128), 0, stream, (const float*)proj, n_split, (size_t)split_stride,
               (size_t)row_stride, q_off, k_off, v_off, prep, token_pos, cos_t, sin_t, n_rot, act, k_scale, q_scale,
               v_ones, H, D, Dv);
  else if (in_dtype == LLMX_BF16)
    launch_pdl(decay_prep_kernel<bf16>, pgrid, dim3(128), 0, stream, (const bf16*)proj, n_split, (size_t)split_stride,
               (size_t)row_stride, q_off, k_off, v_off, prep, token_pos, cos_t, sin_t, n_rot, act, k_scale, q_scale,
               v_ones, H, D, Dv);
  else
    return LLMX_REFUSED(2);
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return (int)e;
  Dv = Dva;                                        // from here on the extra column is a column like the others
  // columns per CTA: as many as still give every SM a CTA or two (a CTA with more columns stages q and k fewer times)
  int cols = 32;
  while (cols > 8 && (long long)n_seqs * H * n_seg * ((Dv + cols - 1) / cols) < 2LL * n_sm) cols >>= 1;
  while (cols > 4 && cols / 2 >= Dv) cols >>= 1;
  const int Dp = (D + 3) & ~3;
  const int col_blocks = (Dv + cols - 1) / cols;
  if ((long long)col_blocks * n_seg > 0x7fffffff) return LLMX_REFUSED(3);
  dim3 grid(col_blocks * n_seg, H, n_seqs), block(cols * 8);
  const size_t smem = (size_t)LA_STAGES * LA_CHUNK * (2 * Dp + cols + (gates ? 4 : 0)) * sizeof(float);
#define GO2(DPT, PASS, GATED)                                                                                          \
  do {                                                                                                                 \
    static bool attr_set = false;                                                                                      \
    if (!attr_set && smem > 48 * 1024) {                                                                               \
      e = cudaFuncSetAttribute(decay_scan_kernel<DPT, PASS, GATED>, cudaFuncAttributeMaxDynamicSharedMemorySize,       \
                               100 * 1024);                                                                            \
      if (e != cudaSuccess) return (int)e;                                                                             \
      attr_set = true;                                                                                                 \
    }                                                                                                                  \
    launch_pdl(decay_scan_kernel<DPT, PASS, GATED>, grid, block, smem, stream, (const float*)prep, out, state, partial, \
               seq_start, seq_slot, decay, gates, (size_t)head_stride, H, D, Dv, cols, col_blocks, seg_len, n_seg);    \
  } while (0)
#define GO1(DPT, PASS)              \
  do {                              \
    if (gates) GO2(DPT, PASS, true); \
    else GO2(DPT, PASS, false);     \
  } while (0)
#define GO(DPT)                    \
  do {                             \
    GO1(DPT, 1);                   \
    if (n_seg > 1) GO1(DPT, 2);    \
  } while (0)
  if (Dp <= 32) GO(4);
  else if (Dp <= 64) GO(8);
  else if (Dp <= 128) GO(16);
  else GO(32);
#undef GO
#undef GO1
#undef GO2
  return LLMX_LAUNCH_STATUS();
}

// ---------------------------------------------------------------------------
// After the recurrence: y[t, j] = o[t, j] * r * gain[j] * act(gate[t, j]) with r = 1 / sqrt(mean(o^2) + eps), the
// mean taken over one head's Dv columns (per_head, usually without a gain) or over all H*Dv columns of the
// token.  One warp per (token, head), or one CTA per token.  float32 throughout; y in the activations' dtype.
// ---------------------------------------------------------------------------
// With `gates` (float32 [T, H, 4], exp(-m) third) a head's o has o_stride = Dv + 1 columns, the last one n . q,
// and o is first divided by max(|n . q|, exp(-m)) + den_eps.
template <typename TIN, typename TO>
__global__ void gated_norm_heads_kernel(const float* __restrict__ o, const TIN* __restrict__ proj, int n_split,
                                        size_t split_stride, size_t row_stride, int g_off,
                                        const float* __restrict__ gain, float eps, int gate_act,
                                        TO* __restrict__ y, int H, int Dv, int o_stride,
                                        const float* __restrict__ gates, float den_eps) {
  pdl_launch_dependents();
  pdl_wait();
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int t = blockIdx.x, h = blockIdx.y * 4 + warp;
  if (h >= H) return;
  const float* orow = o + ((size_t)t * H + h) * o_stride;
  float den = 1.f;
  if (gates) den = fmaxf(fabsf(orow[Dv]), gates[((size_t)t * H + h) * 4 + 2]) + den_eps;
  float ss = 0.f;
  for (int i = lane; i < Dv; i += 32) {
    const float v = gates ? orow[i] / den : orow[i];
    ss += v * v;
  }
  const float r = 1.0f / sqrtf(warp_sum(ss) / (float)Dv + eps);
  const TIN* grow = proj + (size_t)t * row_stride + g_off + h * Dv;
  for (int i = lane; i < Dv; i += 32) {
    float v = (gates ? orow[i] / den : orow[i]) * r;
    if (gain) v *= gain[h * Dv + i];
    y[((size_t)t * H + h) * Dv + i] = from_f32<TO>(v * la_act(la_value(grow, i, n_split, split_stride), gate_act));
  }
}

template <typename TIN, typename TO>
__global__ void __launch_bounds__(256)
gated_norm_row_kernel(const float* __restrict__ o, const TIN* __restrict__ proj, int n_split, size_t split_stride,
                      size_t row_stride, int g_off, const float* __restrict__ gain, float eps, int gate_act,
                      TO* __restrict__ y, int n) {
  __shared__ float red[32];
  pdl_launch_dependents();
  pdl_wait();
  const int t = blockIdx.x;
  const float* orow = o + (size_t)t * n;
  float ss = 0.f;
  for (int i = threadIdx.x; i < n; i += blockDim.x) ss += orow[i] * orow[i];
  const float r = 1.0f / sqrtf(block_sum(ss, red) / (float)n + eps);
  const TIN* grow = proj + (size_t)t * row_stride + g_off;
  for (int i = threadIdx.x; i < n; i += blockDim.x) {
    float v = orow[i] * r;
    if (gain) v *= gain[i];
    y[(size_t)t * n + i] = from_f32<TO>(v * la_act(la_value(grow, i, n_split, split_stride), gate_act));
  }
}

// per_head != 0: the mean of squares is a head's; else the token's.  gain: float32 [H*Dv] or null.  gates (per_head
// only): see the kernel; o is then [T, H, Dv + 1].
LLMX_API int llmx_gated_norm(const float* o, const void* proj, int in_dtype, int n_split, long long split_stride,
                             long long row_stride, int g_off, const float* gain, float eps, int gate_act, int per_head,
                             void* y, int out_dtype, int n_tokens, int H, int Dv, const float* gates, float den_eps,
                             cudaStream_t stream) {
  if (n_tokens <= 0) return 0;
  if (H <= 0 || Dv <= 0 || n_split < 1 || (gates && !per_head)) return LLMX_REFUSED(1);
  const int o_stride = gates ? Dv + 1 : Dv;
  if (gate_act != LA_ACT_SILU && gate_act != LA_ACT_SIGMOID && gate_act != LA_ACT_NONE) return LLMX_REFUSED(1);
#define GO(TIN, TO)                                                                                                  \
  do {                                                                                                               \
    if (per_head)                                                                                                    \
      launch_pdl(gated_norm_heads_kernel<TIN, TO>, dim3(n_tokens, (H + 3) / 4), dim3(128), 0, stream, o,             \
                 (const TIN*)proj, n_split, (size_t)split_stride, (size_t)row_stride, g_off, gain, eps, gate_act,    \
                 (TO*)y, H, Dv, o_stride, gates, den_eps);                                                                                  \
    else                                                                                                             \
      launch_pdl(gated_norm_row_kernel<TIN, TO>, dim3(n_tokens), dim3(256), 0, stream, o, (const TIN*)proj, n_split, \
                 (size_t)split_stride, (size_t)row_stride, g_off, gain, eps, gate_act, (TO*)y, H * Dv);              \
  } while (0)
  const int key = in_dtype * 2 + out_dtype;
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
