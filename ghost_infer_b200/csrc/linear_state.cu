// Linear attention with a matrix of state per head, walked token by token: the recurrence of a gated delta rule and of
// decayed ("lightning") linear attention, one kernel with the differences as parameters.
//
// Per head, with S a K x V matrix of 32-bit numbers kept per sequence, and per token a decay g, a key k (K), a query q (K),
// a value v (V) and, for the delta rule, a write strength beta:
//     S <- g S;   u = delta ? beta (v - S^T k) : v;   S <- S + k u^T;   o = S^T q          (o sees the token's own write)
//  * decay: a constant per head, or exp(-exp(A_log[h]) * softplus(a[t, h] + dt_bias[h])) from a projected row;
//  * beta: sigmoid of a projected row;
//  * q and k may pass silu on the way in, and may be made unit vectors (x / sqrt(sum x^2 + eps)), q times a constant;
//  * query/key head of head h: h / (heads / qk_heads).
// Everything after the loads is 32-bit.  The tokens of a sequence are walked in order whatever the step holds, so a prompt
// cut anywhere, alone or in a batch, gives the same bits.
//
// Work split: grid (heads, sequences, tiles of 32 columns of S).  A column of S (K numbers) belongs to 8 neighbouring lanes,
// lane l holding rows l, l + 8, ...; a column's two dot products end with three exchanges among its lanes.  Tokens go
// through shared memory 16 at a time.  State per slot: [heads][V][K] floats (a column's rows side by side) at the start of
// the slot's row; slot -1 (a padding row of a fixed-size launch) uses the last row of the matrix.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int LS_COLS = 32, LS_LANES = 8, LS_CH = 16;

__device__ __forceinline__ float ls_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float ls_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

template <typename T, int KR>
__global__ void __launch_bounds__(LS_COLS * LS_LANES)
linear_state_kernel(float* __restrict__ o, const T* q, long ldq, const T* k, long ldk, const T* v, long ldv, const T* a_in,
                    long lda, const T* b_in, long ldb, const float* __restrict__ decay_c, const float* __restrict__ dt_bias,
                    float* state, long state_ld, int state_rows, const int* __restrict__ cu_seqlens,
                    const int* __restrict__ seq_slots, int heads, int qk_heads, int K, int V, int in_act, int unit_norm,
                    float norm_eps, float q_scale, int delta) {
  constexpr int Kp = KR * LS_LANES;
  constexpr int NT = LS_COLS * LS_LANES;
  extern __shared__ __align__(16) float sm[];
  float* sq = sm;                      // [LS_CH][Kp]
  float* sk = sq + LS_CH * Kp;         // [LS_CH][Kp]
  float* sv = sk + LS_CH * Kp;         // [LS_CH][LS_COLS]
  float* sg = sv + LS_CH * LS_COLS;    // [LS_CH]
  float* sb = sg + LS_CH;              // [LS_CH]
  gi::pdl_prologue();
  const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * LS_COLS;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  if (qlen <= 0) return;
  const int slot = seq_slots[b];
  float* S_row = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld + (size_t)h * V * K;
  const int hk = h / (heads / qk_heads);
  const int tid = threadIdx.x, col = tid / LS_LANES, lane = tid % LS_LANES;
  const int j = j0 + col;
  float S[KR];
#pragma unroll
  for (int r = 0; r < KR; ++r) {
    const int i = lane + LS_LANES * r;
    S[r] = (j < V && i < K) ? S_row[(size_t)j * K + i] : 0.f;
  }
  const float dc = decay_c[h];
  const float rate = a_in != nullptr ? expf(dc) : 0.f, bias = (a_in != nullptr && dt_bias != nullptr) ? dt_bias[h] : 0.f;
  for (int c0 = 0; c0 < qlen; c0 += LS_CH) {
    const int n = min(LS_CH, qlen - c0);
    const size_t tok = (size_t)tok0 + c0;
    __syncthreads();                   // the chunk before has been used up
    for (int idx = tid; idx < n * Kp; idx += NT) {
      const int t = idx / Kp, i = idx % Kp;
      float qv = 0.f, kv = 0.f;
      if (i < K) {
        qv = gi::ldf(q + (tok + t) * ldq + (size_t)hk * K + i);
        kv = gi::ldf(k + (tok + t) * ldk + (size_t)hk * K + i);
        if (in_act) { qv = ls_silu(qv); kv = ls_silu(kv); }
      }
      sq[idx] = qv;
      sk[idx] = kv;
    }
    for (int idx = tid; idx < n * LS_COLS; idx += NT) {
      const int t = idx / LS_COLS, c = idx % LS_COLS;
      float vv = 0.f;
      if (j0 + c < V) {
        vv = gi::ldf(v + (tok + t) * ldv + (size_t)h * V + j0 + c);
        if (in_act) vv = ls_silu(vv);
      }
      sv[idx] = vv;
    }
    if (tid < n) {
      sg[tid] = a_in != nullptr ? expf(-rate * ls_softplus(gi::ldf(a_in + (tok + tid) * lda + h) + bias)) : dc;
      sb[tid] = b_in != nullptr ? 1.0f / (1.0f + expf(-gi::ldf(b_in + (tok + tid) * ldb + h))) : 1.0f;
    }
    __syncthreads();
    if (unit_norm) {
      const int warp = tid >> 5, wl = tid & 31;
      for (int t = warp; t < n; t += NT / 32) {
        float s1 = 0.f, s2 = 0.f;
        for (int i = wl; i < Kp; i += 32) {
          s1 = fmaf(sq[t * Kp + i], sq[t * Kp + i], s1);
          s2 = fmaf(sk[t * Kp + i], sk[t * Kp + i], s2);
        }
        s1 = gi::warp_sum(s1);
        s2 = gi::warp_sum(s2);
        const float fq = q_scale / sqrtf(s1 + norm_eps), fk = 1.0f / sqrtf(s2 + norm_eps);
        for (int i = wl; i < Kp; i += 32) {
          sq[t * Kp + i] *= fq;
          sk[t * Kp + i] *= fk;
        }
      }
      __syncthreads();
    }
    for (int t = 0; t < n; ++t) {
      const float g = sg[t];
      float kk[KR];
#pragma unroll
      for (int r = 0; r < KR; ++r) kk[r] = sk[t * Kp + lane + LS_LANES * r];
      float u = sv[t * LS_COLS + col];
      if (delta) {
        float d = 0.f;
#pragma unroll
        for (int r = 0; r < KR; ++r) d = fmaf(S[r], kk[r], d);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        u = sb[t] * (u - g * d);
      }
      float acc = 0.f;
#pragma unroll
      for (int r = 0; r < KR; ++r) {
        S[r] = fmaf(kk[r], u, g * S[r]);
        acc = fmaf(S[r], sq[t * Kp + lane + LS_LANES * r], acc);
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      acc += __shfl_xor_sync(0xffffffffu, acc, 4);
      if (lane == 0 && j < V) o[(tok + t) * ((size_t)heads * V) + (size_t)h * V + j] = acc;
    }
  }
  if (j < V) {
#pragma unroll
    for (int r = 0; r < KR; ++r) {
      const int i = lane + LS_LANES * r;
      if (i < K) S_row[(size_t)j * K + i] = S[r];
    }
  }
}

}  // namespace

extern "C" int gi_linear_state(float* o, const void* q, long ldq, const void* k, long ldk, const void* v, long ldv,
                               const void* a_in, long lda, const void* b_in, long ldb, int dtype, const float* decay_c,
                               const float* dt_bias, float* state, long state_ld, int state_rows, const int* cu_seqlens,
                               const int* seq_slots, int n_seqs, int heads, int qk_heads, int K, int V, int in_act,
                               int unit_norm, float norm_eps, float q_scale, int delta, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (heads <= 0 || qk_heads <= 0 || heads % qk_heads || K <= 0 || V <= 0)
    return gi::fail(GI_ERR_ARG, "linear_state: bad sizes (heads %d, query/key heads %d, keys %d, values %d)", heads, qk_heads, K, V);
  if (K > 32 * LS_LANES) return gi::fail(GI_ERR_UNSUPPORTED, "linear_state: keys of %d numbers (at most %d)", K, 32 * LS_LANES);
  if (!o || !q || !k || !v || !decay_c || !state || !cu_seqlens || !seq_slots) return gi::fail(GI_ERR_ARG, "linear_state: a missing pointer");
  if (delta && b_in == nullptr) return gi::fail(GI_ERR_ARG, "linear_state: the delta rule needs its write strengths");
  if (state_ld < (long)heads * K * V) return gi::fail(GI_ERR_ARG, "linear_state: state rows of %ld floats, wanted %ld", state_ld, (long)heads * K * V);
  const dim3 grid(heads, n_seqs, (V + LS_COLS - 1) / LS_COLS), block(LS_COLS * LS_LANES);
  cudaError_t e = cudaSuccess;
#define GI_LS_LAUNCH(KR)                                                                                                  \
  do {                                                                                                                    \
    const size_t smem = (size_t)(2 * LS_CH * (KR) * LS_LANES + LS_CH * LS_COLS + 2 * LS_CH) * sizeof(float);              \
    e = gi::launch(linear_state_kernel<T, KR>, grid, block, smem, (cudaStream_t)stream, o, (const T*)q, ldq, (const T*)k, \
                   ldk, (const T*)v, ldv, (const T*)a_in, lda, (const T*)b_in, ldb, decay_c, dt_bias, state, state_ld,   \
                   state_rows, cu_seqlens, seq_slots, heads, qk_heads, K, V, in_act, unit_norm, norm_eps, q_scale, delta); \
  } while (0)
  GI_DISPATCH_DTYPE(dtype, T, {
    if (K <= 4 * LS_LANES) GI_LS_LAUNCH(4);
    else if (K <= 8 * LS_LANES) GI_LS_LAUNCH(8);
    else if (K <= 16 * LS_LANES) GI_LS_LAUNCH(16);
    else GI_LS_LAUNCH(32);
  });
#undef GI_LS_LAUNCH
  return gi::check(e, "linear_state");
}
