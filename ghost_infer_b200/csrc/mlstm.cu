// The gates of a matrix memory with a running maximum (the mLSTM of xLSTM), walked token by token per head.
//
// Per head, with a cap c on the gates' pre-activations a_t (input) and b_t (forget):
//     i_t = c tanh(a_t / c),   f_t = log sigmoid(c tanh(b_t / c)),
//     m_t = max(f_t + m_(t-1), i_t)                       (m starts at 0),
//     keep_t = exp(f_t + m_(t-1) - m_t),   put_t = exp(i_t - m_t),
//     n_t = keep_t n_(t-1) + put_t k_t                    (n starts at 0),
//     out_t = s / (max(|n_t . (s q_t)|, exp(-m_t)) + 1e-6)    with s the queries' constant scale.
// The matrix itself, S_t = keep_t S_(t-1) + put_t k_t v_t^T and the read-out S_t^T q_t, is the linear-state kernel's work:
// this kernel hands it keep_t and put_t per token and head, and out_t, by which the read-out is multiplied afterwards.
// Everything here is 32-bit.  Per sequence and head the state holds n (K numbers) and m.
//
// grid (heads, sequences), four warps a block.  The tokens of a sequence are taken in chunks: all threads load a chunk's keys,
// queries and gate rows into shared memory (one trip to memory a chunk) and make i and f; one thread walks m through the chunk
// (a maximum and an addition a token); keep and put follow for all tokens at once; one warp walks n (lane l holds entries l,
// l + 32, ... in registers: two multiply-adds an entry and token, the lanes' shares of n . q left in shared memory); the
// shares are added per token in a fixed order.  The arithmetic of a token does not depend on where the chunks begin, so a
// prompt cut anywhere gives the same bits.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T, int NPL, int CH>
__global__ void __launch_bounds__(128)
mlstm_gates_kernel(float* __restrict__ keep_out, float* __restrict__ put_out, float* __restrict__ scale_out, const T* q, long ldq,
                   const T* k, long ldk, const T* gi_in, const T* gf_in, long ldg, const float* __restrict__ bi,
                   const float* __restrict__ bf, float cap, float q_scale, float* state, long state_ld, int state_rows,
                   const int* cu_seqlens, const int* seq_slots, int heads, int K) {
  extern __shared__ float sm[];
  constexpr int Kp = NPL * 32;
  float* sk = sm;                    // [CH][Kp]
  float* sq = sk + CH * Kp;          // [CH][Kp]
  float* sdot = sq + CH * Kp;        // [CH][33]
  float* si = sdot + CH * 33;        // [CH] log input gates, then put
  float* sf = si + CH;               // [CH] log forget gates, then keep
  float* smx = sf + CH;              // [CH] m after each token
  float* spv = smx + CH;             // [CH] m before each token
  __shared__ float m_carry;
  gi::pdl_prologue();
  const int h = blockIdx.x, b = blockIdx.y, tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  if (qlen <= 0) return;
  const int slot = seq_slots[b];
  float* st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld + (size_t)h * (K + 1);
  float n[NPL];
#pragma unroll
  for (int i = 0; i < NPL; ++i) {
    const int e = lane + 32 * i;
    n[i] = (warp == 0 && e < K) ? st[e] : 0.f;
  }
  if (tid == 0) m_carry = st[K];
  const float bias_i = bi != nullptr ? bi[h] : 0.f, bias_f = bf != nullptr ? bf[h] : 0.f;
  // a chunk's rows travel through registers: the next chunk's loads are issued before this chunk's walks begin and land
  // while they run, so a chunk costs its walks alone
  constexpr int R = CH * Kp / 128;
  float kr[R], qr[R], ga = 0.f, gb = 0.f;
  auto fetch = [&](int c0) {
    const int nh = min(CH, qlen - c0);
    const size_t tokc = (size_t)tok0 + c0;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      const int idx = tid + i * 128, t = idx / Kp, e = idx % Kp;
      const bool live = t < nh && e < K;
      kr[i] = live ? gi::ldf(k + (tokc + t) * ldk + (size_t)h * K + e) : 0.f;
      qr[i] = live ? gi::ldf(q + (tokc + t) * ldq + (size_t)h * K + e) : 0.f;
    }
    if (tid < nh) {
      ga = gi::ldf(gi_in + (tokc + tid) * ldg + h);
      gb = gi::ldf(gf_in + (tokc + tid) * ldg + h);
    }
  };
  fetch(0);
  for (int c0 = 0; c0 < qlen; c0 += CH) {
    const int nh = min(CH, qlen - c0);
    const size_t tokc = (size_t)tok0 + c0;
#pragma unroll
    for (int i = 0; i < R; ++i) {
      sk[tid + i * 128] = kr[i];
      sq[tid + i * 128] = qr[i];
    }
    if (tid < nh) {
      const float a = ga + bias_i, bb = gb + bias_f;
      si[tid] = cap * tanhf(a / cap);
      sf[tid] = log_sigmoid_f(cap * tanhf(bb / cap));
    }
    if (c0 + CH < qlen) fetch(c0 + CH);
    __syncthreads();
    if (tid == 0) {
      float m = m_carry;
      for (int t = 0; t < nh; ++t) {
        spv[t] = m;
        m = fmaxf(sf[t] + m, si[t]);
        smx[t] = m;
      }
      m_carry = m;
    }
    __syncthreads();
    if (tid < nh) {
      const float keep = expf(sf[tid] + spv[tid] - smx[tid]), put = expf(si[tid] - smx[tid]);
      sf[tid] = keep;
      si[tid] = put;
      keep_out[(tokc + tid) * heads + h] = keep;
      put_out[(tokc + tid) * heads + h] = put;
    }
    __syncthreads();
    if (warp == 0) {
      for (int t = 0; t < nh; ++t) {
        const float keep = sf[t], put = si[t];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < NPL; ++i) {
          n[i] = fmaf(put, sk[t * Kp + lane + 32 * i], keep * n[i]);
          dot = fmaf(n[i], sq[t * Kp + lane + 32 * i], dot);
        }
        sdot[t * 33 + lane] = dot;
      }
    }
    __syncthreads();
    if (tid < nh) {
      float d = 0.f;
      for (int l = 0; l < 32; ++l) d += sdot[tid * 33 + l];
      d *= q_scale;
      scale_out[(tokc + tid) * heads + h] = q_scale / (fmaxf(fabsf(d), expf(-smx[tid])) + 1e-6f);
    }
    __syncthreads();
  }
  if (warp == 0) {
#pragma unroll
    for (int i = 0; i < NPL; ++i) {
      const int e = lane + 32 * i;
      if (e < K) st[e] = n[i];
    }
  }
  if (tid == 0) st[K] = m_carry;
}

template <typename T, int NPL, int CH>
cudaError_t launch_gates(dim3 grid, cudaStream_t s, float* keep, float* put, float* out_scale, const void* q, long ldq, const void* k,
                         long ldk, const void* gate_i, const void* gate_f, long ldg, const float* bias_i, const float* bias_f, float cap,
                         float q_scale, float* state, long state_ld, int state_rows, const int* cu_seqlens, const int* seq_slots,
                         int heads, int K) {
  const size_t smem = (size_t)(2 * CH * NPL * 32 + CH * 33 + 4 * CH) * sizeof(float);
  return gi::launch(mlstm_gates_kernel<T, NPL, CH>, grid, dim3(128), smem, s, keep, put, out_scale, (const T*)q, ldq, (const T*)k, ldk,
                    (const T*)gate_i, (const T*)gate_f, ldg, bias_i, bias_f, cap, q_scale, state, state_ld, state_rows, cu_seqlens,
                    seq_slots, heads, K);
}

}  // namespace

extern "C" int gi_mlstm_gates(float* keep, float* put, float* out_scale, const void* q, long ldq, const void* k, long ldk,
                              const void* gate_i, const void* gate_f, long ldg, int dtype, const float* bias_i, const float* bias_f,
                              float cap, float q_scale, float* state, long state_ld, int state_rows, const int* cu_seqlens,
                              const int* seq_slots, int n_seqs, int heads, int K, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (heads <= 0 || K <= 0 || K > 512) return gi::fail(GI_ERR_UNSUPPORTED, "mlstm_gates: keys of %d numbers (at most 512)", K);
  if (!(cap > 0.f)) return gi::fail(GI_ERR_ARG, "mlstm_gates: the gates' cap must be positive");
  if (state_ld < (long)heads * (K + 1)) return gi::fail(GI_ERR_ARG, "mlstm_gates: state rows of %ld floats, wanted %ld", state_ld, (long)heads * (K + 1));
  cudaError_t e = cudaSuccess;
  const dim3 grid(heads, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
#define GI_GATES(NPL, CH)                                                                                                      \
  GI_DISPATCH_DTYPE(dtype, T, e = (launch_gates<T, NPL, CH>(grid, s, keep, put, out_scale, q, ldq, k, ldk, gate_i, gate_f, ldg, \
                                                            bias_i, bias_f, cap, q_scale, state, state_ld, state_rows,          \
                                                            cu_seqlens, seq_slots, heads, K)))
  if (K <= 32) GI_GATES(1, 32);
  else if (K <= 64) GI_GATES(2, 32);
  else if (K <= 128) GI_GATES(4, 32);
  else if (K <= 256) GI_GATES(8, 16);
  else GI_GATES(16, 8);
#undef GI_GATES
  return gi::check(e, "mlstm_gates");
}
