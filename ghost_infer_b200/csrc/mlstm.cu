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
// grid (heads, sequences), one warp a block: lane l holds entries l, l + 32, ... of n.  The walk is serial in t; the rows of the
// next tokens do not depend on it, so their loads are issued ahead.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int ML_MAX_PER_LANE = 16;      // keys of up to 512 numbers

__device__ __forceinline__ float log_sigmoid_f(float x) { return fminf(x, 0.f) - log1pf(expf(-fabsf(x))); }

template <typename T>
__global__ void __launch_bounds__(32)
mlstm_gates_kernel(float* __restrict__ keep_out, float* __restrict__ put_out, float* __restrict__ scale_out, const T* q, long ldq,
                   const T* k, long ldk, const T* gi_in, const T* gf_in, long ldg, const float* __restrict__ bi,
                   const float* __restrict__ bf, float cap, float q_scale, float* state, long state_ld, int state_rows,
                   const int* cu_seqlens, const int* seq_slots, int heads, int K) {
  gi::pdl_prologue();
  const int h = blockIdx.x, b = blockIdx.y, lane = threadIdx.x;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  if (qlen <= 0) return;
  const int slot = seq_slots[b];
  float* st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld + (size_t)h * (K + 1);
  float n[ML_MAX_PER_LANE];
#pragma unroll
  for (int i = 0; i < ML_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    n[i] = e < K ? st[e] : 0.f;
  }
  float m = st[K];
  const float bias_i = bi != nullptr ? bi[h] : 0.f, bias_f = bf != nullptr ? bf[h] : 0.f;
  for (int t = 0; t < qlen; ++t) {
    const size_t tok = (size_t)tok0 + t;
    float kk[ML_MAX_PER_LANE], qq[ML_MAX_PER_LANE];
#pragma unroll
    for (int i = 0; i < ML_MAX_PER_LANE; ++i) {
      const int e = lane + 32 * i;
      kk[i] = e < K ? gi::ldf(k + tok * ldk + (size_t)h * K + e) : 0.f;
      qq[i] = e < K ? gi::ldf(q + tok * ldq + (size_t)h * K + e) : 0.f;
    }
    const float a = gi::ldf(gi_in + tok * ldg + h) + bias_i, bb = gi::ldf(gf_in + tok * ldg + h) + bias_f;
    const float ig = cap * tanhf(a / cap);
    const float fg = log_sigmoid_f(cap * tanhf(bb / cap));
    const float m_new = fmaxf(fg + m, ig);
    const float keep = expf(fg + m - m_new), put = expf(ig - m_new);
    float dot = 0.f;
#pragma unroll
    for (int i = 0; i < ML_MAX_PER_LANE; ++i) {
      n[i] = fmaf(put, kk[i], keep * n[i]);
      dot = fmaf(n[i], qq[i], dot);
    }
    dot = gi::warp_sum(dot) * q_scale;
    m = m_new;
    if (lane == 0) {
      keep_out[tok * heads + h] = keep;
      put_out[tok * heads + h] = put;
      scale_out[tok * heads + h] = q_scale / (fmaxf(fabsf(dot), expf(-m_new)) + 1e-6f);
    }
  }
#pragma unroll
  for (int i = 0; i < ML_MAX_PER_LANE; ++i) {
    const int e = lane + 32 * i;
    if (e < K) st[e] = n[i];
  }
  if (lane == 0) st[K] = m;
}

}  // namespace

extern "C" int gi_mlstm_gates(float* keep, float* put, float* out_scale, const void* q, long ldq, const void* k, long ldk,
                              const void* gate_i, const void* gate_f, long ldg, int dtype, const float* bias_i, const float* bias_f,
                              float cap, float q_scale, float* state, long state_ld, int state_rows, const int* cu_seqlens,
                              const int* seq_slots, int n_seqs, int heads, int K, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (heads <= 0 || K <= 0 || K > 32 * ML_MAX_PER_LANE) return gi::fail(GI_ERR_UNSUPPORTED, "mlstm_gates: keys of %d numbers (at most %d)", K, 32 * ML_MAX_PER_LANE);
  if (!(cap > 0.f)) return gi::fail(GI_ERR_ARG, "mlstm_gates: the gates' cap must be positive");
  if (state_ld < (long)heads * (K + 1)) return gi::fail(GI_ERR_ARG, "mlstm_gates: state rows of %ld floats, wanted %ld", state_ld, (long)heads * (K + 1));
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(mlstm_gates_kernel<T>, dim3(heads, n_seqs), dim3(32), 0, (cudaStream_t)stream, keep, put, out_scale, (const T*)q, ldq,
                     (const T*)k, ldk, (const T*)gate_i, (const T*)gate_f, ldg, bias_i, bias_f, cap, q_scale, state, state_ld, state_rows,
                     cu_seqlens, seq_slots, heads, K));
  return gi::check(e, "mlstm_gates");
}
