// Row kernels for layers that keep several copies of the residual stream ("hyper-connections"), read a learned blend of
// them, and write every copy back as a learned mix of the old copies plus a share of the sublayer's output; with a short
// causal convolution in front of every sublayer and a sigmoid gate on what it returns.
//
// The copies of a token lie side by side: x [tokens][S][d], 32-bit.
//  * stream_expand:  x[t][s] = e[t] for every s (all copies start as the embedded token).
//  * stream_sum:     out[r] = sum_s x[row(r)][s] (what the final norm reads), in the order of s.
//  * hyper_read:     u = sum_s a[s] x[t][s];  h[t] = u / sqrt(mean(u^2) + eps) * w in the activation type; optionally a
//                    matrix of 32-bit rows is zeroed in the same pass (the rows the sublayer adds its output into).
//  * input_conv:     c[t] = h[t] + sum_j k[:, j] h[t - taps + 1 + j] per channel, zeros before the sequence's start.  Inputs
//                    older than the step come from the sequence's state (its last taps - 1 inputs, oldest first).
//  * hyper_write:    g = sigmoid(z[t] + b) (z: a projection of h, or absent);  x[t][to] = sum_s M[s][to] x[t][s] + o[to] g y[t],
//                    all copies at once from the old ones.  The block of a sequence's last token of the step also renews the
//                    convolution's state from h (and from the old state where the step brought fewer than taps - 1 tokens).
//  * scale_rows:     x *= c.
// Sums over the copies, the norm, the gate and the mix are 32-bit.  A row's sums follow from the width alone.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int MAX_STREAMS = 16;
constexpr int MAX_TAPS = 8;

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

__global__ void stream_expand_kernel(float* __restrict__ x, const float* __restrict__ e, int S, int d, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / d, c = i % d;
  const float v = e[i];
  for (int s = 0; s < S; ++s) x[(t * S + s) * d + c] = v;
}

__global__ void stream_sum_kernel(float* __restrict__ out, const float* __restrict__ x, const int* __restrict__ rows, int S, int d,
                                  size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t r = i / d, c = i % d;
  const size_t t = rows != nullptr ? (size_t)rows[r] : r;
  float acc = 0.f;
  for (int s = 0; s < S; ++s) acc += x[(t * S + s) * d + c];
  out[i] = acc;
}

// One block per token; the blend of the copies is kept in shared memory between the two passes.
template <typename TO, typename TW>
__global__ void __launch_bounds__(256)
hyper_read_kernel(TO* __restrict__ h, const float* x, const float* __restrict__ a, const TW* __restrict__ w, float* __restrict__ zero,
                  int S, int d, float eps) {
  extern __shared__ float u[];
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const size_t t = blockIdx.x;
  const float* xr = x + t * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x; c < d; c += 256) {
    float acc = 0.f;
    for (int s = 0; s < S; ++s) acc = fmaf(a[s], xr[(size_t)s * d + c], acc);
    u[c] = acc;
    ss = fmaf(acc, acc, ss);
  }
  const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)d + eps);
  for (int c = threadIdx.x; c < d; c += 256) {
    gi::stf(h + t * d + c, u[c] * rs * gi::ldf(w + c));
    if (zero != nullptr) zero[t * d + c] = 0.f;
  }
}

// How many rows directly before row t belong to the same sequence, counted up to `most`.
__device__ __forceinline__ int rows_before(const int* slots, int t, int most) {
  const int slot = slots[t];
  int q = 0;
  while (q < most && t - q - 1 >= 0 && slots[t - q - 1] == slot) ++q;
  return q;
}

template <typename T, typename TW>
__global__ void __launch_bounds__(256)
input_conv_kernel(T* __restrict__ out, const T* h, const TW* __restrict__ k, const float* state, long state_ld, int state_rows,
                  const int* slots, int d, int taps) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const int slot = slots[t];
  const int q = rows_before(slots, t, taps - 1);
  const float* st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld;
  for (int c = blockIdx.y * 256 + threadIdx.x; c < d; c += gridDim.y * 256) {
    const float own = gi::ldf(h + (size_t)t * d + c);
    float acc = own;
    for (int j = 0; j < taps; ++j) {
      const int back = taps - 1 - j;
      // the input `back` tokens ago: a row of this step, or entry (taps - 1 - back + q) of the state
      const float v = back == 0 ? own : (back <= q ? gi::ldf(h + (size_t)(t - back) * d + c) : st[(size_t)(taps - 1 - back + q) * d + c]);
      acc = fmaf(gi::ldf(k + (size_t)c * taps + j), v, acc);
    }
    gi::stf(out + (size_t)t * d + c, acc);
  }
}

template <typename T, typename TW>
__global__ void __launch_bounds__(256)
hyper_write_kernel(float* x, const float* y, const T* z, const TW* __restrict__ zb, const float* __restrict__ M,
                   const float* __restrict__ o, const T* h, float* state, long state_ld, int state_rows, const int* slots,
                   int n_tokens, int S, int d, int taps) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * S * d;
  for (int c = blockIdx.y * 256 + threadIdx.x; c < d; c += gridDim.y * 256) {
    float v = y[(size_t)t * d + c];
    if (z != nullptr) v *= sigmoid_f(gi::ldf(z + (size_t)t * d + c) + (zb != nullptr ? gi::ldf(zb + c) : 0.f));
    float old[MAX_STREAMS];
#pragma unroll
    for (int s = 0; s < MAX_STREAMS; ++s) old[s] = s < S ? xr[(size_t)s * d + c] : 0.f;
    for (int to = 0; to < S; ++to) {
      float acc = 0.f;
#pragma unroll
      for (int s = 0; s < MAX_STREAMS; ++s)
        if (s < S) acc = fmaf(M[s * S + to], old[s], acc);
      xr[(size_t)to * d + c] = fmaf(o[to], v, acc);
    }
  }
  if (state == nullptr || taps <= 1) return;
  const int slot = slots[t];
  if (t + 1 < n_tokens && slots[t + 1] == slot) return;       // not the sequence's last token of this step
  const int q = rows_before(slots, t, taps - 1);
  float* st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld;
  for (int c = blockIdx.y * 256 + threadIdx.x; c < d; c += gridDim.y * 256) {
    float keep[MAX_TAPS - 1];
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i) {
      if (i < taps - 1) {
        const int back = taps - 2 - i;        // entry i is the input `back` tokens before this one
        keep[i] = back <= q ? gi::ldf(h + (size_t)(t - back) * d + c) : st[(size_t)(taps - 1 - back + q) * d + c];
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i)
      if (i < taps - 1) st[(size_t)i * d + c] = keep[i];
  }
}

__global__ void scale_rows_kernel(float* x, float c, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i < total) x[i] *= c;
}

inline unsigned blocks_of(size_t total) { return (unsigned)((total + 255) / 256); }
// few tokens: a row's channels over several blocks
inline unsigned col_blocks(int n_tokens, int d) { return n_tokens >= 128 ? 1u : (unsigned)min(16, (d + 255) / 256); }

}  // namespace

extern "C" int gi_stream_expand(float* x, const float* e, int n_tokens, int streams, int d, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (streams < 1 || d < 1) return gi::fail(GI_ERR_ARG, "stream_expand: bad sizes");
  const size_t total = (size_t)n_tokens * d;
  return gi::check(gi::launch(stream_expand_kernel, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, x, e, streams, d, total),
                   "stream_expand");
}

extern "C" int gi_stream_sum(float* out, const float* x, const int* rows, int n_rows, int streams, int d, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (streams < 1 || d < 1) return gi::fail(GI_ERR_ARG, "stream_sum: bad sizes");
  const size_t total = (size_t)n_rows * d;
  return gi::check(gi::launch(stream_sum_kernel, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, out, x, rows, streams, d, total),
                   "stream_sum");
}

extern "C" int gi_hyper_read(void* h, int dtype, const float* x, const float* blend, const void* w, int w_dtype, float* zero,
                             int n_tokens, int streams, int d, float eps, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (streams < 1 || streams > MAX_STREAMS || d < 1) return gi::fail(GI_ERR_UNSUPPORTED, "hyper_read: %d copies of the stream (at most %d)", streams, MAX_STREAMS);
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return gi::fail(GI_ERR_UNSUPPORTED, "hyper_read: rows of %d values are wider than shared memory", d);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, TO, GI_DISPATCH_DTYPE(w_dtype, TW, {
    auto kern = hyper_read_kernel<TO, TW>;
    if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e == cudaSuccess)
      e = gi::launch(kern, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (TO*)h, x, blend, (const TW*)w, zero, streams, d, eps);
  }));
  return gi::check(e, "hyper_read");
}

extern "C" int gi_input_conv(void* out, const void* h, int dtype, const void* taps_w, int w_dtype, const float* state, long state_ld,
                             int state_rows, const int* slots, int n_tokens, int d, int taps, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (taps < 1 || taps > MAX_TAPS || d < 1) return gi::fail(GI_ERR_UNSUPPORTED, "input_conv: %d taps (1 to %d)", taps, MAX_TAPS);
  if (taps > 1 && (state == nullptr || state_ld < (long)(taps - 1) * d)) return gi::fail(GI_ERR_ARG, "input_conv: no room for the last inputs");
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(input_conv_kernel<T, TW>, dim3(n_tokens, col_blocks(n_tokens, d)), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                     (const T*)h, (const TW*)taps_w, state, state_ld, state_rows, slots, d, taps)));
  return gi::check(e, "input_conv");
}

extern "C" int gi_hyper_write(float* x, const float* y, const void* z, const void* z_bias, int dtype, int w_dtype, const float* mix,
                              const float* share, const void* h, float* state, long state_ld, int state_rows, const int* slots,
                              int n_tokens, int streams, int d, int taps, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (streams < 1 || streams > MAX_STREAMS || d < 1) return gi::fail(GI_ERR_UNSUPPORTED, "hyper_write: %d copies of the stream (at most %d)", streams, MAX_STREAMS);
  if (state != nullptr && (taps < 1 || taps > MAX_TAPS || h == nullptr || state_ld < (long)(taps - 1) * d))
    return gi::fail(GI_ERR_ARG, "hyper_write: the convolution's state needs 1 to %d taps, the inputs and room for them", MAX_TAPS);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(hyper_write_kernel<T, TW>, dim3(n_tokens, col_blocks(n_tokens, d)), dim3(256), 0, (cudaStream_t)stream, x, y,
                     (const T*)z, (const TW*)z_bias, mix, share, (const T*)h, state, state_ld, state_rows, slots, n_tokens, streams, d,
                     taps)));
  return gi::check(e, "hyper_write");
}

extern "C" int gi_scale_rows(float* x, float c, long n_values, void* stream) {
  if (n_values <= 0) return GI_OK;
  return gi::check(gi::launch(scale_rows_kernel, dim3(blocks_of((size_t)n_values)), dim3(256), 0, (cudaStream_t)stream, x, c, (size_t)n_values),
                   "scale_rows");
}
