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
template <typename T> __device__ __forceinline__ float rounded(float v);
template <> __device__ __forceinline__ float rounded<float>(float v) { return v; }
template <> __device__ __forceinline__ float rounded<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

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


// ---- the same three kernels, four neighbouring channels a thread, 16 bytes a load: for widths that are multiples of 4 and
// rows that start on 16-byte boundaries.  A row's sums are formed in an order that follows from the width alone here too.

// hyper_read; with `conv_out` the input convolution as well, for steps of one token a sequence (every older input comes from
// the sequence's state): c = h + sum of taps, h rounded to the activation type first, as the separate kernel reads it.
template <typename TO, typename TW, typename TK>
__global__ void __launch_bounds__(256)
hyper_read4_kernel(TO* __restrict__ h, const float* x, const float* __restrict__ a, const TW* __restrict__ w, float* __restrict__ zero,
                   int S, int d, float eps, TO* __restrict__ conv_out, const TK* __restrict__ k, const float* state, long state_ld,
                   int state_rows, const int* slots, int taps) {
  extern __shared__ __align__(16) float u[];
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const size_t t = blockIdx.x;
  const float* xr = x + t * S * d;
  float ss = 0.f;
  for (int c = threadIdx.x * 4; c < d; c += 1024) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s = 0; s < S; ++s) {
      const float4 v = *reinterpret_cast<const float4*>(xr + (size_t)s * d + c);
      const float as = a[s];
      acc.x = fmaf(as, v.x, acc.x); acc.y = fmaf(as, v.y, acc.y); acc.z = fmaf(as, v.z, acc.z); acc.w = fmaf(as, v.w, acc.w);
    }
    *reinterpret_cast<float4*>(u + c) = acc;
    ss = fmaf(acc.x, acc.x, ss); ss = fmaf(acc.y, acc.y, ss); ss = fmaf(acc.z, acc.z, ss); ss = fmaf(acc.w, acc.w, ss);
  }
  // (a thread's share of the row's sum is four neighbouring channels here, every 256th in the plain kernel: the two kernels
  // differ by rounding; which of them runs follows from the width and the alignment alone, never from the step)
  const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)d + eps);
  const float* st = nullptr;
  if (conv_out != nullptr && taps > 1) {
    const int slot = slots[t];
    st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld;
  }
  for (int c = threadIdx.x * 4; c < d; c += 1024) {
    const float4 uv = *reinterpret_cast<const float4*>(u + c);
    const float4 wv = gi::ld4(w + c);
    float4 hv = make_float4(uv.x * rs * wv.x, uv.y * rs * wv.y, uv.z * rs * wv.z, uv.w * rs * wv.w);
    gi::st4(h + t * d + c, hv);
    if (zero != nullptr) *reinterpret_cast<float4*>(zero + t * d + c) = make_float4(0.f, 0.f, 0.f, 0.f);
    if (conv_out != nullptr) {
      float own[4] = {hv.x, hv.y, hv.z, hv.w};
      float out[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        own[e] = rounded<TO>(own[e]);       // as the stored row holds it
        float acc = own[e];
        for (int j = 0; j < taps; ++j) {
          const float v = j == taps - 1 ? own[e] : st[(size_t)j * d + c + e];
          acc = fmaf(gi::ldf(k + (size_t)(c + e) * taps + j), v, acc);
        }
        out[e] = acc;
      }
      gi::st4(conv_out + t * d + c, make_float4(out[0], out[1], out[2], out[3]));
    }
  }
}

// TAPS > 0: the number of taps is known when the kernel is compiled, and a thread's 4 x TAPS weights arrive as TAPS loads of
// four numbers into registers; TAPS 0: any number of taps, the weights read one by one.
template <typename T, typename TW, int TAPS>
__global__ void __launch_bounds__(256)
input_conv4_kernel(T* __restrict__ out, const T* h, const TW* __restrict__ k, const float* state, long state_ld, int state_rows,
                   const int* slots, int d, int taps_arg) {
  gi::pdl_prologue();
  const int taps = TAPS > 0 ? TAPS : taps_arg;
  const int t = blockIdx.x;
  const int slot = slots[t];
  const int q = rows_before(slots, t, taps - 1);
  const float* st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld;
  for (int c = (blockIdx.y * 256 + threadIdx.x) * 4; c < d; c += gridDim.y * 1024) {
    float kw[TAPS > 0 ? 4 * TAPS : 1];
    if (TAPS > 0) {
#pragma unroll
      for (int i = 0; i < TAPS; ++i) {
        const float4 w4 = gi::ld4(k + (size_t)c * TAPS + 4 * i);
        kw[4 * i] = w4.x; kw[4 * i + 1] = w4.y; kw[4 * i + 2] = w4.z; kw[4 * i + 3] = w4.w;
      }
    }
    const float4 o4 = gi::ld4(h + (size_t)t * d + c);
    const float own[4] = {o4.x, o4.y, o4.z, o4.w};
    float acc[4] = {own[0], own[1], own[2], own[3]};
#pragma unroll
    for (int j = 0; j < (TAPS > 0 ? TAPS : MAX_TAPS); ++j) {
      if (j < taps) {
        const int back = taps - 1 - j;
        float4 v4 = o4;
        if (back > 0) v4 = back <= q ? gi::ld4(h + (size_t)(t - back) * d + c) : *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 - back + q) * d + c);
        const float v[4] = {v4.x, v4.y, v4.z, v4.w};
#pragma unroll
        for (int e = 0; e < 4; ++e) acc[e] = fmaf(TAPS > 0 ? kw[e * (TAPS > 0 ? TAPS : 1) + j] : gi::ldf(k + (size_t)(c + e) * taps + j), v[e], acc[e]);
      }
    }
    gi::st4(out + (size_t)t * d + c, make_float4(acc[0], acc[1], acc[2], acc[3]));
  }
}

// SMAX: the most copies this instance holds in registers (4 or MAX_STREAMS)
template <typename T, typename TW, int SMAX>
__global__ void __launch_bounds__(256)
hyper_write4_kernel(float* x, const float* y, const T* z, const TW* __restrict__ zb, const float* __restrict__ M,
                    const float* __restrict__ o, const T* h, float* state, long state_ld, int state_rows, const int* slots,
                    int n_tokens, int S, int d, int taps) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  float* xr = x + (size_t)t * S * d;
  for (int c = (blockIdx.y * 256 + threadIdx.x) * 4; c < d; c += gridDim.y * 1024) {
    float4 v = *reinterpret_cast<const float4*>(y + (size_t)t * d + c);
    if (z != nullptr) {
      const float4 g = gi::ld4(z + (size_t)t * d + c);
      float4 b = make_float4(0.f, 0.f, 0.f, 0.f);
      if (zb != nullptr) b = gi::ld4(zb + c);
      v.x *= sigmoid_f(g.x + b.x); v.y *= sigmoid_f(g.y + b.y); v.z *= sigmoid_f(g.z + b.z); v.w *= sigmoid_f(g.w + b.w);
    }
    float4 old[SMAX];
#pragma unroll
    for (int s = 0; s < SMAX; ++s)
      if (s < S) old[s] = *reinterpret_cast<const float4*>(xr + (size_t)s * d + c);
    for (int to = 0; to < S; ++to) {
      float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
      for (int s = 0; s < SMAX; ++s)
        if (s < S) {
          const float m = M[s * S + to];
          acc.x = fmaf(m, old[s].x, acc.x); acc.y = fmaf(m, old[s].y, acc.y); acc.z = fmaf(m, old[s].z, acc.z); acc.w = fmaf(m, old[s].w, acc.w);
        }
      const float sh = o[to];
      acc.x = fmaf(sh, v.x, acc.x); acc.y = fmaf(sh, v.y, acc.y); acc.z = fmaf(sh, v.z, acc.z); acc.w = fmaf(sh, v.w, acc.w);
      *reinterpret_cast<float4*>(xr + (size_t)to * d + c) = acc;
    }
  }
  if (state == nullptr || taps <= 1) return;
  const int slot = slots[t];
  if (t + 1 < n_tokens && slots[t + 1] == slot) return;       // not the sequence's last token of this step
  const int q = rows_before(slots, t, taps - 1);
  float* st = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld;
  for (int c = (blockIdx.y * 256 + threadIdx.x) * 4; c < d; c += gridDim.y * 1024) {
    float4 keep[MAX_TAPS - 1];
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i) {
      if (i < taps - 1) {
        const int back = taps - 2 - i;
        keep[i] = back <= q ? gi::ld4(h + (size_t)(t - back) * d + c) : *reinterpret_cast<const float4*>(st + (size_t)(taps - 1 - back + q) * d + c);
      }
    }
#pragma unroll
    for (int i = 0; i < MAX_TAPS - 1; ++i)
      if (i < taps - 1) *reinterpret_cast<float4*>(st + (size_t)i * d + c) = keep[i];
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
// four channels a thread: every thread one group of four where the row is not longer than 64 blocks' worth
inline unsigned col_blocks4(int d) { return (unsigned)max(1, min(64, (d + 1023) / 1024)); }
inline bool aligned16(const void* p) { return (((uintptr_t)p) & 15) == 0; }

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
  return gi_hyper_read_conv(h, dtype, x, blend, w, w_dtype, zero, n_tokens, streams, d, eps, nullptr, nullptr, GI_F32, nullptr, 0, 0,
                            nullptr, 0, stream);
}

// The same and, for a step of one token a sequence, the input convolution in the same launch: conv_out = h + sum of taps,
// the older inputs from the state (see gi_input_conv).  Needs a width that is a multiple of 4 and 16-byte aligned rows.
extern "C" int gi_hyper_read_conv(void* h, int dtype, const float* x, const float* blend, const void* w, int w_dtype, float* zero,
                                  int n_tokens, int streams, int d, float eps, void* conv_out, const void* taps_w, int k_dtype,
                                  const float* state, long state_ld, int state_rows, const int* slots, int taps, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  const bool vec = d % 4 == 0 && aligned16(h) && aligned16(x) && aligned16(w) && aligned16(zero) && aligned16(conv_out) &&
                   aligned16(state) && state_ld % 4 == 0;
  if (conv_out != nullptr) {
    if (!vec) return gi::fail(GI_ERR_UNSUPPORTED, "hyper_read: the convolution in the same launch needs a width that is a multiple of 4 and aligned rows");
    if (taps < 1 || taps > MAX_TAPS || taps_w == nullptr || slots == nullptr || (taps > 1 && (state == nullptr || state_ld < (long)(taps - 1) * d)))
      return gi::fail(GI_ERR_ARG, "hyper_read: the convolution needs 1 to %d taps, its weights, the slots and its state", MAX_TAPS);
  }
  if (streams < 1 || streams > MAX_STREAMS || d < 1) return gi::fail(GI_ERR_UNSUPPORTED, "hyper_read: %d copies of the stream (at most %d)", streams, MAX_STREAMS);
  const size_t smem = (size_t)d * sizeof(float);
  if (smem > 200 * 1024) return gi::fail(GI_ERR_UNSUPPORTED, "hyper_read: rows of %d values are wider than shared memory", d);
  cudaError_t e = cudaSuccess;
  if (vec) {
    GI_DISPATCH_DTYPE(dtype, TO, GI_DISPATCH_DTYPE(w_dtype, TW, GI_DISPATCH_DTYPE(k_dtype, TK, {
      auto kern = hyper_read4_kernel<TO, TW, TK>;
      if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        e = gi::launch(kern, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (TO*)h, x, blend, (const TW*)w, zero, streams, d, eps,
                       (TO*)conv_out, (const TK*)taps_w, state, state_ld, state_rows, slots, taps);
    })));
    return gi::check(e, "hyper_read");
  }
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
  if (d % 4 == 0 && aligned16(out) && aligned16(h) && aligned16(state) && state_ld % 4 == 0) {
    GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
        {
          auto kern = input_conv4_kernel<T, TW, 0>;
          if (taps == 2) kern = input_conv4_kernel<T, TW, 2>;
          else if (taps == 3) kern = input_conv4_kernel<T, TW, 3>;
          else if (taps == 4) kern = input_conv4_kernel<T, TW, 4>;
          e = gi::launch(kern, dim3(n_tokens, col_blocks4(d)), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)h,
                         (const TW*)taps_w, state, state_ld, state_rows, slots, d, taps);
        }));
    return gi::check(e, "input_conv");
  }
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
  if (d % 4 == 0 && aligned16(x) && aligned16(y) && aligned16(z) && aligned16(z_bias) && aligned16(h) && aligned16(state) && state_ld % 4 == 0) {
    GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
        {
          auto kern = streams <= 4 ? hyper_write4_kernel<T, TW, 4> : hyper_write4_kernel<T, TW, MAX_STREAMS>;
          e = gi::launch(kern, dim3(n_tokens, col_blocks4(d)), dim3(256), 0, (cudaStream_t)stream, x, y, (const T*)z, (const TW*)z_bias,
                         mix, share, (const T*)h, state, state_ld, state_rows, slots, n_tokens, streams, d, taps);
        }));
    return gi::check(e, "hyper_write");
  }
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
