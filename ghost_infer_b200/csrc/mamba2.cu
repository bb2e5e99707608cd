// The Mamba-2 (state-space duality) mixer's own steps, between its input and output projections.
//
// The input projection's rows are [z: inner | x: inner | B: G*N | C: G*N | dt: heads], inner = heads * P.
//  * conv:  the channels [x | B | C] pass a causal convolution over `taps` tokens per channel, plus bias, then silu.
//           Inputs before a step's first token come from the sequence's state (zeros for a fresh sequence).
//  * scan:  dt <- softplus(dt + dt_bias); per head (head h reads group h / (heads / G) of B and C)
//           S <- exp(-exp(A_log) dt) S + dt B x^T   (S is N x P),   y = S^T C + D x.
//           Everything here is 32-bit; the tokens of a sequence are walked in order, thirty-two at a time through shared
//           memory; a warp owns two or four columns p of S, its lanes the rows n, kept in registers across the step.
//           One token or a thousand, alone or in a batch, take the same arithmetic in the same order: no bit changes.
//  * gate + norm: y * silu(z), divided by the root mean square of each of `parts` equal parts, times a weight.
// Per-sequence state: one float row per slot, [S: heads * P * N, a column's N rows side by side (a lane's rows are then
// neighbours in memory: a one-token step, which is all loading and storing of S, moves whole lines) | last taps - 1 conv
// inputs: (taps - 1) * channels];
// slot -1 (a padding row of a fixed-size launch) uses the last row of the matrix.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {


__device__ __forceinline__ float silu_f(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float softplus_f(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// grid (token tiles of 8, sequences, channel tiles of 256): a thread takes one channel of eight tokens
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
conv_kernel(T* __restrict__ out, const T* __restrict__ proj, long ld_proj, const TW* __restrict__ w,
            const TW* __restrict__ bias, const float* __restrict__ state, long state_ld, int state_rows,
            const int* __restrict__ cu_seqlens, const int* __restrict__ seq_slots, int inner, int channels, int taps,
            int s_floats) {
  gi::pdl_prologue();
  const int b = blockIdx.y;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  const int i0 = blockIdx.x * 8;
  if (i0 >= qlen) return;
  const int slot = seq_slots[b];
  const float* cs = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld + s_floats;
  const int n_here = min(8, qlen - i0);
  const int c = blockIdx.z * 256 + threadIdx.x;
  if (c < channels) {
    const float bc = gi::ldf(bias + c);
    for (int ii = 0; ii < n_here; ++ii) {
      const int i = i0 + ii;
      float acc = bc;
      for (int j = 0; j < taps; ++j) {
        const int src = i - (taps - 1) + j;
        const float v = src >= 0 ? gi::ldf(proj + (size_t)(tok0 + src) * ld_proj + inner + c)
                                 : cs[(size_t)(src + taps - 1) * channels + c];
        acc = fmaf(gi::ldf(w + (size_t)c * taps + j), v, acc);
      }
      gi::stf(out + (size_t)(tok0 + i) * channels + c, silu_f(acc));
    }
  }
}

// grid (channel blocks, sequences): the state takes the last taps - 1 inputs of [old state | this step's inputs]
template <typename T>
__global__ void conv_update_kernel(const T* __restrict__ proj, long ld_proj, float* __restrict__ state, long state_ld,
                                   int state_rows, const int* __restrict__ cu_seqlens,
                                   const int* __restrict__ seq_slots, int inner, int channels, int taps, int s_floats) {
  gi::pdl_prologue();
  const int b = blockIdx.y;
  const int c = blockIdx.x * blockDim.x + threadIdx.x;
  if (c >= channels) return;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  if (qlen <= 0) return;
  const int slot = seq_slots[b];
  float* cs = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld + s_floats;
  const int keep = taps - 1;
  // place k of the new state is place qlen + k of [old state (keep) | inputs (qlen)]; walking k upwards reads old
  // places qlen + k > k only, which are not yet overwritten
  for (int k = 0; k < keep; ++k) {
    const int at = qlen + k;
    const float v = at < keep ? cs[(size_t)at * channels + c] : gi::ldf(proj + (size_t)(tok0 + at - keep) * ld_proj + inner + c);
    cs[(size_t)k * channels + c] = v;
  }
}

// grid (heads, sequences, column tiles of SC_W * SC_CPW); a warp owns SC_CPW (two or four) columns p of the head's state, its lanes the
// rows (lane l of NPT >= 4 rows owns rows (32 j + l) 4 .. + 3 for j = 0 .. NPT / 4 - 1, so that a warp reads B and C as
// whole 16-byte words side by side; of fewer rows, l NPT .. + NPT - 1), in registers for the whole step.  Tokens go
// through shared memory SC_CH at a time (rows past N padded with zeros, which leave their state at zero); B_t and C_t
// are read once per token for all of a warp's columns.  A token's sum over the rows stays per lane for SC_RB tokens,
// then the 32 (token, column) sums of a warp are added across its lanes in one halving exchange (31 shuffles instead of
// 160), after which lane SC_CPW t + c holds token t, column c.  The order of every sum follows from N alone.
constexpr int SC_W = 4, SC_CH = 32;

// One halving step of the exchange: of 2 * HALF values a lane keeps the half its bit `BIT` of the lane number names and
// adds the other lane's partial sums of the same values.
template <int HALF, int BIT>
__device__ __forceinline__ void halve(float (&v)[32], int lane) {
  const bool upper = (lane & BIT) != 0;
#pragma unroll
  for (int k = 0; k < HALF; ++k) {
    const float send = upper ? v[k] : v[k + HALF];
    const float keep = upper ? v[k + HALF] : v[k];
    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, BIT);
  }
}

template <typename T, typename TW, int NPT, int SC_CPW>
__global__ void __launch_bounds__(SC_W * 32)
scan_kernel(float* __restrict__ y, const T* __restrict__ xbc, const T* __restrict__ proj, long ld_proj,
            const TW* __restrict__ dt_bias, const TW* __restrict__ a_log, const TW* __restrict__ d_skip,
            float* __restrict__ state, long state_ld, int state_rows, const int* __restrict__ cu_seqlens,
            const int* __restrict__ seq_slots, int heads, int P, int N, int groups) {
  constexpr int NP = 32 * NPT;       // rows with padding
  constexpr int SC_COLS = SC_W * SC_CPW, SC_RB = 32 / SC_CPW, SC_CPW_LOG2 = SC_CPW == 2 ? 1 : 2;
  static_assert(SC_CPW == 2 || SC_CPW == 4, "a warp takes 2 or 4 columns");
  extern __shared__ __align__(16) float sm[];
  float* sB = sm;                    // [SC_CH][NP]
  float* sC = sB + SC_CH * NP;       // [SC_CH][NP]
  float* sx = sC + SC_CH * NP;       // [SC_CH][SC_COLS]
  float* sdt = sx + SC_CH * SC_COLS; // [SC_CH]
  float* sdA = sdt + SC_CH;          // [SC_CH]
  gi::pdl_prologue();
  const int h = blockIdx.x, b = blockIdx.y, p0 = blockIdx.z * SC_COLS;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  if (qlen <= 0) return;
  const int slot = seq_slots[b];
  float* S_row = state + (size_t)(slot >= 0 ? slot : state_rows - 1) * state_ld + (size_t)h * N * P;
  const int g = h / (heads / groups);
  const int inner = heads * P, channels = inner + 2 * groups * N;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int pw = p0 + warp * SC_CPW;             // this warp's first column
  // row of this lane's i-th value
  auto row_of = [&](int i) { return NPT >= 4 ? ((i >> 2) * 32 + lane) * 4 + (i & 3) : lane * NPT + i; };
  float S[SC_CPW][NPT];
#pragma unroll
  for (int c = 0; c < SC_CPW; ++c)
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = row_of(i);
      S[c][i] = (pw + c < P && n < N) ? S_row[(size_t)(pw + c) * N + n] : 0.f;
    }
  const float A = -expf(gi::ldf(a_log + h)), D = gi::ldf(d_skip + h), bias = gi::ldf(dt_bias + h);

  for (int c0 = 0; c0 < qlen; c0 += SC_CH) {
    const int nc = min(SC_CH, qlen - c0);
    __syncthreads();
    for (int idx = tid; idx < nc * NP; idx += SC_W * 32) {
      const int t = idx / NP, n = idx % NP;
      float bv = 0.f, cv = 0.f;
      if (n < N) {
        const T* r = xbc + (size_t)(tok0 + c0 + t) * channels + inner + (size_t)g * N + n;
        bv = gi::ldf(r);
        cv = gi::ldf(r + (size_t)groups * N);
      }
      sB[idx] = bv;
      sC[idx] = cv;
    }
    for (int idx = tid; idx < nc * SC_COLS; idx += SC_W * 32) {
      const int t = idx / SC_COLS, j = idx % SC_COLS;
      sx[idx] = (p0 + j < P) ? gi::ldf(xbc + (size_t)(tok0 + c0 + t) * channels + (size_t)h * P + p0 + j) : 0.f;
    }
    for (int t = tid; t < nc; t += SC_W * 32) {
      const float dt = softplus_f(gi::ldf(proj + (size_t)(tok0 + c0 + t) * ld_proj + 2 * inner + 2 * groups * N + h) + bias);
      sdt[t] = dt;
      sdA[t] = expf(A * dt);
    }
    __syncthreads();
    for (int t0 = 0; t0 < nc; t0 += SC_RB) {
      float acc[32];                                  // [SC_RB tokens][SC_CPW columns]
#pragma unroll
      for (int tl = 0; tl < SC_RB; ++tl) {
        const int t = t0 + tl;
#pragma unroll
        for (int c = 0; c < SC_CPW; ++c) acc[tl * SC_CPW + c] = 0.f;
        if (t < nc) {                                 // the same for the whole block
          const float dA = sdA[t], dt = sdt[t];
          float bv[NPT], cv[NPT];
          if (NPT >= 4) {
#pragma unroll
            for (int j = 0; j < NPT / 4; ++j) {
              const float4 b4 = *reinterpret_cast<const float4*>(sB + t * NP + (j * 32 + lane) * 4);
              const float4 c4 = *reinterpret_cast<const float4*>(sC + t * NP + (j * 32 + lane) * 4);
              bv[4 * j] = b4.x; bv[4 * j + 1] = b4.y; bv[4 * j + 2] = b4.z; bv[4 * j + 3] = b4.w;
              cv[4 * j] = c4.x; cv[4 * j + 1] = c4.y; cv[4 * j + 2] = c4.z; cv[4 * j + 3] = c4.w;
            }
          } else {
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
              bv[i] = sB[t * NP + lane * NPT + i];
              cv[i] = sC[t * NP + lane * NPT + i];
            }
          }
#pragma unroll
          for (int i = 0; i < NPT; ++i) bv[i] *= dt;
#pragma unroll
          for (int c = 0; c < SC_CPW; ++c) {
            const float x = sx[t * SC_COLS + warp * SC_CPW + c];
            float a = 0.f;
#pragma unroll
            for (int i = 0; i < NPT; ++i) {
              S[c][i] = fmaf(dA, S[c][i], x * bv[i]);
              a = fmaf(S[c][i], cv[i], a);
            }
            acc[tl * SC_CPW + c] = a;
          }
        }
      }
      halve<16, 16>(acc, lane);
      halve<8, 8>(acc, lane);
      halve<4, 4>(acc, lane);
      halve<2, 2>(acc, lane);
      halve<1, 1>(acc, lane);
      // lane SC_CPW tl + c now holds token t0 + tl, column c
      const int t = t0 + (lane >> SC_CPW_LOG2), c = lane & (SC_CPW - 1);
      if (t < nc && pw + c < P)
        y[(size_t)(tok0 + c0 + t) * inner + (size_t)h * P + pw + c] = acc[0] + D * sx[t * SC_COLS + warp * SC_CPW + c];
    }
  }
#pragma unroll
  for (int c = 0; c < SC_CPW; ++c)
#pragma unroll
    for (int i = 0; i < NPT; ++i) {
      const int n = row_of(i);
      if (pw + c < P && n < N) S_row[(size_t)(pw + c) * N + n] = S[c][i];
    }
}

// grid (tokens, parts)
template <typename TO, typename T, typename TW>
__global__ void __launch_bounds__(256)
gate_norm_kernel(TO* __restrict__ out, const float* __restrict__ y, const T* __restrict__ proj, long ld_proj,
                 const TW* __restrict__ w, int inner, int parts, float eps) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const int t = blockIdx.x, part = blockIdx.y, gw = inner / parts, c0 = part * gw;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gw; i += blockDim.x) {
    const float v = y[(size_t)t * inner + c0 + i] * silu_f(gi::ldf(proj + (size_t)t * ld_proj + c0 + i));
    ss = fmaf(v, v, ss);
  }
  ss = gi::block_sum(ss, scratch);
  const float inv = 1.0f / sqrtf(ss / (float)gw + eps);
  for (int i = threadIdx.x; i < gw; i += blockDim.x) {
    const float v = y[(size_t)t * inner + c0 + i] * silu_f(gi::ldf(proj + (size_t)t * ld_proj + c0 + i));
    gi::stf(out + (size_t)t * inner + c0 + i, v * inv * gi::ldf(w + c0 + i));
  }
}

template <typename T, typename TW, int NPT, int CPW>
int launch_scan(dim3 grid, size_t smem, cudaStream_t s, float* y, const T* xbc, const T* proj, long ld_proj, const TW* dt_bias,
                const TW* a_log, const TW* d_skip, float* state, long state_ld, int state_rows, const int* cu, const int* slots,
                int heads, int P, int N, int groups) {
  auto kern = scan_kernel<T, TW, NPT, CPW>;
  if (smem > 48 * 1024) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "mamba2 scan: %s", cudaGetErrorString(e));
  }
  return gi::check(gi::launch(kern, grid, dim3(SC_W * 32), smem, s, y, xbc, proj, ld_proj, dt_bias, a_log, d_skip, state, state_ld,
                              state_rows, cu, slots, heads, P, N, groups), "mamba2 scan");
}

}  // namespace

extern "C" int gi_mamba2_conv(void* xbc_out, const void* proj, int dtype, long ld_proj, const void* conv_w,
                              const void* conv_b, int w_dtype, const float* state, long state_ld, int state_rows,
                              const int* cu_seqlens, const int* seq_slots, int n_seqs, int max_q_len, int inner,
                              int channels, int taps, int s_floats, void* stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GI_OK;
  if (taps < 1 || channels <= 0 || inner < 0) return gi::fail(GI_ERR_ARG, "mamba2 conv: bad sizes");
  if (n_seqs > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 conv: more than 65535 sequences in one launch");
  if ((channels + 255) / 256 > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 conv: %d channels are more than one launch takes", channels);
  dim3 grid((max_q_len + 7) / 8, n_seqs, (channels + 255) / 256);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(conv_kernel<T, TW>, grid, dim3(256), 0, (cudaStream_t)stream, (T*)xbc_out, (const T*)proj, ld_proj,
                     (const TW*)conv_w, (const TW*)conv_b, state, state_ld, state_rows, cu_seqlens, seq_slots, inner, channels,
                     taps, s_floats)));
  return gi::check(e, "mamba2 conv");
}

extern "C" int gi_mamba2_conv_update(const void* proj, int dtype, long ld_proj, float* state, long state_ld, int state_rows,
                                     const int* cu_seqlens, const int* seq_slots, int n_seqs, int inner, int channels,
                                     int taps, int s_floats, void* stream) {
  if (n_seqs <= 0 || taps <= 1) return GI_OK;
  if (n_seqs > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 conv: more than 65535 sequences in one launch");
  dim3 grid((channels + 127) / 128, n_seqs);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(conv_update_kernel<T>, grid, dim3(128), 0, (cudaStream_t)stream, (const T*)proj, ld_proj, state, state_ld,
                     state_rows, cu_seqlens, seq_slots, inner, channels, taps, s_floats));
  return gi::check(e, "mamba2 conv update");
}

extern "C" int gi_mamba2_scan(float* y, const void* xbc, const void* proj, int dtype, long ld_proj, const void* dt_bias,
                              const void* a_log, const void* d_skip, int w_dtype, float* state, long state_ld,
                              int state_rows, const int* cu_seqlens, const int* seq_slots, int n_seqs, int heads, int P,
                              int N, int groups, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (heads <= 0 || P <= 0 || N <= 0 || groups <= 0 || heads % groups != 0)
    return gi::fail(GI_ERR_ARG, "mamba2 scan: %d heads, %d groups, head size %d, state %d", heads, groups, P, N);
  if (n_seqs > 65535 || heads > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 scan: more than 65535 sequences or heads");
  if (N > 1024) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 scan: a state of %d rows is more than a warp's lanes take", N);
  int npt = 1;
  while (32 * npt < N) npt *= 2;
  // four columns a warp where that still gives every SM several blocks (B_t and C_t are then read once for four columns);
  // two where there are few heads and sequences (one prompt), for twice the warps.  Either way a sum's additions are
  // the same ones in the same order, so the choice changes no bit.
  const int cpw = ((long)heads * n_seqs * ((P + SC_W * 4 - 1) / (SC_W * 4)) >= 400) ? 4 : 2;
  const int cols = SC_W * cpw;
  dim3 grid(heads, n_seqs, (P + cols - 1) / cols);
  if (grid.z > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 scan: head size %d is more than one launch takes", P);
  const size_t smem = (2 * (size_t)SC_CH * 32 * npt + (size_t)SC_CH * cols + 2 * SC_CH) * sizeof(float);
  cudaStream_t s = (cudaStream_t)stream;
  int rc = GI_OK;
#define GI_SCAN_LAUNCH(NPT, CPW)                                                                                       \
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,                                                           \
      rc = (launch_scan<T, TW, NPT, CPW>(grid, smem, s, y, (const T*)xbc, (const T*)proj, ld_proj, (const TW*)dt_bias, \
                                         (const TW*)a_log, (const TW*)d_skip, state, state_ld, state_rows, cu_seqlens, \
                                         seq_slots, heads, P, N, groups))))
#define GI_SCAN_CASE(NPT)                                                                                              \
  case NPT:                                                                                                            \
    if (cpw == 4) GI_SCAN_LAUNCH(NPT, 4);                                                                              \
    else GI_SCAN_LAUNCH(NPT, 2);                                                                                       \
    break;
  switch (npt) {
    GI_SCAN_CASE(1)
    GI_SCAN_CASE(2)
    GI_SCAN_CASE(4)
    GI_SCAN_CASE(8)
    GI_SCAN_CASE(16)
    GI_SCAN_CASE(32)
  }
#undef GI_SCAN_LAUNCH
#undef GI_SCAN_CASE
  return rc;
}

extern "C" int gi_mamba2_gate_norm(void* out, int out_dtype, const float* y, const void* proj, int dtype, long ld_proj,
                                   const void* w, int w_dtype, int n_tokens, int inner, int parts, float eps,
                                   void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (parts <= 0 || inner <= 0 || inner % parts != 0)
    return gi::fail(GI_ERR_ARG, "mamba2 norm: %d values do not divide into %d parts", inner, parts);
  if (parts > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "mamba2 norm: more than 65535 parts");
  dim3 grid(n_tokens, parts);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(out_dtype, TO, GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(gate_norm_kernel<TO, T, TW>, grid, dim3(256), 0, (cudaStream_t)stream, (TO*)out, y, (const T*)proj, ld_proj,
                     (const TW*)w, inner, parts, eps))));
  return gi::check(e, "mamba2 norm");
}
