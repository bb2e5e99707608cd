// Row kernels for attention whose queries and keys are normed head by head, whose values are made unit-RMS vectors, and
// whose heads are gated by one number each; for outputs of a recurrence that are scaled, normed per head and gated; and for
// gated feed-forward rows with clamped halves.
//
//  * head_prepare:   one token's float32 row [q: H * n | k: G * n | v: G * m | ...] of the projection (G = 0: queries only):
//                    biases added and the sums rounded as the projection would have stored them; every head of q and of k
//                    divided by its own root mean square and multiplied by a weight of n numbers shared by the heads; every
//                    head of v divided by its root mean square (no weight); the first `rot` numbers of every head of q and k
//                    rotated (pairs of neighbours, or pairs half the rotated width apart); q into the rows the attention reads,
//                    k and v into the token's place in the paged cache.  Each norm may be switched off.
//  * head_gate:      out[t][h][:] = a[t][h][:] * sigmoid(g[t][h]): one gate per head, from float32 rows.
//  * scaled_norm_gate: v = y[t][h][:] * s[t][h];  out = v / sqrt(mean(v^2) + eps) * w[h][:] * sigmoid(g[t][h][:]).
//  * clamped_glu:    rows [gate: f | up: f]:  g = min(gate, limit), u = clamp(up, -limit, limit);
//                    out = g * sigmoid(alpha g) * (u + 1)      (limit <= 0: no clamps).
// Norms, angles and gates are 32-bit.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float rounded(float v);
template <> __device__ __forceinline__ float rounded<float>(float v) { return v; }
template <> __device__ __forceinline__ float rounded<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }

// One block of 256 threads per token; a warp takes a head at a time.  Shared memory: the row's q, k and v as floats.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
head_prepare_kernel(T* __restrict__ q_out, long ldq, const float* in, long ld, const TW* __restrict__ bq, const TW* __restrict__ bk,
                    const TW* __restrict__ bv, const TW* __restrict__ wq, const TW* __restrict__ wk, int norm_q, int norm_k, int norm_v,
                    float eps, const float2* table, int half, int adjacent, const int* positions, const int* slots,
                    const int* block_table, int max_pages, T* kcache, T* vcache, int n_heads, int n_kv, int hd, int hdv) {
  extern __shared__ float row[];
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const float* r = in + (size_t)t * ld;
  const int qd = n_heads * hd, kd = n_kv * hd, vw = n_kv * hdv;
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int i = threadIdx.x; i < qd + kd + vw; i += 256) {
    float v = r[i];
    const TW* b = i < qd ? bq : (i < qd + kd ? bk : bv);
    if (b != nullptr) v += gi::ldf(b + (i < qd ? i : (i < qd + kd ? i - qd : i - qd - kd)));
    row[i] = rounded<T>(v);
  }
  __syncthreads();
  // heads of q, then of k, then of v: each divided by its own root mean square
  for (int hh = warp; hh < n_heads + 2 * n_kv; hh += 8) {
    const bool is_q = hh < n_heads, is_k = !is_q && hh < n_heads + n_kv;
    const int n = (is_q || is_k) ? hd : hdv;
    float* p = is_q ? row + (size_t)hh * hd : (is_k ? row + qd + (size_t)(hh - n_heads) * hd : row + qd + kd + (size_t)(hh - n_heads - n_kv) * hdv);
    const bool on = is_q ? norm_q : (is_k ? norm_k : norm_v);
    if (!on) continue;
    float ss = 0.f;
    for (int i = lane; i < n; i += 32) ss = fmaf(p[i], p[i], ss);
    const float rs = 1.0f / sqrtf(gi::warp_sum(ss) / (float)n + eps);
    const TW* w = is_q ? wq : (is_k ? wk : nullptr);
    for (int i = lane; i < n; i += 32) p[i] = p[i] * rs * (w != nullptr ? gi::ldf(w + i) : 1.0f);
  }
  __syncthreads();
  const bool write_cache = n_kv > 0;
  const int slot = slots[t];
  const int pos = max(positions[t], 0);
  const int page = (write_cache && slot >= 0) ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
  const int off = pos % PAGE_TOKENS;
  const int rot = 2 * half;
  const float2* cs = table + (size_t)t * half;
  for (int e = threadIdx.x; e < qd + kd; e += 256) {
    const int d = e % hd;
    float val = row[e];
    if (d < rot) {
      float ra, rb;
      if (adjacent) {
        const int dl = d & ~1;
        gi::rotate_pair(row[e - d + dl], row[e - d + dl + 1], cs[dl >> 1], &ra, &rb);
        val = (d & 1) ? rb : ra;
      } else {
        const int i = d < half ? d : d - half;
        gi::rotate_pair(row[e - d + i], row[e - d + i + half], cs[i], &ra, &rb);
        val = d < half ? ra : rb;
      }
    }
    if (e < qd) {
      gi::stf(q_out + (size_t)t * ldq + e, val);
    } else {
      const int i = e - qd, g = i / hd;
      gi::stf(kcache + (((size_t)page * n_kv + g) * PAGE_TOKENS + off) * hd + (i % hd), val);
    }
  }
  for (int i = threadIdx.x; i < vw; i += 256) {
    const int g = i / hdv;
    gi::stf(vcache + (((size_t)page * n_kv + g) * PAGE_TOKENS + off) * hdv + (i % hdv), row[qd + kd + i]);
  }
}

template <typename T>
__global__ void head_gate_kernel(T* __restrict__ out, const T* a, const float* g, long ldg, int n_heads, int hdv, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t w = (size_t)n_heads * hdv, t = i / w, h = (i % w) / hdv;
  gi::stf(out + i, gi::ldf(a + i) * sigmoid_f(g[t * ldg + h]));
}

// grid (tokens, heads); 128 threads sum one head
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
scaled_norm_gate_kernel(T* __restrict__ out, const float* y, const float* s, const float* g, long ldg, const TW* __restrict__ w,
                        int n_heads, int hdv, float eps) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const size_t t = blockIdx.x;
  const int h = blockIdx.y;
  const size_t c0 = (size_t)h * hdv;
  const float* yr = y + t * n_heads * hdv + c0;
  const float sc = s != nullptr ? s[t * n_heads + h] : 1.0f;
  float ss = 0.f;
  for (int i = threadIdx.x; i < hdv; i += 128) {
    const float v = yr[i] * sc;
    ss = fmaf(v, v, ss);
  }
  const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)hdv + eps);
  for (int i = threadIdx.x; i < hdv; i += 128)
    gi::stf(out + t * n_heads * hdv + c0 + i, yr[i] * sc * rs * gi::ldf(w + c0 + i) * sigmoid_f(g[t * ldg + c0 + i]));
}

template <typename T>
__global__ void clamped_glu_kernel(T* __restrict__ out, const T* in, long ld_in, int f, float limit, float alpha, size_t total,
                                   int interleaved) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t t = i / f, c = i % f;
  // gate and up of output c: columns c and f + c, or, interleaved in blocks of 8, (c / 8) * 16 + c % 8 and 8 further
  const size_t gc = interleaved ? (c / 8) * 16 + c % 8 : c;
  float g = gi::ldf(in + t * ld_in + gc), u = gi::ldf(in + t * ld_in + (interleaved ? gc + 8 : f + c));
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
  }
  gi::stf(out + i, g * sigmoid_f(alpha * g) * (u + 1.0f));
}

inline unsigned blocks_of(size_t total) { return (unsigned)((total + 255) / 256); }

}  // namespace

extern "C" int gi_head_prepare(void* q_out, long ldq, int dtype, const float* in, long ld, const void* bq, const void* bk,
                               const void* bv, const void* wq, const void* wk, int w_dtype, int norm_q, int norm_k, int norm_v,
                               float eps, const float* table, int half, int adjacent, const int* positions, const int* slots,
                               const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens, int n_heads,
                               int n_kv, int hd, int hdv, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (n_heads <= 0 || n_kv < 0 || hd <= 0 || hdv <= 0 || half < 0 || 2 * half > hd)
    return gi::fail(GI_ERR_ARG, "head_prepare: bad sizes (heads %d, kv heads %d, head %d, values %d, rotated %d)", n_heads, n_kv, hd, hdv, 2 * half);
  if (adjacent && (hd & 1) && half > 0) return gi::fail(GI_ERR_ARG, "head_prepare: neighbouring pairs need an even head size");
  if (half > 0 && table == nullptr) return gi::fail(GI_ERR_ARG, "head_prepare: rotation without a table of angles");
  if (n_kv > 0 && (!kcache || !vcache || !block_table)) return gi::fail(GI_ERR_ARG, "head_prepare: keys and values without a cache");
  const size_t smem = ((size_t)(n_heads + n_kv) * hd + (size_t)n_kv * hdv) * sizeof(float);
  if (smem > 160 * 1024) return gi::fail(GI_ERR_UNSUPPORTED, "head_prepare: rows of %zu bytes do not fit shared memory", smem);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW, {
    auto kern = head_prepare_kernel<T, TW>;
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return gi::check(e, "head_prepare (shared memory)");
    }
    e = gi::launch(kern, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (T*)q_out, ldq, in, ld, (const TW*)bq, (const TW*)bk,
                   (const TW*)bv, (const TW*)wq, (const TW*)wk, norm_q, norm_k, norm_v, eps, (const float2*)table, half, adjacent,
                   positions, slots, block_table, max_pages, (T*)kcache, (T*)vcache, n_heads, n_kv, hd, hdv);
  }));
  return gi::check(e, "head_prepare");
}

extern "C" int gi_head_gate(void* out, const void* a, int dtype, const float* g, long ldg, int n_rows, int n_heads, int hdv, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (n_heads <= 0 || hdv <= 0) return gi::fail(GI_ERR_ARG, "head_gate: bad sizes");
  const size_t total = (size_t)n_rows * n_heads * hdv;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(head_gate_kernel<T>, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)a, g, ldg, n_heads,
                     hdv, total));
  return gi::check(e, "head_gate");
}

extern "C" int gi_scaled_norm_gate(void* out, int dtype, const float* y, const float* scale, const float* g, long ldg, const void* w,
                                   int w_dtype, int n_rows, int n_heads, int hdv, float eps, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (n_heads <= 0 || hdv <= 0 || n_heads > 65535) return gi::fail(GI_ERR_ARG, "scaled_norm_gate: bad sizes");
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(scaled_norm_gate_kernel<T, TW>, dim3(n_rows, n_heads), dim3(128), 0, (cudaStream_t)stream, (T*)out, y, scale, g, ldg,
                     (const TW*)w, n_heads, hdv, eps)));
  return gi::check(e, "scaled_norm_gate");
}

extern "C" int gi_clamped_glu(void* out, const void* in, long ld_in, int dtype, int n_rows, int f, float limit, float alpha, void* stream) {
  return gi_clamped_glu_rows(out, in, ld_in, dtype, n_rows, f, limit, alpha, 0, stream);
}

extern "C" int gi_clamped_glu_rows(void* out, const void* in, long ld_in, int dtype, int n_rows, int f, float limit, float alpha,
                                   int interleaved, void* stream) {
  if (n_rows <= 0 || f <= 0) return GI_OK;
  if (interleaved && f % 8) return gi::fail(GI_ERR_ARG, "clamped_glu: interleaved rows need a width that is a multiple of 8");
  const size_t total = (size_t)n_rows * f;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(clamped_glu_kernel<T>, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)in, ld_in, f,
                     limit, alpha, total, interleaved));
  return gi::check(e, "clamped_glu");
}
