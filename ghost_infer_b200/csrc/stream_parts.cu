// Row kernels for layers that read the residual stream itself and norm what comes back, and for attention whose
// queries and keys are normed over their whole projection before they are rotated.
//
//  * cast_rows:      the float32 stream in the activation type (what a sublayer without a norm in front reads).
//  * postnorm_add:   x += y / sqrt(mean(y^2) + eps) * w [* s]: the norm sits on a sublayer's OUTPUT; s is a learned
//                    per-channel scale (or absent).  Everything 32-bit.
//  * axpy:           out += alpha * a on float32 rows (mixers side by side, each with a constant weight).
//  * qk_prepare:     one token's float32 row [q | k | v] of the projection: biases added and the sum rounded as the
//                    projection would have stored it; q and k each divided by the root mean square of the WHOLE vector
//                    (all heads together) and multiplied by a weight; the first `rot` numbers of every head rotated
//                    (pairs of neighbours, or pairs half the rotated width apart); q into the rows the attention reads, k and v
//                    into the token's place in the paged cache.  A row may hold queries only (a layer that reads another
//                    layer's keys and values).
//  * gate_mul:       out = a * sigmoid(g) or a * silu(g), element by element.
//  * norm_gate:      out = y / sqrt(mean_group(y^2) + eps) * w * act(g): the norm in groups of `gs` values (one head, or
//                    all heads together), the weight per value of a group or of the row; the gate comes after the norm.
//  * side_gate:      out[t, c] = gelu_tanh(gx[t, c]) * table[token_t, col0 + c]: a slice of a second embedding table
//                    gated by a projection of the stream.
//  * act_rows:       out = gelu(in) in its exact (erf) form.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

template <typename T> __device__ __forceinline__ float rounded(float v);
template <> __device__ __forceinline__ float rounded<float>(float v) { return v; }
template <> __device__ __forceinline__ float rounded<__nv_bfloat16>(float v) { return __bfloat162float(__float2bfloat16_rn(v)); }

__device__ __forceinline__ float sigmoid_f(float v) { return 1.0f / (1.0f + expf(-v)); }
__device__ __forceinline__ float gelu_tanh_f(float z) {
  return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * (z + 0.044715f * z * z * z)));
}
__device__ __forceinline__ float gelu_erf_f(float z) { return 0.5f * z * (1.0f + erff(z * 0.7071067811865476f)); }

__device__ __forceinline__ void st4(float* p, float4 v) { *reinterpret_cast<float4*>(p) = v; }
__device__ __forceinline__ void st4(__nv_bfloat16* p, float4 v) {
  __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
  *reinterpret_cast<uint2*>(p) = make_uint2(*reinterpret_cast<uint32_t*>(&a), *reinterpret_cast<uint32_t*>(&b));
}

// Four values a thread; `vec`: both pointers are 16-byte aligned, so whole groups move as one access each way.
// `zero` (or null): float32 values of the same count that are set to zero in the same pass (the rows a sublayer adds into).
template <typename TO>
__global__ void cast_rows_kernel(TO* __restrict__ out, const float* x, float* __restrict__ zero, size_t total, int vec) {
  gi::pdl_prologue();
  const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (e >= total) return;
  if (vec && e + 4 <= total) {
    st4(out + e, *reinterpret_cast<const float4*>(x + e));
    if (zero != nullptr) *reinterpret_cast<float4*>(zero + e) = make_float4(0.f, 0.f, 0.f, 0.f);
  } else {
    for (size_t i = e; i < total && i < e + 4; ++i) {
      gi::stf(out + i, x[i]);
      if (zero != nullptr) zero[i] = 0.f;
    }
  }
}

// One block per row.  A thread takes groups of four neighbouring values, 1,024 values apart; `vec`: the rows start on
// 16-byte boundaries, so a group is one access.  The order of the row's sum follows from the width alone either way.
// `h_out` (or null): the new rows of x once more in the activation type, what the next sublayer reads; `zero_y`: y is set
// to zero once it is read, for the next sublayer to add into.
template <typename TW, typename TH>
__global__ void __launch_bounds__(256)
postnorm_add_kernel(float* x, float* y, const TW* __restrict__ w, const TW* __restrict__ s, int d, float eps, int vec,
                    TH* __restrict__ h_out, int zero_y) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  float* yr = y + (size_t)blockIdx.x * d;
  float* xr = x + (size_t)blockIdx.x * d;
  TH* hr = h_out != nullptr ? h_out + (size_t)blockIdx.x * d : nullptr;
  float ss = 0.f;
  for (int i = threadIdx.x * 4; i < d; i += 1024) {
    if (vec && i + 4 <= d) {
      const float4 v = *reinterpret_cast<const float4*>(yr + i);
      ss = fmaf(v.x, v.x, ss); ss = fmaf(v.y, v.y, ss); ss = fmaf(v.z, v.z, ss); ss = fmaf(v.w, v.w, ss);
    } else {
      for (int e = i; e < d && e < i + 4; ++e) ss = fmaf(yr[e], yr[e], ss);
    }
  }
  const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)d + eps);
  for (int i = threadIdx.x * 4; i < d; i += 1024) {
    if (vec && i + 4 <= d) {
      const float4 v = *reinterpret_cast<const float4*>(yr + i);
      float4 o = *reinterpret_cast<const float4*>(xr + i);
      float t0 = v.x * rs * gi::ldf(w + i), t1 = v.y * rs * gi::ldf(w + i + 1), t2 = v.z * rs * gi::ldf(w + i + 2),
            t3 = v.w * rs * gi::ldf(w + i + 3);
      if (s != nullptr) { t0 *= gi::ldf(s + i); t1 *= gi::ldf(s + i + 1); t2 *= gi::ldf(s + i + 2); t3 *= gi::ldf(s + i + 3); }
      o.x += t0; o.y += t1; o.z += t2; o.w += t3;
      *reinterpret_cast<float4*>(xr + i) = o;
      if (hr != nullptr) st4(hr + i, o);
      if (zero_y) *reinterpret_cast<float4*>(yr + i) = make_float4(0.f, 0.f, 0.f, 0.f);
    } else {
      for (int e = i; e < d && e < i + 4; ++e) {
        float v = yr[e] * rs * gi::ldf(w + e);
        if (s != nullptr) v *= gi::ldf(s + e);
        const float o = xr[e] + v;
        xr[e] = o;
        if (hr != nullptr) gi::stf(hr + e, o);
        if (zero_y) yr[e] = 0.f;
      }
    }
  }
}

__global__ void axpy_kernel(float* out, const float* a, float alpha, size_t total, int vec) {
  gi::pdl_prologue();
  const size_t e = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4;
  if (e >= total) return;
  if (vec && e + 4 <= total) {
    const float4 v = *reinterpret_cast<const float4*>(a + e);
    float4 o = *reinterpret_cast<const float4*>(out + e);
    o.x = fmaf(alpha, v.x, o.x); o.y = fmaf(alpha, v.y, o.y); o.z = fmaf(alpha, v.z, o.z); o.w = fmaf(alpha, v.w, o.w);
    *reinterpret_cast<float4*>(out + e) = o;
  } else {
    for (size_t i = e; i < total && i < e + 4; ++i) out[i] = fmaf(alpha, a[i], out[i]);
  }
}

// One block per token.  Shared memory: the row's queries and keys as 32-bit numbers.
template <typename T, typename TW>
__global__ void __launch_bounds__(256)
qk_prepare_kernel(T* __restrict__ q_out, long ldq, const float* in, long ld, const TW* __restrict__ bq, const TW* __restrict__ bk,
                  const TW* __restrict__ bv, const TW* __restrict__ wq, const TW* __restrict__ wk, float eps,
                  const float2* table, int half, int adjacent, const int* positions, const int* slots,
                  const int* block_table, int max_pages, T* kcache, T* vcache, int n_heads, int n_kv, int hd, int hdv,
                  int write_cache) {
  extern __shared__ float row[];
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const int t = blockIdx.x;
  const float* r = in + (size_t)t * ld;
  const int qd = n_heads * hd, kd = n_kv * hd, vw = n_kv * hdv;
  float sq = 0.f, sk = 0.f;
  for (int i = threadIdx.x; i < qd + kd; i += 256) {
    float v = r[i];
    if (i < qd) { if (bq != nullptr) v += gi::ldf(bq + i); }
    else if (bk != nullptr) v += gi::ldf(bk + i - qd);
    v = rounded<T>(v);
    row[i] = v;
    if (i < qd) sq = fmaf(v, v, sq); else sk = fmaf(v, v, sk);
  }
  if (wq != nullptr) {
    const float rq = 1.0f / sqrtf(gi::block_sum(sq, scratch) / (float)qd + eps);
    for (int i = threadIdx.x; i < qd; i += 256) row[i] = row[i] * rq * gi::ldf(wq + i);
  }
  if (wk != nullptr && kd > 0) {
    const float rk = 1.0f / sqrtf(gi::block_sum(sk, scratch) / (float)kd + eps);
    for (int i = threadIdx.x; i < kd; i += 256) row[qd + i] = row[qd + i] * rk * gi::ldf(wk + i);
  }
  __syncthreads();
  const int slot = slots[t];
  const int pos = max(positions[t], 0);
  const int page = (write_cache && slot >= 0) ? block_table[(size_t)slot * max_pages + pos / PAGE_TOKENS] : 0;
  const int off = pos % PAGE_TOKENS;
  const int rot = 2 * half;
  const float2* cs = table + (size_t)t * half;
  const int n_rot = write_cache ? qd + kd : qd;
  for (int e = threadIdx.x; e < n_rot; e += 256) {
    const int d = e % hd;
    float val = row[e];
    if (d < rot) {
      float ra, rb;
      if (adjacent) {
        const int dl = d & ~1;      // the even member of this value's pair, inside the head
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
  if (write_cache) {
    for (int i = threadIdx.x; i < vw; i += 256) {
      float v = r[qd + kd + i];
      if (bv != nullptr) v += gi::ldf(bv + i);
      const int g = i / hdv;
      gi::stf(vcache + (((size_t)page * n_kv + g) * PAGE_TOKENS + off) * hdv + (i % hdv), v);
    }
  }
}

template <typename T>
__global__ void gate_mul_kernel(T* __restrict__ out, const T* a, const T* g, long ldg, int f, int act, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / f, c = i % f;
  const float z = gi::ldf(g + m * ldg + c);
  gi::stf(out + i, gi::ldf(a + i) * (act ? z * sigmoid_f(z) : sigmoid_f(z)));
}

// grid (tokens, groups): 128 threads sum one group
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
norm_gate_kernel(T* __restrict__ out, const float* y, const T* g, long ldg, const TW* __restrict__ w, int inner, int gs,
                 int w_per_row, int act, float eps) {
  __shared__ float scratch[33];
  gi::pdl_prologue();
  const size_t t = blockIdx.x;
  const int c0 = blockIdx.y * gs;
  const float* yr = y + t * inner + c0;
  float ss = 0.f;
  for (int i = threadIdx.x; i < gs; i += 128) ss = fmaf(yr[i], yr[i], ss);
  const float rs = 1.0f / sqrtf(gi::block_sum(ss, scratch) / (float)gs + eps);
  for (int i = threadIdx.x; i < gs; i += 128) {
    const float z = gi::ldf(g + t * ldg + c0 + i);
    const float gate = act ? z * sigmoid_f(z) : sigmoid_f(z);
    gi::stf(out + t * inner + c0 + i, yr[i] * rs * gi::ldf(w + (w_per_row ? c0 + i : i)) * gate);
  }
}

template <typename T, typename TW>
__global__ void side_gate_kernel(T* __restrict__ out, const T* gx, long ldg, const TW* __restrict__ table, long ld_table,
                                 const int* tokens, int col0, int dim, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  const size_t m = i / dim, c = i % dim;
  const float e = gi::ldf(table + (size_t)tokens[m] * ld_table + col0 + c);
  gi::stf(out + i, gelu_tanh_f(gi::ldf(gx + m * ldg + c)) * e);
}

template <typename T>
__global__ void act_rows_kernel(T* __restrict__ out, const T* in, long ld_in, int f, size_t total) {
  gi::pdl_prologue();
  const size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= total) return;
  gi::stf(out + i, gelu_erf_f(gi::ldf(in + (i / f) * ld_in + i % f)));
}

inline unsigned blocks_of(size_t total) { return (unsigned)((total + 255) / 256); }

}  // namespace

extern "C" int gi_cast_rows(void* out, int out_dtype, const float* x, long n_values, void* stream) {
  return gi_cast_rows_zero(out, out_dtype, x, nullptr, n_values, stream);
}

extern "C" int gi_cast_rows_zero(void* out, int out_dtype, const float* x, float* zero, long n_values, void* stream) {
  if (n_values <= 0) return GI_OK;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(out_dtype, TO,
      e = gi::launch(cast_rows_kernel<TO>, dim3(blocks_of(((size_t)n_values + 3) / 4)), dim3(256), 0, (cudaStream_t)stream, (TO*)out, x,
                     zero, (size_t)n_values, (int)((((uintptr_t)out | (uintptr_t)x | (uintptr_t)zero) & 15) == 0)));
  return gi::check(e, "cast_rows");
}

extern "C" int gi_postnorm_add(float* x, const float* y, const void* w, const void* scale, int w_dtype, int n_rows, int d,
                               float eps, void* stream) {
  return gi_postnorm_add_ex(x, const_cast<float*>(y), w, scale, w_dtype, n_rows, d, eps, nullptr, GI_F32, 0, stream);
}

extern "C" int gi_postnorm_add_ex(float* x, float* y, const void* w, const void* scale, int w_dtype, int n_rows, int d, float eps,
                                  void* h_out, int h_dtype, int zero_y, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (d <= 0 || !x || !y || !w) return gi::fail(GI_ERR_ARG, "postnorm_add: bad width %d or a missing pointer", d);
  const int vec = (int)(d % 4 == 0 && (((uintptr_t)x | (uintptr_t)y | (uintptr_t)h_out) & 15) == 0);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(w_dtype, TW, GI_DISPATCH_DTYPE(h_dtype, TH,
      e = gi::launch(postnorm_add_kernel<TW, TH>, dim3(n_rows), dim3(256), 0, (cudaStream_t)stream, x, y, (const TW*)w,
                     (const TW*)scale, d, eps, vec, (TH*)h_out, zero_y)));
  return gi::check(e, "postnorm_add");
}

extern "C" int gi_axpy(float* out, const float* a, float alpha, long n_values, void* stream) {
  if (n_values <= 0) return GI_OK;
  cudaError_t e = gi::launch(axpy_kernel, dim3(blocks_of(((size_t)n_values + 3) / 4)), dim3(256), 0, (cudaStream_t)stream, out, a, alpha,
                             (size_t)n_values, (int)((((uintptr_t)out | (uintptr_t)a) & 15) == 0));
  return gi::check(e, "axpy");
}

extern "C" int gi_qk_prepare(void* q_out, long ldq, int dtype, const float* in, long ld, const void* bq, const void* bk,
                             const void* bv, const void* wq, const void* wk, int w_dtype, float eps, const float* table, int half,
                             int adjacent, const int* positions, const int* slots, const int* block_table, int max_pages,
                             void* kcache, void* vcache, int n_tokens, int n_heads, int n_kv, int hd, int hdv, int write_cache,
                             void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (n_heads <= 0 || n_kv < 0 || hd <= 0 || hdv <= 0 || half < 0 || 2 * half > hd)
    return gi::fail(GI_ERR_ARG, "qk_prepare: bad sizes (heads %d, kv heads %d, head %d, values %d, rotated %d)", n_heads, n_kv, hd, hdv, 2 * half);
  if (adjacent && (hd & 1) && half > 0) return gi::fail(GI_ERR_ARG, "qk_prepare: neighbouring pairs need an even head size");
  if (half > 0 && table == nullptr) return gi::fail(GI_ERR_ARG, "qk_prepare: rotation without a table of angles");
  if (write_cache && (n_kv == 0 || !kcache || !vcache || !block_table))
    return gi::fail(GI_ERR_ARG, "qk_prepare: cache write without keys or without a cache");
  const size_t smem = (size_t)(n_heads + n_kv) * hd * sizeof(float);
  if (smem > 160 * 1024) return gi::fail(GI_ERR_UNSUPPORTED, "qk_prepare: rows of %zu bytes do not fit shared memory", smem);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW, {
    auto kern = qk_prepare_kernel<T, TW>;
    if (smem > 48 * 1024) {
      e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e != cudaSuccess) return gi::check(e, "qk_prepare (shared memory)");
    }
    e = gi::launch(kern, dim3(n_tokens), dim3(256), smem, (cudaStream_t)stream, (T*)q_out, ldq, in, ld, (const TW*)bq,
                   (const TW*)bk, (const TW*)bv, (const TW*)wq, (const TW*)wk, eps, (const float2*)table, half, adjacent,
                   positions, slots, block_table, max_pages, (T*)kcache, (T*)vcache, n_heads, n_kv, hd, hdv, write_cache);
  }));
  return gi::check(e, "qk_prepare");
}

extern "C" int gi_gate_mul(void* out, const void* a, const void* g, long ldg, int dtype, int n_rows, int f, int act, void* stream) {
  if (n_rows <= 0 || f <= 0) return GI_OK;
  const size_t total = (size_t)n_rows * f;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(gate_mul_kernel<T>, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)a,
                     (const T*)g, ldg, f, act, total));
  return gi::check(e, "gate_mul");
}

extern "C" int gi_norm_gate(void* out, int dtype, const float* y, const void* g, long ldg, const void* w, int w_dtype, int n_rows,
                            int inner, int group, int w_per_row, int act, float eps, void* stream) {
  if (n_rows <= 0) return GI_OK;
  if (inner <= 0 || group <= 0 || inner % group) return gi::fail(GI_ERR_ARG, "norm_gate: %d values do not divide into groups of %d", inner, group);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(norm_gate_kernel<T, TW>, dim3(n_rows, inner / group), dim3(128), 0, (cudaStream_t)stream, (T*)out, y,
                     (const T*)g, ldg, (const TW*)w, inner, group, w_per_row, act, eps)));
  return gi::check(e, "norm_gate");
}

extern "C" int gi_side_gate(void* out, const void* gx, long ldg, int dtype, const void* table, long ld_table, int w_dtype,
                            const int* tokens, int n_rows, int col0, int dim, void* stream) {
  if (n_rows <= 0 || dim <= 0) return GI_OK;
  const size_t total = (size_t)n_rows * dim;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(side_gate_kernel<T, TW>, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)gx,
                     ldg, (const TW*)table, ld_table, tokens, col0, dim, total)));
  return gi::check(e, "side_gate");
}

extern "C" int gi_act_rows(void* out, const void* in, long ld_in, int dtype, int n_rows, int f, void* stream) {
  if (n_rows <= 0 || f <= 0) return GI_OK;
  const size_t total = (size_t)n_rows * f;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T,
      e = gi::launch(act_rows_kernel<T>, dim3(blocks_of(total)), dim3(256), 0, (cudaStream_t)stream, (T*)out, (const T*)in, ld_in,
                     f, total));
  return gi::check(e, "act_rows");
}
