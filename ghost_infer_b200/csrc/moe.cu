// Routed feed-forward (mixture of experts): every token picks `top` of `experts` small gated feed-forward layers.
//
//  * route:   logits = h W_r^T in 32-bit (one block per token, a warp per expert in turn, a fixed order of additions);
//             the `top` largest logits (the lower index wins a tie); weights = softmax over the chosen logits only;
//             optionally a gate for a shared expert, sigmoid(h . w_sg).
//  * plan:    a stable counting sort of the (token, choice) entries by expert, entirely on the device, so that a step
//             has the same launches whatever the tokens choose (it can be recorded and replayed): per segment of 1,024
//             entries each entry's rank among the earlier entries of its expert and the segment's count per expert;
//             then the experts' offsets; then each entry's place.
//  * products over the sorted rows: a tile of 64 rows belongs to one expert and reads that expert's matrix; the grid has
//             as many row tiles as the worst case needs (entries / 64 + experts) and the others leave at once.  Each output
//             is summed by one thread in k order, so a row's result does not depend on where the sort put it.
//  * combine: residual += sum over the choices (in their order) of weight x expert output, plus the shared expert's
//             output times its gate.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int SEG = 1024;

// Sixteen bytes of a row at once, as floats.
template <typename T> struct Vec16;
template <> struct Vec16<float> {
  static constexpr int N = 4;
  static __device__ __forceinline__ void load(const float* p, float (&v)[8]) {
    const float4 x = *reinterpret_cast<const float4*>(p);
    v[0] = x.x; v[1] = x.y; v[2] = x.z; v[3] = x.w;
  }
};
template <> struct Vec16<__nv_bfloat16> {
  static constexpr int N = 8;
  static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&v)[8]) {
    const uint4 x = *reinterpret_cast<const uint4*>(p);
    const uint32_t r[4] = {x.x, x.y, x.z, x.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      v[2 * i] = __uint_as_float(r[i] << 16);
      v[2 * i + 1] = __uint_as_float(r[i] & 0xffff0000u);
    }
  }
};

// One block per token: the row goes to shared memory as floats once; warp w forms the logits of experts w, w + 4, ...
// (and the last warp's turn after them the shared expert's gate); then the first warp picks.
template <typename T, typename TW>
__global__ void __launch_bounds__(128)
route_kernel(int* __restrict__ ids, float* __restrict__ wts, float* __restrict__ sgate, const T* __restrict__ h, long ldh,
             const TW* __restrict__ w_router, const TW* __restrict__ w_sg, int n_tokens, int width, int experts, int top,
             int vec, int score_mode, const float* __restrict__ correction, float weight_scale) {
  extern __shared__ __align__(16) float sm[];
  float* hs = sm;                          // [width] (rounded up to a multiple of 8)
  float* lg = sm + ((width + 7) / 8) * 8;  // [experts]
  float* ps = lg + experts;                // [experts] (score_mode 2: every expert's share of the softmax over all of them)
  gi::pdl_prologue();
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int t = blockIdx.x;
  const T* hr = h + (size_t)t * ldh;
  for (int i = threadIdx.x; i < width; i += 128) hs[i] = gi::ldf(hr + i);
  __syncthreads();
  const int rows = experts + (w_sg != nullptr ? 1 : 0);
  for (int e = warp; e < rows; e += 4) {
    const TW* wr = e < experts ? w_router + (size_t)e * width : w_sg;
    float acc = 0.f;
    if (vec) {
      constexpr int VN = Vec16<TW>::N;
      for (int i = lane * VN; i < width; i += 32 * VN) {
        float wv[8];
        Vec16<TW>::load(wr + i, wv);
#pragma unroll
        for (int j = 0; j < VN; ++j) acc = fmaf(hs[i + j], wv[j], acc);
      }
    } else {
      for (int i = lane; i < width; i += 32) acc = fmaf(hs[i], gi::ldf(wr + i), acc);
    }
    acc = gi::warp_sum(acc);
    if (lane == 0) {
      if (e < experts) lg[e] = acc;
      else sgate[t] = 1.0f / (1.0f + expf(-acc));
    }
  }
  __syncthreads();
  if (warp != 0) return;
  if (score_mode == 2) {
    // the softmax over all experts; the choice is made by share + correction, the weights use the shares themselves
    float top_z = -INFINITY;
    for (int e = lane; e < experts; e += 32) top_z = fmaxf(top_z, lg[e]);
    top_z = gi::warp_max(top_z);
    float den = 0.f;
    for (int e = lane; e < experts; e += 32) {
      const float p = expf(lg[e] - top_z);
      ps[e] = p;
      den += p;
    }
    den = gi::warp_sum(den);
    for (int e = lane; e < experts; e += 32) {
      const float p = ps[e] / den;
      ps[e] = p;
      lg[e] = p + (correction != nullptr ? correction[e] : 0.f);
    }
    __syncwarp();
  }
  float first = 0.f, sum = 0.f, mine = 0.f;      // lane k keeps the k-th chosen logit (top <= 32)
  for (int k = 0; k < top; ++k) {
    float best = -INFINITY;
    int at = 0x7fffffff;
    for (int e = lane; e < experts; e += 32) {
      const float v = lg[e];
      if (v > best || (v == best && e < at)) { best = v; at = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oa = __shfl_xor_sync(0xffffffffu, at, o);
      if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
    }
    if (at == 0x7fffffff) at = k < experts ? k : 0;      // every logit a NaN: any expert, never an index outside
    if (k == 0) first = best;
    // score_mode 0: the weights are the softmax over the chosen logits; 1: each chosen logit's own sigmoid, as it is
    const float ex = score_mode == 2 ? ps[at < experts ? at : 0]
                                     : (score_mode == 1 ? 1.0f / (1.0f + expf(-best)) : expf(best - first));
    sum += ex;
    if (lane == k) mine = ex;
    if (lane == 0) {
      ids[(size_t)t * top + k] = at;
      if (at < experts) lg[at] = -INFINITY;
    }
    __syncwarp();
  }
  if (lane < top)
    wts[(size_t)t * top + lane] = score_mode == 2 ? mine / (sum + 1e-20f) * weight_scale : (score_mode == 1 ? mine : mine / sum);
}

// ---- plan ------------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(SEG)
rank_kernel(int* __restrict__ local_rank, int* __restrict__ seg_count, const int* __restrict__ ids, int entries, int experts) {
  extern __shared__ int smi[];             // [SEG] ids, [experts] histogram
  int* sid = smi;
  int* hist = smi + SEG;
  gi::pdl_prologue();
  const int seg = blockIdx.x, i = seg * SEG + threadIdx.x;
  const int id = i < entries ? ids[i] : -1;
  sid[threadIdx.x] = id;
  for (int e = threadIdx.x; e < experts; e += SEG) hist[e] = 0;
  __syncthreads();
  if (id >= 0) {
    int r = 0;
    for (int j = 0; j < (int)threadIdx.x; ++j) r += sid[j] == id;
    local_rank[i] = r;
    atomicAdd(&hist[id], 1);                // integer counts: the same whatever the order
  }
  __syncthreads();
  for (int e = threadIdx.x; e < experts; e += SEG) seg_count[(size_t)seg * experts + e] = hist[e];
}

__global__ void __launch_bounds__(1024)
offsets_kernel(int* __restrict__ offsets, int* __restrict__ seg_count, int n_seg, int experts) {
  extern __shared__ int smi[];             // [experts] totals
  gi::pdl_prologue();
  for (int e = threadIdx.x; e < experts; e += blockDim.x) {
    int run = 0;
    for (int s = 0; s < n_seg; ++s) {
      const int c = seg_count[(size_t)s * experts + e];
      seg_count[(size_t)s * experts + e] = run;     // becomes: entries of this expert in earlier segments
      run += c;
    }
    smi[e] = run;
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    int run = 0;
    for (int e = 0; e < experts; ++e) {
      offsets[e] = run;
      run += smi[e];
    }
    offsets[experts] = run;
  }
}

__global__ void __launch_bounds__(SEG)
place_kernel(int* __restrict__ perm, int* __restrict__ inv, const int* __restrict__ offsets, const int* __restrict__ seg_base,
             const int* __restrict__ local_rank, const int* __restrict__ ids, int entries, int experts) {
  gi::pdl_prologue();
  const int seg = blockIdx.x, i = seg * SEG + threadIdx.x;
  if (i >= entries) return;
  const int id = ids[i];
  const int pos = offsets[id] + seg_base[(size_t)seg * experts + id] + local_rank[i];
  perm[pos] = i;
  inv[i] = pos;
}

// ---- products ----------------------------------------------------------------------------------------------------
constexpr int BM = 64, BN = 64, BK = 16, TM = 4, TN = 4;

// Which expert and which rows row tile `ty` holds: experts in order, each with ceil(count / BM) tiles.
__device__ __forceinline__ bool tile_rows(const int* __restrict__ offsets, int experts, int ty, int* e_out, int* r0, int* r1) {
  int tiles = 0;
  for (int e = 0; e < experts; ++e) {
    const int lo = offsets[e], hi = offsets[e + 1];
    const int n = (hi - lo + BM - 1) / BM;
    if (ty < tiles + n) {
      *e_out = e;
      *r0 = lo + (ty - tiles) * BM;
      *r1 = min(hi, *r0 + BM);
      return true;
    }
    tiles += n;
  }
  return false;
}

// What a gated expert keeps of its two sums.  limit <= 0: silu(g) * u.  limit > 0: the clamped form g' = min(g, limit),
// u' = clamp(u, -limit, limit), g' * sigmoid(alpha g') * (u' + 1).
__device__ __forceinline__ float gated_value(float g, float u, float limit, float alpha) {
  if (limit > 0.f) {
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    return g / (1.0f + expf(-alpha * g)) * (u + 1.0f);
  }
  return g / (1.0f + expf(-g)) * u;
}

// DUAL: two accumulators (gate rows n, up rows f + n of the expert's matrix), out = silu(gate) * up in the rows' type.
// else: out (float) = a W^T.
template <typename TA, typename TW, bool DUAL>
__global__ void __launch_bounds__(256)
expert_gemm_kernel(void* __restrict__ out_, const TA* __restrict__ A, long lda, const TW* __restrict__ W, long w_stride,
                   const int* __restrict__ offsets, const int* __restrict__ perm, int top, int experts, int N, int K,
                   int interleaved, int act_out, float limit, float alpha) {
  __shared__ float As[BK][BM + 4];
  __shared__ float Ws[BK][BN + 4];
  __shared__ float Us[DUAL ? BK : 1][BN + 4];
  __shared__ int src[BM];
  gi::pdl_prologue();
  int e, r0, r1;
  if (!tile_rows(offsets, experts, blockIdx.y, &e, &r0, &r1)) return;
  const int tid = threadIdx.x;
  const int n0 = blockIdx.x * BN;
  const TW* We = W + (size_t)e * w_stride;
  if (tid < BM) src[tid] = (r0 + tid < r1) ? (perm != nullptr ? perm[r0 + tid] / top : r0 + tid) : -1;
  __syncthreads();
  const int tx = tid % 16, ty = tid / 16;
  float acc[TM][TN], acu[DUAL ? TM : 1][TN];
#pragma unroll
  for (int i = 0; i < TM; ++i)
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      acc[i][j] = 0.f;
      if (DUAL) acu[i][j] = 0.f;
    }
  for (int k0 = 0; k0 < K; k0 += BK) {
#pragma unroll
    for (int q = 0; q < 4; ++q) {
      const int idx = tid + q * 256;
      const int r = idx / BK, kk = idx % BK, k = k0 + kk;
      float a = 0.f, w = 0.f, u = 0.f;
      if (k < K) {
        if (src[r] >= 0) a = gi::ldf(A + (size_t)src[r] * lda + k);
        if (n0 + r < N) {
          // gate and up rows of output n: rows n and N + n, or, interleaved in blocks of 8, (n / 8) * 16 + n % 8 and 8 further
          const int n = n0 + r;
          const size_t gr = (DUAL && interleaved) ? (size_t)(n / 8) * 16 + n % 8 : (size_t)n;
          w = gi::ldf(We + gr * K + k);
          if (DUAL) u = gi::ldf(We + (interleaved ? gr + 8 : (size_t)N + n) * K + k);
        }
      }
      As[kk][r] = a;
      Ws[kk][r] = w;
      if (DUAL) Us[kk][r] = u;
    }
    __syncthreads();
#pragma unroll
    for (int kk = 0; kk < BK; ++kk) {
      float a[TM], w[TN], u[TN];
#pragma unroll
      for (int i = 0; i < TM; ++i) a[i] = As[kk][ty * TM + i];
#pragma unroll
      for (int j = 0; j < TN; ++j) {
        w[j] = Ws[kk][tx * TN + j];
        if (DUAL) u[j] = Us[kk][tx * TN + j];
      }
#pragma unroll
      for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) {
          acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
          if (DUAL) acu[i][j] = fmaf(a[i], u[j], acu[i][j]);
        }
    }
    __syncthreads();
  }
#pragma unroll
  for (int i = 0; i < TM; ++i) {
    const int r = r0 + ty * TM + i;
    if (r >= r1) continue;
#pragma unroll
    for (int j = 0; j < TN; ++j) {
      const int n = n0 + tx * TN + j;
      if (n >= N) continue;
      if (DUAL) {
        gi::stf((TA*)out_ + (size_t)r * N + n, gated_value(acc[i][j], acu[i][j], limit, alpha));
      } else if (act_out) {          // a plain (ungated) hidden layer: relu squared, in the rows' type
        const float z = fmaxf(acc[i][j], 0.f);
        gi::stf((TA*)out_ + (size_t)r * N + n, z * z);
      } else {
        ((float*)out_)[(size_t)r * N + n] = acc[i][j];
      }
    }
  }
}

// ---- the same products for a step of few rows (one-token steps): bound by the bytes of the experts' matrices ----------
// grid (column tiles of 32, experts); a block stages up to 8 of its expert's rows in shared memory and streams 32 rows
// of the expert's matrix past them, 16 bytes per lane per load; a warp takes 8 columns, its lanes cut K between them
// and their sums meet in a fixed order (a lane's own partial sums in k order, then the warp's tree).  An expert without
// rows leaves at once, so the launch reads only the matrices of experts that were chosen.
constexpr int GEMV_WARPS = 4, GEMV_COLS = 32, GEMV_ROWS = 8, GEMV_MAX_ENTRIES = 512;
constexpr int GEMV_CPW = GEMV_COLS / GEMV_WARPS;     // columns per warp

inline bool gemv_ok(int dtype, int w_dtype, int k, const void* a, const void* w, long lda) {
  const int per = dtype == GI_F32 ? 4 : 8;             // elements per 16-byte load
  return dtype == w_dtype && k % per == 0 && lda % per == 0 && !(((uintptr_t)a | (uintptr_t)w) & 15) &&
         (size_t)GEMV_ROWS * k * (dtype == GI_F32 ? 4 : 2) <= 160 * 1024;
}

template <typename T, bool DUAL>
__global__ void __launch_bounds__(GEMV_WARPS * 32)
expert_gemv_kernel(void* __restrict__ out_, const T* __restrict__ A, long lda, const T* __restrict__ W, long w_stride,
                   const int* __restrict__ offsets, const int* __restrict__ perm, int top, int N, int K, int interleaved,
                   int act_out, float limit, float alpha) {
  extern __shared__ __align__(16) unsigned char smem_raw[];
  T* As = reinterpret_cast<T*>(smem_raw);            // [GEMV_ROWS][K]
  constexpr int VN = Vec16<T>::N;
  gi::pdl_prologue();
  const int e = blockIdx.y;
  const int lo = offsets[e], hi = offsets[e + 1];
  if (hi <= lo) return;
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const T* We = W + (size_t)e * w_stride;
  const int n_base = blockIdx.x * GEMV_COLS + warp * GEMV_CPW;
  for (int r0 = lo; r0 < hi; r0 += GEMV_ROWS) {
    const int rows = min(GEMV_ROWS, hi - r0);
    __syncthreads();
    for (int idx = tid; idx < rows * (K / VN); idx += GEMV_WARPS * 32) {
      const int r = idx / (K / VN), c = idx % (K / VN);
      const int src = perm != nullptr ? perm[r0 + r] / top : r0 + r;
      *reinterpret_cast<uint4*>(As + (size_t)r * K + c * VN) = *reinterpret_cast<const uint4*>(A + (size_t)src * lda + c * VN);
    }
    __syncthreads();
    // four columns at a time, so that a lane has four (eight with the up rows) 16-byte loads in flight per turn
    for (int j0 = 0; j0 < GEMV_CPW; j0 += 4) {
      if (n_base + j0 >= N) break;                      // the same for the whole warp
      const T* wg[4];
      const T* wu[4];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int n = min(n_base + j0 + jj, N - 1);     // a column past the end repeats the last one and is not stored
        const size_t gr = (DUAL && interleaved) ? (size_t)(n / 8) * 16 + n % 8 : (size_t)n;
        wg[jj] = We + gr * K;
        wu[jj] = We + (interleaved ? gr + 8 : (size_t)N + n) * K;
      }
      float acc[4][GEMV_ROWS], acu[DUAL ? 4 : 1][GEMV_ROWS];
#pragma unroll
      for (int jj = 0; jj < 4; ++jj)
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r) {
          acc[jj][r] = 0.f;
          if (DUAL) acu[jj][r] = 0.f;
        }
      for (int k = lane * VN; k < K; k += 32 * VN) {
        float wv[4][8], uv[DUAL ? 4 : 1][8], av[8];
#pragma unroll
        for (int jj = 0; jj < 4; ++jj) {
          Vec16<T>::load(wg[jj] + k, wv[jj]);
          if (DUAL) Vec16<T>::load(wu[jj] + k, uv[jj]);
        }
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r) {
          if (r < rows) {
            Vec16<T>::load(As + (size_t)r * K + k, av);
#pragma unroll
            for (int jj = 0; jj < 4; ++jj)
#pragma unroll
              for (int i = 0; i < VN; ++i) {
                acc[jj][r] = fmaf(av[i], wv[jj][i], acc[jj][r]);
                if (DUAL) acu[jj][r] = fmaf(av[i], uv[jj][i], acu[jj][r]);
              }
          }
        }
      }
#pragma unroll
      for (int jj = 0; jj < 4; ++jj) {
        const int n = n_base + j0 + jj;
#pragma unroll
        for (int r = 0; r < GEMV_ROWS; ++r) {
          if (r >= rows) break;
          const float g = gi::warp_sum(acc[jj][r]);
          if (DUAL) {
            const float u = gi::warp_sum(acu[jj][r]);
            if (lane == 0 && n < N) gi::stf((T*)out_ + (size_t)(r0 + r) * N + n, gated_value(g, u, limit, alpha));
          } else if (lane == 0 && n < N) {
            if (act_out) {
              const float z = fmaxf(g, 0.f);
              gi::stf((T*)out_ + (size_t)(r0 + r) * N + n, z * z);
            } else {
              ((float*)out_)[(size_t)(r0 + r) * N + n] = g;
            }
          }
        }
      }
    }
  }
}

// out[r, :] = in[idx[r] / top, :]: the rows of a step in the order of the sort, for products that want an expert's rows
// side by side.
template <typename T>
__global__ void gather_rows_kernel(T* __restrict__ out, const T* __restrict__ in, long ld_in, const int* __restrict__ idx,
                                   int top, int width, const float* __restrict__ scale) {
  gi::pdl_prologue();
  const int r = blockIdx.x;
  const T* src = in + (size_t)(idx[r] / top) * ld_in;
  if (scale == nullptr) {
    for (int i = threadIdx.x; i < width; i += blockDim.x) out[(size_t)r * width + i] = src[i];
  } else {
    // the entry's weight goes onto what the expert reads (32-bit product, rounded to the rows' type)
    const float s = scale[idx[r]];
    for (int i = threadIdx.x; i < width; i += blockDim.x) gi::stf(out + (size_t)r * width + i, gi::ldf(src + i) * s);
  }
}

__global__ void __launch_bounds__(256)
combine_kernel(float* __restrict__ residual, const float* __restrict__ down, const int* __restrict__ inv,
               const float* __restrict__ wts, const float* __restrict__ shared, const float* __restrict__ sgate, int width,
               int top) {
  gi::pdl_prologue();
  const int t = blockIdx.x;
  for (int i = blockIdx.y * blockDim.x + threadIdx.x; i < width; i += gridDim.y * blockDim.x) {
    float acc = 0.f;
    for (int k = 0; k < top; ++k)      // without weights (they went onto the experts' inputs): the plain sum
      acc = fmaf(wts != nullptr ? wts[(size_t)t * top + k] : 1.0f, down[(size_t)inv[(size_t)t * top + k] * width + i], acc);
    if (shared != nullptr) acc = fmaf(sgate[t], shared[(size_t)t * width + i], acc);
    residual[(size_t)t * width + i] += acc;
  }
}

}  // namespace

extern "C" int gi_moe_route(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                            const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, void* stream) {
  return gi_moe_route_scored(ids, wts, sgate, h, dtype, ldh, w_router, w_sg, w_dtype, n_tokens, width, experts, top, 0, stream);
}

extern "C" int gi_moe_route_scored(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                                   const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, int score_mode,
                                   void* stream) {
  return gi_moe_route_shares(ids, wts, sgate, h, dtype, ldh, w_router, w_sg, w_dtype, n_tokens, width, experts, top, score_mode,
                             nullptr, 1.0f, stream);
}

extern "C" int gi_moe_route_shares(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                                   const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, int score_mode,
                                   const float* correction, float weight_scale, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (score_mode < 0 || score_mode > 2) return gi::fail(GI_ERR_ARG, "router: unknown kind of weights %d", score_mode);
  if (experts < 1 || top < 1 || top > experts || top > 32 || experts > 8192)
    return gi::fail(GI_ERR_UNSUPPORTED, "router: %d of %d experts (at most 32 of 8192)", top, experts);
  if (w_sg != nullptr && sgate == nullptr) return gi::fail(GI_ERR_ARG, "router: a shared gate needs somewhere to go");
  const size_t smem = (((size_t)width + 7) / 8 * 8 + 2 * (size_t)experts) * sizeof(float);
  if (smem > 200 * 1024) return gi::fail(GI_ERR_UNSUPPORTED, "router: rows of %d values are wider than its shared memory", width);
  const int per = w_dtype == GI_F32 ? 4 : 8;
  const int vec = (width % per == 0 && !(((uintptr_t)w_router | (uintptr_t)w_sg) & 15)) ? 1 : 0;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, GI_DISPATCH_DTYPE(w_dtype, TW, {
      auto kern = route_kernel<T, TW>;
      if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
      if (e == cudaSuccess)
        e = gi::launch(kern, dim3(n_tokens), dim3(128), smem, (cudaStream_t)stream, ids, wts, sgate, (const T*)h, ldh,
                       (const TW*)w_router, (const TW*)w_sg, n_tokens, width, experts, top, vec, score_mode, correction, weight_scale);
  }));
  return gi::check(e, "router");
}

extern "C" int gi_moe_plan(int* offsets, int* perm, int* inv, int* scratch, const int* ids, int entries, int experts,
                           void* stream) {
  if (entries <= 0) return GI_OK;
  if (experts < 1 || experts > 8192) return gi::fail(GI_ERR_UNSUPPORTED, "router plan: %d experts (at most 8192)", experts);
  const int n_seg = (entries + SEG - 1) / SEG;
  int* seg_count = scratch;                          // [n_seg][experts]
  int* local_rank = scratch + (size_t)n_seg * experts;   // [entries]
  cudaStream_t s = (cudaStream_t)stream;
  cudaError_t e = gi::launch(rank_kernel, dim3(n_seg), dim3(SEG), (SEG + (size_t)experts) * sizeof(int), s, local_rank, seg_count,
                             ids, entries, experts);
  if (e == cudaSuccess)
    e = gi::launch(offsets_kernel, dim3(1), dim3(experts < 1024 ? ((experts + 31) / 32) * 32 : 1024), (size_t)experts * sizeof(int),
                   s, offsets, seg_count, n_seg, experts);
  if (e == cudaSuccess)
    e = gi::launch(place_kernel, dim3(n_seg), dim3(SEG), 0, s, perm, inv, (const int*)offsets, (const int*)seg_count,
                   (const int*)local_rank, ids, entries, experts);
  return gi::check(e, "router plan");
}

extern "C" int gi_moe_gemm_gate_up(void* out, int dtype, const void* a, long lda, const void* w, int w_dtype, long w_stride,
                                   const int* offsets, const int* perm, int entries, int top, int experts, int f, int k,
                                   int interleaved, void* stream) {
  return gi_moe_gemm_gate_up_clamped(out, dtype, a, lda, w, w_dtype, w_stride, offsets, perm, entries, top, experts, f, k, interleaved,
                                     0.f, 1.0f, stream);
}

extern "C" int gi_moe_gemm_gate_up_clamped(void* out, int dtype, const void* a, long lda, const void* w, int w_dtype, long w_stride,
                                           const int* offsets, const int* perm, int entries, int top, int experts, int f, int k,
                                           int interleaved, float limit, float alpha, void* stream) {
  if (entries <= 0) return GI_OK;
  if (f <= 0 || k <= 0 || top < 1) return gi::fail(GI_ERR_ARG, "expert product: bad sizes");
  if (interleaved && f % 8 != 0) return gi::fail(GI_ERR_ARG, "expert product: interleaved rows need a width that is a multiple of 8");
  if (entries <= GEMV_MAX_ENTRIES && gemv_ok(dtype, w_dtype, k, a, w, lda)) {
    cudaError_t e = cudaSuccess;
    const size_t smem = (size_t)GEMV_ROWS * k * (dtype == GI_F32 ? 4 : 2);
    dim3 grid((f + GEMV_COLS - 1) / GEMV_COLS, experts);
    GI_DISPATCH_DTYPE(dtype, T, {
        auto kern = expert_gemv_kernel<T, true>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
          e = gi::launch(kern, grid, dim3(GEMV_WARPS * 32), smem, (cudaStream_t)stream, out, (const T*)a, lda, (const T*)w, w_stride,
                         offsets, perm, top, f, k, interleaved, 0, limit, alpha);
    });
    return gi::check(e, "expert product (gate, up; few rows)");
  }
  const long tiles = (entries + BM - 1) / BM + experts;
  if (tiles > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "expert product: %d rows are more than one launch takes", entries);
  dim3 grid((f + BN - 1) / BN, (unsigned)tiles);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, TA, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(expert_gemm_kernel<TA, TW, true>, grid, dim3(256), 0, (cudaStream_t)stream, out, (const TA*)a, lda,
                     (const TW*)w, w_stride, offsets, perm, top, experts, f, k, interleaved, 0, limit, alpha)));
  return gi::check(e, "expert product (gate, up)");
}

extern "C" int gi_moe_gemm_down(float* out, const void* a, int dtype, long lda, const void* w, int w_dtype, long w_stride,
                                const int* offsets, int entries, int experts, int n, int k, void* stream) {
  return gi_moe_gemm_rows((void*)out, a, dtype, lda, w, w_dtype, w_stride, offsets, entries, experts, n, k, 0, stream);
}

extern "C" int gi_moe_gemm_rows(void* out, const void* a, int dtype, long lda, const void* w, int w_dtype, long w_stride,
                                const int* offsets, int entries, int experts, int n, int k, int act_out, void* stream) {
  if (entries <= 0) return GI_OK;
  if (act_out != 0 && act_out != 1) return gi::fail(GI_ERR_ARG, "expert product: unknown activation %d", act_out);
  if (n <= 0 || k <= 0) return gi::fail(GI_ERR_ARG, "expert product: bad sizes");
  if (entries <= GEMV_MAX_ENTRIES && gemv_ok(dtype, w_dtype, k, a, w, lda)) {
    cudaError_t e = cudaSuccess;
    const size_t smem = (size_t)GEMV_ROWS * k * (dtype == GI_F32 ? 4 : 2);
    dim3 grid((n + GEMV_COLS - 1) / GEMV_COLS, experts);
    GI_DISPATCH_DTYPE(dtype, T, {
        auto kern = expert_gemv_kernel<T, false>;
        if (smem > 48 * 1024) e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e == cudaSuccess)
          e = gi::launch(kern, grid, dim3(GEMV_WARPS * 32), smem, (cudaStream_t)stream, (void*)out, (const T*)a, lda, (const T*)w,
                         w_stride, offsets, (const int*)nullptr, 1, n, k, 0, act_out, 0.f, 1.0f);
    });
    return gi::check(e, "expert product (down; few rows)");
  }
  const long tiles = (entries + BM - 1) / BM + experts;
  if (tiles > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "expert product: %d rows are more than one launch takes", entries);
  dim3 grid((n + BN - 1) / BN, (unsigned)tiles);
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, TA, GI_DISPATCH_DTYPE(w_dtype, TW,
      e = gi::launch(expert_gemm_kernel<TA, TW, false>, grid, dim3(256), 0, (cudaStream_t)stream, (void*)out, (const TA*)a, lda,
                     (const TW*)w, w_stride, offsets, (const int*)nullptr, 1, experts, n, k, 0, act_out, 0.f, 1.0f)));
  return gi::check(e, "expert product (down)");
}

extern "C" int gi_moe_combine(float* residual, const float* down, const int* inv, const float* wts, const float* shared,
                              const float* sgate, int n_tokens, int width, int top, void* stream) {
  if (n_tokens <= 0) return GI_OK;
  if (shared != nullptr && sgate == nullptr) return gi::fail(GI_ERR_ARG, "expert combine: a shared output needs its gate");
  // few tokens: a row's columns over several blocks
  const int col_blocks = n_tokens >= 256 ? 1 : min(64, (width + 255) / 256);
  return gi::check(gi::launch(combine_kernel, dim3(n_tokens, col_blocks), dim3(256), 0, (cudaStream_t)stream, residual, down, inv, wts, shared,
                              sgate, width, top), "expert combine");
}

extern "C" int gi_moe_gather_rows(void* out, const void* in, int dtype, long ld_in, const int* perm, int entries, int top,
                                  int width, void* stream) {
  return gi_moe_gather_rows_scaled(out, in, dtype, ld_in, perm, nullptr, entries, top, width, stream);
}

extern "C" int gi_moe_gather_rows_scaled(void* out, const void* in, int dtype, long ld_in, const int* perm, const float* scale,
                                         int entries, int top, int width, void* stream) {
  if (entries <= 0) return GI_OK;
  if (top < 1 || width <= 0) return gi::fail(GI_ERR_ARG, "gather: bad sizes");
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, e = gi::launch(gather_rows_kernel<T>, dim3(entries), dim3(256), 0, (cudaStream_t)stream, (T*)out,
                                             (const T*)in, ld_in, perm, top, width, scale));
  return gi::check(e, "gather rows");
}

// A prompt step's experts through the tensor-core products, expert by expert, from offsets the host has read back: for
// every expert with rows, hidden = act(rows W_gate^T) * (rows W_up^T) (gate and up rows interleaved in blocks of 8) and
// out = hidden W_down^T as float, over the expert's stretch of the sorted rows.  Stretches of up to 64 rows take the
// streamed product, longer ones the tiled one.  One call per layer, so that the host's share is the launches alone.
static int experts_tc(float* out, void* hidden, const void* rows, const void* w_gate_up, long gate_up_stride,
                      const void* w_down, long down_stride, const int* host_offsets, int experts, int width, int f,
                      float* scratch, int* counters, int n_counters, void* stream, bool ungated, float limit = 0.f, float alpha = 1.f);

// The same for gated experts in the clamped form (limit > 0; see gi_clamped_glu): every stretch takes the tiled product.
extern "C" int gi_moe_experts_tc_clamped(float* out, void* hidden, const void* rows, const void* w_gate_up, long gate_up_stride,
                                         const void* w_down, long down_stride, const int* host_offsets, int experts, int width,
                                         int f, float limit, float alpha, float* scratch, int* counters, int n_counters, void* stream) {
  if (!(limit > 0.f)) return gi::fail(GI_ERR_ARG, "experts on tensor cores: the clamped form needs a positive limit");
  return experts_tc(out, hidden, rows, w_gate_up, gate_up_stride, w_down, down_stride, host_offsets, experts, width, f, scratch,
                    counters, n_counters, stream, false, limit, alpha);
}

extern "C" int gi_moe_experts_tc(float* out, void* hidden, const void* rows, const void* w_gate_up, long gate_up_stride,
                                 const void* w_down, long down_stride, const int* host_offsets, int experts, int width, int f,
                                 float* scratch, int* counters, int n_counters, void* stream) {
  return experts_tc(out, hidden, rows, w_gate_up, gate_up_stride, w_down, down_stride, host_offsets, experts, width, f, scratch,
                    counters, n_counters, stream, false);
}

// The same for ungated experts: hidden = relu(rows W_up^T)^2 (w_up [experts][f][width]), the activation in the first
// product's epilogue; every stretch takes the tiled product.
extern "C" int gi_moe_experts_tc_ungated(float* out, void* hidden, const void* rows, const void* w_up, long up_stride,
                                         const void* w_down, long down_stride, const int* host_offsets, int experts, int width,
                                         int f, float* scratch, int* counters, int n_counters, void* stream) {
  return experts_tc(out, hidden, rows, w_up, up_stride, w_down, down_stride, host_offsets, experts, width, f, scratch, counters,
                    n_counters, stream, true);
}

static int experts_tc(float* out, void* hidden, const void* rows, const void* w_gate_up, long gate_up_stride,
                      const void* w_down, long down_stride, const int* host_offsets, int experts, int width, int f,
                      float* scratch, int* counters, int n_counters, void* stream, bool ungated, float limit, float alpha) {
  if (experts <= 0 || width <= 0 || f <= 0 || f % 8 != 0 || width % 8 != 0)
    return gi::fail(GI_ERR_UNSUPPORTED, "experts on tensor cores: width %d and hidden width %d must be multiples of 8", width, f);
  const __nv_bfloat16* a = (const __nv_bfloat16*)rows;
  __nv_bfloat16* h = (__nv_bfloat16*)hidden;
  cudaStream_t main_stream = (cudaStream_t)stream;
  // An expert's stretch of a few hundred rows makes fewer tiles than the GPU has SMs, so the longer stretches go round
  // four side streams (an expert's two products one after the other on its stream) between a fork and a join on the
  // caller's stream; the short ones, whose streamed product shares its scratch memory, follow on the caller's stream.
  constexpr int SIDE = 4;
  static cudaStream_t side[gi::MAX_DEVICES_SEEN][SIDE];
  static cudaEvent_t fork_ev[gi::MAX_DEVICES_SEEN], join_ev[gi::MAX_DEVICES_SEEN][SIDE];
  static bool made[gi::MAX_DEVICES_SEEN] = {false};
  int dev = -1;
  bool many = false;
  const int small = (ungated || limit > 0.f) ? 0 : 64;      // stretches of up to this many rows take the streamed product (silu-gated experts only)
  const int up_rows = ungated ? f : 2 * f;
  for (int e = 0; e < experts; ++e) many = many || host_offsets[e + 1] - host_offsets[e] > small;
  cudaStreamCaptureStatus capturing = cudaStreamCaptureStatusNone;
  cudaStreamIsCapturing(main_stream, &capturing);
  bool fan = many && capturing == cudaStreamCaptureStatusNone && cudaGetDevice(&dev) == cudaSuccess && dev >= 0 && dev < gi::MAX_DEVICES_SEEN;
  if (fan && !made[dev]) {
    bool ok = cudaEventCreateWithFlags(&fork_ev[dev], cudaEventDisableTiming) == cudaSuccess;
    for (int i = 0; ok && i < SIDE; ++i)
      ok = cudaStreamCreateWithFlags(&side[dev][i], cudaStreamNonBlocking) == cudaSuccess &&
           cudaEventCreateWithFlags(&join_ev[dev][i], cudaEventDisableTiming) == cudaSuccess;
    if (!ok) { cudaGetLastError(); fan = false; } else made[dev] = true;
  }
  if (fan) {
    if (cudaEventRecord(fork_ev[dev], main_stream) != cudaSuccess) return gi::fail(GI_ERR_CUDA, "experts on tensor cores: fork");
    for (int i = 0; i < SIDE; ++i) cudaStreamWaitEvent(side[dev][i], fork_ev[dev], 0);
  }
  int turn = 0;
  for (int e = 0; e < experts; ++e) {
    const int lo = host_offsets[e], m = host_offsets[e + 1] - lo;
    if (m <= small) continue;
    const __nv_bfloat16* wgu = (const __nv_bfloat16*)w_gate_up + (size_t)e * gate_up_stride;
    const __nv_bfloat16* wd = (const __nv_bfloat16*)w_down + (size_t)e * down_stride;
    cudaStream_t s = fan ? side[dev][turn++ % SIDE] : main_stream;
    // narrower tiles where wide ones would leave most SMs without one
    const int row_tiles = (m + 127) / 128;
    const int tile_up = row_tiles * ((up_rows + 255) / 256) < 64 ? 128 : 256, tile_down = row_tiles * ((width + 255) / 256) < 64 ? 128 : 256;
    int rc = limit > 0.f ? gi_gemm_tc_bf16_clamped(h + (size_t)lo * f, a + (size_t)lo * width, wgu, m, up_rows, width, width, width, f, tile_up,
                                                   limit, alpha, s)
                         : gi_gemm_tc_bf16(h + (size_t)lo * f, ungated ? (GI_TC_STORE_BF16 | GI_ACT_RELU2) : GI_TC_SWIGLU, a + (size_t)lo * width,
                                           wgu, m, up_rows, width, width, width, f, tile_up, s);
    if (rc == GI_OK)
      rc = gi_gemm_tc_bf16(out + (size_t)lo * width, GI_TC_STORE_F32, h + (size_t)lo * f, wd, m, width, f, f, f, width, tile_down, s);
    if (rc != GI_OK) return rc;
  }
  if (fan) {
    for (int i = 0; i < SIDE; ++i) {
      cudaEventRecord(join_ev[dev][i], side[dev][i]);
      cudaStreamWaitEvent(main_stream, join_ev[dev][i], 0);
    }
    if (cudaGetLastError() != cudaSuccess) return gi::fail(GI_ERR_CUDA, "experts on tensor cores: join");
  }
  for (int e = 0; e < experts; ++e) {
    const int lo = host_offsets[e], m = host_offsets[e + 1] - lo;
    if (m <= 0 || m > small) continue;
    const __nv_bfloat16* wgu = (const __nv_bfloat16*)w_gate_up + (size_t)e * gate_up_stride;
    const __nv_bfloat16* wd = (const __nv_bfloat16*)w_down + (size_t)e * down_stride;
    int rc = gi_gemm_stream_bf16(h + (size_t)lo * f, GI_SKINNY_SWIGLU, a + (size_t)lo * width, wgu, scratch, counters, n_counters, m,
                                 2 * f, width, width, width, f, -1, main_stream);
    if (rc == GI_OK)
      rc = gi_gemm_stream_bf16(out + (size_t)lo * width, GI_SKINNY_STORE_F32, h + (size_t)lo * f, wd, scratch, counters, n_counters,
                               m, width, f, f, f, width, -1, main_stream);
    if (rc != GI_OK) return rc;
  }
  return GI_OK;
}
