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
// Work split: grid (heads, sequences, tiles of 32, 16 or 8 columns of S; the widest tile that still gives every SM a
// block is chosen by the launcher).  A column of S (K numbers) belongs to 8 neighbouring lanes; lane l holds rows
// 4 (l + 8 m) .. + 3 for m = 0, 1, ..., so a column's rows are read from the state, and a token's key and query from shared
// memory, sixteen bytes at a time.  The delta rule's S^T k ends with three exchanges among a column's lanes, token by
// token, since the next write depends on it; the read-outs S^T q of eight tokens are exchanged together (seven exchanges
// instead of twenty-four).  The order of every sum follows from K alone: one token or a thousand, alone or in a batch,
// whatever the tile, give the same bits.
// Four more warps of the block prepare the next tokens while these work: together they load a chunk's rows (sixteen bytes a
// thread where the rows allow it, every load before anything is computed from it, so a chunk costs one trip to memory),
// apply silu on the way into shared memory, then the unit norms (one warp per token, in place), the decay and the write
// strength, and write the previous chunk's read-outs to memory in whole lines.  Two buffers in shared memory, one barrier
// of the block per chunk.
// State per slot: [heads][V][K] floats (a column's rows side by side) at the start of the slot's row; slot -1 (a padding row
// of a fixed-size launch) uses the last row of the matrix.
#include <math.h>

#include "api.h"
#include "common.cuh"

namespace {

constexpr int LS_LANES = 8;        // lanes of a column
constexpr int LS_PREP = 128;       // threads that prepare tokens and write read-outs
constexpr int LS_TB = 8;           // read-outs exchanged together

__device__ __forceinline__ float ls_silu(float v) { return v / (1.0f + expf(-v)); }
__device__ __forceinline__ float ls_softplus(float v) { return v > 20.f ? v : log1pf(expf(v)); }

// One halving step among a column's 8 lanes: of 2 * HALF values a lane keeps the half its bit `BIT` of the lane number
// names and adds the other lane's partial sums of the same values.
template <int HALF, int BIT>
__device__ __forceinline__ void ls_halve(float (&v)[LS_TB], int lane) {
  const bool upper = (lane & BIT) != 0;
#pragma unroll
  for (int k = 0; k < HALF; ++k) {
    const float send = upper ? v[k] : v[k + HALF];
    const float keep = upper ? v[k + HALF] : v[k];
    v[k] = keep + __shfl_xor_sync(0xffffffffu, send, BIT);
  }
}

// Sixteen bytes of a row as 32-bit numbers.
__device__ __forceinline__ void ls_load16(const float* p, float (&out)[4]) {
  const float4 v = *reinterpret_cast<const float4*>(p);
  out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
__device__ __forceinline__ void ls_load16(const __nv_bfloat16* p, float (&out)[8]) {
  const uint4 v = *reinterpret_cast<const uint4*>(p);
  const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    out[2 * i] = __uint_as_float(w[i] << 16);
    out[2 * i + 1] = __uint_as_float(w[i] & 0xffff0000u);
  }
}
// The preparing threads among themselves (barrier 1; the block's own barrier is 0).
__device__ __forceinline__ void ls_prep_barrier() { asm volatile("bar.sync 1, %0;" ::"n"(LS_PREP) : "memory"); }

struct LsArgs {
  float* o;
  const void *q, *k, *v, *a_in, *b_in;
  long ldq, ldk, ldv, lda, ldb;
  const float *decay_c, *dt_bias;
  const float *g_direct, *u_direct;      // per token and head, ready made: the decay itself and what multiplies the written value
  float* state;
  long state_ld;
  int state_rows;
  const int *cu_seqlens, *seq_slots;
  int heads, qk_heads, K, V, in_act, unit_norm, vec_state, vec_in;
  float norm_eps, q_scale;
};

// tokens per chunk: two buffers of it stay under 48 KB of shared memory
template <int KR> struct LsChunk { static constexpr int value = KR >= 32 ? 8 : 16; };

// WALK: the step holds sequences of many tokens, and eight whole tokens run without a test between them; without it (steps
// of one token a sequence) the kernel is the same but smaller, so that two blocks fit an SM at every tile width.
// Two blocks an SM for the narrower tiles too: a grid of about as many blocks as SMs times two then runs as one round.
template <typename T, int KR, int COLS, bool DELTA, bool WALK>
__global__ void __launch_bounds__(COLS * LS_LANES + LS_PREP, (COLS <= 16 || !WALK) ? 2 : 1)
linear_state_kernel(const LsArgs a) {
  constexpr int Kp = KR * LS_LANES;            // rows with padding
  constexpr int M = KR / 4;                    // groups of four rows per lane; also a preparing lane's share of a row
  constexpr int NC = COLS * LS_LANES;          // threads that hold S
  constexpr int CH = LsChunk<KR>::value;
  constexpr int BUF = 2 * CH * Kp + 2 * CH * COLS + 2 * CH;
  constexpr int VW = 16 / (int)sizeof(T);      // numbers of a row in sixteen bytes
  static_assert(CH % LS_TB == 0 && CH <= LS_PREP && (CH * Kp) % LS_PREP == 0 && COLS % VW == 0 && CH * COLS / VW <= LS_PREP,
                "whole exchanges; a preparing thread per token, and per group of a chunk's values");
  extern __shared__ __align__(16) float sm[];
  gi::pdl_prologue();
  const int h = blockIdx.x, b = blockIdx.y, j0 = blockIdx.z * COLS;
  const int tok0 = a.cu_seqlens[b], qlen = a.cu_seqlens[b + 1] - tok0;
  if (qlen <= 0) return;
  const int K = a.K, V = a.V;
  const int slot = a.seq_slots[b];
  float* S_row = a.state + (size_t)(slot >= 0 ? slot : a.state_rows - 1) * a.state_ld + (size_t)h * V * K;
  const int hk = h / (a.heads / a.qk_heads);
  const int tid = threadIdx.x;
  const bool prep = tid >= NC;
  const int n_chunks = (qlen + CH - 1) / CH;
  const size_t o_ld = (size_t)a.heads * V;
  const T* qp = (const T*)a.q; const T* kp = (const T*)a.k; const T* vp = (const T*)a.v;
  const T* ap = (const T*)a.a_in; const T* bp = (const T*)a.b_in;
  const float dc = a.decay_c != nullptr ? a.decay_c[h] : 1.0f;
  const float rate = ap != nullptr ? expf(dc) : 0.f, bias = (ap != nullptr && a.dt_bias != nullptr) ? a.dt_bias[h] : 0.f;

  // a chunk's tokens made ready in buffer `buf` by the 128 preparing threads together.  First every thread loads its share
  // of the chunk's rows (sixteen bytes at a time where the rows allow it), all loads before anything is computed from them,
  // so a chunk costs one trip to memory; silu is applied on the way into shared memory.  Then, for unit vectors, one warp
  // per token sums the squares of its row in shared memory and scales it in place.
  auto prepare = [&](int c, float* buf) {
    float* sq = buf; float* sk = sq + CH * Kp; float* sv = sk + CH * Kp; float* sg = sv + CH * COLS; float* sb = sg + CH;
    const int n = min(CH, qlen - c * CH);
    const int pt = tid - NC;
    const size_t tokc = (size_t)tok0 + (size_t)c * CH;
    const bool act = a.in_act != 0;
    // decay and write strength: one thread per token
    float av = 0.f, bv = 0.f;
    if (pt < n) {
      if (ap != nullptr) av = gi::ldf(ap + (tokc + pt) * a.lda + h);
      if (bp != nullptr) bv = gi::ldf(bp + (tokc + pt) * a.ldb + h);
    }
    if (a.vec_in) {
      constexpr int QG = (CH * Kp / VW + LS_PREP - 1) / LS_PREP;     // groups of VW numbers a thread moves, per operand
      const int gpr = K / VW, total = n * gpr;
      float qr[QG][VW], kr[QG][VW];
#pragma unroll
      for (int i = 0; i < QG; ++i) {
        const int g = pt + i * LS_PREP;
        if (g < total) {
          const int t = g / gpr, r0 = (g - t * gpr) * VW;
          ls_load16(qp + (tokc + t) * a.ldq + (size_t)hk * K + r0, qr[i]);
          ls_load16(kp + (tokc + t) * a.ldk + (size_t)hk * K + r0, kr[i]);
        }
      }
      float vr[VW];
      const int vpr = COLS / VW, vt = pt / vpr, vc = (pt - vt * vpr) * VW;     // at most CH * COLS / VW <= 128 groups
      const bool vlive = vt < n && j0 + vc < V;
      if (vlive) ls_load16(vp + (tokc + vt) * a.ldv + (size_t)h * V + j0 + vc, vr);
#pragma unroll
      for (int i = 0; i < QG; ++i) {
        const int g = pt + i * LS_PREP;
        if (g < total) {
          const int t = g / gpr, r0 = (g - t * gpr) * VW;
#pragma unroll
          for (int e = 0; e < VW; e += 4) {
            float4 q4 = make_float4(qr[i][e], qr[i][e + 1], qr[i][e + 2], qr[i][e + 3]);
            float4 k4 = make_float4(kr[i][e], kr[i][e + 1], kr[i][e + 2], kr[i][e + 3]);
            if (act) {
              q4.x = ls_silu(q4.x); q4.y = ls_silu(q4.y); q4.z = ls_silu(q4.z); q4.w = ls_silu(q4.w);
              k4.x = ls_silu(k4.x); k4.y = ls_silu(k4.y); k4.z = ls_silu(k4.z); k4.w = ls_silu(k4.w);
            }
            *reinterpret_cast<float4*>(sq + t * Kp + r0 + e) = q4;
            *reinterpret_cast<float4*>(sk + t * Kp + r0 + e) = k4;
          }
        }
      }
      if (vlive) {
#pragma unroll
        for (int e = 0; e < VW; ++e) sv[vt * COLS + vc + e] = act ? ls_silu(vr[e]) : vr[e];     // V is a multiple of VW here
      }
    } else {
      constexpr int QS = CH * Kp / LS_PREP, VS = (CH * COLS + LS_PREP - 1) / LS_PREP;
      const int total = n * K;
      float qr[QS], kr[QS], vr[VS];
#pragma unroll
      for (int i = 0; i < QS; ++i) {
        const int e = pt + i * LS_PREP;
        if (e < total) {
          const int t = e / K, r = e - t * K;
          qr[i] = gi::ldf(qp + (tokc + t) * a.ldq + (size_t)hk * K + r);
          kr[i] = gi::ldf(kp + (tokc + t) * a.ldk + (size_t)hk * K + r);
        }
      }
#pragma unroll
      for (int i = 0; i < VS; ++i) {
        const int e = pt + i * LS_PREP, t = e / COLS, cc = e % COLS;
        vr[i] = (t < n && j0 + cc < V) ? gi::ldf(vp + (tokc + t) * a.ldv + (size_t)h * V + j0 + cc) : 0.f;
      }
#pragma unroll
      for (int i = 0; i < QS; ++i) {
        const int e = pt + i * LS_PREP;
        if (e < total) {
          const int t = e / K, r = e - t * K;
          sq[t * Kp + r] = act ? ls_silu(qr[i]) : qr[i];
          sk[t * Kp + r] = act ? ls_silu(kr[i]) : kr[i];
        }
      }
#pragma unroll
      for (int i = 0; i < VS; ++i) {
        const int e = pt + i * LS_PREP;
        if (e < n * COLS) sv[e] = act ? ls_silu(vr[i]) : vr[i];
      }
    }
    if (pt < n) {
      sg[pt] = ap != nullptr ? expf(-rate * ls_softplus(av + bias)) : dc;
      sb[pt] = bp != nullptr ? 1.0f / (1.0f + expf(-bv)) : 1.0f;
      if (a.g_direct != nullptr) sg[pt] = a.g_direct[(tokc + pt) * a.heads + h];
      if (a.u_direct != nullptr) sb[pt] = a.u_direct[(tokc + pt) * a.heads + h];
    }
    if (a.unit_norm) {
      ls_prep_barrier();             // the chunk's rows are in shared memory
      const int pw = pt >> 5, pl = pt & 31;
      for (int t = pw; t < n; t += LS_PREP / 32) {
        float qv[M], kv[M];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int i = 0; i < M; ++i) {
          qv[i] = sq[t * Kp + pl + 32 * i];
          kv[i] = sk[t * Kp + pl + 32 * i];
          s1 = fmaf(qv[i], qv[i], s1);
          s2 = fmaf(kv[i], kv[i], s2);
        }
        s1 = gi::warp_sum(s1);
        s2 = gi::warp_sum(s2);
        const float fq = a.q_scale / sqrtf(s1 + a.norm_eps), fk = 1.0f / sqrtf(s2 + a.norm_eps);
#pragma unroll
        for (int i = 0; i < M; ++i) {
          sq[t * Kp + pl + 32 * i] = qv[i] * fq;
          sk[t * Kp + pl + 32 * i] = kv[i] * fk;
        }
      }
    }
  };
  // a chunk's read-outs from buffer `buf` to memory, by the threads [first, first + count)
  auto write_out = [&](int c, const float* buf, int first, int count) {
    const float* so = buf + 2 * CH * Kp + CH * COLS + 2 * CH;
    const int n = min(CH, qlen - c * CH);
    for (int idx = tid - first; idx < n * COLS; idx += count) {
      const int t = idx / COLS, cc = idx % COLS;
      if (j0 + cc < V) a.o[((size_t)tok0 + (size_t)c * CH + t) * o_ld + (size_t)h * V + j0 + cc] = so[idx];
    }
  };

  const int col = tid / LS_LANES, lane = tid % LS_LANES;    // of the threads that hold S
  const int j = j0 + col;
  float S[KR];
  if (prep) {
    if (K < Kp) {                  // rows past K stay zero in both buffers: nothing writes them again
      for (int e = tid - NC; e < 2 * CH * Kp; e += LS_PREP) {
        if (e % Kp >= K) { sm[e] = 0.f; sm[BUF + e] = 0.f; }
      }
      ls_prep_barrier();
    }
    prepare(0, sm);
  } else {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const int i = 4 * (lane + LS_LANES * m);
      if (a.vec_state && j < V && i < K) {
        const float4 s4 = *reinterpret_cast<const float4*>(S_row + (size_t)j * K + i);
        S[4 * m] = s4.x; S[4 * m + 1] = s4.y; S[4 * m + 2] = s4.z; S[4 * m + 3] = s4.w;
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e) S[4 * m + e] = (j < V && i + e < K) ? S_row[(size_t)j * K + i + e] : 0.f;
      }
    }
  }
  for (int c = 0; c < n_chunks; ++c) {
    __syncthreads();             // chunk c is ready in buffer c & 1; the other buffer's tokens and this one's read-outs are used up
    float* buf = sm + (c & 1) * BUF;
    if (prep) {
      if (c > 0) write_out(c - 1, sm + ((c - 1) & 1) * BUF, NC, LS_PREP);
      if (c + 1 < n_chunks) prepare(c + 1, sm + ((c + 1) & 1) * BUF);
      continue;
    }
    const float* sq = buf; const float* sk = sq + CH * Kp; const float* sv = sk + CH * Kp;
    const float* sg = sv + CH * COLS; const float* sb = sg + CH;
    float* so = buf + 2 * CH * Kp + CH * COLS + 2 * CH;
    const int n = min(CH, qlen - c * CH);
    // one token: the state's columns walk on, `out` takes this lane's share of the read-out
    auto token = [&](int t, float& out) {
      const float g = sg[t];
      float kk[KR], qq[KR];
#pragma unroll
      for (int m = 0; m < M; ++m) {
        const float4 k4 = *reinterpret_cast<const float4*>(sk + t * Kp + 4 * (lane + LS_LANES * m));
        const float4 q4 = *reinterpret_cast<const float4*>(sq + t * Kp + 4 * (lane + LS_LANES * m));
        kk[4 * m] = k4.x; kk[4 * m + 1] = k4.y; kk[4 * m + 2] = k4.z; kk[4 * m + 3] = k4.w;
        qq[4 * m] = q4.x; qq[4 * m + 1] = q4.y; qq[4 * m + 2] = q4.z; qq[4 * m + 3] = q4.w;
      }
      float u = sv[t * COLS + col];
      if (DELTA) {
        float d0 = 0.f, d1 = 0.f, d2 = 0.f, d3 = 0.f;     // four chains, then a tree: the order is fixed by K alone
#pragma unroll
        for (int m = 0; m < M; ++m) {
          d0 = fmaf(S[4 * m], kk[4 * m], d0);
          d1 = fmaf(S[4 * m + 1], kk[4 * m + 1], d1);
          d2 = fmaf(S[4 * m + 2], kk[4 * m + 2], d2);
          d3 = fmaf(S[4 * m + 3], kk[4 * m + 3], d3);
        }
        float d = (d0 + d1) + (d2 + d3);
        d += __shfl_xor_sync(0xffffffffu, d, 1);
        d += __shfl_xor_sync(0xffffffffu, d, 2);
        d += __shfl_xor_sync(0xffffffffu, d, 4);
        u = sb[t] * (u - g * d);
      } else if (a.u_direct != nullptr) {
        u *= sb[t];
      }
      float a0 = 0.f, a1 = 0.f, a2 = 0.f, a3 = 0.f;
#pragma unroll
      for (int m = 0; m < M; ++m) {
        S[4 * m] = fmaf(kk[4 * m], u, g * S[4 * m]);
        S[4 * m + 1] = fmaf(kk[4 * m + 1], u, g * S[4 * m + 1]);
        S[4 * m + 2] = fmaf(kk[4 * m + 2], u, g * S[4 * m + 2]);
        S[4 * m + 3] = fmaf(kk[4 * m + 3], u, g * S[4 * m + 3]);
        a0 = fmaf(S[4 * m], qq[4 * m], a0);
        a1 = fmaf(S[4 * m + 1], qq[4 * m + 1], a1);
        a2 = fmaf(S[4 * m + 2], qq[4 * m + 2], a2);
        a3 = fmaf(S[4 * m + 3], qq[4 * m + 3], a3);
      }
      out = (a0 + a1) + (a2 + a3);
    };
    for (int t0 = 0; t0 < n; t0 += LS_TB) {
      float acc[LS_TB];
      if (WALK && t0 + LS_TB <= n) {     // eight whole tokens: nothing to test between them, so the next one's loads start early
#pragma unroll
        for (int tl = 0; tl < LS_TB; ++tl) token(t0 + tl, acc[tl]);
      } else {
#pragma unroll
        for (int tl = 0; tl < LS_TB; ++tl) {
          acc[tl] = 0.f;
          if (t0 + tl < n) token(t0 + tl, acc[tl]);      // the same for the whole block
        }
      }
      ls_halve<4, 4>(acc, lane);
      ls_halve<2, 2>(acc, lane);
      ls_halve<1, 1>(acc, lane);
      // lane l of a column now holds token t0 + l
      if (t0 + lane < n) so[(t0 + lane) * COLS + col] = acc[0];
    }
  }
  __syncthreads();
  write_out(n_chunks - 1, sm + ((n_chunks - 1) & 1) * BUF, 0, NC + LS_PREP);
  if (!prep && j < V) {
#pragma unroll
    for (int m = 0; m < M; ++m) {
      const int i = 4 * (lane + LS_LANES * m);
      if (a.vec_state && i < K) {
        *reinterpret_cast<float4*>(S_row + (size_t)j * K + i) = make_float4(S[4 * m], S[4 * m + 1], S[4 * m + 2], S[4 * m + 3]);
      } else {
#pragma unroll
        for (int e = 0; e < 4; ++e)
          if (i + e < K) S_row[(size_t)j * K + i + e] = S[4 * m + e];
      }
    }
  }
}

int ls_sm_count() {
  static int n[gi::MAX_DEVICES_SEEN] = {};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= gi::MAX_DEVICES_SEEN) return 148;
  if (n[dev] == 0 && cudaDeviceGetAttribute(&n[dev], cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) n[dev] = 148;
  return n[dev];
}

template <typename T, int KR, int COLS>
cudaError_t ls_launch(const LsArgs& a, int n_seqs, bool delta, bool walk, cudaStream_t stream) {
  constexpr int CH = LsChunk<KR>::value;
  const size_t smem = 2 * (size_t)(2 * CH * KR * LS_LANES + 2 * CH * COLS + 2 * CH) * sizeof(float);
  const dim3 grid(a.heads, n_seqs, (a.V + COLS - 1) / COLS), block(COLS * LS_LANES + LS_PREP);
  if (walk)
    return delta ? gi::launch(linear_state_kernel<T, KR, COLS, true, true>, grid, block, smem, stream, a)
                 : gi::launch(linear_state_kernel<T, KR, COLS, false, true>, grid, block, smem, stream, a);
  return delta ? gi::launch(linear_state_kernel<T, KR, COLS, true, false>, grid, block, smem, stream, a)
               : gi::launch(linear_state_kernel<T, KR, COLS, false, false>, grid, block, smem, stream, a);
}

template <typename T, int KR>
cudaError_t ls_pick_tile(const LsArgs& a, int n_seqs, bool delta, bool walk, cudaStream_t stream) {
  // the widest tile that still gives every SM a block: with fewer blocks than SMs the token-by-token walk, whose length a
  // block cannot shorten, runs on a part of the device only
  const long per = (long)a.heads * n_seqs, sms = ls_sm_count();
  if (per * ((a.V + 31) / 32) >= sms || a.V <= 8) return ls_launch<T, KR, 32>(a, n_seqs, delta, walk, stream);
  if (per * ((a.V + 15) / 16) >= sms) return ls_launch<T, KR, 16>(a, n_seqs, delta, walk, stream);
  return ls_launch<T, KR, 8>(a, n_seqs, delta, walk, stream);
}

}  // namespace

extern "C" int gi_linear_state(float* o, const void* q, long ldq, const void* k, long ldk, const void* v, long ldv,
                               const void* a_in, long lda, const void* b_in, long ldb, int dtype, const float* decay_c,
                               const float* dt_bias, float* state, long state_ld, int state_rows, const int* cu_seqlens,
                               const int* seq_slots, int n_seqs, int heads, int qk_heads, int K, int V, int in_act,
                               int unit_norm, float norm_eps, float q_scale, int delta, int n_tokens, void* stream) {
  return gi_linear_state_gated(o, q, ldq, k, ldk, v, ldv, a_in, lda, b_in, ldb, dtype, decay_c, dt_bias, nullptr, nullptr, state,
                               state_ld, state_rows, cu_seqlens, seq_slots, n_seqs, heads, qk_heads, K, V, in_act, unit_norm,
                               norm_eps, q_scale, delta, n_tokens, stream);
}

extern "C" int gi_linear_state_gated(float* o, const void* q, long ldq, const void* k, long ldk, const void* v, long ldv,
                                     const void* a_in, long lda, const void* b_in, long ldb, int dtype, const float* decay_c,
                                     const float* dt_bias, const float* g_direct, const float* u_direct, float* state,
                                     long state_ld, int state_rows, const int* cu_seqlens, const int* seq_slots, int n_seqs,
                                     int heads, int qk_heads, int K, int V, int in_act, int unit_norm, float norm_eps,
                                     float q_scale, int delta, int n_tokens, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (heads <= 0 || qk_heads <= 0 || heads % qk_heads || K <= 0 || V <= 0)
    return gi::fail(GI_ERR_ARG, "linear_state: bad sizes (heads %d, query/key heads %d, keys %d, values %d)", heads, qk_heads, K, V);
  if (K > 32 * LS_LANES) return gi::fail(GI_ERR_UNSUPPORTED, "linear_state: keys of %d numbers (at most %d)", K, 32 * LS_LANES);
  if (!o || !q || !k || !v || (!decay_c && !g_direct) || !state || !cu_seqlens || !seq_slots) return gi::fail(GI_ERR_ARG, "linear_state: a missing pointer");
  if (u_direct != nullptr && delta) return gi::fail(GI_ERR_ARG, "linear_state: ready-made write strengths do not go with the delta rule");
  if (delta && b_in == nullptr) return gi::fail(GI_ERR_ARG, "linear_state: the delta rule needs its write strengths");
  if (state_ld < (long)heads * K * V) return gi::fail(GI_ERR_ARG, "linear_state: state rows of %ld floats, wanted %ld", state_ld, (long)heads * K * V);
  LsArgs a;
  a.o = o; a.q = q; a.k = k; a.v = v; a.a_in = a_in; a.b_in = b_in;
  a.ldq = ldq; a.ldk = ldk; a.ldv = ldv; a.lda = lda; a.ldb = ldb;
  a.decay_c = decay_c; a.dt_bias = dt_bias; a.g_direct = g_direct; a.u_direct = u_direct; a.state = state; a.state_ld = state_ld; a.state_rows = state_rows;
  a.cu_seqlens = cu_seqlens; a.seq_slots = seq_slots;
  a.heads = heads; a.qk_heads = qk_heads; a.K = K; a.V = V; a.in_act = in_act; a.unit_norm = unit_norm;
  // sixteen bytes of a column at a time where every column of every slot starts on such a boundary
  a.vec_state = (K % 4 == 0 && state_ld % 4 == 0 && ((size_t)state & 15) == 0) ? 1 : 0;
  a.norm_eps = norm_eps; a.q_scale = q_scale;
  {
    // sixteen bytes of a row at a time where every piece a block reads starts on such a boundary
    const int vw = dtype == GI_BF16 ? 8 : 4;
    const size_t esz = dtype == GI_BF16 ? 2 : 4;
    a.vec_in = (K % vw == 0 && V % vw == 0 && ldq % vw == 0 && ldk % vw == 0 && ldv % vw == 0 &&
                (((uintptr_t)q | (uintptr_t)k | (uintptr_t)v) & 15) == 0 && esz * vw == 16) ? 1 : 0;
  }
  // more tokens than sequences: some sequence brings several, the step is a prompt step (n_tokens 0: not known)
  const bool walk = n_tokens <= 0 || n_tokens > n_seqs;
  cudaError_t e = cudaSuccess;
  GI_DISPATCH_DTYPE(dtype, T, {
    if (K <= 4 * LS_LANES) e = ls_pick_tile<T, 4>(a, n_seqs, delta != 0, walk, (cudaStream_t)stream);
    else if (K <= 8 * LS_LANES) e = ls_pick_tile<T, 8>(a, n_seqs, delta != 0, walk, (cudaStream_t)stream);
    else if (K <= 16 * LS_LANES) e = ls_pick_tile<T, 16>(a, n_seqs, delta != 0, walk, (cudaStream_t)stream);
    else e = ls_pick_tile<T, 32>(a, n_seqs, delta != 0, walk, (cudaStream_t)stream);
  });
  return gi::check(e, "linear_state");
}
