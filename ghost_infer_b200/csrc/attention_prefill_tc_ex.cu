// The tensor-core prompt attention (see attention_prefill_tc.cu: 64 queries of one head per block, four warps of 16
// rows, key tiles of one page through cp.async into swizzled shared memory, m16n8k16 products, a running softmax in
// base 2 with 32-bit statistics) with what some designs add to attention, each off at its neutral value:
//  * keys and values of different widths (hd, hdv: any multiples of 8 up to 128; tiles are padded with zero columns to
//    64 or 128, which add nothing to a product);
//  * a cap on the scores, s <- cap * tanh(s / cap), in 32-bit (tanh through the approximate exponential: see gi::tanh_fast);
//  * a sink per head: one more term exp(sink) in the denominator, with no key and no value;
//  * chunks: a query sees the keys of its own chunk floor(pos / chunk) only, counted from position 0.
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int BQ = 64;     // queries per block
constexpr int BKV = 64;    // keys per tile = one page
constexpr int WARPS = 4;

template <int HD, int HDV>
__global__ void __launch_bounds__(WARPS * 32)
attn_prefill_tcx_kernel(__nv_bfloat16* __restrict__ out, long ldo, const __nv_bfloat16* __restrict__ q, long ldq,
                       const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                       const int* __restrict__ block_table, int max_pages, const int* __restrict__ cu_seqlens,
                       const int* __restrict__ seq_slots, const int* __restrict__ seq_pos0, int n_heads, int n_kv,
                       float scale, int window, int q_tiles, int hd, int hdv, float softcap, const float* __restrict__ sinks,
                       int chunk, int keep_first) {
  constexpr int CH = HD / 8, CHV = HDV / 8;
  constexpr int TILE_BYTES = BKV * HD * 2, VTILE_BYTES = BKV * HDV * 2;
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                         // [BQ][HD]
  unsigned char* kv_s = smem + BQ * HD * 2;          // [2 stages][K tile | V tile]
  constexpr int STAGE_BYTES = TILE_BYTES + VTILE_BYTES;

  const int b = blockIdx.z, h = blockIdx.y;
  const int tok0 = cu_seqlens[b], qlen = cu_seqlens[b + 1] - tok0;
  const int q0 = (q_tiles - 1 - (int)blockIdx.x) * BQ;          // latest tiles first
  if (q0 >= qlen) return;
  const int slot = seq_slots[b], pos0 = seq_pos0[b];
  const int kvh = h / (n_heads / n_kv);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;
  const int rows_here = min(BQ, qlen - q0);
  const int p_last = pos0 + q0 + rows_here - 1;                 // the block's last position
  int t_first = 0;                                              // the first key any row here may see
  if (window > 0) t_first = max(0, pos0 + q0 - window + 1);
  if (chunk > 0) t_first = max(t_first, ((pos0 + q0) / chunk) * chunk);
  const int kt_begin = (t_first / BKV) * BKV;
  // a window may keep the sequence's first `keep_first` positions visible: their tiles come before the window's own
  const int kept = window > 0 ? keep_first : 0;
  const int kept_tiles = min((kept + BKV - 1) / BKV, kt_begin / BKV);
  const int n_tiles = kept_tiles + (p_last - kt_begin) / BKV + 1;

  auto issue_kv = [&](int tile, int stage) {
    const int kt = tile < kept_tiles ? tile * BKV : kt_begin + (tile - kept_tiles) * BKV;
    const int page = block_table[(size_t)slot * max_pages + kt / PAGE_TOKENS];
    const size_t row0 = ((size_t)page * n_kv + kvh) * PAGE_TOKENS;
    unsigned char* ks = kv_s + (size_t)stage * STAGE_BYTES;
    unsigned char* vs = ks + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < BKV * CH / (WARPS * 32); ++i) {
      const int idx = i * WARPS * 32 + tid;
      const int r = idx / CH, c = idx % CH;
      // rows nobody here sees and the padding columns: zeros, not read
      const int ok = (kt + r <= p_last && (kt + r >= t_first || kt + r < kept) && c * 8 < hd) ? 16 : 0;
      gi::cp_async_16(gi::smem_u32(ks + gi::swz<CH>(r, c)), kcache + (row0 + (ok ? r : 0)) * hd + (ok ? c * 8 : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < BKV * CHV / (WARPS * 32); ++i) {
      const int idx = i * WARPS * 32 + tid;
      const int r = idx / CHV, c = idx % CHV;
      const int ok = (kt + r <= p_last && (kt + r >= t_first || kt + r < kept) && c * 8 < hdv) ? 16 : 0;
      gi::cp_async_16(gi::smem_u32(vs + gi::swz<CHV>(r, c)), vcache + (row0 + (ok ? r : 0)) * hdv + (ok ? c * 8 : 0), ok);
    }
  };

  // queries of this block (rows past the sequence's end: zeros) and the first key tile
#pragma unroll
  for (int i = 0; i < BQ * CH / (WARPS * 32); ++i) {
    const int idx = i * WARPS * 32 + tid;
    const int r = idx / CH, c = idx % CH;
    const int ok = (r < rows_here && c * 8 < hd) ? 16 : 0;
    gi::cp_async_16(gi::smem_u32(q_s + gi::swz<CH>(r, c)), q + (size_t)(tok0 + q0 + (ok ? r : 0)) * ldq + (size_t)h * hd + (ok ? c * 8 : 0), ok);
  }
  issue_kv(0, 0);
  gi::cp_async_commit();

  const int p_row0 = pos0 + q0 + warp * 16 + g;       // position of this thread's first row; the second is 8 further
  const int p_warp_last = pos0 + q0 + warp * 16 + 15;
  const float sl2 = scale * 1.4426950408889634f;
  const float cap_in = softcap > 0.f ? scale / softcap : 0.f, cap_out = softcap * 1.4426950408889634f;
  // the first key of each of this thread's two rows' chunks, and of the warp's first row's
  int c_lo[2] = {0, 0};
  int c_lo_warp = 0;
  if (chunk > 0) {
    c_lo[0] = (p_row0 / chunk) * chunk;
    c_lo[1] = ((p_row0 + 8) / chunk) * chunk;
    c_lo_warp = ((pos0 + q0 + warp * 16) / chunk) * chunk;
  }
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[HDV / 8][4];
#pragma unroll
  for (int i = 0; i < HDV / 8; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;
  uint32_t qf[HD / 16][4];

  for (int tile = 0; tile < n_tiles; ++tile) {
    const int stage = tile & 1;
    if (tile + 1 < n_tiles) issue_kv(tile + 1, stage ^ 1);
    gi::cp_async_commit();
    gi::cp_async_wait<1>();
    __syncthreads();
    if (tile == 0) {
#pragma unroll
      for (int ks = 0; ks < HD / 16; ++ks) {
        const int r = warp * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = ks * 2 + (lane >> 4);
        gi::ldmatrix_x4(qf[ks], gi::smem_u32(q_s + gi::swz<CH>(r, c)));
      }
    }
    const int kt = tile < kept_tiles ? tile * BKV : kt_begin + (tile - kept_tiles) * BKV;
    const unsigned char* ks_ = kv_s + (size_t)stage * STAGE_BYTES;
    const unsigned char* vs_ = ks_ + TILE_BYTES;
    // a warp whose rows all lie before this tile, or whose windows all ended before it, has nothing to do here
    const bool active = kt <= p_warp_last && (window <= 0 || kt + BKV - 1 > p_warp_last - 15 - window || kt < kept) && kt + BKV - 1 >= c_lo_warp;
    if (active) {
      float s[BKV / 8][4];
#pragma unroll
      for (int nt = 0; nt < BKV / 8; ++nt) {
#pragma unroll
        for (int c = 0; c < 4; ++c) s[nt][c] = 0.f;
#pragma unroll
        for (int kp = 0; kp < HD / 32; ++kp) {
          uint32_t kb[4];
          const int r = nt * 8 + (lane & 7), c = kp * 4 + (lane >> 3);
          gi::ldmatrix_x4(kb, gi::smem_u32(ks_ + gi::swz<CH>(r, c)));
          gi::mma_16816(s[nt], qf[kp * 2], kb[0], kb[1]);
          gi::mma_16816(s[nt], qf[kp * 2 + 1], kb[2], kb[3]);
        }
      }
      float tmax[2] = {-INFINITY, -INFINITY};
#pragma unroll
      for (int nt = 0; nt < BKV / 8; ++nt)
#pragma unroll
        for (int c = 0; c < 4; ++c) {
          const int key = kt + nt * 8 + 2 * t + (c & 1);
          const int p = p_row0 + (c >> 1) * 8;
          const bool ok = key <= p && p <= p_last && (window <= 0 || key > p - window || key < kept) && key >= c_lo[c >> 1];
          const float sc = softcap > 0.f ? cap_out * gi::tanh_fast(s[nt][c] * cap_in) : s[nt][c] * sl2;
          s[nt][c] = ok ? sc : -INFINITY;
          tmax[c >> 1] = fmaxf(tmax[c >> 1], s[nt][c]);
        }
      float alpha[2], m_use[2];
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 1));
        tmax[hh] = fmaxf(tmax[hh], __shfl_xor_sync(0xffffffffu, tmax[hh], 2));
        const float m_new = fmaxf(m_run[hh], tmax[hh]);
        alpha[hh] = (m_run[hh] == -INFINITY) ? 0.f : exp2f(m_run[hh] - m_new);   // m_new >= m_run, both finite here
        m_run[hh] = m_new;
        m_use[hh] = (m_new == -INFINITY) ? 0.f : m_new;     // a row that has seen no key yet: every p below is 0
      }
      float psum[2] = {0.f, 0.f};
      uint32_t pf[BKV / 16][4];
#pragma unroll
      for (int nt = 0; nt < BKV / 8; ++nt) {
        const float p0 = exp2f(s[nt][0] - m_use[0]), p1 = exp2f(s[nt][1] - m_use[0]);
        const float p2 = exp2f(s[nt][2] - m_use[1]), p3 = exp2f(s[nt][3] - m_use[1]);
        psum[0] += p0 + p1;
        psum[1] += p2 + p3;
        pf[nt / 2][(nt & 1) * 2] = gi::pack_bf16(p0, p1);
        pf[nt / 2][(nt & 1) * 2 + 1] = gi::pack_bf16(p2, p3);
      }
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 1);
        psum[hh] += __shfl_xor_sync(0xffffffffu, psum[hh], 2);
        l_run[hh] = l_run[hh] * alpha[hh] + psum[hh];
      }
#pragma unroll
      for (int i = 0; i < HDV / 8; ++i) {
        o[i][0] *= alpha[0];
        o[i][1] *= alpha[0];
        o[i][2] *= alpha[1];
        o[i][3] *= alpha[1];
      }
#pragma unroll
      for (int kk = 0; kk < BKV / 16; ++kk) {
#pragma unroll
        for (int dp = 0; dp < HDV / 16; ++dp) {
          uint32_t vb[4];
          const int r = kk * 16 + (lane & 7) + ((lane >> 3) & 1) * 8, c = dp * 2 + (lane >> 4);
          gi::ldmatrix_x4_trans(vb, gi::smem_u32(vs_ + gi::swz<CHV>(r, c)));
          gi::mma_16816(o[dp * 2], pf[kk], vb[0], vb[1]);
          gi::mma_16816(o[dp * 2 + 1], pf[kk], vb[2], vb[3]);
        }
      }
    }
    __syncthreads();     // everyone is done with this stage before the next iteration refills it
  }

#pragma unroll
  for (int hh = 0; hh < 2; ++hh) {
    const int row = warp * 16 + g + hh * 8;
    if (row >= rows_here) continue;
    float a = 1.f;
    if (sinks != nullptr) {
      // the sink: one more term of the denominator (statistics are in base 2), with no value behind it
      const float sk = sinks[h] * 1.4426950408889634f;
      const float m_f = fmaxf(m_run[hh], sk);
      a = (m_run[hh] == -INFINITY) ? 0.f : exp2f(m_run[hh] - m_f);
      l_run[hh] = l_run[hh] * a + exp2f(sk - m_f);
    }
    const float inv = l_run[hh] > 0.f ? a / l_run[hh] : 0.f;
    __nv_bfloat16* orow = out + (size_t)(tok0 + q0 + row) * ldo + (size_t)h * hdv;
#pragma unroll
    for (int i = 0; i < HDV / 8; ++i) {
      if (i * 8 + 2 * t >= hdv) continue;
      __nv_bfloat162 v = __floats2bfloat162_rn(o[i][hh * 2] * inv, o[i][hh * 2 + 1] * inv);
      *reinterpret_cast<__nv_bfloat162*>(orow + i * 8 + 2 * t) = v;
    }
  }
}

template <int HD, int HDV>
int launch(dim3 grid, cudaStream_t s, __nv_bfloat16* out, long ldo, const __nv_bfloat16* q, long ldq, const __nv_bfloat16* kc,
           const __nv_bfloat16* vc, const int* bt, int max_pages, const int* cu, const int* slots, const int* pos0, int H, int KV,
           float scale, int window, int q_tiles, int hd, int hdv, float softcap, const float* sinks, int chunk, int keep_first) {
  constexpr size_t smem = (size_t)BQ * HD * 2 + 2 * ((size_t)BKV * HD * 2 + (size_t)BKV * HDV * 2);
  auto kern = attn_prefill_tcx_kernel<HD, HDV>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention prefill: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  kern<<<grid, WARPS * 32, smem, s>>>(out, ldo, q, ldq, kc, vc, bt, max_pages, cu, slots, pos0, H, KV, scale, window, q_tiles, hd, hdv,
                                      softcap, sinks, chunk, keep_first);
  return gi::check_launch("attention prefill (tensor cores, general)");
}

}  // namespace

extern "C" int gi_attn_prefill_tc_ex(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                                     const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                                     const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd,
                                     float scale, int window, int hdv, float softcap, const float* sinks, int chunk,
                                     void* stream) {
  return gi_attn_prefill_tc_ex2(out, ldo, q, ldq, kcache, vcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, n_seqs,
                                max_q_len, n_heads, n_kv, hd, scale, window, hdv, softcap, sinks, chunk, 0, stream);
}

// The same with a window that keeps the sequence's first `keep_first` positions visible as well.
extern "C" int gi_attn_prefill_tc_ex2(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                                      const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                                      const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd,
                                      float scale, int window, int hdv, float softcap, const float* sinks, int chunk,
                                      int keep_first, void* stream) {
  if (n_seqs <= 0 || max_q_len <= 0) return GI_OK;
  if (keep_first < 0 || (keep_first > 0 && chunk > 0)) return gi::fail(GI_ERR_ARG, "attention: kept first positions go with a window, not with chunks");
  if (hd <= 0 || hd > 128 || hd % 8 || hdv <= 0 || hdv > 128 || hdv % 8)
    return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tensor cores): key size %d, value size %d; multiples of 8 up to 128", hd, hdv);
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (chunk < 0 || softcap < 0.f) return gi::fail(GI_ERR_ARG, "attention: a chunk or a cap cannot be negative");
  if (ldq % 8 != 0 || ldo % 2 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15) || ((uintptr_t)out & 3))
    return gi::fail(GI_ERR_UNSUPPORTED, "attention prefill (tensor cores): queries and cache must be 16-byte aligned");
  if (n_seqs > 65535 || n_heads > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or heads in one launch");
  const int q_tiles = (max_q_len + BQ - 1) / BQ;
  dim3 grid(q_tiles, n_heads, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
#define GI_TCX(HDP, HDVP)                                                                                                  \
  return launch<HDP, HDVP>(grid, s, (__nv_bfloat16*)out, ldo, (const __nv_bfloat16*)q, ldq, (const __nv_bfloat16*)kcache,   \
                           (const __nv_bfloat16*)vcache, block_table, max_pages, cu_seqlens, seq_slots, seq_pos0, n_heads,  \
                           n_kv, scale, window, q_tiles, hd, hdv, softcap, sinks, chunk, keep_first)
  if (hd <= 64 && hdv <= 64) GI_TCX(64, 64);
  if (hd <= 64) GI_TCX(64, 128);
  if (hdv <= 64) GI_TCX(128, 64);
  GI_TCX(128, 128);
#undef GI_TCX
}
