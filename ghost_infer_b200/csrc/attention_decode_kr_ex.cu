// The decode attention with the keys on the rows of the tensor-core tile (see attention_decode_kr.cu: a tile of 16 keys is
// the rows of an m16n8k16 product and up to 8 heads of a group its columns; per-warp cp.async rings; slices merged by
// gi_attn_combine) with what some designs add to attention, each off at its neutral value:
//  * keys and values of different widths (hd, hdv: any multiples of 8 up to 128; tiles are padded with zero columns to
//    64 or 128, which add nothing to a product);
//  * a cap on the scores, s <- cap * tanh(s / cap), in 32-bit (tanh through the approximate exponential: see gi::tanh_fast);
//  * a sink per head: one more term exp(sink) in the denominator, with no key and no value (the first slice takes it in);
//  * chunks: the token sees the keys of its own chunk floor(pos / chunk) only, counted from position 0.
#include <math.h>

#include "api.h"
#include "common.cuh"
#include "mma_utils.cuh"

namespace {

constexpr int KT = 16;       // keys per tile
constexpr int COLS = 8;      // heads per block: the columns of the tile

__device__ __forceinline__ uint32_t movmatrix_trans(uint32_t a) {
  uint32_t d;
  asm volatile("movmatrix.sync.aligned.m8n8.trans.b16 %0, %1;" : "=r"(d) : "r"(a));
  return d;
}

template <int HD, int HDV, int WARPS, int STAGES>
__global__ void __launch_bounds__(WARPS * 32)
attn_decode_krx_kernel(__nv_bfloat16* __restrict__ out, long ldo, float* __restrict__ part_o, float* __restrict__ part_ml,
                      const __nv_bfloat16* q /* written by the kernel before: see gi::pdl_wait */, long ldq,
                      const __nv_bfloat16* __restrict__ kcache, const __nv_bfloat16* __restrict__ vcache,
                      const int* __restrict__ block_table, int max_pages, const int* __restrict__ seq_slots,
                      const int* __restrict__ seq_lens, int n_heads, int n_kv, float scale, int window, int n_splits,
                      int own_tiles, int hd, int hdv, float softcap, const float* __restrict__ sinks, int pos_chunk, int keep_first) {
  constexpr int CH = HD / 8, CHV = HDV / 8;      // 16-byte chunks per row
  constexpr int TILE_BYTES = KT * HD * 2;        // one K tile
  constexpr int VTILE_BYTES = KT * HDV * 2;      // one V tile
  constexpr int STAGE_BYTES = TILE_BYTES + VTILE_BYTES;    // K then V
  constexpr int MT = HD / 16;                    // 16-dim steps of S^T
  constexpr int MTV = HDV / 16;                  // 16-dim row tiles of O^T
  extern __shared__ __align__(128) unsigned char smem[];
  unsigned char* q_s = smem;                                       // [8][HD] bf16, swizzled
  unsigned char* ring = smem + COLS * HD * 2;                      // [WARPS][STAGES][K tile | V tile]
  // Lengths, slots and the block table were uploaded before the step's first kernel, and no kernel of the step
  // writes a cached position other than each sequence's last one: the first tiles are requested before the
  // dependency wait; only the tile that holds the last position waits.
  gi::pdl_launch_dependents();

  const int group = n_heads / n_kv;
  const int chunks = (group + COLS - 1) / COLS;
  const int b = blockIdx.z, kvh = blockIdx.y / chunks, chunk = blockIdx.y % chunks, sp = blockIdx.x;
  const int g0 = chunk * COLS, gcount = min(COLS, group - g0);
  const int h0 = kvh * group + g0;
  const int slot = gi::ld_step(seq_slots + b);
  const int len = gi::ld_step(seq_lens + b);
  const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
  const int g = lane >> 2, t = lane & 3;

  int t_first = 0;
  if (window > 0) t_first = max(0, len - window);
  if (pos_chunk > 0) t_first = max(t_first, ((len - 1) / pos_chunk) * pos_chunk);
  const int t_base = (t_first / KT) * KT;
  // a window may keep the sequence's first `keep_first` positions visible: their tiles are counted before the window's own
  const int kept = window > 0 ? keep_first : 0;
  const int kept_tiles = min((kept + KT - 1) / KT, t_base / KT);
  const int tiles = kept_tiles + (len > t_base ? (len - t_base + KT - 1) / KT : 0);
  const int per = own_tiles > 0 ? own_tiles : (tiles + n_splits - 1) / n_splits;
  const int used = per > 0 ? max(1, (tiles + per - 1) / per) : 1;      // slices of this sequence that hold keys
  const int tile_lo = sp * per, tile_hi = min(tiles, tile_lo + per);
  if (sp >= used) {
    // nothing of this sequence lies in this slice: the combine kernel must find it marked empty
    if (n_splits > 1) {
      for (int r = threadIdx.x; r < gcount; r += WARPS * 32) {
        const size_t pi = ((size_t)b * n_heads + h0 + r) * n_splits + sp;
        part_ml[pi * 2] = -INFINITY;
        part_ml[pi * 2 + 1] = 0.f;
      }
    }
    return;
  }

  unsigned char* my_ring = ring + (size_t)warp * STAGES * STAGE_BYTES;
  const float sl2 = scale * 1.4426950408889634f;
  const float cap_in = softcap > 0.f ? scale / softcap : 0.f, cap_out = softcap * 1.4426950408889634f;

  auto issue = [&](int tile, int stage) {
    const int t0 = tile < kept_tiles ? tile * KT : t_base + (tile - kept_tiles) * KT;
    const int page = slot >= 0 ? gi::ld_step(block_table + (size_t)slot * max_pages + t0 / PAGE_TOKENS) : 0;
    const size_t row0 = ((size_t)page * n_kv + kvh) * PAGE_TOKENS + (t0 % PAGE_TOKENS);
    unsigned char* ks = my_ring + (size_t)stage * STAGE_BYTES;
    unsigned char* vs = ks + TILE_BYTES;
#pragma unroll
    for (int i = 0; i < KT * CH / 32; ++i) {
      const int idx = i * 32 + lane;
      const int r = idx / CH, c = idx % CH;
      // rows outside the visible span and the padding columns are zero-filled, not read
      const int ok = (t0 + r < len && (t0 + r >= t_first || t0 + r < kept) && c * 8 < hd) ? 16 : 0;
      gi::cp_async_16(gi::smem_u32(ks + gi::swz<CH>(r, c)), kcache + (row0 + (ok ? r : 0)) * hd + (ok ? c * 8 : 0), ok);
    }
#pragma unroll
    for (int i = 0; i < KT * CHV / 32; ++i) {
      const int idx = i * 32 + lane;
      const int r = idx / CHV, c = idx % CHV;
      const int ok = (t0 + r < len && (t0 + r >= t_first || t0 + r < kept) && c * 8 < hdv) ? 16 : 0;
      gi::cp_async_16(gi::smem_u32(vs + gi::swz<CHV>(r, c)), vcache + (row0 + (ok ? r : 0)) * hdv + (ok ? c * 8 : 0), ok);
    }
  };

  // per thread: heads 2t and 2t + 1 (index j), keys g and g + 8 of a tile
  float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.f, 0.f};
  float o[MTV][4];                     // O^T: [0], [1] dim 16 mt + g of heads 2t, 2t + 1; [2], [3] dim 16 mt + g + 8
#pragma unroll
  for (int i = 0; i < MTV; ++i)
#pragma unroll
    for (int c = 0; c < 4; ++c) o[i][c] = 0.f;

  // prologue: STAGES - 1 tiles in flight; the tile with the sequence's last position only after the wait
  int next = tile_lo + warp;
  int late_stage = -1;
#pragma unroll
  for (int s = 0; s < STAGES - 1; ++s) {
    if (next < tile_hi) {
      if (next == tiles - 1) late_stage = s;
      else issue(next, s);
    }
    gi::cp_async_commit();
    next += WARPS;
  }
  gi::pdl_wait();
  if (late_stage >= 0) {          // a short slice: its last tile is among the first ones; fetch it now and let it land
    issue(tiles - 1, late_stage);
    gi::cp_async_commit();
    gi::cp_async_wait<0>();
  }
  // queries of the block's heads as rows 0..gcount-1 of an 8-row tile (the others zero)
  for (int idx = tid; idx < COLS * CH; idx += WARPS * 32) {
    const int r = idx / CH, c = idx % CH;
    uint4 v = make_uint4(0, 0, 0, 0);
    if (r < gcount && c * 8 < hd) v = *reinterpret_cast<const uint4*>(q + (size_t)b * ldq + (size_t)(h0 + r) * hd + c * 8);
    *reinterpret_cast<uint4*>(q_s + gi::swz<CH>(r, c)) = v;
  }
  __syncthreads();
  // Q^T as the second operand: for 32 dims at a time, four 8x8 matrices (heads 0-7, dims +0, +8, +16, +24)
  uint32_t qb[HD / 32][4];
#pragma unroll
  for (int kp = 0; kp < HD / 32; ++kp) gi::ldmatrix_x4(qb[kp], gi::smem_u32(q_s + gi::swz<CH>(lane & 7, kp * 4 + (lane >> 3))));

  int stage = 0;
  for (int tile = tile_lo + warp; tile < tile_hi; tile += WARPS) {
    // keep the ring full, then wait for the oldest tile
    if (next < tile_hi) issue(next, (stage + STAGES - 1) % STAGES);
    gi::cp_async_commit();
    next += WARPS;
    gi::cp_async_wait<STAGES - 1>();
    __syncwarp();
    const unsigned char* ks = my_ring + (size_t)stage * STAGE_BYTES;
    const unsigned char* vs = ks + TILE_BYTES;
    const int t0 = tile < kept_tiles ? tile * KT : t_base + (tile - kept_tiles) * KT;

    // S^T = K Q^T: rows are the tile's 16 keys
    float s[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int kk = 0; kk < MT; ++kk) {
      // matrices: (keys 0-7, dims lo), (keys 8-15, dims lo), (keys 0-7, dims hi), (keys 8-15, dims hi)
      uint32_t ka[4];
      gi::ldmatrix_x4(ka, gi::smem_u32(ks + gi::swz<CH>((lane & 7) + ((lane >> 3) & 1) * 8, kk * 2 + (lane >> 4))));
      gi::mma_16816(s, ka, qb[kk >> 1][(kk & 1) * 2], qb[kk >> 1][(kk & 1) * 2 + 1]);
    }
    // mask (two keys per thread) and running softmax (two heads per thread)
    const bool ok0 = t0 + g < len && (t0 + g >= t_first || t0 + g < kept), ok1 = t0 + g + 8 < len && (t0 + g + 8 >= t_first || t0 + g + 8 < kept);
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const float sc = softcap > 0.f ? cap_out * gi::tanh_fast(s[c] * cap_in) : s[c] * sl2;
      s[c] = ((c < 2) ? ok0 : ok1) ? sc : -INFINITY;
    }
    float alpha[2];
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      float tmax = fmaxf(s[j], s[2 + j]);
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 4));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 8));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 16));
      const float m_new = fmaxf(m_run[j], tmax);          // finite: every tile holds at least one live key
      alpha[j] = (m_run[j] == -INFINITY) ? 0.f : exp2f(m_run[j] - m_new);
      m_run[j] = m_new;
    }
    const float p0 = exp2f(s[0] - m_run[0]), p1 = exp2f(s[1] - m_run[1]);
    const float p2 = exp2f(s[2] - m_run[0]), p3 = exp2f(s[3] - m_run[1]);
    l_run[0] = l_run[0] * alpha[0] + (p0 + p2);           // this thread's keys only; lanes are added at the end
    l_run[1] = l_run[1] * alpha[1] + (p1 + p3);
    // P^T from (key g, heads 2t, 2t + 1) to (keys 2t, 2t + 1, head g)
    const uint32_t pb0 = movmatrix_trans(gi::pack_bf16(p0, p1)), pb1 = movmatrix_trans(gi::pack_bf16(p2, p3));
#pragma unroll
    for (int i = 0; i < MTV; ++i) {
      o[i][0] *= alpha[0];
      o[i][1] *= alpha[1];
      o[i][2] *= alpha[0];
      o[i][3] *= alpha[1];
    }
    // O^T += V^T P^T: rows are 16 dims of the head
#pragma unroll
    for (int mt = 0; mt < MTV; ++mt) {
      // transposed matrices: (keys 0-7, dims lo), (keys 0-7, dims hi), (keys 8-15, dims lo), (keys 8-15, dims hi)
      uint32_t va[4];
      gi::ldmatrix_x4_trans(va, gi::smem_u32(vs + gi::swz<CHV>((lane & 7) + (lane >> 4) * 8, mt * 2 + ((lane >> 3) & 1))));
      gi::mma_16816(o[mt], va, pb0, pb1);
    }
    __syncwarp();
    stage = (stage + 1) % STAGES;
  }
  gi::cp_async_wait<0>();
  // the sums over this warp's keys: lanes of equal t hold the same two heads
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 4);
    l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 8);
    l_run[j] += __shfl_xor_sync(0xffffffffu, l_run[j], 16);
  }
  __syncthreads();

  // merge the warps (reusing the ring): natural-log maxima so that the combine kernel can go on
  constexpr int MROW = HDV + 8;
  float* Mo = reinterpret_cast<float*>(ring);            // [WARPS][8][MROW]
  float* Mm = Mo + WARPS * COLS * MROW;                  // [WARPS][8]
  float* Ml = Mm + WARPS * COLS;                         // [WARPS][8]
#pragma unroll
  for (int j = 0; j < 2; ++j) {
    const int r = 2 * t + j;
    if (r >= gcount) continue;
    if (g == 0) {
      Mm[warp * COLS + r] = m_run[j];
      Ml[warp * COLS + r] = l_run[j];
    }
#pragma unroll
    for (int i = 0; i < MTV; ++i) {
      Mo[(warp * COLS + r) * MROW + i * 16 + g] = o[i][j];
      Mo[(warp * COLS + r) * MROW + i * 16 + g + 8] = o[i][2 + j];
    }
  }
  __syncthreads();
  for (int idx = tid; idx < gcount * hdv; idx += WARPS * 32) {
    const int r = idx / hdv, d = idx % hdv;
    float mm = -INFINITY;
#pragma unroll
    for (int w = 0; w < WARPS; ++w) mm = fmaxf(mm, Mm[w * COLS + r]);
    float tot = 0.f, val = 0.f;
    if (mm != -INFINITY) {
#pragma unroll
      for (int w = 0; w < WARPS; ++w) {
        const float mw = Mm[w * COLS + r];
        if (mw == -INFINITY) continue;
        const float wgt = exp2f(mw - mm);
        tot += Ml[w * COLS + r] * wgt;
        val += Mo[(w * COLS + r) * MROW + d] * wgt;
      }
    }
    const int h = h0 + r;
    if (sinks != nullptr && sp == 0) {
      // the sink counts once per (sequence, head): the first slice takes it in (statistics are in base 2 here)
      const float sk = sinks[h] * 1.4426950408889634f;
      const float m_f = fmaxf(mm, sk);
      const float a = (mm == -INFINITY) ? 0.f : exp2f(mm - m_f);
      tot = tot * a + exp2f(sk - m_f);
      val *= a;
      mm = m_f;
    }
    if (n_splits == 1) {
      out[(size_t)b * ldo + (size_t)h * hdv + d] = __float2bfloat16_rn(tot > 0.f ? val / tot : 0.f);
    } else {
      const size_t pi = ((size_t)b * n_heads + h) * n_splits + sp;
      part_o[pi * hdv + d] = val;
      if (d == 0) {
        part_ml[pi * 2] = mm * 0.6931471805599453f;      // back to natural-log units
        part_ml[pi * 2 + 1] = tot;
      }
    }
  }
}

template <int HD, int HDV, int WARPS, int STAGES>
int launch(dim3 grid, cudaStream_t s, __nv_bfloat16* out, long ldo, float* po, float* pml, const __nv_bfloat16* q, long ldq,
           const __nv_bfloat16* kc, const __nv_bfloat16* vc, const int* bt, int max_pages, const int* slots, const int* lens,
           int H, int KV, float scale, int window, int n_splits, int own_tiles, int hd, int hdv, float softcap, const float* sinks,
           int chunk, int keep_first) {
  constexpr size_t ring = (size_t)WARPS * STAGES * (KT * HD * 2 + KT * HDV * 2);
  constexpr size_t merge = (size_t)(WARPS * COLS * (HDV + 8) + 2 * WARPS * COLS) * sizeof(float);
  constexpr size_t smem = COLS * HD * 2 + (ring > merge ? ring : merge);
  auto kern = attn_decode_krx_kernel<HD, HDV, WARPS, STAGES>;
  static bool configured[gi::MAX_DEVICES_SEEN] = {false};
  int dev;
  if (gi::unconfigured_here(configured, &dev)) {
    cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
    if (e != cudaSuccess) return gi::fail(GI_ERR_CUDA, "attention decode: %s", cudaGetErrorString(e));
    if (dev >= 0) configured[dev] = true;
  }
  return gi::check(gi::launch(kern, grid, dim3(WARPS * 32), smem, s, out, ldo, po, pml, q, ldq, kc, vc, bt, max_pages, slots, lens, H, KV,
                              scale, window, n_splits, own_tiles, hd, hdv, softcap, sinks, chunk, keep_first),
                   "attention decode (keys on rows, general)");
}

}  // namespace

// gi_attn_decode_generic_ex's operation on tensor cores: bfloat16, key and value sizes multiples of 8 up to 128.  Slices
// are counted in tiles of 16 keys; they are merged by gi_attn_combine.
extern "C" int gi_attn_decode_kr_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq,
                                    const void* kcache, const void* vcache, const int* block_table, int max_pages,
                                    const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                                    float scale, int window, int n_splits, int own_tiles, int hdv, float softcap,
                                    const float* sinks, int chunk, void* stream) {
  return gi_attn_decode_kr_ex2(out, ldo, part_o, part_ml, q, ldq, kcache, vcache, block_table, max_pages, seq_slots, seq_lens, n_seqs,
                               n_heads, n_kv, hd, scale, window, n_splits, own_tiles, hdv, softcap, sinks, chunk, 0, stream);
}

// The same with a window that keeps the sequence's first `keep_first` positions visible as well.
extern "C" int gi_attn_decode_kr_ex2(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq,
                                     const void* kcache, const void* vcache, const int* block_table, int max_pages,
                                     const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                                     float scale, int window, int n_splits, int own_tiles, int hdv, float softcap,
                                     const float* sinks, int chunk, int keep_first, void* stream) {
  if (n_seqs <= 0) return GI_OK;
  if (keep_first < 0 || (keep_first > 0 && chunk > 0)) return gi::fail(GI_ERR_ARG, "attention: kept first positions go with a window, not with chunks");
  if (own_tiles < 0) return gi::fail(GI_ERR_ARG, "attention: tiles per slice cannot be negative");
  if (hd <= 0 || hd > 128 || hd % 8 || hdv <= 0 || hdv > 128 || hdv % 8)
    return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (keys on rows): key size %d, value size %d; multiples of 8 up to 128", hd, hdv);
  if (n_heads <= 0 || n_kv <= 0 || n_heads % n_kv != 0)
    return gi::fail(GI_ERR_ARG, "attention: %d heads do not divide into %d kv heads", n_heads, n_kv);
  if (chunk < 0 || softcap < 0.f) return gi::fail(GI_ERR_ARG, "attention: a chunk or a cap cannot be negative");
  if (n_splits < 1) return gi::fail(GI_ERR_ARG, "attention: at least one slice");
  if (n_splits > 1 && (!part_o || !part_ml)) return gi::fail(GI_ERR_ARG, "attention: slices need scratch memory");
  if (ldq % 8 != 0 || ((uintptr_t)q & 15) || ((uintptr_t)kcache & 15) || ((uintptr_t)vcache & 15))
    return gi::fail(GI_ERR_UNSUPPORTED, "attention decode (keys on rows): queries and cache must be 16-byte aligned");
  const int group = n_heads / n_kv;
  const int chunks = (group + COLS - 1) / COLS;
  if ((long)n_kv * chunks > 65535 || n_seqs > 65535) return gi::fail(GI_ERR_UNSUPPORTED, "attention: more than 65535 sequences or kv heads in one launch");
  dim3 grid(n_splits, n_kv * chunks, n_seqs);
  cudaStream_t s = (cudaStream_t)stream;
  int rc;
#define GI_DECODE_KRX(HD_, HDV_, W_)                                                                                          \
  rc = launch<HD_, HDV_, W_, 2>(grid, s, (__nv_bfloat16*)out, ldo, part_o, part_ml, (const __nv_bfloat16*)q, ldq,              \
                                (const __nv_bfloat16*)kcache, (const __nv_bfloat16*)vcache, block_table, max_pages, seq_slots, \
                                seq_lens, n_heads, n_kv, scale, window, n_splits, own_tiles, hd, hdv, softcap, sinks, chunk, keep_first)
  if (hd <= 64 && hdv <= 64) GI_DECODE_KRX(64, 64, 6);
  else if (hd <= 64) GI_DECODE_KRX(64, 128, 4);
  else if (hdv <= 64) GI_DECODE_KRX(128, 64, 4);
  else GI_DECODE_KRX(128, 128, 4);
#undef GI_DECODE_KRX
  if (rc != GI_OK) return rc;
  if (n_splits > 1) return gi_attn_combine(out, ldo, GI_BF16, part_o, part_ml, n_seqs, n_heads, hdv, n_splits, stream);
  return GI_OK;
}
