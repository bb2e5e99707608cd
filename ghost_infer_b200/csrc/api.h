// C entry points of the kernel library.  Every function takes device pointers and a CUDA stream,
// launches on that stream without synchronising, and returns 0 or an error code whose text
// gi_last_error() gives.  Nothing here allocates device memory: callers pass outputs and scratch.
#pragma once

#define GI_ABI_VERSION 1

#define GI_GEMM_STORE 0      // out = A * W^T, stored in out_dtype
#define GI_GEMM_ACCUM_F32 1  // out (float) += A * W^T

#ifdef __cplusplus
extern "C" {
#endif

// Partial sums a deferred product left behind (see GI_SKINNY_ACCUM_DEFER): where they are and how the product cut its work.
typedef struct {
  const float* partials;     // null: nothing to settle
  const int* tile_first_cta; // per 128-row tile: the first and the last block that held a piece of it
  const int* tile_last_cta;
  const int* cta_first_tile; // per block: the tile its range began in (that piece sits in the block's slot 0)
  int nt;                    // token-tile width of the product (16, 32 or 64)
} gi_settle_t;

#ifdef __CUDACC__
// Which blocks of a deferred product hold pieces of the 128-column tile of column f.  Blocks take contiguous ranges
// of K blocks, so every block after the first began its range inside the tile (its piece sits in its slot 0); only
// the first block may have come from an earlier tile (slot 1).  The tables are uploaded once per shape and never
// written by a kernel: a kernel may read them before its dependency wait.
struct gi_settle_span {
  int c_first, c_last, first_slot;
};
__device__ __forceinline__ gi_settle_span gi_span_of(const gi_settle_t& st, int f) {
  gi_settle_span s;
  const int tile = f / 128;
  s.c_first = st.tile_first_cta[tile];
  s.c_last = st.tile_last_cta[tile];
  s.first_slot = (s.c_first != s.c_last && tile != st.cta_first_tile[s.c_first]) ? 1 : 0;
  return s;
}
// The address of block c's piece for token m, column f.
__device__ __forceinline__ const float* gi_piece(const gi_settle_t& st, const gi_settle_span& s, int c, int m, int f) {
  const int slot = (c == s.c_first) ? s.first_slot : 0;
  return st.partials + ((size_t)c * 2 + slot) * (128 * st.nt) + (size_t)m * 128 + f % 128;
}
// The sum of a column's pieces in the order of the K ranges.  The loads of up to eight pieces are issued together
// (absent ones count as +0, which changes no sum), so that the sum costs one trip to the L2 cache, not one per piece.
__device__ __forceinline__ float gi_sum_pieces(const gi_settle_t& st, const gi_settle_span& s, int m, int f) {
  float acc = 0.f;
  for (int c0 = s.c_first; c0 <= s.c_last; c0 += 8) {
    float p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) p[j] = (c0 + j <= s.c_last) ? __ldcg(gi_piece(st, s, c0 + j, m, f)) : 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) acc += p[j];
  }
  return acc;
}
// Two columns of the same tile at once (a rotated pair): both columns' loads are in flight together.
__device__ __forceinline__ float2 gi_sum_pieces2(const gi_settle_t& st, const gi_settle_span& s, int m, int fa, int fb) {
  float2 acc = make_float2(0.f, 0.f);
  for (int c0 = s.c_first; c0 <= s.c_last; c0 += 8) {
    float pa[8], pb[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      pa[j] = (c0 + j <= s.c_last) ? __ldcg(gi_piece(st, s, c0 + j, m, fa)) : 0.f;
      pb[j] = (c0 + j <= s.c_last) ? __ldcg(gi_piece(st, s, c0 + j, m, fb)) : 0.f;
    }
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc.x += pa[j];
      acc.y += pb[j];
    }
  }
  return acc;
}
__device__ __forceinline__ float4 gi_sum_pieces4(const gi_settle_t& st, const gi_settle_span& s, int m, int f) {
  float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
  for (int c0 = s.c_first; c0 <= s.c_last; c0 += 8) {
    float4 p[8];
#pragma unroll
    for (int j = 0; j < 8; ++j)
      p[j] = (c0 + j <= s.c_last) ? __ldcg(reinterpret_cast<const float4*>(gi_piece(st, s, c0 + j, m, f))) : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      acc.x += p[j].x;
      acc.y += p[j].y;
      acc.z += p[j].z;
      acc.w += p[j].w;
    }
  }
  return acc;
}
#endif

const char* gi_last_error(void);
int gi_abi_version(void);
// Programmatic dependent launch: kernels of a stream may begin while their predecessor drains (off by default).
void gi_set_pdl(int on);
int gi_get_pdl(void);

int gi_embed(float* out, const void* table, int table_dtype, const int* tokens, int n_tokens, int d, int vocab,
             void* stream);
int gi_rmsnorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows, int n_rows,
               int d, float eps, void* stream);
// The same, first adding deferred partial sums to the rows it reads (and writing the settled rows back to x, unless
// `rows` selects: then x is left as it is and must not be read again).
int gi_rmsnorm_settle(void* out, int out_dtype, float* x, const void* w, int w_dtype, const int* rows, int n_rows,
                      int d, float eps, gi_settle_t settle, void* stream);
int gi_silu_mul(void* out, const void* gate_up, int dtype, int n_rows, int f, int interleaved, void* stream);

int gi_gemm_generic(void* out, int out_dtype, int mode, const void* A, int a_dtype, const void* W, int w_dtype, int M,
                    int N, int K, long lda, long ldw, long ldo, void* stream);

// mode of gi_gemm_skinny_bf16
#define GI_SKINNY_STORE_BF16 0
#define GI_SKINNY_STORE_F32 1
#define GI_SKINNY_ACCUM_F32 2   // out (float) += product
#define GI_SKINNY_SWIGLU 3      // W rows interleaved [8 gate | 8 up]; out[M, N/2] bfloat16 = silu(gate) * up
#define GI_ACT_GELU 0x100       // or-ed into a gated mode (GI_SKINNY_SWIGLU, GI_TC_SWIGLU) of the tcgen05 products: the gate's
                                // activation is gelu in its tanh form instead of silu
#define GI_SKINNY_STORE_DEFER 5 // the same for STORE_BF16: whole tiles are stored, cut tiles stay as partial sums for gi_rope_cache_write
#define GI_SKINNY_ACCUM_DEFER 4 // gi_gemm_stream_bf16 only: as ACCUM_F32, but tiles cut between blocks leave their partial
                                // sums in `scratch` for gi_rmsnorm / gi_settle to add (no exchange between blocks)
int gi_gemm_skinny_bf16(void* out, int mode, const void* A, const void* W, int M, int N, int K, long lda, long ldw,
                        long ldo, void* stream);

// Persistent stream-K tcgen05 product for at most 64 rows of activations (modes as gi_gemm_skinny_bf16).
// `scratch`: gi_gemm_stream_scratch_floats() floats; `counters`: one int per 128 rows of W, zero at first use.
// use_pdl: launch with programmatic stream serialization (weights are prefetched before the dependency wait).
long gi_gemm_stream_scratch_floats(void);
int gi_gemm_stream_bf16(void* out, int mode, const void* A, const void* W, float* scratch, int* counters, int n_counters,
                        int M, int N, int K, long lda, long ldw, long ldo, int use_pdl, void* stream);
// As gi_gemm_stream_bf16; `next_W` [next_N, next_K] (optional) is the matrix that the next streamed product in this
// stream will read: the kernel asks the L2 cache for the first `units_ahead` 16 KB units of each of that launch's blocks
// once its own loads are issued (`next_mode`: the mode of that launch, which decides how it cuts its work).  A wrong
// guess costs bandwidth, never a result; next_W must be valid memory.
int gi_gemm_stream_bf16_ex(void* out, int mode, const void* A, const void* W, float* scratch, int* counters, int n_counters,
                           int M, int N, int K, long lda, long ldw, long ldo, int use_pdl, const void* next_W, int next_N,
                           int next_K, long next_ldw, int next_mode, int units_ahead, void* stream);
int gi_gemm_stream_status(int* status);
// percent > 0: a product that finishes its own sums and has fewer 128-row tiles than SMs, but at least `percent` of
// them, runs one block per tile, so that no tile is cut between blocks; 0: always one block per SM.  Returns the old value.
int gi_gemm_stream_whole_tiles(int percent);
// Time stamps of the streamed products' blocks, for a timeline of a decode step: see gemm_stream.cu.
long gi_gemm_stream_timeline(unsigned long long* buf, int slots);
int gi_gemm_stream_geometry(int M, int N, int K, int* n_ctas, int* kb_per_tile, int* nt);

// x[rows, :] += the partial sums, in the order of the K ranges.  rows: optional selection; n_features = width of x.
int gi_settle(float* x, gi_settle_t settle, const int* rows, int n_rows, int d, void* stream);

// mode of gi_gemm_tc_bf16 (same meanings as the skinny product's)
#define GI_TC_STORE_BF16 0
#define GI_TC_STORE_F32 1
#define GI_TC_ACCUM_F32 2
#define GI_TC_SWIGLU 3
#define GI_TC_QKV_ROPE 4        // gi_gemm_tc_qkv_rope only: queries rotated and stored, keys and values into the cache
// tcgen05 / TMA product for many rows of activations; tile_n is 128 or 256
int gi_gemm_tc_bf16(void* out, int mode, const void* A, const void* W, int M, int N, int K, long lda, long ldw,
                    long ldo, int tile_n, void* stream);
#define GI_ACT_RELU2 0x200      // or-ed into GI_TC_STORE_BF16 (gi_gemm_tc_bf16_bias): out = relu(A W^T + bias)^2 as bfloat16
#define GI_ACT_GELU_ERF 0x400   // or-ed into GI_TC_STORE_BF16: out = gelu(A W^T) in the exact (erf) form as bfloat16, no bias
// gi_gemm_tc_bf16 with `bias` (bfloat16 [N], or null) for the mode GI_TC_STORE_BF16 | GI_ACT_RELU2.
int gi_gemm_tc_bf16_bias(void* out, int mode, const void* A, const void* W, const void* bias, int M, int N, int K, long lda,
                         long ldw, long ldo, int tile_n, void* stream);
// The q/k/v product of a prompt step that rotates and stores in its epilogue (the work of gi_rope_cache_write, the same
// bits): out [M, N] packed rows of which the queries' columns are written; N = (n_heads + 2 n_kv) * hd, hd 64 or 128.
int gi_gemm_tc_qkv_rope(void* out, const void* A, const void* W, int M, int N, int K, long lda, long ldw, long ldo,
                        const float* table, const int* positions, const int* slots, const int* block_table, int max_pages,
                        void* kcache, void* vcache, int n_heads, int n_kv, int hd, int write_cache, void* stream);
// narrower tiles for the columns of an unfilled last round of blocks: on (default) or off
int gi_gemm_tc_tail_tiles(int on);
int gi_gemm_tc_status(int* status);

// table[t, i] = (cos, sin)(positions[t] * inv_freq[i]), float2 [n_tokens, rot / 2]
int gi_rope_table(float* table, const int* positions, const float* inv_freq, int n_tokens, int rot, void* stream);
int gi_rope_cache_write(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots,
                        const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens, int n_heads,
                        int n_kv, int hd, int rot, int adjacent, int write_cache, void* stream);
// The same for rows whose product was deferred (GI_SKINNY_STORE_DEFER): values of tiles that were cut between blocks
// are the sums of the partial sums, rounded to the row's dtype as a stored value would have been.
int gi_rope_cache_write_settle(void* qkv, int dtype, long ld, const float* table, const int* positions, const int* slots,
                               const int* block_table, int max_pages, void* kcache, void* vcache, int n_tokens,
                               int n_heads, int n_kv, int hd, int rot, int adjacent, int write_cache, gi_settle_t settle,
                               void* stream);

int gi_attn_prefill_generic(void* out, long ldo, const void* q, long ldq, int dtype, const void* kcache,
                            const void* vcache, const int* block_table, int max_pages, const int* cu_seqlens,
                            const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv,
                            int hd, float scale, int window, void* stream);
int gi_attn_decode_generic(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, int dtype,
                           const void* kcache, const void* vcache, const int* block_table, int max_pages,
                           const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                           float scale, int window, int n_splits, int own_tiles, void* stream);

// The same two operations with what a model's attention may add, each off at its neutral value: values of another
// width than the keys (hdv; the value cache is [page][kv head][64][hdv], the output [tokens, heads * hdv]), a cap
// on the scores (s <- cap * tanh(s / cap); 0: none), a sink per head (float[heads]: one more term exp(sink) in the
// softmax's denominator, without key or value; null: none) and chunks (a query sees keys of its own chunk
// floor(pos / chunk) only; 0: none).  part_o holds hdv values per (sequence, head, slice).
int gi_attn_prefill_generic_ex(void* out, long ldo, const void* q, long ldq, int dtype, const void* kcache,
                               const void* vcache, const int* block_table, int max_pages, const int* cu_seqlens,
                               const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads,
                               int n_kv, int hd, float scale, int window, int hdv, float softcap, const float* sinks,
                               int chunk, void* stream);
int gi_attn_decode_generic_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, int dtype,
                              const void* kcache, const void* vcache, const int* block_table, int max_pages,
                              const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                              float scale, int window, int n_splits, int own_tiles, int hdv, float softcap,
                              const float* sinks, int chunk, void* stream);

// The same two with the value rows `v_row_stride` numbers apart instead of hdv (a cache whose values are the leading hdv
// numbers of its key rows passes the keys as values and the keys' row length here); keys up to 640 and values up to 512 wide.
int gi_attn_prefill_generic_ex2(void* out, long ldo, const void* q, long ldq, int dtype, const void* kcache,
                                const void* vcache, const int* block_table, int max_pages, const int* cu_seqlens,
                                const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads,
                                int n_kv, int hd, float scale, int window, int hdv, float softcap, const float* sinks,
                                int chunk, long v_row_stride, void* stream);
int gi_attn_decode_generic_ex2(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, int dtype,
                               const void* kcache, const void* vcache, const int* block_table, int max_pages,
                               const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                               float scale, int window, int n_splits, int own_tiles, int hdv, float softcap,
                               const float* sinks, int chunk, long v_row_stride, void* stream);

// ---- layers with a low-rank latent in place of keys and values per head, and what their feed-forwards add.
// y = (x - mean) / sqrt(var + eps) * w per row, 32-bit statistics; `rows` (optional) picks the rows of x.
int gi_layernorm(void* out, int out_dtype, const float* x, const void* w, int w_dtype, const int* rows, int n_rows, int d,
                 float eps, void* stream);
// The same, first adding deferred partial sums to the rows it reads (as gi_rmsnorm_settle does).
int gi_layernorm_settle(void* out, int out_dtype, float* x, const void* w, int w_dtype, const int* rows, int n_rows, int d,
                        float eps, gi_settle_t settle, void* stream);
// out[t, :f] = act(in[t, :f] + bias) (bias optional; act 0: none, 1: relu squared); with `residual` [n_rows, d] also
// residual[t, :] += res_bias in the same launch.
int gi_bias_act(void* out, const void* in, int dtype, long ld_in, const void* bias, int w_dtype, int n_rows, int f, int act,
                float* residual, const void* res_bias, int d, void* stream);
// in[t] = [query latent (rq) | key/value latent (r) | rotary key part (dr)]: cq[t] = rmsnorm(query latent) * wq (skipped
// when rq is 0); the cache row of token t, [r + dr] numbers in pages [page][64][r + dr], = [rmsnorm(latent) * wc | key part
// with its first `rot` numbers turned in neighbouring pairs by table[t]].
int gi_latent_prepare(void* cq, const void* in, int dtype, long ld, const void* wq, const void* wc, int w_dtype, float eps,
                      const float* table, int rot, const int* positions, const int* slots, const int* block_table, int max_pages,
                      void* kcache, int n_tokens, int rq, int r, int dr, int write_cache, void* stream);
// qa[t, h, r : r + dr] = q[t, h, dn : dn + dr] with its first `rot` numbers turned (q rows [heads][dn + dr], qa rows
// [heads][r + dr]).
int gi_latent_query_rot(void* qa, long ldqa, const void* q, long ldq, int dtype, const float* table, int rot, int n_tokens,
                        int n_heads, int dn, int dr, int r, void* stream);
// out[t, h * ohs + n] = sum_k a[t, h * ahs + k] * w[h * whs + n * ldw + k * kstride], n < N, k < K, for every head h; out has
// a's type.  tensor_cores: bfloat16 operands with kstride 1 take `mma.sync`.
int gi_bmm_heads(void* out, long ldo, long ohs, const void* a, long lda, long ahs, int dtype, const void* w, int w_dtype,
                 long whs, long ldw, long kstride, int M, int N, int K, int heads, int tensor_cores, void* stream);
// Causal attention of n_heads heads over one shared row per position, on tensor cores (bfloat16): the cache holds rows of dk
// numbers in pages [page][64][dk]; q rows are [heads][dk]; score = q . row * scale; the value is the row's first dv numbers;
// out rows [heads][dv].  cu_seqlens given: a prompt step (seq_pos0: cached lengths before it).  cu_seqlens null: a one-token
// step (seq_lens: lengths including the token) cut into n_splits slices of the context (own_tiles > 0: that many 64-key
// tiles of each sequence's own span per slice), merged inside; part_o holds dv floats and part_ml 2 per (sequence, head,
// slice).  dk and dv multiples of 8, dk <= 576, dv <= 512.
int gi_attn_latent_tc(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                      const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots, const int* seq_pos0,
                      const int* seq_lens, int n_seqs, int max_q_len, int n_heads, int dk, int dv, float scale, int n_splits,
                      int own_tiles, void* stream);
// table[t, i] = magnitude * (cos, sin)(positions[t] * inv_freq[i])
int gi_rope_table_scaled(float* table, const int* positions, const float* inv_freq, int n_tokens, int rot, float magnitude,
                         void* stream);

// The prompt operation of gi_attn_prefill_generic_ex on tensor cores: bfloat16, key and value sizes multiples of 8 up to 128.
int gi_attn_prefill_tc_ex(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                          const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                          const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd, float scale,
                          int window, int hdv, float softcap, const float* sinks, int chunk, void* stream);

// The one-token operation of gi_attn_decode_generic_ex on tensor cores (keys on the rows of the tile): bfloat16, key and
// value sizes multiples of 8 up to 128; own_tiles counts tiles of 16 keys.
int gi_attn_decode_kr_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                         const void* vcache, const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                         int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits, int own_tiles,
                         int hdv, float softcap, const float* sinks, int chunk, void* stream);

// Keys and values of a step's tokens into the cache without rotation, for packed rows [q: heads * hd | k: kv * hd |
// v: kv * hdv].  `first` (optional, [tokens, kv * hdv], the rows' type): the values are first blended with it,
// v <- (1 - lambda) v + lambda first, in 32-bit, lambda read from device memory; the blended values are also
// written back into the rows.  `copy_to` (optional, same shape): receives the rows' values as they are (for a later
// layer's `first`).
int gi_kv_store(void* qkv, int dtype, long ld, const void* first, const float* lambda, void* copy_to,
                const int* positions, const int* slots, const int* block_table, int max_pages, void* kcache,
                void* vcache, int n_tokens, int n_heads, int n_kv, int hd, int hdv, int write_cache, void* stream);

// ---- Mamba-2 (state-space duality) mixer.  Per-sequence state rows live in one float matrix [rows, row_floats]:
// first heads * N * P floats of S (per head N x P), then channels * (taps - 1) floats of the convolution's last
// inputs (oldest first per channel).  A sequence of slot s uses row s; slot -1 (a padding row) uses the last row.
// proj: the input projection's rows [tokens, 2 * inner + 2 * G * N + heads] = [z | x | B | C | dt], inner = heads * P.
// conv: xbc_out[t, c] = silu(bias[c] + sum_j w[c, j] * in[t - (taps - 1) + j, c]) over channels c of [x | B | C], inputs
// before the step's first token from the state (zero for a fresh sequence); then the state takes the last taps - 1
// inputs (gi_mamba2_conv_update, a launch of its own because it overwrites what the first reads).  Other mixers with a
// short convolution use the two as they are: `inner` is the column of the rows where the `channels` convolved ones start
// (0 and up), `s_floats` the floats of a state row before the convolution's inputs.
int gi_mamba2_conv(void* xbc_out, const void* proj, int dtype, long ld_proj, const void* conv_w, const void* conv_b,
                   int w_dtype, const float* state, long state_ld, int state_rows, const int* cu_seqlens,
                   const int* seq_slots, int n_seqs, int max_q_len, int inner, int channels, int taps, int s_floats,
                   void* stream);
int gi_mamba2_conv_update(const void* proj, int dtype, long ld_proj, float* state, long state_ld, int state_rows,
                          const int* cu_seqlens, const int* seq_slots, int n_seqs, int inner, int channels, int taps,
                          int s_floats, void* stream);
// scan: dt <- softplus(dt + dt_bias); per head S <- exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, everything in
// 32-bit, tokens of a sequence in order, S read from and written back to the state.  y: float [tokens, inner].
int gi_mamba2_scan(float* y, const void* xbc, const void* proj, int dtype, long ld_proj, const void* dt_bias,
                   const void* a_log, const void* d_skip, int w_dtype, float* state, long state_ld, int state_rows,
                   const int* cu_seqlens, const int* seq_slots, int n_seqs, int heads, int P, int N, int groups,
                   void* stream);
// out[t, :] = groupwise_rmsnorm(y[t, :] * silu(z[t, :])) * w, z the first inner columns of proj; `parts` equal parts,
// each divided by its own root mean square (eps inside the root).
int gi_mamba2_gate_norm(void* out, int out_dtype, const float* y, const void* proj, int dtype, long ld_proj,
                        const void* w, int w_dtype, int n_tokens, int inner, int parts, float eps, void* stream);

// ---- routed feed-forward (mixture of experts).
// route: logits = h W_r^T in 32-bit; the `top` largest per token (first wins a tie), weights = softmax over the chosen
// logits; optional shared gate sg[t] = sigmoid(h . w_sg).  ids int[tokens, top], wts float[tokens, top].
int gi_moe_route(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                 const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, void* stream);
// The same with the kind of weights named: 0 as above; 1: every chosen expert's own sigmoid(logit), not renormalized.
int gi_moe_route_scored(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                        const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, int score_mode, void* stream);
// plan: a stable counting sort of the tokens' choices by expert.  offsets int[experts + 1]; perm int[entries] (sorted
// place -> entry t * top + k); inv int[entries] (entry -> sorted place).  scratch: int[(entries + 1023) / 1024 *
// experts * 2 + entries].
int gi_moe_plan(int* offsets, int* perm, int* inv, int* scratch, const int* ids, int entries, int experts, void* stream);
// Products over the sorted rows, each row with its expert's matrix (w + expert * w_stride, [n, k] row-major).
// gate_up: out[r, 0..f) = silu(a[src(r)] Wg^T) * (a[src(r)] Wu^T), W = [gate (f rows); up (f rows)], src(r) = perm[r] / top.
// down: out[r, :] = a[r] W^T stored as float.
int gi_moe_gemm_gate_up(void* out, int dtype, const void* a, long lda, const void* w, int w_dtype, long w_stride,
                        const int* offsets, const int* perm, int entries, int top, int experts, int f, int k,
                        int interleaved, void* stream);    // interleaved: W's rows in blocks [8 gate | 8 up]
// out[r, :] = in[perm[r] / top, :] (the step's rows in sorted order, an expert's rows side by side).
int gi_moe_gather_rows(void* out, const void* in, int dtype, long ld_in, const int* perm, int entries, int top, int width,
                       void* stream);
int gi_moe_gemm_down(float* out, const void* a, int dtype, long lda, const void* w, int w_dtype, long w_stride,
                     const int* offsets, int entries, int experts, int n, int k, void* stream);
// gi_moe_gemm_down with a choice of what is stored: act_out 0: the sums as float; 1: relu(sum)^2 in the rows' type (the
// hidden layer of an ungated expert).
int gi_moe_gemm_rows(void* out, const void* a, int dtype, long lda, const void* w, int w_dtype, long w_stride,
                     const int* offsets, int entries, int experts, int n, int k, int act_out, void* stream);
// gi_moe_gather_rows with every gathered row multiplied by scale[perm[r]] (one float per entry; null: as they are).
int gi_moe_gather_rows_scaled(void* out, const void* in, int dtype, long ld_in, const int* perm, const float* scale,
                              int entries, int top, int width, void* stream);
// The experts of a prompt step through the tcgen05 products, one expert's stretch of the sorted rows after another, from
// offsets on the HOST (int[experts + 1]); bfloat16, gate and up rows interleaved.  hidden: bfloat16 [entries, f] scratch.
int gi_moe_experts_tc(float* out, void* hidden, const void* rows, const void* w_gate_up, long gate_up_stride,
                      const void* w_down, long down_stride, const int* host_offsets, int experts, int width, int f,
                      float* scratch, int* counters, int n_counters, void* stream);
// The same for ungated experts, hidden = relu(rows W_up^T)^2 with w_up [experts][f][width].
int gi_moe_experts_tc_ungated(float* out, void* hidden, const void* rows, const void* w_up, long up_stride, const void* w_down,
                              long down_stride, const int* host_offsets, int experts, int width, int f, float* scratch,
                              int* counters, int n_counters, void* stream);
// residual[t, :] += sum_k wts[t, k] * down[inv[t * top + k], :] (k in order; wts null: every weight 1) + sgate[t] *
// shared[t, :] (if given).
int gi_moe_combine(float* residual, const float* down, const int* inv, const float* wts, const float* shared,
                   const float* sgate, int n_tokens, int width, int top, void* stream);

// act(gate) * up over rows [gate | up] (or blocks [8 gate | 8 up]); act 0: silu, 1: the tanh form of gelu.
int gi_act_mul(void* out, const void* gate_up, int dtype, int n_rows, int f, int interleaved, int act, void* stream);
// x[t, :] = table[tokens[t], :] * scale.
int gi_embed_scaled(float* out, const void* table, int table_dtype, const int* tokens, int n_tokens, int d, int vocab,
                    float scale, void* stream);
// own_tiles > 0: slice s of a sequence holds tiles [s * own_tiles, (s + 1) * own_tiles) of 32 keys of its own span,
// whatever n_splits is (which must cover the longest span); 0: each span is cut into n_splits equal slices.

// bfloat16, head size 64 or 128: the same operation as gi_attn_prefill_generic, on tensor cores
int gi_attn_prefill_tc(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                       const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                       const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd, float scale,
                       int window, void* stream);
// bfloat16, head size 128: the same on tcgen05 tensor cores (scores and output accumulate in tensor memory).
// q_rows: rows of the packed q/k/v matrix; cache_pages: pages the cache tensors hold.
int gi_attn_prefill_t5(void* out, long ldo, const void* q, long ldq, long q_rows, const void* kcache, const void* vcache,
                       long cache_pages, const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                       const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd, float scale, int window,
                       void* stream);
// query tiles two to a block (the i-th from the end with the i-th from the start): 0 never, 1 where the launch then
// is one round of blocks (default), 2 always
// gi_attn_prefill_t5 with a cap on the scores, a sink per head and chunks of positions (see gi_attn_prefill_generic_ex).
int gi_attn_prefill_t5_ex(void* out, long ldo, const void* q, long ldq, long q_rows, const void* kcache, const void* vcache,
                          long cache_pages, const int* block_table, int max_pages, const int* cu_seqlens,
                          const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd,
                          float scale, int window, float softcap, const float* sinks, int chunk, void* stream);
int gi_attn_prefill_t5_pairing(int mode);
int gi_attn_prefill_t5_status(int* status);
// bfloat16, head size 64 or 128: the same operation as gi_attn_decode_generic, on tensor cores
int gi_attn_decode_tc(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                      const void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                      const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window,
                      int n_splits, void* stream);
// the same with a choice of tile: 32 keys (one block per SM) or 16 keys (two blocks per SM)
int gi_attn_decode_tc_ex(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                         const void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                         const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window,
                         int n_splits, int tile_keys, void* stream);
// the same with the slices merged inside the kernel by the block that finishes last (counters: one int per sequence x
// kv head x chunk of 16 heads, zero before the first use; nullptr: merged by a second kernel), and, with own_tiles > 0,
// slices of that many tiles of each sequence's own span instead of n_splits equal ones
int gi_attn_decode_tc_merged(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters, const void* q,
                             long ldq, const void* kcache, const void* vcache, const int* block_table, int max_pages,
                             const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale,
                             int window, int n_splits, int own_tiles, int tile_keys, int stages, void* stream);
// stages: depth of each warp's ring of tiles, 2 to 4 (0: the default for the head size)
// The same on rows that are not rotated yet: `qkv` holds one packed [q | k | v] row per sequence as the q/k/v product
// left it (`settle`: its pending partial sums), `table` [sequences][rot / 2] the (cos, sin) of each sequence's newest
// position.  The kernel rotates q and k (pairs (i, i + rot / 2)) and stores k and v at position length - 1 itself:
// gi_rope_cache_write's work for a decode step, inside the attention's launch.
int gi_attn_decode_tc_rope(void* out, long ldo, float* part_o, float* part_ml, int* counters, int n_counters, const void* qkv,
                           long ld, void* kcache, void* vcache, const int* block_table, int max_pages, const int* seq_slots,
                           const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits,
                           int own_tiles, int tile_keys, int stages, const float* table, int rot, gi_settle_t settle,
                           void* stream);
// The decode attention with the keys on the rows of the tensor-core tile and up to 8 heads on its columns (half the
// products per key for groups of up to 8 heads); slices are merged by gi_attn_combine.  warps: 4, 6 or 8 a block;
// stages: 2 or 3 tiles deep per warp.
int gi_attn_decode_kr(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                      const void* vcache, const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                      int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits, int own_tiles,
                      int warps, int stages, void* stream);
int gi_attn_combine(void* out, long ldo, int dtype, const float* part_o, const float* part_ml, int n_seqs, int n_heads,
                    int hd, int n_splits, void* stream);

int gi_sample(int* out_tokens, const float* logits, long ld, int n_rows, int vocab, float temperature, int top_k,
              float top_p, unsigned long long* rng_state, const int* state_index, void* stream);

// ---- layers that read the stream itself and norm a sublayer's output (stream_parts.cu) ---------------------------------
// out (activation type) = x (float32), n_values numbers.
int gi_cast_rows(void* out, int out_dtype, const float* x, long n_values, void* stream);
// x[r] += y[r] / sqrt(mean(y[r]^2) + eps) * w [* scale], float32 rows of d numbers; scale may be null.
int gi_postnorm_add(float* x, const float* y, const void* w, const void* scale, int w_dtype, int n_rows, int d, float eps,
                    void* stream);
// gi_cast_rows that also sets `zero` (float32, n_values, or null) to zero; gi_postnorm_add that also writes the new rows
// of x in the type `h_dtype` to `h_out` (or null) and, with `zero_y`, sets y to zero once it is read.
int gi_cast_rows_zero(void* out, int out_dtype, const float* x, float* zero, long n_values, void* stream);
int gi_postnorm_add_ex(float* x, float* y, const void* w, const void* scale, int w_dtype, int n_rows, int d, float eps,
                       void* h_out, int h_dtype, int zero_y, void* stream);
// out += alpha * a over n_values float32 numbers.
int gi_axpy(float* out, const float* a, float alpha, long n_values, void* stream);
// One token's float32 row [q: n_heads * hd | k: n_kv * hd | v: n_kv * hdv] (n_kv 0: queries only): biases (each may be
// null), RMS norm over the whole of q and of k with weights wq / wk (null: no norm), rotation of the first 2 * half numbers
// of every head by `table` [tokens][half] of (cos, sin) (adjacent: pairs (2i, 2i + 1); else (i, i + half)), q into q_out,
// k and v into the token's place in the pages.
int gi_qk_prepare(void* q_out, long ldq, int dtype, const float* in, long ld, const void* bq, const void* bk, const void* bv,
                  const void* wq, const void* wk, int w_dtype, float eps, const float* table, int half, int adjacent,
                  const int* positions, const int* slots, const int* block_table, int max_pages, void* kcache, void* vcache,
                  int n_tokens, int n_heads, int n_kv, int hd, int hdv, int write_cache, void* stream);
// out = a * sigmoid(g) (act 0) or a * silu(g) (act 1); a and out are contiguous [n_rows, f].
int gi_gate_mul(void* out, const void* a, const void* g, long ldg, int dtype, int n_rows, int f, int act, void* stream);
// out = y / sqrt(mean over each group of `group` values (y^2) + eps) * w * act(g); w has `group` values (w_per_row 0) or `inner`.
int gi_norm_gate(void* out, int dtype, const float* y, const void* g, long ldg, const void* w, int w_dtype, int n_rows, int inner,
                 int group, int w_per_row, int act, float eps, void* stream);
// out[t, c] = gelu_tanh(gx[t, c]) * table[tokens[t], col0 + c], c < dim.
int gi_side_gate(void* out, const void* gx, long ldg, int dtype, const void* table, long ld_table, int w_dtype, const int* tokens,
                 int n_rows, int col0, int dim, void* stream);
// out = gelu(in), the exact form, [n_rows, f].
int gi_act_rows(void* out, const void* in, long ld_in, int dtype, int n_rows, int f, void* stream);

// ---- linear attention with a matrix of state per head (linear_state.cu) -------------------------------------------------
// o float32 [tokens, heads * V].  q, k: rows with qk_heads * K numbers at the pointer; v: heads * V.  a_in / b_in: rows with
// one number per head (null: a constant decay decay_c[h] / no write strength).  With a_in, decay_c holds A_log.
// n_tokens: the rows of the step (0: not known); as many as sequences means one token each, and a smaller kernel runs.
int gi_linear_state(float* o, const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, const void* a_in,
                    long lda, const void* b_in, long ldb, int dtype, const float* decay_c, const float* dt_bias, float* state,
                    long state_ld, int state_rows, const int* cu_seqlens, const int* seq_slots, int n_seqs, int heads,
                    int qk_heads, int K, int V, int in_act, int unit_norm, float norm_eps, float q_scale, int delta,
                    int n_tokens, void* stream);

// The same with the gates ready made: g_direct / u_direct float32 [tokens, heads] (either may be null) give the decay of every
// token and head as it is, and a number that multiplies what the token writes (S <- g S + k (u v)^T; not with the delta rule).
int gi_linear_state_gated(float* o, const void* q, long ldq, const void* k, long ldk, const void* v, long ldv, const void* a_in,
                          long lda, const void* b_in, long ldb, int dtype, const float* decay_c, const float* dt_bias,
                          const float* g_direct, const float* u_direct, float* state, long state_ld, int state_rows,
                          const int* cu_seqlens, const int* seq_slots, int n_seqs, int heads, int qk_heads, int K, int V, int in_act,
                          int unit_norm, float norm_eps, float q_scale, int delta, int n_tokens, void* stream);

// ---- a matrix memory with a running maximum (mlstm.cu) ------------------------------------------------------------------
// Per token and head: keep = exp(f + m_prev - m), put = exp(i - m), out_scale = s / (max(|n . (s q)|, exp(-m)) + 1e-6), with
// i = cap tanh((gate_i + bias_i) / cap), f = log sigmoid(cap tanh((gate_f + bias_f) / cap)), m = max(f + m_prev, i),
// n = keep n_prev + put k.  q, k: rows with heads * K numbers at the pointer; gate_i, gate_f: rows with one number per head.
// state: per slot and head K + 1 floats (n, m) at the pointer, rows state_ld apart; the last of state_rows rows serves slot -1.
int gi_mlstm_gates(float* keep, float* put, float* out_scale, const void* q, long ldq, const void* k, long ldk, const void* gate_i,
                   const void* gate_f, long ldg, int dtype, const float* bias_i, const float* bias_f, float cap, float q_scale,
                   float* state, long state_ld, int state_rows, const int* cu_seqlens, const int* seq_slots, int n_seqs, int heads,
                   int K, void* stream);

// ---- several copies of the residual stream (hyper_streams.cu) -----------------------------------------------------------
// x float32 [tokens][streams][d].
int gi_stream_expand(float* x, const float* e, int n_tokens, int streams, int d, void* stream);
// out[r] = sum over the copies of x[rows[r]] (rows null: every token in order).
int gi_stream_sum(float* out, const float* x, const int* rows, int n_rows, int streams, int d, void* stream);
// h[t] = rmsnorm(sum_s blend[s] x[t][s]) * w in `dtype`; `zero` (or null): float32 [tokens][d] set to zero in the same pass.
int gi_hyper_read(void* h, int dtype, const float* x, const float* blend, const void* w, int w_dtype, float* zero, int n_tokens,
                  int streams, int d, float eps, void* stream);
// gi_hyper_read and, for a step of one token a sequence, the input convolution in the same launch (conv_out, or null).
int gi_hyper_read_conv(void* h, int dtype, const float* x, const float* blend, const void* w, int w_dtype, float* zero, int n_tokens,
                       int streams, int d, float eps, void* conv_out, const void* taps_w, int k_dtype, const float* state,
                       long state_ld, int state_rows, const int* slots, int taps, void* stream);
// out[t] = h[t] + sum_j taps_w[:, j] h[t - taps + 1 + j] per channel (taps_w [d][taps]); inputs before the step come from the
// sequence's state (float32 [taps - 1][d] per slot, oldest first; rows state_ld apart, the last row serves slot -1).  Rows of
// one sequence are neighbours in the step and carry the same slot.
int gi_input_conv(void* out, const void* h, int dtype, const void* taps_w, int w_dtype, const float* state, long state_ld,
                  int state_rows, const int* slots, int n_tokens, int d, int taps, void* stream);
// x[t][to] = sum_s mix[s][to] x[t][s] + share[to] * y[t] * sigmoid(z[t] + z_bias) (z null: no gate); with `state`, the block of
// a sequence's last token renews the convolution's state from `h` (the rows input_conv read).
int gi_hyper_write(float* x, const float* y, const void* z, const void* z_bias, int dtype, int w_dtype, const float* mix,
                   const float* share, const void* h, float* state, long state_ld, int state_rows, const int* slots, int n_tokens,
                   int streams, int d, int taps, void* stream);
int gi_scale_rows(float* x, float c, long n_values, void* stream);

// ---- attention normed head by head, gated heads, clamped gated rows (head_parts.cu) -------------------------------------
// One token's float32 row [q: n_heads * hd | k: n_kv * hd | v: n_kv * hdv | ...] (n_kv 0: queries only): biases (each may be
// null), per-head RMS norms of q and k with weights wq / wk of hd numbers shared by the heads (norm_q / norm_k; a null weight
// is 1), per-head RMS norm of v without a weight (norm_v), rotation as in gi_qk_prepare, q into q_out, k and v into the pages.
int gi_head_prepare(void* q_out, long ldq, int dtype, const float* in, long ld, const void* bq, const void* bk, const void* bv,
                    const void* wq, const void* wk, int w_dtype, int norm_q, int norm_k, int norm_v, float eps, const float* table,
                    int half, int adjacent, const int* positions, const int* slots, const int* block_table, int max_pages,
                    void* kcache, void* vcache, int n_tokens, int n_heads, int n_kv, int hd, int hdv, void* stream);
// out[t][h][:] = a[t][h][:] * sigmoid(g[t * ldg + h]).
int gi_head_gate(void* out, const void* a, int dtype, const float* g, long ldg, int n_rows, int n_heads, int hdv, void* stream);
// v = y[t][h][:] * scale[t][h] (scale null: 1); out = v / sqrt(mean(v^2) + eps) * w[h][:] * sigmoid(g[t * ldg + h * hdv + :]).
int gi_scaled_norm_gate(void* out, int dtype, const float* y, const float* scale, const float* g, long ldg, const void* w, int w_dtype,
                        int n_rows, int n_heads, int hdv, float eps, void* stream);
// rows [gate: f | up: f] -> min(gate, limit) * sigmoid(alpha * that) * (clamp(up, -limit, limit) + 1); limit <= 0: no clamps.
int gi_clamped_glu(void* out, const void* in, long ld_in, int dtype, int n_rows, int f, float limit, float alpha, void* stream);

// ---- additions to the routed feed-forward and the plain attention -------------------------------------------------------
// score_mode 2: shares = softmax over ALL experts; the `top` largest of share + correction (null: 0) are chosen; weights =
// the chosen shares / (their sum + 1e-20) * weight_scale.
int gi_moe_route_shares(int* ids, float* wts, float* sgate, const void* h, int dtype, long ldh, const void* w_router,
                        const void* w_sg, int w_dtype, int n_tokens, int width, int experts, int top, int score_mode,
                        const float* correction, float weight_scale, void* stream);
// gi_moe_gemm_gate_up with the clamped form of the gated value for limit > 0 (see gi_clamped_glu).
int gi_moe_gemm_gate_up_clamped(void* out, int dtype, const void* a, long lda, const void* w, int w_dtype, long w_stride,
                                const int* offsets, const int* perm, int entries, int top, int experts, int f, int k,
                                int interleaved, float limit, float alpha, void* stream);
// gi_attn_decode_kr_ex / gi_attn_prefill_tc_ex with a window that keeps the sequence's first `keep_first` positions visible.
int gi_attn_decode_kr_ex2(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, const void* kcache,
                          const void* vcache, const int* block_table, int max_pages, const int* seq_slots, const int* seq_lens,
                          int n_seqs, int n_heads, int n_kv, int hd, float scale, int window, int n_splits, int own_tiles, int hdv,
                          float softcap, const float* sinks, int chunk, int keep_first, void* stream);
int gi_attn_prefill_tc_ex2(void* out, long ldo, const void* q, long ldq, const void* kcache, const void* vcache,
                           const int* block_table, int max_pages, const int* cu_seqlens, const int* seq_slots,
                           const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd, float scale,
                           int window, int hdv, float softcap, const float* sinks, int chunk, int keep_first, void* stream);
int gi_attn_prefill_t5_ex2(void* out, long ldo, const void* q, long ldq, long q_rows, long q_cols, const void* kcache,
                           const void* vcache, long cache_pages, const int* block_table, int max_pages, const int* cu_seqlens,
                           const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads, int n_kv, int hd,
                           float scale, int window, float softcap, const float* sinks, int chunk, int keep_first, void* stream);
// gi_clamped_glu over rows whose gate and up columns are interleaved in blocks of 8 ([8 gate | 8 up] ...), if `interleaved`.
int gi_clamped_glu_rows(void* out, const void* in, long ld_in, int dtype, int n_rows, int f, float limit, float alpha, int interleaved,
                        void* stream);
// gi_gemm_stream_bf16's gated mode with the clamped form of the gated value (a product of up to 64 rows).
int gi_gemm_stream_bf16_clamped(void* out, const void* A, const void* W, float* scratch, int* counters, int n_counters, int M, int N,
                                int K, long lda, long ldw, long ldo, float limit, float alpha, void* stream);
// gi_gemm_tc_bf16's gated mode with the clamped form of the gated value (see gi_clamped_glu); W's gate and up rows interleaved
// in blocks of 8.  And a prompt step's clamped gated experts through it, stretch by stretch (see gi_moe_experts_tc).
int gi_gemm_tc_bf16_clamped(void* out, const void* A, const void* W, int M, int N, int K, long lda, long ldw, long ldo, int tile_n,
                            float limit, float alpha, void* stream);
int gi_moe_experts_tc_clamped(float* out, void* hidden, const void* rows, const void* w_gate_up, long gate_up_stride,
                              const void* w_down, long down_stride, const int* host_offsets, int experts, int width, int f,
                              float limit, float alpha, float* scratch, int* counters, int n_counters, void* stream);
// The plain attention kernels with a window that keeps the sequence's first `keep_first` positions visible as well.
int gi_attn_prefill_generic_ex3(void* out, long ldo, const void* q, long ldq, int dtype, const void* kcache,
                                const void* vcache, const int* block_table, int max_pages, const int* cu_seqlens,
                                const int* seq_slots, const int* seq_pos0, int n_seqs, int max_q_len, int n_heads,
                                int n_kv, int hd, float scale, int window, int hdv, float softcap, const float* sinks,
                                int chunk, long v_row_stride, int keep_first, void* stream);
int gi_attn_decode_generic_ex3(void* out, long ldo, float* part_o, float* part_ml, const void* q, long ldq, int dtype,
                               const void* kcache, const void* vcache, const int* block_table, int max_pages,
                               const int* seq_slots, const int* seq_lens, int n_seqs, int n_heads, int n_kv, int hd,
                               float scale, int window, int n_splits, int own_tiles, int hdv, float softcap,
                               const float* sinks, int chunk, long v_row_stride, int keep_first, void* stream);

#ifdef __cplusplus
}
#endif
