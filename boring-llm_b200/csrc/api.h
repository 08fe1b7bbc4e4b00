// C interface of the kernel library. Every function returns 0 on success; otherwise
// bl_last_error() describes what was refused or what failed. Pointers are device pointers
// unless a comment says otherwise; `stream` is a cudaStream_t.
#pragma once
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

const char* bl_last_error(void);
int bl_device_check(void);   // 0 when the current device can run this library (compute capability 10.x)

// out[t, :] = table[ids[t], :] as 32-bit floats (the residual stream).
int bl_embed(const void* table, int table_dtype, const int* ids, float* out,
             int T, int d, int vocab, void* stream);

// y[r, :] = x[row_idx ? row_idx[r] : r, :] / sqrt(mean(x^2) + eps) * w, statistics in 32-bit.
int bl_rmsnorm(const float* x, const int* row_idx, const void* w, int w_dtype, void* y, int y_dtype,
               int rows, int d, float eps, void* stream);

// Plain matrix product on CUDA cores, 32-bit accumulation in ascending k for every output element:
// out[M, N] = epilogue(x[M, K] . W[N, K]^T). For BL_EPI_SWIGLU W has 2N rows (gate, then up), and `bias`, which that epilogue
// does not add, may point to two 32-bit numbers {kind, limit} on the device that name the gated activation (BL_GLU_* of
// common.cuh; null: SiLU). The same holds for every product below that takes a bias and this epilogue.
int bl_gemm_plain(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias, int bias_dtype,
                  void* out, int out_dtype, int M, int N, int K, int epilogue, void* stream);

// Splits rows of joined [q | k | v] projections, rotates q and k by position (inside each head, pair j is
// (j, j + n_rot/2) for pair_layout 0 and (2j, 2j + 1) for pair_layout 1; angle = float(position) * inv_freq[j],
// cos and sin times mscale) and writes k and v into the pages of the token's request. k_cache/v_cache may be
// null: then only q is produced.
int bl_rope_kv_write(const float* qkv, const int* positions, const int* tok_req, const int* block_table,
                     int max_pages, const float* inv_freq, int rot_half, float mscale,
                     void* q_out, void* k_cache, void* v_cache, int dtype,
                     int T, int H, int KV, int dh, int page_size, int pair_layout, void* stream);

// Plain paged causal attention: one warp per (token, head), keys visited in ascending position.
// Token t of request r = tok_req[t] stands at position ctx_len[r] - (cu_q[r+1] - cu_q[r]) + (t - cu_q[r])
// and sees keys j <= position with j + window > position (window 0: all of them).
int bl_attention_plain(const void* q, const void* k_cache, const void* v_cache, int dtype,
                       const int* tok_req, const int* cu_q, const int* ctx_len, const int* block_table,
                       int max_pages, void* out, int T, int H, int KV, int dh, int page_size,
                       int window, float scale, void* stream);

// x[r, :] += v[:] for every row of the 32-bit residual stream (the bias of a projection that adds into it).
int bl_add_row_vector(float* x, const void* v, int v_dtype, int rows, int d, void* stream);

// out_ids[r] = index of the first maximum of logits[r, :].
int bl_argmax(const float* logits, int* out_ids, int rows, int vocab, void* stream);

// One token per row: greedy where temperature[r] <= 0, else temperature sampling with the optional
// top_k (0: off), top_p (>= 1: off) and min_p (0: off) cuts over candidates in descending logit order;
// uniform[r] in [0, 1) is the row's random number (unused by greedy rows).
int bl_sample(const float* logits, int rows, int vocab, const float* temperature, const int* top_k,
              const float* top_p, const float* min_p, const float* uniform, int* out_ids, void* stream);

// logits[r, t] is divided by penalty[r] when positive, multiplied otherwise, for each token t in
// tokens[offsets[r] .. offsets[r+1]) (the host lists each distinct token once).
int bl_repeat_penalty(float* logits, int rows, int vocab, const int* tokens, const int* offsets,
                      const float* penalty, void* stream);

// Matrix product for few rows (decode): bfloat16 x[M, K] and W[N, K] read once from global memory straight
// into tensor-core registers. K must be a multiple of 8, x and W 16-byte aligned. Same epilogues as bl_gemm_plain.
int bl_gemm_skinny(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                   int M, int N, int K, int epilogue, void* stream);
int bl_gemm_skinny_norm_parts(int N);
int bl_gemm_skinny_residual_norm(const void* x, const void* w, void* out, int M, int N, int K, const void* norm_w,
                                 int norm_w_dtype, void* hw, float* ss, void* stream);
int bl_gemm_skinny_scaled(const void* hw, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                          int M, int N, int K, int epilogue, const float* ss, int parts, float eps, void* stream);

// Tensor-core paged attention (bfloat16, pages of 16 tokens, head sizes 16/32/48/64/96/128).
int bl_attention_mma_supported(int dh, int page_size);
// Prefill shape: tiles[n_tiles][2] = (request, first token of a 64-token tile within the request's new tokens).
int bl_attention_prefill(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                         const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                         void* out, int H, int KV, int dh, int page_size, int window, float scale, void* stream);
// The same on tcgen05 tensor cores with TMA-fed tiles and scores and outputs in tensor memory (attention_tcgen05.cu):
// head size 64 and pages of 16 only. tiles[n_tiles][2] = (request, first token of a 128-row tile). T: rows of
// q and out; n_pages: pages in k_cache / v_cache. *status = 0 unless a block gave up on a bounded wait since the last
// call (synchronises the device).
int bl_attention_prefill_tc_supported(int dh, int page_size);
int bl_attention_prefill_tc(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                            const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                            void* out, int T, int n_pages, int H, int KV, int dh, int page_size, int window, float scale,
                            void* stream);
int bl_attention_prefill_tc_status(int* status);
// Blocks of bl_attention_decode that the current device holds at once for this head size (0: not built).
int bl_attention_decode_resident_blocks(int dh);
// Decode shape: reqs[n] = requests with one new token; their keys are cut into n_splits slices. With scratch == null
// (up to 16 slices) the slices of a request are the blocks of one thread-block cluster and merge their partial results
// through distributed shared memory; with scratch (up to 256 slices) the last block to finish merges them from
// scratch: bl_attention_decode_scratch_floats(n, H, dh, n_splits) floats (none for one slice).
long long bl_attention_decode_scratch_floats(int n, int H, int dh, int n_splits);
// counters: n * KV * ceil((H / KV) / 16) ints that are zero at the call and zero again when it is done.
int bl_attention_decode(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                        const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                        int n_splits, float* scratch, int* counters, void* out, int H, int KV, int dh, int page_size,
                        int window, float scale, void* stream);

// The decode shape with TMA-fed rings (attention_decode.cu): head sizes 64 and 128, pages of 16, 1..16 slices that are
// the blocks of one cluster; the MMAs' columns are the query heads of a key/value head (8 or 16 a block). n_pages:
// pages in k_cache / v_cache. early != 0: the launch may start under its predecessor's tail (programmatic dependent
// launch). *status = 0 unless a warp gave up on a bounded wait since the last call (synchronises
// the device). resident_blocks: blocks the device holds at once for this head size and heads per key/value head.
int bl_attention_decode_tma_supported(int dh, int page_size);
int bl_attention_decode_tma_resident_blocks(int dh, int heads_per_kv);
// Clusters of `cluster` blocks that the device runs at once for this shape (0: cannot be launched).
int bl_attention_decode_tma_max_clusters(int dh, int heads_per_kv, int cluster);
int bl_attention_decode_tma(const void* q, const void* k_cache, const void* v_cache, int n_pages, const int* cu_q,
                            const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                            int n_splits, void* out, int H, int KV, int dh, int page_size, int window, float scale,
                            int early, void* stream);
int bl_attention_decode_tma_status(int* status);

// cs[t, j] = cos(positions[t] * inv_freq[j]) * mscale, sn likewise, j < rot_half: the rotation of a step's tokens,
// worked out once for all layers.
int bl_rope_table(const int* positions, const float* inv_freq, int rot_half, float mscale, float* cs, float* sn, int T,
                  void* stream);
// The joined q/k/v product on pairs of SMs (gemm_tcgen05_pair.cu) with bias, rotation (pairs j, j + dh / 2; cs, sn:
// [M, dh / 2] from bl_rope_table) and the writes of q and of k and v into the pages of each token's request folded
// into its epilogue. Head size 64 or 128, pages of 16; null caches: nothing is cached; bias may be null.
int bl_gemm_tc_pair_qkv_rope_supported(int H, int KV, int dh, int page_size, int K);
// ss != null: x holds rows whose RMS norm is pending (bl_gemm_tc_pair_residual_norm); row m of the product is scaled
// by 1 / sqrt(sum(ss[m, :parts]) * inv_dim + eps) before the bias.
int bl_gemm_tc_pair_qkv_rope(const void* x, const void* w, const void* bias, int bias_dtype, int M, int K,
                             const int* tok_req, const int* positions, const int* block_table, int max_pages,
                             const float* cs, const float* sn, void* q_out, void* k_cache, void* v_cache,
                             int H, int KV, int dh, int page_size, const float* ss, int parts, float inv_dim, float eps,
                             void* stream);
// An RMS norm between two products without a pass of its own: the product that adds into the 32-bit residual stream
// also writes hw = bfloat16(out * norm_w) and per-row sums of squares by tile (ss[M, bl_gemm_tc_pair_norm_parts(M, N)]);
// the products that read the normed rows take hw and scale their accumulator rows by the row's 1 / sqrt(mean + eps).
int bl_gemm_tc_pair_norm_parts(int M, int N);
int bl_gemm_tc_pair_residual_norm(const void* x, const void* w, void* out, int M, int N, int K, const void* norm_w,
                                  int norm_w_dtype, void* hw, float* ss, void* stream);
int bl_gemm_tc_pair_swiglu_scaled(const void* hw, const void* w, void* out, int M, int N, int K, const float* ss,
                                  int parts, float inv_dim, float eps, void* stream);

// Matrix product for many rows (prefill) on tcgen05 tensor cores with TMA-fed shared-memory tiles and the
// accumulator in tensor memory. bfloat16 x[M, K] and W[N, K]; K a multiple of 8, x and W 16-byte aligned.
int bl_gemm_tc(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
               int M, int N, int K, int epilogue, void* stream);
// *status = 0 unless a block of bl_gemm_tc gave up on a bounded wait since the last call (synchronises the device).
int bl_gemm_tc_status(int* status);

// Few rows (up to 64) times very many columns (an output head), no epilogue: W is the M side of tcgen05.mma and
// streams through a deep TMA ring once, x stays in shared memory, blocks are persistent (gemm_tcgen05_cols.cu).
int bl_gemm_tc_cols_supported(int M, int N, int K);
int bl_gemm_tc_cols(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, void* stream);
int bl_gemm_tc_cols_status(int* status);

// Fused kernels for steps with few rows (decode_fused.cu): the RMS norm in front of a product, and the split,
// rotation and cache write behind the q/k/v product, folded into the product.
int bl_norm_gemm_supported(int K);
int bl_norm_gemm(const float* x, const int* row_idx, const void* norm_w, int norm_w_dtype, float eps,
                 const void* w, const void* bias, int bias_dtype, void* out, int M, int N, int K,
                 int epilogue, void* stream);
int bl_norm_qkv_rope(const float* x, const void* norm_w, int norm_w_dtype, float eps, const void* w_qkv,
                     const void* bias, int bias_dtype, const int* positions, const int* tok_req,
                     const int* block_table, int max_pages, const float* inv_freq, float mscale,
                     void* q_out, void* k_cache, void* v_cache, int M, int K, int H, int KV, int dh,
                     int page_size, int pair_layout, void* stream);
// Programmatic dependent launch for the small kernels of a step (on by default): 0 launches them the ordinary way.
void bl_set_dependent_launch(int on);

// Writes the GPU's nanosecond timer to buf[slot] once everything before it on the stream has finished.
int bl_stamp(unsigned long long* buf, int slot, void* stream);

// The same product on pairs of SMs (tcgen05 cta_group::2, clusters of two blocks, 256 x 256 tiles): twice the
// arithmetic per byte loaded into shared memory. Same contract as bl_gemm_tc.
int bl_gemm_tc_pair(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                    int M, int N, int K, int epilogue, void* stream);
int bl_gemm_tc_pair_status(int* status);

// The same product for shapes with few output tiles: a cluster of up to eight blocks shares a tile of 128 rows and
// cuts K among its blocks; the partial tiles are added up in block order through distributed shared memory
// (gemm_tcgen05_splitk.cu). Same contract as bl_gemm_tc. bl_gemm_tc_splitk_split: how many blocks would share a tile
// (1: K is not cut, the kernel has nothing over bl_gemm_tc).
int bl_gemm_tc_splitk_split(int M, int N, int K, int epilogue);
int bl_gemm_tc_splitk(const void* x, const void* w, const void* bias, int bias_dtype, void* out, int out_dtype,
                      int M, int N, int K, int epilogue, void* stream);
int bl_gemm_tc_splitk_status(int* status);

// The tensor-core attention kernels with what may follow the softmax: sinks[H] (null: none), a learned score per head
// whose exponential joins the denominator once, unscaled, without a value (the slices of a decode row count it once, at
// their merge); gate (null: none), 32-bit logits with rows ld_gate apart: head h of token t is multiplied by
// sigmoid(gate[t * ld_gate + h]). Otherwise as the functions without `_tail`.
int bl_attention_prefill_tail(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                              const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                              void* out, int H, int KV, int dh, int page_size, int window, float scale,
                              const void* sinks, int sink_dtype, const float* gate, int ld_gate, void* stream);
int bl_attention_prefill_tc_tail(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                 const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                                 void* out, int T, int n_pages, int H, int KV, int dh, int page_size, int window, float scale,
                                 const void* sinks, int sink_dtype, const float* gate, int ld_gate, void* stream);
int bl_attention_decode_tail(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                             const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                             int n_splits, float* scratch, int* counters, void* out, int H, int KV, int dh, int page_size,
                             int window, float scale, const void* sinks, int sink_dtype, const float* gate, int ld_gate,
                             void* stream);
// The tcgen05 prompt kernel, the TMA-fed decode kernel and the `mma.sync` kernels with a cap c > 0 on the scaled scores as well, s <- c tanh(s / c), before the softmax (0: none).
int bl_attention_prefill_cap(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                             const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                             void* out, int H, int KV, int dh, int page_size, int window, float scale,
                             const void* sinks, int sink_dtype, const float* gate, int ld_gate, float softcap, void* stream);
int bl_attention_prefill_tc_cap(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                                const int* ctx_len, const int* block_table, int max_pages, const int* tiles, int n_tiles,
                                void* out, int T, int n_pages, int H, int KV, int dh, int page_size, int window, float scale,
                                const void* sinks, int sink_dtype, const float* gate, int ld_gate, float softcap, void* stream);
int bl_attention_decode_tma_cap(const void* q, const void* k_cache, const void* v_cache, int n_pages, const int* cu_q,
                                const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                                int n_splits, void* out, int H, int KV, int dh, int page_size, int window, float scale,
                                int early, const void* sinks, int sink_dtype, const float* gate, int ld_gate, float softcap,
                                void* stream);
int bl_attention_decode_cap(const void* q, const void* k_cache, const void* v_cache, const int* cu_q,
                            const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                            int n_splits, float* scratch, int* counters, void* out, int H, int KV, int dh, int page_size,
                            int window, float scale, const void* sinks, int sink_dtype, const float* gate, int ld_gate,
                            float softcap, void* stream);
int bl_attention_decode_tma_tail(const void* q, const void* k_cache, const void* v_cache, int n_pages, const int* cu_q,
                                 const int* ctx_len, const int* block_table, int max_pages, const int* reqs, int n,
                                 int n_splits, void* out, int H, int KV, int dh, int page_size, int window, float scale,
                                 int early, const void* sinks, int sink_dtype, const float* gate, int ld_gate, void* stream);

// The plain product with rows of x that are `ldx` values apart (a column range of a wider matrix as the input).
int bl_gemm_plain_ld(const void* x, int x_dtype, int ldx, const void* w, int w_dtype, const void* bias, int bias_dtype,
                     void* out, int out_dtype, int M, int N, int K, int epilogue, void* stream);

// bl_attention_plain with options: values of head size dv (keys and queries: dh); sinks[H] (null: none): exp(sinks[h])
// joins head h's softmax denominator once, unscaled, without a value; gate (null: none): head h of token t is
// multiplied by sigmoid(gate[t * ld_gate + h]). out: [T, H * dv].
int bl_attention_plain_ext(const void* q, const void* k_cache, const void* v_cache, int dtype,
                           const int* tok_req, const int* cu_q, const int* ctx_len, const int* block_table,
                           int max_pages, void* out, int T, int H, int KV, int dh, int dv, int page_size, int window,
                           float scale, const void* sinks, int sink_dtype, const float* gate, int ld_gate, void* stream);
// ... and a cap c > 0 on the scores: s <- c tanh(s / c) on the scaled score, before the softmax (0: none).
int bl_attention_plain_cap(const void* q, const void* k_cache, const void* v_cache, int dtype,
                           const int* tok_req, const int* cu_q, const int* ctx_len, const int* block_table,
                           int max_pages, void* out, int T, int H, int KV, int dh, int dv, int page_size, int window,
                           float scale, const void* sinks, int sink_dtype, const float* gate, int ld_gate, float softcap, void* stream);

// y[r, :] = (x[src, :] - mean) / sqrt(var + eps) * w + b (b may be null), src = row_idx ? row_idx[r] : r; var is the
// mean of the squared deviations; statistics in 32-bit.
int bl_layernorm(const float* x, const int* row_idx, const void* w, int w_dtype, const void* b, int b_dtype,
                 void* y, int y_dtype, int rows, int d, float eps, void* stream);
// x[r, :] += layer norm(sub[r, :] * sigmoid(gate[r * ld_gate + :] + gate_bias[:])) * w + b: a gate on a sublayer's
// result, the norm behind the sublayer and the residual sum. gate, gate_bias and b may be null.
int bl_gated_norm_residual(float* x, const float* sub, const float* gate, int ld_gate, const void* gate_bias, int gb_dtype,
                           const void* w, int w_dtype, const void* b, int b_dtype, int rows, int d, float eps, void* stream);
// Up to three row-wise steps in one launch, each optional (null pointers leave a step out), for widths that
// bl_norm_chain_supported takes and 16-byte aligned operands: A (sub != null) x += layer norm(sub * sigmoid(gate +
// gate_bias)) * w + b; B (streams != null) mix_out = sum_{j < n - 1} coeffs[j] * streams[j] + coeffs[n - 1] * row, the row
// being stream n - 1 (x); C (w2 != null) y = layer norm(row) * w2 + b2. Bit for bit what the three kernels give.
int bl_norm_chain_supported(int d, int ld_gate);
int bl_norm_chain(float* x, const float* sub, const float* gate, int ld_gate, const void* gate_bias, int gb_dtype,
                  const void* w, int w_dtype, const void* b, int b_dtype, float eps, const float* streams, long long stride,
                  const void* coeffs, int c_dtype, int n, float* mix_out, const void* w2, int w2_dtype, const void* b2,
                  int b2_dtype, float eps2, void* y, int y_dtype, int rows, int d, void* stream);
// out[e] = sum_{j < n} coeffs[j] * streams[j * stride + e], e < count.
int bl_depth_mix(const float* streams, long long stride, const void* coeffs, int c_dtype, int n, float* out,
                 long long count, void* stream);
// y[r, c] = act(x[r, c]) for r < rows, c < cols; rows ld_x and ld_y values apart (y may be x).
#define BL_ACT_SILU 0
#define BL_ACT_GELU_ERF 1
#define BL_ACT_GELU_TANH 2
int bl_activation(const void* x, int x_dtype, long long ld_x, void* y, int y_dtype, long long ld_y, int rows, int cols,
                  int act, void* stream);

// Rows proj[T, ld] hold a token's joined projections: q in columns 0 .. H * dk, k from off_k (KV * dk), v from off_v
// (KV * dv). RMS norm of the whole q row and of the whole k row (weights q_norm_w [H * dk], k_norm_w [KV * dk]; null:
// no norm), rotation of the first 2 * rot_half dimensions of every head by angle float(position) * inv_freq[j], q to
// q_out [T, H * dk], k and v into the pages of the token's request (null caches: not written).
int bl_qk_norm_rope_write(const float* proj, int ld, int off_k, int off_v, const void* q_norm_w, int qw_dtype,
                          const void* k_norm_w, int kw_dtype, float eps, const int* positions, const int* tok_req,
                          const int* block_table, int max_pages, const float* inv_freq, int rot_half, int pair_layout,
                          void* q_out, void* k_cache, void* v_cache, int dtype, int T, int H, int KV, int dk, int dv,
                          int page_size, void* stream);

// Linear recurrences over a matrix state per head kept in state slots (recurrent.cu). Request r owns tokens
// cu_q[r] .. cu_q[r + 1] - 1 and the slot slots[r]; its state S [H, dk, dv] starts at state + slots[r] * slot_stride.
// q, k: [T, G * dk] (query/key head of head h: h / (H / G)), v: [T, H * dv], a: [T, H * dk] (the decays, see
// bl_gemm_plain_decay), beta: [T, H] logits (delta rule only), each with its own row stride; out: [T, H * dv] 32-bit.
#define BL_RULE_GLA 0      // S <- diag(a) S + k v^T; o = S^T (q * q_scale)
#define BL_RULE_DELTA 1    // S <- diag(a) S; u = sigmoid(beta) (v - S^T k); S <- S + k u^T; o = S^T (q * q_scale)
#define BL_RULE_BONUS 2    // o = (S^T q + beta v) * q_scale; S <- diag(a) S + k v^T  (the read-out sees the state BEFORE the token's write; beta: a given number per token and head)
int bl_gemm_plain_decay(const float* x, int ldx, const void* w, int w_dtype, const void* bias, int bias_dtype,
                        float* out, int M, int N, int K, const float* coef, int group, float sign, void* stream);
int bl_recurrent_scan(int rule, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                      const float* a, int lda, const float* beta, int ldb, float q_scale, float* state, long long slot_stride, const int* slots, const int* cu_q, int R,
                      float* out, int H, int G, int dk, int dv, void* stream);
// The same with long portions cut into nc parts that run side by side (requests with 256 tokens or more in the step;
// linear attention with key sizes that bl_recurrent_scan_can_split takes): every part first runs from a zero state, then
// from the request's state folded through the parts before it, and a fold leaves the slot (the delta rule's fold, a
// product with the part's key x key transition, runs between the passes). scratch: bl_recurrent_scan_parts_scratch
// floats. nc 1: bl_recurrent_scan.
long long bl_recurrent_scan_parts_scratch(int rule, int R, int nc, int H, int dk, int dv);
int bl_recurrent_scan_can_split(int rule, int H, int dk, int dv);   // 0, or the blocks one request's portion runs on
int bl_recurrent_scan_parts(int rule, const float* q, int ldq, const float* k, int ldk, const float* v, int ldv,
                            const float* a, int lda, const float* beta, int ldb, float q_scale, float* state,
                            long long slot_stride, const int* slots, const int* cu_q, int R, float* out, int H, int G,
                            int dk, int dv, int nc, float* scratch, void* stream);
// y[t, h, :] = o[t, h, :] / sqrt(mean(o^2) + eps) * w[:] * gate(g[t * ld_gate + h * dv + :]) (gate null: none).
#define BL_GATE_SIGMOID 0
#define BL_GATE_SILU 1
int bl_head_norm_gate(const float* o, const void* w, int w_dtype, const float* gate, int ld_gate, int gate_kind,
                      void* y, int y_dtype, int T, int H, int dv, float eps, void* stream);
// y[t, ch] = silu(sum_i taps[ch, i] * x[t - (n_taps - 1) + i, ch]) over a request's tokens, the inputs before the
// step's first token taken from the slot's tail [n_taps - 1, C] (oldest first); then heads 0 .. unit_heads - 1 of dk
// columns become unit vectors (x / sqrt(sum x^2 + unit_eps)), the first scaled_heads of them times q_scale.
int bl_conv_silu_unit(const float* x, int ld, const float* taps, int n_taps, const float* tail, long long slot_stride,
                      const int* slots, const int* tok_req, const int* cu_q, float* y, int T, int C, int unit_heads,
                      int scaled_heads, int dk, float q_scale, float unit_eps, void* stream);
// bl_conv_silu_unit with a bias per channel (null: none) that each channel's sum starts from.
int bl_conv_silu_unit_bias(const float* x, int ld, const float* taps, int n_taps, const float* tail, long long slot_stride,
                           const int* slots, const int* tok_req, const int* cu_q, float* y, int T, int C, int unit_heads,
                           int scaled_heads, int dk, float q_scale, float unit_eps, const void* bias, int bias_dtype, void* stream);
// In front of a recurrence with a fixed decay per head: q (columns 0 ..) and k (from off_k) of proj rotated by position
// (pairs (i, i + rot_half) of each head's first 2 * rot_half values), k times k_scale, decay_out[t, h, :] = head_decay[h].
int bl_rope_decay_prep(const float* proj, int ld, int off_k, const int* positions, const float* inv_freq, int rot_half,
                       const float* head_decay, float k_scale, float* q_out, float* k_out, float* decay_out, int T, int H, int dk,
                       void* stream);
// In front of a selective state-space recurrence: dt = softplus(raw[t, h] + dt_bias[h]); decay_out[t, h, :n_state] =
// exp(-rate[h] * dt); v_out[t, h, :] = dt * x[t, h, :].
int bl_ssd_prep(const float* raw, int ld_raw, const void* dt_bias, int bias_dtype, const float* rate, const float* x, int ld_x,
                float* decay_out, float* v_out, int T, int H, int n_state, int dv, void* stream);
// y = rms_norm_in_parts((o + skip[c / dv] * x) * silu(z)) * w: the gate in front of the norm, n_parts equal parts of a row of
// `width` values each normed by its own root mean square. x / skip, z and w may be null.
int bl_gated_group_norm(const float* o, const float* x, int ld_x, const void* skip, int skip_dtype, int dv, const float* z, int ld_z,
                        const void* w, int w_dtype, void* y, int y_dtype, int T, int width, int n_parts, float eps, void* stream);
// The tail of every request with tokens becomes its last n_taps - 1 inputs (after bl_conv_silu_unit has read it).
int bl_conv_tail_update(const float* x, int ld, int n_taps, float* tail, long long slot_stride, const int* slots,
                        const int* cu_q, int R, int C, void* stream);

// bl_head_norm_gate with options: the heads of a row of o lie o_head_stride values apart; w_per_head != 0: w holds H * dv
// values (a weight per head and channel); floor (null: none) [T, H]: o[t, h, :dv] is divided by
// max(|o[t, h, dv]|, floor[t, h]) + 1e-6 before the norm (o_head_stride >= dv + 1).
int bl_head_norm_gate_ext(const float* o, int o_head_stride, const void* w, int w_dtype, int w_per_head, const float* floor,
                          const float* gate, int ld_gate, int gate_kind, void* y, int y_dtype, int T, int H, int dv, float eps,
                          void* stream);
// The gates of a matrix memory with exponential gating, the tokens of each request in order. proj [T, ld] holds k at
// off_k (H * dk), v at off_v (H * dv) and the gates' pre-activations at off_i and off_f (H each). Per token and head:
// i = cap tanh((zi + bias_i) / cap), f = log sigmoid(cap tanh((zf + bias_f) / cap)), m' = max(f + m, i) (m [H] is kept in
// the request's slot at off_m floats from its start; a zeroed slot is the start of a sequence), a = e^(f + m - m'),
// e = e^(i - m'). gates [3, T, H]: a, e, e^(-m'). What bl_recurrent_scan (BL_RULE_GLA, value size dv + 1) then reads:
// decay [T, H * dk] = a for every key channel, k_out [T, H * dk] = e k, v_out [T, H * (dv + 1)] = (v, 1): the state's last
// value column is the normaliser n' = a n + e k, the read-out's last column n' . q.
int bl_memory_gates(const float* proj, int ld, int off_k, int off_v, int off_i, int off_f, const void* bias_i, int bi_dtype,
                    const void* bias_f, int bf_dtype, float cap, float* state, long long slot_stride, long long off_m,
                    const int* slots, const int* cu_q, int R, int T, float* gates, float* decay, float* k_out, float* v_out,
                    int H, int dk, int dv, void* stream);
// out[s, t, :] = x[t, :] + (x'[t, :] - x[t, :]) * mu[s, :] (mu 32-bit [n_mix, d]), s < n_mix, x' the row of the request's token before; for a
// step's first token of a request it is prev + slots[r] * slot_stride [d] (bl_conv_tail_update with two taps keeps it).
int bl_shift_mix(const float* x, int ld, const float* mu, int n_mix, const float* prev, long long slot_stride,
                 const int* slots, const int* tok_req, const int* cu_q, void* out, int out_dtype, int T, int d, void* stream);
// out[t, h] = sum_c u[h, c] * k[t, h, c] * q[t, h, c] (the beta of BL_RULE_BONUS for a bonus per head and key channel).
int bl_bonus_dot(const float* q, int ldq, const float* k, int ldk, const void* u, int u_dtype, float* out, int T, int H, int dk,
                 void* stream);

// bl_qk_norm_rope_write with the norm's scope as an argument: per_head 0: one RMS norm over a token's whole q row (weights
// [H * dk]) and one over its whole k row ([KV * dk]); per_head != 0: a norm over each head's dk values, the weights [dk]
// shared by the heads. q_head_scale (null: none): 32-bit [H], head h of q is multiplied by q_head_scale[h] as it is written
// (a factor per head on the scores, of either sign, costs the attention kernels nothing this way).
int bl_qk_norm_rope_write_scope(const float* proj, int ld, int off_k, int off_v, const void* q_norm_w, int qw_dtype,
                                const void* k_norm_w, int kw_dtype, float eps, int per_head, const int* positions,
                                const int* tok_req, const int* block_table, int max_pages, const float* inv_freq,
                                int rot_half, int pair_layout, void* q_out, void* k_cache, void* v_cache, int dtype, int T,
                                int H, int KV, int dk, int dv, int page_size, const float* q_head_scale, void* stream);
// out[m, n] = exp(-exp(u[m, :] . W[n, :] + bias[n])), u = tanh(x) where x_tanh != 0 (x: 32-bit rows ldx apart).
int bl_gemm_plain_decay_exp(const float* x, int ldx, int x_tanh, const void* w, int w_dtype, const void* bias, int bias_dtype,
                            float* out, int M, int N, int K, void* stream);

// Layers with the norm behind the sublayer (post_norm.cu): x += LN(s) * w (no bias), s = a, or, with b != null,
// s = (a / rms(a) * wa + b / rms(b) * wb) / 2 (rms with rms_eps inside the root); y (null: none): the new rows of x in
// y_dtype as well. bl_cast_rows: y = x in y_dtype. bl_softcap: x = cap * tanh(x / cap) in place.
int bl_post_norm_residual(float* x, const float* a, const void* wa, int wa_dtype, const float* b, const void* wb, int wb_dtype,
                          float rms_eps, const void* w, int w_dtype, float eps, void* y, int y_dtype, int rows, int d, void* stream);
int bl_cast_rows(const float* x, void* y, int y_dtype, long long count, void* stream);
// out = (a / rms(a) * wa + b / rms(b) * wb) / 2 row by row (32-bit): the mean of two sublayer results, each RMS-normed first.
int bl_pair_rms_mean(const float* a, const void* wa, int wa_dtype, const float* b, const void* wb, int wb_dtype, float rms_eps,
                     float* out, int rows, int d, void* stream);
int bl_softcap(float* x, long long count, float cap, void* stream);
// x += ca * a + cb * b (32-bit, `count` values); x[r, :] += sigmoid(gate[r * ld_gate]) * a[r, :] (one gate logit per row).
int bl_add_scaled_pair(float* x, const float* a, float ca, const float* b, float cb, long long count, void* stream);
int bl_add_row_gated(float* x, const float* a, const float* gate, long long ld_gate, int rows, int d, void* stream);
// y = xIELU(x) on 32-bit sums, args = {softplus(p), 1/2 + softplus(q)} on the device: v > 0: args[0] v^2 + v / 2, else
// args[1] (e^v - 1 - v) + v / 2.
int bl_xielu(const float* x, long long ld_x, void* y, int y_dtype, long long ld_y, int rows, int cols, const float* args, void* stream);

// Attention over the query's own chunk of positions with the heads' softmax weights mixed afterwards (attention_talk.cu).
// Position i sees j in [i - i % chunk, i] (chunk 0: from 0; window > 0 also j > i - window); score = q . k * scale *
// head_scale[head] (null: 1). A [T, H, KV, dv] 32-bit: head g's softmax applied to the values of every key/value head;
// bl_talk_mix: out[t, h, :] = sum_g talk[h, g] A[t, g, kv(h), :].
int bl_attention_talk_plain(const void* q, const void* k_cache, const void* v_cache, int dtype, const int* tok_req,
                            const int* cu_q, const int* ctx_len, const int* block_table, int max_pages, float* A, int T, int H,
                            int KV, int dh, int dv, int page_size, int chunk, int window, float scale, const void* head_scale,
                            int hs_dtype, void* stream);
int bl_talk_mix(const void* A, int a_dtype, const void* talk, int talk_dtype, void* out, int out_dtype, int T, int H, int KV, int dv,
                void* stream);
// The same on tensor cores (attention_mma.cu: bfloat16, pages of 16, head sizes 16/32/48/64/96/128, values of the keys'
// head size, positive head_scale in 32-bit): tiles / reqs as bl_attention_prefill / bl_attention_decode (up to 16 slices,
// merged inside clusters); spread [T, H, KV, dh] bfloat16.
int bl_attention_prefill_talk(const void* q, const void* k_cache, const void* v_cache, const int* cu_q, const int* ctx_len,
                              const int* block_table, int max_pages, const int* tiles, int n_tiles, void* spread, int H, int KV,
                              int dh, int page_size, int chunk, int window, float scale, const float* head_scale, void* stream);
int bl_attention_decode_talk(const void* q, const void* k_cache, const void* v_cache, const int* cu_q, const int* ctx_len,
                             const int* block_table, int max_pages, const int* reqs, int n, int n_splits, void* spread, int H,
                             int KV, int dh, int page_size, int chunk, int window, float scale, const float* head_scale, void* stream);

// Routed experts (moe.cu). bl_moe_route: z [T, ldz] 32-bit router logits; s = sigmoid(z), choice = s + correction (null:
// none); experts in n_groups runs of neighbours, a group's score the sum of its two largest choice scores, the `keep` best
// groups stay open; ids [T, top] the `top` largest choice scores among them in descending order, wts [T, top] their s.
// bl_expert_gemm_plain: out[p, :] = epilogue(x[p / x_div, :] . W[ids[p]]^T), W[e] = w + e * expert_stride elements
// ([N, K], or [2N, K] gate rows then up rows for BL_EPI_SWIGLU, whose gated activation `act` names: {kind, limit} on the
// device, null for SiLU). bl_moe_combine: out[t, :] = (add ? out[t, :] : 0) + sum_k wts[t, k] y[t * top + k, :].
int bl_moe_route(const float* z, int ldz, const void* correction, int corr_dtype, int T, int E, int top, int n_groups, int keep,
                 int* ids, float* wts, void* stream);
int bl_expert_gemm_plain(const void* x, int x_dtype, int x_div, const void* w, int w_dtype, long long expert_stride, const int* ids,
                         void* out, int out_dtype, int P, int N, int K, int epilogue, const float* act, void* stream);
int bl_moe_combine(const float* y, const float* wts, float* out, int T, int top, int d, int add, void* stream);
// The same with further choices. bl_moe_route_ext: score_kind BL_SCORE_SIGMOID, or BL_SCORE_SOFTMAX (softmax of z over all E);
// group_top 2: a group's score is the sum of its two largest choice scores, 1: its largest. Identity experts are the expert
// numbers from n_real on: no matrix, no row in a product; the weighted sums take the token's input row x[t, :] for them.
#define BL_SCORE_SIGMOID 0
#define BL_SCORE_SOFTMAX 1
int bl_moe_route_ext(const float* z, int ldz, const void* correction, int corr_dtype, int T, int E, int top, int n_groups, int keep,
                     int* ids, float* wts, int score_kind, int group_top, void* stream);
int bl_expert_gemm_plain_some(const void* x, int x_dtype, int x_div, const void* w, int w_dtype, long long expert_stride,
                              const int* ids, void* out, int out_dtype, int P, int N, int K, int epilogue, const float* act,
                              int n_real, void* stream);
int bl_moe_combine_some(const float* y, const float* wts, float* out, int T, int top, int d, int add, const int* ids, int n_real,
                        const void* x, int x_dtype, void* stream);
int bl_moe_combine_rows_some(const float* y, const int* pos, const float* wts, float* out, int T, int top, int d, int add,
                             const void* x, int x_dtype, void* stream);
// The same on tensor cores: the pairs (token, chosen expert) are laid out expert by expert in tiles of `tile` rows
// (bl_moe_plan: pos [P] the row of each pair, row_src [max_tiles * tile] the pair of each row or -1, tile_expert
// [max_tiles] the expert of each tile or -1; max_tiles >= ceil(P / tile) + E), the tokens' rows are gathered there
// (bl_gather_rows, bfloat16 rows of a multiple of 8 values), bl_gemm_tc_grouped multiplies every tile of 128 rows by its
// expert's matrix (gemm_tcgen05.cu), and bl_moe_combine_rows adds up a token's rows y[pos[t * top + k]].
int bl_moe_plan(const int* ids, int P, int E, int tile, int max_tiles, int* pos, int* row_src, int* tile_expert, void* stream);
int bl_gather_rows(const void* x, const int* row_src, int div, void* dst, int rows, int cols, void* stream);
int bl_gemm_tc_grouped(const void* x, const void* w, void* out, int out_dtype, int M, int N, int K, int epilogue, int n_experts,
                       const int* tile_expert, const float* act, void* stream);
int bl_moe_combine_rows(const float* y, const int* pos, const float* wts, float* out, int T, int top, int d, int add, void* stream);

// ids[t, :] = table[tokens[t], :] (table [vocabulary, top] of expert numbers), wts[t, :] = 1 / top (moe.cu).
int bl_table_route(const int* table, const int* tokens, int T, int top, int* ids, float* wts, void* stream);

// out = table[ids] * scale (elementwise.cu).
int bl_embed_scaled(const void* table, int table_dtype, const int* ids, float* out, int T, int d, int vocab, float scale, void* stream);

// y[r, c] = glu(kind, x[r, c], x[r, cols + c], limit) on 32-bit sums (norm_gate.cu; the kinds are in common.cuh).
int bl_glu_act(const float* x, long long ld_x, void* y, int y_dtype, long long ld_y, int rows, int cols, int kind, float limit,
               void* stream);

// Attention over one cached latent per token (latent.cu). bl_latent_prep: per row of the joined product's 32-bit sums,
// cq = RMS norm of columns [off_q, off_q + q_rank) times q_norm_w (cq null: skipped), and into the token's page the row
// [RMS norm of columns [off_kv, off_kv + rank) times kv_norm_w | the next rot_dim columns, the first 2 * rot_half of them
// rotated in pairs (j, j + rot_half) by float(position) * inv_freq[j], cos and sin times mscale] (cache null: skipped);
// cache [pages, page_size, rank + rot_dim]. bl_head_gemm_plain: out[t, h, n] = sum_k x[t, h, k] W[h][n, k] (* sigmoid(gate[t, h * N + n])),
// every operand by its strides in elements. bl_rope_heads: out[t, h, out_off + .] = q[t, h, off + .] (n values, the
// first 2 * rot_half rotated); with n_lead > 0 also lead_out[t, h, .] = lead[t, h, .] (n_lead values of every head, `lead` strided as q,
// lead_out of out's dtype with strides of its own).
// bl_latent_attention_plain: q [T, H, dk], out [T, H, dv]: softmax over the visible cached rows (window 0: all) of
// q . row * scale with an optional sink per head in the denominator, applied to the rows' first dv values.
int bl_latent_prep(const float* proj, int ld, int off_q, int q_rank, int off_kv, int rank, int rot_dim, int rot_half, const void* q_norm_w,
                   int qw_dtype, const void* kv_norm_w, int kw_dtype, float eps, const int* positions, const int* tok_req,
                   const int* block_table, int max_pages, int page_size, const float* inv_freq, float mscale, void* cq, void* cache,
                   int dtype, int T, void* stream);
int bl_head_gemm_plain(const void* x, int x_dtype, long long ldx, long long x_head, const void* w, int w_dtype, long long w_head,
                       long long w_n, long long w_k, void* out, int out_dtype, long long ld_out, long long out_head, int T, int H,
                       int N, int K, const float* gate, long long ld_gate, void* stream);
int bl_rope_heads(const float* q, long long ld, long long head_stride, int off, const int* positions, const float* inv_freq,
                  int n, int rot_half, float mscale, void* out, int out_dtype, long long ld_out, long long out_head, int out_off, int T,
                  int H, const float* lead, int n_lead, void* lead_out, long long ld_lead, long long lead_head, void* stream);
int bl_latent_attention_plain(const void* q, const void* cache, int dtype, const int* tok_req, const int* cu_q, const int* ctx_len,
                              const int* block_table, int max_pages, void* out, int T, int H, int dk, int dv, int page_size,
                              int window, float scale, const void* sinks, int sink_dtype, void* stream);

// The same attention on tensor cores (latent_mma.cu): queries q_lat [H, Tp, rank] and q_rot [H, Tp, rot] and the result out
// [H, Tp, rank] lie head-major, bfloat16; `work` is the step's list of 64-token tiles [n][2] (request, first token) of
// requests with several new tokens, or, with `single`, the list [n] of requests with one; those may cut their keys into
// n_splits slices (a block each) that meet in part_o [n * H, n_splits, rank] and part_ml [n * H, n_splits, 2] and a merge kernel.
int bl_latent_attention_mma_supported(int rank, int rot, int page_size);
int bl_latent_attention_mma(const void* q_lat, const void* q_rot, const void* cache, const int* cu_q, const int* ctx_len,
                            const int* block_table, int max_pages, const int* work, int n_work, int single, void* out, int H, int Tp,
                            int rank, int rot, int page_size, int window, float scale, const void* sinks, int sink_dtype, int n_splits,
                            float* part_o, float* part_ml, void* stream);
// tile[i] = i / per for n_heads * per tiles; out[t, h * N + n] = hv[h, t, n] (* sigmoid(gate[t, h * N + n])) with hv [H, Tp, N] (latent.cu).
int bl_head_tiles(int* tile, int n_heads, int per, void* stream);
int bl_heads_gate_rows(const float* hv, const float* gate, long long ld_gate, void* out, int out_dtype, int T, int H, int N, int Tp,
                       void* stream);

#ifdef __cplusplus
}
#endif
