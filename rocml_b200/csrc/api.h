// The C interface of the kernel library.  Every function launches on `stream` and returns 0,
// a cudaError_t value, or one of the RB_ERR_* codes of common.cuh; nothing here allocates.
// Element type codes: 0 = float32, 1 = bfloat16.
#pragma once
#ifdef __cplusplus
extern "C" {
#endif

int rb_embedding(const int* ids, const void* table, int table_dtype, float* out, int T, int H, int vocab,
                 int* status, void* stream);

int rb_add_rmsnorm(float* resid, const float* delta, int n_delta, long long delta_stride, const void* w,
                   int w_dtype, void* out, int out_dtype, const int* rows, int n_rows, int H, float eps,
                   int write_back, const void* w2, void* out2, const float* delta_b, int n_delta_b,
                   long long delta_b_stride, void* stream);

int rb_silu_mul(const void* in, int in_dtype, int n_in, long long in_stride, void* out, int out_dtype, int rows,
                int I, int paired, void* stream);

// Embedding rows times `scale` plus, when inv_freq is given, a sinusoid position vector (even entries sine, odd
// cosine of positions[t] * inv_freq[i / 2]); `copy` (optional) receives the same rows.
int rb_embedding_pos(const int* ids, const void* table, int table_dtype, float* out, float* copy, int T, int H,
                     int vocab, float scale, const int* positions, const float* inv_freq, int* status, void* stream);

// resid += sum of delta partial sums (+ other) (+ vec, broadcast over the rows); each may be absent.
int rb_residual_inject(float* resid, const float* delta, int n_delta, long long delta_stride, const float* other,
                       const void* vec, int vec_dtype, int T, int H, void* stream);

// resid += rmsnorm(d) * w_post; out = rmsnorm(resid) * w_next when w_next is given.  d is the sum of the delta
// partial sums, or, with row_of, the weighted sum of a token's rows of delta: sum_j weights[t, j] *
// delta[row_of[t, j]] (delta_stride is then the row stride, top the choices a token).
int rb_postnorm_add_norm(float* resid, const float* delta, int n_delta, long long delta_stride, const int* row_of,
                         const float* weights, int top, const void* w_post, float eps_post, const void* w_next,
                         float eps_next, int w_dtype, void* out, int out_dtype, int n_rows, int H, void* stream);

// [gate | up] halves -> out; kind 0: silu(g) * u; kind 1: min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u) + 1);
// kind 2: gelu(g) * u, gelu in its tanh form.
// paired: gates and ups alternate in blocks of 16 columns instead of lying in two halves.
int rb_gated_act(const void* in, int in_dtype, int n_in, long long in_stride, long long in_ld, void* out, int out_dtype,
                 long long out_ld, int rows, int I, int kind, float limit, float alpha, int paired, void* stream);

int rb_scale(float* x, long long n, float factor, void* stream);

// out[t, h, :out_w] = in[t, h, :out_w] * gate for heads of in_w (>= out_w) values; gate float32 [T, heads * gate_w]
// (gate_w 1: one a head, out_w: one a value), or the sigmoid of `raw` (such columns of projection rows, n_in
// partial sums), or absent.
int rb_head_gate(const void* in, long long ld_in, int in_w, void* out, long long ld_out, int out_w, const float* gate,
                 int gate_w, const void* raw, int raw_dtype, int n_in, long long in_stride, long long row_stride,
                 int heads, int T, int dtype, void* stream);

// A latent-attention layer's projection rows [queries | latent | gate logits]: latent normalised into the paged
// cache, queries (when q_out is given) and sigmoid(gates) written out (latent.cu).
int rb_latent_prep(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_width, int rank,
                   int n_gate, const void* w, int w_dtype, float eps, void* q_out, int q_stride, float* gate_out,
                   void* cache, int act_dtype, const int* positions, const int* slot_of_token, const int* block_table,
                   int max_pages, int T, void* stream);

// Routed experts (routing.cu).  Router logits z[T, E] = x[T, K] . w[E, K]^T with 32-bit FMA, w float32.
int rb_router_logits(const void* x, int x_dtype, long long ldx, const float* w, float* z, int ldz, int T, int E, int K,
                     void* stream);
// n_groups > 1: only experts of the keep_groups best groups of neighbours can be chosen (a group's score: its two
// largest scores added); renormalize: weights divided by their sum + norm_eps.
int rb_moe_route(const float* z, int ldz, const void* bias, int bias_dtype, const int* slot_of_token, int T, int E,
                 int top, int* ids, float* weights, int* place, int* counts, int n_groups, int keep_groups,
                 int renormalize, float norm_eps, void* stream);
int rb_moe_plan(const int* counts, int E, int tile_rows, int max_tiles, int* starts, int* tile_group, void* stream);
int rb_moe_gather(const void* x, int dtype, int H, const int* ids, const int* place, const int* starts, int T, int top,
                  void* rows, int* row_of, void* stream);
// extra (optional): [n_extra][T, H] partial sums added to every token's row, times sigmoid(extra_gate[t * ld]) when
// extra_gate is given.
int rb_moe_combine(const float* y, long long ldy, const int* row_of, const float* weights, int T, int top, float* out,
                   int H, const float* extra, int n_extra, long long extra_stride, const float* extra_gate,
                   int extra_gate_ld, void* stream);

// Linear attention with a fixed decay per head (linear_attention.cu).  The step's tokens go through
// S = decay[h] * S + k v^T, o = S^T q per (sequence, head), the state [slots, heads, dim, vdim] float32 read and
// written in place; q, k, v are columns q_off, k_off, v_off of the projection rows (n_in partial sums added first);
// act 1: silu on q and k (act_qk) or v (act_v); k is multiplied by k_scale.  out float32 [T, heads * vdim].
int rb_decay_scan(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_off, int k_off,
                  int v_off, int heads, int dim, int vdim, int act_qk, int act_v, float k_scale, const float* decay,
                  float* state, const int* seq_slot, const int* cu_q, int B, float* out, int ld_out, void* stream);
// The same for sequences that bring exactly one token each (a decode step): the state streams through registers.
int rb_decay_step(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_off, int k_off,
                  int v_off, int heads, int dim, int vdim, int act_qk, int act_v, float k_scale, const float* decay,
                  float* state, const int* seq_slot, const int* cu_q, int B, float* out, int ld_out, void* stream);
// The same for prompts, by blocks of 64 tokens that run side by side: work float32 [max_blocks, heads, dim, vdim],
// max_blocks >= the sum over the sequences of ceil(tokens / 64).  Head sizes up to 128.
int rb_decay_scan_blocks(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_off, int k_off,
                         int v_off, int heads, int dim, int vdim, int act_qk, int act_v, float k_scale, const float* decay,
                         float* state, const int* seq_slot, const int* cu_q, int B, int max_blocks, float* work, float* out,
                         int ld_out, void* stream);
// out = o / rms(o over each of `groups` column groups) (* w) * act(gate), gate = columns g_off.. of the projection
// rows; gate_act 0: none, 1: silu, 2: sigmoid.
int rb_group_norm_gate(const float* o, int ld_o, const void* proj, int proj_dtype, int n_in, long long in_stride,
                       int row_stride, int g_off, const void* w, int w_dtype, float eps, int groups, int W, int gate_act,
                       void* out, int out_dtype, int ld_out, const int* slot_of_token, int T, void* stream);

// Many small products in one launch, by head or by tiles of sorted rows (grouped_matmul.cu).
int rb_grouped_matmul(const void* x, int x_dtype, long long ldx, int x_col_stride, const void* w, int w_dtype,
                      long long w_group_stride, void* out, int out_dtype, long long ldo, int o_col_stride, int M, int N,
                      int K, int groups, const int* tile_group, int tile_rows, const float* row_scale, int row_scale_ld,
                      int act, float limit, float alpha, void* stream);

// Keeps the stream busy for about that long (at most a second): the profiler's gate.
int rb_hold(long long microseconds, void* stream);
int rb_cast(const void* in, int in_dtype, void* out, int out_dtype, long long n, void* stream);

int rb_qk_norm_rope_cache(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, void* q_out,
                          int act_dtype, int q_stride, int T, int nq, int nkv, int hd, const void* q_norm_w,
                          const void* k_norm_w, int w_dtype, float eps, const float* inv_freq, int rot_dim,
                          const int* positions, const int* slot_of_token, const int* block_table, int max_pages,
                          void* k_cache, void* v_cache, int write_kv, const void* cos_sin, int vd, int hdp,
                          int interleaved, int n_gate, float* gate_out, int post_norm, const float* v_first,
                          const float* v_lambda, float* v_out, void* stream);

int rb_rope_table(const int* positions, const float* inv_freq, int T, int half, float mag, void* out, void* stream);

int rb_gemm_generic(const void* x, int x_dtype, const void* w, int w_dtype, const void* bias, void* out,
                    int out_dtype, int M, int N, int K, long long ldx, long long ldo, int splits,
                    long long split_stride, void* stream);

// The limit, in clock cycles, of every barrier wait in the tensor-core products (cycles <= 0: the default,
// about two seconds), and a switch for tests of the give-up path: while it is set a few-token product
// never requests its first K block, so the warp that waits for it runs into the limit, records
// RB_ERR_TIMEOUT in the status word and the block unwinds.
void rb_gemm_tcgen05_set_wait(long long cycles, int withhold_first_stage);
int rb_gemm_tcgen05(const void* x, const void* w, const float* bias, void* out, int out_dtype, int M, int N,
                    int K, long long ldx, long long ldo, int splits, long long split_stride, int stages,
                    int gated, int* status, void* stream);

int rb_gemm_tcgen05_gated_pair(const void* x, const void* w, const float* bias, void* h, int M, int N, int K,
                               long long ldx, long long ldh, const float* row_sumsq, int row_groups,
                               long long row_sumsq_ld, float row_eps, int stages, int* status, void* stream);

int rb_gemm_tcgen05_residual(const void* x, const void* w, const float* bias, int M, int N, int K, long long ldx,
                             int splits, float* resid, long long ld_resid, const void* next_w, int next_w_f32,
                             void* xhat, long long ld_xhat, float* sumsq, long long ld_sumsq, int stages,
                             int* status, void* stream);

int rb_gemm_tcgen05_qkv_rope(const void* x, const void* w, const float* bias, int M, int N, int K, long long ldx,
                             void* q_out, long long q_ld, void* k_cache, void* v_cache, const int* positions,
                             const int* slot_of_token, const int* block_table, int max_pages, const void* q_norm_w,
                             const void* k_norm_w, int norm_w_f32, float norm_eps, const float* cos_sin, int nq,
                             int nkv, int stages, int* status, void* stream);

// The persistent product over tiles of 128 sorted rows, each with the weight of its group (see the definition).
int rb_gemm_tcgen05_grouped(const void* x, const void* w, void* out, int out_dtype, int R, int N, int K, int groups,
                            long long ldx, long long ldo, const int* tile_group, int gated, int act_kind,
                            float act_limit, float act_alpha, int* status, void* stream);

int rb_gemm_tcgen05_add(const void* x, const void* w, const float* bias, float* resid, int M, int N, int K,
                        long long ldx, long long ld_resid, int stages, int* status, void* stream);

int rb_attention_generic(const void* q, int q_stride, void* out, int o_stride, int dtype, const void* k_cache,
                         const void* v_cache, const int* block_table, int max_pages, const int* seq_slot,
                         const int* cu_q, const int* kv_len, int B, int max_q_len, int nq, int nkv, int hd,
                         float scale, int window, int keep, float sink, int chunk, int n_chunks, float* part_acc,
                         float* part_ml, int cross, void* stream);

int rb_attention_prefill(const void* q, int q_stride, void* out, int o_stride, const void* k_cache,
                         const void* v_cache, const int* block_table, int max_pages, const int* seq_slot,
                         const int* cu_q, const int* kv_len, int B, int max_q_len, int nq, int nkv, int hd, float scale,
                         int window, int keep, float sink, void* stream);

int rb_attention_prefill_tc5(const void* q, int q_stride, int T, void* out, int o_stride, const void* k_cache,
                             const void* v_cache, int n_pages, const int* block_table, int max_pages,
                             const int* seq_slot, const int* cu_q, const int* kv_len, int B, int max_q_len, int nq,
                             int nkv, int hd, float scale, int window, int keep, float sink, int heads_first, int* status,
                             const void* gate, long long gate_row_stride, int cross, void* stream);

int rb_attention_decode(const void* q, int q_stride, const void* k_cache, const void* v_cache,
                        const int* block_table, int max_pages, const int* seq_slot, const int* cu_q,
                        const int* kv_len, int B, int nq, int nkv, int hd, float scale, int window, int keep, float sink,
                        int n_chunks, int pages_per_block, float* part_acc, float* part_ml, int* counters, void* out,
                        int o_stride, const void* gate, int gate_f32, int gate_n_in, long long gate_in_stride,
                        long long gate_row_stride, int cross, void* stream);

int rb_attention_decode_fused(const float* proj, int n_in, long long in_stride, int row_stride, const void* q_norm_w,
                              const void* k_norm_w, int w_f32, float eps, const float* cos_sin, int write_kv,
                              const float* row_sumsq, int row_groups, long long row_sumsq_ld, float row_eps,
                              int row_width, void* k_cache, void* v_cache, const int* block_table, int max_pages, const int* seq_slot,
                              const int* cu_q, const int* kv_len, int B, int nq, int nkv, int hd, float scale,
                              int window, int n_chunks, int pages_per_block, float* part_acc, float* part_ml,
                              int* counters, void* out, int o_stride, int keep, float sink, int rot_dim, int post_norm,
                              const float* v_first, const float* v_lambda, float* v_keep, const void* gate, int gate_f32,
                              int gate_n_in, long long gate_in_stride, long long gate_row_stride, void* stream);

int rb_attention_merge(const float* part_acc, const float* part_ml, void* out, int o_stride, int dtype,
                       const int* positions, const int* slot_of_token, int T, int nq, int hd, int chunk,
                       int n_chunks, int window, int keep, float sink, void* stream);

int rb_argmax(const float* logits, long long row_stride, int rows, int V, int* out, float* scratch_v,
              int* scratch_i, int slices, void* stream);

int rb_sample(float* logits, long long row_stride, int n, int V, const void* rows, const int* history, int* out,
              void* stream);

// Reader of safetensors files (safetensors_reader.cu): open and check the header, list the tensors, copy one
// tensor's bytes to host or device memory, close.
void* rb_st_open(const char* path, char* err, int err_len);
int rb_st_count(const void* handle);
int rb_st_entry(const void* handle, int i, const char** name, const char** dtype, int* rank, long long* shape,
                long long* nbytes);
int rb_st_metadata_count(const void* handle);
int rb_st_metadata(const void* handle, int i, const char** key, const char** value);
int rb_st_read(void* handle, int i, void* dst, long long dst_bytes, int on_device, void* stream);
void rb_st_close(void* handle);

// A layer whose norm follows the sum (postln.cu): resid <- rmsnorm(alpha * resid + gain * sum of the delta partial sums) * w,
// in place, 32-bit; `out` (optional) receives the rows in the activations' type.  gain may be absent (ones).  next_out
// (optional, of out_dtype; only when every row is its sequence's only one): row + (next_kept[slot] - row) * next_mu, and
// next_kept[slot] receives the row.
int rb_postln(float* resid, const float* delta, int n_delta, long long delta_stride, const float* gain, const float* w,
              float alpha, float eps, void* out, int out_dtype, const int* slot_of_token, int n_rows, int H,
              const float* next_mu, float* next_kept, void* next_out, void* stream);
// out[t] = x[t] + (x[t - 1] - x[t]) * mu, the row before a sequence's first coming from (and the last going to) kept[slot].
int rb_token_shift(const float* x, const float* mu, float* kept, const int* seq_slot, const int* cu_q, int n_seqs,
                   int max_q_len, void* out, int out_dtype, int H, void* stream);

// A state-space mixer (ssm.cu).  Causal convolution over `channels` columns from col0 of the projection rows, taps
// [channels][taps] (the last is the current token's), the inputs before a step's first token in kept[slot][taps-1][channels];
// act 1: silu.  out float32 [T, channels].
int rb_causal_conv(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int col0, int channels,
                   int taps, const float* w, const float* bias, int act, float* kept, const int* seq_slot, const int* cu_q,
                   int n_seqs, int max_q_len, float* out, int ld_out, void* stream);
// S = exp(-exp(a_log) dt) S + dt B x^T, y = S^T C + skip * x, dt = softplus(raw + dt_bias); x, B, C columns of u (float32),
// raw columns of the projection rows; state float32 [slots][heads][n][p].
int rb_ssm_scan(const float* u, int ld_u, int x_off, int b_off, int c_off, const void* raw, int raw_dtype, int n_in,
                long long in_stride, int row_stride, int dt_off, const float* dt_bias, const float* a_log, const float* skip,
                int heads, int groups, int n, int p, float* state, const int* seq_slot, const int* cu_q, int n_seqs,
                int one_token_each, float* out, int ld_out, void* stream);
// The same by blocks of 64 tokens side by side (prompts).  work: float32 [n_blocks][heads][n][p], block_decay: float32
// [n_blocks][heads], cb: float32 [n_blocks][groups][64][64], n_blocks >= the sum over sequences of ceil(tokens / 64).
int rb_ssm_scan_blocks(const float* u, int ld_u, int x_off, int b_off, int c_off, const void* raw, int raw_dtype, int n_in,
                       long long in_stride, int row_stride, int dt_off, const float* dt_bias, const float* a_log,
                       const float* skip, int heads, int groups, int n, int p, float* state, const int* seq_slot,
                       const int* cu_q, int n_seqs, int n_blocks, float* work, float* block_decay, float* cb, float* out,
                       int ld_out, void* stream);
// out = rmsnorm over each of `groups` parts of (y * act(z)) * w; z columns of the projection rows; act 1 silu, 2 sigmoid.
int rb_gate_group_norm(const float* y, int ld_y, const void* proj, int proj_dtype, int n_in, long long in_stride,
                       int row_stride, int z_off, const float* w, float eps, int groups, int W, int gate_act, void* out,
                       int out_dtype, int ld_out, const int* slot_of_token, int T, void* stream);

// Latent attention with a query latent and a rotated key part (latent.cu).
int rb_latent_rot_prep(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_rank, int rank,
                       int rot, int n_gate, const float* wq, const float* wc, float eps, void* cq_out, int cq_stride,
                       float* gate_out, void* cache, int dp, int act_dtype, const float* cos_sin, const int* positions,
                       const int* slot_of_token, const int* block_table, int max_pages, int T, void* stream);
int rb_latent_q_rot(const void* q, int q_stride, int heads, int dim, int rot, int rank, int dp, const float* cos_sin,
                    void* folded, int f_stride, int dtype, const int* slot_of_token, int T, void* stream);

// Attention with a norm over the whole q and k projections and head weights mixed after the softmax (talking_heads.cu).
int rb_wide_norm_rope_cache(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int nq, int nkv,
                            int hd, int vd, int hdp, const float* wq, const float* wk, float eps, const float* factor,
                            const float* cos_sin, int rot, int neighbours, void* q_out, int q_stride, void* k_cache,
                            void* v_cache, int act_dtype, const int* positions, const int* slot_of_token,
                            const int* block_table, int max_pages, int T, void* stream);
int rb_talk_mix(const void* o, int o_stride, const float* mix, void* out, int out_stride, int nq, int nkv, int hdp, int vd,
                int dtype, const int* slot_of_token, int T, void* stream);

#ifdef __cplusplus
}
#endif
