/* The C interface of the kernel library (liblitinfer_b200_*.so), as litinfer_b200/kernels.py calls it through ctypes.
 *
 * All pointers are device pointers unless said otherwise; tensors are row-major and contiguous; dtype 0 is float32,
 * 1 bfloat16; every launch goes to `stream`.  A function returns 0, or non-zero with the text in li_last_error(), and
 * launches nothing in that case: sizes a kernel cannot take are refused, never computed wrongly.
 * LitInfer's counterpart is include/llaisys/*.h (ops.h, models/qwen2.h): one C entry per operator.
 */
#pragma once
#include <cuda_runtime.h>

#ifdef __cplusplus
extern "C" {
#endif

/* ---- api.cu ---- */
/* The message of the last call that returned non-zero (a static buffer; copy it before the next call). */
const char* li_last_error();

/* 0 if the current device is a B200 (sm_100); the library has code for no other. */
int li_check_device();
/* Which of the launches that follow may NOT begin while the kernel before them still runs (programmatic dependent
 * launch): a mask of 1 tcgen05 GEMMs, 2 weight-streaming products, 4 attention, 8 the rest; 0 lets all overlap (the
 * default), 15 none.  The step function sets it per step.  LITINFER_B200_PDL=0 in the environment keeps all off. */
void li_pdl_allow(int kinds_off);

/* ---- resident block tables (elementwise.cu) ---- */
/* resident [rows, cols] int32: a row per state slot, the last row all sink page.  updates: a count, then triples (slot,
 * logical page, page id).  Applies the triples of each of the S sequences' slots, then copies the first max_blocks
 * entries of each sequence's row into out [S, max_blocks]. */
int li_table_gather(int* resident, int rows, int cols, const int* updates, int update_cap, const int* slots, int* out, int S, int
    max_blocks, int trash_page, cudaStream_t stream);

/* ---- attention.cu ---- */
/* Causal grouped-query attention of a step's tokens over the paged cache.  qkv [T, (nh + 2 nkv) dh] with q
 * rotated; out [T, nh dh]; token t of sequence s at position p sees the cached keys max(0, p - window + 1) .. p
 * through block_table[s]; singles: how many sequences of a step with longer portions have one token (negative: not
 * known); units (may be NULL): the work list of the kernel for long portions, made with the step's metadata (two counts,
 * two unused words, then per entry: sequence, tile of 128 tokens, part | parts << 8, unused), with the number of entries
 * to launch when the single tokens go to the decode kernel and when they do not.  softcap > 0: scores become
 * softcap * tanh(score / softcap); slopes [nh] (may be NULL): slopes[h] * (p - key) is taken off the score of head h;
 * gate [T, nh] in the run dtype (may be NULL): head h's output is multiplied by 1 / (1 + exp(-gate[t, h])).
 * keep_first > 0 (with a window): keys 0 .. keep_first - 1 stay visible behind the window; sinks [nh] (may be NULL):
 * exp(sinks[h]) joins the softmax's denominator of head h once, with no key and no value. */
int li_paged_attention(const void* qkv, void* out, const void* kcache, const void* vcache, int dtype, const int*
    block_table, int max_blocks, const int* q_start, const int* ctx_lens, const int* seq_of_token, const int*
    positions, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages, float scale, int window, int
    max_q_len, int max_ctx_len, const int* old_lens, int singles, const int* units, int slots_portions, int slots_all,
    float softcap, const float* slopes, const void* gate, int keep_first, const float* sinks, cudaStream_t stream);

/* The same through one implementation: 0 general, 1 decode, 2 mma.sync tiles, 3 tcgen05 tiles (tests and
 * measurements). */
int li_paged_attention_with(int which, const void* qkv, void* out, const void* kcache, const void* vcache, int dtype,
    const int* block_table, int max_blocks, const int* q_start, const int* ctx_lens, const int* seq_of_token, const
    int* positions, int T, int S, int nh, int nkv, int dh, int page_size, int num_pages, float scale, int window, int
    max_q_len, int max_ctx_len, const int* old_lens, int singles, const int* units, int slots_portions, int slots_all,
    float softcap, const float* slopes, const void* gate, int keep_first, const float* sinks, cudaStream_t stream);

/* ---- decode_step.cu: a decode step as one persistent kernel (decode_step.h has the structures) ---- */
struct LiDecodeStep;
int li_decode_step_accepts(int M, int hidden, int heads, int kv_heads, int head_dim, int intermediate, int vocab, int page_size);
int li_decode_step_plan(int M, int hidden, int heads, int kv_heads, int head_dim, int splits, int* stage_k, int* stages, int* x_cols, int*
    scratch_bytes);
int li_decode_step(const LiDecodeStep* step, cudaStream_t stream);

/* ---- elementwise.cu ---- */
/* out[t] = table[ids[t]] as float. */
int li_embedding(const void* table, int dtype, const int* ids, float* out, int T, int H, int V, cudaStream_t stream);

/* x[t] += pairs[row] with row = (prev * mul_prev + ids[t] * mul_cur) mod buckets, prev the token before t in its sequence:
 * ids[t - 1] inside a portion, for a portion's first token the sequence's last token of the step before (state [slots,
 * state_stride] int32, element 0), and row `buckets` for a sequence's first token (position 0).  The state moves on to the
 * portion's last token in the same launch.  pairs [buckets + 1, H] in the run dtype. */
int li_add_pair_rows(float* x, const void* pairs, int dtype, const int* ids, const int* positions, const int* q_start,
    const int* seq_of_token, const int* slots, int* state, long long state_stride, int buckets, long long mul_prev, long long mul_cur,
    int T, int H, cudaStream_t stream);

/* out = x / sqrt(mean(x^2) + eps) * w, rows of H; out in the run dtype. */
int li_rmsnorm(const float* x, const float* w, float eps, void* out, int dtype, int T, int H, cudaStream_t stream);

/* x += delta (in place, float), then out = rmsnorm(x). */
int li_add_rmsnorm(float* x, const void* delta, int dtype, const float* w, float eps, void* out, int T, int H,
    cudaStream_t stream);

/* out[r] = rmsnorm(x[rows[r]]): the final norm on the rows whose logits are wanted. */
int li_gather_rmsnorm(const float* x, const int* rows, const float* w, float eps, void* out, int dtype, int R, int T,
    int H, cudaStream_t stream);

/* x += delta over n elements. */
int li_residual_add(float* x, const void* delta, int dtype, long long n, cudaStream_t stream);

/* out[r, :] = src[rows[r], :] for n_rows rows of `width` floats. */
int li_gather_rows(const float* src, const int* rows, float* out, int n_src, int n_rows, long long width, cudaStream_t stream);

/* x *= factor over n floats (an embedding scale). */
int li_scale_inplace(float* x, long long n, float factor, cudaStream_t stream);

/* x = cap * tanh(x / cap) over n floats (a cap on the logits). */
int li_logit_cap(float* x, long long n, float cap, cudaStream_t stream);

/* out[t, i] = up * gate / (1 + exp(-gate)), gate_up [T, 2 I] as gate | up. */
int li_swiglu(const void* gate_up, void* out, int dtype, int T, int I, cudaStream_t stream);

/* out = hprime * rinv per row, rinv from the partial sums of squares ssq[M, nparts] (the norm that rides on two
 * products, applied on its own). */
int li_apply_row_scale(const void* hprime, const float* ssq, int nparts, int width, float eps, void* out, int M, int
    H, cudaStream_t stream);

/* out[t, i] = g / (1 + exp(-alpha g)) * (u + 1) with g = min(gate, limit), u = clamp(up, -limit, limit); gate_up
 * [T, 2 I] as gate | up. */
int li_glu_clamped(const void* gate_up, void* out, int dtype, int T, int I, float limit, float alpha, cudaStream_t stream);

/* out = a N(z) + b N(z^2) + c N(z^3) + e per row of z [T, n], powers element by element, N(v) = v / sqrt(mean(v^2) + eps),
 * coef = {a, b, c, e} float on the device. */
int li_polynorm(const void* z, int dtype, const float* coef, float eps, void* out, int T, int n, cudaStream_t stream);

/* x [T, n] *= sigmoid(gate [T, gate_stride] at column gate_off + i / group), in float, one rounding. */
int li_mul_sigmoid(void* x, const void* gate, int dtype, int gate_stride, int gate_off, int group, int T, int n, cudaStream_t stream);

/* out = sa a + sb b over n elements of the run dtype (the sum in float). */
int li_weighted_sum2(const void* a, const void* b, float sa, float sb, void* out, int dtype, long long n, cudaStream_t stream);

/* ---- hyper.cu: the residual stream as s parallel streams xs [T, s, H] (float) ---- */
/* out[r] = RMSNorm(sum_s in_w[s] xs[rows[r], s]) * w; in_w NULL: the plain sum; rows NULL: every row in order. */
int li_hc_read_norm(const float* xs, const float* in_w, const int* rows, const float* w, float eps, void* out, int dtype, int R,
    int T, int s, int H, cudaStream_t stream);

/* xs[t, r] = sum_s mix[s, r] xs[t, s] + out_w[r] y[t] (all streams from the old ones); then, unless next_out is NULL,
 * next_out[t] = RMSNorm(sum_r next_in[r] xs[t, r]) * next_w.  y2 not NULL: the output is s1 y + s2 y2. */
int li_hc_update(float* xs, const void* y, const void* y2, float s1, float s2, int dtype, const float* mix, const float* out_w,
    const float* next_in, const float* next_w, float eps, void* next_out, int T, int s, int H, cudaStream_t stream);

/* xs[t, a] = x[t] for every stream a. */
int li_hc_expand(const float* x, float* xs, int T, int s, int H, cudaStream_t stream);

/* x[t] += table[positions[t]]: learned absolute positions, table [P, H] in the run dtype. */
int li_add_position_rows(float* x, const void* table, int dtype, const int* positions, int T, int H, int P, cudaStream_t stream);

/* ---- recurrent.cu: mixers with a state of fixed size per request (state [slots, state_stride] float) ---- */
/* out[t, c] = silu(b[c] + sum_k w[c, k] in_(t - taps + 1 + k)[c]) over the C channels at column in_off of in [T,
 * in_stride]; inputs before a sequence's portion come from its state (the last taps - 1 inputs, oldest first, at
 * state_off).  shift: every sequence has one token, and its state moves on in the same launch. */
int li_causal_conv_silu(const void* in, int dtype, int in_stride, int in_off, const float* w, const float* b, float* state,
    long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
    void* out, int T, int C, int taps, int shift, cudaStream_t stream);

/* Moves every sequence's convolution state on by its portion (after li_causal_conv_silu has read it). */
int li_conv_state_shift(const void* in, int dtype, int in_stride, int in_off, float* state, long long state_stride, long long state_off,
    const int* q_start, const int* slots, int S, int C, int taps, cudaStream_t stream);

/* Per head S [N, P]: S = exp(-exp(A_log) dt) S + dt B x^T, y = S^T C + D x, dt = softplus(dt_raw + dt_bias); xbc
 * [T, C] holds x | B | C; a sequence's tokens in order, its state read and written once (kept as [heads][P][N]). */
int li_ssm_scan(const void* xbc, int dtype, int C, const void* dt_raw, int dt_stride, const float* dt_bias, const float* A_log,
    const float* D, float* state, long long state_stride, const int* q_start, const int* slots, float* y, int S, int heads,
    int P, int N, int groups, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream);

/* Per head S [d, dv]: S = decay S + k v^T, out = S^T q, with q, k, v = silu of the columns at q_off, k_off, v_off
 * of qkv [T, stride]; the state is kept as [heads][dv][d]. */
int li_decay_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* decay, float* state,
    long long state_stride, const int* q_start, const int* slots, float* out, int S, int heads, int d, int dv,
    const int* seg, int mode, float* chunk_state, cudaStream_t stream);

/* Long portions in chunks (seg: quadruples of begin, end, chunk, slot; S = their number): the scans run with mode 1 (every
 * chunk from zeros, its end state to chunk_state, for li_ssm_scan its decay to chunk_decay), then li_scan_carry (runs:
 * triples of first chunk, chunks, slot; a chunk's decay given, or token_decay[head] ^ length) turns chunk_state into the states the chunks start from and moves the slots on,
 * then the scans with mode 2 (outputs).  Mode 0 without seg: every sequence in one piece. */
int li_scan_carry(float* state, long long state_stride, float* chunk_state, const float* chunk_decay, const float* token_decay,
    const int* seg, const int* runs, int nruns, int heads, int per_head, int period, cudaStream_t stream);

/* Per head S [d, dv] with a decay per token and key channel: S = diag(a) S + k v^T, out = S^T (q q_scale), with
 * a = sigmoid(z)^inv_tau from the float logits za [T, za_stride] at column za_off (heads x d); q, k, v are the columns at
 * q_off, k_off, v_off of qkv [T, stride] as they are; the state is kept as [heads][dv][d]; chunk_decay [chunks, heads, d]
 * (li_scan_carry with period d). */
int li_gla_scan(const void* qkv, int dtype, int stride, int q_off, int k_off, int v_off, const float* za, int za_stride, int za_off,
    float inv_tau, float q_scale, float* state, long long state_stride, const int* q_start, const int* slots, float* out,
    int S, int heads, int d, int dv, const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream);

/* The gated delta rule, per head S [d, dv]: S = diag(g) S, u = beta (v - S^T k), S = S + k u^T, out = S^T q.  li_delta_prepare
 * makes per token what does not depend on the state: the causal convolution (conv_w [channels, taps], older inputs from the
 * state at state_off) and silu of the channels q | k | v (kv_heads d, kv_heads d, heads dv) at column col0 of proj [T, stride];
 * q and k as unit vectors (x / sqrt(sum x^2 + unit_eps), q times q_scale) and k . q into prep_qk [T, kv_heads, 2 DP + 4];
 * g = exp(-exp(A_log[h]) softplus(za [T, za_stride] at za_off + h d + i)) and beta = sigmoid(proj[b_off + h]) into prep_g
 * [T, heads, DP + 4]; v [T, heads dv]; all float, DP = 32, 64, 128 or 256 (the first that holds d).  shift: every sequence has
 * one token and the convolution's state moves on here.  li_delta_scan walks; head h uses key head h / (heads / kv_heads); the
 * state is kept as [heads][dv][d]. */
int li_delta_prepare(const void* proj, int dtype, int stride, int col0, int b_off, const float* conv_w, int taps, float* state,
    long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
    const float* za, int za_stride, int za_off, const float* A_log, float q_scale, float unit_eps, float* prep_qk,
    float* prep_g, float* v, int T, int heads, int kv_heads, int d, int dv, int shift, cudaStream_t stream);
void li_delta_force_columns(int columns);   /* 0: columns a warp of the walk by the launch's size; 2, 4 or 8, for tests and measurements */
int li_delta_scan(const float* prep_qk, const float* prep_g, const float* v, float* state, long long state_stride, const int* q_start,
    const int* slots, float* out, int S, int heads, int kv_heads, int d, int dv, cudaStream_t stream);

/* Per channel c a state S [N]: S = exp(dt_c A[c, :]) S + dt_c x_c B, y_c = (S . C + D[c] x_c) silu(z_c), with
 * dt = softplus(dt_raw) (float, [T, dt_stride]), A = -exp(A_log) [inner, N]; x at column x_off of [T, x_stride], B and C
 * (N each) at b_off and c_off of bc [T, bc_stride], the gate z at z_off of [T, z_stride]; y [T, inner] in the run dtype; the
 * state is kept as [inner][N]; chunk_decay [chunks, inner, N] (li_scan_carry with one head and period inner N). */
int li_channel_scan(const void* x, int dtype, int x_stride, int x_off, const void* bc, int bc_stride, int b_off, int c_off,
    const float* dt_raw, int dt_stride, const void* z, int z_stride, int z_off, const float* A_log, const float* D,
    float* state, long long state_stride, const int* q_start, const int* slots, void* y, int S, int inner, int N,
    const int* seg, int mode, float* chunk_state, float* chunk_decay, cudaStream_t stream);

/* RMSNorm of y [T, n] (float) in `groups` equal parts, times w; mode 0: y is first multiplied by silu(gate), mode 1:
 * the result is multiplied by sigmoid(gate), mode 2: by silu(gate); gate [T, gate_stride] at column gate_off, in the run dtype like out. */
int li_gated_rmsnorm(const float* y, const void* gate, int dtype, int gate_stride, int gate_off, const float* w, float eps, int mode,
    void* out, int T, int n, int groups, cudaStream_t stream);

/* ---- gemm_tcgen05.cu ---- */
/* Measurements: 0 keeps the rotary epilogue to paired tiles. */
void li_tcgen05_rope_single_tiles(int on);

/* Tests and measurements: force a tile shape of the tcgen05 product (0: by shape). */
void li_tcgen05_force_tile(int tile);

/* Tests and measurements: force the splits of k of the tcgen05 product (0: by shape). */
void li_tcgen05_force_ksplit(int n);

/* ---- gemv_bf16.cu ---- */
/* The weight-streaming product for callers that may not allocate (see no_alloc.h). */
int li_linear_gemv_static(const void* a, const void* w, const float* bias, void* out, int dtype_out, int M, int N, int
    K, cudaStream_t stream);

/* ---- gemv_tcgen05.cu ---- */
/* Measurements: force the splits of k of the swapped tcgen05 product (0: by shape). */
void li_gemv_tcgen05_force_ksplit(int n);

/* ---- linear.cu ---- */
/* out[M, N] = a[M, K] w[N, K]^T (+ bias), epilogue 0 none / 1 SwiGLU over interleaved gate|up rows; float32 in
 * float32 out, or bfloat16 in, bfloat16 or float out. */
int li_linear(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M, int N,
    int K, int epilogue, cudaStream_t stream);

/* 1 if li_linear_scaled takes this product. */
int li_linear_scaled_accepts(const void* a, const void* w, const void* out, int dtype_in, int M, int N, int K);

/* li_linear with each row of a scaled by rinv from partial sums of squares (a deferred RMSNorm). */
int li_linear_scaled(const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out, int M,
    int N, int K, int epilogue, const float* ssq, int nparts, int width, float eps, cudaStream_t stream);

/* How many partial sums per row li_linear_add_scaled leaves for this product (0: it refuses it). */
int li_linear_add_scaled_parts(const void* a, const void* w, const void* x32, const void* hprime, int dtype_in, int M,
    int N, int K);

/* x32 += a w^T (+ bias); hprime = bfloat16(norm_weight * x32); ssq_out[row, part] = sums of x32^2 over the part's
 * columns. */
int li_linear_add_scaled(const void* a, const void* w, const float* bias, float* x32, const float* norm_weight, void*
    hprime, float* ssq_out, int dtype_in, int M, int N, int K, cudaStream_t stream);

/* li_linear through one implementation (tests and measurements). */
int li_linear_with(int which, const void* a, const void* w, const float* bias, void* out, int dtype_in, int dtype_out,
    int M, int N, int K, int epilogue, cudaStream_t stream);

/* ---- rope.cu ---- */
/* out[t, j] = (cos, sin)(positions[t] / denom[j]). */
int li_rope_table(const int* positions, const float* denom, int half, float* out, int T, cudaStream_t stream);

/* Rotate q in place, rotate k and store it, store v (transposed) at slot_mapping[t] of the paged caches. */
int li_rope_kv_write(void* qkv, int dtype, const int* positions, const float* denom, int rotary_dim, const int*
    slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh, int page_size, int num_pages, int write,
    cudaStream_t stream);

/* The q|k|v product followed by li_rope_kv_write, as one kernel where the shape allows. */
int li_linear_rope_kv(const void* a, const void* w, const float* bias, void* qkv, int dtype, const int* positions,
    const float* denom, int rotary_dim, const int* slot_mapping, void* kcache, void* vcache, int T, int K, int nh, int
    nkv, int dh, int page_size, int num_pages, int write, int allow_fused, const float* ssq, int nparts, int width,
    float eps, const float* cos_sin, cudaStream_t stream);

/* ---- norm_pair.cu: norms before and after a sublayer in one pass over the residual stream ---- */
/* Per row: x += post(y) (post: a norm of y [R, H] with the weight w_post; NULL: x += y; y NULL: nothing is added), then
 * out = next(x) if w_next is given (without it, out, if given, takes x as it is in the run dtype).  A norm is centered (mean taken off, variance as the mean of squared deviations:
 * layer norm without bias) or not (RMS norm).  rows (may be NULL; only without y): out[r] = next(x[rows[r]]).
 * y_places (may be NULL): token r's y is the sum over j < y_top of y[y_places[r y_top + j]] (times y_weights[...] if given). */
int li_norm_add_norm(float* x, const void* y, int dtype, const float* w_post, int post_centered, float eps_post, const float* w_next,
    int next_centered, float eps_next, void* out, const int* rows, int R, int n_src, int H, const int* y_places,
    int y_top, const float* y_weights, cudaStream_t stream);

/* x[t] += row for every token. */
int li_add_row(float* x, const float* row, int T, int H, cudaStream_t stream);

/* RMS norm of the columns col .. col + n - 1 of in [T, ld_in] (mean of squares over `width` elements), written to out
 * [T, ld_out] at col_a and, if col_b >= 0, at col_b too. */
int li_rmsnorm_cols(const void* in, int dtype, int ld_in, int col, int n, int width, const float* w, float eps, void* out, int ld_out,
    int col_a, int col_b, int T, cudaStream_t stream);

/* ---- qkv_post.cu: between the q|k|v product and attention ---- */
/* A short causal convolution per channel (conv_w [(nh + 2 nkv) dh, taps]; inputs before a portion from state [slots,
 * state_stride] at state_off), an RMS norm per query and key head (q_norm, k_norm [dh], mean over norm_width elements),
 * the rotation of the first rotary_dim elements, q to out, k and v into the paged cache.  Every step is optional.
 * row_rinv (may be NULL) [T, 2]: the norm is over the whole projection of q (column 0) and of k (column 1) instead: the
 * factor is given, and q_norm [nh dh], k_norm [nkv dh] hold a weight per channel.  nkv 0 (with write 0): proj and out hold
 * queries only.  out_ld: elements of a row of out (0: as many as a row of proj).
 * shift: every sequence of the step has one token, and the state moves on in the same launch.  to_cache 0: keys and values
 * go to their columns of out, not into the cache. */
int li_conv_norm_rope_kv(const void* proj, void* out, int dtype, const float* conv_w, int taps, float* state,
    long long state_stride, long long state_off, const int* q_start, const int* seq_of_token, const int* slots,
    const float* q_norm, const float* k_norm, float eps, int norm_width, const float* row_rinv, const int* positions,
    const float* denom, int rotary_dim, const int* slot_mapping, void* kcache, void* vcache, int T, int nh, int nkv, int dh,
    int page_size, int num_pages, int write, int shift, int to_cache, int out_ld, cudaStream_t stream);

/* Latent attention with a rotated part, per token: c = rmsnorm(low[col_c : col_c + R]) * w into the key and the value head of
 * out [T, (nh + 2) dl]; the shared key part low[col_r : col_r + dr] rotated behind c in the key head; every query head's
 * rotated part q[h (d + dr) + d ...] rotated behind the head's first R columns; the rest of the heads zero.  Pair i turns by
 * float(pos) / denom[i]; interleaved: pair (2i, 2i + 1), else (i, i + dr / 2); cosine and sine times magnitude. */
int li_latent_rope_post(const void* low, int dtype, int ld_low, int col_c, int col_r, const void* q, int ld_q, int d, const float* w, float eps,
    const int* positions, const float* denom, float magnitude, int interleaved, void* out, int T, int nh, int R, int dr,
    int dl, cudaStream_t stream);

/* out[t, j] = 1 / sqrt(sum of squares of the columns col_j .. col_j + n_j - 1 of x [T, ld] / width_j + eps), j = 0, 1 (n_1
 * 0: one range): the factor of an RMS norm over a whole projection, for li_conv_norm_rope_kv's row_rinv. */
int li_row_rinv(const void* x, int dtype, int ld, int col0, int n0, int width0, int col1, int n1, int width1, float eps, float* out,
    int T, cudaStream_t stream);

/* ---- grouped.cu: products in groups, routing of a mixture of experts ---- */
/* out_g = a_g w_g^T, w [G, N, K].  row_offsets [G + 1] (device): group g owns those rows of a [M, lda] and out [M, ldc].
 * row_offsets NULL: every group takes all M rows, inputs at column g * a_gcol, outputs at column g * c_gcol.
 * tile_group (may be NULL): with runs of rows that start at multiples of 128, the group of every tile of 128 rows (-1: none);
 * large bfloat16 products then run on tcgen05 tiles.  epilogue 1 (bfloat16): gate and up rows of every matrix interleaved in
 * eights, out rows of N / 2 activations up * gate / (1 + exp(-gate)). */
int li_grouped_linear(const void* a, int lda, int a_gcol, const void* w, void* out, int ldc, int c_gcol, const int* row_offsets,
    const int* tile_group, int dtype, int M, int N, int K, int G, int epilogue, const float* glu_params,
    cudaStream_t stream);

/* ids, weights [T, top]: the experts with the largest sigmoid(logits [T, E]) and those scores (scoring 0), or the experts
 * with the largest logits and the softmax over the chosen logits alone (scoring 1). */
int li_moe_route(const float* logits, int scoring, int T, int E, int top, int* ids, float* weights, cudaStream_t stream);

/* The same choice for a router over all experts at once with groups: s = softmax(logits [T, E]); choice scores s + correction
 * (may be NULL); the experts form `groups` equal groups of neighbours, a group's score is its largest choice score, only the
 * `keep` best groups' experts can be chosen; the `top` largest choice scores choose; weights = s of the chosen / (their sum +
 * 1e-20) * scale. */
int li_moe_route_grouped(const float* logits, const float* correction, int T, int E, int top, int groups, int keep, float scale, int* ids,
    float* weights, cudaStream_t stream);

/* Stable sort of n (token, choice) pairs by expert: offsets [E + 1], pair_at (pair at a sorted place, -1: none), place_of [n].
 * Every expert's run starts at a multiple of pad; pair_at has `places` entries; tile_group (may be NULL) [n_tiles]: the expert of
 * every tile of pad rows, -1 for the experts from `matrices` on (experts without matrices, whose rows pass as they are). */
int li_moe_sort(const int* ids, int n, int E, int matrices, int pad, int* offsets, int* pair_at, int* place_of, int* tile_group, int n_tiles,
    int places, cudaStream_t stream);

/* out [n, H]: row r is h[pair_at[r] / top], times weights[pair_at[r]] if weights is given; zeros where pair_at[r] < 0. */
int li_moe_gather(const void* h, int dtype, const int* pair_at, const float* weights, int n, int top, int H, void* out, cudaStream_t stream);

/* y [T, H]: y[t] = sum_k rows[place_of[t * top + k]] (times weights[t * top + k] if weights is given). */
int li_moe_combine(const void* rows, int dtype, const int* place_of, const float* weights, int T, int top, int H, void* y,
    cudaStream_t stream);

/* ---- sampling.cu ---- */
/* out[r] = the first maximum of logits[r]. */
int li_argmax(const float* logits, int* out, int R, int V, cudaStream_t stream);

/* out[r] = a draw from logits[r] under (temperature, top_k, top_p, seed, output index) packed in params; Gumbel-
 * max with a counter-based generator, independent of the batch. */
int li_sample(const float* logits, const int* params, int* out, int R, int V, cudaStream_t stream);

/* ---- fill_random.cu ---- */
/* out[i] = mean + std * n(key, i), n standard normal from a counter-based generator (a pure function of key and i). */
int li_fill_normal(void* out, int dtype, long long n, unsigned long long key, float mean, float std, cudaStream_t stream);

/* out[i] = an integer in [0, range) from (key, i). */
int li_fill_randint(int* out, long long n, unsigned long long key, int range, cudaStream_t stream);

/* ---- tcgen05_host.cu ---- */
/* 0, or the status a tcgen05 kernel left when one of its bounded waits ran out. */
int li_tcgen05_status();

/* Tests: clear the status word; make a bounded wait run out on purpose (one thread, a barrier nobody arrives on,
 * a limit in microseconds): the status then reads 99. */
void li_tcgen05_clear_status();

/* Progress marks of kernels launched with their debug flag (host memory, readable while they run). */
int li_tcgen05_progress(int* out, int n);
int li_tcgen05_wait_selftest(int limit_us, cudaStream_t stream);

#ifdef __cplusplus
}
#endif
