/* C ABI of libb200hybrid.so: the operators of hybrid decoders (latent attention with a sink, decayed linear attention,
 * routed experts, grouped RMS norm, short causal convolution, depth-weighted residual history; windowed attention with
 * grouped key/value heads, residual add + RMS norm, learned positions; parallel blocks with two norms, convolved rotary
 * attention whose values are its keys, a selective state-space mixer, sigmoid-routed experts; parallel blocks with one norm
 * and a token shift, two mixers side by side, chunked rotary attention with scores mixed across heads, a recurrence with a
 * decay per key channel and token, a router that chooses among groups of experts) for sm_100a.
 *
 * Conventions shared by all entries: raw device pointers, sizes as int, `stream` a cudaStream_t, return 0 on success, a
 * negative b200h_status for refused arguments, a positive cudaError_t for a failed launch; b200h_last_error() says why.
 * `dtype` is the type T of projection outputs and weights: B200H_BF16 or B200H_F32.  The residual stream, norm weights,
 * router weights, recurrent state and everything named `float` below are 32-bit floats whatever T is.
 * A step has n rows; row t belongs to batch entry tok_seq[t], at position tok_pos[t]; cu_q[s] is entry s's first row. */
#ifndef B200_HYBRID_H
#define B200_HYBRID_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
#define B200H_API extern "C" __attribute__((visibility("default")))
#else
#define B200H_API

/* ---- parallel blocks with one norm and a token shift, side-by-side mixers, recurrence with a decay per channel and token ---- */

/* out[t] = table[tokens[t]] + second[row] (float), row = (previous token * mul_prev + tokens[t] * mul_cur) mod buckets, or `buckets`
 * (the table's last row) at position 0.  The token before an entry's first row is the int at prev + seq_slot[s] * slot_stride (in
 * a float's place), which then becomes the entry's last token of this step. */
B200H_API int b200h_embed_hashed(const void* tokens, const void* table, const void* second, int buckets, int mul_prev, int mul_cur, void* prev,
                                 int64_t slot_stride, const void* tok_seq, const void* tok_pos, const void* cu_q, const void* seq_slot,
                                 void* out, int n, int batch, int width, int dtype, void* stream);

/* x[t] += branch_scale * (left[t] / rms(left[t]) * wl + right[t] / rms(right[t]) * wr) + sum_p ff[t, p]; then, if w is given,
 * hf[t] = x[t] / rms(x[t]) * w (float) and h[t] the same as T.  left, right: T [n, width] (both or neither) with wl, wr float
 * [width]; ff: T (or float when ff_is_f32) [n, parts, width] or NULL; h, hf optional. */
B200H_API int b200h_branch_residual_norm(void* x, const void* left, const void* right, const void* wl, const void* wr, float branch_scale,
                                         const void* ff, int ff_is_f32, int parts, const void* w, int n, int width, float eps, void* h,
                                         void* hf, int dtype, void* stream);

/* Token shift of normed rows h (float [n, width]): a[t] = h[t] + (h[t-1] - h[t]) * shift (shift float [width] or NULL: a = h), and
 * for m < nmu blends[m][t] = a[t] + (a[t-1] - a[t]) * mu[m] (mu float [nmu, width]; a, blends T, blends [nmu, n, width]; a optional).
 * The rows before an entry's first come from its state (float [2, width] = its last h and a at state + seq_slot[s] * slot_stride;
 * zeros at a sequence's start), which is then advanced by the step. */
B200H_API int b200h_token_shift(const void* h, const void* shift, const void* mu, int nmu, void* state, int64_t slot_stride,
                                const void* tok_seq, const void* cu_q, const void* seq_slot, int n, int batch, int width, void* a,
                                void* blends, int dtype, void* stream);

/* Per head, S a [dim, vdim] float matrix per sequence:  w_t = exp(-exp(d_t + w0)) per key channel;
 * out_t = (S + diag(bonus) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T.  r, k (heads * dim columns) and v (heads * vdim) are T
 * with row stride ld; d float [n, heads * dim]; w0, bonus float [heads * dim]; state float [heads, vdim, dim] at state + seq_slot[s] *
 * slot_stride, read and advanced; decay: float [n, heads * dim] scratch; out float [n, heads * vdim]. */
B200H_API int b200h_channel_decay_scan(const void* r, const void* k, const void* v, int64_t ld, const void* d, const void* w0,
                                       const void* bonus, void* state, int64_t slot_stride, const void* cu_q, const void* seq_slot, int n,
                                       int batch, int heads, int dim, int vdim, void* decay, void* out, int dtype, void* stream);

/* y[t] = unit_rms_per_group(o[t]) * w * act(gate[t]) as T: the norm BEFORE the gate; o float [n, count], `groups` equal parts,
 * gate T with row stride ld_gate; act 0 sigmoid, 1 silu. */
B200H_API int b200h_group_norm_gate(const void* o, const void* w, const void* gate, int64_t ld_gate, int n, int count, int groups, int act,
                                    float eps, void* y, int dtype, void* stream);

/* x <- z > 0 ? softplus(p) z^2 + z / 2 : (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 in place (T); params = {p, q} floats on the device. */
B200H_API int b200h_xielu(void* x, int64_t count, const void* params, int dtype, void* stream);

/* x <- tanh(x) in place (T). */
B200H_API int b200h_tanh(void* x, int64_t count, int dtype, void* stream);

/* Router with sigmoid scores s and groups of neighbouring experts: choice score = s + correction (float [experts] or NULL); a
 * group's score = the sum of its group_top largest choice scores; only experts of the `keep` best of `groups` equal groups can be
 * chosen; ids = the `top` largest choice scores; wts = the chosen s (without correction), / (their sum + 1e-20) if renorm, * scale. */
B200H_API int b200h_route_grouped(const void* x, int x_dtype, const void* router, const void* correction, int n, int width, int experts,
                                  int top, int groups, int keep, int group_top, int renorm, float scale, void* ids, void* wts, void* stream);

#endif

#define B200H_BF16 1
#define B200H_F32 2
#define B200H_MAX_TAPS 16

enum b200h_status { B200H_ERR_INVALID_ARG = -1, B200H_ERR_UNSUPPORTED = -2 };

/* Rotation of interleaved pairs (2i, 2i+1), i < pairs, by the angle position * freqs[i]; cos and sin times magnitude.
 * freqs: `pairs` doubles in device memory. */
typedef struct b200h_rotary {
    const void* freqs;
    int pairs;
    float magnitude;
} b200h_rotary;

/* One latent-attention layer of one step.
 * Cache entry of a position inside its page (page address + layer_off): the normed latent as T at [pos % block_len][kv_rank],
 * and, rot_off bytes further, the rotated shared key part as float at [pos % block_len][rot_dim]. */
typedef struct b200h_latent_args {
    int n, heads, dim, rot_dim, vdim, kv_rank, q_rank, block_len;
    float scale, eps;
    b200h_rotary rot;
    const void* dq;          /* T [n, ld_dq]: query latent before its norm (q_rank columns) */
    int64_t ld_dq;
    const void* dkv;         /* T [n, ld_dkv]: kv_rank latent columns, then rot_dim shared key columns */
    int64_t ld_dkv;
    const void* q_norm;      /* float [q_rank] */
    const void* kv_norm;     /* float [kv_rank] */
    void* cq;                /* T [n, q_rank]: out of b200h_latent_prep */
    const void* q;           /* T [n, ld_q]: per head dim plain then rot_dim rotated columns */
    int64_t ld_q;
    const void* sink;        /* float [heads] */
    const void* q_lat;       /* float [n, heads, kv_rank]: the plain query parts carried into the latent's coordinates (uk_h^T q) */
    void* q_rot;             /* float [n, heads, rot_dim]: out of b200h_rotate_query */
    void* o_lat;             /* float [n, heads, splits, kv_rank] scratch: unnormalised partial of every key range */
    void* ml;                /* float [n, heads, splits, 2] scratch: running maximum and denominator of every key range */
    int splits;              /* key ranges per row (whole pages each), >= 1 */
    void* o_heads;           /* T [heads, n, kv_rank]: out of b200h_latent_attention, the normalised weighted sum of latents */
    const void* tok_seq;     /* int [n] */
    const void* tok_pos;     /* int [n] */
    const void* block_ptrs;  /* int64: page addresses, entry s's pages from cu_blocks[s] */
    const void* cu_blocks;   /* int [batch + 1] */
    int64_t layer_off, rot_off;
    int dtype;
    void* stream;
} b200h_latent_args;

B200H_API const char* b200h_last_error(void);

/* out[t] = table[tokens[t]] * scale (float). */
B200H_API int b200h_embed(const void* tokens, const void* table, float scale, void* out, int n, int width, int dtype, void* stream);

/* out[t] = x[t] + sum_j w[:, j] * x[t - taps + 1 + j] as T, x float [n, width], w float [width, taps]; rows before an entry's first
 * come from its state (float [taps - 1, width] at state + seq_slot[s] * slot_stride), which is then advanced by the step. */
B200H_API int b200h_causal_conv(const void* x, const void* w, void* state, int64_t slot_stride, const void* tok_seq, const void* cu_q,
                                const void* seq_slot, void* out, int n, int batch, int width, int taps, int dtype, void* stream);

/* x[t] += w * (sum_p m[t, p]) / rms per group; m is T (or float when m_is_f32) [n, parts, width]; x_t (optional): x as T. */
B200H_API int b200h_residual_group_norm(void* x, const void* m, int m_is_f32, int parts, const void* w, int n, int width, int groups,
                                        float eps, void* x_t, int dtype, void* stream);

/* out[r] = w * x[rows[r]] / rms per group as T (rows NULL: the first `count` rows). */
B200H_API int b200h_group_norm_rows(const void* x, const void* rows, const void* w, int count, int width, int groups, float eps, void* out,
                                    int dtype, void* stream);

/* hist[terms - 1] <- x; x <- sum_j coef[j] * hist[j] (j < terms); hist[j] starts hist_stride floats after hist[j - 1]. */
B200H_API int b200h_depth_mix(void* x, void* hist, int64_t hist_stride, const void* coef, int terms, int64_t count, void* stream);

/* Norm of both latents, rotation of the shared key part, cache store (fills cq). */
B200H_API int b200h_latent_prep(const b200h_latent_args* args);
/* Rotation of the per-head rotated query parts (fills q_rot). */
B200H_API int b200h_rotate_query(const b200h_latent_args* args);
/* Causal attention over the cached latents with the sink: score = scale * (q_lat . c + q_rot . kr) (fills o_heads). */
B200H_API int b200h_latent_attention(const b200h_latent_args* args);
/* y[t, h * vdim + v] = o[h, t, v] * sigmoid(gate[t, h * vdim + v]) as T; o float [heads, n, vdim] (the expanded values). */
B200H_API int b200h_head_gate(const void* o, const void* gate, int64_t ld_gate, int n, int heads, int vdim, void* y, int dtype, void* stream);

/* Per head S <- decay S + silu(k) silu(v)^T, out = S^T silu(q) (float [n, heads, vdim]); q, k, v are T with row stride ld;
 * state float [heads, vdim, dim] at state + seq_slot[s] * slot_stride, read and advanced. */
B200H_API int b200h_decay_attention(const void* q, const void* k, const void* v, int64_t ld, const void* decay, void* state,
                                    int64_t slot_stride, const void* cu_q, const void* seq_slot, int batch, int heads, int dim, int vdim,
                                    void* out, int dtype, void* stream);

/* y[t] = o[t] / rms(o[t]) * w * sigmoid(gate[t]) as T over `count` columns. */
B200H_API int b200h_gated_rms(const void* o, const void* w, const void* gate, int64_t ld_gate, int n, int count, float eps, void* y,
                              int dtype, void* stream);

/* softmax(router x) over all experts; ids / wts [n, top]: the top largest and their scores. */
B200H_API int b200h_route(const void* x, const void* router, int n, int width, int experts, int top, void* ids, void* wts, void* stream);
/* The same with x as float or T (x_dtype) and a choice of scores: score_fn 0 = softmax over all experts, 1 = sigmoid of every
 * logit on its own (the weights are the chosen experts' sigmoids, not renormalised). */
B200H_API int b200h_route_scored(const void* x, int x_dtype, const void* router, int n, int width, int experts, int top, int score_fn,
                                 void* ids, void* wts, void* stream);

/* Routed experts for a step of few rows (an expert's weights are read once for all rows that chose it), e = ids[t, k], w = wts[t, k]:
 *   act 0, scale_input 0:  out[t, k] = w * down_e (silu(gate_e x[t]) * (up_e x[t]))
 *   act 1 (no gate matrix): out[t, k] = w * down_e relu(up_e x[t])^2
 *   scale_input 1: the score multiplies the expert's input instead, expert_e(w x[t]); it is applied to the first products
 *   (linear in x), so the scaled input is never rounded to T. */
typedef struct b200h_expert_args {
    int n, width, ff, experts, top, dtype;
    const void* x;           /* T [n, width] */
    const void* gate;        /* T [experts, ff, width] */
    const void* up;          /* T [experts, ff, width] */
    const void* down;        /* T [experts, width, ff] */
    const void* ids;         /* int [n, top] */
    const void* wts;         /* float [n, top] */
    void* out;               /* float [n, top, width] */
    void* mid;               /* T [n * top, ff] scratch */
    void* counts;            /* int [experts] scratch */
    void* lists;             /* int [experts, n * top] scratch */
    void* stream;
    int act;                 /* 0: silu(gate) * up; 1: relu(up)^2 (gate is not read) */
    int scale_input;         /* 0: the score scales the expert's output; 1: its input */
} b200h_expert_args;
B200H_API int b200h_experts(const b200h_expert_args* args);

/* out = silu(g) * u element by element (T, `count` elements): between an expert's gate / up GEMMs and its down GEMM. */
B200H_API int b200h_silu_mul(const void* g, const void* u, void* out, int64_t count, int dtype, void* stream);

/* out[slot[r]] = wts[slot[r]] * src[r]: rows grouped by expert (src T [rows, width]) back to their (row, choice) places
 * (out float [rows, width], wts float [rows] or NULL for 1, slot int [rows]). */
B200H_API int b200h_weighted_scatter(const void* src, const void* slot, const void* wts, void* out, int rows, int width, int dtype,
                                     void* stream);

/* out[r] = index of the largest of logits[r, :vocab] (float, row stride ld; ties: the lowest index). */
B200H_API int b200h_argmax(const void* logits, int64_t ld, int rows, int vocab, void* out, void* stream);

/* ---- pre-norm blocks: learned positions, residual add + RMS norm, windowed attention with grouped key/value heads ---- */

/* x[t] += table[idx ? idx[t] : fixed] (x float [n, width], table T [rows, width], idx int [n] or NULL). */
B200H_API int b200h_add_rows(void* x, const void* table, const void* idx, int fixed, int n, int width, int dtype, void* stream);

/* x[t] += m[t] + extra (m T [n, width] or NULL, extra T [width] or NULL); then, if h is given, h[t] = x[t] / rms(x[t]) * w
 * (float [n, width]; w float [width] holds the full factor, i.e. one plus the stored deviation where a design stores that). */
B200H_API int b200h_residual_norm(void* x, const void* m, const void* extra, const void* w, int n, int width, float eps, void* h,
                                  int dtype, void* stream);

/* x <- relu(x)^2 in place (T, `count` elements). */
B200H_API int b200h_relu2(void* x, int64_t count, int dtype, void* stream);

/* One layer of softmax attention over a sliding window of a paged key/value cache, for one step.
 * Query head h reads key/value head h / (heads / kv_heads).  For the query at position i and a key at position j,
 * max(0, i - window + 1) <= j <= i (window 0: every j <= i):
 *   s = scale * (q . k);  s <- softcap * tanh(s / softcap) if softcap > 0;  s <- s - r1[h] * ln(1 + r2[h] * (i - j)) if r1;
 *   weight = softmax over j (with exp(sink[h]) added to the denominator if sink: a score that carries no value);
 *   weight_h <- sum_g talk[h, g] * weight_g if talk;  out_h = sum_j weight_h(j) * v_j;
 *   y = out * sigmoid(gate) if gate.
 * Cache entry of a position inside its page (page address + layer_off): the normed key as T at [pos % block_len][kv_heads * dim],
 * and, v_off bytes further, the value as T at [pos % block_len][kv_heads * vdim]. */
typedef struct b200h_window_args {
    int n, heads, kv_heads, dim, vdim, block_len, window, splits;
    float scale, softcap, eps;
    const void* q;           /* T [n, ld]: heads * dim columns */
    const void* k;           /* T [n, ld]: kv_heads * dim columns */
    const void* v;           /* T [n, ld]: kv_heads * vdim columns */
    int64_t ld;
    const void* bias;        /* float [heads * dim + kv_heads * dim + kv_heads * vdim] or NULL: added to q | k | v before anything else */
    const void* q_norm;      /* float [heads * dim] or NULL: RMS norm over the whole query projection */
    const void* k_norm;      /* float [kv_heads * dim] or NULL */
    void* qn;                /* float [n, heads * dim]: out of b200h_window_prep */
    const void* r1;          /* float [heads] or NULL */
    const void* r2;          /* float [heads] */
    const void* talk;        /* float [heads, heads] or NULL */
    const void* gate;        /* T [n, ld_gate] or NULL */
    int64_t ld_gate;
    void* ml;                /* float [n, heads, splits, 2] scratch */
    void* o_part;            /* float [n, splits, heads * vdim] scratch */
    void* scores;            /* float [n, heads, score_ld] scratch: a row's scores, indexed by key position - the row's first visible key */
    int64_t score_ld;        /* >= the most keys a row of the step sees: min(window, largest position + 1), all positions when window is 0 */
    void* y;                 /* T [n, heads * vdim]: out of b200h_window_attention */
    const void* tok_seq;     /* int [n] */
    const void* tok_pos;     /* int [n] */
    const void* block_ptrs;  /* int64: page addresses, entry s's pages from cu_blocks[s] */
    const void* cu_blocks;   /* int [batch + 1] */
    int64_t layer_off, v_off;
    int dtype;
    void* stream;
    const void* sink;        /* float [heads] or NULL */
    int chunk;               /* > 0: a query sees only keys j with j / chunk == i / chunk (chunks counted from position 0) */
    int talk_scores;         /* 1: talk mixes the heads' SCORES before the softmax (s_h <- sum_g talk[h, g] * s_g) instead of their weights */
    int gate_heads;          /* 1: gate is T [n, ld_gate] with ONE column per head instead of one per output column */
} b200h_window_args;
/* Bias, norm of query and key, cache store of key and value (fills qn). */
B200H_API int b200h_window_prep(const b200h_window_args* args);
/* The same for an attention that norms PER HEAD and rotates: bias, then every head of q and k divided by its root mean square over
 * dim and multiplied by q_norm / k_norm (float [dim], shared by all heads; NULL: no norm), then the rotation rot of every head; cache
 * store of key and (biased) value (fills qn). */
B200H_API int b200h_head_rope_prep(const b200h_window_args* args, const b200h_rotary* rot);
/* Attention of the step's rows over the cache (fills y); the step's own rows must have been stored by a prep entry. */
B200H_API int b200h_window_attention(const b200h_window_args* args);

/* ---- parallel blocks (both sublayers read the same stream), convolved rotary attention, state-space mixer ---- */

/* x[t] += mult * (mix[t] + sum_p ff[t, p]) + add[t] + extra, then h1[t] = x[t] / rms(x[t]) * w1 and h2[t] = ... * w2 as T.
 * mix T [n, width], ff float [n, parts, width], add float [n, width], extra T [width], h1, h2: each optional (NULL);
 * w1 / w2 float [width] hold the full factor; h2f (optional, with h2): the second norm as float too. */
B200H_API int b200h_parallel_residual_norm(void* x, const void* mix, const void* ff, int parts, float mult, const void* add, const void* extra,
                                           const void* w1, const void* w2, int n, int width, float eps, void* h1, void* h2, void* h2f,
                                           int dtype, void* stream);

/* out[t, c] = act(bias[c] + sum_j w[c, j] * u[t - taps + 1 + j, c]) as float [n, channels]; u T with row stride ld; w float
 * [channels, taps]; bias float [channels] or NULL; act 0 none, 1 silu.  Rows before an entry's first come from its state (float
 * [taps - 1, channels] at state + seq_slot[s] * slot_stride), which is then advanced by the step. */
B200H_API int b200h_short_conv(const void* u, int64_t ld, const void* w, const void* bias, int act, void* state, int64_t slot_stride,
                               const void* tok_seq, const void* cu_q, const void* seq_slot, void* out, int n, int batch, int channels,
                               int taps, int dtype, void* stream);

/* Per head h (group h / (heads / groups)): dt = softplus(dt + dt_bias[h]); S <- exp(-exp(a_log[h]) dt) S + dt B x^T;
 * out = S^T C + skip[h] x (float [n, heads * vdim]).  xbc float [n, heads * vdim + 2 * groups * nstate] = x | B | C;
 * dt T with row stride ld_dt, one column per head; state float [heads, vdim, nstate] at state + seq_slot[s] * slot_stride;
 * steps: float [n, heads, 2] scratch (every row's step size and decay, computed once per head). */
B200H_API int b200h_ssm_scan(const void* xbc, const void* dt, int64_t ld_dt, const void* dt_bias, const void* a_log, const void* skip,
                             void* state, int64_t slot_stride, const void* cu_q, const void* seq_slot, int n, int batch, int heads, int vdim,
                             int nstate, int groups, void* steps, void* out, int dtype, void* stream);

/* out[t] = unit_rms_per_group(y[t] * silu(gate[t])) * w as T; y float [n, count], gate T with row stride ld_gate, `groups` equal parts. */
B200H_API int b200h_gate_group_norm(const void* y, const void* gate, int64_t ld_gate, const void* w, int n, int count, int groups, float eps,
                                    void* out, int dtype, void* stream);

/* Preparation of an attention layer whose stacked projection qk (T [n, ld]: heads * dim query columns, then kv_heads * dim key
 * columns) passes a short causal convolution per channel (conv float [channels, taps], state float [taps - 1, channels] per slot),
 * then a rotation of every head's first 2 * rot.pairs dimensions, then a division by the head's root mean square.  The cache gets
 * the normed key (T, at layer_off) and, as the VALUE, the convolved key before rotation and norm (T, at layer_off + v_off),
 * laid out as b200h_window_args describes; qn gets the queries (float [n, heads * dim]). */
typedef struct b200h_conv_prep_args {
    int n, batch, heads, kv_heads, dim, taps, block_len;
    float eps;
    b200h_rotary rot;
    const void* qk;
    int64_t ld;
    const void* conv;
    void* state;
    int64_t slot_stride;
    void* qn;
    const void* tok_seq;     /* int [n] */
    const void* tok_pos;     /* int [n] */
    const void* cu_q;        /* int [batch + 1] */
    const void* seq_slot;    /* int [batch] */
    const void* block_ptrs;
    const void* cu_blocks;
    int64_t layer_off, v_off;
    int dtype;
    void* stream;
} b200h_conv_prep_args;
B200H_API int b200h_conv_rope_prep(const b200h_conv_prep_args* args);

/* x <- cap * tanh(x / cap) in place (float). */
B200H_API int b200h_softcap(void* x, int64_t count, float cap, void* stream);

/* u[r, :] <- relu(scale[r] * u[r, :])^2 in place (u T [rows, cols], scale float [rows] or NULL). */
B200H_API int b200h_scaled_relu2(void* u, const void* scale, int rows, int cols, int dtype, void* stream);


/* ---- parallel blocks with one norm and a token shift, side-by-side mixers, recurrence with a decay per channel and token ---- */

/* out[t] = table[tokens[t]] + second[row] (float), row = (previous token * mul_prev + tokens[t] * mul_cur) mod buckets, or `buckets`
 * (the table's last row) at position 0.  The token before an entry's first row is the int at prev + seq_slot[s] * slot_stride (in
 * a float's place), which then becomes the entry's last token of this step. */
B200H_API int b200h_embed_hashed(const void* tokens, const void* table, const void* second, int buckets, int mul_prev, int mul_cur, void* prev,
                                 int64_t slot_stride, const void* tok_seq, const void* tok_pos, const void* cu_q, const void* seq_slot,
                                 void* out, int n, int batch, int width, int dtype, void* stream);

/* x[t] += branch_scale * (left[t] / rms(left[t]) * wl + right[t] / rms(right[t]) * wr) + sum_p ff[t, p]; then, if w is given,
 * hf[t] = x[t] / rms(x[t]) * w (float) and h[t] the same as T.  left, right: T [n, width] (both or neither) with wl, wr float
 * [width]; ff: T (or float when ff_is_f32) [n, parts, width] or NULL; h, hf optional. */
B200H_API int b200h_branch_residual_norm(void* x, const void* left, const void* right, const void* wl, const void* wr, float branch_scale,
                                         const void* ff, int ff_is_f32, int parts, const void* w, int n, int width, float eps, void* h,
                                         void* hf, int dtype, void* stream);

/* Token shift of normed rows h (float [n, width]): a[t] = h[t] + (h[t-1] - h[t]) * shift (shift float [width] or NULL: a = h), and
 * for m < nmu blends[m][t] = a[t] + (a[t-1] - a[t]) * mu[m] (mu float [nmu, width]; a, blends T, blends [nmu, n, width]; a optional).
 * The rows before an entry's first come from its state (float [2, width] = its last h and a at state + seq_slot[s] * slot_stride;
 * zeros at a sequence's start), which is then advanced by the step. */
B200H_API int b200h_token_shift(const void* h, const void* shift, const void* mu, int nmu, void* state, int64_t slot_stride,
                                const void* tok_seq, const void* cu_q, const void* seq_slot, int n, int batch, int width, void* a,
                                void* blends, int dtype, void* stream);

/* Per head, S a [dim, vdim] float matrix per sequence:  w_t = exp(-exp(d_t + w0)) per key channel;
 * out_t = (S + diag(bonus) k_t v_t^T)^T r_t;  S <- diag(w_t) S + k_t v_t^T.  r, k (heads * dim columns) and v (heads * vdim) are T
 * with row stride ld; d float [n, heads * dim]; w0, bonus float [heads * dim]; state float [heads, vdim, dim] at state + seq_slot[s] *
 * slot_stride, read and advanced; decay: float [n, heads * dim] scratch; out float [n, heads * vdim]. */
B200H_API int b200h_channel_decay_scan(const void* r, const void* k, const void* v, int64_t ld, const void* d, const void* w0,
                                       const void* bonus, void* state, int64_t slot_stride, const void* cu_q, const void* seq_slot, int n,
                                       int batch, int heads, int dim, int vdim, void* decay, void* out, int dtype, void* stream);

/* y[t] = unit_rms_per_group(o[t]) * w * act(gate[t]) as T: the norm BEFORE the gate; o float [n, count], `groups` equal parts,
 * gate T with row stride ld_gate; act 0 sigmoid, 1 silu. */
B200H_API int b200h_group_norm_gate(const void* o, const void* w, const void* gate, int64_t ld_gate, int n, int count, int groups, int act,
                                    float eps, void* y, int dtype, void* stream);

/* x <- z > 0 ? softplus(p) z^2 + z / 2 : (1/2 + softplus(q)) (exp(z) - 1 - z) + z / 2 in place (T); params = {p, q} floats on the device. */
B200H_API int b200h_xielu(void* x, int64_t count, const void* params, int dtype, void* stream);

/* x <- tanh(x) in place (T). */
B200H_API int b200h_tanh(void* x, int64_t count, int dtype, void* stream);

/* Router with sigmoid scores s and groups of neighbouring experts: choice score = s + correction (float [experts] or NULL); a
 * group's score = the sum of its group_top largest choice scores; only experts of the `keep` best of `groups` equal groups can be
 * chosen; ids = the `top` largest choice scores; wts = the chosen s (without correction), / (their sum + 1e-20) if renorm, * scale. */
B200H_API int b200h_route_grouped(const void* x, int x_dtype, const void* router, const void* correction, int n, int width, int experts,
                                  int top, int groups, int keep, int group_top, int renorm, float scale, void* ids, void* wts, void* stream);

#endif
