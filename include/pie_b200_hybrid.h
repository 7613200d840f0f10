/* pie_b200_hybrid.h -- C ABI of libpie_b200_hybrid.so: sm_100a operators for models that mix recurrent and attention
 * layers over dense (unquantized) weights.  Built from csrc/hyb_*.cu; the page allocator of pie_b200.h is linked in too,
 * so a program that serves such a model needs this one library only.
 *
 * Conventions
 *   - every pointer is a DEVICE pointer; calls are asynchronous on `stream` (cudaStream_t as void*), allocate nothing,
 *     never synchronise and can be captured in CUDA graphs; the return value is a pie_status (pie_b200.h);
 *   - a step is RAGGED: T token rows, row t belongs to sequence tok_seq[t]; sequence i owns rows
 *     seq_start[i] .. seq_start[i] + seq_len[i] - 1 (consecutive positions seq_ctx[i] ..), keeps its recurrent state in
 *     slot seq_slot[i] and its keys / values in the 64-token pages named by row i of the block table;
 *   - dtype codes are PIE_DTYPE_BF16 / PIE_DTYPE_F32.  "act" tensors (inputs of matrix products, the key / value pages)
 *     are bf16 when the model is served in bf16 and fp32 when it runs in exact mode; the residual streams, norms,
 *     softmax, recurrent state and every gate of a recurrence are fp32 in both;
 *   - small parameters (norm weights, mixing weights, convolution taps, decay parameters) are fp32 arrays.
 */
#ifndef PIE_B200_HYBRID_H_
#define PIE_B200_HYBRID_H_

#include <stddef.h>
#include <stdint.h>

#include "pie_b200.h"

#ifdef __cplusplus
extern "C" {
#endif

int pieh_abi_version(void);
const char* pieh_last_cuda_error(void);
unsigned long long pieh_launch_count(void);
/* non-zero after a tensor-core pipeline gave up a bounded wait (the kernel returned early; its output is invalid).
 * Synchronises the device. */
unsigned int pieh_pipeline_error(void);
/* on: every operator is launched as a programmatic dependent of the launch before it on its stream (its blocks may become
 * resident early and wait at their top); captured into CUDA graphs as such.  Off by default. */
void pieh_set_pdl(int on);

/* epilogues of pieh_linear */
enum {
  PIEH_EPI_NONE = 0,
  PIEH_EPI_RELU2 = 1,    /* y <- max(y, 0)^2                                   */
  PIEH_EPI_SOFTCAP = 2,  /* y <- cap * tanh(y / cap)                           */
  PIEH_EPI_STREAMS = 3,  /* out is the residual [M, S, N] fp32: x[m, t, n] <- sum_s mix[s, t] x[m, s, n] + outw[t] * y */
  PIEH_EPI_GLU = 4,      /* gated pair (pieh_linear_glu only): out [M, N / 2]                                        */
  PIEH_EPI_SIGMUL = 5,   /* y <- y * sigmoid(gate[m, n])   (pieh_linear_batched only)                                */
  PIEH_EPI_TANH = 6,     /* y <- tanh(y)                   (pieh_linear_act only)                                    */
  PIEH_EPI_XIELU = 7     /* y <- a y^2 + y / 2 (y > 0),  b (e^y - 1 - y) + y / 2 (y <= 0)   (pieh_linear_act only)    */
};

/* ragged step descriptor, shared by the recurrent and the attention operators (all arrays int32, device) */
typedef struct pieh_batch {
  int T;                   /* token rows in the step                          */
  int n_seq;               /* sequences in the step                           */
  const int32_t* tok_seq;  /* [T]      sequence index of each row             */
  const int32_t* tok_pos;  /* [T]      position of each row in its sequence   */
  const int32_t* seq_start;/* [n_seq]  first row of the sequence              */
  const int32_t* seq_len;  /* [n_seq]  rows of the sequence in this step      */
  const int32_t* seq_ctx;  /* [n_seq]  tokens of the sequence before this step*/
  const int32_t* seq_slot; /* [n_seq]  state slot of the sequence             */
  const int32_t* block_table; /* [n_seq, bt_stride] page ids                  */
  int bt_stride;
  int n_tiles;             /* 64-row query tiles: every sequence's rows cut into runs of <= 64 (0: no tile list)  */
  const int32_t* tile_seq; /* [n_tiles] sequence of the tile                  */
  const int32_t* tile_row; /* [n_tiles] first row of the tile                 */
} pieh_batch;

/* y[m, n] = sum_k x[m, k] w[n, k] (+ bias[n]), fp32 accumulation.  w_dtype bf16: x is rounded to bf16 (if it is not
 * already) and the products are exact; w_dtype f32: plain fp32 multiply-add, no reduced-precision matrix mode.
 * bias fp32 or NULL.  epi_a: cap (SOFTCAP); STREAMS: out_ld = S * N is implied, mix [S, S] and outw [S] fp32, S <= 8. */
int pieh_linear(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld, const void* w,
                int w_dtype, const float* bias, int M, int N, int K, int epilogue, float epi_a, const float* mix,
                const float* outw, int S, void* stream);

/* pieh_linear with an activation that takes up to two constants: NONE, RELU2, TANH, or XIELU with a = act_a, b = act_b
 * (the caller passes the finished coefficients, e.g. softplus of learned numbers). */
int pieh_linear_act(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld, const void* w,
                    int w_dtype, const float* bias, int M, int N, int K, int act, float act_a, float act_b, void* stream);

/* nb independent products in one launch (one per head, say): for z < nb
 *   out[z * out_bs + m * out_ld + n] = sum_k x[z * x_bs + m * x_ld + k] * w[z * w_bs + n * K + k]
 * (strides in elements), with the same dtype rules as pieh_linear.  epilogue NONE, RELU2 or SIGMUL; SIGMUL multiplies by
 * sigmoid(gate[z * gate_bs + m * gate_ld + n]), gate fp32 logits. */
int pieh_linear_batched(void* out, int out_dtype, long long out_ld, long long out_bs, const void* x, int x_dtype,
                        long long x_ld, long long x_bs, const void* w, int w_dtype, long long w_bs, int nb, int M, int N,
                        int K, int epilogue, const float* gate, long long gate_ld, long long gate_bs, void* stream);

/* xs[t, s, :] = table[tokens[t], :] for every stream s.  xs fp32 [T, S, W]. */
int pieh_embed_streams(float* xs, const void* table, int table_dtype, const int32_t* tokens, int T, int S, int W,
                       int vocab, void* stream);
/* out[r, :] = rms_norm(sum_s in_w[s] xs[row(r), s, :]) * (unit_offset + norm_w);  in_w NULL = all ones; rows NULL =
 * identity.  out is an act tensor [R, W]. */
int pieh_stream_norm(void* out, int out_dtype, const float* xs, const int32_t* rows, const float* in_w,
                     const float* norm_w, float unit_offset, float eps, int R, int S, int W, void* stream);
/* xs[t, u, :] <- sum_s mix[s, u] xs[t, s, :] + outw[u] * y[t, :]   (y fp32 [T, W]) */
int pieh_stream_update(float* xs, const float* y, const float* mix, const float* outw, int T, int S, int W, void* stream);

/* ---- gated delta rule ----------------------------------------------------------------------------------------------
 * proj fp32 [T, ld]: columns [q (G dk) | k (G dk) | v (H dv) | gate (H dv) | b (H) | a (H)] of the fused projection. */
typedef struct pieh_delta {
  int H, G, dk, dv, taps;
  const float* conv_w;   /* [(2 G dk + H dv), taps]; last tap multiplies the current token */
  const float* A_log;    /* [H] */
  const float* dt_bias;  /* [H] */
  const float* out_norm; /* [dv] */
  float eps;             /* of the output norm */
  float* conv_state;     /* [slots, taps - 1, 2 G dk + H dv] fp32, oldest first */
  float* state;          /* [slots, H, dk, dv] fp32 */
} pieh_delta;
/* convolution + silu, unit-length q (times dk^-1/2) and k, beta and decay per head; then the convolution history of
 * every sequence moves on.  q, k fp32 [T, G, dk]; v fp32 [T, H, dv]; beta, decay fp32 [T, H]. */
int pieh_delta_prepare(float* q, float* k, float* v, float* beta, float* decay, const float* proj, long long ld,
                       const pieh_delta* d, const pieh_batch* b, void* stream);
/* the recurrence over each sequence's rows, state read from and written back to its slot (a sequence with no context
 * starts from zero whatever the slot holds); o fp32 [T, H, dv]. */
int pieh_delta_scan(float* o, const float* q, const float* k, const float* v, const float* beta, const float* decay,
                    const pieh_delta* d, const pieh_batch* b, void* stream);
/* out[t, h, :] = o[t, h, :] / rms(o[t, h, :]) * out_norm * silu(gate[t, h, :]); gate = proj + gate_off, row stride ld */
int pieh_delta_gate(void* out, int out_dtype, const float* o, const float* proj, long long ld, long long gate_off,
                    const pieh_delta* d, int T, void* stream);

/* ---- differential attention with a sliding window over 64-token pages ----------------------------------------------
 * proj fp32 [T, ld]: columns [q (H, 2, d) | k (G, 2, d) | v (G, dv)]. */
typedef struct pieh_attn {
  int H, G, d, dv;
  int rot_dims;            /* leading features of each map that rotate (adjacent pairs); 0 = none */
  const double* rot_freqs; /* [rot_dims / 2] angle per position */
  const float* q_norm;     /* [d] plain weight, or NULL = no query / key norm */
  const float* k_norm;
  float eps;
  float scale, softcap;    /* softcap 0 = none */
  int window;              /* visible keys per query (itself included); 0 = all earlier ones */
  float lambda;            /* weight of the second map */
  float out_scale;         /* applied after the per-head unit-rms of (map1 - lambda map2) */
  void* k_pages;           /* [pages, 64, G, 2 d] act dtype */
  void* v_pages;           /* [pages, 64, G, dv]  act dtype */
  int kv_dtype;
} pieh_attn;
/* norm + rotation of q and k; k and v appended to the pages at each row's position.  q_out fp32 [T, H, 2, d]. */
int pieh_attn_prepare(float* q_out, const float* proj, long long ld, const pieh_attn* a, const pieh_batch* b,
                      void* stream);
/* out[t, h, :] act [T, H dv]: both maps' windowed softmax attention over the pages, combined and normalised. */
int pieh_attn_run(void* out, int out_dtype, const float* q, const pieh_attn* a, const pieh_batch* b, void* stream);

/* ---- gated linear units -------------------------------------------------------------------------------------------
 * w [N, K] holds the gate and the linear half INTERLEAVED: row 2 j is gate row j, row 2 j + 1 the linear ("up") row j.
 * out[m, j] = g' * sigmoid(alpha * g') * (u' + up_offset), with g' = min(g, limit), u' = clamp(u, -limit, limit) when
 * limit > 0 and g' = g, u' = u when limit == 0.  alpha 1, limit 0, up_offset 0 is silu(g) * u.  out is [M, N / 2]. */
int pieh_linear_glu(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld, const void* w,
                    int w_dtype, int M, int N, int K, float alpha, float limit, float up_offset, void* stream);

/* ---- learned absolute positions and the post-norm residual ----------------------------------------------------------
 * x[t, :] = table[tokens[t], :] + pos_table[positions[t], :] (fp32), act[t, :] = the same rounded to the act dtype
 * (act may be NULL).  pos_table NULL: no position term. */
int pieh_embed_positions(float* x, void* act, int act_dtype, const void* table, const void* pos_table, int table_dtype,
                         const int32_t* tokens, const int32_t* positions, int T, int W, int vocab, int max_positions,
                         void* stream);
/* A sublayer's output joins the residual through its OWN norm:  x[t, :] += rms_norm(y[t, :]) * norm_w,  then
 * act[t, :] = x[t, :] in the act dtype (the next sublayer's matrix-product input; may be NULL).
 * y is either a plain fp32 [T, W] tensor (parts = NULL) or gathered on the fly from a mixture:
 *   y[t, :] = sum_k part_w[t, k] * parts[part_row[t * top + k], :]  +  (shared ? shared_gate[t * gate_ld] * shared[t, :] : 0)
 * shared_gate holds LOGITS (the sigmoid is taken here). */
typedef struct pieh_mix_sum {
  const float* parts;        /* [rows, W] fp32 or NULL */
  const int32_t* part_row;   /* [T * top] */
  const float* part_w;       /* [T * top] */
  int top;
  const float* shared;       /* [T, W] fp32 or NULL */
  const float* shared_gate;  /* logits, element t * gate_ld */
  long long gate_ld;
} pieh_mix_sum;
int pieh_postnorm_add(float* x, void* act, int act_dtype, const float* y, const pieh_mix_sum* mix, const float* norm_w,
                      float eps, int T, int W, void* stream);

/* ---- attention with a linear distance bias, a softmax sink and an output gate, over 64-token pages -------------------
 * proj fp32 [T, ld]: q at column 0 (H d), k at k_off (G d), v at v_off (G dv; v_off == k_off: the values are the
 * projected keys), gate logits at g_off (H dv; g_off < 0: no gate).
 *   q' = rms_norm(q over all H d features) * q_norm * (1 + temp_coef * ln(floor((p + 1) / temp_every) + 1))
 *   k' = rms_norm(k over all G d features) * k_norm            (q_norm / k_norm NULL: no norm; temp_every 0: no factor)
 *   s_ij = q'_i . k'_j * scale - slopes[h] * (i - j),   j <= i  (and i - j < window when window > 0)
 *   p_ij = exp(s_ij) / (sink + sum_j exp(s_ij))                 (sink 1: one extra term of score 0 without a value)
 *   out[i, h, :] = sum_j p_ij v_j * sigmoid(gate[i, h, :]) */
typedef struct pieh_bias_attn {
  int H, G, d, dv;
  long long k_off, v_off, g_off;
  const float* q_norm;     /* [H d] */
  const float* k_norm;     /* [G d] */
  float eps;
  float scale;
  float temp_coef;
  double temp_every;     /* positions per temperature step (need not be whole); 0 = no temperature */
  const float* slopes;     /* [H] or NULL = no distance bias */
  int sink;
  int window;
  void* k_pages;           /* [pages, 64, G, d]  act dtype */
  void* v_pages;           /* [pages, 64, G, dv] act dtype */
  int kv_dtype;
  /* optional pieces (all zero / NULL: off) */
  const float* sinks;      /* [H] learned sink logits: the denominator gains exp(sinks[h]) (unscaled, once) instead of the
                              score-0 term of `sink` */
  int gate_heads;          /* 1: the gate at g_off holds ONE logit per head ([H]) instead of one per output feature */
  int rot_dims;            /* leading features of every query / key head that rotate, feature i paired with i + rot_dims / 2 */
  const float* rot_cs;     /* [T, rot_dims / 2, 2] (cos, sin) of each row's angles: pieh_rot_table */
  const float* v_mix;      /* device scalar lambda: v <- (1 - lambda) v + lambda v_keep[t] before the pages are written */
  float* v_keep;           /* [T, G dv] fp32: read when v_mix is set; otherwise, if not NULL, this call's values are left here */
  int sigmoid;             /* 1: no softmax -- a visible key weighs sigmoid(s_ij + score_bias[h]), the weights are not normalised
                              over the keys and there is no sink */
  const float* score_bias; /* [H] added to the score inside the sigmoid (NULL: none) */
} pieh_bias_attn;
/* q_out fp32 [T, H, d]; k' and v appended to the pages at each row's position.  Rotation (after the norms) turns the pair
 * (u, v) = (x[i], x[i + rot_dims / 2]) into (u cos - v sin, v cos + u sin). */
int pieh_bias_attn_prepare(float* q_out, const float* proj, long long ld, const pieh_bias_attn* a, const pieh_batch* b,
                           void* stream);
/* cs[t, i] = (cos, sin)(positions[t] * freqs[i]), the angle formed in double precision.  cs fp32 [T, half, 2]. */
int pieh_rot_table(float* cs, const int32_t* positions, const double* freqs, int T, int half, void* stream);
/* out act [T, H dv]; proj is read for the gate.  dv <= 512. */
int pieh_bias_attn_run(void* out, int out_dtype, const float* q, const float* proj, long long ld,
                       const pieh_bias_attn* a, const pieh_batch* b, void* stream);

/* ---- mixture of experts ---------------------------------------------------------------------------------------------
 * Routing of T tokens over E experts from fp32 router logits z [T, ld]:  s = sigmoid(z); the experts form n_groups equal
 * groups of neighbours, a group scores the sum of its two largest s (its only one when a group is one expert), the
 * keep_groups best groups stay eligible, and the `top` eligible experts with the largest s are chosen with weight
 * s * scale (no renormalisation).  Ties go to the lower index.
 * The plan sorts the T * top (token, choice) pairs by expert into SLOTS: slot_row[s] = token row, slot_expert[s],
 * pair_slot[t * top + k] = slot, pair_w[t * top + k] = weight; tiles64 / tiles128 list the runs of <= 64 / 128 slots of
 * one expert as [count, (expert, first slot, slots) ...] for the grouped products. */
typedef struct pieh_moe_plan {
  int E, top, n_groups, keep_groups;
  float scale;
  int32_t* slot_row;     /* [T * top] */
  int32_t* slot_expert;  /* [T * top] */
  int32_t* pair_slot;    /* [T * top] */
  float* pair_w;         /* [T * top] */
  int32_t* tiles64;      /* [1 + 3 * (T * top / 64 + E)]  */
  int32_t* tiles128;     /* [1 + 3 * (T * top / 128 + E)] */
  int32_t* counters;     /* [2 * E + 2] scratch */
  int softmax_top;       /* 1: no groups, no sigmoid: the `top` largest LOGITS are chosen and weigh softmax over the chosen
                            logits only (times scale) */
} pieh_moe_plan;
int pieh_moe_route(const float* z, long long ld, const pieh_moe_plan* p, int T, void* stream);
/* Grouped product over the slots: out[s, :] = x[row(s), :] W_e(s)^T with W_e = w + e * w_stride elements, row(s) =
 * slot_row[s] when gather_rows else s.  P = T * top slots.  glu 1: as pieh_linear_glu (silu when alpha 1, limit 0);
 * glu 2: no pair, out = max(y, 0)^2;  glu 0: plain. */
int pieh_moe_linear(void* out, int out_dtype, long long out_ld, const void* x, int x_dtype, long long x_ld, const void* w,
                    int w_dtype, long long w_stride, int P, int N, int K, int gather_rows, int glu, float alpha,
                    float limit, float up_offset, const pieh_moe_plan* p, void* stream);

/* ---- parallel pre-norm blocks with a causal input convolution ------------------------------------------------------
 * x[t, :] = table[tokens[t], :] * scale   (fp32 residual) */
int pieh_embed_scaled(float* x, const void* table, int table_dtype, const int32_t* tokens, float scale, int T, int W,
                      int vocab, void* stream);
/* The residual takes a block's output and the NEXT block's norm is formed in the same pass:
 *   x[t, :] += (y ? y[t, :] : 0) + (mix ? mixture as in pieh_postnorm_add : 0)      (a NULL shared_gate: the shared rows count fully)
 *   h[t, :]  = x[t, :] / sqrt(mean(x[t, :]^2) + eps) * norm_w                          (skipped when h or norm_w is NULL)
 * x, h fp32 [T, W]. */
int pieh_residual_norm(float* x, const float* y, const pieh_mix_sum* mix, float* h, const float* norm_w, float eps, int T,
                       int W, void* stream);
/* Causal convolution over time on every channel, added to its input, for up to 4 tap sets that read the same h:
 *   out_k[t, c] = h[t, c] + sum_j w_k[c, j] * h[t - taps + 1 + j, c]        (rows before the sequence's start are zero)
 * The last taps - 1 rows of h of every sequence are its state (fp32, oldest first, in the sequence's slot); the call reads
 * the state for rows that reach back before the step and then moves it on. */
typedef struct pieh_canon {
  int taps, n_out;
  const float* w[4];   /* [W, taps] fp32 each */
  void* out[4];        /* act [T, W] each */
  float* state;        /* [slots, taps - 1, W] fp32 (unused when taps == 1) */
} pieh_canon;
int pieh_canon_conv(const pieh_canon* c, int out_dtype, const float* h, int W, const pieh_batch* b, void* stream);

/* ---- minGRU: a gated recurrence whose gates read the current token only ------------------------------------------------
 * proj fp32 [T, ld]: columns [z logits | u | gate], `width` each.  z = sigmoid(.), candidate = u + 1/2 (u >= 0) or
 * sigmoid(u) (u < 0), S_t = (1 - z) S_(t-1) + z candidate per channel, out[t, :] = S_t * silu(gate).  state fp32
 * [slots, width]: read unless the sequence has no context, written back at the end.  scratch: fp32 [3, n_tiles, width], used
 * when a sequence brings more than 64 rows (the batch's tile list cuts them into runs that are scanned in parallel); NULL:
 * always the one-pass kernel. */
int pieh_mingru_scan(void* out, int out_dtype, const float* proj, long long ld, int width, float* state, float* scratch,
                     const pieh_batch* b, void* stream);

/* ---- latent attention: the cached latent and the query latent ------------------------------------------------------------
 * proj fp32 [T, ld]: the query latent at column 0 (q_rank) and the key / value latent at kv_off (kv_rank).  Both get an
 * RMS norm with a plain weight; the query latent goes to cq_out (act [T, q_rank]), the other to the pages
 * [pages, 64, kv_rank] at each row's position.  The attention over the latent itself is pieh_bias_attn_run with one
 * key / value head of kv_rank features whose key and value pages are the same pool. */
int pieh_latent_prepare(void* cq_out, int out_dtype, const float* proj, long long ld, int q_rank, long long kv_off,
                        int kv_rank, const float* q_norm, const float* kv_norm, float eps, void* pages, int kv_dtype,
                        const pieh_batch* b, void* stream);

/* ---- sandwich-norm residual: a sublayer's output passes its own norm on the way into the residual, and the next
 * sublayer's input norm is formed in the same pass ------------------------------------------------------------------------
 *   x[t, :] += mult * rms_norm(y[t, :]) * post_w          y plain fp32 [T, W], or the mixture of pieh_postnorm_add (a NULL
 *                                                          shared_gate: the shared rows count fully); skipped when both are NULL
 *   x[t, :] += add_rows[t, :] + add_vec[:]                 each optional (a looped stack re-injects its input this way)
 *   h[t, :]  = rms_norm(x[t, :]) * next_w                  act dtype; skipped when h or next_w is NULL */
int pieh_sandwich_add(float* x, const float* y, const pieh_mix_sum* mix, const float* post_w, float mult,
                      const float* add_rows, const float* add_vec, void* h, int h_dtype, const float* next_w, float eps,
                      int T, int W, void* stream);

/* out[t, c] = norm-and-gate of x[t, :] in `groups` equal parts of group_size features, each by its own root mean square:
 *   gate_first 0:  x / rms(x) * w * f(gate)          gate_first 1:  (x f(gate)) / rms(x f(gate)) * w
 * f: gate_fn 0 none (gate may be NULL), 1 sigmoid, 2 silu.  x fp32 row stride x_ld, gate fp32 row stride gate_ld,
 * w [groups * group_size], out act [T, groups * group_size]. */
int pieh_gated_group_norm(void* out, int out_dtype, const float* x, long long x_ld, const float* gate, long long gate_ld,
                          const float* w, int groups, int group_size, float eps, int gate_fn, int gate_first, int T,
                          void* stream);

/* ---- generalized delta rule: per-channel decay and a removal term along the unit key ---------------------------------------
 * proj fp32 [T, ld] holds r at r_off, k at k_off (H dk each), v at v_off (H dv) and the removal logits at a_off (H dk).
 *   w = exp(-decay_scale * sigmoid(decay_logits)),  a = sigmoid(a_logits + a_bias),  u = k / sqrt(|k|^2 + key_eps)  per head
 *   S_t = diag(w) S_(t-1) - (a * u)(u^T S_(t-1)) + k v^T      (S [dk, dv]; both corrections read the old state)
 *   o_t = S_t^T r */
typedef struct pieh_gdelta {
  int H, dk, dv;
  long long r_off, k_off, v_off, a_off;
  const float* a_bias;   /* [H dk] or NULL */
  float decay_scale, key_eps;
  float* state;          /* [slots, H, dk, dv] fp32 */
} pieh_gdelta;
/* decay, u, au fp32 [T, H, dk]; decay_logits fp32 [T, dl_ld] (their bias already added). */
int pieh_gdelta_prepare(float* decay, float* u, float* au, const float* proj, long long ld, const float* decay_logits,
                        long long dl_ld, const pieh_gdelta* d, int T, void* stream);
/* the recurrence over each sequence's rows (state from and back to its slot; no context: from zero).  o fp32 [T, H, dv]. */
int pieh_gdelta_scan(float* o, const float* proj, long long ld, const float* decay, const float* u, const float* au,
                     const pieh_gdelta* d, const pieh_batch* b, void* stream);

/* ---- selective state space layer in its scalar-decay ("state-space duality") form --------------------------------------------
 * proj fp32 [T, ld]: the convolved channels [x (H P) | B (G N) | C (G N)] start at xbc_off, the H step-size logits at dt_off.
 *   channels <- silu(causal conv over time + conv_b)         history of taps - 1 rows per sequence slot, zeros before the start
 *   dt = softplus(dt_logit + dt_bias),  decay = exp(-exp(A_log) dt)              per head
 *   S_t = decay S_(t-1) + dt B_t x_t^T   (S [N, P], head h reads group h / (H / G));   y_t = S_t^T C_t + D x_t */
typedef struct pieh_ssd {
  int H, P, N, G, taps;
  long long xbc_off, dt_off;
  const float* conv_w;   /* [H P + 2 G N, taps]; the last tap multiplies the current token */
  const float* conv_b;   /* [H P + 2 G N] or NULL */
  const float* dt_bias;  /* [H] */
  const float* A_log;    /* [H] */
  const float* D;        /* [H] */
  float* conv_state;     /* [slots, taps - 1, H P + 2 G N] fp32, oldest first (unused when taps == 1) */
  float* state;          /* [slots, H, N, P] fp32 */
} pieh_ssd;
/* xbc fp32 [T, H P + 2 G N] after convolution and silu; dtd fp32 [T, H, 2] = (dt, decay); then the histories move on. */
int pieh_ssd_prepare(float* xbc, float* dtd, const float* proj, long long ld, const pieh_ssd* s, const pieh_batch* b,
                     void* stream);
/* y fp32 [T, H P]. */
int pieh_ssd_scan(float* y, const float* xbc, const float* dtd, const pieh_ssd* s, const pieh_batch* b, void* stream);

#ifdef __cplusplus
}
#endif
#endif
