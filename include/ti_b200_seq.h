/*
 * ti_b200_seq.h -- C ABI of libturboinfer_b200_seq.so: the layered sequence engine.
 *
 * A decoder is described layer by layer (ti_seq_layer_desc) instead of by one fixed block, and it is stepped over a RAGGED
 * batch: every step brings the next tokens of some of the live sequences -- a portion of a prompt for one, a single decoded
 * token for another -- and all of them run together.  The engine owns
 *   - a page pool for the attention layers' keys and values (64 tokens a page, one page table per sequence shared by all
 *     attention layers; pages return to the free list when a sequence is closed and are handed out again),
 *   - state slots for the recurrent layers (one slot per live sequence, reused the same way),
 *   - the step function, the continuous-batching generation loop on top of it and the on-device sampler.
 * Conventions as in ti_b200.h: 0 = success, ti_seq_last_error() has the message, no CPU fallback, opaque 64-bit handles.
 * Linear weights are [out, in] row-major and applied as W x.
 */
#ifndef TI_B200_SEQ_H
#define TI_B200_SEQ_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef uint64_t ti_seq_model_t;

enum {
    TI_SEQ_MIXER_ATTENTION = 0, /* softmax attention over cached keys / values (windowed, grouped, rotary) */
    TI_SEQ_MIXER_WKV = 1,       /* token-shifted linear recurrence, output read before the state is updated, bonus term */
    TI_SEQ_MIXER_GLA = 2,       /* gated linear attention: S <- diag(a) S + k v^T, o = S^T q, a = sigmoid(.)^(1/tau) per key channel */
    TI_SEQ_MIXER_HGRN2 = 3,     /* the same recurrence with the forget gate f as decay and 1 - f as the written key */
    TI_SEQ_MIXER_LATENT = 4     /* softmax attention whose keys / values are linear images of a cached low-rank vector + one shared rotated key part */
};
enum {
    TI_SEQ_ACT_RELU = 0, TI_SEQ_ACT_SILU = 1, TI_SEQ_ACT_GELU_TANH = 2,
    TI_SEQ_ACT_XIELU = 3 /* a z^2 + z / 2 for z > 0, b (exp(z) - 1 - z) + z / 2 otherwise; a = softplus(act[0]), b = 1/2 + softplus(act[1]) */
};
enum {
    TI_SEQ_FF_GLU = 0,      /* down(act(gate h) * up h) */
    TI_SEQ_FF_POLYNORM = 1, /* down(a N(z) + b N(z^2) + c N(z^3) + e), z = up h, N = division by the RMS over the inner size */
    TI_SEQ_FF_EXPERTS = 2,  /* routed gated experts (+ identity experts, + a shared expert) */
    TI_SEQ_FF_DENSE = 3     /* down(act(up h)) with ff_act (its learned numbers, if it has any, in "mlp.act") */
};
enum {
    TI_SEQ_ROUTE_SOFTMAX_ALL = 0, /* softmax over all router outputs, choice by score + correction inside the best groups, weights renormalised */
    TI_SEQ_ROUTE_TOP_LOGITS = 1   /* logits + bias ("mlp.router.b"); the `top` largest are chosen, weights = softmax over the chosen logits */
};
enum {
    TI_SEQ_QK_NORM_NONE = 0,
    TI_SEQ_QK_NORM_HEAD = 1,   /* q and k divided by their RMS per head (after rotation), no weights */
    TI_SEQ_QK_NORM_WHOLE = 2   /* RMS over the whole projection (all heads at once) times a plain weight "mix.q.norm" / "mix.k.norm" */
};
enum {
    TI_SEQ_NORMS_AROUND = 0, /* a norm in front of every sublayer ("norm1", "norm2") and one behind it ("norm1b", "norm2b") */
    TI_SEQ_NORMS_BEHIND = 1, /* the sublayers read the residual stream itself; one norm behind each ("norm1", "norm2") */
    TI_SEQ_NORMS_FRONT = 2   /* one norm in front of every sublayer ("norm1", "norm2"), none behind it */
};
enum {
    TI_SEQ_NORM_SCALAR = 0 /* one gain for all coordinates */, TI_SEQ_NORM_ONE_PLUS = 1 /* per-coordinate gain stored as w, applied as 1 + w */,
    TI_SEQ_NORM_VECTOR = 2 /* per-coordinate gain applied as it is stored */
};
enum {
    TI_SEQ_SINK_NONE = 0,
    TI_SEQ_SINK_LEARNED = 1, /* the softmax denominator has one more term exp(sink[head]) ("mix.sink") without key or value */
    TI_SEQ_SINK_ZERO = 2     /* the same term with a fixed score of 0: p_j = exp(s_j) / (1 + sum exp(s)); no tensor */
};
enum { TI_SEQ_BF16 = 0, TI_SEQ_F32 = 1 };   /* compute mode of a model, and element type of a tensor handed to set_tensor */

typedef struct ti_seq_layer_desc {
    int32_t mixer;           /* TI_SEQ_MIXER_* */
    int32_t heads, kv_heads; /* query heads, key/value heads (wkv: heads only) */
    int32_t dim, vdim;       /* per-head query/key size, value size (wkv: dim only) */
    int32_t window;          /* attention: a position sees itself and the window - 1 before it; 0 = everything before it */
    int32_t rot_dims;        /* leading coordinates of each head that are rotated, paired (2i, 2i+1); 0 = no rotation */
    float rot_base;
    int32_t rot_scaled;      /* 1: wavelength-dependent slow-down of the frequencies with the four numbers below */
    float rot_factor, rot_low, rot_high, rot_original;
    int32_t qk_norm;         /* TI_SEQ_QK_NORM_* */
    int32_t out_gate;        /* 1: head output times sigmoid of a per-head projection of the mixer input */
    float scale;             /* attention score scale */
    int32_t decay_rank;      /* wkv: inner size of the decay's two-matrix projection */
    int32_t ff;              /* feed-forward inner size, 0 = the layer has no feed-forward */
    int32_t ff_act;          /* TI_SEQ_ACT_* of the gate branch */
    /* -- gated linear recurrences (gla, hgrn2): heads, dim (key channels), vdim (value channels) above -- */
    float decay_tau;         /* gla: decay = sigmoid(z)^(1 / tau); its two-matrix projection has inner size decay_rank */
    /* -- latent attention: dim = unrotated query/key size, rot_dims = rotated part (one key part shared by the heads), vdim -- */
    int32_t kv_rank;         /* size of the cached low-rank vector */
    int32_t kv_from;         /* -1: the layer projects and caches its own; j: it reads layer j's cache (j before this layer) */
    int32_t sink;            /* TI_SEQ_SINK_* */
    /* -- feed-forward -- */
    int32_t ff_kind;         /* TI_SEQ_FF_*; `ff` is the inner size of the dense forms and of one routed expert */
    int32_t experts;         /* routed experts with weights */
    int32_t identity;        /* router outputs behind them whose expert returns its input */
    int32_t top;             /* experts a token uses */
    int32_t groups, groups_keep; /* experts (identity included) form `groups` equal groups of neighbours; only the best `groups_keep` can be chosen */
    int32_t shared_ff;       /* inner size of the expert every token uses, scaled by a sigmoid of one more projection; 0 = none */
    /* -- around the sublayers -- */
    int32_t res_gate;        /* 1: every sublayer's result is multiplied by sigmoid(R h + b) of its input before the norm behind it */
    /* -- attention: what happens to a score between the dot product and the softmax, and which keys a row sees -- */
    float softcap;           /* > 0: score <- cap * tanh(score / cap) after scaling */
    int32_t talk;            /* 1: the heads' scores of a (query, key) pair are mixed before masking, score_h <- sum_g T[h][g] score_g, T = "mix.talk" [heads][heads] */
    int32_t keep_first;      /* with a window: keys at positions < keep_first stay visible to every later row */
    /* (`sink` above also applies to TI_SEQ_MIXER_ATTENTION: "mix.sink" [heads]) */
    /* -- feed-forward, routed experts -- */
    int32_t route_kind;      /* TI_SEQ_ROUTE_* */
    int32_t shared_plain;    /* 1: the shared expert is added as it is (no sigmoid scale, no "mlp.shared.sg") */
    /* -- around the sublayers -- */
    int32_t conv_taps;       /* >= 1: the mixer reads h + conv(h), a causal depth-wise convolution over the last `conv_taps` inputs of the
                                sequence ("canon1" [width][taps], zeros before position 0); the last taps - 1 inputs are sequence state */
    int32_t layer_scale;     /* 1: each sublayer's normed result is multiplied coordinate by coordinate by "ls1" / "ls2" before the residual sum */
    int32_t conv_ff;         /* 1 (with conv_taps >= 1): the feed-forward reads through a convolution of its own too ("canon2") */
    /* -- rotation, attention and latent attention -- */
    int32_t rot_half;        /* 1: rotated coordinate i pairs with i + rot_dims / 2 instead of (2i, 2i + 1) */
    float rot_linear;        /* > 0: every frequency is divided by this number (independent of the wavelength) */
    /* -- attention -- */
    int32_t proj_bias;       /* 1: the q, k, v and output projections add biases ("mix.q.b", "mix.k.b", "mix.v.b", "mix.o.b") */
    int32_t v_norm;          /* 1: every value head is divided by its RMS (no weight) before it is cached */
    int32_t head_temp;       /* 1: the scaled score of query head h is multiplied by "mix.temp"[h] */
    /* -- latent attention (`window` and `out_gate` above apply to it as well: "mix.g" [heads][width]) -- */
    int32_t q_rank;          /* > 0: queries through a low-rank vector: q = Uq norm(Dq h) ("mix.dq" [q_rank][width], "mix.dq.norm",
                                "mix.uq" [heads * (dim + rot_dims)][q_rank]); 0: "mix.q" */
} ti_seq_layer_desc;

typedef struct ti_seq_model_desc {
    int32_t vocab, width, n_layers;
    int32_t loop_start, loop_stop, loop_times; /* layers [start, stop) run `times` times with the same weights and their own
                                                  cache / state per pass, each pass entered through the input projection of
                                                  [x; embedding]; times = 0: no looped block */
    float norm_eps, logit_scale;
    int32_t mode;            /* TI_SEQ_BF16 / TI_SEQ_F32 */
    int32_t max_tokens;      /* tokens the page pool holds (each sequence's count rounds up to whole pages) */
    int32_t max_seqs;        /* state slots = sequences that can be live at once */
    int32_t norm_kind;       /* TI_SEQ_NORM_* of the norms around the sublayers and in front of the head */
    float logit_softcap;     /* > 0: logits <- cap * tanh(logits / cap) */
    int32_t side_dim;        /* > 0: after every layer a per-token side input is added: side.embed[token][layer * side_dim ...] gated by
                                gelu_tanh(side.gate x), projected back and RMS-normed with a plain per-coordinate weight */
    int32_t norm_place;      /* TI_SEQ_NORMS_* */
    float pos_base;          /* > 0: a sinusoidal position vector is added to the embedding: entry 2i = sin(p * base^(-2i/width)),
                                entry 2i + 1 = cos of the same angle */
    int32_t tied_head;       /* 1: the logits are products with the embedding table (no "head" tensor) */
    int32_t loop_plain;      /* 1: the passes of the looped block follow one another directly (no "loop.in" projection) */
    int32_t streams;         /* >= 1: hyper-connections.  The residual is `streams` copies X_s of the embedding output; sublayer q of a layer
                                reads u = sum_s hcq.in[s] X_s and, with its result y, all copies are rewritten at once from the old ones:
                                X_t <- sum_s hcq.mix[s][t] X_s + hcq.out[t] y ("l<i>.hc1.*" mixer, "l<i>.hc2.*" feed-forward); the model's
                                output is sum_s X_s.  Needs TI_SEQ_NORMS_FRONT.  0: one residual stream, x <- x + y */
} ti_seq_model_desc;

int ti_seq_init(int device);
const char* ti_seq_last_error(void);
uint64_t ti_seq_launch_count(void);

int ti_seq_model_new(const ti_seq_model_desc* desc, const ti_seq_layer_desc* layers, ti_seq_model_t* out);
/* tensor names: "embed", "side.embed", "loop.in", "final.norm", "head", "l<i>.norm1|norm1b|norm2|norm2b", "l<i>.rg1|rg2[.b]",
 * "l<i>.ls1|ls2", "l<i>.canon1|canon2", "l<i>.hc1|hc2.in|out|mix", "l<i>.mix.<x>", "l<i>.mlp.<x>", "l<i>.side.<x>";
 * `dtype` is the element type of `data` (TI_SEQ_BF16: raw bfloat16 bits, TI_SEQ_F32) */
int ti_seq_model_set_tensor(ti_seq_model_t m, const char* name, int32_t dtype, const void* data, const int64_t* shape, int32_t ndim);
/* uniform(-amp, amp) + offset generated on the device from (seed, element index): benchmark-size models */
int ti_seq_model_set_tensor_synthetic(ti_seq_model_t m, const char* name, const int64_t* shape, int32_t ndim, uint64_t seed, float amp,
                                      float offset);
/* number of tensors the description requires, and the name / shape of the i-th */
int ti_seq_model_tensor_count(ti_seq_model_t m, int32_t* n);
int ti_seq_model_tensor_info(ti_seq_model_t m, int32_t i, char* name, size_t cap, int64_t* shape, int32_t* ndim);
int ti_seq_model_finalize(ti_seq_model_t m);
int ti_seq_model_free(ti_seq_model_t m);

/* a sequence takes a state slot when opened; its pages are allocated as its tokens arrive; close gives both back */
int ti_seq_open(ti_seq_model_t m, int32_t* seq);
int ti_seq_close(ti_seq_model_t m, int32_t seq);
int ti_seq_length(ti_seq_model_t m, int32_t seq, int32_t* tokens);
int ti_seq_pool_info(ti_seq_model_t m, int32_t* free_pages, int32_t* total_pages, int32_t* free_slots, int32_t* page_tokens);
/* physical pages of a sequence (for tests of page reuse); returns the count in *n */
int ti_seq_pages(ti_seq_model_t m, int32_t seq, int32_t* pages, int32_t cap, int32_t* n);

/* One step: entry e brings counts[e] tokens of sequence seqs[e] (tokens are concatenated in `tokens`).  want_rows are row
 * indices into the concatenated tokens whose logits are copied to logits_host [n_want][vocab] (may be 0 / NULL). */
int ti_seq_step(ti_seq_model_t m, int32_t n_entries, const int32_t* seqs, const int32_t* counts, const int32_t* tokens, int32_t n_want,
                const int32_t* want_rows, float* logits_host);
/* The same step, then a token is sampled on the device from the logits of each entry's LAST row (temperature 0 = greedy
 * arg-max; top_k 0 = no top-k; top_p 1 = no nucleus cut); sample_index[e] is the RNG counter of that pick. */
int ti_seq_step_sample(ti_seq_model_t m, int32_t n_entries, const int32_t* seqs, const int32_t* counts, const int32_t* tokens,
                       float temperature, int32_t top_k, float top_p, uint64_t seed, const int32_t* sample_index, int32_t* out_tokens,
                       float* out_logprobs);

/* Continuous-batching generation: n_req prompts (concatenated in `prompts`, lens[i] tokens each), up to max_new new tokens
 * each.  Requests are admitted while a state slot and pages are free; every step runs the decode tokens of the running
 * requests plus prompt portions up to `step_tokens` rows in total; a request ends at max_new tokens or on eos (eos < 0: never).
 * out_tokens [n_req][max_new], out_lens [n_req]. */
int ti_seq_generate(ti_seq_model_t m, int32_t n_req, const int32_t* prompts, const int32_t* lens, int32_t max_new, int32_t step_tokens,
                    float temperature, int32_t top_k, float top_p, uint64_t seed, int32_t eos, int32_t* out_tokens, int32_t* out_lens);

/* debugging / tests: when enabled, every step keeps the residual stream after each layer run; read gives
 * [layer runs][rows of the last step][width] */
int ti_seq_debug_layers(ti_seq_model_t m, int32_t enable);
int ti_seq_debug_layers_read(ti_seq_model_t m, float* out, size_t cap_floats, int32_t* runs, int32_t* rows);
/* CUDA-event time of the last step (device work only), ms */
int ti_seq_last_step_ms(ti_seq_model_t m, float* ms);
/* writes a buffer larger than L2 (benchmarks: cold caches between timed steps) */
int ti_seq_flush_l2(void);
/* bytes of weights one step streams (every matrix once) and bytes of cache + state per cached token / per sequence */
int ti_seq_model_bytes(ti_seq_model_t m, double* weight_bytes, double* kv_bytes_per_token, double* state_bytes_per_seq);

#ifdef __cplusplus
}
#endif
#endif
