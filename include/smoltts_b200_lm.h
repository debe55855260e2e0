/*
 * smoltts_b200 -- C ABI of the hybrid language-model engine (libsmoltts_b200_lm.so): decoder-only models whose layers
 * mix tokens either by softmax attention over a paged key/value pool (keys and values themselves, or one compressed
 * latent per position from which every head's keys and values follow) or by a recurrent matrix state kept in
 * per-sequence slots; feed-forwards are dense or a routed mixture of small experts.  Same conventions as smoltts_b200.h: plain C types, every pointer is a DEVICE pointer owned by the caller unless
 * said otherwise, every compute call is asynchronous on the given cudaStream_t (passed as void*), no allocation after
 * create, 0 / negative SMOL_ERR_* return codes with smol_lm_last_error().
 *
 * One step runs a ragged batch: any number of sequences, each bringing its next tokens (a portion of a prompt or one
 * decoded token), against the pages and the state slot the caller's scheduler gave it.
 *
 * Element type: `dtype` 0 = bfloat16 matrices, GEMM inputs and key/value pool (fp32 accumulation), 1 = float32
 * everywhere (plain FMA arithmetic, no reduced-precision matrix mode).  In both, the residual stream, every norm, the
 * attention scores and weights, and everything inside the recurrence are fp32.
 */
#ifndef SMOLTTS_B200_LM_H
#define SMOLTTS_B200_LM_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define SMOL_LM_ABI_VERSION 4

enum { SMOL_LM_BF16 = 0, SMOL_LM_F32 = 1 };
/* token mixers */
enum {
    SMOL_LM_MIX_SINK_ATTENTION = 0,    /* grouped-query attention, q/k norms, distance penalty, softmax sink, per-channel gate */
    SMOL_LM_MIX_GENERAL_DELTA = 1,     /* generalized delta rule, state [dim, dim] per head */
    SMOL_LM_MIX_LATENT_ATTENTION = 2,  /* attention through a cached latent: queries and keys/values are low-rank, part of each
                                          head's query/key is rotated by position, one gate per head */
    SMOL_LM_MIX_GATED_LINEAR = 3,      /* linear attention with a decay per key channel, state [dim, vdim] per head */
    SMOL_LM_MIX_STATE_SPACE = 4,       /* state-space recurrence with one decay per head and step: a short causal convolution in
                                          front, state [n_state, vdim] per head plus the convolution's last inputs in the slot */
    SMOL_LM_MIX_SIGMOID_ATTENTION = 5, /* grouped-query attention without a softmax: the weight of a visible key is sigmoid(score +
                                          head bias), the heads' weight maps are mixed by a [heads, heads] matrix; rotated and
                                          norm-divided queries and keys, the values being the key projection; one gate per head */
    SMOL_LM_MIX_LIGHTNING = 6,         /* linear attention with one constant decay per head over silu'd q, k, v; state [dim, vdim]
                                          per head; RMS norm over all heads together and a sigmoid gate per channel */
    SMOL_LM_MIX_HGRN2 = 7              /* linear attention whose forget gate f (bounded below per channel) also writes: key = 1 - f;
                                          state [dim, vdim] per head; RMS norm per head */
};
/* feed-forward kinds */
enum {
    SMOL_LM_MLP_NONE = 0,
    SMOL_LM_MLP_POLYNORM = 1,          /* up, PolyNorm, down */
    SMOL_LM_MLP_GATED = 2,             /* down(act(gate) * up) */
    SMOL_LM_MLP_EXPERTS = 3            /* routed mixture of gated experts, some router outputs standing for the input itself */
};
/* activations of the gated feed-forwards */
enum {
    SMOL_LM_ACT_GELU_TANH = 0,
    SMOL_LM_ACT_SILU = 1,
    SMOL_LM_ACT_CLAMPED = 2,           /* g = min(gate, limit), u = clamp(up, -limit, limit): g * sigmoid(act_alpha * g) * (u + 1) */
    SMOL_LM_ACT_RELU_SQUARED = 3       /* max(z, 0)^2 */
};
/* how a router turns its logits into scores */
enum { SMOL_LM_ROUTE_SOFTMAX = 0, SMOL_LM_ROUTE_SIGMOID = 1 };
/* how a layer wraps its sublayers */
enum {
    SMOL_LM_BLOCK_SANDWICH = 0,        /* x += ls * norm_b(sublayer(norm_a(x))): norms with one-plus weight vectors, layer scales */
    SMOL_LM_BLOCK_POSTNORM = 1,        /* x = g * rms_divide(alpha * x + sublayer(x)): one gain per norm; after each layer the
                                          stream becomes a weighted sum of the embedding output and every layer's result */
    SMOL_LM_BLOCK_PRENORM = 2          /* x += sublayer(norm(x)) with the norm SmolLmConfig.norm_kind names; a run flagged
                                          SMOL_LM_RUN_ADD_EMBED starts from x + the embedding output */
};
/* the norm of the pre-norm block */
enum {
    SMOL_LM_NORM_RMS = 0,              /* x / rms(x) * weight */
    SMOL_LM_NORM_DYT = 1               /* tanh(alpha * x) * weight + shift: no mean, no variance */
};
/* per-run flags (SmolLmConfig.run_flags) */
enum { SMOL_LM_RUN_ADD_EMBED = 1 };    /* the embedding output is added to the stream before this run */

/* One layer: sizes, constants and weights.  Matrices (`const void*`) have the engine's element type and are [out, in]
 * row-major; vectors (`const float*`) are always fp32. */
typedef struct SmolLmLayer {
    int32_t mixer;            /* SMOL_LM_MIX_* */
    int32_t heads, kv_heads;  /* query heads; key/value heads (recurrent mixer: = heads) */
    int32_t dim, vdim;        /* per-head key size and value size (recurrent mixer: vdim = dim) */
    int32_t rank;             /* recurrent mixer: inner size of the low-rank decay projection */
    int32_t mlp, ff;          /* SMOL_LM_MLP_*, feed-forward size */
    float score_scale;        /* attention: multiplies q.k */
    float decay_coef;         /* recurrent: decay = exp(-decay_coef * sigmoid(.)) */
    float unit_eps;           /* recurrent: unit key = k / sqrt(sum k^2 + unit_eps) */
    /* fused input projection [n_in, width]; attention rows: q | k | v | gate; recurrent rows: r | k | v | gate | rate | decay-inner */
    const void* w_in;
    const void* w_out;        /* [width, heads * vdim] */
    const void* w_up;         /* [ff, width] */
    const void* w_down;       /* [width, ff] */
    const float *norm1, *norm1b, *norm2, *norm2b;   /* one-plus RMS-norm weights [width] (pre / post of each sublayer) */
    const float *ls1, *ls2;                         /* layer scales [width] */
    const float *q_norm, *k_norm;                   /* attention: plain RMS-norm weights [dim] */
    const float *dist_r1, *dist_r2, *sink;          /* attention: distance penalty r1 ln(1 + r2 (i - j)) and sink logit, [heads] */
    const float *rate_bias;                         /* recurrent: [heads * dim] */
    const float *decay_w2, *decay_bias;             /* recurrent: second decay matrix TRANSPOSED, [rank, heads * dim] fp32; [heads * dim] */
    const float *out_norm;                          /* recurrent: plain weight after the per-head RMS division [heads * dim] */
    const float *act;                               /* PolyNorm coefficients a, b, c, e */
    /* --- latent attention, gated linear recurrence, gated and routed feed-forwards --- */
    int32_t rot_dim;          /* latent attention: rotated query/key coordinates per head (after the `dim` unrotated ones) */
    int32_t rot_dims;         /* of these, the leading coordinates the rotation acts on (even, <= rot_dim; the rest pass unchanged) */
    int32_t q_rank, kv_rank;  /* latent attention: sizes of the query latent and of the cached key/value latent */
    int32_t mlp_act;          /* SMOL_LM_ACT_* of a gated feed-forward or of the experts */
    int32_t n_experts;        /* routed: experts with weights */
    int32_t n_identity;       /* routed: further router outputs whose "expert" returns its input */
    int32_t top_k;            /* routed: router outputs used per token */
    int32_t n_groups, keep_groups;  /* routed: outputs form n_groups equal groups of neighbours, chosen from the best keep_groups */
    float rot_base;           /* rotation angle of pair i at position p: p * rot_base^(-2i / rot_dims) */
    float decay_tau;          /* gated linear: decay = sigmoid(z)^(1 / decay_tau) */
    float router_scale;       /* routed: multiplies the normalised weights */
    /* latent attention: w_in rows are query-latent [q_rank] | key/value latent [kv_rank] | shared rotated key [rot_dim] | gate [heads];
     * gated linear: w_in rows are q | k [heads*dim each] | v | gate [heads*vdim each] | decay-inner [rank], and score_scale multiplies q;
     * decay_w2 / decay_bias are used as in the delta rule (second decay matrix transposed, fp32) */
    const void* w_q_up;       /* latent attention: [heads * (dim + rot_dim), q_rank] */
    const void* w_k_up_t;     /* latent attention: per head the key expansion TRANSPOSED, [heads][kv_rank][dim] */
    const void* w_v_up;       /* latent attention: [heads * vdim, kv_rank] */
    const float *q_lat_norm, *kv_lat_norm;   /* latent attention: plain RMS-norm weights [q_rank], [kv_rank] */
    const void* w_experts_in; /* routed: [n_experts][2 * ff][width], gate rows then up rows; gated: w_up holds [2 * ff][width] likewise */
    const void* w_experts_out;/* routed: [n_experts][width][ff] */
    const float* w_router;    /* routed: [n_experts + n_identity][width] fp32 */
    const float* route_bias;  /* routed: added to the scores for the choice only [n_experts + n_identity] */
    const float* depth_mix;   /* post-norm block: weights of the embedding output and of every layer result so far [run + 2] */
    /* --- options of the softmax attention (SMOL_LM_MIX_SINK_ATTENTION) --- */
    int32_t window;           /* a query at position i sees the keys 0 <= i - j < window (0: every earlier key) */
    int32_t norm_whole;       /* 1: q_norm [heads * dim] and k_norm [kv_heads * dim] act over the whole projection (one root
                                 mean square for all heads) instead of per head */
    int32_t no_gate;          /* 1: the input projection holds no gate rows and the result is not gated */
    float softcap;            /* score <- softcap * tanh(score / softcap) after the scale (0: none) */
    const float* dist_slope;  /* linear distance penalty slope * (i - j) taken off the score, [heads] (NULL: none) */
    /* --- every mixer --- */
    const float* in_bias;     /* bias of the fused input projection [rows of w_in] (NULL: none) */
    const float* out_bias;    /* added to the output projection's result [width] (NULL: none) */
    float mix_scale;          /* softmax attention and state-space recurrence: multiplies the mixer's result before the
                                 output projection (used as it is: set it to 1 for a plain mixer) */
    /* A second mixer that runs beside this one on the same input (HOST pointer, copied by create; NULL: none).  Only its
     * mixer fields are read.  w_in then holds the rows of this mixer followed by the side mixer's, in_bias likewise, and
     * w_out is [width, this mixer's columns + the side mixer's columns]: the two results, each times its mix_scale, are
     * summed by the one output projection.  Softmax attention and the state-space recurrence can be paired. */
    const struct SmolLmLayer* side;
    /* --- state-space recurrence: w_in rows are gate z [heads*vdim] | x [heads*vdim] | B [bc_groups*n_state] | C [likewise] | dt [heads];
     *     x, B and C pass a causal convolution per channel and silu; dt = softplus(dt + dt_bias); per head (sharing B and C
     *     with the heads of its group)  S <- exp(-exp(a_log) dt) S + dt B x^T,  y = S^T C + skip * x;  then y * silu(z), an RMS
     *     division in norm_parts equal parts of the heads*vdim channels, times out_norm [heads*vdim] --- */
    int32_t n_state, bc_groups, conv_taps, norm_parts;
    const float* conv_w;      /* [heads*vdim + 2*bc_groups*n_state][conv_taps], the last tap multiplies the current token */
    const float* conv_b;      /* [heads*vdim + 2*bc_groups*n_state] */
    const float *dt_bias, *a_log, *skip;   /* [heads] each */
    /* --- feed-forward options --- */
    float act_limit, act_alpha;   /* SMOL_LM_ACT_CLAMPED */
    int32_t router_score;     /* SMOL_LM_ROUTE_* (route_bias may be NULL) */
    int32_t router_plain;     /* 1: a chosen output's weight is its score itself, not the score over the chosen scores' sum */
    int32_t route_input;      /* 1: the weight multiplies the expert's input rather than its output */
    /* --- pre-norm block: the Dynamic-Tanh norms use norm1 / norm2 as weights, with these shifts [width] and alphas (one number each) --- */
    const float *norm1_shift, *norm1_alpha, *norm2_shift, *norm2_alpha;
    /* --- sigmoid attention (w_in rows: q [heads*dim] | k [kv_heads*dim] | gate [heads]; in_bias as usual; vdim = dim).
     *     Per head: q and k + bias, rotated on their leading rot_dims coordinates (pair (2i, 2i+1) by pos * f_i, f_i = rot_base^(-2i/rot_dims)
     *     stretched as below), then divided by their root mean square; the cached value is k + bias before both.
     *     weight_g(i, j) = sigmoid(q_i.k_j * score_scale + head_bias[g]) for j <= i with floor(j / chunk) == floor(i / chunk) (chunk 0:
     *     every j <= i); head h applies sum_g talk[h][g] * weight_g to the values of its key/value head; times sigmoid(gate_h). --- */
    int32_t chunk;
    const float* head_bias;   /* [heads] */
    const float* talk;        /* [heads][heads] fp32 */
    /* frequency stretching of every rotating mixer (rot_stretch 0: none): wavelengths 2 pi / f above rot_original / rot_low use f / rot_stretch, those below
     * rot_original / rot_high keep f, between them s = (rot_original / wavelength - rot_low) / (rot_high - rot_low) blends
     * (1 - s) f / rot_stretch + s f */
    float rot_stretch, rot_low, rot_high, rot_original;
    /* --- lightning attention (w_in rows: q | k [heads*dim each] | v | gate [heads*vdim each]); out_norm [heads*vdim] --- */
    const float* head_decay;  /* [heads] */
    /* --- HGRN2 (w_in rows: q | forget [heads*dim each] | v [heads*vdim]); rate_bias [heads*dim] joins the forget rows,
     *     f = lower + (1 - lower) sigmoid(.); out_norm [vdim] shared by the heads --- */
    const float* forget_lower;   /* [heads*dim] */
    /* --- mixers side by side, each with its own output projection: when proj_norm is set on the layer's own mixer, it and the
     *     side mixer each multiply their own w_out [width, own columns]; each result is divided by its root mean square over the
     *     width and multiplied by its proj_norm [width] and its mix_scale; the two are added.  (Pre-norm block.) --- */
    const float* proj_norm;
    /* --- feed-forward options --- */
    int32_t ff_plain;         /* 1: the experts and the shared expert are down(act(up)) with no gate rows: w_experts_in is
                                 [n_experts][ff][width], w_shared_in [shared_ff][width] */
    int32_t group_rank_top;   /* routed: a group is ranked by the sum of its group_rank_top best choice scores (0 or 1: its best) */
    int32_t shared_ff;        /* routed: size of an expert every token uses, added with weight 1 (0: none) */
    const void* w_shared_in;  /* [2 * shared_ff (gate rows, up rows) or shared_ff (ff_plain)][width] */
    const void* w_shared_out; /* [width][shared_ff] */
} SmolLmLayer;

typedef struct SmolLmConfig {
    int32_t dtype;            /* SMOL_LM_BF16 / SMOL_LM_F32 */
    int32_t vocab, width;
    int32_t n_layers;         /* entries of the layer array */
    int32_t n_runs;           /* layer runs per token: a looped layer counts once per pass; each run owns its cache or state */
    int32_t page_size;        /* positions per key/value page */
    int32_t max_step_tokens;  /* rows of the workspace: most tokens one step may bring */
    int32_t max_step_seqs;    /* most sequences in one step */
    int32_t max_want;         /* most logits rows asked for in one step */
    int32_t max_context;      /* most positions one sequence may hold (sizes the scratch of the few-token attention path) */
    int32_t use_graph;        /* 1: steps of few tokens (decoding) are captured once per shape into a CUDA graph and replayed */
    float embed_scale, norm_eps;
    int32_t block;            /* SMOL_LM_BLOCK_* */
    float residual_alpha;     /* post-norm block: multiplies the stream before the sublayer's output is added */
    float logit_scale;        /* multiplies the logits */
    int32_t norm_plain;       /* sandwich block: 1 = the norms' weight vectors are used as they are, 0 = one is added to them */
    int32_t norm_kind;        /* pre-norm block: SMOL_LM_NORM_* */
    const int32_t* run_flags; /* HOST array [n_runs] of SMOL_LM_RUN_* bits, copied by create (NULL: none set) */
} SmolLmConfig;

typedef struct SmolLmGlobals {
    const void* embed;        /* [vocab, width] */
    const void* head;         /* [vocab, width] */
    const float* final_norm;  /* sandwich block: [width] one-plus weight; post-norm block: one gain */
    const float* embed_norm;  /* post-norm block: one gain of the norm after the embedding */
    const float *final_norm_shift, *final_norm_alpha;   /* Dynamic-Tanh final norm: shift [width], alpha (one number) */
} SmolLmGlobals;

/* A ragged batch.  All arrays live on the device. */
typedef struct SmolLmStep {
    int32_t n_tokens, n_seqs, n_want, max_pages;
    /* what the host knows about the step, used to choose kernels and grids (0 = unknown: the safe choice is made):
     * fewest / most tokens any sequence brings, and the largest position in the step */
    int32_t min_seq_tokens, max_seq_tokens, max_pos;
    const int32_t* tokens;       /* [n_tokens] ids, sequences one after the other */
    const int32_t* tok_seq;      /* [n_tokens] index of the token's sequence in this step */
    const int32_t* tok_pos;      /* [n_tokens] position in its sequence, counted from 0 */
    const int32_t* seq_start;    /* [n_seqs + 1] first row of each sequence */
    const int32_t* seq_pos0;     /* [n_seqs] positions the sequence already holds (0: a new sequence, state starts at zero) */
    const int32_t* seq_slot;     /* [n_seqs] state slot */
    const int32_t* block_table;  /* [n_seqs][max_pages] pages of each sequence, in order */
    const int32_t* want_rows;    /* [n_want] rows whose logits are wanted */
    float* logits;               /* [n_want][vocab] */
    float* trace;                /* NULL, or [n_runs][n_tokens][width]: the residual stream after every layer run */
} SmolLmStep;

typedef struct SmolLm SmolLm;

int smol_lm_abi_version(void);
size_t smol_lm_struct_bytes(int which);          /* sizeof of SmolLmLayer (0), SmolLmConfig (1), SmolLmGlobals (2), SmolLmStep (3): a binding checks its mirror */
const char* smol_lm_last_error(void);

/* layers / run_layer are HOST arrays, copied.  run_layer[n] = index of the layer that run n executes. */
int smol_lm_create(const SmolLmConfig* cfg, const SmolLmLayer* layers, const int32_t* run_layer, SmolLm** out);
void smol_lm_destroy(SmolLm* m);

size_t smol_lm_page_bytes(const SmolLm* m);       /* one page: page_size positions of every attention run's keys and values (or latents) */
size_t smol_lm_slot_bytes(const SmolLm* m);       /* one slot: the fp32 matrix states (and convolution inputs) of every recurrent run */
size_t smol_lm_workspace_bytes(const SmolLm* m);

int smol_lm_bind(SmolLm* m, const SmolLmGlobals* g, void* d_workspace, size_t workspace_bytes, void* d_pages, int32_t n_pages,
                 void* d_slots, int32_t n_slots);

int smol_lm_step(SmolLm* m, const SmolLmStep* s, void* stream);

/* Sampling of `rows` logits rows with the library's integer-weight sampler (temperature / top-k / top-p / min-p, Philox
 * counters seed, d_seq_id[row], d_step[row]); temp 0 = arg-max.  n <= 32768. */
int smol_lm_sample(SmolLm* m, const float* d_logits, int32_t rows, int32_t n, float temp, int32_t top_k, float top_p, float min_p,
                   uint64_t seed, const int32_t* d_seq_id, const int32_t* d_step, int32_t* d_out, void* stream);

/* Stand-alone operations of the engine, for tests and benchmarks: y fp32 [M, N] = a [M, K] . w [N, K]^T in the engine's element type. */
int smol_lm_linear(SmolLm* m, const void* d_a, const void* d_w, float* d_y, int32_t M, int32_t N, int32_t K, void* stream);

int64_t smol_lm_launch_count(const SmolLm* m);
int32_t* smol_lm_error_word(SmolLm* m);           /* device word, nonzero after a step that addressed outside its pools */

#ifdef __cplusplus
}
#endif
#endif
