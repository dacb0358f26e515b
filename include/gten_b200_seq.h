/* gten_b200_seq.h -- C-ABI of libgten_b200_seq.so: layer-list sequence models on one B200 (sm_100a).
 *
 * The hot path of include/gten_b200.h is one fixed graph (TinyLlama) with the reference's quantised arithmetic.  This
 * library runs models that are DESCRIBED: a list of layers, each either a parallel block (one norm, a token mixer made of
 * weighted branches, an optional gated feed-forward, both fed through a short causal convolution of the normalised
 * stream) or a pair of sequential sublayers that read the stream itself and are normalised on their way back into it
 * (mixer, then a dense or routed feed-forward); an optional weight-shared loop over a range of layers, an optional hashed
 * bigram embedding, an optional embedding scale.  Weights are bfloat16; the compute mode is bfloat16 operands with fp32
 * accumulation (tensor cores) or true fp32.
 *
 * It shares the context, the stream, the allocator and the error convention with gten_b200.h (the gtb_* calls of that
 * header are exported by this library as well): 0 on success, a message in gtb_last_error() otherwise.
 *
 * State lives in SLOTS, like the batched decode of gtb_engine_batch_*: a slot owns one sequence's position, previous
 * token, per-layer-run K/V cache, recurrent state and convolution history.  A STEP feeds any number of segments
 * (slot, next tokens) in one pass over the weights; the rows of all segments share every matrix product.
 */
#ifndef GTEN_B200_SEQ_H
#define GTEN_B200_SEQ_H
#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum { GTB_SEQ_BF16 = 0, GTB_SEQ_F32 = 1 };                       /* compute mode */
enum { GTB_MIX_SIGMOID_ATTN = 1, GTB_MIX_RETENTION = 2, GTB_MIX_MINGRU = 3, GTB_MIX_SOFTMAX_ATTN = 4, GTB_MIX_LATENT_ATTN = 5 };   /* branch kinds of a token mixer */
enum { GTB_BLOCK_PARALLEL = 0, GTB_BLOCK_POSTNORM = 1, GTB_BLOCK_PRENORM = 2, GTB_BLOCK_SANDWICH = 3 };   /* layer styles */
enum { GTB_FF_GEGLU = 0, GTB_FF_POLYNORM = 1, GTB_FF_EXPERTS = 2, GTB_FF_GATED_EXPERTS = 3, GTB_FF_SWIGLU = 4, GTB_FF_GROUP_EXPERTS = 5 };   /* feed-forward kinds */
enum { GTB_NORM_RMS = 0, GTB_NORM_DYT = 1, GTB_NORM_LAYER = 2 };          /* norm of a pre-norm / sandwich layer and of the model's output */
enum { GTB_ROT_HALVES = 0, GTB_ROT_INTERLEAVED = 1 };             /* which entries a rotary pair takes: (i, i + dims/2) or (2i, 2i + 1) */

/* One branch of a token mixer.  Tensors of branch b of layer i are "l<i>.mix.<name>.{q,k,v,o,...}".
 *  GTB_MIX_SIGMOID_ATTN: causal attention over the slot's K/V cache, `heads` query heads sharing `kv_heads` key/value
 *    heads in consecutive groups; weight of key j = sigmoid(scale * q.k_j + pb[head]), no normalisation over keys;
 *    qk_norm: q and k scaled to unit RMS per head (eps of the model).  Tensors q, k, v, pb, o.
 *  GTB_MIX_RETENTION: S <- decay[head] * S + k v^T, o = S^T q per head (fp32 state per slot); rotary positions on the
 *    first rot_dims dimensions of q and k (pairs i, i + rot_dims/2, angle pos * rot_base^(-2i/rot_dims)); k multiplied
 *    by `scale` after rotation; out_norm: o scaled to unit RMS per head; gated: o *= silu(g h).  Tensors q, k, v, g, o.
 *  GTB_MIX_MINGRU: S <- (1 - z) S + z c per channel (fp32 state per slot, `dim` channels, heads = 1), z = logistic(z h + z.b),
 *    c = u + 1/2 for u >= 0 and logistic(u) below with u = x h + x.b; output o (S * silu(g h)).  Tensors z, z.b, x, x.b, g, o.
 *  GTB_MIX_SOFTMAX_ATTN: softmax attention over the slot's K/V cache with grouped heads.  qk_norm 2: q and k to unit RMS per head
 *    times the weight q.norm / k.norm [dim] (1: unit RMS only); rotary positions on the first rot_dims entries in rot_layout, with
 *    frequencies rot_base^(-2i/rot_dims) rescaled when rot_factor > 0 (wavelengths above rot_original / rot_low divided by
 *    rot_factor, those below rot_original / rot_high kept, a linear blend in rot_original / wavelength between); score =
 *    scale q.k, then softcap * tanh(score / softcap) when softcap > 0; window > 0: position i sees tokens i - window < j <= i and,
 *    when pool > 0, one mean key / mean value for every block [b pool, (b + 1) pool) that ends at or before i - window; sink: the
 *    denominator also holds exp(sink[head]); gated 2: output times logistic(g h) (1: silu) before the out projection; kv_from >= 0:
 *    no k / v tensors, keys and values are those of layer kv_from's cache (an earlier GTB_MIX_SOFTMAX_ATTN layer with the same
 *    kv_heads, dim, vdim).  Tensors q, k, v, q.norm, k.norm, sink, g, o.
 *  GTB_MIX_LATENT_ATTN: softmax attention whose keys and values are up-projections of one latent per token.  Every head has `dim`
 *    plain and `rope_dim` rotated query/key entries ([plain | rotated] per head in q) and `vdim` value entries.  dkv h has kv_rank +
 *    rope_dim rows: the first kv_rank, scaled to unit RMS (eps of the model) times dkv.norm, are the latent c; the last rope_dim,
 *    rotated, are one key part shared by all heads.  Plain keys uk c and values uv c per head; score = scale (q_plain . k_plain +
 *    q_rot . k_rot).  q_rank > 0: q = uq (unit-RMS(dq h) * dq.norm) instead of q h.  Rotation on the first rot_dims (<= rope_dim)
 *    entries of the rotated part in rot_layout.  window, sink as for GTB_MIX_SOFTMAX_ATTN (no pooled blocks); gated 3: head a's output
 *    times logistic(g h)_a, g with one row per head.  The slot caches only c and the rotated key part ([kv_rank + rope_dim] per token).
 *    Tensors q | dq, dq.norm, uq; dkv, dkv.norm, uk, uv, sink, g, o.
 *  In sandwich layers (GTB_BLOCK_SANDWICH) GTB_MIX_SOFTMAX_ATTN and GTB_MIX_RETENTION take further parameters:
 *    softmax attention -- qk_norm 3: ONE RMS norm over the whole q projection (and one over the whole k projection) with weights q.norm
 *    [heads * maps * dim], k.norm [kv_heads * maps * dim]; rot_divide > 0: every rotary frequency is divided by it; chunk > 0: position i
 *    sees j <= i only when floor(i / chunk) = floor(j / chunk); gated 3: one logistic gate per head (g [heads][width]); bias: q, k, v
 *    projections add the vectors q.b, k.b, v.b; out_scale weighs the branch.  maps 2 (differential attention): every head has two query
 *    parts and every K/V head two key parts of `dim` entries ([part 1 | part 2] per head), each pair a softmax attention of its own over
 *    the same values; with lambda = exp(lq1 . lk1) - exp(lq2 . lk2) + diff (tensors lq1, lk1, lq2, lk2 [dim]) the head's output is
 *    (a1 - lambda a2) scaled to unit RMS over its vdim entries (eps of the model) times (1 - diff), then gated.  The cache of a maps-2 layer
 *    holds both key parts; kv_from names a layer of the same style with the same kv_heads, maps, dim, vdim.
 *    retention -- act 1: q, k, v <- silu(q), silu(k), silu(v) before the recurrence; out_norm 2: the concatenated heads are scaled to
 *    unit RMS TOGETHER and multiplied by the weight `norm` [heads * vdim]; gated 2: times logistic(g h). */
typedef struct {
    int kind;
    char name[16];
    int heads, kv_heads, dim, vdim;
    float scale;
    int qk_norm;
    int rot_dims;
    float rot_base;
    int out_norm, gated;
    float out_scale;                 /* weight of this branch in the mixer's sum */
    const float* decay;              /* [heads], host; copied */
    int rot_layout;                  /* GTB_ROT_* */
    float rot_factor, rot_low, rot_high, rot_original;     /* rot_factor = 0: plain frequencies */
    float softcap;                   /* 0: none */
    int window, pool;                /* 0: every earlier token / no pooled blocks */
    int sink;                        /* 1: learned per-head sink in the softmax denominator */
    int kv_from;                     /* -1: own keys and values */
    int rope_dim, kv_rank, q_rank;   /* GTB_MIX_LATENT_ATTN */
    int chunk;                       /* > 0: keys of the query's own chunk of positions only */
    int maps;                        /* 0 / 1: plain softmax attention; 2: differential attention */
    float diff;                      /* maps 2: the constant in lambda and in the output factor (1 - diff) */
    int bias;                        /* 1: q, k, v projections have bias vectors */
    int act;                         /* retention: 1 = silu on q, k, v */
    float rot_divide;                /* > 0: rotary frequencies are divided by it */
} gtb_seq_branch;

/* Tensors of layer i beyond its branches'.  Parallel blocks: "l<i>.norm1" (one gain), "l<i>.mlp.{gate,up,down}", "l<i>.canon{1,2}".
 * Post-norm layers: "l<i>.norm1", "l<i>.norm2" [width] (norm2 only with a feed-forward); GTB_FF_POLYNORM: "l<i>.mlp.up" [ff][width],
 * "l<i>.mlp.down" [width][ff], "l<i>.mlp.act" [4]; GTB_FF_EXPERTS: "l<i>.mlp.router" [experts + identity][width], "l<i>.mlp.correction"
 * [experts + identity], "l<i>.mlp.e<j>.up" [ff][width], "l<i>.mlp.e<j>.down" [width][ff].  A branch with an empty name has its tensors
 * directly under "l<i>.mix.".
 * Pre-norm layers: "l<i>.norm<q>" [width] and, for GTB_NORM_DYT, "l<i>.norm<q>.alpha" [] and "l<i>.norm<q>.b" [width]; with streams > 0
 * "l<i>.hc<q>.in" [streams], "l<i>.hc<q>.out" [streams], "l<i>.hc<q>.mix" [streams][streams] (q = 1: mixer, 2: feed-forward);
 * GTB_FF_GEGLU: "l<i>.mlp.{gate,up,down}"; GTB_FF_GATED_EXPERTS: "l<i>.mlp.router" [experts][width], "l<i>.mlp.e<j>.{gate,up,down}" and,
 * when shared_ff > 0, "l<i>.mlp.shared.{gate,up,down}" with inner width shared_ff and "l<i>.mlp.shared.sg" [1][width]. */
typedef struct {
    int n_branches;                  /* 1 or 2 */
    gtb_seq_branch branch[2];
    int ff;                          /* 0: no feed-forward; else its inner width (of one expert for GTB_FF_EXPERTS) */
    int style;                       /* GTB_BLOCK_PARALLEL: x += mixer(h) + ff(h), h = gain-norm(x) (+ convolutions);
                                      * GTB_BLOCK_POSTNORM: x += norm1(mixer(x)); x += norm2(ff(x)), norms with weight vectors (1 + w),
                                      * one branch, out_scale unused;
                                      * GTB_BLOCK_PRENORM: x += mixer(norm1(x)); x += ff(norm2(x)), norm of kind norm_kind; with config.streams > 0
                                      * the stream is kept in `streams` copies: sublayer q reads u = sum_s hc<q>.in[s] x_s and all copies are
                                      * rewritten at once from the old ones, x_t <- sum_s hc<q>.mix[s][t] x_s + hc<q>.out[t] y.  One branch
                                      * (GTB_MIX_LATENT_ATTN);
                                      * GTB_BLOCK_SANDWICH: x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))), four norms of kind norm_kind
                                      * (GTB_NORM_LAYER or GTB_NORM_RMS with a plain weight); one or two branches (GTB_MIX_SOFTMAX_ATTN,
                                      * GTB_MIX_RETENTION), each weighted by its out_scale */
    int ff_kind;                     /* GTB_FF_GEGLU: down(gelu_tanh(gate h) * (up h)); GTB_FF_POLYNORM: down(a N(z) + b N(z^2) + c N(z^3) + e),
                                      * z = up h, N = unit RMS over the ff values, (a, b, c, e) = tensor mlp.act; GTB_FF_EXPERTS: router outputs
                                      * 0 .. experts-1 are experts e<i>.down(relu(e<i>.up h)^2), the `identity` outputs after them return h;
                                      * s = softmax(router h), the `top` largest s + correction are chosen and weighted with their s;
                                      * GTB_FF_GATED_EXPERTS: experts e<i>.down(silu(e<i>.gate h) * (e<i>.up h)); s = logistic(router h) in fp32, the
                                      * `top` largest s are chosen (ties to the lower index) and weighted with s / (sum of the chosen s + 1e-20);
                                      * shared_ff > 0: an expert of that inner width runs for every row, times logistic(shared.sg h);
                                      * GTB_FF_SWIGLU: down(silu(gate h) * (up h));
                                      * GTB_FF_GROUP_EXPERTS: experts e<i>.down(relu(e<i>.up h)^2); s = logistic(router h) in fp32; the experts form
                                      * route_groups equal groups of neighbours, a group ranks by the sum of its two largest s, only experts of the
                                      * route_keep best groups can be chosen; the `top` largest s among them are chosen (ties to the lower index) and
                                      * weighted with route_scale * s (not renormalised); shared_ff > 0: one more expert of the same form and that
                                      * inner width runs for every row with weight 1 */
    int experts, top, identity;
    int norm_kind;                   /* GTB_BLOCK_PRENORM: GTB_NORM_RMS (x / rms(x) * w) or GTB_NORM_DYT (tanh(alpha x) * w + b, no statistics);
                                      * GTB_BLOCK_SANDWICH: GTB_NORM_RMS or GTB_NORM_LAYER ((x - mean) / sqrt(variance + eps) * w + b) */
    int shared_ff;
    int route_groups, route_keep;    /* GTB_FF_GROUP_EXPERTS (0 groups counts as 1, 0 kept as all) */
    float route_scale;
} gtb_seq_layer;

typedef struct {
    int vocab, width, n_layers;
    float eps;
    int taps;                        /* causal per-channel convolution in front of each sublayer; 0: none */
    int bigram_buckets, bigram_mul_prev, bigram_mul_cur;   /* buckets = 0: no bigram table */
    int loop_start, loop_stop, loop_times;                 /* times = 0: no loop */
    int mode;                        /* GTB_SEQ_BF16 / GTB_SEQ_F32 */
    int n_slots, max_ctx;            /* sequences held at once; positions per slot */
    int max_rows;                    /* rows per pass over the weights (longer steps are cut into passes); 0: default */
    float embed_scale;               /* embedding rows are multiplied by this (0 counts as 1) */
    int final_norm;                  /* 0: one gain; 1: weight vector stored around zero (1 + w); 2: Dynamic Tanh, tensors final.norm, final.norm.alpha, final.norm.b;
                                      * 3: layer norm, tensors final.norm, final.norm.b */
    int streams;                     /* pre-norm layers: copies of the residual stream under hyper-connections (all equal to the embedding output at
                                      * the start, summed at the end); 0: one stream, plain residual sum */
    float logit_softcap;             /* > 0: logits <- cap * tanh(logits / cap) */
} gtb_seq_config;

typedef struct gtb_seq_model* gtb_seq_t;

int gtb_seq_create(gtb_seq_t* out, const gtb_seq_config* cfg, const gtb_seq_layer* layers);
int gtb_seq_destroy(gtb_seq_t m);
/* one tensor of the checkpoint by its name; bf16 (dtype 0) or int32/fp32 payloads are not needed by this family.
 * shape is checked against the description */
int gtb_seq_set_tensor(gtb_seq_t m, const char* name, const void* h_bf16, const int64_t* shape, int ndim);
int gtb_seq_finalize(gtb_seq_t m);                                 /* fails and names the first tensor that is missing */
int gtb_seq_n_runs(gtb_seq_t m, int* n);                           /* layer runs per token (a looped layer counts each pass) */

/* slots */
int gtb_seq_slot_reset(gtb_seq_t m, int slot);                     /* empty sequence: position 0, zero state */
int gtb_seq_slot_position(gtb_seq_t m, int slot, int* pos);

/* The step function.  Segment s feeds seg_len[s] tokens (consecutive in h_tokens) to slot seg_slot[s], continuing from the
 * slot's state; a slot appears at most once.  want_rows: indices into the step's rows (0 .. sum(seg_len)-1, ascending) whose
 * logits are written to h_logits [n_want][vocab] (may be 0).  Rows beyond max_rows are run as further passes. */
int gtb_seq_step(gtb_seq_t m, int n_seg, const int32_t* seg_slot, const int32_t* seg_len, const int32_t* h_tokens,
                 int n_want, const int32_t* want_rows, float* h_logits);
/* same, and the last row of every segment is sampled greedily on the device (first maximum): h_next [n_seg] */
int gtb_seq_step_greedy(gtb_seq_t m, int n_seg, const int32_t* seg_slot, const int32_t* seg_len, const int32_t* h_tokens,
                        int32_t* h_next);
/* n greedy steps of the given slots without a host round trip: each slot feeds its last sampled token (set by
 * gtb_seq_step_greedy or a previous call); tokens land in h_out [n_slots_in][n_steps].  A slot that samples eos_id (>= 0)
 * keeps repeating it and its state stops advancing. */
int gtb_seq_decode(gtb_seq_t m, int n, const int32_t* slots, int n_steps, int eos_id, int32_t* h_out);
/* the k (<= 64) largest logits of segment s's last row of the last step, largest first, ties to the lower id */
int gtb_seq_topk(gtb_seq_t m, int seg, int k, float* h_values, int32_t* h_ids);
/* logits of segment s's last row of the last gtb_seq_step_greedy / gtb_seq_decode call */
int gtb_seq_last_logits(gtb_seq_t m, int seg, float* h_logits);

/* options: "capture" (1: the residual stream after every layer run of the last pass is kept for gtb_seq_read_capture),
 * "tensor" (1, default: bf16 matrix products of >= "tensor_min_rows" rows on tcgen05; 0: SIMT kernels only),
 * "tensor_min_rows" (default 64), "graph" (1, default: gtb_seq_decode replays a CUDA graph per step),
 * "fused_attn" (1, default: tiled kernels of the mixers on prompt portions -- tensor-core attention in bf16 mode, chunked
 * retention and minGRU, expanded keys and values for latent attention; decode rows of latent attention on tensor cores in bf16 mode;
 * 0: the row-at-a-time kernels), "grouped_experts" (1, default: rows sorted by expert and multiplied as groups
 * on passes of tensor_min_rows rows or more; 0: one weight stream per row and choice), "fused_norm" (1, default: norm and input convolution in one kernel on passes of 32 rows or more; 0: two kernels) */
int gtb_seq_set_option(gtb_seq_t m, const char* name, int value);
int gtb_seq_read_capture(gtb_seq_t m, int run, int row, float* h_out);    /* [width] */
/* self-test and timing of the bf16 tensor-core product on host data: C [M][N] = A [M][K] . W [N][K]^T (+ the incoming C when accumulate);
 * operands are placed with a row stride of K + ld_extra elements; *ms = mean device time of `iters` further runs */
int gtb_seq_selftest_gemm(const void* h_A, const void* h_W, float* h_C, int M, int N, int K, int ld_extra, int accumulate, int iters, float* ms);
int gtb_seq_weight_bytes(gtb_seq_t m, size_t* nbytes);
int gtb_seq_state_bytes_per_slot(gtb_seq_t m, size_t* nbytes);

#ifdef __cplusplus
}
#endif
#endif /* GTEN_B200_SEQ_H */
