// gtb_seq.cu -- host side of libgten_b200_seq.so (include/gten_b200_seq.h): model description, weight placement, slot state,
// the step function (one pass over the weights for the rows of any number of segments), greedy decode loop, top-k.
//
// Layout decisions:
//  * per layer THREE matrix products: [all branch projections] <- operand A (h + conv_a(h)); [gate | up] <- operand B (h + conv_b(h));
//    x += [branch outputs (already weighted) | gelu(gate) * up] . [o_0 | o_1 | down]^T  -- the branch out-projections and the down
//    projection are concatenated along K, so the residual update is ONE product that accumulates into the fp32 stream.
//  * every operand / weight row is zero-padded to a multiple of 64 elements (one tensor-core k-block, 16-byte aligned rows).
//  * a looped layer has one set of weights and one set of state (cache, recurrent state, conv history) per pass: a "run".
//  * post-norm layers (GTB_BLOCK_POSTNORM) run their two sublayers one after the other: [branch projections] <- x, mixer, out
//    projection into a fresh block Y, x += norm1(Y); then the feed-forward the same way.  Experts' up matrices are stacked along N
//    ([experts * ff][width]) and their down matrices are stored one after the other ([experts][width][ff padded to 64]), which is what
//    both the per-row kernels and the grouped product read.
//  * pre-norm layers (GTB_BLOCK_PRENORM) keep the stream in `streams` copies XS [streams][max_rows][width]; one kernel per sublayer
//    boundary applies the finished sublayer's update to all copies and forms the next sublayer's normalised input.  Latent attention
//    caches [latent | rotated key part] per token ([n_slots][max_ctx][c_ld]); gated experts store [gate | up] of every expert as one
//    block of 2 ff rows ([experts][2 ff][width]), the shared expert's gate as one more row of the router matrix.
//  * sandwich layers (GTB_BLOCK_SANDWICH) run like post-norm layers with a norm on both sides of each sublayer: one kernel per sublayer
//    boundary adds norm_b(sublayer output) to the stream and writes the next sublayer's normalised input.  Their mixers are the branch
//    kernels of the other styles (softmax attention, retention) side by side, each weighted by out_scale in the out-projection operand.
//    Group-limited experts reuse the stacked layout of the post-norm experts; the shared expert is cut along its inner width into parts of
//    one expert's size that follow the routed experts in the same stacks, so every row simply has `top + parts` choices.
#include <math.h>
#include <string.h>

#include <map>
#include <string>
#include <vector>

#include "../../include/gten_b200_seq.h"
#include "gtb_internal.h"
#include "gtb_sample.cuh"
#include "gtb_seq_gemm.h"
#include "gtb_seq_kernels.cuh"
#include "gtb_seq_mixers.cuh"
#include "gtb_seq_mixers_tiled.cuh"
#include "gtb_seq_latent.cuh"
#include "gtb_seq_sandwich.cuh"

using namespace gtb;
using namespace gtb::seq;

namespace {

inline int pad64(int k) { return (k + 63) / 64 * 64; }
constexpr int SPLIT_MAX_ROWS = 64;          // passes of at most this many rows may split a row's keys over several CTAs

struct TensorDest {
    int kind = 0;              // 0: bf16 matrix block, 1: fp32 vector (converted)
    void* dst = nullptr;
    int rows = 0, cols = 0;    // expected logical shape ([rows] for vectors with cols == 0)
    int ld = 0;                // destination row stride in elements (matrix)
    bool scalar = false;       // shape []
    int group = 0, group_stride = 0;   // matrix rows placed in groups of `group` rows, `group_stride` rows apart (0: contiguous)
    int split_cols = 0;                // > 0: columns placed in blocks of split_cols, block j at dst + j * split_stride elements
    size_t split_stride = 0;
    bool loaded = false;
};

struct BranchW {
    gtb_seq_branch d{};
    std::vector<float> decay, inv_freq;
    int q_off = 0, k_off = 0, v_off = 0, g_off = 0, a_off = 0;
    int kq = 0, kk = 0, kv = 0;   // projection widths
    float* d_pb = nullptr;
    float* d_decay = nullptr;
    float* d_inv_freq = nullptr;
    float *d_qnorm = nullptr, *d_knorm = nullptr, *d_sink = nullptr;
    // latent attention
    bf16 *w_uq = nullptr, *w_uk = nullptr, *w_uv = nullptr;
    float* d_kvnorm = nullptr;
    int kv_off = 0, c_ld = 0, rank_p = 0, qrank_p = 0;
    // sandwich layers
    float* d_onorm = nullptr;                       // retention: weight of the norm over the concatenated heads
    float* d_lam[4] = {nullptr, nullptr, nullptr, nullptr};     // differential attention: lq1, lk1, lq2, lk2
};

struct LayerW {
    gtb_seq_layer d{};
    BranchW br[2];
    int n1 = 0;                // columns of the fused branch projection
    int kout = 0, kout_p = 0;  // K of the fused out projection
    int ff = 0;
    bf16 *w_mix = nullptr, *w_gu = nullptr, *w_out = nullptr, *canon_a = nullptr, *canon_b = nullptr;
    float* d_gain = nullptr;
    bool gu_inter = false;     // gate and up rows interleaved in groups of 32 (what the fused tensor-core epilogue reads)
    // post-norm style
    float *d_bias = nullptr;   // bias of the fused branch projection [n1] (minGRU), or null
    float *norm1 = nullptr, *norm2 = nullptr;
    bf16 *w_up = nullptr, *w_down = nullptr, *w_router = nullptr;
    float *d_act = nullptr, *d_corr = nullptr;
    int kfp = 0;               // inner width of the feed-forward (of one expert), padded to 64
    int n_out = 0;             // router outputs: experts + identity (gated experts: + 1 for the shared expert's gate)
    // pre-norm style
    float *nb[2] = {nullptr, nullptr}, *na[2] = {nullptr, nullptr};     // Dynamic Tanh: bias vectors and alpha of norm1 / norm2
    float* hc[2] = {nullptr, nullptr};                                  // hyper-connection weights [in | out | mix] of the two sublayers
    bf16 *w_sh_gu = nullptr, *w_sh_down = nullptr;                      // shared expert
    int sff = 0, sff_p = 0;
    bool sh_inter = false, e_inter = false;                             // [gate | up] rows interleaved in groups of 32
    // sandwich style
    float *sn_w[4] = {nullptr, nullptr, nullptr, nullptr}, *sn_b[4] = {nullptr, nullptr, nullptr, nullptr};     // norm1, norm1b, norm2, norm2b
    int n_sh = 0, e_total = 0;                                          // parts of the shared expert; routed experts + parts
};

struct Run {
    int layer = 0, pass = -1;  // pass >= 0: inside the loop
    bool enters_pass = false;  // the loop's entry projection comes before this run
    void *kc[2] = {nullptr, nullptr}, *vc[2] = {nullptr, nullptr};
    float* state[2] = {nullptr, nullptr};
    float* tail = nullptr;
    float *pk = nullptr, *pv = nullptr;     // mean key / value of every completed block of `pool` tokens [n_slots][max_blocks][kv_heads * dim|vdim]
    int max_blocks = 0;
};

}  // namespace

struct gtb_seq_model {
    gtb_seq_config cfg{};
    std::vector<LayerW> L;
    std::vector<Run> runs;
    std::map<std::string, TensorDest> tensors;
    std::vector<void*> allocs;
    bool finalized = false;
    int wp = 0;                                  // padded width
    size_t weight_bytes = 0, state_bytes = 0;
    bf16 *embed = nullptr, *bigram = nullptr, *head = nullptr, *loop_in = nullptr;
    float *loop_step = nullptr, *final_gain = nullptr, *final_b = nullptr, *final_a = nullptr;
    // pre-norm style: copies of the stream, latent attention workspace, shared expert
    int ns = 1;                                  // copies of the stream
    bool prenorm = false, sandwich = false;
    float* qk_sc = nullptr;                      // scales of the whole-projection q / k norm [max_rows][2]
    float *xs = nullptr, *hc_one = nullptr, *latQ = nullptr, *latQA = nullptr, *Y2 = nullptr, *shw = nullptr;
    void *opQ = nullptr, *opO = nullptr;
    float* latX = nullptr;                       // expanded [plain keys | values] of one segment's visible range, fp32 [max_ctx][heads * (dim + vdim)]
    bf16 *latKx = nullptr, *latVx = nullptr;     // the same as bf16 heads [n_slots][max_ctx][heads][dim + rope | vdim], shared by the layers
    int lat_kx_max = 0, lat_vx_max = 0, lat_x_max = 0;
    int lat_q_max = 0, lat_qa_max = 0, lat_qr_max = 0, lat_ol_max = 0;
    // workspace of a pass
    int max_rows = 0, n1_max = 0, ff_max = 0, kout_p_max = 0, ro_max = 0;
    float* Y = nullptr;                          // fresh output block of an accumulating tensor-core product [max_rows][width]
    float *x = nullptr, *x0 = nullptr, *h = nullptr, *P = nullptr, *G = nullptr, *O = nullptr, *logits = nullptr;
    void *opA = nullptr, *opB = nullptr, *opC = nullptr, *opL = nullptr, *opH = nullptr;
    float* attn_part = nullptr;                  // split decode attention: partial sums [splits][SPLIT_MAX_ROWS][heads * vdim]
    int attn_splits = 1;
    float* retU = nullptr;                       // chunked retention: per-chunk contributions / states [chunks][heads][dim][vdim]
    size_t retU_floats = 0;
    float* sattn_part = nullptr;                 // split softmax attention: partial (max, denominator, values) [32][SPLIT_MAX_ROWS][heads][vdim + 2]
    float* gruAB = nullptr;                      // chunked minGRU: per-chunk maps [chunks][2][width]
    size_t gruAB_floats = 0;
    float* rl = nullptr;                         // router logits [max_rows][n_out_max]
    int* sel_idx = nullptr;                      // chosen router outputs [max_rows][top_max]
    float* sel_w = nullptr;
    void* act = nullptr;                         // expert activations [max_rows * top_max][kfp_max]
    // grouped experts (bf16 mode): rows sorted by expert, groups aligned to 128 rows
    int mpad_max = 0, e_max = 0;
    bf16 *Xg = nullptr, *actg = nullptr;         // [mpad_max][wp], [mpad_max][kfp_max]
    float *Yg = nullptr, *rw = nullptr;          // [mpad_max][width], [mpad_max]
    int *pair_dst = nullptr, *tile_e = nullptr;  // [max_rows * top_max], [mpad_max / 128]
    int n_out_max = 0, top_max = 0, kfp_max = 0, g_cols = 0;
    bool grouped_experts = true;
    float* cap = nullptr;                        // [runs][max_rows][width]
    bool capture = false;
    int cap_rows = 0;
    // tables
    int* d_tab = nullptr;                        // one upload per pass: seg_slot | seg_row0 | seg_len | row_seg | tok | want
    int* h_tab = nullptr;                        // pinned
    int tab_cap = 0;
    int *d_row_pos = nullptr, *d_row_prev = nullptr, *d_hist = nullptr;
    SlotState* d_slots = nullptr;
    std::vector<int> host_pos;
    std::vector<char> host_stopped_unknown;
    int last_nseg = 0;                           // rows of `logits` that hold segment-last rows (greedy / decode)
    bool use_tensor = true;
    int tensor_min_rows = 64;
    bool use_graph = true;
    bool fused_attn = true;
    bool fused_norm = true;
    SeqGemmPlan* gp = nullptr;
    // decode graph
    cudaGraphExec_t graph = nullptr;
    std::vector<int> graph_slots;
    int graph_eos = -2;
};

namespace {

int dalloc(gtb_seq_model* m, void** p, size_t n, bool zero = true) {
    if (n == 0) n = 16;
    GTB_CUDA(cudaMalloc(p, n));
    if (zero) GTB_CUDA(cudaMemsetAsync(*p, 0, n, ctx().stream));
    m->allocs.push_back(*p);
    ctx().mem += (int64_t)n;
    return GTB_OK;
}
template <typename T> int dalloc_t(gtb_seq_model* m, T** p, size_t count) { return dalloc(m, reinterpret_cast<void**>(p), count * sizeof(T)); }

void want_matrix(gtb_seq_model* m, const std::string& name, bf16* dst, int rows, int cols, int ld) {
    TensorDest d; d.kind = 0; d.dst = dst; d.rows = rows; d.cols = cols; d.ld = ld;
    m->tensors[name] = d;
    m->weight_bytes += (size_t)rows * cols * 2;
}
void want_vector(gtb_seq_model* m, const std::string& name, float* dst, int rows, int cols, bool scalar = false) {
    TensorDest d; d.kind = 1; d.dst = dst; d.rows = rows; d.cols = cols; d.scalar = scalar;
    m->tensors[name] = d;
    m->weight_bytes += (size_t)std::max(rows, 1) * std::max(cols, 1) * 2;
}

size_t osz(const gtb_seq_model* m) { return m->cfg.mode == GTB_SEQ_F32 ? 4 : 2; }
// fp32 values of recurrent state one slot holds for a branch
size_t state_floats(const gtb_seq_branch& d) { return d.kind == GTB_MIX_MINGRU ? (size_t)d.dim : (size_t)d.heads * d.dim * d.vdim; }
constexpr int GRU_CHUNK = 32;               // rows per chunk of the chunked minGRU scan

// C = (acc ? C : 0) + bias + A . W^T on the library stream; picks the tensor-core kernel, the few-row kernel or the SIMT tile kernel
template <typename OT>
int product(gtb_seq_model* m, const void* A, int lda, const bf16* W, int ldw, float* C, int ldc, int M, int N, int Kp, const float* bias, int acc) {
    cudaStream_t st = ctx().stream;
    const OT* a = reinterpret_cast<const OT*>(A);
    if (sizeof(OT) == 2 && m->use_tensor && M >= m->tensor_min_rows && m->gp) {
        // An accumulating epilogue reads C one row per thread (the TMEM lane layout): measured 4x the whole product's time.  So the
        // tensor-core kernel always writes a fresh [M][N] block and a coalesced kernel adds it to the stream.
        float* dst = (acc && N <= m->cfg.width) ? m->Y : C;
        int rc = seq_gemm_bf16(m->gp, A, lda, W, ldw, dst, dst == C ? ldc : N, M, N, Kp, bias, dst == C ? acc : 0);
        if (rc == 0 && dst != C) {
            const size_t n4 = (size_t)M * N;
            k_add_block<<<(unsigned)((n4 + 255) / 256), 256, 0, st>>>(C, ldc, m->Y, N, M);
            GTB_LAUNCHED();
        }
        if (rc != -1) return rc;                 // -1: shape not supported by that kernel
    }
    if (M <= 8) {
        if (M <= 1) k_gemv_rows<OT, 1, 4><<<(N + 3) / 4, 256, 0, st>>>(a, lda, W, ldw, C, ldc, M, N, Kp, bias, acc);
        else if (M <= 2) k_gemv_rows<OT, 2, 4><<<(N + 3) / 4, 256, 0, st>>>(a, lda, W, ldw, C, ldc, M, N, Kp, bias, acc);
        else if (M <= 4) k_gemv_rows<OT, 4, 4><<<(N + 3) / 4, 256, 0, st>>>(a, lda, W, ldw, C, ldc, M, N, Kp, bias, acc);
        else k_gemv_rows<OT, 8, 4><<<(N + 3) / 4, 256, 0, st>>>(a, lda, W, ldw, C, ldc, M, N, Kp, bias, acc);
    } else {
        dim3 grid((N + SG_BN - 1) / SG_BN, (M + SG_BM - 1) / SG_BM);
        k_gemm_simt<OT><<<grid, 256, 0, st>>>(a, lda, W, ldw, C, ldc, M, N, Kp, bias, acc);
    }
    GTB_LAUNCHED();
    return GTB_OK;
}

AttnBranch attn_args(const gtb_seq_model* m, const BranchW& b) {
    AttnBranch a{};
    a.heads = b.d.heads; a.kv_heads = b.d.kv_heads; a.dim = b.d.dim; a.vdim = b.d.vdim;
    a.scale = b.d.scale; a.eps = m->cfg.eps; a.out_scale = b.d.out_scale; a.qk_norm = b.d.qk_norm;
    a.q_off = b.q_off; a.k_off = b.k_off; a.v_off = b.v_off; a.a_off = b.a_off; a.pb = b.d_pb; a.max_ctx = m->cfg.max_ctx;
    return a;
}
RetBranch ret_args(const gtb_seq_model* m, const BranchW& b) {
    RetBranch a{};
    a.heads = b.d.heads; a.dim = b.d.dim; a.vdim = b.d.vdim; a.scale = b.d.scale; a.eps = m->cfg.eps; a.out_scale = b.d.out_scale;
    a.rot_dims = b.d.rot_dims; a.inv_freq = b.d_inv_freq; a.decay = b.d_decay; a.out_norm = b.d.out_norm; a.gated = b.d.gated;
    a.q_off = b.q_off; a.k_off = b.k_off; a.v_off = b.v_off; a.g_off = b.g_off; a.a_off = b.a_off;
    return a;
}

// chunked retention (prompt portions): chunk length, value-slice width and shared memory of its two matrix kernels
struct RetChunk { int C, vs; size_t smem_kv, smem_out; bool ok; };
RetChunk ret_chunk(const gtb_seq_branch& d) {
    RetChunk r;
    r.C = d.dim <= 128 ? 64 : 32;
    r.vs = std::min(d.vdim, r.C);         // a state slice [dim][vs] must fit where the keys [dim][C] were
    const size_t dp = (d.dim + 3) & ~3, vsp = (r.vs + 3) & ~3;
    r.smem_kv = ((size_t)r.C * dp + (size_t)r.C * vsp) * sizeof(float);
    r.smem_out = (2 * (size_t)(r.C + 4) * d.dim + (size_t)r.C * vsp + (size_t)r.C * r.C) * sizeof(float);     // the incoming state reuses the keys' space
    r.ok = r.smem_out <= 200 * 1024;
    return r;
}

template <int DP, int VP, int HPC>
int launch_sigattn_mma(const PassTables& t, const AttnBranch& a, int S, int n_tiles, const float* P, int ldp, const bf16* kc, const bf16* vc, bf16* out, int ld_out) {
    const size_t smem = ((HPC + 2) * 64 * (size_t)(DP + 8) + 2 * 64 * (size_t)(VP + 8)) * 2;      // queries + two stages of keys and values
    static bool attr = false;
    if (!attr) { GTB_CUDA(cudaFuncSetAttribute(k_sigattn_mma<DP, VP, HPC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr = true; }
    k_sigattn_mma<DP, VP, HPC><<<dim3(n_tiles, a.heads / HPC), 128 * HPC, smem, ctx().stream>>>(t, a, S, P, ldp, kc, vc, out, ld_out);
    GTB_LAUNCHED();
    return GTB_OK;
}
int sigattn_mma(const PassTables& t, const AttnBranch& a, int S, int n_tiles, const float* P, int ldp, const bf16* kc, const bf16* vc, bf16* out, int ld_out) {
    const int dp = a.dim <= 32 ? 32 : a.dim <= 64 ? 64 : 128, vp = a.vdim <= 32 ? 32 : a.vdim <= 64 ? 64 : 128;
    // (HPC = 2 -- two query heads of a group sharing a CTA's K/V tiles -- was measured equal to one head per CTA at 32 heads x 2048 rows)
#define SA_CASE(D, V) if (dp == D && vp == V) return launch_sigattn_mma<D, V, 1>(t, a, S, n_tiles, P, ldp, kc, vc, out, ld_out)
    SA_CASE(32, 32); SA_CASE(32, 64); SA_CASE(32, 128); SA_CASE(64, 32); SA_CASE(64, 64); SA_CASE(64, 128); SA_CASE(128, 32); SA_CASE(128, 64); SA_CASE(128, 128);
#undef SA_CASE
    return -1;
}

// row-by-row retention (decode rows, short portions): value channels per CTA, CTA shape, slices, shared memory
struct RetLaunch { dim3 block; size_t smem; int vs, nvs; };
RetLaunch ret_launch(const gtb_seq_branch& d) {
    RetLaunch r;
    r.vs = std::min(d.vdim, d.dim > 512 ? 32 : 64);
    r.nvs = (d.vdim + r.vs - 1) / r.vs;
    const int bx = (r.vs + 31) / 32 * 32;
    int ny = std::max(1, std::min(std::min(512 / bx, d.dim), 16));
    r.block = dim3(bx, ny);
    r.smem = ((size_t)d.dim * r.vs + 4 * (size_t)d.dim + (size_t)ny * r.vs) * sizeof(float);
    return r;
}

template <int DP, int VP>
int launch_sattn_mma(const PassTables& t, const SoftAttn& a, int S, int n_tiles, const float* P, int ldp, const bf16* kc, const bf16* vc, const float* pk, const float* pv,
                     bf16* out, int ld_out, float* out_f, int ld_f) {
    const size_t smem = (3 * 64 * (size_t)(DP + 8) + 2 * 64 * (size_t)(VP + 8)) * 2;      // queries + two stages of keys and values
    static bool attr = false;
    if (!attr) { GTB_CUDA(cudaFuncSetAttribute(k_sattn_mma<DP, VP>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); attr = true; }
    k_sattn_mma<DP, VP><<<dim3(n_tiles, a.heads * sa_maps(a)), 128, smem, ctx().stream>>>(t, a, S, P, ldp, kc, vc, pk, pv, out, ld_out, out_f, ld_f);
    GTB_LAUNCHED();
    return GTB_OK;
}
// out_f != null: the units' outputs go there in fp32 ([rows][ld_f], unit-major) without gate or weight instead of `out`
int sattn_mma(const PassTables& t, const SoftAttn& a, int S, int n_tiles, const float* P, int ldp, const bf16* kc, const bf16* vc, const float* pk, const float* pv,
              bf16* out, int ld_out, float* out_f = nullptr, int ld_f = 0) {
    const int dp = a.dim <= 32 ? 32 : a.dim <= 64 ? 64 : 128, vp = a.vdim <= 32 ? 32 : a.vdim <= 64 ? 64 : 128;
#define SA_CASE(D, V) if (dp == D && vp == V) return launch_sattn_mma<D, V>(t, a, S, n_tiles, P, ldp, kc, vc, pk, pv, out, ld_out, out_f, ld_f)
    SA_CASE(32, 32); SA_CASE(32, 64); SA_CASE(32, 128); SA_CASE(64, 32); SA_CASE(64, 64); SA_CASE(64, 128); SA_CASE(128, 32); SA_CASE(128, 64); SA_CASE(128, 128);
#undef SA_CASE
    return -1;
}

GruBranch gru_args(const BranchW& b) {
    GruBranch a{};
    a.width = b.d.dim; a.z_off = b.q_off; a.x_off = b.k_off; a.g_off = b.g_off; a.a_off = b.a_off;
    return a;
}
SoftAttn soft_args(const gtb_seq_model* m, const BranchW& b, const Run& run) {
    SoftAttn a{};
    a.heads = b.d.heads; a.kv_heads = b.d.kv_heads; a.dim = b.d.dim; a.vdim = b.d.vdim;
    a.scale = b.d.scale; a.eps = m->cfg.eps; a.softcap = b.d.softcap;
    a.qk_norm = b.d.qk_norm; a.q_norm = b.d_qnorm; a.k_norm = b.d_knorm;
    a.rot_dims = b.d.rot_dims; a.rot_layout = b.d.rot_layout; a.inv_freq = b.d_inv_freq;
    a.window = b.d.window; a.pool = (b.d.window > 0) ? b.d.pool : 0; a.sink = b.d_sink; a.gate = b.d.gated;
    a.q_off = b.q_off; a.k_off = b.k_off; a.v_off = b.v_off; a.g_off = b.g_off; a.a_off = b.a_off;
    a.own_kv = b.d.kv_from < 0; a.max_ctx = m->cfg.max_ctx; a.max_blocks = run.max_blocks;
    a.maps = b.d.maps > 1 ? b.d.maps : 1; a.chunk = b.d.chunk; a.out_scale = b.d.out_scale; a.qk_sc = m->qk_sc;
    if (a.maps > 1) { a.gate = 0; a.out_scale = 1.0f; }       // the maps are combined, gated and weighted afterwards
    return a;
}

// One layer of the post-norm style on R rows: x += norm1(mixer(x)); x += norm2(ff(x)).  opA holds the stream as a product operand
// when x_in_opA (the residual update of the previous sublayer wrote it) and always does on return.
template <typename OT>
int run_postnorm_layer(gtb_seq_model* m, const PassTables& t, int R, int S, const Run& run, const LayerW& l, bool portions, const int* seg_lens, int n_qtiles, bool x_in_opA) {
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    const int W = c.width, wp = m->wp;
    OT *opA = (OT*)m->opA, *opC = (OT*)m->opC;
    if (!x_in_opA) {
        k_copy_operand<OT><<<R, 256, 0, st>>>(m->x, W, opA, (OT*)nullptr, wp);
        GTB_LAUNCHED();
    }
    int rc = product<OT>(m, opA, wp, l.w_mix, wp, m->P, l.n1, R, l.n1, wp, l.d_bias, 0);
    if (rc) return rc;
    const BranchW& b = l.br[0];
    if (b.d.kind == GTB_MIX_MINGRU) {
        const GruBranch a = gru_args(b);
        const int cb = (a.width + 127) / 128;
        if (portions) {
            int n_chunks = 0;
            for (int s = 0; s < S; s++) n_chunks += (seg_lens[s] + GRU_CHUNK - 1) / GRU_CHUNK;
            if ((size_t)n_chunks * 2 * a.width > m->gruAB_floats) return gtb::fail(GTB_ERR_STATE, "chunk workspace too small");
            k_mingru_chunk<<<dim3(n_chunks, cb), 128, 0, st>>>(t, a, m->P, l.n1, S, GRU_CHUNK, m->gruAB);
            GTB_LAUNCHED();
            k_mingru_chunk_out<OT><<<dim3(n_chunks, cb), 128, 0, st>>>(t, a, m->P, l.n1, S, GRU_CHUNK, m->gruAB, run.state[0], opC, l.kout_p);
            GTB_LAUNCHED();
            k_mingru_store<<<dim3(S, cb), 128, 0, st>>>(t, a, S, GRU_CHUNK, m->gruAB, run.state[0]);
            GTB_LAUNCHED();
        } else {
            k_mingru<OT><<<dim3(S, cb), 128, 0, st>>>(t, a, m->P, l.n1, run.state[0], opC, l.kout_p);
            GTB_LAUNCHED();
        }
    } else {
        const SoftAttn a = soft_args(m, b, run);
        k_sattn_prep<OT><<<dim3(R, (a.heads + 2 * a.kv_heads + 3) / 4), 128, 0, st>>>(t, a, m->P, l.n1, (OT*)run.kc[0], (OT*)run.vc[0]);
        GTB_LAUNCHED();
        if (a.pool > 0) {
            k_pool_update<OT><<<R, 128, 0, st>>>(t, a, (const OT*)run.kc[0], (const OT*)run.vc[0], run.pk, run.pv);
            GTB_LAUNCHED();
        }
        int done = -1;
        if (portions && sizeof(OT) == 2 && a.dim <= 128 && a.vdim <= 128)
            done = sattn_mma(t, a, S, n_qtiles, m->P, l.n1, (const bf16*)run.kc[0], (const bf16*)run.vc[0], run.pk, run.pv, (bf16*)opC, l.kout_p);
        if (done > 0) return done;
        if (done < 0 && !portions && R <= SPLIT_MAX_ROWS && m->sattn_part) {
            // decode rows: one CTA per 128 keys of the longest key list this layer can meet (window tokens + pooled blocks), at most 32
            const int max_keys = a.window > 0 ? std::min(c.max_ctx, a.window + (a.pool > 0 ? c.max_ctx / a.pool : 0)) : c.max_ctx;
            const int splits = std::max(1, std::min(32, (max_keys + 127) / 128));
            if (splits > 1) {
                k_sattn_split<OT><<<dim3(R, a.heads, splits), 128, (a.dim + 128 + 33) * sizeof(float), st>>>(t, a, m->P, l.n1, (const OT*)run.kc[0], (const OT*)run.vc[0], run.pk, run.pv, m->sattn_part, R);
                GTB_LAUNCHED();
                k_sattn_join<OT><<<dim3(R, a.heads), 128, 0, st>>>(a, m->P, l.n1, m->sattn_part, R, splits, opC, l.kout_p);
                GTB_LAUNCHED();
                done = 0;
            }
        }
        if (done < 0) {
            k_sattn<OT><<<dim3(R, a.heads), 128, (a.dim + 128 + 33) * sizeof(float), st>>>(t, a, m->P, l.n1, (const OT*)run.kc[0], (const OT*)run.vc[0], run.pk, run.pv, opC, l.kout_p);
            GTB_LAUNCHED();
        }
    }
    rc = product<OT>(m, opC, l.kout_p, l.w_out, l.kout_p, m->Y, W, R, W, l.kout_p, nullptr, 0);
    if (rc) return rc;
    // few rows and a routed feed-forward next: the residual update also computes the router's logits from the fp32 row it has just formed
    // and picks the experts (two launches less per layer on a decode step)
    RouteNext rn{};
    const bool routed = l.ff > 0 && l.d.ff_kind == GTB_FF_EXPERTS;
    const size_t rn_smem = routed ? ((size_t)W + 3 * l.n_out) * sizeof(float) : 0;
    if (routed && R <= 8 && rn_smem <= 40 * 1024) { rn.w = l.w_router; rn.ldw = wp; rn.n_out = l.n_out; rn.top = l.d.top; rn.corr = l.d_corr; rn.sel_idx = m->sel_idx; rn.sel_w = m->sel_w; }
    k_postnorm_add<OT><<<R, 256, rn.w ? rn_smem : 0, st>>>(m->Y, W, c.eps, l.norm1, nullptr, nullptr, 0, 0, nullptr, nullptr, m->x, opA, wp, rn);
    GTB_LAUNCHED();
    if (l.ff == 0) return GTB_OK;
    if (l.d.ff_kind == GTB_FF_POLYNORM) {
        rc = product<OT>(m, opA, wp, l.w_up, wp, m->G, l.ff, R, l.ff, wp, nullptr, 0);
        if (rc) return rc;
        k_polynorm<OT><<<R, 256, 0, st>>>(m->G, l.ff, l.ff, c.eps, l.d_act, opC, l.kfp);
        GTB_LAUNCHED();
        rc = product<OT>(m, opC, l.kfp, l.w_down, l.kfp, m->Y, W, R, W, l.kfp, nullptr, 0);
        if (rc) return rc;
        k_postnorm_add<OT><<<R, 256, 0, st>>>(m->Y, W, c.eps, l.norm2, nullptr, nullptr, 0, 0, nullptr, nullptr, m->x, opA, wp, RouteNext{});
        GTB_LAUNCHED();
        return GTB_OK;
    }
    const int E = l.d.experts, top = l.d.top;
    if (!rn.w) {
        rc = product<OT>(m, opA, wp, l.w_router, wp, m->rl, l.n_out, R, l.n_out, wp, nullptr, 0);
        if (rc) return rc;
        k_moe_route<<<R, 32, 2 * l.n_out * sizeof(float), st>>>(m->rl, l.n_out, l.n_out, l.d_corr, top, m->sel_idx, m->sel_w);
        GTB_LAUNCHED();
    }
    const int n_pairs = R * top, mpad = (n_pairs + 127) / 128 * 128 + E * 128;
    if (sizeof(OT) == 2 && E > 0 && m->grouped_experts && m->use_tensor && m->gp && m->Xg && R >= m->tensor_min_rows && mpad <= m->mpad_max) {
        // rows sorted by expert, two grouped tensor-core products (up with the weighted relu^2 epilogue, down), the choices of a row summed
        // in the residual update
        k_moe_group<<<1, 1024, 2 * E * sizeof(int), st>>>(m->sel_idx, n_pairs, E, m->pair_dst, m->tile_e, mpad / 128);
        GTB_LAUNCHED();
        k_moe_gather<<<n_pairs, 128, 0, st>>>((const bf16*)opA, wp, top, m->pair_dst, m->sel_w, m->Xg, m->rw);
        GTB_LAUNCHED();
        rc = seq_gemm_bf16_grouped(m->gp, m->Xg, wp, l.w_up, wp, mpad, l.ff, wp, E, m->tile_e, nullptr, 0, m->actg, l.kfp, m->rw);
        if (rc == 0) rc = seq_gemm_bf16_grouped(m->gp, m->actg, l.kfp, l.w_down, l.kfp, mpad, W, l.kfp, E, m->tile_e, m->Yg, W, nullptr, 0, nullptr);
        if (rc > 0) return rc;
        if (rc == 0) {
            k_postnorm_add<OT><<<R, 256, 0, st>>>(nullptr, W, c.eps, l.norm2, m->sel_idx, m->sel_w, top, E, m->Yg, m->pair_dst, m->x, opA, wp, RouteNext{});
            GTB_LAUNCHED();
            return GTB_OK;
        }
    }
    if (E > 0) {
        // a warp per output column; with few (row, choice) pairs every column group gets its own CTA so that the experts' matrices stream at
        // full width, with many pairs the grid is wide already
        const int cta_budget = std::max(1, 4096 / std::max(1, R * top));
        k_moe_up_rows<OT><<<dim3(R * top, std::max(1, std::min(cta_budget, (l.kfp + 7) / 8))), 256, 0, st>>>(opA, wp, wp, l.w_up, wp, l.ff, l.kfp, E, top, m->sel_idx, m->sel_w, (OT*)m->act);
        GTB_LAUNCHED();
        k_moe_down_rows<OT><<<dim3(R, std::max(1, std::min(std::max(1, 4096 / R), (W + 7) / 8))), 256, 0, st>>>((const OT*)m->act, l.kfp, l.w_down, W, E, top, m->sel_idx, m->Y, W);
        GTB_LAUNCHED();
    } else {
        GTB_CUDA(cudaMemsetAsync(m->Y, 0, (size_t)R * W * sizeof(float), st));
    }
    k_postnorm_add<OT><<<R, 256, 0, st>>>(m->Y, W, c.eps, l.norm2, m->sel_idx, m->sel_w, top, E, nullptr, nullptr, m->x, opA, wp, RouteNext{});
    GTB_LAUNCHED();
    return GTB_OK;
}

// One retention branch on R rows: projections in m->P, output into the out-projection operand.  Prompt portions run chunk-wise, everything
// else row by row from the slot's state.
template <typename OT>
int run_retention(gtb_seq_model* m, const PassTables& t, int R, int S, const Run& run, int bi, const LayerW& l, bool portions, const int* seg_lens) {
    cudaStream_t st = ctx().stream;
    const BranchW& b = l.br[bi];
    OT* opC = (OT*)m->opC;
    const RetBranch a = ret_args(m, b);
    const RetChunk rcfg = ret_chunk(b.d);
    const bool chunks = portions && rcfg.ok;
    if (b.d.act) {
        // in place, in one pass over q | k | v (neighbours in the projection): activating inside the chunk kernels instead was measured
        // slower (they read q and k twice; 41 us more in them against 23 us for this kernel at 2048 rows x 8 heads of 128)
        const int n = b.v_off + a.heads * a.vdim - b.q_off;
        k_silu_cols<<<(unsigned)(((size_t)R * n + 255) / 256), 256, 0, st>>>(m->P, l.n1, b.q_off, n, R);
        GTB_LAUNCHED();
    }
    auto post = [&]() -> int {
        if (b.d.out_norm == 2) k_ret_post_all<OT><<<R, 256, 0, st>>>(a, b.d_onorm, m->O, m->P, l.n1, opC, l.kout_p);
        else k_ret_post<OT><<<dim3(R, (a.heads + 3) / 4), 128, 0, st>>>(a, m->O, m->P, l.n1, opC, l.kout_p);
        GTB_LAUNCHED();
        return GTB_OK;
    };
    if (chunks) {
        int n_chunks = 0;
        for (int s = 0; s < S; s++) n_chunks += (seg_lens[s] + rcfg.C - 1) / rcfg.C;
        const size_t need = (size_t)n_chunks * a.heads * a.dim * a.vdim;
        if (need > m->retU_floats) return gtb::fail(GTB_ERR_STATE, "chunk workspace too small (%zu > %zu floats)", need, m->retU_floats);
        const int nvs = (a.vdim + rcfg.vs - 1) / rcfg.vs;
        if (a.rot_dims > 0 || a.scale != 1.0f) {
            k_ret_rotate<<<R, 128, 0, st>>>(t, a, m->P, l.n1);
            GTB_LAUNCHED();
        }
        if (rcfg.smem_kv > 48 * 1024) GTB_CUDA(cudaFuncSetAttribute(k_ret_chunk_kv, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rcfg.smem_kv));
        k_ret_chunk_kv<<<dim3(n_chunks, a.heads, nvs), 256, rcfg.smem_kv, st>>>(t, a, m->P, l.n1, S, rcfg.C, rcfg.vs, m->retU);
        GTB_LAUNCHED();
        k_ret_scan<<<dim3(S, a.heads, (a.dim * a.vdim + 255) / 256), 256, 0, st>>>(t, a, S, rcfg.C, m->retU, run.state[bi]);
        GTB_LAUNCHED();
        if (rcfg.smem_out > 48 * 1024) GTB_CUDA(cudaFuncSetAttribute(k_ret_chunk_out, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rcfg.smem_out));
        k_ret_chunk_out<<<dim3(n_chunks, a.heads, nvs), 256, rcfg.smem_out, st>>>(t, a, m->P, l.n1, S, rcfg.C, rcfg.vs, m->retU, m->O);
        GTB_LAUNCHED();
        return post();
    }
    const RetLaunch rl = ret_launch(b.d);
    if (rl.smem > 48 * 1024) GTB_CUDA(cudaFuncSetAttribute(k_retention, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)rl.smem));
    k_retention<<<dim3(S, a.heads, rl.nvs), rl.block, rl.smem, st>>>(t, a, m->P, l.n1, run.state[bi], m->O, rl.vs);
    GTB_LAUNCHED();
    return post();
}

// ---- sandwich layers ---------------------------------------------------------------------------------------------------------
NormArgs sw_norm(const gtb_seq_model* m, const LayerW& l, int q) {          // q: 0 norm1, 1 norm1b, 2 norm2, 3 norm2b
    NormArgs n{};
    n.kind = l.d.norm_kind; n.w = l.sn_w[q]; n.b = l.sn_b[q]; n.eps = m->cfg.eps;
    return n;
}

// the residual update with the fewest kept values per thread that hold a row of this width
template <typename OT>
void sandwich_add(int R, size_t smem, const float* Y, const float* Y2, const float* Yg, const int* pair_dst, int top, int W, const NormArgs& post, float* x, const NormArgs& next,
                  OT* op, int ld_op, const GroupRouteNext& rn) {
    cudaStream_t st = ctx().stream;
    if (W <= 1024) k_sandwich_add<OT, 1><<<R, 256, smem, st>>>(Y, Y2, Yg, pair_dst, top, W, post, x, next, op, ld_op, rn);
    else if (W <= 2048) k_sandwich_add<OT, 2><<<R, 256, smem, st>>>(Y, Y2, Yg, pair_dst, top, W, post, x, next, op, ld_op, rn);
    else k_sandwich_add<OT, 4><<<R, 256, smem, st>>>(Y, Y2, Yg, pair_dst, top, W, post, x, next, op, ld_op, rn);
}

// One softmax-attention branch of a sandwich layer on R rows: projections in m->P, output into the out-projection operand.
template <typename OT>
int run_soft_branch(gtb_seq_model* m, const PassTables& t, int R, int S, const Run& run, int bi, const LayerW& l, bool portions, int n_qtiles) {
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    const BranchW& b = l.br[bi];
    OT* opC = (OT*)m->opC;
    const SoftAttn a = soft_args(m, b, run);
    const int M = a.maps, units = a.heads * M, nk = a.own_kv ? a.kv_heads * M : 0;
    if (a.qk_norm == 3) {
        k_proj_rms<<<R, 256, 0, st>>>(m->P, l.n1, a.q_off, units * a.dim, a.k_off, nk * a.dim, c.eps, m->qk_sc);
        GTB_LAUNCHED();
    }
    k_sattn_prep<OT><<<dim3(R, (units + nk + (a.own_kv ? a.kv_heads : 0) + 3) / 4), 128, 0, st>>>(t, a, m->P, l.n1, (OT*)run.kc[bi], (OT*)run.vc[bi]);
    GTB_LAUNCHED();
    // two maps per head: the units' outputs stay fp32 (their difference is taken afterwards), unit-major in m->O
    float* of = M > 1 ? m->O : nullptr;
    const int ldf = units * a.vdim;
    SoftAttn af = a;
    af.a_off = 0;
    const size_t smem = (a.dim + 128 + 33) * sizeof(float);
    int done = -1;
    if (portions && sizeof(OT) == 2 && a.dim <= 128 && a.vdim <= 128)
        done = sattn_mma(t, a, S, n_qtiles, m->P, l.n1, (const bf16*)run.kc[bi], (const bf16*)run.vc[bi], nullptr, nullptr, (bf16*)opC, l.kout_p, of, ldf);
    if (done > 0) return done;
    if (done < 0 && !portions && R <= SPLIT_MAX_ROWS && m->sattn_part) {
        int max_keys = c.max_ctx;
        if (a.window > 0) max_keys = std::min(max_keys, a.window);
        if (a.chunk > 0) max_keys = std::min(max_keys, a.chunk);
        const int splits = std::max(1, std::min(32, (max_keys + 127) / 128));
        if (splits > 1) {
            k_sattn_split<OT><<<dim3(R, units, splits), 128, smem, st>>>(t, a, m->P, l.n1, (const OT*)run.kc[bi], (const OT*)run.vc[bi], nullptr, nullptr, m->sattn_part, R);
            GTB_LAUNCHED();
            if (of) k_sattn_join<float><<<dim3(R, units), 128, 0, st>>>(af, m->P, l.n1, m->sattn_part, R, splits, of, ldf);
            else k_sattn_join<OT><<<dim3(R, units), 128, 0, st>>>(a, m->P, l.n1, m->sattn_part, R, splits, opC, l.kout_p);
            GTB_LAUNCHED();
            done = 0;
        }
    }
    if (done < 0) {
        if (of) k_sattn<OT, float><<<dim3(R, units), 128, smem, st>>>(t, af, m->P, l.n1, (const OT*)run.kc[bi], (const OT*)run.vc[bi], nullptr, nullptr, of, ldf);
        else k_sattn<OT, OT><<<dim3(R, units), 128, smem, st>>>(t, a, m->P, l.n1, (const OT*)run.kc[bi], (const OT*)run.vc[bi], nullptr, nullptr, opC, l.kout_p);
        GTB_LAUNCHED();
    }
    if (of) {
        DiffArgs d{};
        d.heads = a.heads; d.dim = a.dim; d.vdim = a.vdim; d.diff = b.d.diff; d.eps = c.eps; d.out_scale = b.d.out_scale != 0.0f ? b.d.out_scale : 1.0f;
        d.lq1 = b.d_lam[0]; d.lk1 = b.d_lam[1]; d.lq2 = b.d_lam[2]; d.lk2 = b.d_lam[3];
        d.gate = b.d.gated; d.g_off = b.g_off; d.a_off = b.a_off;
        k_diff_combine<OT><<<dim3(R, (a.heads + 3) / 4), 128, 0, st>>>(d, of, m->P, l.n1, opC, l.kout_p);
        GTB_LAUNCHED();
    }
    return GTB_OK;
}

// One layer of the sandwich style on R rows: x += norm1b(mixer(norm1(x))); x += norm2b(ff(norm2(x))).  opA holds norm1(x) on entry; on
// return it holds `next` of the new stream (the following layer's norm1) when next.w is set.
template <typename OT>
int run_sandwich_layer(gtb_seq_model* m, const PassTables& t, int R, int S, const Run& run, const LayerW& l, bool portions, const int* seg_lens, int n_qtiles,
                       const NormArgs& next) {
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    const int W = c.width, wp = m->wp;
    OT *opA = (OT*)m->opA, *opC = (OT*)m->opC;
    int rc = product<OT>(m, opA, wp, l.w_mix, wp, m->P, l.n1, R, l.n1, wp, l.d_bias, 0);
    if (rc) return rc;
    for (int bi = 0; bi < l.d.n_branches; bi++) {
        if (l.br[bi].d.kind == GTB_MIX_SOFTMAX_ATTN) rc = run_soft_branch<OT>(m, t, R, S, run, bi, l, portions, n_qtiles);
        else rc = run_retention<OT>(m, t, R, S, run, bi, l, portions, seg_lens);
        if (rc) return rc;
    }
    rc = product<OT>(m, opC, l.kout_p, l.w_out, l.kout_p, m->Y, W, R, W, l.kout_p, nullptr, 0);
    if (rc) return rc;
    // few rows and a routed feed-forward next: the residual update also computes the router's logits from the operand row it has just formed
    // and picks the experts (two launches less per layer on a decode step)
    GroupRouteNext rn{};
    const int groups = std::max(1, l.d.route_groups), keep = l.d.route_keep > 0 ? l.d.route_keep : groups;
    const bool routed = l.ff > 0 && l.d.ff_kind == GTB_FF_GROUP_EXPERTS;
    const size_t rn_smem = routed ? ((size_t)W + 3 * l.d.experts + groups) * sizeof(float) : 0;
    if (routed && R <= 8 && rn_smem <= 40 * 1024) {
        rn.w = l.w_router; rn.ldw = wp; rn.n_exp = l.d.experts; rn.n_groups = groups; rn.keep = keep; rn.top = l.d.top; rn.n_always = l.n_sh; rn.scale = l.d.route_scale;
        rn.sel_idx = m->sel_idx; rn.sel_w = m->sel_w;
    }
    sandwich_add<OT>(R, rn.w ? rn_smem : 0, m->Y, nullptr, nullptr, nullptr, 0, W, sw_norm(m, l, 1), m->x, l.ff > 0 ? sw_norm(m, l, 2) : next, opA, wp, rn);
    GTB_LAUNCHED();
    if (l.ff == 0) return GTB_OK;
    if (l.d.ff_kind == GTB_FF_SWIGLU) {
        bool act_done = false;
        if (sizeof(OT) == 2 && m->use_tensor && m->gp && R >= m->tensor_min_rows && l.gu_inter) {
            rc = seq_gemm_bf16_gated(m->gp, opA, wp, l.w_gu, wp, opC, l.kfp, 0, R, 2 * l.ff, wp, 1, nullptr);
            if (rc > 0) return rc;
            if (rc == 0) { ctx().launches++; act_done = true; }
        }
        if (!act_done) {
            rc = product<OT>(m, opA, wp, l.w_gu, wp, m->G, 2 * l.ff, R, 2 * l.ff, wp, nullptr, 0);
            if (rc) return rc;
            k_swiglu_rows<OT><<<dim3(R, std::max(1, std::min((l.kfp + 255) / 256, std::max(1, 2048 / R)))), 256, 0, st>>>(m->G, l.ff, l.gu_inter ? 1 : 0, nullptr, opC, l.kfp);
            GTB_LAUNCHED();
        }
        rc = product<OT>(m, opC, l.kfp, l.w_down, l.kfp, m->Y, W, R, W, l.kfp, nullptr, 0);
        if (rc) return rc;
        sandwich_add<OT>(R, 0, m->Y, nullptr, nullptr, nullptr, 0, W, sw_norm(m, l, 3), m->x, next, opA, wp, GroupRouteNext{});
        GTB_LAUNCHED();
        return GTB_OK;
    }
    // group-limited experts; the parts of the shared expert are choices top .. top + n_sh - 1 of every row
    const int E = l.d.experts, Et = l.e_total, top = l.d.top + l.n_sh;
    if (!rn.w) {
        rc = product<OT>(m, opA, wp, l.w_router, wp, m->rl, E, R, E, wp, nullptr, 0);
        if (rc) return rc;
        k_moe_route_grouped<<<R, 32, (2 * E + groups) * sizeof(float), st>>>(m->rl, E, E, groups, keep, l.d.top, l.d.route_scale, l.n_sh, m->sel_idx, m->sel_w);
        GTB_LAUNCHED();
    }
    const int n_pairs = R * top, mpad = (n_pairs + 127) / 128 * 128 + Et * 128;
    if (sizeof(OT) == 2 && m->grouped_experts && m->use_tensor && m->gp && m->Xg && R >= m->tensor_min_rows && mpad <= m->mpad_max) {
        k_moe_group<<<1, 1024, 2 * Et * sizeof(int), st>>>(m->sel_idx, n_pairs, Et, m->pair_dst, m->tile_e, mpad / 128);
        GTB_LAUNCHED();
        k_moe_gather<<<n_pairs, 128, 0, st>>>((const bf16*)opA, wp, top, m->pair_dst, m->sel_w, m->Xg, m->rw);
        GTB_LAUNCHED();
        rc = seq_gemm_bf16_grouped(m->gp, m->Xg, wp, l.w_up, wp, mpad, l.ff, wp, Et, m->tile_e, nullptr, 0, m->actg, l.kfp, m->rw);
        if (rc == 0) rc = seq_gemm_bf16_grouped(m->gp, m->actg, l.kfp, l.w_down, l.kfp, mpad, W, l.kfp, Et, m->tile_e, m->Yg, W, nullptr, 0, nullptr);
        if (rc > 0) return rc;
        if (rc == 0) {
            sandwich_add<OT>(R, 0, nullptr, nullptr, m->Yg, m->pair_dst, top, W, sw_norm(m, l, 3), m->x, next, opA, wp, GroupRouteNext{});
            GTB_LAUNCHED();
            return GTB_OK;
        }
    }
    const int cta_budget = std::max(1, 4096 / std::max(1, R * top));
    k_moe_up_rows<OT><<<dim3(R * top, std::max(1, std::min(cta_budget, (l.kfp + 7) / 8))), 256, 0, st>>>(opA, wp, wp, l.w_up, wp, l.ff, l.kfp, Et, top, m->sel_idx, m->sel_w, (OT*)m->act);
    GTB_LAUNCHED();
    k_moe_down_rows<OT><<<dim3(R, std::max(1, std::min(std::max(1, 4096 / R), (W + 7) / 8))), 256, 0, st>>>((const OT*)m->act, l.kfp, l.w_down, W, Et, top, m->sel_idx, m->Y, W);
    GTB_LAUNCHED();
    sandwich_add<OT>(R, 0, m->Y, nullptr, nullptr, nullptr, 0, W, sw_norm(m, l, 3), m->x, next, opA, wp, GroupRouteNext{});
    GTB_LAUNCHED();
    return GTB_OK;
}

// ---- pre-norm layers ---------------------------------------------------------------------------------------------------------
// a finished sublayer whose update of the stream copies has not been applied yet
struct PendingUpdate {
    const float* Y = nullptr;  const float* Y2 = nullptr;             // the sublayer's output (Y2: a second share, the shared expert)
    const float* Yg = nullptr; const int* pair_dst = nullptr; int top = 0;   // grouped experts: rows of Yg to sum instead of Y
    const float* hc = nullptr; int src_ns = 1;
};

NormArgs norm_args(const gtb_seq_model* m, const LayerW& l, int q) {
    NormArgs n{};
    n.kind = l.d.norm_kind; n.w = q == 0 ? l.norm1 : l.norm2; n.b = l.nb[q]; n.alpha = l.na[q]; n.eps = m->cfg.eps;
    return n;
}
// applies the pending update (if any) to the copies and forms the next sublayer's input in opA (hc_next: its [in | out | mix]; null: none)
template <typename OT>
int hc_boundary(gtb_seq_model* m, int R, PendingUpdate& pend, const float* hc_next, const NormArgs& nrm, float* xsum) {
    const int W = m->cfg.width;
    const bool whole_row = hc_next && nrm.kind == GTB_NORM_RMS;       // the RMS norm sums over the row inside one CTA
    const int V = W % 4 == 0 ? 4 : 1;
    const int gy = whole_row ? 1 : std::max(1, std::min((W / V + 255) / 256, std::max(1, 2048 / R)));
#define HC_LAUNCH(VV, NN) k_hc_step<OT, VV, NN><<<dim3(R, gy), 256, 0, ctx().stream>>>(m->xs, (size_t)m->max_rows * W, m->ns, pend.src_ns, W, pend.Y, pend.Y2, pend.Yg, \
                                                                                      pend.pair_dst, pend.top, pend.hc, hc_next, nrm, (OT*)m->opA, m->wp, xsum)
    if (V == 4) { if (m->ns <= 2) HC_LAUNCH(4, 2); else if (m->ns <= 4) HC_LAUNCH(4, 4); else HC_LAUNCH(4, 8); }
    else { if (m->ns <= 2) HC_LAUNCH(1, 2); else if (m->ns <= 4) HC_LAUNCH(1, 4); else HC_LAUNCH(1, 8); }
#undef HC_LAUNCH
    GTB_LAUNCHED();
    pend = PendingUpdate{};
    pend.src_ns = m->ns;
    return GTB_OK;
}

LatAttn lat_args(const gtb_seq_model* m, const BranchW& b) {
    LatAttn a{};
    a.heads = b.d.heads; a.dim = b.d.dim; a.rope = b.d.rope_dim; a.vdim = b.d.vdim; a.rank = b.d.kv_rank; a.q_rank = b.d.q_rank;
    a.rot_dims = b.d.rot_dims; a.rot_layout = b.d.rot_layout; a.inv_freq = b.d_inv_freq; a.kv_norm = b.d_kvnorm; a.q_norm = b.d_qnorm;
    a.eps = m->cfg.eps; a.q_off = b.q_off; a.kv_off = b.kv_off; a.g_off = b.g_off; a.a_off = b.a_off; a.c_ld = b.c_ld; a.max_ctx = m->cfg.max_ctx;
    return a;
}
// the absorbed form as a softmax attention with one K/V head over the latent cache: keys [latent | rotated part], values the latent
SoftAttn lat_soft_args(const gtb_seq_model* m, const BranchW& b) {
    SoftAttn a{};
    a.heads = b.d.heads; a.kv_heads = 1; a.dim = b.d.kv_rank + b.d.rope_dim; a.vdim = b.d.kv_rank;
    a.scale = b.d.scale; a.eps = m->cfg.eps; a.window = b.d.window; a.sink = b.d_sink;
    a.k_ld = a.v_ld = b.c_ld; a.own_kv = 1; a.max_ctx = m->cfg.max_ctx;
    return a;
}

template <int VPW>
int launch_lat_dec_mma(const PassTables& t, const SoftAttn& a, int R, int splits, const float* QA, int ldqa, const bf16* cache, float* part) {
    const int DP = (a.dim + 15) & ~15;
    const size_t smem = (size_t)(16 + 64) * (DP + 8) * 2 + 16 * (64 + 8) * 2 + 64 * sizeof(float);
    static size_t allowed = 48 * 1024;
    if (smem > 200 * 1024) return -1;
    if (smem > allowed) { GTB_CUDA(cudaFuncSetAttribute(k_lat_dec_mma<VPW>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem)); allowed = smem; }
    k_lat_dec_mma<VPW><<<dim3(R, (a.heads + 15) / 16, splits), 128, smem, ctx().stream>>>(t, a, QA, ldqa, cache, part, R);
    GTB_LAUNCHED();
    return GTB_OK;
}
// -1: sizes outside the kernel (the caller takes the row kernels)
int lat_dec_mma(const PassTables& t, const SoftAttn& a, int R, int splits, const float* QA, int ldqa, const bf16* cache, float* part) {
    if (a.vdim <= 128) return launch_lat_dec_mma<32>(t, a, R, splits, QA, ldqa, cache, part);
    if (a.vdim <= 256) return launch_lat_dec_mma<64>(t, a, R, splits, QA, ldqa, cache, part);
    if (a.vdim <= 512) return launch_lat_dec_mma<128>(t, a, R, splits, QA, ldqa, cache, part);
    return -1;
}

// One pre-norm layer on R rows.  pend carries the update of the sublayer before it (none for the first layer) and leaves with this
// layer's last sublayer pending; cap_prev: where the sum of the copies after the previous layer goes (capture), or null.
template <typename OT>
int run_prenorm_layer(gtb_seq_model* m, const PassTables& t, int R, int S, const Run& run, const LayerW& l, bool portions, const int* seg_lens, const int* seg_slots,
                      int n_qtiles, PendingUpdate& pend, float* cap_prev) {
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    const int W = c.width, wp = m->wp;
    OT *opA = (OT*)m->opA, *opC = (OT*)m->opC;
    int rc = hc_boundary<OT>(m, R, pend, l.hc[0], norm_args(m, l, 0), cap_prev);
    if (rc) return rc;
    rc = product<OT>(m, opA, wp, l.w_mix, wp, m->P, l.n1, R, l.n1, wp, nullptr, 0);
    if (rc) return rc;
    const BranchW& b = l.br[0];
    // prompt portions in bf16 mode: keys and values of the visible range are expanded from the cached latents and the heads run the
    // tensor-core softmax attention; everything else runs the absorbed form on the row kernels
    const bool expand = portions && sizeof(OT) == 2 && seg_slots && m->latKx && b.d.dim + b.d.rope_dim <= 128 && b.d.vdim <= 128;
    {
        const LatAttn a = lat_args(m, b);
        const int hd = a.dim + a.rope;
        k_lat_prep<OT><<<dim3(R, a.q_rank > 0 ? 2 : 1), 128, 0, st>>>(t, a, m->P, l.n1, (OT*)run.kc[0], (OT*)m->opQ, b.qrank_p);
        GTB_LAUNCHED();
        const float* Q = m->P;
        int ldq = l.n1, q0 = b.q_off;
        if (a.q_rank > 0) {
            ldq = a.heads * hd + a.heads;         // room for the heads' gate logits behind the queries (the tiled path reads them there)
            rc = product<OT>(m, m->opQ, b.qrank_p, b.w_uq, b.qrank_p, m->latQ, ldq, R, a.heads * hd, b.qrank_p, nullptr, 0);
            if (rc) return rc;
            Q = m->latQ; q0 = 0;
        }
        if (expand) {
            const int ld_qr = a.heads * hd + a.heads, nx = a.heads * (a.dim + a.vdim);
            k_lat_qrot<<<R, 128, 0, st>>>(t, a, Q, ldq, q0, m->P, l.n1, m->latQ, ld_qr);
            GTB_LAUNCHED();
            for (int s = 0; s < S; s++) {
                const int slot = seg_slots[s], p0 = m->host_pos[slot];
                const int lo = b.d.window > 0 ? std::max(0, p0 - b.d.window + 1) : 0, n = p0 + seg_lens[s] - lo;
                const bf16* src = (const bf16*)run.kc[0] + ((size_t)slot * c.max_ctx + lo) * b.c_ld;
                rc = product<OT>(m, src, b.c_ld, b.w_uk, b.rank_p, m->latX, nx, n, nx, b.rank_p, nullptr, 0);      // uk and uv rows are one matrix
                if (rc) return rc;
                k_lat_pack<<<n, 256, 0, st>>>(a, m->latX, n, slot, lo, (const bf16*)run.kc[0], m->latKx, m->latVx);
                GTB_LAUNCHED();
            }
            SoftAttn sa{};
            sa.heads = sa.kv_heads = a.heads; sa.dim = hd; sa.vdim = a.vdim; sa.scale = b.d.scale; sa.eps = c.eps; sa.window = b.d.window; sa.sink = b.d_sink;
            sa.gate = b.d.gated; sa.q_off = 0; sa.g_off = a.heads * hd; sa.a_off = b.a_off; sa.own_kv = 1; sa.max_ctx = c.max_ctx;
            rc = sattn_mma(t, sa, S, n_qtiles, m->latQ, ld_qr, m->latKx, m->latVx, nullptr, nullptr, (bf16*)opC, l.kout_p);
            if (rc > 0) return rc;
            if (rc < 0) return gtb::fail(GTB_ERR_STATE, "head sizes outside the tiled attention kernel");
        }
    }
    if (!expand) {
        const LatAttn a = lat_args(m, b);
        const int hd = a.dim + a.rope;
        const float* Q = a.q_rank > 0 ? m->latQ : m->P;
        const int ldq = a.q_rank > 0 ? a.heads * hd + a.heads : l.n1, q0 = a.q_rank > 0 ? 0 : b.q_off;
        k_lat_qabs<<<dim3(R, a.heads, (a.rank + 127) / 128), 128, (hd + 512) * sizeof(float), st>>>(t, a, Q, ldq, q0, b.w_uk, b.rank_p, m->latQA);
        GTB_LAUNCHED();
        const SoftAttn sa = lat_soft_args(m, b);
        const int ldqa = a.heads * sa.dim, ld_ol = (a.heads * a.rank + 7) / 8 * 8;
        const size_t smem = (sa.dim + 128 + 33) * sizeof(float);
        bool done = false;
        if (sizeof(OT) == 2 && m->fused_attn && !portions && R <= SPLIT_MAX_ROWS && m->sattn_part) {
            // decode rows in bf16 mode: 16 heads per CTA on tensor cores, one CTA per 64 keys of the longest key list this layer can meet
            const int max_keys = sa.window > 0 ? std::min(c.max_ctx, sa.window) : c.max_ctx;
            const int splits = std::max(1, std::min(32, (max_keys + 63) / 64));
            rc = lat_dec_mma(t, sa, R, splits, m->latQA, ldqa, (const bf16*)run.kc[0], m->sattn_part);
            if (rc > 0) return rc;
            if (rc == 0) {
                k_sattn_join<OT><<<dim3(R, sa.heads), 128, 0, st>>>(sa, m->latQA, ldqa, m->sattn_part, R, splits, (OT*)m->opO, ld_ol);
                GTB_LAUNCHED();
                done = true;
            }
        }
        if (!done && !portions && R <= SPLIT_MAX_ROWS && m->sattn_part) {
            const int max_keys = sa.window > 0 ? std::min(c.max_ctx, sa.window) : c.max_ctx;
            const int splits = std::max(1, std::min(32, (max_keys + 127) / 128));
            if (splits > 1) {
                k_sattn_split<OT><<<dim3(R, sa.heads, splits), 128, smem, st>>>(t, sa, m->latQA, ldqa, (const OT*)run.kc[0], (const OT*)run.kc[0], nullptr, nullptr, m->sattn_part, R);
                GTB_LAUNCHED();
                k_sattn_join<OT><<<dim3(R, sa.heads), 128, 0, st>>>(sa, m->latQA, ldqa, m->sattn_part, R, splits, (OT*)m->opO, ld_ol);
                GTB_LAUNCHED();
                done = true;
            }
        }
        if (!done) {
            k_sattn<OT><<<dim3(R, sa.heads), 128, smem, st>>>(t, sa, m->latQA, ldqa, (const OT*)run.kc[0], (const OT*)run.kc[0], nullptr, nullptr, (OT*)m->opO, ld_ol);
            GTB_LAUNCHED();
        }
        const int n_out = a.heads * a.vdim;
        k_lat_vup<OT><<<dim3(R, std::max(1, std::min(std::max(1, 4096 / R), (n_out + 7) / 8))), 256, 0, st>>>(a, (const OT*)m->opO, ld_ol, b.w_uv, b.rank_p, m->P, l.n1, b.d.gated, opC, l.kout_p);
        GTB_LAUNCHED();
    }
    rc = product<OT>(m, opC, l.kout_p, l.w_out, l.kout_p, m->Y, W, R, W, l.kout_p, nullptr, 0);
    if (rc) return rc;
    pend.Y = m->Y; pend.hc = l.hc[0];
    if (l.ff == 0) return GTB_OK;
    rc = hc_boundary<OT>(m, R, pend, l.hc[1], norm_args(m, l, 1), nullptr);
    if (rc) return rc;
    if (l.d.ff_kind == GTB_FF_GEGLU) {
        bool act_done = false;
        if (sizeof(OT) == 2 && m->use_tensor && m->gp && R >= m->tensor_min_rows && l.gu_inter) {
            rc = seq_gemm_bf16_geglu(m->gp, opA, wp, l.w_gu, wp, opC, l.kfp, 0, R, 2 * l.ff, wp);
            if (rc > 0) return rc;
            if (rc == 0) { ctx().launches++; act_done = true; }
        }
        if (!act_done) {
            rc = product<OT>(m, opA, wp, l.w_gu, wp, m->G, 2 * l.ff, R, 2 * l.ff, wp, nullptr, 0);
            if (rc) return rc;
            const size_t n = (size_t)R * l.ff;
            k_geglu<OT><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(m->G, l.ff, opC, l.kfp, 0, R, l.gu_inter ? 1 : 0);
            GTB_LAUNCHED();
        }
        rc = product<OT>(m, opC, l.kfp, l.w_down, l.kfp, m->Y, W, R, W, l.kfp, nullptr, 0);
        if (rc) return rc;
        pend.Y = m->Y; pend.hc = l.hc[1];
        return GTB_OK;
    }
    // gated routed experts: router (and the shared expert's gate) in one product, fp32 accumulation
    const int E = l.d.experts, top = l.d.top;
    rc = product<OT>(m, opA, wp, l.w_router, wp, m->rl, l.n_out, R, l.n_out, wp, nullptr, 0);
    if (rc) return rc;
    k_moe_route_sigmoid<<<R, 32, E * sizeof(float), st>>>(m->rl, l.n_out, E, top, m->sel_idx, m->sel_w, l.sff > 0 ? m->shw : nullptr);
    GTB_LAUNCHED();
    if (l.sff > 0) {
        bool act_done = false;
        if (sizeof(OT) == 2 && m->use_tensor && m->gp && R >= m->tensor_min_rows && l.sh_inter) {
            rc = seq_gemm_bf16_gated(m->gp, opA, wp, l.w_sh_gu, wp, opC, l.sff_p, 0, R, 2 * l.sff, wp, 1, m->shw);
            if (rc > 0) return rc;
            if (rc == 0) { ctx().launches++; act_done = true; }
        }
        if (!act_done) {
            rc = product<OT>(m, opA, wp, l.w_sh_gu, wp, m->G, 2 * l.sff, R, 2 * l.sff, wp, nullptr, 0);
            if (rc) return rc;
            k_swiglu_rows<OT><<<dim3(R, std::max(1, std::min((l.sff_p + 255) / 256, std::max(1, 2048 / R)))), 256, 0, st>>>(m->G, l.sff, l.sh_inter ? 1 : 0, m->shw, opC, l.sff_p);
            GTB_LAUNCHED();
        }
        rc = product<OT>(m, opC, l.sff_p, l.w_sh_down, l.sff_p, m->Y2, W, R, W, l.sff_p, nullptr, 0);
        if (rc) return rc;
        pend.Y2 = m->Y2;
    }
    const int n_pairs = R * top, mpad = (n_pairs + 127) / 128 * 128 + E * 128;
    if (sizeof(OT) == 2 && m->grouped_experts && m->use_tensor && m->gp && m->Xg && l.e_inter && R >= m->tensor_min_rows && mpad <= m->mpad_max) {
        // rows sorted by expert; the gate-and-up product writes w * silu(gate) * up per (row, choice), the down product one output row per pair,
        // and the next boundary sums a row's pairs
        k_moe_group<<<1, 1024, 2 * E * sizeof(int), st>>>(m->sel_idx, n_pairs, E, m->pair_dst, m->tile_e, mpad / 128);
        GTB_LAUNCHED();
        k_moe_gather<<<n_pairs, 128, 0, st>>>((const bf16*)opA, wp, top, m->pair_dst, m->sel_w, m->Xg, m->rw);
        GTB_LAUNCHED();
        rc = seq_gemm_bf16_grouped_gated(m->gp, m->Xg, wp, l.w_up, wp, mpad, 2 * l.ff, wp, E, m->tile_e, m->actg, l.kfp, m->rw, 1);
        if (rc == 0) rc = seq_gemm_bf16_grouped(m->gp, m->actg, l.kfp, l.w_down, l.kfp, mpad, W, l.kfp, E, m->tile_e, m->Yg, W, nullptr, 0, nullptr);
        if (rc > 0) return rc;
        if (rc == 0) {
            pend.Yg = m->Yg; pend.pair_dst = m->pair_dst; pend.top = top; pend.hc = l.hc[1];
            return GTB_OK;
        }
    }
    {
        const int cta_budget = std::max(1, 4096 / std::max(1, R * top));
        k_moe_gu_rows<OT><<<dim3(R * top, std::max(1, std::min(cta_budget, (l.kfp + 7) / 8))), 256, 0, st>>>(opA, wp, wp, l.w_up, wp, l.ff, l.kfp, l.e_inter ? 1 : 0, top, m->sel_idx, m->sel_w, (OT*)m->act);
        GTB_LAUNCHED();
        k_moe_down_rows<OT><<<dim3(R, std::max(1, std::min(std::max(1, 4096 / R), (W + 7) / 8))), 256, 0, st>>>((const OT*)m->act, l.kfp, l.w_down, W, E, top, m->sel_idx, m->Y, W);
        GTB_LAUNCHED();
    }
    pend.Y = m->Y; pend.hc = l.hc[1];
    return GTB_OK;
}

// the launch sequence of one pass: R rows of S segments whose tables are already on the device
template <typename OT>
int run_pass(gtb_seq_model* m, const PassTables& t, int R, int S, bool from_pending, int n_want, const int* d_want, const int* seg_lens = nullptr,
             const int* seg_slots = nullptr) {
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    const int W = c.width, wp = m->wp;
    OT *opA = (OT*)m->opA, *opB = (OT*)m->opB, *opC = (OT*)m->opC, *opL = (OT*)m->opL, *opH = (OT*)m->opH;
    // prompt portions (the host knows the segment lengths and they are long on average) take the tiled kernels of the mixers
    const bool portions = seg_lens != nullptr && m->fused_attn && R >= 16 * S;
    int n_qtiles = 0;
    if (portions) for (int s = 0; s < S; s++) n_qtiles += (seg_lens[s] + 63) / 64;
    k_plan<<<(R + 127) / 128, 128, 0, st>>>(t, R, from_pending ? 1 : 0);
    GTB_LAUNCHED();
    const bool first_reads_x = m->L[m->runs[0].layer].d.style == GTB_BLOCK_POSTNORM;
    const float emb_scale = c.embed_scale != 0.0f ? c.embed_scale : 1.0f;
    if (m->sandwich && c.bigram_buckets == 0) {     // embedding and the first layer's input norm in one kernel; every later norm comes out of a residual update
        k_embed_norm<OT><<<R, 256, 0, st>>>(t, m->embed, W, emb_scale, sw_norm(m, m->L[m->runs[0].layer], 0), m->x, opA, wp);
        GTB_LAUNCHED();
    } else {
        k_embed<OT><<<R, 256, 0, st>>>(t, m->embed, m->bigram, c.bigram_buckets, c.bigram_mul_prev, c.bigram_mul_cur, W, emb_scale,
                                       m->prenorm ? m->xs : m->x, c.loop_times > 0 ? m->x0 : nullptr, first_reads_x ? opA : (OT*)nullptr, wp);
        GTB_LAUNCHED();
        if (m->sandwich) {
            k_norm_rows<OT><<<R, 256, 0, st>>>(m->x, W, sw_norm(m, m->L[m->runs[0].layer], 0), nullptr, opA, wp);
            GTB_LAUNCHED();
        }
    }
    bool x_in_opA = first_reads_x;
    PendingUpdate pend;                       // pre-norm layers: the embedding fills the first copy of the stream only
    for (size_t u = 0; u < m->runs.size(); u++) {
        const Run& run = m->runs[u];
        const LayerW& l = m->L[run.layer];
        if (l.d.style == GTB_BLOCK_SANDWICH) {
            const NormArgs next = u + 1 < m->runs.size() ? sw_norm(m, m->L[m->runs[u + 1].layer], 0) : NormArgs{};
            int rc = run_sandwich_layer<OT>(m, t, R, S, run, l, portions, seg_lens, n_qtiles, next);
            if (rc) return rc;
            if (m->capture) {
                GTB_CUDA(cudaMemcpyAsync(m->cap + u * (size_t)m->max_rows * W, m->x, (size_t)R * W * sizeof(float), cudaMemcpyDeviceToDevice, st));
                m->cap_rows = R;
            }
            continue;
        }
        if (l.d.style == GTB_BLOCK_PRENORM) {
            float* cap_prev = (m->capture && u > 0) ? m->cap + (u - 1) * (size_t)m->max_rows * W : nullptr;
            int rc = run_prenorm_layer<OT>(m, t, R, S, run, l, portions, seg_lens, seg_slots, n_qtiles, pend, cap_prev);
            if (rc) return rc;
            if (u + 1 == m->runs.size()) {     // the last update, and the sum of the copies for the output norm
                rc = hc_boundary<OT>(m, R, pend, nullptr, NormArgs{}, m->x);
                if (rc) return rc;
                if (m->capture) {
                    GTB_CUDA(cudaMemcpyAsync(m->cap + u * (size_t)m->max_rows * W, m->x, (size_t)R * W * sizeof(float), cudaMemcpyDeviceToDevice, st));
                    m->cap_rows = R;
                }
            }
            continue;
        }
        if (l.d.style == GTB_BLOCK_POSTNORM) {
            int rc = run_postnorm_layer<OT>(m, t, R, S, run, l, portions, seg_lens, n_qtiles, x_in_opA);
            if (rc) return rc;
            x_in_opA = true;
            if (m->capture) {
                GTB_CUDA(cudaMemcpyAsync(m->cap + u * (size_t)m->max_rows * W, m->x, (size_t)R * W * sizeof(float), cudaMemcpyDeviceToDevice, st));
                m->cap_rows = R;
            }
            continue;
        }
        x_in_opA = false;
        if (run.enters_pass) {
            k_concat2<OT><<<R, 256, 0, st>>>(m->x, m->x0, W, opL, pad64(2 * W));
            GTB_LAUNCHED();
            int rc = product<OT>(m, opL, pad64(2 * W), m->loop_in, pad64(2 * W), m->x, W, R, W, pad64(2 * W), m->loop_step + (size_t)run.pass * W, 0);
            if (rc) return rc;
        }
        OT* ob = l.ff > 0 ? opB : nullptr;
        const bool nc_fused = c.taps > 0 && c.taps <= 8 && m->fused_norm && R >= 32;     // few rows: two kernels with channel-wide grids are quicker
        if (nc_fused) {
            k_norm_canon<OT><<<R, 256, 0, st>>>(t, m->x, W, c.eps, l.d_gain, c.taps, l.canon_a, l.ff > 0 ? l.canon_b : nullptr, run.tail, m->h, opA, ob, wp);
            GTB_LAUNCHED();
        } else {
            k_rmsnorm_scalar<float><<<R, 256, 0, st>>>(m->x, W, c.eps, l.d_gain, nullptr, m->h, W);
            GTB_LAUNCHED();
        }
        if (c.taps > 0) {
            if (!nc_fused) {
                k_canon<OT><<<dim3(R, (W + 255) / 256), 256, 0, st>>>(t, m->h, W, c.taps, l.canon_a, l.ff > 0 ? l.canon_b : nullptr, run.tail, opA, ob, wp);
                GTB_LAUNCHED();
            }
            if (c.taps > 1) {
                k_canon_tail<<<dim3(S, (W + 255) / 256), 256, 0, st>>>(t, m->h, W, c.taps, run.tail);
                GTB_LAUNCHED();
            }
        } else {
            k_copy_operand<OT><<<R, 256, 0, st>>>(m->h, W, opA, ob, wp);
            GTB_LAUNCHED();
        }
        int rc = product<OT>(m, opA, wp, l.w_mix, wp, m->P, l.n1, R, l.n1, wp, nullptr, 0);
        if (rc) return rc;
        bool ff_done = false;
        if (l.ff > 0) {
            // tensor-core pass: gelu(gate) * up comes out of the product's epilogue as the out-projection operand
            if (sizeof(OT) == 2 && m->use_tensor && m->gp && R >= m->tensor_min_rows && l.gu_inter) {
                rc = seq_gemm_bf16_geglu(m->gp, opB, wp, l.w_gu, wp, opC, l.kout_p, l.kout - l.ff, R, 2 * l.ff, wp);
                if (rc > 0) return rc;
                if (rc == 0) { ctx().launches++; ff_done = true; }
            }
            if (!ff_done) {
                rc = product<OT>(m, opB, wp, l.w_gu, wp, m->G, 2 * l.ff, R, 2 * l.ff, wp, nullptr, 0);
                if (rc) return rc;
            }
        }
        for (int bi = 0; bi < l.d.n_branches; bi++) {
            const BranchW& b = l.br[bi];
            if (b.d.kind == GTB_MIX_SIGMOID_ATTN) {
                const AttnBranch a = attn_args(m, b);
                k_attn_prep<OT><<<dim3(R, (a.heads + 2 * a.kv_heads + 3) / 4), 128, 0, st>>>(t, a, m->P, l.n1, (OT*)run.kc[bi], (OT*)run.vc[bi]);
                GTB_LAUNCHED();
                int done = -1;
                if (portions && sizeof(OT) == 2 && a.dim <= 128 && a.vdim <= 128)
                    done = sigattn_mma(t, a, S, n_qtiles, m->P, l.n1, (const bf16*)run.kc[bi], (const bf16*)run.vc[bi], (bf16*)opC, l.kout_p);
                if (done > 0) return done;
                if (done < 0 && !portions && m->attn_splits > 1 && R <= SPLIT_MAX_ROWS) {
                    // (a group-major variant -- one CTA scoring a key for all query heads of its K/V head -- was measured slower at 32 heads
                    // and 8 splits: 8x fewer CTAs on a latency-bound step)
                    k_sigattn_split<OT><<<dim3(R, a.heads, m->attn_splits), 128, (a.dim + 128) * sizeof(float), st>>>(t, a, m->P, l.n1, (const OT*)run.kc[bi], (const OT*)run.vc[bi], m->attn_part, R);
                    GTB_LAUNCHED();
                    k_sigattn_join<OT><<<dim3(R, (a.heads * a.vdim + 255) / 256), 256, 0, st>>>(a, m->attn_part, R, m->attn_splits, opC, l.kout_p);
                    GTB_LAUNCHED();
                    done = 0;
                }
                if (done < 0) {
                    k_sigattn<OT><<<dim3(R, a.heads), 128, (a.dim + 128) * sizeof(float), st>>>(t, a, m->P, l.n1, (const OT*)run.kc[bi], (const OT*)run.vc[bi], opC, l.kout_p);
                    GTB_LAUNCHED();
                }
            } else {
                int rc2 = run_retention<OT>(m, t, R, S, run, bi, l, portions, seg_lens);
                if (rc2) return rc2;
            }
        }
        if (l.ff > 0 && !ff_done) {
            const size_t n = (size_t)R * l.ff;
            k_geglu<OT><<<(unsigned)((n + 255) / 256), 256, 0, st>>>(m->G, l.ff, opC, l.kout_p, l.kout - l.ff, R, l.gu_inter ? 1 : 0);
            GTB_LAUNCHED();
        }
        rc = product<OT>(m, opC, l.kout_p, l.w_out, l.kout_p, m->x, W, R, W, l.kout_p, nullptr, 1);
        if (rc) return rc;
        if (m->capture) {
            GTB_CUDA(cudaMemcpyAsync(m->cap + u * (size_t)m->max_rows * W, m->x, (size_t)R * W * sizeof(float), cudaMemcpyDeviceToDevice, st));
            m->cap_rows = R;
        }
    }
    if (n_want > 0) {
        if (c.final_norm == 3) {
            NormArgs fn{};
            fn.kind = GTB_NORM_LAYER; fn.w = m->final_gain; fn.b = m->final_b; fn.eps = c.eps;
            k_norm_rows<OT><<<n_want, 256, 0, st>>>(m->x, W, fn, d_want, opH, wp);
        } else if (c.final_norm == 2) {
            NormArgs fn{};
            fn.kind = GTB_NORM_DYT; fn.w = m->final_gain; fn.b = m->final_b; fn.alpha = m->final_a;
            k_dyt_rows<OT><<<n_want, 256, 0, st>>>(m->x, W, fn, d_want, opH, wp);
        } else if (c.final_norm) k_rmsnorm_weight<OT><<<n_want, 256, 0, st>>>(m->x, W, c.eps, m->final_gain, 1, d_want, opH, wp);
        else k_rmsnorm_scalar<OT><<<n_want, 256, 0, st>>>(m->x, W, c.eps, m->final_gain, d_want, opH, wp);
        GTB_LAUNCHED();
        int rc = product<OT>(m, opH, wp, m->head, wp, m->logits, c.vocab, n_want, c.vocab, wp, nullptr, 0);
        if (rc) return rc;
        if (c.logit_softcap > 0.0f) {
            const size_t n = (size_t)n_want * c.vocab;
            k_softcap<<<(unsigned)((n + 255) / 256), 256, 0, st>>>(m->logits, n, c.logit_softcap);
            GTB_LAUNCHED();
        }
    }
    k_commit<<<(S + 127) / 128, 128, 0, st>>>(t, S);
    GTB_LAUNCHED();
    return GTB_OK;
}

}  // namespace

// the table buffer of a pass: ints [seg_slot S | seg_row0 S | seg_len S | row_seg R | tok R | want R]
static PassTables tables(gtb_seq_model* m, int S, int R) {
    PassTables t{};
    int* b = m->d_tab;
    t.seg_slot = b; t.seg_row0 = b + S; t.seg_len = b + 2 * S; t.row_seg = b + 3 * S; t.tok = b + 3 * S + R;
    t.row_pos = m->d_row_pos; t.row_prev = m->d_row_prev; t.slots = m->d_slots;
    return t;
}

extern "C" {

int gtb_seq_create(gtb_seq_t* out, const gtb_seq_config* cfg, const gtb_seq_layer* layers) {
    GTB_CHECK_INIT();
    GTB_ARG(out && cfg && layers);
    GTB_ARG(cfg->vocab > 0 && cfg->width > 0 && cfg->n_layers > 0 && cfg->n_slots > 0 && cfg->max_ctx > 0);
    GTB_ARG(cfg->mode == GTB_SEQ_BF16 || cfg->mode == GTB_SEQ_F32);
    GTB_ARG(cfg->taps >= 0 && cfg->taps <= 64);
    if (cfg->loop_times > 0) GTB_ARG(cfg->loop_start >= 0 && cfg->loop_start < cfg->loop_stop && cfg->loop_stop <= cfg->n_layers);
    gtb_seq_model* m = new gtb_seq_model();
    m->cfg = *cfg;
    gtb_seq_config& c = m->cfg;
    if (c.max_rows <= 0) c.max_rows = 2048;
    m->max_rows = c.max_rows;
    const int W = c.width, wp = pad64(W);
    m->wp = wp;
    int rc = GTB_OK;
#define TRY(e) do { rc = (e); if (rc) { gtb_seq_destroy(m); return rc; } } while (0)
#define REQ(cond) do { if (!(cond)) { gtb_seq_destroy(m); return gtb::fail(GTB_ERR_ARG, "model description rejected: %s", #cond); } } while (0)
    TRY(dalloc_t(m, &m->embed, (size_t)c.vocab * W));
    want_matrix(m, "embed", m->embed, c.vocab, W, W);
    if (c.bigram_buckets > 0) {
        TRY(dalloc_t(m, &m->bigram, (size_t)(c.bigram_buckets + 1) * W));
        want_matrix(m, "bigram", m->bigram, c.bigram_buckets + 1, W, W);
    }
    TRY(dalloc_t(m, &m->head, (size_t)c.vocab * wp));
    want_matrix(m, "head", m->head, c.vocab, W, wp);
    REQ(c.final_norm >= 0 && c.final_norm <= 3);
    REQ(c.streams >= 0 && c.streams <= HC_MAX && c.logit_softcap >= 0.0f);
    TRY(dalloc_t(m, &m->final_gain, c.final_norm ? W : 1));
    if (c.final_norm) want_vector(m, "final.norm", m->final_gain, W, 0);
    else want_vector(m, "final.norm", m->final_gain, 0, 0, true);
    if (c.final_norm == 3) {
        TRY(dalloc_t(m, &m->final_b, W));
        want_vector(m, "final.norm.b", m->final_b, W, 0);
    }
    if (c.final_norm == 2) {
        TRY(dalloc_t(m, &m->final_b, W));
        TRY(dalloc_t(m, &m->final_a, 1));
        want_vector(m, "final.norm.b", m->final_b, W, 0);
        want_vector(m, "final.norm.alpha", m->final_a, 0, 0, true);
    }
    m->ns = c.streams > 0 ? c.streams : 1;
    m->prenorm = layers[0].style == GTB_BLOCK_PRENORM;
    m->sandwich = layers[0].style == GTB_BLOCK_SANDWICH;
    if (m->prenorm && c.streams == 0) {
        TRY(dalloc_t(m, &m->hc_one, 3));
        const float one[3] = {1.0f, 1.0f, 1.0f};
        GTB_CUDA(cudaMemcpyAsync(m->hc_one, one, sizeof one, cudaMemcpyHostToDevice, ctx().stream));
        GTB_CUDA(cudaStreamSynchronize(ctx().stream));
    }
    if (c.loop_times > 0) {
        TRY(dalloc_t(m, &m->loop_in, (size_t)W * pad64(2 * W)));
        want_matrix(m, "loop.in", m->loop_in, W, 2 * W, pad64(2 * W));
        TRY(dalloc_t(m, &m->loop_step, (size_t)c.loop_times * W));
        want_vector(m, "loop.step", m->loop_step, c.loop_times, W);
    }
    m->L.resize(c.n_layers);
    for (int i = 0; i < c.n_layers; i++) {
        LayerW& l = m->L[i];
        l.d = layers[i];
        const bool post = l.d.style == GTB_BLOCK_POSTNORM, pre = l.d.style == GTB_BLOCK_PRENORM, sw = l.d.style == GTB_BLOCK_SANDWICH;
        REQ(l.d.style == GTB_BLOCK_PARALLEL || post || pre || sw);
        REQ(pre == m->prenorm);                  // the copies of the stream belong to the whole model: pre-norm layers do not mix with the other styles
        REQ(sw == m->sandwich);                  // a sandwich layer hands its successor a normalised operand
        REQ(!(pre || sw) || (c.loop_times == 0 && c.taps == 0));
        REQ(l.d.n_branches >= 1 && l.d.n_branches <= (post || pre ? 1 : 2));
        REQ(l.d.ff >= 0);
        if (sw) REQ((l.d.norm_kind == GTB_NORM_RMS || l.d.norm_kind == GTB_NORM_LAYER) && (l.d.ff == 0 || l.d.ff_kind == GTB_FF_SWIGLU || l.d.ff_kind == GTB_FF_GROUP_EXPERTS));
        else if (pre) REQ((l.d.norm_kind == GTB_NORM_RMS || l.d.norm_kind == GTB_NORM_DYT) && (l.d.ff == 0 || l.d.ff_kind == GTB_FF_GEGLU || l.d.ff_kind == GTB_FF_GATED_EXPERTS));
        else REQ(post ? (l.d.ff == 0 || l.d.ff_kind == GTB_FF_POLYNORM || l.d.ff_kind == GTB_FF_EXPERTS) : l.d.ff_kind == GTB_FF_GEGLU);
        l.ff = l.d.ff;
        const std::string lp = "l" + std::to_string(i) + ".";
        int n1 = 0, ko = 0;
        for (int bi = 0; bi < l.d.n_branches; bi++) {
            BranchW& b = l.br[bi];
            b.d = l.d.branch[bi];
            gtb_seq_branch& d = b.d;
            REQ(pre ? d.kind == GTB_MIX_LATENT_ATTN : post ? (d.kind == GTB_MIX_MINGRU || d.kind == GTB_MIX_SOFTMAX_ATTN) :
                sw ? (d.kind == GTB_MIX_SOFTMAX_ATTN || d.kind == GTB_MIX_RETENTION) : (d.kind == GTB_MIX_SIGMOID_ATTN || d.kind == GTB_MIX_RETENTION));
            if (d.kind == GTB_MIX_LATENT_ATTN) {
                REQ(d.heads > 0 && d.dim > 0 && d.rope_dim >= 0 && d.vdim > 0 && d.kv_rank > 0 && d.q_rank >= 0 && d.window >= 0);
                REQ(d.kv_rank <= 512 && d.kv_rank + d.rope_dim <= 1024);        // the absorbed form runs on the row kernels of softmax attention
                REQ(d.rot_dims >= 0 && d.rot_dims <= d.rope_dim && d.rot_dims % 2 == 0 && (d.gated == 0 || d.gated == 3));
                d.kv_heads = 1; d.kv_from = -1; d.pool = 0;
                const int hd = d.dim + d.rope_dim, nq = d.q_rank > 0 ? d.q_rank : d.heads * hd;
                b.q_off = n1; b.kv_off = n1 + nq; b.g_off = b.kv_off + d.kv_rank + d.rope_dim;
                n1 = b.g_off + (d.gated ? d.heads : 0);
                b.a_off = ko; ko += d.heads * d.vdim;
                b.rank_p = pad64(d.kv_rank); b.qrank_p = d.q_rank > 0 ? pad64(d.q_rank) : 0;
                b.c_ld = std::max((d.kv_rank + d.rope_dim + 7) / 8 * 8, b.rank_p);
                if (d.rot_dims > 0) {
                    b.inv_freq.resize(d.rot_dims / 2);
                    for (int k = 0; k < d.rot_dims / 2; k++) b.inv_freq[k] = (float)pow((double)d.rot_base, -2.0 * k / d.rot_dims);
                    TRY(dalloc_t(m, &b.d_inv_freq, b.inv_freq.size()));
                    GTB_CUDA(cudaMemcpyAsync(b.d_inv_freq, b.inv_freq.data(), b.inv_freq.size() * sizeof(float), cudaMemcpyHostToDevice, ctx().stream));
                }
                m->lat_q_max = std::max(m->lat_q_max, d.heads * hd + d.heads);
                if (hd <= 128 && d.vdim <= 128) {
                    m->lat_kx_max = std::max(m->lat_kx_max, d.heads * hd);
                    m->lat_vx_max = std::max(m->lat_vx_max, d.heads * d.vdim);
                    m->lat_x_max = std::max(m->lat_x_max, d.heads * (d.dim + d.vdim));
                }
                m->lat_qa_max = std::max(m->lat_qa_max, d.heads * (d.kv_rank + d.rope_dim));
                m->lat_qr_max = std::max(m->lat_qr_max, b.qrank_p);
                m->lat_ol_max = std::max(m->lat_ol_max, (d.heads * d.kv_rank + 7) / 8 * 8);
                continue;
            }
            if (d.kind == GTB_MIX_MINGRU) {
                REQ(d.dim > 0);
                d.heads = d.kv_heads = 1; d.vdim = d.dim; d.rot_dims = 0;
                b.q_off = n1; b.k_off = n1 + d.dim; b.g_off = n1 + 2 * d.dim; n1 += 3 * d.dim;      // update gate | candidate | output gate
                b.a_off = ko; ko += d.dim;
                continue;
            }
            REQ(d.heads > 0 && d.dim > 0 && d.vdim > 0 && d.dim <= 1024 && d.vdim <= 512);
            if (d.kind == GTB_MIX_RETENTION) d.kv_heads = d.heads;
            REQ(d.kv_heads > 0 && d.heads % d.kv_heads == 0);
            REQ(d.rot_dims >= 0 && d.rot_dims <= d.dim && d.rot_dims % 2 == 0);
            if (d.kind != GTB_MIX_SOFTMAX_ATTN || !sw) { REQ(d.maps <= 1 && d.chunk == 0 && d.bias == 0 && d.rot_divide == 0.0f && d.qk_norm <= 2); d.maps = 1; }
            if (d.kind != GTB_MIX_RETENTION || !sw) REQ(d.act == 0 && d.out_norm <= 1);
            if (d.maps < 1) d.maps = 1;
            b.kq = d.heads * d.maps * d.dim; b.kk = d.kv_heads * d.maps * d.dim; b.kv = d.kv_heads * d.vdim;
            if (d.kind == GTB_MIX_SOFTMAX_ATTN) {
                REQ(d.qk_norm >= 0 && d.qk_norm <= 3 && d.gated >= 0 && d.gated <= 3 && d.window >= 0 && d.pool >= 0 && d.softcap >= 0.0f);
                REQ(d.maps <= 2 && d.chunk >= 0 && d.rot_divide >= 0.0f && (d.gated != 3 || sw));
                if (d.maps == 2) REQ(d.pool == 0 && d.sink == 0 && (d.gated == 0 || d.gated == 3));
                if (!sw) d.out_scale = 1.0f;
                REQ(d.kv_from < i);
                if (d.kv_from >= 0) {
                    REQ(c.loop_times == 0);
                    const LayerW& src = m->L[d.kv_from];
                    REQ(src.d.style == l.d.style && src.d.n_branches == 1 && src.br[0].d.kind == GTB_MIX_SOFTMAX_ATTN && src.br[0].d.kv_from < 0);
                    REQ(src.br[0].d.kv_heads == d.kv_heads && src.br[0].d.dim == d.dim && src.br[0].d.vdim == d.vdim && src.br[0].d.maps == d.maps);
                    REQ(l.d.n_branches == 1);
                } else d.kv_from = -1;
                b.q_off = n1; n1 += b.kq;
                if (d.kv_from < 0) { b.k_off = n1; n1 += b.kk; b.v_off = n1; n1 += b.kv; }
                if (d.gated) { b.g_off = n1; n1 += d.gated == 3 ? d.heads : d.heads * d.vdim; }
                b.a_off = ko; ko += d.heads * d.vdim;
                if (d.maps == 2) m->ro_max = std::max(m->ro_max, 2 * d.heads * d.vdim);
                if (d.rot_dims > 0) {
                    // frequencies in double, rounded once: base^(-2k/dims); long wavelengths slowed down by rot_factor, a linear blend between
                    b.inv_freq.resize(d.rot_dims / 2);
                    for (int k = 0; k < d.rot_dims / 2; k++) {
                        double f = pow((double)d.rot_base, -2.0 * k / d.rot_dims);
                        if (d.rot_factor > 0.0f) {
                            const double wl = 2.0 * M_PI / f, orig = d.rot_original, lo = d.rot_low, hi = d.rot_high, fac = d.rot_factor;
                            if (wl > orig / lo) f = f / fac;
                            else if (!(wl < orig / hi)) { const double sm = (orig / wl - lo) / (hi - lo); f = (1.0 - sm) * f / fac + sm * f; }
                        }
                        if (d.rot_divide > 0.0f) f /= (double)d.rot_divide;
                        b.inv_freq[k] = (float)f;
                    }
                    TRY(dalloc_t(m, &b.d_inv_freq, b.inv_freq.size()));
                    GTB_CUDA(cudaMemcpyAsync(b.d_inv_freq, b.inv_freq.data(), b.inv_freq.size() * sizeof(float), cudaMemcpyHostToDevice, ctx().stream));
                }
                continue;
            }
            b.q_off = n1; b.k_off = n1 + b.kq; b.v_off = b.k_off + b.kk; n1 = b.v_off + b.kv;
            if (d.kind == GTB_MIX_RETENTION) REQ(d.gated >= 0 && d.gated <= (sw ? 2 : 1) && d.out_norm >= 0);
            if (d.kind == GTB_MIX_RETENTION && d.gated) { b.g_off = n1; n1 += d.heads * d.vdim; }
            b.a_off = ko; ko += d.heads * d.vdim;
            if (d.kind == GTB_MIX_RETENTION) {
                REQ(d.decay != nullptr);
                REQ(ret_launch(d).smem <= 200 * 1024);
                b.decay.assign(d.decay, d.decay + d.heads);
                d.decay = nullptr;
                TRY(dalloc_t(m, &b.d_decay, d.heads));
                GTB_CUDA(cudaMemcpyAsync(b.d_decay, b.decay.data(), d.heads * sizeof(float), cudaMemcpyHostToDevice, ctx().stream));
                if (d.rot_dims > 0) {
                    // (same stream as the allocation's zero fill: a copy on another stream could be overtaken by it)
                    b.inv_freq.resize(d.rot_dims / 2);
                    for (int k = 0; k < d.rot_dims / 2; k++) b.inv_freq[k] = (float)pow((double)d.rot_base, -2.0 * k / d.rot_dims);
                    TRY(dalloc_t(m, &b.d_inv_freq, b.inv_freq.size()));
                    GTB_CUDA(cudaMemcpyAsync(b.d_inv_freq, b.inv_freq.data(), b.inv_freq.size() * sizeof(float), cudaMemcpyHostToDevice, ctx().stream));
                }
            }
        }
        GTB_CUDA(cudaStreamSynchronize(ctx().stream));       // the vectors above are read from members that may move; wait for the copies
        l.n1 = n1;
        l.kout = (post || pre || sw) ? ko : ko + l.ff;
        l.kout_p = pad64(l.kout);
        TRY(dalloc_t(m, &l.w_mix, (size_t)n1 * wp));
        TRY(dalloc_t(m, &l.w_out, (size_t)W * l.kout_p));
        for (int bi = 0; bi < l.d.n_branches; bi++) {
            BranchW& b = l.br[bi];
            const gtb_seq_branch& d = b.d;
            const std::string bp = lp + "mix." + (d.name[0] ? std::string(d.name) + "." : std::string());
            if (d.kind == GTB_MIX_MINGRU) {
                TRY(dalloc_t(m, &l.d_bias, n1));
                want_matrix(m, bp + "z", l.w_mix + (size_t)b.q_off * wp, d.dim, W, wp);
                want_matrix(m, bp + "x", l.w_mix + (size_t)b.k_off * wp, d.dim, W, wp);
                want_matrix(m, bp + "g", l.w_mix + (size_t)b.g_off * wp, d.dim, W, wp);
                want_vector(m, bp + "z.b", l.d_bias + b.q_off, d.dim, 0);
                want_vector(m, bp + "x.b", l.d_bias + b.k_off, d.dim, 0);
                want_matrix(m, bp + "o", l.w_out + b.a_off, W, d.dim, l.kout_p);
                continue;
            }
            if (d.kind == GTB_MIX_LATENT_ATTN) {
                const int hd = d.dim + d.rope_dim;
                if (d.q_rank > 0) {
                    want_matrix(m, bp + "dq", l.w_mix + (size_t)b.q_off * wp, d.q_rank, W, wp);
                    TRY(dalloc_t(m, &b.d_qnorm, d.q_rank));
                    want_vector(m, bp + "dq.norm", b.d_qnorm, d.q_rank, 0);
                    TRY(dalloc_t(m, &b.w_uq, (size_t)d.heads * hd * b.qrank_p));
                    want_matrix(m, bp + "uq", b.w_uq, d.heads * hd, d.q_rank, b.qrank_p);
                } else {
                    want_matrix(m, bp + "q", l.w_mix + (size_t)b.q_off * wp, d.heads * hd, W, wp);
                }
                want_matrix(m, bp + "dkv", l.w_mix + (size_t)b.kv_off * wp, d.kv_rank + d.rope_dim, W, wp);
                TRY(dalloc_t(m, &b.d_kvnorm, d.kv_rank));
                want_vector(m, bp + "dkv.norm", b.d_kvnorm, d.kv_rank, 0);
                TRY(dalloc_t(m, &b.w_uk, (size_t)d.heads * (d.dim + d.vdim) * b.rank_p));      // uv follows uk: one product expands keys and values
                b.w_uv = b.w_uk + (size_t)d.heads * d.dim * b.rank_p;
                want_matrix(m, bp + "uk", b.w_uk, d.heads * d.dim, d.kv_rank, b.rank_p);
                want_matrix(m, bp + "uv", b.w_uv, d.heads * d.vdim, d.kv_rank, b.rank_p);
                if (d.sink) { TRY(dalloc_t(m, &b.d_sink, d.heads)); want_vector(m, bp + "sink", b.d_sink, d.heads, 0); }
                if (d.gated) want_matrix(m, bp + "g", l.w_mix + (size_t)b.g_off * wp, d.heads, W, wp);
                want_matrix(m, bp + "o", l.w_out + b.a_off, W, d.heads * d.vdim, l.kout_p);
                continue;
            }
            want_matrix(m, bp + "q", l.w_mix + (size_t)b.q_off * wp, b.kq, W, wp);
            const bool own_kv = !(d.kind == GTB_MIX_SOFTMAX_ATTN && d.kv_from >= 0);
            if (own_kv) {
                want_matrix(m, bp + "k", l.w_mix + (size_t)b.k_off * wp, b.kk, W, wp);
                want_matrix(m, bp + "v", l.w_mix + (size_t)b.v_off * wp, b.kv, W, wp);
            }
            if (d.bias) {                           // bias vectors of the fused projection; columns without one stay zero
                if (!l.d_bias) TRY(dalloc_t(m, &l.d_bias, n1));
                want_vector(m, bp + "q.b", l.d_bias + b.q_off, b.kq, 0);
                if (own_kv) { want_vector(m, bp + "k.b", l.d_bias + b.k_off, b.kk, 0); want_vector(m, bp + "v.b", l.d_bias + b.v_off, b.kv, 0); }
            }
            if ((d.kind == GTB_MIX_RETENTION || d.kind == GTB_MIX_SOFTMAX_ATTN) && d.gated)
                want_matrix(m, bp + "g", l.w_mix + (size_t)b.g_off * wp, (d.kind == GTB_MIX_SOFTMAX_ATTN && d.gated == 3) ? d.heads : d.heads * d.vdim, W, wp);
            if (d.kind == GTB_MIX_RETENTION && d.out_norm == 2) { TRY(dalloc_t(m, &b.d_onorm, d.heads * d.vdim)); want_vector(m, bp + "norm", b.d_onorm, d.heads * d.vdim, 0); }
            want_matrix(m, bp + "o", l.w_out + b.a_off, W, d.heads * d.vdim, l.kout_p);
            if (d.kind == GTB_MIX_SIGMOID_ATTN) {
                TRY(dalloc_t(m, &b.d_pb, d.heads));
                want_vector(m, bp + "pb", b.d_pb, d.heads, 0);
            }
            if (d.kind == GTB_MIX_SOFTMAX_ATTN) {
                if (d.qk_norm == 2) {
                    TRY(dalloc_t(m, &b.d_qnorm, d.dim));
                    want_vector(m, bp + "q.norm", b.d_qnorm, d.dim, 0);
                    if (own_kv) { TRY(dalloc_t(m, &b.d_knorm, d.dim)); want_vector(m, bp + "k.norm", b.d_knorm, d.dim, 0); }
                }
                if (d.qk_norm == 3) {               // one weight per entry of the whole projection
                    TRY(dalloc_t(m, &b.d_qnorm, b.kq));
                    want_vector(m, bp + "q.norm", b.d_qnorm, b.kq, 0);
                    if (own_kv) { TRY(dalloc_t(m, &b.d_knorm, b.kk)); want_vector(m, bp + "k.norm", b.d_knorm, b.kk, 0); }
                    if (!m->qk_sc) TRY(dalloc_t(m, &m->qk_sc, (size_t)m->max_rows * 2));
                }
                if (d.maps == 2) {
                    const char* nm[4] = {"lq1", "lk1", "lq2", "lk2"};
                    for (int q = 0; q < 4; q++) { TRY(dalloc_t(m, &b.d_lam[q], d.dim)); want_vector(m, bp + nm[q], b.d_lam[q], d.dim, 0); }
                }
                if (d.sink) { TRY(dalloc_t(m, &b.d_sink, d.heads)); want_vector(m, bp + "sink", b.d_sink, d.heads, 0); }
            }
        }
        if (sw) {
            const char* nn[4] = {"norm1", "norm1b", "norm2", "norm2b"};
            for (int q = 0; q < (l.ff > 0 ? 4 : 2); q++) {
                TRY(dalloc_t(m, &l.sn_w[q], W));
                want_vector(m, lp + nn[q], l.sn_w[q], W, 0);
                if (l.d.norm_kind == GTB_NORM_LAYER) { TRY(dalloc_t(m, &l.sn_b[q], W)); want_vector(m, lp + nn[q] + ".b", l.sn_b[q], W, 0); }
            }
            if (l.ff > 0) {
                l.kfp = pad64(l.ff);
                m->kfp_max = std::max(m->kfp_max, l.kfp);
                if (l.d.ff_kind == GTB_FF_SWIGLU) {
                    TRY(dalloc_t(m, &l.w_gu, (size_t)2 * l.ff * wp));
                    TRY(dalloc_t(m, &l.w_down, (size_t)W * l.kfp));
                    l.gu_inter = l.ff % 32 == 0;
                    want_matrix(m, lp + "mlp.gate", l.w_gu, l.ff, W, wp);
                    want_matrix(m, lp + "mlp.up", l.w_gu + (size_t)(l.gu_inter ? 32 : l.ff) * wp, l.ff, W, wp);
                    if (l.gu_inter)
                        for (const char* nm : {"mlp.gate", "mlp.up"}) { TensorDest& d = m->tensors[lp + nm]; d.group = 32; d.group_stride = 64; }
                    want_matrix(m, lp + "mlp.down", l.w_down, W, l.ff, l.kfp);
                    m->g_cols = std::max(m->g_cols, 2 * l.ff);
                    m->kout_p_max = std::max(m->kout_p_max, l.kfp);
                } else {
                    const int E = l.d.experts, G = std::max(1, l.d.route_groups), keep = l.d.route_keep > 0 ? l.d.route_keep : G;
                    REQ(E > 0 && E <= 4096 && l.d.identity == 0 && l.d.top > 0 && l.d.shared_ff >= 0 && E % G == 0 && keep <= G && l.d.top <= keep * (E / G));
                    l.sff = l.d.shared_ff;
                    l.n_sh = (l.sff + l.ff - 1) / l.ff;              // the shared expert in parts of one expert's inner width
                    l.e_total = E + l.n_sh;
                    REQ(l.d.top + l.n_sh <= 64);
                    l.n_out = E;
                    TRY(dalloc_t(m, &l.w_router, (size_t)E * wp));
                    want_matrix(m, lp + "mlp.router", l.w_router, E, W, wp);
                    TRY(dalloc_t(m, &l.w_up, (size_t)l.e_total * l.ff * wp));
                    TRY(dalloc_t(m, &l.w_down, (size_t)l.e_total * W * l.kfp));
                    for (int e = 0; e < E; e++) {
                        const std::string ep = lp + "mlp.e" + std::to_string(e) + ".";
                        want_matrix(m, ep + "up", l.w_up + (size_t)e * l.ff * wp, l.ff, W, wp);
                        want_matrix(m, ep + "down", l.w_down + (size_t)e * W * l.kfp, W, l.ff, l.kfp);
                    }
                    if (l.sff > 0) {
                        // rows of shared.up continue the stack (the last part's missing rows stay zero); columns of shared.down go part by part
                        want_matrix(m, lp + "mlp.shared.up", l.w_up + (size_t)E * l.ff * wp, l.sff, W, wp);
                        want_matrix(m, lp + "mlp.shared.down", l.w_down + (size_t)E * W * l.kfp, W, l.sff, l.kfp);
                        TensorDest& d = m->tensors[lp + "mlp.shared.down"];
                        d.split_cols = l.ff; d.split_stride = (size_t)W * l.kfp;
                    }
                    m->n_out_max = std::max(m->n_out_max, E);
                    m->top_max = std::max(m->top_max, l.d.top + l.n_sh);
                    m->e_max = std::max(m->e_max, l.e_total);
                }
            }
        } else if (pre) {
            const int ns = m->ns;
            for (int q = 0; q < (l.ff > 0 ? 2 : 1); q++) {
                const std::string np = lp + (q == 0 ? "norm1" : "norm2"), hp = lp + (q == 0 ? "hc1." : "hc2.");
                float*& nw = q == 0 ? l.norm1 : l.norm2;
                TRY(dalloc_t(m, &nw, W));
                want_vector(m, np, nw, W, 0);
                if (l.d.norm_kind == GTB_NORM_DYT) {
                    TRY(dalloc_t(m, &l.nb[q], W));
                    TRY(dalloc_t(m, &l.na[q], 1));
                    want_vector(m, np + ".b", l.nb[q], W, 0);
                    want_vector(m, np + ".alpha", l.na[q], 0, 0, true);
                }
                if (c.streams > 0) {
                    TRY(dalloc_t(m, &l.hc[q], (size_t)ns * (2 + ns)));
                    want_vector(m, hp + "in", l.hc[q], ns, 0);
                    want_vector(m, hp + "out", l.hc[q] + ns, ns, 0);
                    want_vector(m, hp + "mix", l.hc[q] + 2 * ns, ns, ns);
                } else l.hc[q] = m->hc_one;
            }
            if (l.ff > 0) {
                l.kfp = pad64(l.ff);
                m->kfp_max = std::max(m->kfp_max, l.kfp);
                if (l.d.ff_kind == GTB_FF_GEGLU) {
                    TRY(dalloc_t(m, &l.w_gu, (size_t)2 * l.ff * wp));
                    TRY(dalloc_t(m, &l.w_down, (size_t)W * l.kfp));
                    l.gu_inter = l.ff % 32 == 0;
                    want_matrix(m, lp + "mlp.gate", l.w_gu, l.ff, W, wp);
                    want_matrix(m, lp + "mlp.up", l.w_gu + (size_t)(l.gu_inter ? 32 : l.ff) * wp, l.ff, W, wp);
                    if (l.gu_inter)
                        for (const char* nm : {"mlp.gate", "mlp.up"}) { TensorDest& d = m->tensors[lp + nm]; d.group = 32; d.group_stride = 64; }
                    want_matrix(m, lp + "mlp.down", l.w_down, W, l.ff, l.kfp);
                    m->g_cols = std::max(m->g_cols, 2 * l.ff);
                    m->kout_p_max = std::max(m->kout_p_max, l.kfp);
                } else {
                    const int E = l.d.experts;
                    REQ(E > 0 && E <= 4096 && l.d.identity == 0 && l.d.top > 0 && l.d.top <= E && l.d.top <= 64 && l.d.shared_ff >= 0);
                    l.sff = l.d.shared_ff;
                    l.n_out = E + (l.sff > 0 ? 1 : 0);
                    TRY(dalloc_t(m, &l.w_router, (size_t)l.n_out * wp));
                    want_matrix(m, lp + "mlp.router", l.w_router, E, W, wp);
                    if (l.sff > 0) want_matrix(m, lp + "mlp.shared.sg", l.w_router + (size_t)E * wp, 1, W, wp);
                    TRY(dalloc_t(m, &l.w_up, (size_t)E * 2 * l.ff * wp));
                    TRY(dalloc_t(m, &l.w_down, (size_t)E * W * l.kfp));
                    l.e_inter = l.ff % 32 == 0;
                    for (int e = 0; e < E; e++) {
                        const std::string ep = lp + "mlp.e" + std::to_string(e) + ".";
                        bf16* base = l.w_up + (size_t)e * 2 * l.ff * wp;
                        want_matrix(m, ep + "gate", base, l.ff, W, wp);
                        want_matrix(m, ep + "up", base + (size_t)(l.e_inter ? 32 : l.ff) * wp, l.ff, W, wp);
                        if (l.e_inter)
                            for (const char* nm : {"gate", "up"}) { TensorDest& d = m->tensors[ep + nm]; d.group = 32; d.group_stride = 64; }
                        want_matrix(m, ep + "down", l.w_down + (size_t)e * W * l.kfp, W, l.ff, l.kfp);
                    }
                    m->n_out_max = std::max(m->n_out_max, l.n_out);
                    m->top_max = std::max(m->top_max, l.d.top);
                    m->e_max = std::max(m->e_max, E);
                    if (l.sff > 0) {
                        l.sff_p = pad64(l.sff);
                        l.sh_inter = l.sff % 32 == 0;
                        TRY(dalloc_t(m, &l.w_sh_gu, (size_t)2 * l.sff * wp));
                        TRY(dalloc_t(m, &l.w_sh_down, (size_t)W * l.sff_p));
                        want_matrix(m, lp + "mlp.shared.gate", l.w_sh_gu, l.sff, W, wp);
                        want_matrix(m, lp + "mlp.shared.up", l.w_sh_gu + (size_t)(l.sh_inter ? 32 : l.sff) * wp, l.sff, W, wp);
                        if (l.sh_inter)
                            for (const char* nm : {"mlp.shared.gate", "mlp.shared.up"}) { TensorDest& d = m->tensors[lp + nm]; d.group = 32; d.group_stride = 64; }
                        want_matrix(m, lp + "mlp.shared.down", l.w_sh_down, W, l.sff, l.sff_p);
                        m->g_cols = std::max(m->g_cols, 2 * l.sff);
                        m->kout_p_max = std::max(m->kout_p_max, l.sff_p);
                    }
                }
            }
        } else if (post) {
            TRY(dalloc_t(m, &l.norm1, W));
            want_vector(m, lp + "norm1", l.norm1, W, 0);
            if (l.ff > 0) {
                TRY(dalloc_t(m, &l.norm2, W));
                want_vector(m, lp + "norm2", l.norm2, W, 0);
                l.kfp = pad64(l.ff);
                m->kfp_max = std::max(m->kfp_max, l.kfp);
                if (l.d.ff_kind == GTB_FF_POLYNORM) {
                    TRY(dalloc_t(m, &l.w_up, (size_t)l.ff * wp));
                    TRY(dalloc_t(m, &l.w_down, (size_t)W * l.kfp));
                    TRY(dalloc_t(m, &l.d_act, 4));
                    want_matrix(m, lp + "mlp.up", l.w_up, l.ff, W, wp);
                    want_matrix(m, lp + "mlp.down", l.w_down, W, l.ff, l.kfp);
                    want_vector(m, lp + "mlp.act", l.d_act, 4, 0);
                    m->g_cols = std::max(m->g_cols, l.ff);
                    m->kout_p_max = std::max(m->kout_p_max, l.kfp);
                } else {
                    const int E = l.d.experts, I = l.d.identity;
                    REQ(E >= 0 && I >= 0 && E + I > 0 && E + I <= 4096 && l.d.top > 0 && l.d.top <= E + I && l.d.top <= 64);
                    l.n_out = E + I;
                    TRY(dalloc_t(m, &l.w_router, (size_t)l.n_out * wp));
                    TRY(dalloc_t(m, &l.d_corr, l.n_out));
                    want_matrix(m, lp + "mlp.router", l.w_router, l.n_out, W, wp);
                    want_vector(m, lp + "mlp.correction", l.d_corr, l.n_out, 0);
                    TRY(dalloc_t(m, &l.w_up, (size_t)std::max(E, 1) * l.ff * wp));
                    TRY(dalloc_t(m, &l.w_down, (size_t)std::max(E, 1) * W * l.kfp));
                    for (int e = 0; e < E; e++) {
                        const std::string ep = lp + "mlp.e" + std::to_string(e) + ".";
                        want_matrix(m, ep + "up", l.w_up + (size_t)e * l.ff * wp, l.ff, W, wp);
                        want_matrix(m, ep + "down", l.w_down + (size_t)e * W * l.kfp, W, l.ff, l.kfp);
                    }
                    m->n_out_max = std::max(m->n_out_max, l.n_out);
                    m->top_max = std::max(m->top_max, l.d.top);
                    m->e_max = std::max(m->e_max, E);
                }
            }
        } else {
            if (l.ff > 0) {
                TRY(dalloc_t(m, &l.w_gu, (size_t)2 * l.ff * wp));
                l.gu_inter = l.ff % 32 == 0;
                want_matrix(m, lp + "mlp.gate", l.w_gu, l.ff, W, wp);
                want_matrix(m, lp + "mlp.up", l.w_gu + (size_t)(l.gu_inter ? 32 : l.ff) * wp, l.ff, W, wp);
                if (l.gu_inter)
                    for (const char* nm : {"mlp.gate", "mlp.up"}) { TensorDest& d = m->tensors[lp + nm]; d.group = 32; d.group_stride = 64; }
                want_matrix(m, lp + "mlp.down", l.w_out + ko, W, l.ff, l.kout_p);
                m->ff_max = std::max(m->ff_max, l.ff);
            }
            TRY(dalloc_t(m, &l.d_gain, 1));
            want_vector(m, lp + "norm1", l.d_gain, 0, 0, true);
            if (c.taps > 0) {
                TRY(dalloc_t(m, &l.canon_a, (size_t)W * c.taps));
                want_matrix(m, lp + "canon1", l.canon_a, W, c.taps, c.taps);
                if (l.ff > 0) {
                    TRY(dalloc_t(m, &l.canon_b, (size_t)W * c.taps));
                    want_matrix(m, lp + "canon2", l.canon_b, W, c.taps, c.taps);
                }
            }
        }
        m->n1_max = std::max(m->n1_max, n1);
        m->kout_p_max = std::max(m->kout_p_max, l.kout_p);
        for (int bi = 0; bi < l.d.n_branches; bi++)
            if (l.br[bi].d.kind == GTB_MIX_RETENTION) m->ro_max = std::max(m->ro_max, l.br[bi].d.heads * l.br[bi].d.vdim);
    }
    // the order of layer runs
    auto add_run = [&](int layer, int pass, bool enters) { Run r; r.layer = layer; r.pass = pass; r.enters_pass = enters; m->runs.push_back(r); };
    if (c.loop_times > 0) {
        for (int i = 0; i < c.loop_start; i++) add_run(i, -1, false);
        for (int p = 0; p < c.loop_times; p++)
            for (int i = c.loop_start; i < c.loop_stop; i++) add_run(i, p, i == c.loop_start);
        for (int i = c.loop_stop; i < c.n_layers; i++) add_run(i, -1, false);
    } else {
        for (int i = 0; i < c.n_layers; i++) add_run(i, -1, false);
    }
    for (const Run& r : m->runs) REQ(!(r.enters_pass && m->L[r.layer].d.style == GTB_BLOCK_POSTNORM));      // a loop pass opens with a parallel block
    // state of every run, for every slot
    const size_t es = osz(m);
    for (Run& r : m->runs) {
        const LayerW& l = m->L[r.layer];
        size_t per_slot = 0;
        for (int bi = 0; bi < l.d.n_branches; bi++) {
            const gtb_seq_branch& d = l.br[bi].d;
            if (d.kind == GTB_MIX_LATENT_ATTN) {
                const size_t cb = (size_t)c.max_ctx * l.br[bi].c_ld * es;
                TRY(dalloc(m, &r.kc[bi], cb * c.n_slots));
                per_slot += cb;
            } else if (d.kind == GTB_MIX_SIGMOID_ATTN || d.kind == GTB_MIX_SOFTMAX_ATTN) {
                if (d.kind == GTB_MIX_SOFTMAX_ATTN && d.kv_from >= 0) {
                    // no loop (checked above), so run j is layer j: the source layer's cache, appended to earlier in the same pass
                    r.kc[bi] = m->runs[d.kv_from].kc[0];
                    r.vc[bi] = m->runs[d.kv_from].vc[0];
                } else {
                    const size_t kb = (size_t)c.max_ctx * d.kv_heads * std::max(1, d.maps) * d.dim * es, vb = (size_t)c.max_ctx * d.kv_heads * d.vdim * es;
                    TRY(dalloc(m, &r.kc[bi], kb * c.n_slots));
                    TRY(dalloc(m, &r.vc[bi], vb * c.n_slots));
                    per_slot += kb + vb;
                }
                if (d.kind == GTB_MIX_SOFTMAX_ATTN && d.window > 0 && d.pool > 0) {      // pooled blocks follow this layer's own block size
                    r.max_blocks = c.max_ctx / d.pool + 1;
                    const size_t kb = (size_t)r.max_blocks * d.kv_heads * d.dim * sizeof(float), vb = (size_t)r.max_blocks * d.kv_heads * d.vdim * sizeof(float);
                    TRY(dalloc(m, (void**)&r.pk, kb * c.n_slots));
                    TRY(dalloc(m, (void**)&r.pv, vb * c.n_slots));
                    per_slot += kb + vb;
                }
            } else {
                const size_t sb = state_floats(d) * sizeof(float);
                TRY(dalloc(m, (void**)&r.state[bi], sb * c.n_slots));
                per_slot += sb;
            }
        }
        if (c.taps > 1) {
            TRY(dalloc_t(m, &r.tail, (size_t)c.n_slots * (c.taps - 1) * W));
            per_slot += (size_t)(c.taps - 1) * W * sizeof(float);
        }
        m->state_bytes += per_slot;
    }
    // workspace
    const size_t R = m->max_rows;
    TRY(dalloc_t(m, &m->x, R * W));
    TRY(dalloc_t(m, &m->x0, R * W));
    TRY(dalloc_t(m, &m->h, R * W));
    TRY(dalloc_t(m, &m->Y, R * W));
    TRY(dalloc_t(m, &m->P, R * m->n1_max));
    TRY(dalloc_t(m, &m->G, R * std::max(std::max(2 * m->ff_max, m->g_cols), 1)));
    TRY(dalloc_t(m, &m->O, R * std::max(m->ro_max, 1)));
    for (const LayerW& l : m->L)
        for (int bi = 0; bi < l.d.n_branches; bi++)
            if (l.br[bi].d.kind == GTB_MIX_RETENTION && ret_chunk(l.br[bi].d).ok) {
                const gtb_seq_branch& d = l.br[bi].d;
                const size_t chunks = R / ret_chunk(d).C + c.n_slots + 1;
                m->retU_floats = std::max(m->retU_floats, chunks * d.heads * d.dim * d.vdim);
            }
    if (m->retU_floats) TRY(dalloc_t(m, &m->retU, m->retU_floats));
    for (const LayerW& l : m->L)
        if (l.br[0].d.kind == GTB_MIX_MINGRU) m->gruAB_floats = std::max(m->gruAB_floats, (R / GRU_CHUNK + c.n_slots + 1) * 2 * (size_t)l.br[0].d.dim);
    if (m->gruAB_floats) TRY(dalloc_t(m, &m->gruAB, m->gruAB_floats));
    {
        size_t hv = 0;
        for (const LayerW& l : m->L)
            if (l.br[0].d.kind == GTB_MIX_SOFTMAX_ATTN) hv = std::max(hv, (size_t)l.br[0].d.heads * std::max(1, l.br[0].d.maps) * (l.br[0].d.vdim + 2));
            else if (l.br[0].d.kind == GTB_MIX_LATENT_ATTN) hv = std::max(hv, (size_t)l.br[0].d.heads * (l.br[0].d.kv_rank + 2));
        if (hv > 0 && c.max_ctx > 128) TRY(dalloc_t(m, &m->sattn_part, 32 * SPLIT_MAX_ROWS * hv));
    }
    if (m->n_out_max > 0) {
        TRY(dalloc_t(m, &m->rl, R * m->n_out_max));
        TRY(dalloc_t(m, &m->sel_idx, R * m->top_max));
        TRY(dalloc_t(m, &m->sel_w, R * m->top_max));
        TRY(dalloc(m, &m->act, R * m->top_max * m->kfp_max * es));
        if (c.mode == GTB_SEQ_BF16 && m->e_max > 0) {
            m->mpad_max = (int)((R * m->top_max + 127) / 128 * 128) + m->e_max * 128;
            TRY(dalloc_t(m, &m->Xg, (size_t)m->mpad_max * wp));
            TRY(dalloc_t(m, &m->actg, (size_t)m->mpad_max * m->kfp_max));
            TRY(dalloc_t(m, &m->Yg, (size_t)m->mpad_max * W));
            TRY(dalloc_t(m, &m->rw, m->mpad_max));
            TRY(dalloc_t(m, &m->pair_dst, R * m->top_max));
            TRY(dalloc_t(m, &m->tile_e, m->mpad_max / 128));
        }
    }
    {   // key splits of decode-time attention: one CTA per 128 keys of a full slot, at most 32
        int hv = 0;
        for (const LayerW& l : m->L)
            for (int bi = 0; bi < l.d.n_branches; bi++)
                if (l.br[bi].d.kind == GTB_MIX_SIGMOID_ATTN) hv = std::max(hv, l.br[bi].d.heads * l.br[bi].d.vdim);
        m->attn_splits = std::max(1, std::min(32, c.max_ctx / 128));
        if (hv > 0 && m->attn_splits > 1) TRY(dalloc_t(m, &m->attn_part, (size_t)m->attn_splits * SPLIT_MAX_ROWS * hv));
    }
    if (m->prenorm) {
        TRY(dalloc_t(m, &m->xs, (size_t)m->ns * R * W));
        TRY(dalloc_t(m, &m->Y2, R * W));
        TRY(dalloc_t(m, &m->shw, R));
        TRY(dalloc_t(m, &m->latQ, R * std::max(m->lat_q_max, 1)));
        TRY(dalloc_t(m, &m->latQA, R * std::max(m->lat_qa_max, 1)));
        TRY(dalloc(m, &m->opQ, R * std::max(m->lat_qr_max, 8) * es));
        TRY(dalloc(m, &m->opO, R * std::max(m->lat_ol_max, 8) * es));
        if (c.mode == GTB_SEQ_BF16 && m->lat_kx_max > 0) {
            TRY(dalloc_t(m, &m->latX, (size_t)c.max_ctx * m->lat_x_max));
            TRY(dalloc_t(m, &m->latKx, (size_t)c.n_slots * c.max_ctx * m->lat_kx_max));
            TRY(dalloc_t(m, &m->latVx, (size_t)c.n_slots * c.max_ctx * m->lat_vx_max));
        }
    }
    TRY(dalloc_t(m, &m->logits, R * c.vocab));
    TRY(dalloc(m, &m->opA, R * wp * es));
    TRY(dalloc(m, &m->opB, R * wp * es));
    TRY(dalloc(m, &m->opC, R * m->kout_p_max * es));
    TRY(dalloc(m, &m->opL, R * pad64(2 * W) * es));
    TRY(dalloc(m, &m->opH, R * wp * es));
    m->tab_cap = 3 * c.n_slots + 3 * (int)R + 16;
    TRY(dalloc_t(m, &m->d_tab, m->tab_cap));
    GTB_CUDA(cudaHostAlloc((void**)&m->h_tab, m->tab_cap * sizeof(int), cudaHostAllocDefault));
    TRY(dalloc_t(m, &m->d_row_pos, R));
    TRY(dalloc_t(m, &m->d_row_prev, R));
    TRY(dalloc_t(m, &m->d_hist, (size_t)c.n_slots * 2));
    TRY(dalloc_t(m, &m->d_slots, c.n_slots));
    m->host_pos.assign(c.n_slots, 0);
    for (int s = 0; s < c.n_slots; s++) TRY(gtb_seq_slot_reset(m, s));
    if (c.mode == GTB_SEQ_BF16) seq_gemm_create(&m->gp);     // a failure leaves gp null: SIMT kernels only
#undef TRY
#undef REQ
    GTB_CUDA(cudaStreamSynchronize(ctx().stream));
    *out = m;
    return GTB_OK;
}

int gtb_seq_destroy(gtb_seq_t m) {
    if (!m) return GTB_OK;
    cudaStreamSynchronize(ctx().stream);
    if (m->graph) cudaGraphExecDestroy(m->graph);
    if (m->gp) seq_gemm_destroy(m->gp);
    for (void* p : m->allocs) cudaFree(p);
    if (m->h_tab) cudaFreeHost(m->h_tab);
    delete m;
    return GTB_OK;
}

int gtb_seq_set_tensor(gtb_seq_t m, const char* name, const void* h_bf16, const int64_t* shape, int ndim) {
    GTB_CHECK_INIT();
    GTB_ARG(m && name && h_bf16 && ndim >= 0 && ndim <= 2);
    auto it = m->tensors.find(name);
    if (it == m->tensors.end()) return gtb::fail(GTB_ERR_ARG, "tensor '%s' does not belong to this model", name);
    TensorDest& d = it->second;
    const int64_t r = ndim >= 1 ? shape[0] : 0, cc = ndim >= 2 ? shape[1] : 0;
    bool ok;
    if (d.scalar) ok = ndim == 0 || (ndim == 1 && r == 1);
    else if (d.kind == 1 && d.cols == 0) ok = ndim == 1 && r == d.rows;
    else ok = ndim == 2 && r == d.rows && cc == d.cols;
    if (!ok) return gtb::fail(GTB_ERR_ARG, "tensor '%s': shape does not fit the description (expected [%d, %d])", name, d.rows, d.cols);
    if (d.kind == 0) {
        if (d.group > 0) {
            for (int r0 = 0; r0 < d.rows; r0 += d.group)
                GTB_CUDA(cudaMemcpy2D((bf16*)d.dst + (size_t)(r0 / d.group) * d.group_stride * d.ld, (size_t)d.ld * 2,
                                      (const bf16*)h_bf16 + (size_t)r0 * d.cols, (size_t)d.cols * 2, (size_t)d.cols * 2, std::min(d.group, d.rows - r0), cudaMemcpyHostToDevice));
        } else if (d.split_cols > 0) {
            for (int c0 = 0; c0 < d.cols; c0 += d.split_cols)
                GTB_CUDA(cudaMemcpy2D((bf16*)d.dst + (size_t)(c0 / d.split_cols) * d.split_stride, (size_t)d.ld * 2, (const bf16*)h_bf16 + c0, (size_t)d.cols * 2,
                                      (size_t)std::min(d.split_cols, d.cols - c0) * 2, d.rows, cudaMemcpyHostToDevice));
        } else {
            GTB_CUDA(cudaMemcpy2D(d.dst, (size_t)d.ld * 2, h_bf16, (size_t)d.cols * 2, (size_t)d.cols * 2, d.rows, cudaMemcpyHostToDevice));
        }
    } else {
        const size_t n = d.scalar ? 1 : (size_t)d.rows * std::max(d.cols, 1);
        std::vector<float> f(n);
        const uint16_t* s = reinterpret_cast<const uint16_t*>(h_bf16);
        for (size_t i = 0; i < n; i++) { const uint32_t u = (uint32_t)s[i] << 16; memcpy(&f[i], &u, 4); }
        GTB_CUDA(cudaMemcpy(d.dst, f.data(), n * sizeof(float), cudaMemcpyHostToDevice));
    }
    d.loaded = true;
    return GTB_OK;
}

int gtb_seq_finalize(gtb_seq_t m) {
    GTB_ARG(m);
    for (auto& kv : m->tensors)
        if (!kv.second.loaded) return gtb::fail(GTB_ERR_STATE, "tensor '%s' has not been loaded", kv.first.c_str());
    m->finalized = true;
    return GTB_OK;
}

int gtb_seq_n_runs(gtb_seq_t m, int* n) { GTB_ARG(m && n); *n = (int)m->runs.size(); return GTB_OK; }

int gtb_seq_slot_reset(gtb_seq_t m, int slot) {
    GTB_CHECK_INIT();
    GTB_ARG(m && slot >= 0 && slot < m->cfg.n_slots);
    cudaStream_t st = ctx().stream;
    const SlotState z{0, -1, 0, 0};
    GTB_CUDA(cudaMemcpyAsync(m->d_slots + slot, &z, sizeof z, cudaMemcpyHostToDevice, st));
    GTB_CUDA(cudaStreamSynchronize(st));                    // z is a local
    for (Run& r : m->runs) {
        const LayerW& l = m->L[r.layer];
        for (int bi = 0; bi < l.d.n_branches; bi++)
            if (r.state[bi]) {
                const size_t sb = state_floats(l.br[bi].d) * sizeof(float);
                GTB_CUDA(cudaMemsetAsync((char*)r.state[bi] + sb * slot, 0, sb, st));
            }
        if (r.tail) {
            const size_t tb = (size_t)(m->cfg.taps - 1) * m->cfg.width * sizeof(float);
            GTB_CUDA(cudaMemsetAsync((char*)r.tail + tb * slot, 0, tb, st));
        }
    }
    m->host_pos[slot] = 0;
    return GTB_OK;
}

int gtb_seq_slot_position(gtb_seq_t m, int slot, int* pos) {
    GTB_CHECK_INIT();
    GTB_ARG(m && pos && slot >= 0 && slot < m->cfg.n_slots);
    SlotState s;
    GTB_CUDA(cudaMemcpyAsync(&s, m->d_slots + slot, sizeof s, cudaMemcpyDeviceToHost, ctx().stream));
    GTB_CUDA(cudaStreamSynchronize(ctx().stream));
    *pos = s.pos;
    m->host_pos[slot] = s.pos;
    return GTB_OK;
}

static int step_impl(gtb_seq_t m, int n_seg, const int32_t* seg_slot, const int32_t* seg_len, const int32_t* h_tokens, int n_want,
                     const int32_t* want_rows, float* h_logits, bool greedy, int32_t* h_next) {
    GTB_CHECK_INIT();
    GTB_ARG(m && n_seg > 0 && n_seg <= m->cfg.n_slots && seg_slot && seg_len && h_tokens);
    if (!m->finalized) return gtb::fail(GTB_ERR_STATE, "gtb_seq_finalize has not succeeded");
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    std::vector<char> seen(c.n_slots, 0);
    long long total = 0;
    for (int s = 0; s < n_seg; s++) {
        GTB_ARG(seg_slot[s] >= 0 && seg_slot[s] < c.n_slots && !seen[seg_slot[s]] && seg_len[s] > 0);
        seen[seg_slot[s]] = 1;
        if (m->host_pos[seg_slot[s]] + seg_len[s] > c.max_ctx)
            return gtb::fail(GTB_ERR_ARG, "slot %d: %d + %d tokens exceed max_ctx %d", seg_slot[s], m->host_pos[seg_slot[s]], seg_len[s], c.max_ctx);
        total += seg_len[s];
    }
    for (long long i = 0; i < total; i++) GTB_ARG(h_tokens[i] >= 0 && h_tokens[i] < c.vocab);
    if (greedy) { GTB_ARG(h_next); n_want = 0; }
    for (int i = 0; i < n_want; i++) GTB_ARG(want_rows[i] >= 0 && want_rows[i] < total && (i == 0 || want_rows[i] > want_rows[i - 1]));
    if (n_want > 0) GTB_ARG(h_logits);
    // passes: walk the segments, cutting at max_rows rows
    int seg = 0, off = 0, wi = 0, row_base = 0;
    std::vector<int> next(n_seg, 0);
    while (seg < n_seg) {
        int* tb = m->h_tab;
        std::vector<int> ps, pr0, pl, pseg_of;      // this pass's segments
        int R = 0;
        int s = seg, o = off;
        while (s < n_seg && R < m->max_rows) {
            const int take = std::min(seg_len[s] - o, m->max_rows - R);
            ps.push_back(seg_slot[s]); pr0.push_back(R); pl.push_back(take); pseg_of.push_back(s);
            R += take; o += take;
            if (o == seg_len[s]) { s++; o = 0; }
        }
        const int S = (int)ps.size();
        std::vector<int> want_local, last_rows;
        while (wi < n_want && want_rows[wi] < row_base + R) want_local.push_back(want_rows[wi++] - row_base);
        std::vector<int> greedy_segs;
        if (greedy)
            for (int k = 0; k < S; k++) {
                const int gs = pseg_of[k];
                const bool ends = (gs < s) || (gs == s && o == 0);       // the segment's last row is inside this pass
                if (ends) { want_local.push_back(pr0[k] + pl[k] - 1); greedy_segs.push_back(k); }
            }
        int* p = tb;
        memcpy(p, ps.data(), S * 4); p += S;
        memcpy(p, pr0.data(), S * 4); p += S;
        memcpy(p, pl.data(), S * 4); p += S;
        for (int k = 0; k < S; k++) for (int i = 0; i < pl[k]; i++) *p++ = k;
        memcpy(p, h_tokens + row_base, R * 4); p += R;
        const int nw = (int)want_local.size();
        if (nw) memcpy(p, want_local.data(), nw * 4);
        const int n_ints = 3 * S + 2 * R + nw;
        GTB_CUDA(cudaMemcpyAsync(m->d_tab, tb, n_ints * sizeof(int), cudaMemcpyHostToDevice, st));
        const PassTables t = tables(m, S, R);
        const int* d_want = m->d_tab + 3 * S + 2 * R;
        int rc;
        // greedy passes: logits rows are ordered like greedy_segs; the argmax kernel needs a segment per logits row, so it runs on
        // a table of its own below
        if (c.mode == GTB_SEQ_F32) rc = run_pass<float>(m, t, R, S, false, nw, d_want, pl.data(), ps.data());
        else rc = run_pass<bf16>(m, t, R, S, false, nw, d_want, pl.data(), ps.data());
        if (rc) return rc;
        if (greedy && nw) {
            // segment table restricted to the segments that ended: reuse the upload buffer behind the pass's tables
            int* q = m->h_tab + n_ints;
            for (int k : greedy_segs) *q++ = ps[k];
            GTB_CUDA(cudaMemcpyAsync(m->d_tab + n_ints, m->h_tab + n_ints, nw * sizeof(int), cudaMemcpyHostToDevice, st));
            PassTables ta = t;
            ta.seg_slot = m->d_tab + n_ints;
            k_argmax_rows<<<nw, 1024, 0, st>>>(m->logits, c.vocab, ta, -1, m->d_hist, 1, 0);
            GTB_LAUNCHED();
            std::vector<int> got(nw);
            GTB_CUDA(cudaMemcpyAsync(got.data(), m->d_hist, nw * sizeof(int), cudaMemcpyDeviceToHost, st));
            GTB_CUDA(cudaStreamSynchronize(st));
            for (int i = 0; i < nw; i++) h_next[pseg_of[greedy_segs[i]]] = got[i];
            m->last_nseg = nw;
        } else if (nw) {
            GTB_CUDA(cudaMemcpyAsync(h_logits + (size_t)(wi - nw) * c.vocab, m->logits, (size_t)nw * c.vocab * sizeof(float), cudaMemcpyDeviceToHost, st));
            GTB_CUDA(cudaStreamSynchronize(st));
        } else {
            GTB_CUDA(cudaStreamSynchronize(st));       // the pinned table buffer is reused by the next pass
        }
        for (int k = 0; k < S; k++) m->host_pos[ps[k]] += pl[k];
        row_base += R;
        seg = s; off = o;
    }
    (void)next;
    if (m->gp) {
        int bad = 0;
        int rc = seq_gemm_status(m->gp, &bad);
        if (rc) return rc;
        if (bad) return gtb::fail(GTB_ERR_STATE, "a tensor-core product gave up on a pipeline wait; results of this step are not valid");
    }
    return GTB_OK;
}

int gtb_seq_step(gtb_seq_t m, int n_seg, const int32_t* seg_slot, const int32_t* seg_len, const int32_t* h_tokens, int n_want,
                 const int32_t* want_rows, float* h_logits) {
    return step_impl(m, n_seg, seg_slot, seg_len, h_tokens, n_want, want_rows, h_logits, false, nullptr);
}

int gtb_seq_step_greedy(gtb_seq_t m, int n_seg, const int32_t* seg_slot, const int32_t* seg_len, const int32_t* h_tokens, int32_t* h_next) {
    return step_impl(m, n_seg, seg_slot, seg_len, h_tokens, 0, nullptr, nullptr, true, h_next);
}

int gtb_seq_decode(gtb_seq_t m, int n, const int32_t* slots, int n_steps, int eos_id, int32_t* h_out) {
    GTB_CHECK_INIT();
    GTB_ARG(m && n > 0 && n <= m->cfg.n_slots && n <= m->max_rows && slots && n_steps > 0 && h_out);
    if (!m->finalized) return gtb::fail(GTB_ERR_STATE, "gtb_seq_finalize has not succeeded");
    cudaStream_t st = ctx().stream;
    const gtb_seq_config& c = m->cfg;
    std::vector<char> seen(c.n_slots, 0);
    for (int i = 0; i < n; i++) {
        GTB_ARG(slots[i] >= 0 && slots[i] < c.n_slots && !seen[slots[i]]);
        seen[slots[i]] = 1;
        if (m->host_pos[slots[i]] + n_steps > c.max_ctx)
            return gtb::fail(GTB_ERR_ARG, "slot %d: %d + %d tokens exceed max_ctx %d", slots[i], m->host_pos[slots[i]], n_steps, c.max_ctx);
    }
    const bool same = m->graph && m->graph_eos == eos_id && m->graph_slots.size() == (size_t)n && std::equal(slots, slots + n, m->graph_slots.begin());
    // tables of a decode pass: segment i = slot i, one row each, wanted rows = all
    int* p = m->h_tab;
    for (int i = 0; i < n; i++) *p++ = slots[i];
    for (int i = 0; i < n; i++) *p++ = i;
    for (int i = 0; i < n; i++) *p++ = 1;
    for (int i = 0; i < n; i++) *p++ = i;      // row_seg
    for (int i = 0; i < n; i++) *p++ = 0;      // tok (from pending)
    for (int i = 0; i < n; i++) *p++ = i;      // want
    GTB_CUDA(cudaMemcpyAsync(m->d_tab, m->h_tab, 6 * n * sizeof(int), cudaMemcpyHostToDevice, st));
    const PassTables t = tables(m, n, n);
    const int* d_want = m->d_tab + 5 * n;
    int* d_out = nullptr;
    GTB_CUDA(cudaMalloc((void**)&d_out, (size_t)n * n_steps * sizeof(int)));
    auto one = [&]() -> int {
        int rc = c.mode == GTB_SEQ_F32 ? run_pass<float>(m, t, n, n, true, n, d_want) : run_pass<bf16>(m, t, n, n, true, n, d_want);
        if (rc) return rc;
        k_argmax_rows<<<n, 1024, 0, st>>>(m->logits, c.vocab, t, eos_id, m->d_hist, 1, 0);
        GTB_LAUNCHED();
        return GTB_OK;
    };
    int rc = GTB_OK;
    if (m->use_graph && !m->capture) {
        if (!same) {
            if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
            const int64_t l0 = ctx().launches;
            cudaGraph_t g = nullptr;
            GTB_CUDA(cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal));
            rc = one();
            cudaError_t ce = cudaStreamEndCapture(st, &g);
            ctx().launches = l0;
            if (rc) { if (g) cudaGraphDestroy(g); cudaFree(d_out); return rc; }
            if (ce != cudaSuccess) { cudaFree(d_out); return gtb::fail(GTB_ERR_CUDA, "graph capture failed: %s", cudaGetErrorString(ce)); }
            ce = cudaGraphInstantiate(&m->graph, g, 0);
            cudaGraphDestroy(g);
            if (ce != cudaSuccess) { cudaFree(d_out); return gtb::fail(GTB_ERR_CUDA, "graph instantiation failed: %s", cudaGetErrorString(ce)); }
            m->graph_slots.assign(slots, slots + n);
            m->graph_eos = eos_id;
        }
    }
    for (int k = 0; k < n_steps && rc == GTB_OK; k++) {
        if (m->use_graph && !m->capture) {
            cudaError_t ce = cudaGraphLaunch(m->graph, st);
            if (ce != cudaSuccess) rc = gtb::fail(GTB_ERR_CUDA, "graph launch failed: %s", cudaGetErrorString(ce));
            ctx().launches += 1;
        } else {
            rc = one();
        }
        if (rc == GTB_OK) {
            cudaError_t ce = cudaMemcpy2DAsync(d_out + k, (size_t)n_steps * sizeof(int), m->d_hist, sizeof(int), sizeof(int), n, cudaMemcpyDeviceToDevice, st);
            if (ce != cudaSuccess) rc = gtb::fail(GTB_ERR_CUDA, "copy failed: %s", cudaGetErrorString(ce));
        }
    }
    if (rc == GTB_OK) {
        cudaError_t ce = cudaMemcpyAsync(h_out, d_out, (size_t)n * n_steps * sizeof(int), cudaMemcpyDeviceToHost, st);
        if (ce == cudaSuccess) ce = cudaStreamSynchronize(st);
        if (ce != cudaSuccess) rc = gtb::fail(GTB_ERR_CUDA, "copy failed: %s", cudaGetErrorString(ce));
    }
    cudaFree(d_out);
    if (rc) return rc;
    m->last_nseg = n;
    for (int i = 0; i < n; i++) { int pos; gtb_seq_slot_position(m, slots[i], &pos); }
    return GTB_OK;
}

int gtb_seq_topk(gtb_seq_t m, int seg, int k, float* h_values, int32_t* h_ids) {
    GTB_CHECK_INIT();
    GTB_ARG(m && seg >= 0 && seg < m->last_nseg && k > 0 && k <= 64 && k <= m->cfg.vocab && h_values && h_ids);
    float* dv = nullptr;
    GTB_CUDA(cudaMalloc((void**)&dv, 64 * (sizeof(float) + sizeof(int32_t))));
    int32_t* di = reinterpret_cast<int32_t*>(dv + 64);
    k_topk<<<1, 1024, 0, ctx().stream>>>(m->logits + (size_t)seg * m->cfg.vocab, m->cfg.vocab, k, dv, di);
    ctx().launches++;
    cudaError_t e = cudaMemcpyAsync(h_values, dv, k * sizeof(float), cudaMemcpyDeviceToHost, ctx().stream);
    if (e == cudaSuccess) e = cudaMemcpyAsync(h_ids, di, k * sizeof(int32_t), cudaMemcpyDeviceToHost, ctx().stream);
    if (e == cudaSuccess) e = cudaStreamSynchronize(ctx().stream);
    cudaFree(dv);
    if (e != cudaSuccess) return gtb::fail(GTB_ERR_CUDA, "top-k failed: %s", cudaGetErrorString(e));
    return GTB_OK;
}

int gtb_seq_last_logits(gtb_seq_t m, int seg, float* h_logits) {
    GTB_CHECK_INIT();
    GTB_ARG(m && seg >= 0 && seg < m->last_nseg && h_logits);
    GTB_CUDA(cudaMemcpyAsync(h_logits, m->logits + (size_t)seg * m->cfg.vocab, m->cfg.vocab * sizeof(float), cudaMemcpyDeviceToHost, ctx().stream));
    GTB_CUDA(cudaStreamSynchronize(ctx().stream));
    return GTB_OK;
}

int gtb_seq_set_option(gtb_seq_t m, const char* name, int value) {
    GTB_ARG(m && name);
    const std::string n = name;
    if (n == "capture") {
        m->capture = value != 0;
        if (m->capture && !m->cap) {
            int rc = dalloc_t(m, &m->cap, m->runs.size() * (size_t)m->max_rows * m->cfg.width);
            if (rc) return rc;
        }
    } else if (n == "tensor") m->use_tensor = value != 0;
    else if (n == "tensor_min_rows") m->tensor_min_rows = std::max(1, value);
    else if (n == "graph") m->use_graph = value != 0;
    else if (n == "fused_attn") m->fused_attn = value != 0;
    else if (n == "fused_norm") m->fused_norm = value != 0;
    else if (n == "grouped_experts") m->grouped_experts = value != 0;
    else return gtb::fail(GTB_ERR_ARG, "unknown option '%s'", name);
    if (m->graph) { cudaGraphExecDestroy(m->graph); m->graph = nullptr; }
    return GTB_OK;
}

int gtb_seq_read_capture(gtb_seq_t m, int run, int row, float* h_out) {
    GTB_CHECK_INIT();
    GTB_ARG(m && m->cap && run >= 0 && run < (int)m->runs.size() && row >= 0 && row < m->cap_rows && h_out);
    GTB_CUDA(cudaMemcpyAsync(h_out, m->cap + ((size_t)run * m->max_rows + row) * m->cfg.width, m->cfg.width * sizeof(float), cudaMemcpyDeviceToHost, ctx().stream));
    GTB_CUDA(cudaStreamSynchronize(ctx().stream));
    return GTB_OK;
}

// self-test / timing of the bf16 tensor-core product on host data: C = A . W^T (+ C0 when accumulate), ld = K + ld_extra elements
int gtb_seq_selftest_gemm(const void* h_A, const void* h_W, float* h_C, int M, int N, int K, int ld_extra, int accumulate, int iters, float* ms) {
    GTB_CHECK_INIT();
    GTB_ARG(h_A && h_W && h_C && M > 0 && N > 0 && K > 0 && K % 64 == 0 && ld_extra >= 0 && ld_extra % 8 == 0 && iters >= 1);
    SeqGemmPlan* gp = nullptr;
    int rc = seq_gemm_create(&gp);
    if (rc) return rc;
    const int ld = K + ld_extra;
    bf16 *dA = nullptr, *dW = nullptr;
    float* dC = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t st = ctx().stream;
    auto done = [&](int code) { cudaFree(dA); cudaFree(dW); cudaFree(dC); if (e0) cudaEventDestroy(e0); if (e1) cudaEventDestroy(e1); seq_gemm_destroy(gp); return code; };
    if (cudaMalloc((void**)&dA, (size_t)M * ld * 2) != cudaSuccess || cudaMalloc((void**)&dW, (size_t)N * ld * 2) != cudaSuccess ||
        cudaMalloc((void**)&dC, (size_t)M * N * 4) != cudaSuccess) return done(gtb::fail(GTB_ERR_CUDA, "cudaMalloc failed"));
    cudaMemset(dA, 0, (size_t)M * ld * 2);
    cudaMemset(dW, 0, (size_t)N * ld * 2);
    cudaMemcpy2D(dA, (size_t)ld * 2, h_A, (size_t)K * 2, (size_t)K * 2, M, cudaMemcpyHostToDevice);
    cudaMemcpy2D(dW, (size_t)ld * 2, h_W, (size_t)K * 2, (size_t)K * 2, N, cudaMemcpyHostToDevice);
    cudaMemcpy(dC, h_C, (size_t)M * N * 4, cudaMemcpyHostToDevice);
    cudaDeviceSynchronize();          // the copies above ran on the default stream, the product runs on the library stream
    rc = seq_gemm_bf16(gp, dA, ld, dW, ld, dC, N, M, N, K, nullptr, accumulate);
    if (rc) return done(rc == -1 ? gtb::fail(GTB_ERR_ARG, "shape not supported by the tensor-core product") : rc);
    cudaMemcpyAsync(h_C, dC, (size_t)M * N * 4, cudaMemcpyDeviceToHost, st);
    cudaEventCreate(&e0); cudaEventCreate(&e1);
    cudaEventRecord(e0, st);
    // accumulate >= 2: timing runs accumulate too and a 256 MB buffer is rewritten before each (operands come from HBM, not L2)
    void* flush = nullptr;
    float total = 0.0f;
    if (accumulate >= 2 && cudaMalloc(&flush, (size_t)256 << 20) != cudaSuccess) flush = nullptr;
    if (flush) {
        for (int i = 0; i < iters; i++) {
            cudaMemsetAsync(flush, i, (size_t)256 << 20, st);
            cudaEventRecord(e0, st);
            seq_gemm_bf16(gp, dA, ld, dW, ld, dC, N, M, N, K, nullptr, 1);
            cudaEventRecord(e1, st);
            cudaStreamSynchronize(st);
            float t = 0.0f;
            cudaEventElapsedTime(&t, e0, e1);
            total += t;
        }
        cudaFree(flush);
        cudaEventRecord(e0, st);
    } else {
        for (int i = 0; i < iters; i++) seq_gemm_bf16(gp, dA, ld, dW, ld, dC, N, M, N, K, nullptr, 0);
    }
    cudaEventRecord(e1, st);
    if (cudaStreamSynchronize(st) != cudaSuccess) return done(gtb::fail(GTB_ERR_CUDA, "the product failed: %s", cudaGetErrorString(cudaGetLastError())));
    if (ms) { cudaEventElapsedTime(ms, e0, e1); *ms = (flush ? total : *ms) / iters; }
    int bad = 0;
    seq_gemm_status(gp, &bad);
    return done(bad ? gtb::fail(GTB_ERR_STATE, "the product gave up on a pipeline wait") : GTB_OK);
}

int gtb_seq_weight_bytes(gtb_seq_t m, size_t* nbytes) { GTB_ARG(m && nbytes); *nbytes = m->weight_bytes; return GTB_OK; }
int gtb_seq_state_bytes_per_slot(gtb_seq_t m, size_t* nbytes) { GTB_ARG(m && nbytes); *nbytes = m->state_bytes; return GTB_OK; }

}  // extern "C"
