// gtb_seq_gemm.cu -- bf16 matrix product of the layer-list sequence models on the 5th-generation tensor cores.
//
//     C[M][N] = (acc ? C : 0) + bias + A[M][K] . W[N][K]^T        A, W bf16 (K contiguous), C fp32
//
// Same structure as the batched-prefill product of the TinyLlama path (gtb_prefill.cu), with bf16 operands and a plain fp32
// epilogue: persistent CTAs (one per SM) walk the 128 x BN output tiles; warp 0 is the TMA producer (128-byte swizzled 128 x 64 and
// BN x 64 boxes through a ring of mbarrier stages), one thread of warp 1 issues tcgen05.mma kind::f16 (M128 x N(BN) x K16, fp32
// accumulators in a double-buffered TMEM allocation) and releases stages / publishes accumulators with tcgen05.commit, warps 2-9
// read their 32 TMEM lanes back with tcgen05.ld and write C -- the epilogue of tile i overlaps the main loop of tile i + 1.
// Rows and columns beyond M and N come in as zeros (TMA out-of-bounds fill) and are not stored; K is a multiple of 64 because every
// operand of these models is padded to that.
//
// Every mbarrier wait is bounded: a wait that does not complete raises the CTA's abort flag, every role leaves its loop, the
// TMEM allocation is released and the kernel returns with a status word set that the host reads after the launch.
//
// The fused variant (EPI_GEGLU) takes W = gate rows and up rows interleaved in groups of 32 and writes gelu_tanh(gate) * up as a
// bf16 operand block: the feed-forward activation never exists in fp32 in HBM.
//
// Grouped products (routed experts): the rows of A are sorted into groups that start on multiples of 128 rows, a device table gives
// every M tile its group (or -1: nothing to do), and group g multiplies with rows [g N, (g + 1) N) of W.  EPI_RELU2 writes
// row_w[row] * relu(acc)^2 as a bf16 operand block (the expert's activation, already weighted with the router's score).
#include "gtb_seq_gemm.h"

#include <cuda_bf16.h>

#include "gtb_internal.h"
#include "gtb_tc.cuh"

namespace gtb {
namespace seq {

constexpr int SQ_BM = 128, SQ_BK = 64, SQ_THREADS = 320, SQ_EPI_THREADS = 256;
enum { SQ_EPI_F32 = 0, SQ_EPI_GEGLU = 1, SQ_EPI_RELU2 = 2 };

template <int BN> struct SqCfg {
    static constexpr int STAGES = (BN == 256) ? 4 : 6;
    static constexpr uint32_t A_BYTES = SQ_BM * SQ_BK * 2;
    static constexpr uint32_t B_BYTES = BN * SQ_BK * 2;
    static constexpr uint32_t STAGE_BYTES = A_BYTES + B_BYTES;
    static constexpr uint32_t SMEM = STAGES * STAGE_BYTES + 1024 + 256;
    // kind::f16 instruction descriptor: D fp32 (bit 4), A and B bf16 (format 1 at bits 7-9 and 10-12), both K-major,
    // N >> 3 at bits 17-22, M >> 4 at bits 24-28
    static constexpr uint32_t IDESC = (1u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(SQ_BM >> 4) << 24);
};

struct SqEpi {
    float* C;
    int ldc;
    const float* bias;
    int accumulate;
    __nv_bfloat16* act;      // EPI_GEGLU: output operand [M][ld_act], written at column act_off + (pair index)
    int ld_act, act_off;
    int* status;
    const int* tile_group;   // grouped product: group of every M tile (-1: skip), or null
    int group_rows;          // rows of W per group
    const float* row_w;      // EPI_RELU2: weight of every row of A; EPI_GEGLU: optional weight of every row
    int act_kind;            // EPI_GEGLU: 0 = gelu_tanh(gate) * up, 1 = silu(gate) * up
};

// bounded wait: false when the barrier did not complete (or another role gave up)
__device__ __forceinline__ bool sq_wait(uint32_t bar, uint32_t parity, volatile int* abort_flag) {
    for (int it = 0; it < (1 << 24); it++) {
        if (mbar_try_wait(bar, parity)) return true;
        if ((it & 1023) == 1023 && *abort_flag) return false;
    }
    *abort_flag = 1;
    return false;
}

// tanh on the special-function unit: relative error ~2^-11, below the bf16 rounding of the value that is stored
__device__ __forceinline__ float sq_gelu(float z) {
    const float c = 0.7978845608028654f;
    float th;
    asm("tanh.approx.f32 %0, %1;" : "=f"(th) : "f"(c * (z + 0.044715f * z * z * z)));
    return 0.5f * z * (1.0f + th);
}

// silu(z) = z / (1 + 2^(-z log2 e)) on the special-function unit; the value is rounded to bf16 right after
__device__ __forceinline__ float sq_silu(float z) { return __fdividef(z, 1.0f + __expf(-z)); }
__device__ __forceinline__ float sq_gate(float z, int kind) { return kind ? sq_silu(z) : sq_gelu(z); }

template <int BN, int EPI>
__global__ void __launch_bounds__(SQ_THREADS, 1)
k_seq_gemm(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB, int M, int N, int K, const SqEpi ep) {
    using Cfg = SqCfg<BN>;
    constexpr int ST = Cfg::STAGES;
    extern __shared__ unsigned char smem_raw[];
    unsigned char* smem = reinterpret_cast<unsigned char*>(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    uint64_t* bars = reinterpret_cast<uint64_t*>(smem + ST * Cfg::STAGE_BYTES);
    uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 2 * ST + 4);
    volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
    const uint32_t smem_base = smem_u32(smem), bar_base = smem_u32(bars);
    auto bar_full = [&](int s) { return bar_base + 8u * s; };
    auto bar_empty = [&](int s) { return bar_base + 8u * (ST + s); };
    auto bar_tfull = [&](int a) { return bar_base + 8u * (2 * ST + a); };
    auto bar_tempty = [&](int a) { return bar_base + 8u * (2 * ST + 2 + a); };

    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int n_mt = (M + SQ_BM - 1) / SQ_BM, n_nt = (N + BN - 1) / BN;
    const int n_tiles = n_mt * n_nt, nkb = K / SQ_BK;

    if (threadIdx.x == 0) {
        for (int s = 0; s < ST; s++) { mbar_init(bar_full(s), 1); mbar_init(bar_empty(s), 1); }
        for (int a = 0; a < 2; a++) { mbar_init(bar_tfull(a), 1); mbar_init(bar_tempty(a), SQ_EPI_THREADS); }
        *abort_flag = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(smem_u32(tmem_slot), 2 * BN);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem_base = *tmem_slot;

    if (warp == 0) {
        if (lane == 0) {        // ---------------- TMA producer
            tma_prefetch_desc(&tmA);
            tma_prefetch_desc(&tmB);
            uint32_t s = 0, ph = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                const int mt = tile % n_mt, nt = tile / n_mt;         // consecutive CTAs share one slice of W
                const int grp = ep.tile_group ? ep.tile_group[mt] : 0;
                if (grp < 0) continue;
                const int wrow = grp * ep.group_rows + nt * BN;
                for (int kb = 0; kb < nkb; kb++) {
                    if (!(ok = sq_wait(bar_empty(s), ph ^ 1, abort_flag))) break;
                    mbar_expect_tx(bar_full(s), Cfg::STAGE_BYTES);
                    const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES;
                    tma_load_2d(sa, &tmA, bar_full(s), kb * SQ_BK, mt * SQ_BM);
                    tma_load_2d(sa + Cfg::A_BYTES, &tmB, bar_full(s), kb * SQ_BK, wrow);
                    if (++s == ST) { s = 0; ph ^= 1; }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {        // ---------------- MMA issuer
            uint32_t s = 0, ph = 0;
            int it = 0;
            bool ok = true;
            for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
                if (ep.tile_group && ep.tile_group[tile % n_mt] < 0) continue;      // skipped tiles take no accumulator stage
                const int cur = it++, as = cur & 1;
                if (!(ok = sq_wait(bar_tempty(as), ((cur >> 1) & 1) ^ 1, abort_flag))) break;
                tc_fence_after();
                const uint32_t d_tmem = tmem_base + (uint32_t)(as * BN);
                for (int kb = 0; kb < nkb; kb++) {
                    if (!(ok = sq_wait(bar_full(s), ph, abort_flag))) break;
                    tc_fence_after();
                    const uint32_t sa = smem_base + s * Cfg::STAGE_BYTES, sb = sa + Cfg::A_BYTES;
#pragma unroll
                    for (int k = 0; k < SQ_BK / 16; k++)
                        umma_f16(d_tmem, umma_desc_sw128(sa + k * 32), umma_desc_sw128(sb + k * 32), Cfg::IDESC, (kb | k) != 0);
                    umma_commit(bar_empty(s));
                    if (kb == nkb - 1) umma_commit(bar_tfull(as));
                    if (++s == ST) { s = 0; ph ^= 1; }
                }
            }
        }
        __syncwarp();
    } else {                    // ---------------- epilogue warps
        const int lg = warp & 3;                                    // TMEM lanes 32 * (warp % 4) .. + 31
        const int chalf = (warp - 2) >> 2;                          // which half of the tile's columns
        int it = 0;
        bool ok = true;
        for (int tile = blockIdx.x; ok && tile < n_tiles; tile += gridDim.x) {
            const int mt = tile % n_mt, nt = tile / n_mt;
            if (ep.tile_group && ep.tile_group[mt] < 0) continue;
            const int cur = it++, as = cur & 1;
            if (!(ok = sq_wait(bar_tfull(as), (cur >> 1) & 1, abort_flag))) break;
            tc_fence_after();
            const int row = mt * SQ_BM + lg * 32 + lane;
            const uint32_t tacc = tmem_base + ((uint32_t)(lg * 32) << 16) + (uint32_t)(as * BN);
            if (EPI == SQ_EPI_F32) {
#pragma unroll 1
                for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); c++) {
                    const int col = nt * BN + c * 32;
                    float v[32];
                    tmem_ld32(tacc + (uint32_t)(c * 32), v);
                    if (row < M && col < N) {
                        float* dst = ep.C + (size_t)row * ep.ldc + col;
                        const int nc = min(32, N - col);
                        if (nc == 32 && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4) {
                                float4 o = make_float4(v[j], v[j + 1], v[j + 2], v[j + 3]);
                                if (ep.bias) { o.x += ep.bias[col + j]; o.y += ep.bias[col + j + 1]; o.z += ep.bias[col + j + 2]; o.w += ep.bias[col + j + 3]; }
                                if (ep.accumulate) { const float4 p = *reinterpret_cast<const float4*>(dst + j); o.x += p.x; o.y += p.y; o.z += p.z; o.w += p.w; }
                                *reinterpret_cast<float4*>(dst + j) = o;
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < nc) {
                                    float o = v[j];
                                    if (ep.bias) o += ep.bias[col + j];
                                    if (ep.accumulate) o += dst[j];
                                    dst[j] = o;
                                }
                        }
                    }
                }
            } else if (EPI == SQ_EPI_RELU2) {
                const float wt = row < M ? ep.row_w[row] : 0.0f;
#pragma unroll 1
                for (int c = chalf * (BN / 64); c < (chalf + 1) * (BN / 64); c++) {
                    const int col = nt * BN + c * 32;
                    float v[32];
                    tmem_ld32(tacc + (uint32_t)(c * 32), v);
                    if (row < M && col < N) {
                        __nv_bfloat16* dst = ep.act + (size_t)row * ep.ld_act + ep.act_off + col;
                        const int nc = min(32, N - col);
                        if (nc == 32 && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint32_t w[4];
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    const float a0 = fmaxf(v[j + 2 * q], 0.0f), a1 = fmaxf(v[j + 2 * q + 1], 0.0f);
                                    const __nv_bfloat162 pr = __floats2bfloat162_rn(wt * a0 * a0, wt * a1 * a1);
                                    w[q] = *reinterpret_cast<const uint32_t*>(&pr);
                                }
                                *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < nc) { const float a0 = fmaxf(v[j], 0.0f); dst[j] = __float2bfloat16_rn(wt * a0 * a0); }
                        }
                    }
                }
            } else {
                // 64 accumulator columns = 32 gate columns followed by their 32 up columns
                const float wt = (ep.row_w && row < M) ? ep.row_w[row] : 1.0f;
                const int ak = ep.act_kind;
#pragma unroll 1
                for (int c2 = chalf * (BN / 128); c2 < (chalf + 1) * (BN / 128); c2++) {
                    const int col = nt * BN + c2 * 64;
                    float g[32], u[32];
                    tmem_ld32(tacc + (uint32_t)(c2 * 64), g);
                    tmem_ld32(tacc + (uint32_t)(c2 * 64 + 32), u);
                    if (row < M && col < N) {
                        const int c0 = col >> 1;                   // first of the 32 activation channels
                        __nv_bfloat16* dst = ep.act + (size_t)row * ep.ld_act + ep.act_off + c0;
                        const int nc = min(32, (N >> 1) - c0);
                        if (nc == 32 && ((((uintptr_t)dst) & 15) == 0)) {
#pragma unroll
                            for (int j = 0; j < 32; j += 8) {
                                uint32_t w[4];
#pragma unroll
                                for (int q = 0; q < 4; q++) {
                                    const __nv_bfloat162 v = __floats2bfloat162_rn(wt * sq_gate(g[j + 2 * q], ak) * u[j + 2 * q], wt * sq_gate(g[j + 2 * q + 1], ak) * u[j + 2 * q + 1]);
                                    w[q] = *reinterpret_cast<const uint32_t*>(&v);
                                }
                                *reinterpret_cast<uint4*>(dst + j) = make_uint4(w[0], w[1], w[2], w[3]);
                            }
                        } else {
#pragma unroll
                            for (int j = 0; j < 32; j++)
                                if (j < nc) dst[j] = __float2bfloat16_rn(wt * sq_gate(g[j], ak) * u[j]);
                        }
                    }
                }
            }
            tc_fence_before();
            mbar_arrive(bar_tempty(as));
        }
    }
    tc_fence_before();
    __syncthreads();
    if (threadIdx.x == 0 && *abort_flag && ep.status) atomicExch(ep.status, 1);
    if (warp == 1) tmem_dealloc(tmem_base, 2 * BN);
}

// ---------------------------------------------------------------------------------------------------------------- host
typedef CUresult (*PFN_tmapEncodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                        const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                        CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

struct SeqGemmPlan {
    PFN_tmapEncodeTiled enc = nullptr;
    int* d_status = nullptr;
    bool attr[2][3] = {{false, false, false}, {false, false, false}};
};

int seq_gemm_create(SeqGemmPlan** out) {
    *out = nullptr;
    void* p = nullptr;
    cudaDriverEntryPointQueryResult qres;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &qres) != cudaSuccess || qres != cudaDriverEntryPointSuccess)
        return fail(GTB_ERR_CUDA, "cuTensorMapEncodeTiled is not available from this driver");
    SeqGemmPlan* g = new SeqGemmPlan();
    g->enc = reinterpret_cast<PFN_tmapEncodeTiled>(p);
    if (cudaMalloc((void**)&g->d_status, sizeof(int)) != cudaSuccess) { delete g; return fail(GTB_ERR_CUDA, "cudaMalloc failed"); }
    cudaMemsetAsync(g->d_status, 0, sizeof(int), ctx().stream);
    *out = g;
    return GTB_OK;
}

void seq_gemm_destroy(SeqGemmPlan* p) {
    if (!p) return;
    if (p->d_status) cudaFree(p->d_status);
    delete p;
}

int seq_gemm_status(SeqGemmPlan* p, int* status) {
    GTB_CUDA(cudaMemcpyAsync(status, p->d_status, sizeof(int), cudaMemcpyDeviceToHost, ctx().stream));
    GTB_CUDA(cudaStreamSynchronize(ctx().stream));
    return GTB_OK;
}

static int make_map(SeqGemmPlan* p, CUtensorMap* m, const void* base, int rows, int cols, int ld, int box_rows) {
    const cuuint64_t gdim[2] = {(cuuint64_t)cols, (cuuint64_t)rows};
    const cuuint64_t gstr[1] = {(cuuint64_t)ld * 2};
    const cuuint32_t box[2] = {(cuuint32_t)SQ_BK, (cuuint32_t)box_rows};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult r = p->enc(m, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), gdim, gstr, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return fail(GTB_ERR_CUDA, "cuTensorMapEncodeTiled failed (%d) for a %d x %d matrix", (int)r, rows, cols);
    return GTB_OK;
}

template <int BN, int EPI>
static int launch(SeqGemmPlan* p, const CUtensorMap& ta, const CUtensorMap& tb, int M, int N, int K, const SqEpi& ep) {
    using Cfg = SqCfg<BN>;
    bool& attr = p->attr[BN == 256][EPI];
    if (!attr) {
        GTB_CUDA(cudaFuncSetAttribute(k_seq_gemm<BN, EPI>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)Cfg::SMEM));
        attr = true;
    }
    const int n_tiles = ((M + SQ_BM - 1) / SQ_BM) * ((N + BN - 1) / BN);
    const int grid = n_tiles < ctx().sm_count ? n_tiles : ctx().sm_count;
    k_seq_gemm<BN, EPI><<<grid, SQ_THREADS, Cfg::SMEM, ctx().stream>>>(ta, tb, M, N, K, ep);
    GTB_LAUNCHED();
    return GTB_OK;
}

static int run(SeqGemmPlan* p, int epi, const void* A, int lda, const void* W, int ldw, int M, int N, int K, const SqEpi& ep) {
    if (!p || K <= 0 || (K % SQ_BK) || (lda % 8) || (ldw % 8) || (((uintptr_t)A | (uintptr_t)W) & 15)) return -1;
    // 256-wide tiles when they still give every SM a tile; otherwise 128-wide
    const int mt = (M + SQ_BM - 1) / SQ_BM;
    // (the 128-wide MMA reads as much of A from shared memory per FLOP as the 256-wide one reads of A and W together: it runs at about
    // half the rate, so it only pays when 256-wide tiles would leave most SMs idle)
    const int bn = (N > 128 && mt * ((N + 255) / 256) * 2 >= ctx().sm_count) ? 256 : 128;
    CUtensorMap ta, tb;
    int rc = make_map(p, &ta, A, M, K, lda, SQ_BM);
    if (rc) return rc;
    rc = make_map(p, &tb, W, N, K, ldw, bn);
    if (rc) return rc;
    if (epi == SQ_EPI_F32) return bn == 256 ? launch<256, SQ_EPI_F32>(p, ta, tb, M, N, K, ep) : launch<128, SQ_EPI_F32>(p, ta, tb, M, N, K, ep);
    return bn == 256 ? launch<256, SQ_EPI_GEGLU>(p, ta, tb, M, N, K, ep) : launch<128, SQ_EPI_GEGLU>(p, ta, tb, M, N, K, ep);
}

int seq_gemm_bf16(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, float* C, int ldc, int M, int N, int K, const float* bias, int accumulate) {
    SqEpi ep{};
    ep.C = C; ep.ldc = ldc; ep.bias = bias; ep.accumulate = accumulate; ep.status = p ? p->d_status : nullptr;
    return run(p, SQ_EPI_F32, A, lda, W, ldw, M, N, K, ep);
}

int seq_gemm_bf16_grouped(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, int M_pad, int N, int K, int n_groups, const int* tile_group,
                          float* C, int ldc, void* act, int ld_act, const float* row_w) {
    if (!p || K <= 0 || (K % SQ_BK) || (lda % 8) || (ldw % 8) || (((uintptr_t)A | (uintptr_t)W) & 15) || (M_pad % SQ_BM) || n_groups <= 0) return -1;
    SqEpi ep{};
    ep.C = C; ep.ldc = ldc; ep.act = reinterpret_cast<__nv_bfloat16*>(act); ep.ld_act = ld_act; ep.status = p->d_status;
    ep.tile_group = tile_group; ep.group_rows = N; ep.row_w = row_w;
    const int mt = M_pad / SQ_BM;
    const int bn = (N > 128 && mt * ((N + 255) / 256) * 2 >= ctx().sm_count) ? 256 : 128;
    CUtensorMap ta, tb;
    int rc = make_map(p, &ta, A, M_pad, K, lda, SQ_BM);
    if (rc) return rc;
    rc = make_map(p, &tb, W, n_groups * N, K, ldw, bn);
    if (rc) return rc;
    if (act) return bn == 256 ? launch<256, SQ_EPI_RELU2>(p, ta, tb, M_pad, N, K, ep) : launch<128, SQ_EPI_RELU2>(p, ta, tb, M_pad, N, K, ep);
    return bn == 256 ? launch<256, SQ_EPI_F32>(p, ta, tb, M_pad, N, K, ep) : launch<128, SQ_EPI_F32>(p, ta, tb, M_pad, N, K, ep);
}

int seq_gemm_bf16_geglu(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, void* act, int ld_act, int act_off, int M, int N2, int K) {
    return seq_gemm_bf16_gated(p, A, lda, W, ldw, act, ld_act, act_off, M, N2, K, 0, nullptr);
}

int seq_gemm_bf16_gated(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, void* act, int ld_act, int act_off, int M, int N2, int K, int act_kind,
                        const float* row_w) {
    if (N2 % 64) return -1;                      // whole (32 gate, 32 up) groups only
    SqEpi ep{};
    ep.act = reinterpret_cast<__nv_bfloat16*>(act); ep.ld_act = ld_act; ep.act_off = act_off; ep.status = p ? p->d_status : nullptr;
    ep.act_kind = act_kind; ep.row_w = row_w;
    return run(p, SQ_EPI_GEGLU, A, lda, W, ldw, M, N2, K, ep);
}

int seq_gemm_bf16_grouped_gated(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, int M_pad, int N2, int K, int n_groups, const int* tile_group,
                                void* act, int ld_act, const float* row_w, int act_kind) {
    if (!p || K <= 0 || (K % SQ_BK) || (lda % 8) || (ldw % 8) || (((uintptr_t)A | (uintptr_t)W) & 15) || (M_pad % SQ_BM) || n_groups <= 0 || (N2 % 64) || !act) return -1;
    SqEpi ep{};
    ep.act = reinterpret_cast<__nv_bfloat16*>(act); ep.ld_act = ld_act; ep.status = p->d_status;
    ep.tile_group = tile_group; ep.group_rows = N2; ep.row_w = row_w; ep.act_kind = act_kind;
    const int mt = M_pad / SQ_BM;
    const int bn = (N2 > 128 && mt * ((N2 + 255) / 256) * 2 >= ctx().sm_count) ? 256 : 128;
    CUtensorMap ta, tb;
    int rc = make_map(p, &ta, A, M_pad, K, lda, SQ_BM);
    if (rc) return rc;
    rc = make_map(p, &tb, W, n_groups * N2, K, ldw, bn);
    if (rc) return rc;
    return bn == 256 ? launch<256, SQ_EPI_GEGLU>(p, ta, tb, M_pad, N2, K, ep) : launch<128, SQ_EPI_GEGLU>(p, ta, tb, M_pad, N2, K, ep);
}

}  // namespace seq
}  // namespace gtb
