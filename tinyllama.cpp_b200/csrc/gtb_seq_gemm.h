// gtb_seq_gemm.h -- tensor-core matrix product of the layer-list sequence models (gtb_seq_gemm.cu):
// C[M][N] = (acc ? C : 0) + bias + A[M][K] . W[N][K]^T, bf16 operands, fp32 accumulation and output.
#pragma once
#include <stdint.h>

namespace gtb {
namespace seq {

struct SeqGemmPlan;
int seq_gemm_create(SeqGemmPlan** out);
void seq_gemm_destroy(SeqGemmPlan* p);
// returns -1 (nothing launched) when the shape is outside what the kernel takes: K and the leading dimensions must be multiples
// of 64 elements, the bases 16-byte aligned
int seq_gemm_bf16(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, float* C, int ldc, int M, int N, int K, const float* bias, int accumulate);
// fused feed-forward input: W holds gate rows and up rows interleaved in groups of 32 (N2 = 2 ff rows, a multiple of 64);
// act[row][act_off + c] = bf16(gelu_tanh(gate_c) * up_c) -- the product never reaches HBM in fp32
int seq_gemm_bf16_geglu(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, void* act, int ld_act, int act_off, int M, int N2, int K);
// the same with a choice of activation (act_kind 0: gelu_tanh(gate) * up, 1: silu(gate) * up) and an optional weight per row of A
int seq_gemm_bf16_gated(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, void* act, int ld_act, int act_off, int M, int N2, int K, int act_kind,
                        const float* row_w);
// grouped and gated: group g multiplies with rows [g N2, (g + 1) N2) of W (its gate and up rows interleaved in groups of 32);
// act[row][c] = bf16(row_w[row] * act(gate_c) * up_c) for c < N2 / 2
int seq_gemm_bf16_grouped_gated(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, int M_pad, int N2, int K, int n_groups, const int* tile_group,
                                void* act, int ld_act, const float* row_w, int act_kind);
// grouped product for routed experts: A [M_pad][K] holds rows sorted into groups that start on multiples of 128 rows, tile_group
// (device) [M_pad / 128] names every M tile's group or -1 (tile skipped, its output rows untouched); group g multiplies with rows
// [g N, (g + 1) N) of W.  act != null: act[row][c] = bf16(row_w[row] * relu(.)^2) for c < N; else C[row][c] (fp32, ldc) is written
int seq_gemm_bf16_grouped(SeqGemmPlan* p, const void* A, int lda, const void* W, int ldw, int M_pad, int N, int K, int n_groups, const int* tile_group,
                          float* C, int ldc, void* act, int ld_act, const float* row_w);
// 1 if a kernel of this plan gave up on a wait since the plan was created (its results are then not valid)
int seq_gemm_status(SeqGemmPlan* p, int* status);

}  // namespace seq
}  // namespace gtb
