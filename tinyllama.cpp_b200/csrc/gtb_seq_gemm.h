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
// 1 if a kernel of this plan gave up on a wait since the plan was created (its results are then not valid)
int seq_gemm_status(SeqGemmPlan* p, int* status);

}  // namespace seq
}  // namespace gtb
