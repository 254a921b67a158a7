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

}  // namespace seq
}  // namespace gtb
