// Paired-CTA (tcgen05 cta_group::2) bf16 GEMM, see gemm_pair.cu. Same contract as
// sb_gemm_bf16: operand layouts, leading dimensions in elements, out_mode 0 bf16 store,
// 1 fp32 store, 2 fp32 accumulate.
#pragma once
#include "host_util.h"

namespace sb {

int gemm_pair_bf16(const void* A, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N, int K,
                   int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode, cudaStream_t stream, int batch = 1,
                   long stride_a = 0, long stride_b = 0, long stride_c = 0);

}  // namespace sb
