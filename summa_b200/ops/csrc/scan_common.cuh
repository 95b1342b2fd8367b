// Pieces shared by the selective-scan forward and backward kernels.
#pragma once
#include "sm100.cuh"

namespace sb {

// Steps per segment = spacing of the state checkpoints the forward pass keeps for the backward pass.
constexpr int SCAN_SEG = 16;

// Raw bf16 inputs of one segment are fetched with 16-byte asynchronous copies while the previous segment is
// being computed (`vec` = every row start and stride is 16-byte aligned; otherwise plain scalar loads fill the
// same staging buffer). A chunk outside the tensor is zero-filled.
__device__ __forceinline__ void scan_stage_rows(uint32_t dst_smem, __nv_bfloat16* dst, const __nv_bfloat16* src,
                                                long ld, long row0, int rows_valid, int rows, int col0, int cols,
                                                int cols_valid, bool vec, int tid, int nthreads) {
  const int cpr = cols / 8;            // 16-byte chunks per row
  for (int i = tid; i < rows * cpr; i += nthreads) {
    const int r = i / cpr, k = i - r * cpr;
    const bool ok = r < rows_valid && 8 * k < cols_valid;
    const __nv_bfloat16* g = src + (ok ? (row0 + r) * ld + col0 + 8 * k : 0);
    if (vec) {
      cp_async16_zfill(dst_smem + (uint32_t)(r * cols + 8 * k) * 2u, g, ok ? 16 : 0);
    } else {
#pragma unroll
      for (int e = 0; e < 8; ++e)
        dst[r * cols + 8 * k + e] = (ok && 8 * k + e < cols_valid) ? g[e] : __float2bfloat16(0.f);
    }
  }
}

}  // namespace sb
