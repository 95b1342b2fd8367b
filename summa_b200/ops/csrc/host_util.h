// Host-side helpers shared by the launchers: TMA tensor-map encoding through the
// driver entry point (no link-time dependency on libcuda), the device error word,
// and the argument-check macro that turns a bad call into a negative return code.
#pragma once
#include <cuda.h>
#include <cuda_runtime.h>
#include <stdint.h>
#include <stdio.h>

namespace sb {

enum : int {
  SB_OK = 0,
  SB_ERR_ARG = -1,        // shape / alignment / dtype rejected on the host
  SB_ERR_CUDA = -2,       // a CUDA runtime call failed
  SB_ERR_TMAP = -3,       // cuTensorMapEncodeTiled rejected the layout
  SB_ERR_TOO_LARGE = -4,  // exceeds a documented capacity
};

#define SB_CHECK_ARG(cond)                                                             \
  do {                                                                                 \
    if (!(cond)) {                                                                     \
      fprintf(stderr, "summa_b200: argument check failed: %s (%s:%d)\n", #cond, __FILE__, __LINE__); \
      return sb::SB_ERR_ARG;                                                           \
    }                                                                                  \
  } while (0)

#define SB_CHECK_CUDA(expr)                                                            \
  do {                                                                                 \
    cudaError_t _e = (expr);                                                           \
    if (_e != cudaSuccess) {                                                           \
      fprintf(stderr, "summa_b200: %s failed: %s (%s:%d)\n", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
      return sb::SB_ERR_CUDA;                                                          \
    }                                                                                  \
  } while (0)

typedef CUresult (*PFN_encodeTiled)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*,
                                    const cuuint64_t*, const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

PFN_encodeTiled get_encode_fn();

// Tiled tensor map over a row-major tensor of `rank` dims. dims/box are given
// innermost-first; strides_bytes[i] is the byte stride of dim i+1 (rank-1 entries).
// elem: 2 = bf16, 4 = fp32, 1 = uint8. swizzle128: 128-byte swizzle (inner box must
// span exactly 128 bytes) or none.
int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128, bool is_float32 = false);

inline int make_tmap_2d(CUtensorMap* out, const void* base, int elem_bytes, uint64_t inner, uint64_t outer,
                        uint64_t row_pitch_bytes, uint32_t box_inner, uint32_t box_outer, bool swizzle128,
                        bool is_float32 = false) {
  uint64_t dims[2] = {inner, outer};
  uint64_t strides[1] = {row_pitch_bytes};
  uint32_t box[2] = {box_inner, box_outer};
  return make_tmap(out, base, elem_bytes, 2, dims, strides, box, swizzle128, is_float32);
}

int num_sms();

// Device error word of the current device (lazily allocated once per device).
unsigned int* error_word();

}  // namespace sb
