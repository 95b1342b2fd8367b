// Host utilities: tensor-map encoder lookup, SM count cache, device error word.
#include "host_util.h"
#include "sm100.cuh"

#include <mutex>

namespace sb {

unsigned int* error_word() {
  static unsigned int* words[64] = {nullptr};
  static std::mutex mu;
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  std::lock_guard<std::mutex> lock(mu);
  if (!words[dev]) {
    unsigned int* p = nullptr;
    if (cudaMalloc(&p, sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(p, 0, sizeof(unsigned int));
    words[dev] = p;
  }
  return words[dev];
}

PFN_encodeTiled get_encode_fn() {
  static PFN_encodeTiled fn = nullptr;
  static std::once_flag once;
  std::call_once(once, [] {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
        q == cudaDriverEntryPointSuccess) {
      fn = reinterpret_cast<PFN_encodeTiled>(p);
    }
  });
  return fn;
}

int make_tmap(CUtensorMap* out, const void* base, int elem_bytes, int rank, const uint64_t* dims,
              const uint64_t* strides_bytes, const uint32_t* box, bool swizzle128, bool is_float32) {
  PFN_encodeTiled enc = get_encode_fn();
  if (!enc) {
    fprintf(stderr, "summa_b200: cuTensorMapEncodeTiled entry point not found\n");
    return SB_ERR_TMAP;
  }
  if ((reinterpret_cast<uintptr_t>(base) & 15) != 0) {
    fprintf(stderr, "summa_b200: TMA base %p is not 16-byte aligned\n", base);
    return SB_ERR_ARG;
  }
  cuuint64_t gdims[5];
  cuuint64_t gstrides[4];
  cuuint32_t gbox[5];
  cuuint32_t estr[5];
  for (int i = 0; i < rank; ++i) {
    gdims[i] = dims[i];
    gbox[i] = box[i];
    estr[i] = 1;
    if (i + 1 < rank) {
      gstrides[i] = strides_bytes[i];
      if (gstrides[i] % 16 != 0) {
        fprintf(stderr, "summa_b200: TMA stride %llu (dim %d) is not a multiple of 16 bytes\n",
                (unsigned long long)gstrides[i], i + 1);
        return SB_ERR_ARG;
      }
    }
  }
  CUtensorMapDataType dt = elem_bytes == 2 ? CU_TENSOR_MAP_DATA_TYPE_BFLOAT16
                           : elem_bytes == 4 ? (is_float32 ? CU_TENSOR_MAP_DATA_TYPE_FLOAT32 : CU_TENSOR_MAP_DATA_TYPE_UINT32)
                                             : CU_TENSOR_MAP_DATA_TYPE_UINT8;
  CUresult r = enc(out, dt, rank, const_cast<void*>(base), gdims, gstrides, gbox, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                   swizzle128 ? CU_TENSOR_MAP_SWIZZLE_128B : CU_TENSOR_MAP_SWIZZLE_NONE,
                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
  if (r != CUDA_SUCCESS) {
    fprintf(stderr, "summa_b200: cuTensorMapEncodeTiled failed (%d): rank %d dims [%llu,%llu] box [%u,%u]\n", (int)r,
            rank, (unsigned long long)gdims[0], (unsigned long long)(rank > 1 ? gdims[1] : 0), gbox[0],
            rank > 1 ? gbox[1] : 0);
    return SB_ERR_TMAP;
  }
  return SB_OK;
}

int num_sms() {
  static int cached[64] = {0};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
  if (cached[dev] == 0) {
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    cached[dev] = n;
  }
  return cached[dev];
}

}  // namespace sb

// Reads and clears the device error word (bit 1: mbarrier timeout, bit 2: peer flag
// timeout, bit 4: bad argument seen on device). Synchronises the device.
extern "C" int sb_read_error_flag(unsigned int* out) {
  unsigned int v = 0;
  unsigned int* w = sb::error_word();
  if (!w) return sb::SB_ERR_CUDA;
  SB_CHECK_CUDA(cudaDeviceSynchronize());
  SB_CHECK_CUDA(cudaMemcpy(&v, w, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) SB_CHECK_CUDA(cudaMemset(w, 0, sizeof(v)));
  *out = v;
  return sb::SB_OK;
}

extern "C" int sb_num_sms() { return sb::num_sms(); }

// Binds `dev`'s primary context to the calling thread for this library's runtime.
// Threads that never made a runtime call (autograd worker threads) have no current
// context, and tensor-map encoding needs one.
extern "C" int sb_set_device(int dev) {
  SB_CHECK_CUDA(cudaSetDevice(dev));
  SB_CHECK_CUDA(cudaFree(nullptr));
  return sb::SB_OK;
}
