// Group-quantised 4-bit weights (group 128 along the input dimension, bf16 scales).
//   packed `[K/2, N]` uint8: byte (k2, n) holds k = 2*k2 in the low nibble and k = 2*k2+1
//   in the high nibble, code q in [0, 15] meaning (q - 8) * scale[k / 128, n].
// Kernels:
//   int4_gemv      y[M,N] (+)= x[M,K] @ dequant(W) for decode-sized M (<= 8 rows per pass),
//                  split over K across blocks (fp32 atomics into a zeroed accumulator) so
//                  that even a tensor-parallel weight shard fills the GPU; the weight is
//                  read exactly once per pass in 4-byte lanes (coalesced along N)
//   int4_finish    accumulator -> bf16 (+ optional residual)
//   int4_dequant   packed -> bf16 `[K, N]` for the prefill path (tensor-core GEMM)
//   argmax_rows    greedy sampling: argmax over the vocabulary per row
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int GV_KSLICE = 512;     // k range per block (4 groups)
constexpr int GV_MAXM = 8;

// grid: (ceil(N / 512), K / GV_KSLICE, ceil(M / 8)); block 128 threads, thread = 4 columns
__global__ void __launch_bounds__(128)
int4_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ packed,
                 const __nv_bfloat16* __restrict__ scales, float* __restrict__ acc_out, int M, int N, int K, long ldx) {
  __shared__ float xs[GV_MAXM][GV_KSLICE];
  const int n0 = (blockIdx.x * 128 + threadIdx.x) * 4;
  const int k0 = blockIdx.y * GV_KSLICE;
  const int m0 = blockIdx.z * GV_MAXM;
  const int mrows = min(GV_MAXM, M - m0);
  for (int i = threadIdx.x; i < GV_MAXM * GV_KSLICE; i += 128) {
    const int m = i / GV_KSLICE, k = i % GV_KSLICE;
    xs[m][k] = (m < mrows && k0 + k < K) ? __bfloat162float(x[(long)(m0 + m) * ldx + k0 + k]) : 0.f;
  }
  __syncthreads();
  if (n0 >= N) return;
  float acc[GV_MAXM][4];
#pragma unroll
  for (int m = 0; m < GV_MAXM; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[m][c] = 0.f;
  const int kend = min(GV_KSLICE, K - k0);
  for (int g0 = 0; g0 < kend; g0 += 128) {
    float part[GV_MAXM][4];
#pragma unroll
    for (int m = 0; m < GV_MAXM; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) part[m][c] = 0.f;
    const uint8_t* wp = packed + (long)((k0 + g0) >> 1) * N + n0;
#pragma unroll 4
    for (int k2 = 0; k2 < 64; ++k2) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(wp + (long)k2 * N);
      const int kk = g0 + 2 * k2;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t byte = (w >> (8 * c)) & 0xffu;
        const float lo = static_cast<float>(static_cast<int>(byte & 15u) - 8);
        const float hi = static_cast<float>(static_cast<int>(byte >> 4) - 8);
#pragma unroll
        for (int m = 0; m < GV_MAXM; ++m) part[m][c] = fmaf(xs[m][kk], lo, fmaf(xs[m][kk + 1], hi, part[m][c]));
      }
    }
    const uint2 sv = *reinterpret_cast<const uint2*>(scales + (long)((k0 + g0) >> 7) * N + n0);
    const float sc[4] = {bf16_lo(sv.x), bf16_hi(sv.x), bf16_lo(sv.y), bf16_hi(sv.y)};
#pragma unroll
    for (int m = 0; m < GV_MAXM; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[m][c] = fmaf(part[m][c], sc[c], acc[m][c]);
  }
  for (int m = 0; m < mrows; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) atomicAdd(acc_out + (long)(m0 + m) * N + n0 + c, acc[m][c]);
}

__global__ void int4_finish_kernel(const float* __restrict__ acc, const __nv_bfloat16* __restrict__ residual,
                                   __nv_bfloat16* __restrict__ y, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float v = acc[i];
    if (residual) v += __bfloat162float(residual[i]);
    y[i] = __float2bfloat16(v);
  }
}

// thread = 4 columns x 2 rows (one packed word)
__global__ void int4_dequant_kernel(const uint8_t* __restrict__ packed, const __nv_bfloat16* __restrict__ scales,
                                    __nv_bfloat16* __restrict__ out, int K, int N) {
  const long total = (long)(K / 2) * (N / 4);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int k2 = i / (N / 4);
    const int n0 = (i - (long)k2 * (N / 4)) * 4;
    const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + (long)k2 * N + n0);
    const uint2 sv = *reinterpret_cast<const uint2*>(scales + (long)((2 * k2) >> 7) * N + n0);
    const float sc[4] = {bf16_lo(sv.x), bf16_hi(sv.x), bf16_lo(sv.y), bf16_hi(sv.y)};
    float lo[4], hi[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t byte = (w >> (8 * c)) & 0xffu;
      lo[c] = static_cast<float>(static_cast<int>(byte & 15u) - 8) * sc[c];
      hi[c] = static_cast<float>(static_cast<int>(byte >> 4) - 8) * sc[c];
    }
    *reinterpret_cast<uint2*>(out + (long)(2 * k2) * N + n0) = make_uint2(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]));
    *reinterpret_cast<uint2*>(out + (long)(2 * k2 + 1) * N + n0) = make_uint2(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
  }
}

// one block per row: argmax over `vocab` logits (fp32 or bf16), lowest index wins ties
template <typename T>
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const T* __restrict__ logits, long* __restrict__ out, int vocab, long ld) {
  const T* row = logits + (long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += 256) {
    const float v = static_cast<float>(row[i]);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  __shared__ float sb_[8];
  __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sb_[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sb_[w] > best || (sb_[w] == best && si[w] < bi)) { best = sb_[w]; bi = si[w]; }
    out[blockIdx.x] = bi;
  }
}

}  // namespace sb

using namespace sb;

// y[M,N] = x[M,K] @ dequant(packed, scales) (+ residual). acc: fp32 scratch `[M, N]`.
// M <= 64, K % 128 == 0, N % 4 == 0.
extern "C" int sb_int4_gemv(const void* x, const void* packed, const void* scales, float* acc, const void* residual,
                            void* y, int M, int N, int K, long ldx, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 64 && K % 128 == 0 && N % 4 == 0 && N > 0);
  SB_CHECK_CUDA(cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)M * N, st));
  dim3 grid((N + 511) / 512, (K + GV_KSLICE - 1) / GV_KSLICE, (M + GV_MAXM - 1) / GV_MAXM);
  int4_gemv_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, (const uint8_t*)packed, (const __nv_bfloat16*)scales,
                                         acc, M, N, K, ldx);
  const long n = (long)M * N;
  int4_finish_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(acc, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, n);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_int4_dequant(const void* packed, const void* scales, void* out, int K, int N, cudaStream_t st) {
  SB_CHECK_ARG(K % 128 == 0 && N % 4 == 0);
  const long total = (long)(K / 2) * (N / 4);
  long blocks = (total + 255) / 256;
  if (blocks > num_sms() * 16L) blocks = num_sms() * 16L;
  int4_dequant_kernel<<<(int)blocks, 256, 0, st>>>((const uint8_t*)packed, (const __nv_bfloat16*)scales,
                                                   (__nv_bfloat16*)out, K, N);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_argmax_rows(const void* logits, long* out, int rows, int vocab, long ld, int is_bf16, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && vocab > 0);
  if (is_bf16) argmax_rows_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((const __nv_bfloat16*)logits, out, vocab, ld);
  else argmax_rows_kernel<float><<<rows, 256, 0, st>>>((const float*)logits, out, vocab, ld);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
