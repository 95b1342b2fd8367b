// HQUANT binary / ternary group codes: groups of 128 over the FLATTENED tensor, one fp16
// scale per group (codec: `summa-train/src/quantization.rs:447-501,691-771`).
//   binary   1 bit / weight, LSB first, bit 1 -> +scale, bit 0 -> -scale, scale = mean |w|
//   ternary  2 bits / weight, code 0 -> -scale, 1 -> 0, 2 -> +scale; scale and support are
//            the L2-optimal prefix of the magnitudes sorted in descending order
// Kernels:
//   fake_quant     quantise-dequantise in one pass for quantisation-aware training (the
//                  straight-through estimator lives in the autograd wrapper): one warp per
//                  group, 4 elements per lane; the ternary form sorts the 128 magnitudes with a
//                  register/shuffle bitonic network, scans them and picks the best prefix
//   hquant_dequant codes -> bf16 / fp32 (prefill path and host-oracle parity)
//   hquant_gemv    y[M,N] = x[M,K] @ decode(W) for decode-sized M straight from the codes
//                  (N % 128 == 0, so a group never straddles two rows of W); split over K with
//                  fp32 atomics, the weight is read once per pass of 4 rows of x
#include <cuda_fp16.h>

#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int HQ_BINARY = 0;
constexpr int HQ_TERNARY = 1;

template <typename T> __device__ __forceinline__ float hq_load(const T* p, long i);
template <> __device__ __forceinline__ float hq_load<float>(const float* p, long i) { return p[i]; }
template <> __device__ __forceinline__ float hq_load<__nv_bfloat16>(const __nv_bfloat16* p, long i) {
  return __bfloat162float(p[i]);
}
template <typename T> __device__ __forceinline__ void hq_store(T* p, long i, float v);
template <> __device__ __forceinline__ void hq_store<float>(float* p, long i, float v) { p[i] = v; }
template <> __device__ __forceinline__ void hq_store<__nv_bfloat16>(__nv_bfloat16* p, long i, float v) {
  p[i] = __float2bfloat16(v);
}

// Descending bitonic sort of 128 values held 4 per lane (element index = 4 * lane + slot).
__device__ __forceinline__ void bitonic128_desc(float (&v)[4], int lane) {
#pragma unroll
  for (int k = 2; k <= 128; k <<= 1) {
#pragma unroll
    for (int j = k >> 1; j > 0; j >>= 1) {
      if (j >= 4) {
        const int lj = j >> 2;
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int i = 4 * lane + s;
          const float o = __shfl_xor_sync(0xffffffffu, v[s], lj);
          const bool keep_max = ((i & k) == 0) == ((i & j) == 0);
          v[s] = keep_max ? fmaxf(v[s], o) : fminf(v[s], o);
        }
      } else {
#pragma unroll
        for (int s = 0; s < 4; ++s) {
          const int p = s ^ j;
          if (p > s) {
            const int i = 4 * lane + s;
            const bool first_max = (i & k) == 0;       // slot s is the lower index of the pair
            const float a = v[s], b = v[p];
            v[s] = first_max ? fmaxf(a, b) : fminf(a, b);
            v[p] = first_max ? fminf(a, b) : fmaxf(a, b);
          }
        }
      }
    }
  }
}

// grid-stride over groups, one warp per group
template <typename T, int FMT>
__global__ void __launch_bounds__(256) fake_quant_kernel(const T* __restrict__ w, T* __restrict__ out, long n) {
  const int lane = threadIdx.x & 31;
  const long groups = (n + 127) >> 7;
  const long warp0 = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const long nwarps = ((long)gridDim.x * blockDim.x) >> 5;
  for (long g = warp0; g < groups; g += nwarps) {
    const long base = (g << 7) + 4 * lane;
    float x[4];
#pragma unroll
    for (int s = 0; s < 4; ++s) x[s] = base + s < n ? hq_load<T>(w, base + s) : 0.f;
    float scale, thresh;
    if (FMT == HQ_BINARY) {
      const long real = min(128L, n - (g << 7));
      scale = warp_sum(fabsf(x[0]) + fabsf(x[1]) + fabsf(x[2]) + fabsf(x[3])) / static_cast<float>(real);
      thresh = 0.f;
    } else {
      float m[4] = {fabsf(x[0]), fabsf(x[1]), fabsf(x[2]), fabsf(x[3])};
      bitonic128_desc(m, lane);
      // inclusive prefix sums in sorted order
      float c[4];
      c[0] = m[0]; c[1] = c[0] + m[1]; c[2] = c[1] + m[2]; c[3] = c[2] + m[3];
      float tot = c[3];
#pragma unroll
      for (int o = 1; o < 32; o <<= 1) {
        const float up = __shfl_up_sync(0xffffffffu, tot, o);
        if (lane >= o) tot += up;
      }
      const float excl = tot - c[3];
      float best = -1.f;
      int bi = 0;
#pragma unroll
      for (int s = 0; s < 4; ++s) {
        c[s] += excl;
        const float gain = c[s] * c[s] / static_cast<float>(4 * lane + s + 1);
        if (gain > best) { best = gain; bi = 4 * lane + s; }
      }
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float ob = __shfl_xor_sync(0xffffffffu, best, o);
        const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
        if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
      }
      const int slot = bi & 3;
      const float csel = slot == 0 ? c[0] : slot == 1 ? c[1] : slot == 2 ? c[2] : c[3];
      const float msel = slot == 0 ? m[0] : slot == 1 ? m[1] : slot == 2 ? m[2] : m[3];
      scale = __shfl_sync(0xffffffffu, csel, bi >> 2) / static_cast<float>(bi + 1);
      thresh = __shfl_sync(0xffffffffu, msel, bi >> 2);
    }
#pragma unroll
    for (int s = 0; s < 4; ++s) {
      if (base + s >= n) continue;
      float q;
      if (FMT == HQ_BINARY) q = x[s] >= 0.f ? scale : -scale;
      else q = (x[s] != 0.f && fabsf(x[s]) >= thresh) ? copysignf(scale, x[s]) : 0.f;
      hq_store<T>(out, base + s, q);
    }
  }
}

// thread = 8 consecutive elements (one binary code byte / two ternary code bytes)
template <typename T, int FMT>
__global__ void __launch_bounds__(256)
hquant_dequant_kernel(const uint8_t* __restrict__ codes, const __half* __restrict__ scales, T* __restrict__ out, long n) {
  const long n8 = (n + 7) >> 3;
  for (long t = blockIdx.x * (long)blockDim.x + threadIdx.x; t < n8; t += (long)gridDim.x * blockDim.x) {
    const float s = __half2float(scales[t >> 4]);
    uint32_t c;
    if (FMT == HQ_BINARY) c = codes[t];
    else c = codes[2 * t] | (static_cast<uint32_t>(codes[2 * t + 1]) << 8);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const long i = 8 * t + j;
      if (i >= n) break;
      float v;
      if (FMT == HQ_BINARY) v = ((c >> j) & 1u) ? s : -s;
      else { const uint32_t q = (c >> (2 * j)) & 3u; v = q == 2u ? s : (q == 0u ? -s : 0.f); }
      hq_store<T>(out, i, v);
    }
  }
}

constexpr int HG_KSLICE = 128;
constexpr int HG_MAXM = 4;
constexpr int HG_THREADS = 64;

// grid: (ceil(N / 512), ceil(K / 128), ceil(M / 4)); thread = 8 columns
template <int FMT>
__global__ void __launch_bounds__(HG_THREADS)
hquant_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ codes,
                   const __half* __restrict__ scales, float* __restrict__ acc_out, int M, int N, int K, long ldx) {
  __shared__ float xs[HG_MAXM][HG_KSLICE];
  const int n0 = (blockIdx.x * HG_THREADS + threadIdx.x) * 8;
  const int k0 = blockIdx.y * HG_KSLICE;
  const int m0 = blockIdx.z * HG_MAXM;
  const int mrows = min(HG_MAXM, M - m0);
  for (int i = threadIdx.x; i < HG_MAXM * HG_KSLICE; i += HG_THREADS) {
    const int m = i / HG_KSLICE, k = i % HG_KSLICE;
    xs[m][k] = (m < mrows && k0 + k < K) ? __bfloat162float(x[(long)(m0 + m) * ldx + k0 + k]) : 0.f;
  }
  __syncthreads();
  if (n0 >= N) return;
  float acc[HG_MAXM][8];
#pragma unroll
  for (int m = 0; m < HG_MAXM; ++m)
#pragma unroll
    for (int c = 0; c < 8; ++c) acc[m][c] = 0.f;
  const int kend = min(HG_KSLICE, K - k0);
#pragma unroll 4
  for (int kk = 0; kk < kend; ++kk) {
    const long e = (long)(k0 + kk) * N + n0;                // flat element index of the first column
    const float s = __half2float(scales[e >> 7]);
    uint32_t c;
    if (FMT == HQ_BINARY) c = codes[e >> 3];
    else c = *reinterpret_cast<const uint16_t*>(codes + (e >> 2));
    float t[HG_MAXM];
#pragma unroll
    for (int m = 0; m < HG_MAXM; ++m) t[m] = xs[m][kk] * s;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      if (FMT == HQ_BINARY) {
        const uint32_t flip = ((~c >> j) & 1u) << 31;
#pragma unroll
        for (int m = 0; m < HG_MAXM; ++m) acc[m][j] += __uint_as_float(__float_as_uint(t[m]) ^ flip);
      } else {
        const uint32_t q = (c >> (2 * j)) & 3u;
        const float f = q == 2u ? 1.f : (q == 0u ? -1.f : 0.f);
#pragma unroll
        for (int m = 0; m < HG_MAXM; ++m) acc[m][j] = fmaf(t[m], f, acc[m][j]);
      }
    }
  }
  for (int m = 0; m < mrows; ++m)
#pragma unroll
    for (int j = 0; j < 8; ++j) atomicAdd(acc_out + (long)(m0 + m) * N + n0 + j, acc[m][j]);
}

__global__ void hquant_finish_kernel(const float* __restrict__ acc, const __nv_bfloat16* __restrict__ residual,
                                     __nv_bfloat16* __restrict__ y, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float v = acc[i];
    if (residual) v += __bfloat162float(residual[i]);
    y[i] = __float2bfloat16(v);
  }
}

}  // namespace sb

using namespace sb;

static int hq_blocks(long work_items, int per_block) {
  long b = (work_items + per_block - 1) / per_block;
  const long cap = num_sms() * 16L;
  return (int)(b < 1 ? 1 : (b > cap ? cap : b));
}

// out = dequant(quant(w)) with the codec's scale estimator. fmt: 0 binary, 1 ternary.
extern "C" int sb_fake_quant(const void* w, void* out, long n, int fmt, int is_bf16, cudaStream_t st) {
  SB_CHECK_ARG(n > 0 && (fmt == HQ_BINARY || fmt == HQ_TERNARY));
  const int blocks = hq_blocks((n + 127) / 128, 8);
  if (is_bf16) {
    if (fmt == HQ_BINARY) fake_quant_kernel<__nv_bfloat16, HQ_BINARY><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)out, n);
    else fake_quant_kernel<__nv_bfloat16, HQ_TERNARY><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)w, (__nv_bfloat16*)out, n);
  } else {
    if (fmt == HQ_BINARY) fake_quant_kernel<float, HQ_BINARY><<<blocks, 256, 0, st>>>((const float*)w, (float*)out, n);
    else fake_quant_kernel<float, HQ_TERNARY><<<blocks, 256, 0, st>>>((const float*)w, (float*)out, n);
  }
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// codes + fp16 scales -> n elements of bf16 (out_bf16 = 1) or fp32
extern "C" int sb_hquant_dequant(const void* codes, const void* scales, void* out, long n, int fmt, int out_bf16,
                                 cudaStream_t st) {
  SB_CHECK_ARG(n > 0 && (fmt == HQ_BINARY || fmt == HQ_TERNARY));
  const int blocks = hq_blocks((n + 7) / 8, 256);
  const uint8_t* c = (const uint8_t*)codes;
  const __half* s = (const __half*)scales;
  if (out_bf16) {
    if (fmt == HQ_BINARY) hquant_dequant_kernel<__nv_bfloat16, HQ_BINARY><<<blocks, 256, 0, st>>>(c, s, (__nv_bfloat16*)out, n);
    else hquant_dequant_kernel<__nv_bfloat16, HQ_TERNARY><<<blocks, 256, 0, st>>>(c, s, (__nv_bfloat16*)out, n);
  } else {
    if (fmt == HQ_BINARY) hquant_dequant_kernel<float, HQ_BINARY><<<blocks, 256, 0, st>>>(c, s, (float*)out, n);
    else hquant_dequant_kernel<float, HQ_TERNARY><<<blocks, 256, 0, st>>>(c, s, (float*)out, n);
  }
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// y[M,N] bf16 = x[M,K] @ decode(W[K,N]) (+ residual); acc: zeroed fp32 [M,N] scratch.
extern "C" int sb_hquant_gemv(const void* x, const void* codes, const void* scales, float* acc, const void* residual,
                              void* y, int M, int N, int K, long ldx, int fmt, cudaStream_t st) {
  SB_CHECK_ARG(M > 0 && K > 0 && N > 0 && N % 128 == 0 && (fmt == HQ_BINARY || fmt == HQ_TERNARY));
  dim3 grid((N + HG_THREADS * 8 - 1) / (HG_THREADS * 8), (K + HG_KSLICE - 1) / HG_KSLICE, (M + HG_MAXM - 1) / HG_MAXM);
  if (fmt == HQ_BINARY)
    hquant_gemv_kernel<HQ_BINARY><<<grid, HG_THREADS, 0, st>>>((const __nv_bfloat16*)x, (const uint8_t*)codes,
                                                               (const __half*)scales, acc, M, N, K, ldx);
  else
    hquant_gemv_kernel<HQ_TERNARY><<<grid, HG_THREADS, 0, st>>>((const __nv_bfloat16*)x, (const uint8_t*)codes,
                                                                (const __half*)scales, acc, M, N, K, ldx);
  const long n = (long)M * N;
  hquant_finish_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(acc, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, n);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// ---------------------------------------------------------------------------- W4 GEMV for 1..4 rows
// Batch-1..4 decode: y[M,N] = x[M,K] @ dequant(W) (+ residual) in ONE launch, no atomics, no
// accumulator pass. Weights in the k8-repacked form (`[K/8, N]` uint32, see quant.cu). A CTA owns
// 32 * CPL output columns and the whole K range: its 8 warps take the 128-k scale groups round
// robin, a lane holds CPL adjacent columns and issues 16 independent loads per group (the 16 k8
// rows), x sits in shared memory as bf16 and is read as broadcast 16-byte words, the warps'
// partial sums meet in shared memory, and the residual add and bf16 conversion happen in place.
namespace sb {

constexpr int WS_WARPS = 8;

template <int MR, int CPL>
__global__ void __launch_bounds__(WS_WARPS * 32)
w4_gemv_small_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ wk8,
                     const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ residual,
                     __nv_bfloat16* __restrict__ y, int M, int N, int K, long ldx) {
  extern __shared__ __align__(16) unsigned char ws_smem[];
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(ws_smem);                 // [MR][K]
  float* red = reinterpret_cast<float*>(ws_smem + (size_t)MR * K * 2);           // [WS_WARPS][MR][32 * CPL]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 32 * CPL + lane * CPL;
  // stage x (rows beyond M are zero)
  const int k8n = K >> 3;
  for (int i = threadIdx.x; i < MR * k8n; i += WS_WARPS * 32) {
    const int m = i / k8n, c = i - m * k8n;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < M) v = *reinterpret_cast<const uint4*>(x + (long)m * ldx + 8 * c);
    reinterpret_cast<uint4*>(xs + (size_t)m * K)[c] = v;
  }
  __syncthreads();
  float acc[MR][CPL];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPL; ++c) acc[m][c] = 0.f;
  const bool live = n0 < N;
  const int groups = K >> 7;
  for (int g = warp; g < groups; g += WS_WARPS) {
    // sum of x over the group (for the -8 offset of the codes): lanes split the 128 values
    float xsum[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      const uint2 v = reinterpret_cast<const uint2*>(xs + (size_t)m * K + 128 * g)[lane];
      xsum[m] = warp_sum(bf16_lo(v.x) + bf16_hi(v.x) + bf16_lo(v.y) + bf16_hi(v.y));
    }
    if (!live) continue;
    uint32_t w[16][CPL];
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const uint32_t* p = wk8 + (long)(16 * g + r) * N + n0;
      if (CPL == 4) { const uint4 t = *reinterpret_cast<const uint4*>(p); w[r][0] = t.x; w[r][1 % CPL] = t.y; w[r][2 % CPL] = t.z; w[r][3 % CPL] = t.w; }
      else if (CPL == 2) { const uint2 t = *reinterpret_cast<const uint2*>(p); w[r][0] = t.x; w[r][1 % CPL] = t.y; }
      else w[r][0] = *p;
    }
    float sc[CPL];
#pragma unroll
    for (int c = 0; c < CPL; ++c) sc[c] = __bfloat162float(scales[(long)g * N + n0 + c]);
    float part[MR][CPL];
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int c = 0; c < CPL; ++c) part[m][c] = 0.f;
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      float xv[MR][8];
#pragma unroll
      for (int m = 0; m < MR; ++m) {
        const uint4 v = reinterpret_cast<const uint4*>(xs + (size_t)m * K + 128 * g)[r];      // broadcast
        xv[m][0] = bf16_lo(v.x); xv[m][1] = bf16_hi(v.x); xv[m][2] = bf16_lo(v.y); xv[m][3] = bf16_hi(v.y);
        xv[m][4] = bf16_lo(v.z); xv[m][5] = bf16_hi(v.z); xv[m][6] = bf16_lo(v.w); xv[m][7] = bf16_hi(v.w);
      }
#pragma unroll
      for (int c = 0; c < CPL; ++c) {
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint32_t pr = ((w[r][c] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;      // bf16 pair (128 + q)
          const float q0 = __uint_as_float(pr << 16), q1 = __uint_as_float(pr & 0xFFFF0000u);
#pragma unroll
          for (int m = 0; m < MR; ++m) part[m][c] = fmaf(xv[m][2 * i], q0, fmaf(xv[m][2 * i + 1], q1, part[m][c]));
        }
      }
    }
#pragma unroll
    for (int m = 0; m < MR; ++m)
#pragma unroll
      for (int c = 0; c < CPL; ++c) acc[m][c] = fmaf(part[m][c] - 136.f * xsum[m], sc[c], acc[m][c]);
  }
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPL; ++c) red[(warp * MR + m) * 32 * CPL + lane * CPL + c] = acc[m][c];
  __syncthreads();
  for (int i = threadIdx.x; i < MR * 32 * CPL; i += WS_WARPS * 32) {
    const int m = i / (32 * CPL), c = i - m * 32 * CPL;
    const int n = blockIdx.x * 32 * CPL + c;
    if (m >= M || n >= N) continue;
    float v = 0.f;
#pragma unroll
    for (int wq = 0; wq < WS_WARPS; ++wq) v += red[(wq * MR + m) * 32 * CPL + c];
    if (residual) v += __bfloat162float(residual[(long)m * N + n]);
    y[(long)m * N + n] = __float2bfloat16(v);
  }
}

template <int MR, int CPL>
static int launch_w4_small(const void* x, const void* wk8, const void* scales, const void* residual, void* y, int M,
                           int N, int K, long ldx, cudaStream_t st) {
  const size_t smem = (size_t)MR * K * 2 + (size_t)WS_WARPS * MR * 32 * CPL * 4;
  auto kern = w4_gemv_small_kernel<MR, CPL>;
  static size_t allowed = 48 * 1024;          // per instantiation: raise the dynamic shared memory limit once
  if (smem > allowed) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    allowed = 200 * 1024;
  }
  const int grid = (N + 32 * CPL - 1) / (32 * CPL);
  kern<<<grid, WS_WARPS * 32, smem, st>>>((const __nv_bfloat16*)x, (const uint32_t*)wk8, (const __nv_bfloat16*)scales,
                                          (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, M, N, K, ldx);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

// y[M,N] bf16 = x[M,K] @ dequant(k8-repacked int4 g128 weights) (+ residual), M <= 4, K % 128 == 0,
// N % 4 == 0, x rows 16-byte aligned. One launch.
extern "C" int sb_w4_gemv_small(const void* x, const void* wk8, const void* scales, const void* residual, void* y,
                                int M, int N, int K, long ldx, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 4 && K > 0 && K % 128 == 0 && N > 0 && N % 4 == 0 && ldx % 8 == 0);
  SB_CHECK_ARG((size_t)4 * K * 2 + 8 * 4 * 128 * 4 <= 200 * 1024);
  // columns per lane: wide loads when there are enough columns to fill the GPU with CTAs
  const int sms = sb::num_sms();
  const int cpl = (N / 128 >= 2 * sms) ? 4 : ((N / 64 >= sms && N % 64 == 0) ? 2 : 1);
  // a ragged tail of columns is handled by the `live` / bounds tests (lanes past N idle)
  const int mr = M <= 1 ? 1 : (M <= 2 ? 2 : 4);
#define SB_W4S(MR, CPL) return sb::launch_w4_small<MR, CPL>(x, wk8, scales, residual, y, M, N, K, ldx, st)
  if (cpl == 4) { if (mr == 1) SB_W4S(1, 4); if (mr == 2) SB_W4S(2, 4); SB_W4S(4, 4); }
  if (cpl == 2) { if (mr == 1) SB_W4S(1, 2); if (mr == 2) SB_W4S(2, 2); SB_W4S(4, 2); }
  if (mr == 1) SB_W4S(1, 1);
  if (mr == 2) SB_W4S(2, 1);
  SB_W4S(4, 1);
#undef SB_W4S
}

// ---------------------------------------------------------------------------- W4 GEMV, K split over a cluster
// Same product, but the K range of a column block is cut over the CTAs of a thread-block cluster
// (up to 8), so that a 4096-column projection puts ~30 warps on every SM instead of 8. Each CTA
// streams its K slice (4 warps, scale groups round robin, the next group's 16 loads are issued
// before the current group is consumed), the slices meet through distributed shared memory in the
// cluster's first CTA, which adds the residual and writes bf16. Optional fused RMSNorm of x: the
// CTAs exchange their partial sums of squares over the cluster and scale their slice by
// rstd * gamma (rounded to bf16, as the separate norm kernel would) before the product.
#include <cooperative_groups.h>

namespace sb {
namespace cg = cooperative_groups;

constexpr int WC_WARPS = 4;

// Epilogue of the qkv projection of a decode step: rotary embedding at the device-side position and
// the append of k / v to the cache, as the separate kernel of `attention_decode.cu` does them.
struct RopeAppend {
  const float* cos_t;      // [max_pos, D/2]; null = plain epilogue
  const float* sin_t;
  __nv_bfloat16* kc;       // caches `[B, cap, Hkv, D]` addressed through the strides below
  __nv_bfloat16* vc;
  const int* pos_ptr;
  int Hq, Hkv, D, cap;
  long c_sb, c_ss, c_sh;
};

// Row-parallel projection of a tensor-parallel decode step: the all-reduce of the partial outputs happens
// in this kernel's epilogue over NVLink peer memory. The CTA that owns a block of output columns stores its
// fp32 partial into slot [rank] of EVERY rank's inbox, raises that block's flag on every rank, waits
// (bounded) for the block's flags of all ranks and sums the slots in rank order (bit-identical on all
// ranks), adds the residual and writes bf16. No grid-wide barrier: blocks finish independently. Inboxes are
// double buffered by call parity; the call number lives in device memory (graph replay).
constexpr int AR_MAX_RANKS = 8;
struct ArFuse {
  float* inbox[AR_MAX_RANKS];        // every rank's inbox: [2 parities][world][4 rows][n_pad] fp32
  uint32_t* flags[AR_MAX_RANKS];     // every rank's flags: [column block][AR_MAX_RANKS]
  unsigned int* epoch_word;          // call number (device, owned by the kernel)
  unsigned int* counter;             // CTA arrival counter for the epoch bump
  unsigned int* err;
  int rank, world;                   // world == 0: plain epilogue
  long n_pad;
};

// GATED (CPL = 2 only): W is `[K, 2I]` = [gate | value]; a lane's two columns are n and I + n and the
// output is silu(gate) * value, `[M, I]` (the SwiGLU of a decode step without its own launch).
template <int MR, int CPL, bool GATED>
__global__ void __launch_bounds__(WC_WARPS * 32)
w4_gemv_cluster_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ wk8,
                       const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ residual,
                       __nv_bfloat16* __restrict__ y, int M, int N, int K, long ldx, int gpc,
                       const float* __restrict__ gamma, float eps, const RopeAppend rope, const ArFuse ar) {
  extern __shared__ __align__(16) unsigned char wc_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();
  const int crank = (int)cluster.block_rank();
  const int groups = K >> 7;
  const int g_lo = crank * gpc, g_hi = min(groups, g_lo + gpc);
  const int kslice = gpc * 128;
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(wc_smem);                          // [MR][kslice]
  float* red = reinterpret_cast<float*>(wc_smem + (size_t)MR * kslice * 2);               // [WC_WARPS][MR][32*CPL]
  float* part = red + WC_WARPS * MR * 32 * CPL;                                           // [MR][32*CPL]
  float* ssq = part + MR * 32 * CPL;                                                      // [MR] (+pad)
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = GATED ? blockIdx.x * 32 + lane : blockIdx.x * 32 * CPL + lane * CPL;
  const int cstride = GATED ? (N >> 1) : 1;                                               // distance of a lane's columns
  const int kbase = g_lo * 128;
  const int k8n = max(0, (g_hi - g_lo) * 16);                                             // 8-element chunks in my slice
  const bool live = n0 < (GATED ? (N >> 1) : N);
  uint32_t wcur[16][CPL], wnxt[16][CPL];
  auto load_group = [&](uint32_t (&w)[16][CPL], int g) {
#pragma unroll
    for (int r = 0; r < 16; ++r) {
      const uint32_t* p = wk8 + (long)(16 * g + r) * N + n0;
      if (GATED) { w[r][0] = __ldcs(p); w[r][1 % CPL] = __ldcs(p + cstride); }
      else if (CPL == 4) { const uint4 t = __ldcs(reinterpret_cast<const uint4*>(p)); w[r][0] = t.x; w[r][1 % CPL] = t.y; w[r][2 % CPL] = t.z; w[r][3 % CPL] = t.w; }
      else if (CPL == 2) { const uint2 t = __ldcs(reinterpret_cast<const uint2*>(p)); w[r][0] = t.x; w[r][1 % CPL] = t.y; }
      else w[r][0] = __ldcs(p);
    }
  };
  // The weights do not depend on the preceding kernel: under programmatic dependent launch the first
  // group is already on its way while that kernel finishes; x is only read after the wait.
  asm volatile("griddepcontrol.launch_dependents;");
  int g = g_lo + warp;
  if (live && g < g_hi) load_group(wcur, g);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // the previous call of this kernel has completed (and bumped the call number) once the wait returns
  const uint32_t ar_epoch = ar.world > 1 ? *reinterpret_cast<volatile unsigned int*>(ar.epoch_word) + 1u : 0u;
  // ---- stage my slice of x; with a fused norm also its sum of squares
  float sq[MR];
#pragma unroll
  for (int m = 0; m < MR; ++m) sq[m] = 0.f;
  for (int i = threadIdx.x; i < MR * k8n; i += WC_WARPS * 32) {
    const int m = i / k8n, c = i - m * k8n;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < M) v = *reinterpret_cast<const uint4*>(x + (long)m * ldx + kbase + 8 * c);
    reinterpret_cast<uint4*>(xs + (size_t)m * kslice)[c] = v;
    if (gamma != nullptr) {
      const float a0 = bf16_lo(v.x), a1 = bf16_hi(v.x), a2 = bf16_lo(v.y), a3 = bf16_hi(v.y);
      const float a4 = bf16_lo(v.z), a5 = bf16_hi(v.z), a6 = bf16_lo(v.w), a7 = bf16_hi(v.w);
      const float s = a0 * a0 + a1 * a1 + a2 * a2 + a3 * a3 + a4 * a4 + a5 * a5 + a6 * a6 + a7 * a7;
#pragma unroll
      for (int mm = 0; mm < MR; ++mm) if (mm == m) sq[mm] += s;
    }
  }
  if (gamma != nullptr) {
    if (threadIdx.x < MR) ssq[threadIdx.x] = 0.f;
    __syncthreads();
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      const float s = warp_sum(sq[m]);
      if (lane == 0) atomicAdd(&ssq[m], s);
    }
    cluster.sync();                                   // every CTA's partial sum of squares is in its `ssq`
    float rstd[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      float t = 0.f;
      for (int r = 0; r < S; ++r) t += cluster.map_shared_rank(ssq, r)[m];
      rstd[m] = rsqrtf(t / static_cast<float>(K) + eps);
    }
    for (int i = threadIdx.x; i < MR * k8n * 4; i += WC_WARPS * 32) {       // pairs of elements
      const int m = i / (k8n * 4), c = i - m * (k8n * 4);
      uint32_t* p = reinterpret_cast<uint32_t*>(xs + (size_t)m * kslice) + c;
      const uint32_t v = *p;
      const float2 gm = *reinterpret_cast<const float2*>(gamma + kbase + 2 * c);
      float r = 0.f;
#pragma unroll
      for (int mm = 0; mm < MR; ++mm) if (mm == m) r = rstd[mm];
      *p = pack_bf16(bf16_lo(v) * r * gm.x, bf16_hi(v) * r * gm.y);
    }
  }
  __syncthreads();
  // ---- stream my groups
  float acc[MR][CPL];
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPL; ++c) acc[m][c] = 0.f;
  for (; g < g_hi; g += WC_WARPS) {
    const int gn = g + WC_WARPS;
    if (live && gn < g_hi) load_group(wnxt, gn);
    const __nv_bfloat16* xg = xs + (size_t)(g - g_lo) * 128;
    float xsum[MR];
#pragma unroll
    for (int m = 0; m < MR; ++m) {
      const uint2 v = reinterpret_cast<const uint2*>(xg + (size_t)m * kslice)[lane];
      xsum[m] = warp_sum(bf16_lo(v.x) + bf16_hi(v.x) + bf16_lo(v.y) + bf16_hi(v.y));
    }
    if (live) {
      float sc[CPL];
#pragma unroll
      for (int c = 0; c < CPL; ++c) sc[c] = __bfloat162float(scales[(long)g * N + n0 + c * cstride]);
      float pt[MR][CPL];
#pragma unroll
      for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CPL; ++c) pt[m][c] = 0.f;
#pragma unroll
      for (int r = 0; r < 16; ++r) {
        float xv[MR][8];
#pragma unroll
        for (int m = 0; m < MR; ++m) {
          const uint4 v = reinterpret_cast<const uint4*>(xg + (size_t)m * kslice)[r];
          xv[m][0] = bf16_lo(v.x); xv[m][1] = bf16_hi(v.x); xv[m][2] = bf16_lo(v.y); xv[m][3] = bf16_hi(v.y);
          xv[m][4] = bf16_lo(v.z); xv[m][5] = bf16_hi(v.z); xv[m][6] = bf16_lo(v.w); xv[m][7] = bf16_hi(v.w);
        }
#pragma unroll
        for (int c = 0; c < CPL; ++c) {
#pragma unroll
          for (int i = 0; i < 4; ++i) {
            const uint32_t pr = ((wcur[r][c] >> (4 * i)) & 0x000F000Fu) | 0x43004300u;
            const float q0 = __uint_as_float(pr << 16), q1 = __uint_as_float(pr & 0xFFFF0000u);
#pragma unroll
            for (int m = 0; m < MR; ++m) pt[m][c] = fmaf(xv[m][2 * i], q0, fmaf(xv[m][2 * i + 1], q1, pt[m][c]));
          }
        }
      }
#pragma unroll
      for (int m = 0; m < MR; ++m)
#pragma unroll
        for (int c = 0; c < CPL; ++c) acc[m][c] = fmaf(pt[m][c] - 136.f * xsum[m], sc[c], acc[m][c]);
#pragma unroll
      for (int r = 0; r < 16; ++r)
#pragma unroll
        for (int c = 0; c < CPL; ++c) wcur[r][c] = wnxt[r][c];
    }
  }
  // ---- CTA reduction, then cluster reduction into rank 0
#pragma unroll
  for (int m = 0; m < MR; ++m)
#pragma unroll
    for (int c = 0; c < CPL; ++c) red[(warp * MR + m) * 32 * CPL + lane * CPL + c] = acc[m][c];
  __syncthreads();
  for (int i = threadIdx.x; i < MR * 32 * CPL; i += WC_WARPS * 32) {
    float v = 0.f;
#pragma unroll
    for (int wq = 0; wq < WC_WARPS; ++wq) v += red[wq * MR * 32 * CPL + i];
    part[i] = v;
  }
  cluster.sync();                                       // all partial tiles are in shared memory
  bool released = false;
  if (crank == 0 && GATED) {
    const int I = N >> 1;
    for (int i = threadIdx.x; i < MR * 32; i += WC_WARPS * 32) {
      const int m = i >> 5, l = i & 31;
      const int n = blockIdx.x * 32 + l;
      float gt = 0.f, vl = 0.f;
      for (int r = 0; r < S; ++r) {
        const float* rp = cluster.map_shared_rank(part, r) + m * 64 + 2 * l;
        gt += rp[0];
        vl += rp[1 % CPL];
      }
      // the unfused path stores gate and value as bf16 before the activation
      gt = __bfloat162float(__float2bfloat16(gt));
      vl = __bfloat162float(__float2bfloat16(vl));
      if (m < M && n < I) y[(long)m * I + n] = __float2bfloat16(gt / (1.f + __expf(-gt)) * vl);
    }
  } else if (crank == 0 && rope.cos_t != nullptr) {
    // pairs of adjacent columns (interleaved rotary convention); columns of a CTA start on an even n
    const int pos = min(*rope.pos_ptr, rope.cap - 1);
    const int D = rope.D, half = D >> 1;
    for (int i = threadIdx.x; i < MR * 16 * CPL; i += WC_WARPS * 32) {
      const int m = i / (16 * CPL), c = 2 * (i - m * 16 * CPL);
      const int n = blockIdx.x * 32 * CPL + c;
      if (m >= M || n >= N) continue;
      float a = 0.f, b = 0.f;
      for (int r = 0; r < S; ++r) {
        const float* rp = cluster.map_shared_rank(part, r) + m * 32 * CPL + c;
        a += rp[0];
        b += rp[1];
      }
      a = __bfloat162float(__float2bfloat16(a));        // the projection's output is bf16 before the rotation
      b = __bfloat162float(__float2bfloat16(b));
      const int h = n / D, d = n - h * D;
      if (h < rope.Hq + rope.Hkv) {
        const float cs = rope.cos_t[(long)pos * half + (d >> 1)], sn = rope.sin_t[(long)pos * half + (d >> 1)];
        const float ra = a * cs - b * sn, rb = a * sn + b * cs;
        a = ra;
        b = rb;
      }
      const uint32_t packed = pack_bf16(a, b);
      if (h < rope.Hq) {
        *reinterpret_cast<uint32_t*>(y + (long)m * N + n) = packed;
      } else {
        const bool is_k = h < rope.Hq + rope.Hkv;
        const int hk = is_k ? h - rope.Hq : h - rope.Hq - rope.Hkv;
        __nv_bfloat16* dst = (is_k ? rope.kc : rope.vc) + (long)m * rope.c_sb + (long)pos * rope.c_ss + (long)hk * rope.c_sh + d;
        *reinterpret_cast<uint32_t*>(dst) = packed;
      }
    }
  } else if (crank == 0 && ar.world > 1) {
    const long slot = 4 * ar.n_pad;
    const long poff = (long)(ar_epoch & 1u) * ar.world * slot;
    // (a) my partial of this column block into slot [rank] of every rank's inbox
    for (int i = threadIdx.x; i < MR * 32 * CPL; i += WC_WARPS * 32) {
      const int m = i / (32 * CPL), c = i - m * 32 * CPL;
      const int n = blockIdx.x * 32 * CPL + c;
      float v = 0.f;
      for (int r = 0; r < S; ++r) v += cluster.map_shared_rank(part, r)[i];
      if (m < M && n < N) {
        const long at = poff + (long)ar.rank * slot + (long)m * ar.n_pad + n;
        for (int d = 0; d < ar.world; ++d) ar.inbox[d][at] = v;
      }
    }
    // the other CTAs of the cluster are only needed for their tiles: let them go now, so that the SM slots of
    // a whole cluster are not held while this CTA waits for the peers (the exchange would otherwise be
    // serialised once per wave of clusters)
    cluster.sync();
    released = true;
    if (threadIdx.x == 0) {
      __threadfence_system();                            // my partial is visible everywhere before any flag
      for (int d = 0; d < ar.world; ++d)
        *reinterpret_cast<volatile uint32_t*>(ar.flags[d] + (long)blockIdx.x * AR_MAX_RANKS + ar.rank) = ar_epoch;
    }
    // (b) wait for this block's partials of all ranks (bounded), then sum in rank order
    if ((int)threadIdx.x < ar.world) {
      if (!wait_flag_sys(ar.flags[ar.rank] + (long)blockIdx.x * AR_MAX_RANKS + threadIdx.x, ar_epoch)) atomicOr(ar.err, 2u);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < MR * 32 * CPL; i += WC_WARPS * 32) {
      const int m = i / (32 * CPL), c = i - m * 32 * CPL;
      const int n = blockIdx.x * 32 * CPL + c;
      if (m < M && n < N) {
        float v = 0.f;
        for (int src = 0; src < ar.world; ++src)
          v += __ldcg(ar.inbox[ar.rank] + poff + (long)src * slot + (long)m * ar.n_pad + n);
        if (residual) v += __bfloat162float(residual[(long)m * N + n]);
        y[(long)m * N + n] = __float2bfloat16(v);
      }
    }
  } else if (crank == 0) {
    for (int i = threadIdx.x; i < MR * 32 * CPL; i += WC_WARPS * 32) {
      const int m = i / (32 * CPL), c = i - m * 32 * CPL;
      const int n = blockIdx.x * 32 * CPL + c;
      float v = 0.f;
      for (int r = 0; r < S; ++r) v += cluster.map_shared_rank(part, r)[i];
      if (m < M && n < N) {
        if (residual) v += __bfloat162float(residual[(long)m * N + n]);
        y[(long)m * N + n] = __float2bfloat16(v);
      }
    }
  }
  if (!released) cluster.sync();                        // nobody leaves while rank 0 still reads its tile
  if (ar.world > 1 && threadIdx.x == 0) {               // the last CTA of the grid bumps the call number
    __threadfence();
    if (atomicAdd(ar.counter, 1u) == gridDim.x * gridDim.y - 1) {
      *ar.counter = 0;
      *ar.epoch_word = ar_epoch;
    }
  }
}

template <int MR, int CPL, bool GATED = false>
static int launch_w4_cluster(const void* x, const void* wk8, const void* scales, const void* residual, void* y, int M,
                             int N, int K, long ldx, const float* gamma, float eps, cudaStream_t st,
                             const RopeAppend* rope_args = nullptr, const ArFuse* ar_args = nullptr) {
  RopeAppend rope = {};
  if (rope_args) rope = *rope_args;
  ArFuse ar = {};
  if (ar_args) ar = *ar_args;
  const int groups = K / 128;
  const int blocks = GATED ? (N / 2 + 31) / 32 : (N + 32 * CPL - 1) / (32 * CPL);
  // split K until every warp still has a group and the grid holds about 6 CTAs (24 warps) per SM
  int S = 1;
  while (S < 8 && groups / (2 * S) >= WC_WARPS && (long)blocks * 2 * S <= 8L * num_sms()) S *= 2;
  const int gpc = (groups + S - 1) / S;
  const size_t smem = (size_t)MR * gpc * 128 * 2 + (size_t)(WC_WARPS + 1) * MR * 32 * CPL * 4 + 64;
  auto kern = w4_gemv_cluster_kernel<MR, CPL, GATED>;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    allowed = 200 * 1024;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks, S, 1);
  cfg.blockDim = dim3(WC_WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = S;
  attr[0].val.clusterDim.z = 1;
  // programmatic dependent launch: this grid may start while its predecessor in the stream still runs;
  // it touches nothing the predecessor produces (and writes nothing) before `griddepcontrol.wait`
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  SB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)x, (const uint32_t*)wk8,
                                   (const __nv_bfloat16*)scales, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, M,
                                   N, K, ldx, gpc, gamma, eps, rope, ar));
  return SB_OK;
}

}  // namespace sb

// As sb_w4_gemv_small, with the K range split over a thread-block cluster. gamma (fp32 [K]) != null
// fuses y = rmsnorm(x; gamma, eps) @ W.
extern "C" int sb_w4_gemv_cluster(const void* x, const void* wk8, const void* scales, const void* residual, void* y,
                                  int M, int N, int K, long ldx, const float* gamma, float eps, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 4 && K > 0 && K % 128 == 0 && N > 0 && N % 4 == 0 && ldx % 8 == 0);
  const int sms = sb::num_sms();
  const int cpl = (N / 128 >= 4 * sms) ? 4 : ((N / 64 >= 2 * sms && N % 64 == 0) ? 2 : 1);
  const int mr = M <= 1 ? 1 : (M <= 2 ? 2 : 4);
#define SB_W4C(MR, CPL) return sb::launch_w4_cluster<MR, CPL>(x, wk8, scales, residual, y, M, N, K, ldx, gamma, eps, st)
  if (cpl == 4) { if (mr == 1) SB_W4C(1, 4); if (mr == 2) SB_W4C(2, 4); SB_W4C(4, 4); }
  if (cpl == 2) { if (mr == 1) SB_W4C(1, 2); if (mr == 2) SB_W4C(2, 2); SB_W4C(4, 2); }
  if (mr == 1) SB_W4C(1, 1);
  if (mr == 2) SB_W4C(2, 1);
  SB_W4C(4, 1);
#undef SB_W4C
}

// y[M, I] = silu(g) * v with [g | v] = (rmsnorm(x) or x) @ dequant(W[K, 2I]): the gated in-projection of a
// decode step, activation included. M <= 4, K % 128 == 0, I % 4 == 0.
extern "C" int sb_w4_gemv_cluster_swiglu(const void* x, const void* wk8, const void* scales, void* y, int M, int N,
                                         int K, long ldx, const float* gamma, float eps, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 4 && K > 0 && K % 128 == 0 && N > 0 && N % 8 == 0 && ldx % 8 == 0);
  if (M <= 1) return sb::launch_w4_cluster<1, 2, true>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st);
  if (M <= 2) return sb::launch_w4_cluster<2, 2, true>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st);
  return sb::launch_w4_cluster<4, 2, true>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st);
}

// The qkv projection of a decode step with its RoPE and KV-cache append in the epilogue: q heads are
// rotated and written to y `[M, N]` (k / v columns of y are not written), k heads are rotated and stored
// at k_cache[b, *pos], v heads at v_cache[b, *pos]. cache_strides = (batch, position, head) in elements.
extern "C" int sb_w4_gemv_cluster_rope(const void* x, const void* wk8, const void* scales, void* y, int M, int N, int K,
                                       long ldx, const float* gamma, float eps, const float* cos_t, const float* sin_t,
                                       void* k_cache, void* v_cache, const int* pos_ptr, int Hq, int Hkv, int D,
                                       const long* cache_strides, int cap, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 4 && K > 0 && K % 128 == 0 && N == (Hq + 2 * Hkv) * D && D % 2 == 0 && ldx % 8 == 0);
  SB_CHECK_ARG(cos_t && sin_t && k_cache && v_cache && pos_ptr && cap > 0);
  sb::RopeAppend r;
  r.cos_t = cos_t; r.sin_t = sin_t; r.kc = (__nv_bfloat16*)k_cache; r.vc = (__nv_bfloat16*)v_cache; r.pos_ptr = pos_ptr;
  r.Hq = Hq; r.Hkv = Hkv; r.D = D; r.cap = cap;
  r.c_sb = cache_strides[0]; r.c_ss = cache_strides[1]; r.c_sh = cache_strides[2];
  if (M <= 1) return sb::launch_w4_cluster<1, 1>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st, &r);
  if (M <= 2) return sb::launch_w4_cluster<2, 1>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st, &r);
  return sb::launch_w4_cluster<4, 1>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st, &r);
}

// ---------------------------------------------------------------------------- W4 GEMV, dequantisation into mma fragments
// The profile of the CUDA-core GEMV above (N 28672, K 4096, one row) shows the integer pipe at 61 % and
// DRAM at 22 % of peak: nibble extraction plus bf16 -> fp32 conversion plus two FMAs per weight pair is
// an instruction-issue bound, not a bandwidth bound. Here the extracted pair `(128 + q_even, 128 + q_odd)`
// (one funnel shift and one LOP3) IS the A fragment of a `mma.sync.m16n8k16` (rows = 16 output columns,
// k = 16 codes), the B fragment holds up to 8 rows of x, and the -136 offset is removed per scale group
// with the sum of x over the group: 2 integer instructions per weight pair and no CUDA-core FMA.
// The warp-level mma is used as the dot-product unit of a bandwidth-bound GEMV (1..8 rows); the
// compute-bound shapes (prefill, training) are on tcgen05.
namespace sb {

constexpr int WM_WARPS = 4;

__device__ __forceinline__ void mma_bf16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

// grid (ceil(N / 32), S), cluster (1, S, 1), 128 threads. CTA = 32 output columns x its K slice (gpc groups);
// the 4 warps take the slice's scale groups round robin.
//
// Fragment mapping. The contraction of an mma does not care which of its 16 k slots holds which k, nor which
// of its 16 rows holds which output column, as long as A and B agree. Lane (g, t) = (lane / 4, lane % 4)
// therefore loads ONE 16-byte vector per 32-k block: the words of k8 row 4 j + t for its four columns
// 4 g .. 4 g + 3 (512 contiguous-per-row bytes per warp instruction, every byte used once), and feeds
//   tile A: row g = column 4 g, row g + 8 = column 4 g + 1;   tile B: columns 4 g + 2, 4 g + 3
//   k step 1: slots (t, t + 4) = pairs 0, 1 of its word;      k step 2: pairs 2, 3
// so its B fragments are x[row g][8 (4 j + t) .. + 8): one 16-byte shared load for both k steps.
__global__ void __launch_bounds__(WM_WARPS * 32)
w4_gemv_mma_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ wk8,
                   const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ residual,
                   __nv_bfloat16* __restrict__ y, int M, int N, int K, long ldx, int gpc,
                   const float* __restrict__ gamma, float eps) {
  extern __shared__ __align__(16) unsigned char wm_smem[];
  cg::cluster_group cluster = cg::this_cluster();
  const int S = (int)cluster.num_blocks();
  const int crank = (int)cluster.block_rank();
  const int groups = K >> 7;
  const int g_lo = crank * gpc, g_hi = min(groups, g_lo + gpc);
  const int kslice = gpc * 128;
  const int xld = kslice + 32;      // row stride of xs: 64 bytes of padding keep the B-fragment loads of two rows on distinct banks
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(wm_smem);                 // [M][xld]
  float* xsum = reinterpret_cast<float*>(wm_smem + (size_t)M * xld * 2);      // [gpc][8]
  float* red = xsum + gpc * 8;                                                   // [WM_WARPS][32 n][8 m]
  float* part = red + WM_WARPS * 256;                                            // [32 n][8 m]
  float* ssq = part + 256;                                                       // [8]
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int nb = blockIdx.x * 32;
  const int cb = nb + 4 * gq;                                                    // my four columns
  const int kbase = g_lo * 128;
  const int k8n = max(0, (g_hi - g_lo) * 16);
  const bool live = cb < N;                                                      // N % 4 == 0
  uint4 wc[4], wn[4];
  auto load_group = [&](uint4 (&w)[4], int g) {
#pragma unroll
    for (int j = 0; j < 4; ++j)
      w[j] = live ? __ldcs(reinterpret_cast<const uint4*>(wk8 + (long)(16 * g + 4 * j + tq) * N + cb)) : make_uint4(0u, 0u, 0u, 0u);
  };
  asm volatile("griddepcontrol.launch_dependents;");
  int g = g_lo + warp;
  if (g < g_hi) load_group(wc, g);
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // ---- stage the M rows of x, optional fused RMSNorm, per-group sums
  for (int i = threadIdx.x; i < M * k8n; i += WM_WARPS * 32) {
    const int m = i / k8n, c = i - m * k8n;
    reinterpret_cast<uint4*>(xs + (size_t)m * xld)[c] = *reinterpret_cast<const uint4*>(x + (long)m * ldx + kbase + 8 * c);
  }
  if (gamma != nullptr) {
    __syncthreads();
    for (int m = warp; m < M; m += WM_WARPS) {
      float sq = 0.f;
      for (int c = lane; c < k8n * 4; c += 32) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(xs + (size_t)m * xld)[c];
        sq += bf16_lo(v) * bf16_lo(v) + bf16_hi(v) * bf16_hi(v);
      }
      sq = warp_sum(sq);
      if (lane == 0) ssq[m] = sq;
    }
    cluster.sync();
    for (int m = warp; m < M; m += WM_WARPS) {
      float t = 0.f;
      for (int r = 0; r < S; ++r) t += cluster.map_shared_rank(ssq, r)[m];
      const float rstd = rsqrtf(t / static_cast<float>(K) + eps);
      for (int c = lane; c < k8n * 4; c += 32) {
        uint32_t* p = reinterpret_cast<uint32_t*>(xs + (size_t)m * xld) + c;
        const uint32_t v = *p;
        const float2 gm = *reinterpret_cast<const float2*>(gamma + kbase + 2 * c);
        *p = pack_bf16(bf16_lo(v) * rstd * gm.x, bf16_hi(v) * rstd * gm.y);
      }
    }
  }
  __syncthreads();
  // (group, row) sums of x: four lanes per item, 32 elements each
  for (int i = threadIdx.x; i < (g_hi - g_lo) * 8 * 4; i += WM_WARPS * 32) {
    const int q = i & 3, m = (i >> 2) & 7, gg = i >> 5;
    float s = 0.f;
    if (m < M) {
      const uint4* p = reinterpret_cast<const uint4*>(xs + (size_t)m * xld + gg * 128 + 32 * q);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint4 v = p[c];
        s += (bf16_lo(v.x) + bf16_hi(v.x)) + (bf16_lo(v.y) + bf16_hi(v.y)) + (bf16_lo(v.z) + bf16_hi(v.z)) + (bf16_lo(v.w) + bf16_hi(v.w));
      }
    }
    s += __shfl_xor_sync(0xffffffffu, s, 1);
    s += __shfl_xor_sync(0xffffffffu, s, 2);
    if (q == 0) xsum[gg * 8 + m] = s;
  }
  __syncthreads();
  // ---- stream my groups
  float accA[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f};
  const __nv_bfloat16* xrow = xs + (size_t)min(gq, M - 1) * xld;  // B fragment: column gq = row gq of x (zero beyond M)
  for (; g < g_hi; g += WM_WARPS) {
    const int gn = g + WM_WARPS;
    if (gn < g_hi) load_group(wn, gn);
    float dA[4] = {0.f, 0.f, 0.f, 0.f}, dB[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      uint4 xb = *reinterpret_cast<const uint4*>(xrow + (g - g_lo) * 128 + 8 * (4 * j + tq));
      if (gq >= M) xb = make_uint4(0u, 0u, 0u, 0u);
      const uint32_t w0 = wc[j].x, w1 = wc[j].y, w2 = wc[j].z, w3 = wc[j].w;
      uint32_t a[4];
      a[0] = (w0 & 0x000F000Fu) | 0x43004300u;
      a[1] = (w1 & 0x000F000Fu) | 0x43004300u;
      a[2] = ((w0 >> 4) & 0x000F000Fu) | 0x43004300u;
      a[3] = ((w1 >> 4) & 0x000F000Fu) | 0x43004300u;
      mma_bf16_16816(dA, a, xb.x, xb.y);
      a[0] = ((w0 >> 8) & 0x000F000Fu) | 0x43004300u;
      a[1] = ((w1 >> 8) & 0x000F000Fu) | 0x43004300u;
      a[2] = ((w0 >> 12) & 0x000F000Fu) | 0x43004300u;
      a[3] = ((w1 >> 12) & 0x000F000Fu) | 0x43004300u;
      mma_bf16_16816(dA, a, xb.z, xb.w);
      a[0] = (w2 & 0x000F000Fu) | 0x43004300u;
      a[1] = (w3 & 0x000F000Fu) | 0x43004300u;
      a[2] = ((w2 >> 4) & 0x000F000Fu) | 0x43004300u;
      a[3] = ((w3 >> 4) & 0x000F000Fu) | 0x43004300u;
      mma_bf16_16816(dB, a, xb.x, xb.y);
      a[0] = ((w2 >> 8) & 0x000F000Fu) | 0x43004300u;
      a[1] = ((w3 >> 8) & 0x000F000Fu) | 0x43004300u;
      a[2] = ((w2 >> 12) & 0x000F000Fu) | 0x43004300u;
      a[3] = ((w3 >> 12) & 0x000F000Fu) | 0x43004300u;
      mma_bf16_16816(dB, a, xb.z, xb.w);
    }
    float sc[4] = {0.f, 0.f, 0.f, 0.f};
    if (live) {
      const uint2 sv = *reinterpret_cast<const uint2*>(scales + (long)g * N + cb);
      sc[0] = bf16_lo(sv.x); sc[1] = bf16_hi(sv.x); sc[2] = bf16_lo(sv.y); sc[3] = bf16_hi(sv.y);
    }
    const float2 xsm = *reinterpret_cast<const float2*>(xsum + (g - g_lo) * 8 + 2 * tq);
    const float o0 = 136.f * xsm.x, o1 = 136.f * xsm.y;
    accA[0] = fmaf(dA[0] - o0, sc[0], accA[0]);     // column 4 g,     rows 2 t, 2 t + 1 of x
    accA[1] = fmaf(dA[1] - o1, sc[0], accA[1]);
    accA[2] = fmaf(dA[2] - o0, sc[1], accA[2]);     // column 4 g + 1
    accA[3] = fmaf(dA[3] - o1, sc[1], accA[3]);
    accB[0] = fmaf(dB[0] - o0, sc[2], accB[0]);     // column 4 g + 2
    accB[1] = fmaf(dB[1] - o1, sc[2], accB[1]);
    accB[2] = fmaf(dB[2] - o0, sc[3], accB[2]);     // column 4 g + 3
    accB[3] = fmaf(dB[3] - o1, sc[3], accB[3]);
#pragma unroll
    for (int j = 0; j < 4; ++j) wc[j] = wn[j];
  }
  // ---- reductions: warps -> CTA tile [32 n][8 m] -> cluster
  {
    float* r = red + warp * 256 + (4 * gq) * 8 + 2 * tq;
    *reinterpret_cast<float2*>(r) = make_float2(accA[0], accA[1]);
    *reinterpret_cast<float2*>(r + 8) = make_float2(accA[2], accA[3]);
    *reinterpret_cast<float2*>(r + 16) = make_float2(accB[0], accB[1]);
    *reinterpret_cast<float2*>(r + 24) = make_float2(accB[2], accB[3]);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < 256; i += WM_WARPS * 32) part[i] = red[i] + red[256 + i] + red[512 + i] + red[768 + i];
  cluster.sync();
  if (crank == 0) {
    for (int i = threadIdx.x; i < 256; i += WM_WARPS * 32) {
      const int nl = i >> 3, m = i & 7;
      const int n = nb + nl;
      if (m < M && n < N) {
        float v = 0.f;
        for (int r = 0; r < S; ++r) v += cluster.map_shared_rank(part, r)[i];
        if (residual) v += __bfloat162float(residual[(long)m * N + n]);
        y[(long)m * N + n] = __float2bfloat16(v);
      }
    }
  }
  cluster.sync();
}

}  // namespace sb

// y[M,N] = (rmsnorm(x) or x)[M,K] @ dequant(W) (+ residual), M <= 8, K % 128 == 0, N % 4 == 0. One launch.
extern "C" int sb_w4_gemv_mma(const void* x, const void* wk8, const void* scales, const void* residual, void* y, int M,
                              int N, int K, long ldx, const float* gamma, float eps, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(M >= 1 && M <= 8 && K > 0 && K % 128 == 0 && N > 0 && N % 4 == 0 && ldx % 8 == 0);
  const int groups = K / 128;
  const int blocks = (N + 31) / 32;
  int S = 1;
  while (S < 8 && groups / (2 * S) >= WM_WARPS && (long)blocks * 2 * S <= 8L * num_sms()) S *= 2;
  const int gpc = (groups + S - 1) / S;
  const size_t smem = (size_t)M * (gpc * 128 + 32) * 2 + (size_t)(gpc * 8 + WM_WARPS * 256 + 256 + 8) * 4;
  SB_CHECK_ARG(smem <= 200 * 1024);
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(w4_gemv_mma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    allowed = 200 * 1024;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(blocks, S, 1);
  cfg.blockDim = dim3(WM_WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = S;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  SB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, w4_gemv_mma_kernel, (const __nv_bfloat16*)x, (const uint32_t*)wk8,
                                   (const __nv_bfloat16*)scales, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, M,
                                   N, K, ldx, gpc, gamma, eps));
  return SB_OK;
}

// ---------------------------------------------------------------------------- W4 GEMV, persistent streaming form
// The same projections as ONE resident grid: a CTA (8 warps) stages x once (optional fused RMSNorm, the
// per-group sums of x), then walks its share of the 32-column blocks; inside a block the warps take the scale
// groups round robin and use the 16-byte-vector fragment mapping of w4_gemv_mma_kernel, the weights arriving
// through a per-warp ring of asynchronous copies three groups ahead. Per block the warps' tiles meet in shared
// memory and the epilogue adds the residual or applies SwiGLU (a gated block is 16 gate columns + the matching
// 16 value columns). Measured on a B200 (N 28672, K 4096, one row: 31 us against 33 us for the cluster kernel,
// DRAM 24 % of peak, the integer pipe at 45 % still the busiest unit) it is level with the cluster kernel launch
// by launch and slower inside the decode step's graph, where a resident grid leaves the next kernel's prologue
// nothing to overlap with; the decode path therefore stays on the cluster kernel and this one is an explicit
// alternative (sb_w4_gemv_stream).
namespace sb {

constexpr int WP_WARPS = 8;

__device__ __forceinline__ void mma_f16_16816(float (&d)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0, %1, %2, %3}, {%4, %5, %6, %7}, {%8, %9}, "
               "{%0, %1, %2, %3};"
               : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
constexpr int WP_STAGES = 4;      // ring depth per warp: 3 scale groups (6 KB) in flight while one is consumed

template <int MR, bool GATED>
__global__ void __launch_bounds__(WP_WARPS * 32)
w4_gemv_stream_kernel(const __nv_bfloat16* __restrict__ x, const uint32_t* __restrict__ wk8,
                      const __nv_bfloat16* __restrict__ scales, const __nv_bfloat16* __restrict__ residual,
                      __nv_bfloat16* __restrict__ y, int M, int N, int K, long ldx, int nblocks,
                      const float* __restrict__ gamma, float eps) {
  extern __shared__ __align__(16) unsigned char wp_smem[];
  const int G = K >> 7;
  const int xld = K + 32;                    // 64 bytes of padding: the B-fragment loads of two rows of x miss each other's banks
  __nv_bfloat16* xs = reinterpret_cast<__nv_bfloat16*>(wp_smem);                  // [MR][xld]: bf16 as loaded, then fp16 in place
  float* xsum = reinterpret_cast<float*>(wp_smem + (size_t)MR * xld * 2);         // [G][MR]
  float* red = xsum + G * MR;                                                     // [WP_WARPS][MR][32]
  float* part = red + WP_WARPS * MR * 32;                                         // [MR][32]
  float* ssq = part + MR * 32;                                                    // [MR] (+ pad to 16 bytes)
  // [WP_WARPS][WP_STAGES][4][32] weight vectors in flight (16-byte aligned)
  uint4* ring = reinterpret_cast<uint4*>((reinterpret_cast<uintptr_t>(ssq + MR) + 15) & ~static_cast<uintptr_t>(15));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int gq = lane >> 2, tq = lane & 3;
  const int I = N >> 1;                                                           // gated: W = [gate | value]
  // first of this lane's four columns in block `blk`
  auto col_of = [&](int blk) {
    if (GATED) return (gq < 4 ? 0 : I) + blk * 16 + 4 * (gq & 3);
    return blk * 32 + 4 * gq;
  };
  auto live_of = [&](int blk) { return GATED ? blk * 16 + 4 * (gq & 3) < I : blk * 32 + 4 * gq < N; };
  // The weights reach the lanes through a per-warp ring in shared memory filled by 16-byte asynchronous copies,
  // WP_STAGES - 1 scale groups ahead (each lane later reads back exactly the 16 bytes it asked for, so the ring
  // needs no layout): the bytes in flight per SM, not the instruction count, decide a weight-streaming GEMV.
  const int ngw = warp < G ? (G - warp + WP_WARPS - 1) / WP_WARPS : 0;            // my groups per block
  const int nmine = blockIdx.x < nblocks ? (nblocks - blockIdx.x + gridDim.x - 1) / gridDim.x : 0;
  const int total = nmine * ngw;                                                  // my (block, group) items, in order
  uint4* myring = ring + (size_t)warp * WP_STAGES * 128;
  int iq = 0, ib = blockIdx.x, ig = warp;                                         // next item to issue: number, block, group
  auto issue = [&]() {
    if (iq < total) {
      const bool live = live_of(ib);
      const uint32_t* p = wk8 + (long)(16 * ig + tq) * N + (live ? col_of(ib) : 0);
      const uint32_t dst = smem_u32(myring + (iq % WP_STAGES) * 128 + lane);
#pragma unroll
      for (int j = 0; j < 4; ++j) cp_async16_zfill(dst + j * 512, p + (long)4 * j * N, live ? 16 : 0);
      ++iq;
      ig += WP_WARPS;
      if (ig >= G) { ig = warp; ib += gridDim.x; }
    }
    cp_async_commit();
  };
  asm volatile("griddepcontrol.launch_dependents;");
#pragma unroll
  for (int q = 0; q < WP_STAGES - 1; ++q) issue();
  asm volatile("griddepcontrol.wait;" ::: "memory");
  // ---- stage x once per CTA, optional fused RMSNorm, per-group sums
  const int k8n = K >> 3;
  for (int i = threadIdx.x; i < MR * k8n; i += WP_WARPS * 32) {
    const int m = i / k8n, c = i - m * k8n;
    uint4 v = make_uint4(0u, 0u, 0u, 0u);
    if (m < M) v = *reinterpret_cast<const uint4*>(x + (long)m * ldx + 8 * c);
    reinterpret_cast<uint4*>(xs + (size_t)m * xld)[c] = v;
  }
  __syncthreads();
  if (gamma != nullptr) {
    for (int m = warp; m < MR; m += WP_WARPS) {
      float sq = 0.f;
      for (int c = lane; c < k8n * 4; c += 32) {
        const uint32_t v = reinterpret_cast<const uint32_t*>(xs + (size_t)m * xld)[c];
        sq += bf16_lo(v) * bf16_lo(v) + bf16_hi(v) * bf16_hi(v);
      }
      sq = warp_sum(sq);
      if (lane == 0) ssq[m] = sq;
    }
    __syncthreads();
  }
  // x as fp16 in place (every bf16 value of sane magnitude is exact in fp16; the clamp keeps the rest finite),
  // with the fused norm applied on the way: rstd * gamma, rounded to bf16 first as the separate norm kernel does
  for (int i = threadIdx.x; i < MR * k8n * 4; i += WP_WARPS * 32) {               // pairs of elements
    const int m = i / (k8n * 4), c = i - m * (k8n * 4);
    uint32_t* p = reinterpret_cast<uint32_t*>(xs + (size_t)m * xld) + c;
    const uint32_t v = *p;
    float a = bf16_lo(v), b = bf16_hi(v);
    if (gamma != nullptr) {
      const float2 gm = *reinterpret_cast<const float2*>(gamma + 2 * c);
      const float r = rsqrtf(ssq[m] / static_cast<float>(K) + eps);
      a = __bfloat162float(__float2bfloat16(a * r * gm.x));
      b = __bfloat162float(__float2bfloat16(b * r * gm.y));
    }
    const __half2 h = __floats2half2_rn(fminf(fmaxf(a, -65504.f), 65504.f), fminf(fmaxf(b, -65504.f), 65504.f));
    *p = *reinterpret_cast<const uint32_t*>(&h);
  }
  __syncthreads();
  // Per (group, row): the sum of x over the k whose code is used in place (k % 4 < 2) and over those whose code
  // is used times 16 (k % 4 >= 2). Four lanes per item, 32 elements each; the trip count is rounded up so that
  // whole warps reach the shuffles.
  for (int i = threadIdx.x; i < ((G * MR * 4 + 31) & ~31); i += WP_WARPS * 32) {
    const bool valid = i < G * MR * 4;
    const int q = i & 3, gm_ = valid ? i >> 2 : 0;
    const int m = gm_ % MR, gg = gm_ / MR;
    const uint4* p = reinterpret_cast<const uint4*>(xs + (size_t)m * xld + gg * 128 + 32 * q);
    float su = 0.f, ss = 0.f;
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint4 v = p[c];
      const float2 f0 = __half22float2(*reinterpret_cast<const __half2*>(&v.x)), f1 = __half22float2(*reinterpret_cast<const __half2*>(&v.y));
      const float2 f2 = __half22float2(*reinterpret_cast<const __half2*>(&v.z)), f3 = __half22float2(*reinterpret_cast<const __half2*>(&v.w));
      su += (f0.x + f0.y) + (f2.x + f2.y);
      ss += (f1.x + f1.y) + (f3.x + f3.y);
    }
    su += __shfl_xor_sync(0xffffffffu, su, 1);
    ss += __shfl_xor_sync(0xffffffffu, ss, 1);
    su += __shfl_xor_sync(0xffffffffu, su, 2);
    ss += __shfl_xor_sync(0xffffffffu, ss, 2);
    if (valid && q == 0) xsum[gg * MR + m] = 1032.f * su + 72.f * ss;              // what the magic numbers add to the product
  }
  __syncthreads();
  // ---- the CTA's column blocks
  // B fragment: column gq = row gq of x; the columns beyond MR repeat the last row (their outputs are never read)
  const __nv_bfloat16* xrow = xs + (size_t)min(gq, MR - 1) * xld;
  const int m0 = 2 * tq, m1 = 2 * tq + 1;                                         // the rows of x this lane's accumulators belong to
  int q = 0;
  for (int cur = blockIdx.x; cur < nblocks; cur += gridDim.x) {
    float accA[4] = {0.f, 0.f, 0.f, 0.f}, accB[4] = {0.f, 0.f, 0.f, 0.f};
    const bool live = live_of(cur);
    const int cb = col_of(cur);
    for (int gi = 0; gi < ngw; ++gi, ++q) {
      const int g = warp + WP_WARPS * gi;
      issue();
      cp_async_wait_group<WP_STAGES - 1>();                                       // item q has landed
      __syncwarp();
      uint4 wc[4];
#pragma unroll
      for (int j = 0; j < 4; ++j) wc[j] = myring[(q % WP_STAGES) * 128 + j * 32 + lane];
      // fp16 magic numbers: (w & 0x000F000F) | 0x64006400 is the pair (1024 + q, 1024 + q'), and the next nibble
      // up, left where it is, (w & 0x00F000F0) | 0x64006400, is (1024 + 16 q, 1024 + 16 q'), which meets x / 16
      // in the B fragment: one shift per word instead of three, and the whole offset leaves with `xsum`.
      float dA[4] = {0.f, 0.f, 0.f, 0.f}, dB[4] = {0.f, 0.f, 0.f, 0.f};
      const uint32_t sixteenth = 0x2C002C00u;                                     // fp16 pair (1/16, 1/16)
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const uint4 xb = *reinterpret_cast<const uint4*>(xrow + g * 128 + 8 * (4 * j + tq));
        uint32_t xy, xw;
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(xy) : "r"(xb.y), "r"(sixteenth));
        asm("mul.rn.f16x2 %0, %1, %2;" : "=r"(xw) : "r"(xb.w), "r"(sixteenth));
        const uint32_t w0 = wc[j].x, w1 = wc[j].y, w2 = wc[j].z, w3 = wc[j].w;
        const uint32_t v0 = w0 >> 8, v1 = w1 >> 8, v2 = w2 >> 8, v3 = w3 >> 8;
        uint32_t a[4];
        a[0] = (w0 & 0x000F000Fu) | 0x64006400u;
        a[1] = (w1 & 0x000F000Fu) | 0x64006400u;
        a[2] = (w0 & 0x00F000F0u) | 0x64006400u;
        a[3] = (w1 & 0x00F000F0u) | 0x64006400u;
        mma_f16_16816(dA, a, xb.x, xy);
        a[0] = (v0 & 0x000F000Fu) | 0x64006400u;
        a[1] = (v1 & 0x000F000Fu) | 0x64006400u;
        a[2] = (v0 & 0x00F000F0u) | 0x64006400u;
        a[3] = (v1 & 0x00F000F0u) | 0x64006400u;
        mma_f16_16816(dA, a, xb.z, xw);
        a[0] = (w2 & 0x000F000Fu) | 0x64006400u;
        a[1] = (w3 & 0x000F000Fu) | 0x64006400u;
        a[2] = (w2 & 0x00F000F0u) | 0x64006400u;
        a[3] = (w3 & 0x00F000F0u) | 0x64006400u;
        mma_f16_16816(dB, a, xb.x, xy);
        a[0] = (v2 & 0x000F000Fu) | 0x64006400u;
        a[1] = (v3 & 0x000F000Fu) | 0x64006400u;
        a[2] = (v2 & 0x00F000F0u) | 0x64006400u;
        a[3] = (v3 & 0x00F000F0u) | 0x64006400u;
        mma_f16_16816(dB, a, xb.z, xw);
      }
      float sc[4] = {0.f, 0.f, 0.f, 0.f};
      if (live) {
        const uint2 sv = *reinterpret_cast<const uint2*>(scales + (long)g * N + cb);
        sc[0] = bf16_lo(sv.x); sc[1] = bf16_hi(sv.x); sc[2] = bf16_lo(sv.y); sc[3] = bf16_hi(sv.y);
      }
      const float o0 = m0 < MR ? xsum[g * MR + m0] : 0.f, o1 = m1 < MR ? xsum[g * MR + m1] : 0.f;
      accA[0] = fmaf(dA[0] - o0, sc[0], accA[0]);
      accA[1] = fmaf(dA[1] - o1, sc[0], accA[1]);
      accA[2] = fmaf(dA[2] - o0, sc[1], accA[2]);
      accA[3] = fmaf(dA[3] - o1, sc[1], accA[3]);
      accB[0] = fmaf(dB[0] - o0, sc[2], accB[0]);
      accB[1] = fmaf(dB[1] - o1, sc[2], accB[1]);
      accB[2] = fmaf(dB[2] - o0, sc[3], accB[2]);
      accB[3] = fmaf(dB[3] - o1, sc[3], accB[3]);
    }
    // warps -> CTA tile part[m][32]: plain blocks by column, gated blocks as (gate, value) pairs
    {
      const int j0 = GATED ? 8 * (gq & 3) + (gq >> 2) : 4 * gq;                   // tile index of my first column
      const int js = GATED ? 2 : 1;                                               // and the distance of my next ones
      if (m0 < MR) {
        float* r = red + (warp * MR + m0) * 32 + j0;
        r[0] = accA[0]; r[js] = accA[2]; r[2 * js] = accB[0]; r[3 * js] = accB[2];
      }
      if (m1 < MR) {
        float* r = red + (warp * MR + m1) * 32 + j0;
        r[0] = accA[1]; r[js] = accA[3]; r[2 * js] = accB[1]; r[3 * js] = accB[3];
      }
    }
    __syncthreads();
    for (int i = threadIdx.x; i < MR * 32; i += WP_WARPS * 32) {
      float v = 0.f;
#pragma unroll
      for (int wq = 0; wq < WP_WARPS; ++wq) v += red[wq * MR * 32 + i];
      part[i] = v;
    }
    __syncthreads();
    // ---- epilogue of block `cur`
    if (GATED) {
      for (int i = threadIdx.x; i < MR * 16; i += WP_WARPS * 32) {
        const int m = i >> 4, l = i & 15;
        const int n = cur * 16 + l;
        // the unfused path stores gate and value as bf16 before the activation
        const float gt = __bfloat162float(__float2bfloat16(part[m * 32 + 2 * l]));
        const float vl = __bfloat162float(__float2bfloat16(part[m * 32 + 2 * l + 1]));
        if (m < M && n < I) y[(long)m * I + n] = __float2bfloat16(gt / (1.f + __expf(-gt)) * vl);
      }
    } else {
      for (int i = threadIdx.x; i < MR * 32; i += WP_WARPS * 32) {
        const int m = i >> 5, n = cur * 32 + (i & 31);
        if (m < M && n < N) {
          float v = part[i];
          if (residual) v += __bfloat162float(residual[(long)m * N + n]);
          y[(long)m * N + n] = __float2bfloat16(v);
        }
      }
    }
  }
}

template <int MR, bool GATED>
static int launch_w4_stream(const void* x, const void* wk8, const void* scales, const void* residual, void* y, int M,
                            int N, int K, long ldx, const float* gamma, float eps, cudaStream_t st) {
  const int nblocks = GATED ? (N / 2 + 15) / 16 : (N + 31) / 32;
  const size_t smem = (size_t)MR * (K + 32) * 2 + (size_t)((K / 128) * MR + (WP_WARPS + 1) * MR * 32 + 16) * 4 +
                      (size_t)WP_WARPS * WP_STAGES * 2048;
  SB_CHECK_ARG(smem <= 200 * 1024);
  auto kern = w4_gemv_stream_kernel<MR, GATED>;
  static size_t allowed = 48 * 1024;
  if (smem > allowed) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024));
    allowed = 200 * 1024;
  }
  const int per_sm = smem <= 100 * 1024 ? 2 : 1;
  const int grid = nblocks < per_sm * num_sms() ? nblocks : per_sm * num_sms();
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(grid, 1, 1);
  cfg.blockDim = dim3(WP_WARPS * 32, 1, 1);
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[1];
  // programmatic dependent launch: this grid may start while its predecessor in the stream still runs;
  // it touches nothing the predecessor produces (and writes nothing) before `griddepcontrol.wait`
  attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 1;
  SB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, kern, (const __nv_bfloat16*)x, (const uint32_t*)wk8,
                                   (const __nv_bfloat16*)scales, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, M,
                                   N, K, ldx, nblocks, gamma, eps));
  return SB_OK;
}

}  // namespace sb

// y[M,N] = (rmsnorm(x) or x)[M,K] @ dequant(W) (+ residual), or with gated != 0 y[M,N/2] = silu(g) * v for
// W = [gate | value], on the persistent streaming kernel. M <= 4, K % 128 == 0, N % 4 == 0 (gated: N % 8 == 0).
// An alternative to sb_w4_gemv_cluster / sb_w4_gemv_cluster_swiglu: level with them launch by launch, behind them
// inside a decode step's graph (a resident grid gives the next kernel's prologue nothing to overlap with).
extern "C" int sb_w4_gemv_stream(const void* x, const void* wk8, const void* scales, const void* residual, void* y,
                                 int M, int N, int K, long ldx, const float* gamma, float eps, int gated,
                                 cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 4 && K > 0 && K % 128 == 0 && N > 0 && N % (gated ? 8 : 4) == 0 && ldx % 8 == 0);
#define SB_W4P(MR)                                                                                                   \
  return gated ? sb::launch_w4_stream<MR, true>(x, wk8, scales, nullptr, y, M, N, K, ldx, gamma, eps, st)           \
               : sb::launch_w4_stream<MR, false>(x, wk8, scales, residual, y, M, N, K, ldx, gamma, eps, st)
  if (M <= 1) SB_W4P(1);
  if (M <= 2) SB_W4P(2);
  SB_W4P(4);
#undef SB_W4P
}

// Row-parallel decode projection with its all-reduce fused: y[M,N] = sum over ranks of x_r[M,K_r] @ W_r (+ residual).
// inbox / flags: host arrays of `world` peer-mapped pointers (inbox: 2 * world * 4 * n_pad floats per rank,
// flags: ceil(n_pad / 32) * 8 words per rank, zero at start); epoch_word / counter: device words, zero at start.
// Every rank must make the same sequence of calls with the same N.
extern "C" int sb_w4_gemv_cluster_allreduce(const void* x, const void* wk8, const void* scales, const void* residual,
                                            void* y, int M, int N, int K, long ldx, const void* const* inbox,
                                            const void* const* flags, unsigned int* epoch_word, unsigned int* counter,
                                            long n_pad, int rank, int world, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 4 && K > 0 && K % 128 == 0 && N > 0 && N % 4 == 0 && ldx % 8 == 0);
  SB_CHECK_ARG(world >= 2 && world <= sb::AR_MAX_RANKS && rank >= 0 && rank < world && n_pad >= N && epoch_word && counter);
  sb::ArFuse ar = {};
  for (int i = 0; i < world; ++i) { ar.inbox[i] = (float*)inbox[i]; ar.flags[i] = (uint32_t*)flags[i]; }
  ar.epoch_word = epoch_word; ar.counter = counter; ar.err = sb::error_word();
  ar.rank = rank; ar.world = world; ar.n_pad = n_pad;
  if (!ar.err) return sb::SB_ERR_CUDA;
  // one column-block width for all ranks and calls (the flags are per 32-column block): CPL = 1
  if (M <= 1) return sb::launch_w4_cluster<1, 1>(x, wk8, scales, residual, y, M, N, K, ldx, nullptr, 0.f, st, nullptr, &ar);
  if (M <= 2) return sb::launch_w4_cluster<2, 1>(x, wk8, scales, residual, y, M, N, K, ldx, nullptr, 0.f, st, nullptr, &ar);
  return sb::launch_w4_cluster<4, 1>(x, wk8, scales, residual, y, M, N, K, ldx, nullptr, 0.f, st, nullptr, &ar);
}
