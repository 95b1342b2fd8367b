// Memory-bound fused kernels: RMSNorm (+residual add) forward/backward, q/k RMSNorm +
// interleaved RoPE forward/backward, SwiGLU forward/backward, y*silu(z) forward/backward,
// fused AdamW over flat buffers. All read/write bf16 activations with 16-byte vector
// accesses and keep statistics in fp32; each launch covers the tensor once.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

__device__ __forceinline__ float siluf(float x) { return x / (1.f + __expf(-x)); }
__device__ __forceinline__ float sigmoidf_(float x) { return 1.f / (1.f + __expf(-x)); }

struct bf16x8 {
  uint4 v;
  __device__ __forceinline__ void unpack(float* f) const {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
  }
  __device__ __forceinline__ void pack(const float* f) {
    v.x = pack_bf16(f[0], f[1]); v.y = pack_bf16(f[2], f[3]); v.z = pack_bf16(f[4], f[5]); v.w = pack_bf16(f[6], f[7]);
  }
};

// ------------------------------------------------------------------ RMSNorm
// One warp per row; H % 8 == 0. Optional residual: s = x + r is written (bf16) and normed.
template <bool ADD>
__global__ void rmsnorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ res,
                                   const float* __restrict__ gamma, __nv_bfloat16* __restrict__ y,
                                   __nv_bfloat16* __restrict__ sum_out, float* __restrict__ rstd_out, int rows, int H,
                                   float eps) {
  asm volatile("griddepcontrol.launch_dependents;");     // lets a dependent-launch successor start its prologue
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const size_t base = static_cast<size_t>(warp) * H;
  float ss = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    float f[8];
    a.unpack(f);
    if (ADD) {
      bf16x8 b;
      b.v = *reinterpret_cast<const uint4*>(res + base + c);
      float g[8];
      b.unpack(g);
#pragma unroll
      for (int i = 0; i < 8; ++i) f[i] += g[i];
      a.pack(f);
      a.unpack(f);   // the stream is bf16: normalise the rounded sum
      *reinterpret_cast<uint4*>(sum_out + base + c) = a.v;
    }
#pragma unroll
    for (int i = 0; i < 8; ++i) ss += f[i] * f[i];
  }
  ss = warp_sum(ss);
  const float rstd = rsqrtf(ss / H + eps);
  if (lane == 0 && rstd_out) rstd_out[warp] = rstd;
  const __nv_bfloat16* src = ADD ? sum_out : x;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a;
    a.v = *reinterpret_cast<const uint4*>(src + base + c);
    float f[8];
    a.unpack(f);
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c);
    const float4 g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    f[0] *= rstd * g0.x; f[1] *= rstd * g0.y; f[2] *= rstd * g0.z; f[3] *= rstd * g0.w;
    f[4] *= rstd * g1.x; f[5] *= rstd * g1.y; f[6] *= rstd * g1.z; f[7] *= rstd * g1.w;
    a.pack(f);
    *reinterpret_cast<uint4*>(y + base + c) = a.v;
  }
}

// dx = rstd * (g*dy) - x * rstd^3 * mean(g*dy*x)  (+ dres when the op had a residual output)
template <bool ADD_GRAD>
__global__ void rmsnorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                   const __nv_bfloat16* __restrict__ dsum, const float* __restrict__ gamma,
                                   const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, int rows, int H) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const size_t base = static_cast<size_t>(warp) * H;
  const float rstd = rstd_in[warp];
  float dot = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a, b;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    b.v = *reinterpret_cast<const uint4*>(dy + base + c);
    float fx[8], fd[8];
    a.unpack(fx);
    b.unpack(fd);
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c);
    const float4 g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) dot += g[i] * fd[i] * fx[i];
  }
  dot = warp_sum(dot);
  const float coef = dot * rstd * rstd * rstd / H;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a, b;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    b.v = *reinterpret_cast<const uint4*>(dy + base + c);
    float fx[8], fd[8], o[8];
    a.unpack(fx);
    b.unpack(fd);
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c);
    const float4 g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    const float g[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = rstd * g[i] * fd[i] - coef * fx[i];
    if (ADD_GRAD) {
      bf16x8 e;
      e.v = *reinterpret_cast<const uint4*>(dsum + base + c);
      float fe[8];
      e.unpack(fe);
#pragma unroll
      for (int i = 0; i < 8; ++i) o[i] += fe[i];
    }
    a.pack(o);
    *reinterpret_cast<uint4*>(dx + base + c) = a.v;
  }
}

// dx and dgamma in ONE pass over x and dy (H <= 1536, the shared-memory tile of the block reduction): a warp walks its rows with the row held in registers
// (one read of x and dy for the dot product, the dx formula and the dgamma contribution), keeps its lanes'
// dgamma columns in registers across all its rows, the block's 8 warps meet in shared memory and each column
// costs one atomic per block. The two-kernel form read x and dy a second time from HBM for dgamma.
template <int NV, bool ADD_GRAD>
__global__ void __launch_bounds__(256, NV <= 4 ? 2 : 1)
rmsnorm_bwd_fused_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                         const __nv_bfloat16* __restrict__ dsum, const float* __restrict__ gamma,
                         const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx,
                         float* __restrict__ dgamma, int rows, int H) {
  __shared__ float red[8][256 * NV];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  const int gw = blockIdx.x * 8 + w, nw = gridDim.x * 8;
  float dg[NV][8];
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) dg[k][i] = 0.f;
  // gamma is re-read where it is used (4-6 KB, resident in L1): it would cost 8 NV registers otherwise
  auto load_gamma = [&](int c, float (&g)[8]) {
    const float4 g0 = *reinterpret_cast<const float4*>(gamma + c), g1 = *reinterpret_cast<const float4*>(gamma + c + 4);
    g[0] = g0.x; g[1] = g0.y; g[2] = g0.z; g[3] = g0.w; g[4] = g1.x; g[5] = g1.y; g[6] = g1.z; g[7] = g1.w;
  };
  for (int row = gw; row < rows; row += nw) {
    const size_t base = static_cast<size_t>(row) * H;
    const float rstd = rstd_in[row];
    float fx[NV][8], fd[NV][8];
    float dot = 0.f;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = lane * 8 + 256 * k;
      bf16x8 a, b;
      a.v = make_uint4(0u, 0u, 0u, 0u);
      b.v = a.v;
      if (c < H) {
        a.v = *reinterpret_cast<const uint4*>(x + base + c);
        b.v = *reinterpret_cast<const uint4*>(dy + base + c);
      }
      a.unpack(fx[k]);
      b.unpack(fd[k]);
      if (c < H) {
        float g[8];
        load_gamma(c, g);
#pragma unroll
        for (int i = 0; i < 8; ++i) dot += g[i] * fd[k][i] * fx[k][i];
      }
    }
    dot = warp_sum(dot);
    const float coef = dot * rstd * rstd * rstd / H;
#pragma unroll
    for (int k = 0; k < NV; ++k) {
      const int c = lane * 8 + 256 * k;
      if (c >= H) continue;
      float o[8], g[8];
      load_gamma(c, g);
#pragma unroll
      for (int i = 0; i < 8; ++i) {
        o[i] = rstd * g[i] * fd[k][i] - coef * fx[k][i];
        dg[k][i] = fmaf(fd[k][i] * fx[k][i], rstd, dg[k][i]);
      }
      if (ADD_GRAD) {
        bf16x8 e;
        e.v = *reinterpret_cast<const uint4*>(dsum + base + c);
        float fe[8];
        e.unpack(fe);
#pragma unroll
        for (int i = 0; i < 8; ++i) o[i] += fe[i];
      }
      bf16x8 r;
      r.pack(o);
      *reinterpret_cast<uint4*>(dx + base + c) = r.v;
    }
  }
#pragma unroll
  for (int k = 0; k < NV; ++k)
#pragma unroll
    for (int i = 0; i < 8; ++i) red[w][lane * 8 + 256 * k + i] = dg[k][i];
  __syncthreads();
  for (int c = threadIdx.x; c < 256 * NV && c < H; c += 256) {
    float a = 0.f;
#pragma unroll
    for (int ww = 0; ww < 8; ++ww) a += red[ww][c];
    atomicAdd(dgamma + c, a);
  }
}

template <int NV>
static void launch_rmsnorm_bwd_fused(const void* x, const void* dy, const void* dsum, const float* gamma,
                                     const float* rstd, void* dx, float* dgamma, int rows, int H, cudaStream_t st) {
  const int blocks = min((rows + 7) / 8, 2 * num_sms());
  if (dsum)
    rmsnorm_bwd_fused_kernel<NV, true><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                               (const __nv_bfloat16*)dsum, gamma, rstd,
                                                               (__nv_bfloat16*)dx, dgamma, rows, H);
  else
    rmsnorm_bwd_fused_kernel<NV, false><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, nullptr,
                                                                gamma, rstd, (__nv_bfloat16*)dx, dgamma, rows, H);
}

// dgamma[c] += sum_rows dy * x * rstd. Block = 32 x 8 threads over a 64-column strip.
__global__ void rmsnorm_dgamma_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                      const float* __restrict__ rstd, float* __restrict__ dgamma, int rows, int H,
                                      int rows_per_block) {
  __shared__ float red[8][64];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + tx * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float a0 = 0.f, a1 = 0.f;
  if (col < H) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const uint32_t vx = *reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(r) * H + col);
      const uint32_t vd = *reinterpret_cast<const uint32_t*>(dy + static_cast<size_t>(r) * H + col);
      const float s = rstd[r];
      a0 += bf16_lo(vx) * bf16_lo(vd) * s;
      a1 += bf16_hi(vx) * bf16_hi(vd) * s;
    }
  }
  red[ty][tx * 2] = a0;
  red[ty][tx * 2 + 1] = a1;
  __syncthreads();
  if (ty == 0) {
#pragma unroll
    for (int i = 1; i < 8; ++i) {
      a0 += red[i][tx * 2];
      a1 += red[i][tx * 2 + 1];
    }
    if (col < H) {
      atomicAdd(dgamma + col, a0);
      atomicAdd(dgamma + col + 1, a1);
    }
  }
}

// RoPE without QK-norm: no row statistics are needed, so every thread rotates 4 adjacent
// pairs (16 bytes) on its own and a warp covers 512 contiguous bytes.
template <int D, bool BACKWARD>
__global__ void qk_rope_vec_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                                   const float* __restrict__ cos_t, const float* __restrict__ sin_t, long T, int S,
                                   int heads, int ld, int pos0) {
  constexpr int TPH = D / 8;                       // threads per head
  const long total = T * heads * TPH;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int part = i % TPH;
    const long th = i / TPH;
    const int h = th % heads;
    const long t = th / heads;
    const size_t off = static_cast<size_t>(t) * ld + static_cast<size_t>(h) * D + part * 8;
    const int pos = pos0 + static_cast<int>(t % S);
    const uint4 w = *reinterpret_cast<const uint4*>(in + off);
    const float4 c = *reinterpret_cast<const float4*>(cos_t + static_cast<size_t>(pos) * (D / 2) + part * 4);
    float4 sn = *reinterpret_cast<const float4*>(sin_t + static_cast<size_t>(pos) * (D / 2) + part * 4);
    if (BACKWARD) { sn.x = -sn.x; sn.y = -sn.y; sn.z = -sn.z; sn.w = -sn.w; }   // inverse rotation
    uint4 r;
    r.x = pack_bf16(bf16_lo(w.x) * c.x - bf16_hi(w.x) * sn.x, bf16_lo(w.x) * sn.x + bf16_hi(w.x) * c.x);
    r.y = pack_bf16(bf16_lo(w.y) * c.y - bf16_hi(w.y) * sn.y, bf16_lo(w.y) * sn.y + bf16_hi(w.y) * c.y);
    r.z = pack_bf16(bf16_lo(w.z) * c.z - bf16_hi(w.z) * sn.z, bf16_lo(w.z) * sn.z + bf16_hi(w.z) * c.z);
    r.w = pack_bf16(bf16_lo(w.w) * c.w - bf16_hi(w.w) * sn.w, bf16_lo(w.w) * sn.w + bf16_hi(w.w) * c.w);
    *reinterpret_cast<uint4*>(out + off) = r;
  }
}

// ------------------------------------------------------------------ q/k RMSNorm + RoPE
// Works on the fused qkv activation `[T, (Hq + 2 Hkv) * D]` (row stride = ld). One warp
// per (token, head) over the Hq + Hkv rotating heads; lane l owns D/32 consecutive
// elements (D = 64 or 128 -> 1 or 2 adjacent pairs). Output goes to `out` with the same
// row layout (in place when out == qkv). pos = pos0 + (t % S).
template <int D, bool NORM, bool BACKWARD>
__global__ void qk_rope_kernel(const __nv_bfloat16* __restrict__ in, __nv_bfloat16* __restrict__ out,
                               const __nv_bfloat16* __restrict__ pre,  // BACKWARD && NORM: forward input
                               const float* __restrict__ q_gamma, const float* __restrict__ k_gamma,
                               float* __restrict__ rstd_io,            // [T, Hq+Hkv] (NORM)
                               float* __restrict__ dq_gamma, float* __restrict__ dk_gamma,
                               const float* __restrict__ cos_t, const float* __restrict__ sin_t, int T, int S, int Hq,
                               int Hkv, int ld, int pos0, float eps) {
  constexpr int E = D / 32;   // elements per lane (2 or 4)
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const int heads = Hq + Hkv;
  const bool active = gw < T * heads;
  float dg[E];
#pragma unroll
  for (int i = 0; i < E; ++i) dg[i] = 0.f;
  const float* gamma = nullptr;
  bool is_q = true;
  if (active) {
    const int t = gw / heads, h = gw - t * heads;
    is_q = h < Hq;
    const size_t off = static_cast<size_t>(t) * ld + static_cast<size_t>(h) * D + lane * E;
    const int pos = pos0 + (t % S);
    float v[E], c[E / 2], s[E / 2];
    if (E == 2) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(in + off);
      v[0] = bf16_lo(w); v[1] = bf16_hi(w);
    } else {
      const uint2 w = *reinterpret_cast<const uint2*>(in + off);
      v[0] = bf16_lo(w.x); v[1] = bf16_hi(w.x); v[2] = bf16_lo(w.y); v[3] = bf16_hi(w.y);
    }
#pragma unroll
    for (int i = 0; i < E / 2; ++i) {
      c[i] = cos_t[static_cast<size_t>(pos) * (D / 2) + lane * (E / 2) + i];
      s[i] = sin_t[static_cast<size_t>(pos) * (D / 2) + lane * (E / 2) + i];
    }
    if (NORM) gamma = is_q ? q_gamma : k_gamma;
    if (!BACKWARD) {
      if (NORM) {
        float ss = 0.f;
#pragma unroll
        for (int i = 0; i < E; ++i) ss += v[i] * v[i];
        ss = warp_sum(ss);
        const float rstd = rsqrtf(ss / D + eps);
        if (lane == 0) rstd_io[gw] = rstd;
#pragma unroll
        for (int i = 0; i < E; ++i) {
          // round to bf16 between the norm and the rotation, as separate ops would
          v[i] = __bfloat162float(__float2bfloat16(v[i] * rstd * gamma[lane * E + i]));
        }
      }
#pragma unroll
      for (int i = 0; i < E / 2; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        v[2 * i] = a * c[i] - b * s[i];
        v[2 * i + 1] = a * s[i] + b * c[i];
      }
    } else {
      // inverse rotation of the incoming gradient
#pragma unroll
      for (int i = 0; i < E / 2; ++i) {
        const float a = v[2 * i], b = v[2 * i + 1];
        v[2 * i] = a * c[i] + b * s[i];
        v[2 * i + 1] = -a * s[i] + b * c[i];
      }
      if (NORM) {
        float x[E];
        if (E == 2) {
          const uint32_t w = *reinterpret_cast<const uint32_t*>(pre + off);
          x[0] = bf16_lo(w); x[1] = bf16_hi(w);
        } else {
          const uint2 w = *reinterpret_cast<const uint2*>(pre + off);
          x[0] = bf16_lo(w.x); x[1] = bf16_hi(w.x); x[2] = bf16_lo(w.y); x[3] = bf16_hi(w.y);
        }
        const float rstd = rstd_io[gw];
        float dot = 0.f;
#pragma unroll
        for (int i = 0; i < E; ++i) {
          const float g = gamma[lane * E + i];
          dot += g * v[i] * x[i];
          dg[i] = v[i] * x[i] * rstd;
        }
        dot = warp_sum(dot);
        const float coef = dot * rstd * rstd * rstd / D;
#pragma unroll
        for (int i = 0; i < E; ++i) v[i] = rstd * gamma[lane * E + i] * v[i] - coef * x[i];
      }
    }
    if (E == 2) {
      *reinterpret_cast<uint32_t*>(out + off) = pack_bf16(v[0], v[1]);
    } else {
      *reinterpret_cast<uint2*>(out + off) = make_uint2(pack_bf16(v[0], v[1]), pack_bf16(v[2], v[3]));
    }
  }
  if (BACKWARD && NORM) {
    // block-level reduction of the gain gradients, then one atomic per element per block
    __shared__ float acc[2][D];
    for (int i = threadIdx.x; i < 2 * D; i += blockDim.x) (&acc[0][0])[i] = 0.f;
    __syncthreads();
    if (active) {
#pragma unroll
      for (int i = 0; i < E; ++i) atomicAdd(&acc[is_q ? 0 : 1][lane * E + i], dg[i]);
    }
    __syncthreads();
    for (int i = threadIdx.x; i < D; i += blockDim.x) {
      if (acc[0][i] != 0.f) atomicAdd(dq_gamma + i, acc[0][i]);
      if (acc[1][i] != 0.f) atomicAdd(dk_gamma + i, acc[1][i]);
    }
  }
}

// ------------------------------------------------------------------ SwiGLU / y*silu(z)
// x `[rows, 2I]` = [gate | value] with row stride ldx; y `[rows, I]`.
__global__ void swiglu_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long rows, int I,
                                  long ldx) {
  const long n8 = rows * (I / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (I / 8);
    const int c = static_cast<int>(i - r * (I / 8)) * 8;
    bf16x8 g, v;
    g.v = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    v.v = *reinterpret_cast<const uint4*>(x + r * ldx + I + c);
    float fg[8], fv[8];
    g.unpack(fg);
    v.unpack(fv);
#pragma unroll
    for (int k = 0; k < 8; ++k) fg[k] = siluf(fg[k]) * fv[k];
    g.pack(fg);
    *reinterpret_cast<uint4*>(y + r * I + c) = g.v;
  }
}

__global__ void swiglu_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                  __nv_bfloat16* __restrict__ dx, long rows, int I, long ldx) {
  const long n8 = rows * (I / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (I / 8);
    const int c = static_cast<int>(i - r * (I / 8)) * 8;
    bf16x8 g, v, d;
    g.v = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    v.v = *reinterpret_cast<const uint4*>(x + r * ldx + I + c);
    d.v = *reinterpret_cast<const uint4*>(dy + r * I + c);
    float fg[8], fv[8], fd[8], og[8], ov[8];
    g.unpack(fg);
    v.unpack(fv);
    d.unpack(fd);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = sigmoidf_(fg[k]);
      const float sl = fg[k] * sg;
      ov[k] = fd[k] * sl;
      og[k] = fd[k] * fv[k] * (sg + sl * (1.f - sg));
    }
    g.pack(og);
    v.pack(ov);
    *reinterpret_cast<uint4*>(dx + r * 2 * I + c) = g.v;
    *reinterpret_cast<uint4*>(dx + r * 2 * I + I + c) = v.v;
  }
}

// ------------------------------------------------------------------ gated / plain activations of the other families
// ACT: 0 silu, 1 gelu (erf), 2 gelu (tanh approximation), 3 relu. Values and derivatives in fp32.
template <int ACT>
__device__ __forceinline__ float act_value(float x) {
  if (ACT == 0) return siluf(x);
  if (ACT == 1) return 0.5f * x * (1.f + erff(x * 0.70710678118654752f));
  if (ACT == 2) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    return 0.5f * x * (1.f + tanhf(u));
  }
  return fmaxf(x, 0.f);
}
template <int ACT>
__device__ __forceinline__ float act_slope(float x) {
  if (ACT == 0) {
    const float sg = sigmoidf_(x);
    return sg + x * sg * (1.f - sg);
  }
  if (ACT == 1) return 0.5f * (1.f + erff(x * 0.70710678118654752f)) + x * 0.3989422804014327f * __expf(-0.5f * x * x);
  if (ACT == 2) {
    const float u = 0.7978845608028654f * (x + 0.044715f * x * x * x);
    const float t = tanhf(u);
    return 0.5f * (1.f + t) + 0.5f * x * (1.f - t * t) * 0.7978845608028654f * (1.f + 0.134145f * x * x);
  }
  return x > 0.f ? 1.f : 0.f;
}

// GATED: x `[rows, 2I]` = [gate | value] (row stride ldx), y `[rows, I]` = act(gate) * value.
// plain:  x `[rows, I]` (row stride ldx), y `[rows, I]` = act(x).
template <int ACT, bool GATED>
__global__ void act_fwd_kernel(const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ y, long rows, int I, long ldx) {
  const long n8 = rows * (I / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (I / 8);
    const int c = static_cast<int>(i - r * (I / 8)) * 8;
    bf16x8 g, v;
    g.v = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    float fg[8], fv[8];
    g.unpack(fg);
    if (GATED) {
      v.v = *reinterpret_cast<const uint4*>(x + r * ldx + I + c);
      v.unpack(fv);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) fg[k] = GATED ? act_value<ACT>(fg[k]) * fv[k] : act_value<ACT>(fg[k]);
    g.pack(fg);
    *reinterpret_cast<uint4*>(y + r * I + c) = g.v;
  }
}

template <int ACT, bool GATED>
__global__ void act_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                               __nv_bfloat16* __restrict__ dx, long rows, int I, long ldx) {
  const long n8 = rows * (I / 8);
  const int od = GATED ? 2 * I : I;        // dx is contiguous
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (I / 8);
    const int c = static_cast<int>(i - r * (I / 8)) * 8;
    bf16x8 g, v, d;
    g.v = *reinterpret_cast<const uint4*>(x + r * ldx + c);
    d.v = *reinterpret_cast<const uint4*>(dy + r * I + c);
    float fg[8], fv[8], fd[8], og[8], ov[8];
    g.unpack(fg);
    d.unpack(fd);
    if (GATED) {
      v.v = *reinterpret_cast<const uint4*>(x + r * ldx + I + c);
      v.unpack(fv);
    }
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      if (GATED) {
        ov[k] = fd[k] * act_value<ACT>(fg[k]);
        og[k] = fd[k] * fv[k] * act_slope<ACT>(fg[k]);
      } else {
        og[k] = fd[k] * act_slope<ACT>(fg[k]);
      }
    }
    g.pack(og);
    *reinterpret_cast<uint4*>(dx + r * od + c) = g.v;
    if (GATED) {
      v.pack(ov);
      *reinterpret_cast<uint4*>(dx + r * od + I + c) = v.v;
    }
  }
}

// ------------------------------------------------------------------ LayerNorm
// One warp per row, statistics in fp32 (two-pass variance, as the oracle computes it): y = (x - mean) rstd gamma + beta.
__global__ void layernorm_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ gamma,
                                     const float* __restrict__ beta, __nv_bfloat16* __restrict__ y,
                                     float* __restrict__ mean_out, float* __restrict__ rstd_out, int rows, int H, float eps) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const size_t base = static_cast<size_t>(warp) * H;
  float s = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) s += f[i];
  }
  const float mean = warp_sum(s) / H;
  float q = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    float f[8];
    a.unpack(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) q += (f[i] - mean) * (f[i] - mean);
  }
  const float rstd = rsqrtf(warp_sum(q) / H + eps);
  if (lane == 0 && mean_out != nullptr) { mean_out[warp] = mean; rstd_out[warp] = rstd; }
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    float f[8], o[8];
    a.unpack(f);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = (f[i] - mean) * rstd * gamma[c + i] + (beta != nullptr ? beta[c + i] : 0.f);
    a.pack(o);
    *reinterpret_cast<uint4*>(y + base + c) = a.v;
  }
}

// dx = rstd (g - mean(g) - xhat mean(g xhat)) with g = dy gamma, xhat = (x - mean) rstd.
__global__ void layernorm_bwd_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                     const float* __restrict__ gamma, const float* __restrict__ mean_in,
                                     const float* __restrict__ rstd_in, __nv_bfloat16* __restrict__ dx, int rows, int H) {
  const int warp = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (warp >= rows) return;
  const size_t base = static_cast<size_t>(warp) * H;
  const float mean = mean_in[warp], rstd = rstd_in[warp];
  float sg = 0.f, sgx = 0.f;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a, b;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    b.v = *reinterpret_cast<const uint4*>(dy + base + c);
    float fx[8], fd[8];
    a.unpack(fx);
    b.unpack(fd);
#pragma unroll
    for (int i = 0; i < 8; ++i) {
      const float g = fd[i] * gamma[c + i];
      sg += g;
      sgx += g * (fx[i] - mean) * rstd;
    }
  }
  sg = warp_sum(sg) / H;
  sgx = warp_sum(sgx) / H;
  for (int c = lane * 8; c < H; c += 256) {
    bf16x8 a, b;
    a.v = *reinterpret_cast<const uint4*>(x + base + c);
    b.v = *reinterpret_cast<const uint4*>(dy + base + c);
    float fx[8], fd[8], o[8];
    a.unpack(fx);
    b.unpack(fd);
#pragma unroll
    for (int i = 0; i < 8; ++i) o[i] = rstd * (fd[i] * gamma[c + i] - sg - (fx[i] - mean) * rstd * sgx);
    a.pack(o);
    *reinterpret_cast<uint4*>(dx + base + c) = a.v;
  }
}

// dgamma[c] += sum_rows dy xhat, dbeta[c] += sum_rows dy. Block = 32 x 8 threads over a 64-column strip.
__global__ void layernorm_dparams_kernel(const __nv_bfloat16* __restrict__ x, const __nv_bfloat16* __restrict__ dy,
                                         const float* __restrict__ mean, const float* __restrict__ rstd,
                                         float* __restrict__ dgamma, float* __restrict__ dbeta, int rows, int H,
                                         int rows_per_block) {
  __shared__ float red[8][4][64 / 2 + 1];
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  const int col = blockIdx.x * 64 + tx * 2;
  const int r0 = blockIdx.y * rows_per_block;
  const int r1 = min(rows, r0 + rows_per_block);
  float g0 = 0.f, g1 = 0.f, b0 = 0.f, b1 = 0.f;
  if (col < H) {
    for (int r = r0 + ty; r < r1; r += 8) {
      const uint32_t vx = *reinterpret_cast<const uint32_t*>(x + static_cast<size_t>(r) * H + col);
      const uint32_t vd = *reinterpret_cast<const uint32_t*>(dy + static_cast<size_t>(r) * H + col);
      const float m = mean[r], s = rstd[r];
      g0 += bf16_lo(vd) * (bf16_lo(vx) - m) * s;
      g1 += bf16_hi(vd) * (bf16_hi(vx) - m) * s;
      b0 += bf16_lo(vd);
      b1 += bf16_hi(vd);
    }
  }
  red[ty][0][tx] = g0; red[ty][1][tx] = g1; red[ty][2][tx] = b0; red[ty][3][tx] = b1;
  __syncthreads();
  if (ty == 0 && col < H) {
#pragma unroll
    for (int i = 1; i < 8; ++i) { g0 += red[i][0][tx]; g1 += red[i][1][tx]; b0 += red[i][2][tx]; b1 += red[i][3][tx]; }
    atomicAdd(dgamma + col, g0);
    atomicAdd(dgamma + col + 1, g1);
    if (dbeta != nullptr) { atomicAdd(dbeta + col, b0); atomicAdd(dbeta + col + 1, b1); }
  }
}

// out = y * silu(z); y, z may be strided views (row strides ldy / ldz), out contiguous.
__global__ void mul_silu_fwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                                    __nv_bfloat16* __restrict__ out, long rows, int C, long ldy, long ldz) {
  const long n8 = rows * (C / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (C / 8);
    const int c = static_cast<int>(i - r * (C / 8)) * 8;
    bf16x8 a, b;
    a.v = *reinterpret_cast<const uint4*>(y + r * ldy + c);
    b.v = *reinterpret_cast<const uint4*>(z + r * ldz + c);
    float fa[8], fb[8];
    a.unpack(fa);
    b.unpack(fb);
#pragma unroll
    for (int k = 0; k < 8; ++k) fa[k] *= siluf(fb[k]);
    a.pack(fa);
    *reinterpret_cast<uint4*>(out + r * C + c) = a.v;
  }
}

__global__ void mul_silu_bwd_kernel(const __nv_bfloat16* __restrict__ y, const __nv_bfloat16* __restrict__ z,
                                    const __nv_bfloat16* __restrict__ dout, __nv_bfloat16* __restrict__ dy,
                                    __nv_bfloat16* __restrict__ dz, long rows, int C, long ldy, long ldz, long lddy,
                                    long lddz) {
  const long n8 = rows * (C / 8);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8; i += (long)gridDim.x * blockDim.x) {
    const long r = i / (C / 8);
    const int c = static_cast<int>(i - r * (C / 8)) * 8;
    bf16x8 a, b, d;
    a.v = *reinterpret_cast<const uint4*>(y + r * ldy + c);
    b.v = *reinterpret_cast<const uint4*>(z + r * ldz + c);
    d.v = *reinterpret_cast<const uint4*>(dout + r * C + c);
    float fa[8], fb[8], fd[8], oy[8], oz[8];
    a.unpack(fa);
    b.unpack(fb);
    d.unpack(fd);
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float sg = sigmoidf_(fb[k]);
      const float sl = fb[k] * sg;
      oy[k] = fd[k] * sl;
      oz[k] = fd[k] * fa[k] * (sg + sl * (1.f - sg));
    }
    a.pack(oy);
    b.pack(oz);
    *reinterpret_cast<uint4*>(dy + r * lddy + c) = a.v;
    *reinterpret_cast<uint4*>(dz + r * lddz + c) = b.v;
  }
}

// ------------------------------------------------------------------ fused AdamW
// fp32 master / m / v over a flat range; grad fp32 (scaled by grad_scale, e.g. the clip
// coefficient read from device memory); writes the bf16 compute copy when given.
__global__ void adamw_kernel(float* __restrict__ master, float* __restrict__ m, float* __restrict__ v,
                             const float* __restrict__ grad, __nv_bfloat16* __restrict__ param_bf16, long n,
                             const float* __restrict__ grad_scale_ptr, float lr, float beta1, float beta2, float eps,
                             float wd, float bc1, float bc2) {
  const float gs = grad_scale_ptr ? *grad_scale_ptr : 1.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float g = grad[i] * gs;
    float p = master[i];
    const float mi = beta1 * m[i] + (1.f - beta1) * g;
    const float vi = beta2 * v[i] + (1.f - beta2) * g * g;
    m[i] = mi;
    v[i] = vi;
    const float mhat = mi / bc1;
    const float vhat = vi / bc2;
    p = p - lr * wd * p - lr * mhat / (sqrtf(vhat) + eps);
    master[i] = p;
    if (param_bf16) param_bf16[i] = __float2bfloat16(p);
  }
}

// sum of squares of an fp32 range into out[0] (atomic), for the global gradient norm.
__global__ void sumsq_kernel(const float* __restrict__ x, long n, float* __restrict__ out) {
  float acc = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    const float a = x[i];
    acc += a * a;
  }
  acc = warp_sum(acc);
  __shared__ float red[32];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = acc;
  __syncthreads();
  if (w == 0) {
    acc = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    acc = warp_sum(acc);
    if (lane == 0) atomicAdd(out, acc);
  }
}

// ------------------------------------------------------------------ Muon: momentum and parameter update over pointer lists
// A shape group's matrices are separate views of the flat buffers, so each kernel takes device arrays of pointers
// (one per matrix) and every matrix has `per` elements (a multiple of 4).
//   momentum: g = grad * scale; v = mu v + g; u = g + mu v (Nesterov blend) as bf16 into the stacked operand of the
//             Newton-Schulz chain; the gradient is zeroed on the way (it has been consumed).
__global__ void muon_momentum_kernel(float* const* __restrict__ grads, float* __restrict__ v, __nv_bfloat16* __restrict__ u,
                                     long per, const float* __restrict__ scale_ptr, float mu) {
  const float scale = *scale_ptr;
  float* g = grads[blockIdx.y];
  float* vm = v + (long)blockIdx.y * per;
  __nv_bfloat16* um = u + (long)blockIdx.y * per;
  for (long i = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4; i < per; i += (long)gridDim.x * blockDim.x * 4) {
    float4 gg = *reinterpret_cast<const float4*>(g + i);
    float4 vv = *reinterpret_cast<const float4*>(vm + i);
    gg.x *= scale; gg.y *= scale; gg.z *= scale; gg.w *= scale;
    vv.x = fmaf(mu, vv.x, gg.x); vv.y = fmaf(mu, vv.y, gg.y); vv.z = fmaf(mu, vv.z, gg.z); vv.w = fmaf(mu, vv.w, gg.w);
    *reinterpret_cast<float4*>(vm + i) = vv;
    uint2 o;
    o.x = pack_bf16(fmaf(mu, vv.x, gg.x), fmaf(mu, vv.y, gg.y));
    o.y = pack_bf16(fmaf(mu, vv.z, gg.z), fmaf(mu, vv.w, gg.w));
    *reinterpret_cast<uint2*>(um + i) = o;
    *reinterpret_cast<float4*>(g + i) = make_float4(0.f, 0.f, 0.f, 0.f);
  }
}

//   apply: master -= step * update (bf16, stacked); param = bf16(master).
__global__ void muon_apply_kernel(float* const* __restrict__ masters, __nv_bfloat16* const* __restrict__ params,
                                  const __nv_bfloat16* __restrict__ upd, long per, float step) {
  float* m = masters[blockIdx.y];
  __nv_bfloat16* pm = params[blockIdx.y];
  const __nv_bfloat16* um = upd + (long)blockIdx.y * per;
  for (long i = (blockIdx.x * (long)blockDim.x + threadIdx.x) * 4; i < per; i += (long)gridDim.x * blockDim.x * 4) {
    float4 mm = *reinterpret_cast<const float4*>(m + i);
    const uint2 uu = *reinterpret_cast<const uint2*>(um + i);
    mm.x -= step * bf16_lo(uu.x); mm.y -= step * bf16_hi(uu.x); mm.z -= step * bf16_lo(uu.y); mm.w -= step * bf16_hi(uu.y);
    *reinterpret_cast<float4*>(m + i) = mm;
    uint2 o;
    o.x = pack_bf16(mm.x, mm.y);
    o.y = pack_bf16(mm.z, mm.w);
    *reinterpret_cast<uint2*>(pm + i) = o;
  }
}

static inline int grid_for(long work_items, int block) {
  long g = (work_items + block - 1) / block;
  const long cap = static_cast<long>(num_sms()) * 16;
  if (g > cap) g = cap;
  if (g < 1) g = 1;
  return static_cast<int>(g);
}

}  // namespace sb

using namespace sb;

extern "C" int sb_rmsnorm_fwd(const void* x, const void* res, const float* gamma, void* y, void* sum_out,
                              float* rstd, int rows, int H, float eps, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && H > 0 && H % 8 == 0);
  const int blocks = (rows + 7) / 8;
  if (res) {
    rmsnorm_fwd_kernel<true><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)res, gamma,
                                                     (__nv_bfloat16*)y, (__nv_bfloat16*)sum_out, rstd, rows, H, eps);
  } else {
    rmsnorm_fwd_kernel<false><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, nullptr, gamma, (__nv_bfloat16*)y,
                                                      nullptr, rstd, rows, H, eps);
  }
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// dx = d(rmsnorm)/dx applied to dy (+ dsum when given); dgamma (fp32, pre-zeroed or
// accumulating) += sum_rows dy * x * rstd.
extern "C" int sb_rmsnorm_bwd(const void* x, const void* dy, const void* dsum, const float* gamma, const float* rstd,
                              void* dx, float* dgamma, int rows, int H, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && H > 0 && H % 8 == 0);
  if (dgamma && H <= 1536) {
    switch ((H + 255) / 256) {
      case 1: launch_rmsnorm_bwd_fused<1>(x, dy, dsum, gamma, rstd, dx, dgamma, rows, H, st); break;
      case 2: launch_rmsnorm_bwd_fused<2>(x, dy, dsum, gamma, rstd, dx, dgamma, rows, H, st); break;
      case 3: launch_rmsnorm_bwd_fused<3>(x, dy, dsum, gamma, rstd, dx, dgamma, rows, H, st); break;
      case 4: launch_rmsnorm_bwd_fused<4>(x, dy, dsum, gamma, rstd, dx, dgamma, rows, H, st); break;
      case 5: launch_rmsnorm_bwd_fused<5>(x, dy, dsum, gamma, rstd, dx, dgamma, rows, H, st); break;
      default: launch_rmsnorm_bwd_fused<6>(x, dy, dsum, gamma, rstd, dx, dgamma, rows, H, st); break;
    }
    SB_CHECK_CUDA(cudaGetLastError());
    return SB_OK;
  }
  const int blocks = (rows + 7) / 8;
  if (dsum) {
    rmsnorm_bwd_kernel<true><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                     (const __nv_bfloat16*)dsum, gamma, rstd, (__nv_bfloat16*)dx, rows, H);
  } else {
    rmsnorm_bwd_kernel<false><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, nullptr, gamma,
                                                      rstd, (__nv_bfloat16*)dx, rows, H);
  }
  if (dgamma) {
    const int rpb = 512;
    dim3 grid((H + 63) / 64, (rows + rpb - 1) / rpb);
    rmsnorm_dgamma_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, rstd, dgamma, rows, H,
                                                rpb);
  }
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Forward (backward = 0) or backward (1) of optional per-head RMSNorm followed by
// interleaved RoPE over the q and k heads of a fused qkv activation.
extern "C" int sb_qk_rope(const void* in, void* out, const void* pre, const float* q_gamma, const float* k_gamma,
                          float* rstd, float* dq_gamma, float* dk_gamma, const float* cos_t, const float* sin_t, int T,
                          int S, int Hq, int Hkv, int D, int ld, int pos0, float eps, int backward, cudaStream_t st) {
  SB_CHECK_ARG(D == 64 || D == 128);
  SB_CHECK_ARG(T > 0 && S > 0 && ld % 4 == 0);
  const bool norm = q_gamma != nullptr;
  const long warps = static_cast<long>(T) * (Hq + Hkv);
  const int blocks = static_cast<int>((warps + 7) / 8);
#define SB_ROPE(DD, NN, BB)                                                                                          \
  qk_rope_kernel<DD, NN, BB><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)in, (__nv_bfloat16*)out,                   \
                                                     (const __nv_bfloat16*)pre, q_gamma, k_gamma, rstd, dq_gamma,      \
                                                     dk_gamma, cos_t, sin_t, T, S, Hq, Hkv, ld, pos0, eps)
  if (!norm && ld % 8 == 0) {
    const long items = static_cast<long>(T) * (Hq + Hkv) * (D / 8);
    const int vb = grid_for(items, 256);
    const __nv_bfloat16* i_ = (const __nv_bfloat16*)in;
    __nv_bfloat16* o_ = (__nv_bfloat16*)out;
    if (D == 64) {
      if (backward) qk_rope_vec_kernel<64, true><<<vb, 256, 0, st>>>(i_, o_, cos_t, sin_t, T, S, Hq + Hkv, ld, pos0);
      else qk_rope_vec_kernel<64, false><<<vb, 256, 0, st>>>(i_, o_, cos_t, sin_t, T, S, Hq + Hkv, ld, pos0);
    } else {
      if (backward) qk_rope_vec_kernel<128, true><<<vb, 256, 0, st>>>(i_, o_, cos_t, sin_t, T, S, Hq + Hkv, ld, pos0);
      else qk_rope_vec_kernel<128, false><<<vb, 256, 0, st>>>(i_, o_, cos_t, sin_t, T, S, Hq + Hkv, ld, pos0);
    }
  } else if (D == 64) {
    if (norm) { if (backward) SB_ROPE(64, true, true); else SB_ROPE(64, true, false); }
    else      { if (backward) SB_ROPE(64, false, true); else SB_ROPE(64, false, false); }
  } else {
    if (norm) { if (backward) SB_ROPE(128, true, true); else SB_ROPE(128, true, false); }
    else      { if (backward) SB_ROPE(128, false, true); else SB_ROPE(128, false, false); }
  }
#undef SB_ROPE
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_swiglu_fwd(const void* x, void* y, long rows, int I, long ldx, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && I % 8 == 0 && ldx % 8 == 0);
  swiglu_fwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, I,
                                                                  ldx);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_swiglu_bwd(const void* x, const void* dy, void* dx, long rows, int I, long ldx, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && I % 8 == 0 && ldx % 8 == 0);
  swiglu_bwd_kernel<<<grid_for(rows * (I / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,
                                                                  (__nv_bfloat16*)dx, rows, I, ldx);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// act: 0 silu, 1 gelu, 2 gelu_tanh, 3 relu. gated: x `[rows, 2I]` = [gate | value] -> y `[rows, I]`; plain: x `[rows, I]`.
extern "C" int sb_act_fwd(const void* x, void* y, long rows, int I, long ldx, int act, int gated, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && I % 8 == 0 && ldx % 8 == 0 && act >= 0 && act <= 3);
  const int grid = grid_for(rows * (I / 8), 256);
#define SB_ACT(A)                                                                                                        \
  if (gated) act_fwd_kernel<A, true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, I, ldx);   \
  else act_fwd_kernel<A, false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (__nv_bfloat16*)y, rows, I, ldx)
  if (act == 0) { SB_ACT(0); } else if (act == 1) { SB_ACT(1); } else if (act == 2) { SB_ACT(2); } else { SB_ACT(3); }
#undef SB_ACT
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// dx contiguous: `[rows, 2I]` (gated) or `[rows, I]`.
extern "C" int sb_act_bwd(const void* x, const void* dy, void* dx, long rows, int I, long ldx, int act, int gated,
                          cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && I % 8 == 0 && ldx % 8 == 0 && act >= 0 && act <= 3);
  const int grid = grid_for(rows * (I / 8), 256);
#define SB_ACT(A)                                                                                                   \
  if (gated) act_bwd_kernel<A, true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,      \
                                                          (__nv_bfloat16*)dx, rows, I, ldx);                       \
  else act_bwd_kernel<A, false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy,           \
                                                      (__nv_bfloat16*)dx, rows, I, ldx)
  if (act == 0) { SB_ACT(0); } else if (act == 1) { SB_ACT(1); } else if (act == 2) { SB_ACT(2); } else { SB_ACT(3); }
#undef SB_ACT
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// y = layernorm(x; gamma, beta (may be null), eps); mean / rstd (fp32 `[rows]`, may be null) are kept for the backward.
extern "C" int sb_layernorm_fwd(const void* x, const float* gamma, const float* beta, void* y, float* mean, float* rstd,
                                int rows, int H, float eps, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && H > 0 && H % 8 == 0 && ((mean == nullptr) == (rstd == nullptr)));
  layernorm_fwd_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, gamma, beta, (__nv_bfloat16*)y, mean, rstd,
                                                        rows, H, eps);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// dx, and dgamma / dbeta (fp32, accumulate: zero them first; dbeta may be null).
extern "C" int sb_layernorm_bwd(const void* x, const void* dy, const float* gamma, const float* mean, const float* rstd,
                                void* dx, float* dgamma, float* dbeta, int rows, int H, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && H > 0 && H % 8 == 0);
  layernorm_bwd_kernel<<<(rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, gamma, mean, rstd,
                                                        (__nv_bfloat16*)dx, rows, H);
  if (dgamma != nullptr) {
    const int rpb = 512;
    dim3 grid((H + 63) / 64, (rows + rpb - 1) / rpb);
    layernorm_dparams_kernel<<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, (const __nv_bfloat16*)dy, mean, rstd, dgamma,
                                                   dbeta, rows, H, rpb);
  }
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_mul_silu_fwd(const void* y, const void* z, void* out, long rows, int C, long ldy, long ldz,
                               cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && C % 8 == 0 && ldy % 8 == 0 && ldz % 8 == 0);
  mul_silu_fwd_kernel<<<grid_for(rows * (C / 8), 256), 256, 0, st>>>((const __nv_bfloat16*)y, (const __nv_bfloat16*)z,
                                                                    (__nv_bfloat16*)out, rows, C, ldy, ldz);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_mul_silu_bwd(const void* y, const void* z, const void* dout, void* dy, void* dz, long rows, int C,
                               long ldy, long ldz, long lddy, long lddz, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && C % 8 == 0 && ldy % 8 == 0 && ldz % 8 == 0 && lddy % 8 == 0 && lddz % 8 == 0);
  mul_silu_bwd_kernel<<<grid_for(rows * (C / 8), 256), 256, 0, st>>>(
      (const __nv_bfloat16*)y, (const __nv_bfloat16*)z, (const __nv_bfloat16*)dout, (__nv_bfloat16*)dy,
      (__nv_bfloat16*)dz, rows, C, ldy, ldz, lddy, lddz);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Muon momentum over `n` matrices of `per` elements each: grads = device array of n fp32 pointers (16-byte aligned),
// v `[n, per]` fp32, u `[n, per]` bf16 (output), scale_ptr a device scalar. per % 4 == 0. The gradients are zeroed.
extern "C" int sb_muon_momentum(const void* grads, float* v, void* u, int n, long per, const float* scale_ptr, float mu,
                                cudaStream_t st) {
  SB_CHECK_ARG(n > 0 && n <= 65535 && per > 0 && per % 4 == 0);
  int bx = (int)((per / 4 + 255) / 256);
  if (bx > 512) bx = 512;
  muon_momentum_kernel<<<dim3(bx, n), 256, 0, st>>>((float* const*)grads, v, (__nv_bfloat16*)u, per, scale_ptr, mu);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Muon update: masters / params = device arrays of n pointers (fp32 masters, bf16 compute copies), upd `[n, per]` bf16.
extern "C" int sb_muon_apply(const void* masters, const void* params, const void* upd, int n, long per, float step,
                             cudaStream_t st) {
  SB_CHECK_ARG(n > 0 && n <= 65535 && per > 0 && per % 4 == 0);
  int bx = (int)((per / 4 + 255) / 256);
  if (bx > 512) bx = 512;
  muon_apply_kernel<<<dim3(bx, n), 256, 0, st>>>((float* const*)masters, (__nv_bfloat16* const*)params,
                                                 (const __nv_bfloat16*)upd, per, step);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_adamw(float* master, float* m, float* v, const float* grad, void* param_bf16, long n,
                        const float* grad_scale_ptr, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                        float bc2, cudaStream_t st) {
  SB_CHECK_ARG(n > 0);
  adamw_kernel<<<grid_for(n, 256), 256, 0, st>>>(master, m, v, grad, (__nv_bfloat16*)param_bf16, n, grad_scale_ptr, lr,
                                                 beta1, beta2, eps, wd, bc1, bc2);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_sumsq(const float* x, long n, float* out, cudaStream_t st) {
  SB_CHECK_ARG(n > 0);
  sumsq_kernel<<<grid_for(n, 256), 256, 0, st>>>(x, n, out);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
