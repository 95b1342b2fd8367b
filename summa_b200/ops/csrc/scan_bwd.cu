// Mamba-1 kernels, backward side: segmented selective-scan backward and the depthwise
// conv1d (+SiLU) backward.
//
// Scan backward uses the forward layout (lane = channel, warp = 8 states, state and its
// gradient in registers). Segments of 32 steps are visited last to first; each
// starts from the forward pass's checkpoint and rebuilds its states in two levels: one sweep
// records the state at every 8th step (registers), then each 8-step group is replayed
// (its 8 pre-step states go to a per-thread column of shared memory, so the step loops stay
// rolled: small code, 128 registers, two blocks per SM) and swept in reverse.
// Per step the B_t / C_t gradients (sums over channels) are reduced over the warp's 32
// channels with a 16-shuffle recursive-halving reduction and written as one partial tile
// per 32-channel block, which a second kernel sums; the delta / u gradients (sums over
// states) are combined across warps in shared memory. No global atomics touch the
// `[B, T, N]` or `[B, T, C]` tensors.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int SCANB_SEG = 32;
constexpr int SCANB_SUB = 8;
constexpr int SCANB_THREADS = 256;

__device__ __forceinline__ float softplusb_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

struct ScanBwdParams {
  const __nv_bfloat16 *u, *delta, *Bm, *Cm, *dy;
  const float *A, *ckpt, *dh_out;          // dh_out: grad wrt final state [B,C,N] or null
  float *ddt_part, *du_part;               // [NS][B][T][C] partial sums over this block's states
  float *dB_part, *dC_part;                // [C/32 tiles][B][T][N]
  float *dA, *dD;                          // [C,N], [C] (atomic accumulate over batch)
  float* dh0;                              // [B,C,N] or null
  int B, T, C;
  long ld_u, ld_d, ld_b, ld_c, ld_dy;
};

// Sum V per-lane values over the 32 lanes of a warp with V + log2(32/V) ... shuffles
// (recursive halving): afterwards lane L holds the total of value index
// bitreverse-free mapping idx(L) = ((L>>4)&1)*V/2 + ((L>>3)&1)*V/4 + ... (see reduce_index).
template <int V>
__device__ __forceinline__ float warp_reduce_values(float (&v)[V], int lane) {
  if constexpr (V == 1) {
    float x = v[0];
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) x += __shfl_xor_sync(0xffffffffu, x, o);
    return x;
  } else {
    // generic: halve the value count at offsets 16, 8, 4, ... then finish with plain adds
    float cur[V];
#pragma unroll
    for (int i = 0; i < V; ++i) cur[i] = v[i];
    int off = 16;
    int cnt = V;
#pragma unroll
    for (int lvl = 0; lvl < 5; ++lvl) {
      if (cnt > 1) {
        const bool hi = (lane & off) != 0;
        const int half = cnt / 2;
#pragma unroll
        for (int i = 0; i < V / 2; ++i) {
          if (i < half) {
            const float send = hi ? cur[i] : cur[i + half];
            const float keep = hi ? cur[i + half] : cur[i];
            cur[i] = keep + __shfl_xor_sync(0xffffffffu, send, off);
          }
        }
        cnt = half;
      } else {
        cur[0] += __shfl_xor_sync(0xffffffffu, cur[0], off);
      }
      off >>= 1;
    }
    return cur[0];
  }
}
// which of the V values lane `lane` ends up holding after warp_reduce_values<V>
template <int V>
__device__ __forceinline__ int reduce_index(int lane) {
  int idx = 0, off = 16, cnt = V;
#pragma unroll
  for (int lvl = 0; lvl < 5; ++lvl) {
    if (cnt > 1) {
      cnt >>= 1;
      if (lane & off) idx += cnt;
    }
    off >>= 1;
  }
  return idx;
}

// Lane = channel, warp = 8 consecutive states; a block covers 32 channels x NB states of
// one batch row (blockIdx.z selects which NB-state slice when N > NB).
template <int N, int NB>
__global__ void __launch_bounds__(32 * (NB / 8), NB >= 64 ? 2 : 4)
selective_scan_bwd_kernel(const ScanBwdParams p) {
  constexpr int NPT = 8;
  constexpr int NW = NB / NPT;
  constexpr int THREADS = 32 * NW;
  constexpr int CH = 32;
  constexpr int NSUB = SCANB_SEG / SCANB_SUB;
  extern __shared__ float sm[];
  float* s_dt = sm;                         // [SEG][CH] softplus(delta)
  float* s_u = s_dt + SCANB_SEG * CH;
  float* s_dy = s_u + SCANB_SEG * CH;
  float* s_ddt = s_dy + SCANB_SEG * CH;     // outputs (sums over this block's states)
  float* s_duo = s_ddt + SCANB_SEG * CH;
  float* s_B = s_duo + SCANB_SEG * CH;      // [SEG][NB]
  float* s_C = s_B + SCANB_SEG * NB;
  float* s_hp = s_C + SCANB_SEG * NB;       // [SUB][NPT][THREADS] pre-step states of the group being swept
  const int tid = threadIdx.x;
  const int ch = tid & 31, wn = tid >> 5;
  const int b = blockIdx.y;
  const int c = blockIdx.x * CH + ch;
  const bool c_ok = c < p.C;
  const int nb0 = blockIdx.z * NB;          // first state of this block
  const int n0 = nb0 + wn * NPT;            // first state of this thread
  float A2[NPT], Av[NPT], dh[NPT], dAacc[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    Av[j] = c_ok ? p.A[(long)c * N + n0 + j] : 0.f;
    A2[j] = Av[j] * 1.4426950408889634f;
    dh[j] = (c_ok && p.dh_out) ? p.dh_out[((long)b * p.C + c) * N + n0 + j] : 0.f;
    dAacc[j] = 0.f;
  }
  float dDacc = 0.f;
  const int ridx = reduce_index<2 * NPT>(ch);          // which (tensor, j) this lane stores
  const int nseg = (p.T + SCANB_SEG - 1) / SCANB_SEG;
  for (int seg = nseg - 1; seg >= 0; --seg) {
    const int t0 = seg * SCANB_SEG;
    const int steps = min(SCANB_SEG, p.T - t0);
    __syncthreads();
    for (int i = tid; i < SCANB_SEG * CH; i += THREADS) {
      const int tt = i >> 5, cc = i & 31;
      const int cgl = blockIdx.x * CH + cc;
      float dtv = 0.f, uv = 0.f, dyv = 0.f;
      if (tt < steps && cgl < p.C) {
        const long row = (long)b * p.T + t0 + tt;
        dtv = softplusb_(__bfloat162float(p.delta[row * p.ld_d + cgl]));
        uv = __bfloat162float(p.u[row * p.ld_u + cgl]);
        dyv = __bfloat162float(p.dy[row * p.ld_dy + cgl]);
      }
      s_dt[i] = dtv; s_u[i] = uv; s_dy[i] = dyv; s_ddt[i] = 0.f; s_duo[i] = 0.f;
    }
    for (int i = tid; i < SCANB_SEG * NB; i += THREADS) {
      const int tt = i / NB, n = i % NB;
      float bv = 0.f, cv = 0.f;
      if (tt < steps) {
        const long row = (long)b * p.T + t0 + tt;
        bv = __bfloat162float(p.Bm[row * p.ld_b + nb0 + n]);
        cv = __bfloat162float(p.Cm[row * p.ld_c + nb0 + n]);
      }
      s_B[i] = bv; s_C[i] = cv;
    }
    __syncthreads();
    const int nl = wn * NPT;                 // state offset inside the block's shared tiles
    // ---- level 1: states at every 8th step
    float hs[NSUB][NPT];
    {
      float h[NPT];
      const float* ck = p.ckpt + (((long)b * nseg + seg) * p.C + (c_ok ? c : 0)) * N + n0;
#pragma unroll
      for (int j = 0; j < NPT; ++j) h[j] = c_ok ? ck[j] : 0.f;
#pragma unroll
      for (int sb_ = 0; sb_ < NSUB; ++sb_) {
#pragma unroll
        for (int j = 0; j < NPT; ++j) hs[sb_][j] = h[j];
        if (sb_ == NSUB - 1) break;
#pragma unroll 1
        for (int k = 0; k < SCANB_SUB; ++k) {
          const int tt = sb_ * SCANB_SUB + k;
          const float dtv = s_dt[tt * CH + ch], duv = dtv * s_u[tt * CH + ch];
#pragma unroll
          for (int j = 0; j < NPT; ++j) h[j] = fmaf(exp2f(dtv * A2[j]), h[j], duv * s_B[tt * NB + nl + j]);
        }
      }
    }
    // ---- level 2: replay each 8-step group, then sweep it in reverse
#pragma unroll
    for (int sb_ = NSUB - 1; sb_ >= 0; --sb_) {
      if (sb_ * SCANB_SUB >= steps) continue;
      {
        float h[NPT];
#pragma unroll
        for (int j = 0; j < NPT; ++j) { h[j] = hs[sb_][j]; s_hp[(0 * NPT + j) * THREADS + tid] = h[j]; }
#pragma unroll 1
        for (int k = 0; k < SCANB_SUB - 1; ++k) {
          const int tt = sb_ * SCANB_SUB + k;
          const float dtv = s_dt[tt * CH + ch], duv = dtv * s_u[tt * CH + ch];
#pragma unroll
          for (int j = 0; j < NPT; ++j) {
            h[j] = fmaf(exp2f(dtv * A2[j]), h[j], duv * s_B[tt * NB + nl + j]);
            s_hp[((k + 1) * NPT + j) * THREADS + tid] = h[j];
          }
        }
      }
#pragma unroll 1
      for (int k = SCANB_SUB - 1; k >= 0; --k) {
        const int tt = sb_ * SCANB_SUB + k;
        if (tt >= steps) continue;        // uniform across the block
        const float dtv = s_dt[tt * CH + ch], uv = s_u[tt * CH + ch], dyv = s_dy[tt * CH + ch];
        const float duv = dtv * uv;
        float ddt = 0.f, duacc = 0.f;
        float red[2 * NPT];               // [0,NPT): dB contributions, [NPT,2NPT): dC contributions
#pragma unroll
        for (int j = 0; j < NPT; ++j) {
          const float bv = s_B[tt * NB + nl + j], cv = s_C[tt * NB + nl + j];
          const float dA = exp2f(dtv * A2[j]);
          const float hprev = s_hp[(k * NPT + j) * THREADS + tid];
          const float ht = fmaf(dA, hprev, duv * bv);
          const float g = fmaf(cv, dyv, dh[j]);
          red[j] = g * duv;
          red[NPT + j] = ht * dyv;
          const float ddA = g * hprev * dA;
          ddt = fmaf(ddA, Av[j], fmaf(g * uv, bv, ddt));
          duacc = fmaf(g * dtv, bv, duacc);
          dAacc[j] = fmaf(ddA, dtv, dAacc[j]);
          dh[j] = g * dA;
        }
        // sums over the warp's 32 channels: 16 values, 16 shuffles; each result lands in 2 lanes
        const float tot = warp_reduce_values<2 * NPT>(red, ch);
        if ((ch & 1) == 0) {
          const long o = (((long)blockIdx.x * p.B + b) * p.T + t0 + tt) * N + n0;
          if (ridx < NPT) p.dB_part[o + ridx] = tot;
          else p.dC_part[o + ridx - NPT] = tot;
        }
        if (NW == 1) { s_ddt[tt * CH + ch] = ddt; s_duo[tt * CH + ch] = duacc; }
        else { atomicAdd(&s_ddt[tt * CH + ch], ddt); atomicAdd(&s_duo[tt * CH + ch], duacc); }
        if (wn == 0 && blockIdx.z == 0) dDacc = fmaf(dyv, uv, dDacc);
      }
    }
    __syncthreads();
    {
      float* pd = p.ddt_part + ((long)blockIdx.z * p.B + b) * p.T * p.C;
      float* pu = p.du_part + ((long)blockIdx.z * p.B + b) * p.T * p.C;
      for (int i = tid; i < steps * CH; i += THREADS) {
        const int tt = i >> 5, cc = i & 31;
        const int cgl = blockIdx.x * CH + cc;
        if (cgl < p.C) {
          const long o = ((long)t0 + tt) * p.C + cgl;
          pd[o] = s_ddt[i];
          pu[o] = s_duo[i];
        }
      }
    }
  }
  if (c_ok) {
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
      atomicAdd(p.dA + (long)c * N + n0 + j, dAacc[j]);
      if (p.dh0) p.dh0[((long)b * p.C + c) * N + n0 + j] = dh[j];
    }
    if (wn == 0 && blockIdx.z == 0) atomicAdd(p.dD + c, dDacc);
  }
}

// out[b,t,n] (bf16, row stride ld) = sum over channel tiles of the partial tiles
__global__ void scan_reduce_parts_kernel(const float* __restrict__ part, __nv_bfloat16* __restrict__ out, int tiles,
                                         long per_tile, int N, long ld) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < per_tile; i += (long)gridDim.x * blockDim.x) {
    float a = 0.f;
    for (int t = 0; t < tiles; ++t) a += part[(long)t * per_tile + i];
    const long row = i / N;
    out[row * ld + (i - row * N)] = __float2bfloat16(a);
  }
}

// ddelta = (sum_s ddt_part[s]) * sigmoid(delta);  du = sum_s du_part[s] + D * dy
__global__ void scan_combine_kernel(const float* __restrict__ ddt_part, const float* __restrict__ du_part,
                                    const __nv_bfloat16* __restrict__ delta, const __nv_bfloat16* __restrict__ dy,
                                    const float* __restrict__ D, __nv_bfloat16* __restrict__ ddelta,
                                    __nv_bfloat16* __restrict__ du, int ns, long rows, int C, long ld_d, long ld_dy) {
  const long total = rows * C;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const long r = i / C;
    const int c = i - r * C;
    float a = 0.f, e = 0.f;
    for (int s = 0; s < ns; ++s) { a += ddt_part[(long)s * total + i]; e += du_part[(long)s * total + i]; }
    const float raw = __bfloat162float(delta[r * ld_d + c]);
    const float sg = 1.f / (1.f + __expf(-raw));
    ddelta[i] = __float2bfloat16(a * sg);
    du[i] = __float2bfloat16(fmaf(D[c], __bfloat162float(dy[r * ld_dy + c]), e));
  }
}

template <int N, int NB>
static int launch_scan_bwd(const ScanBwdParams& p, cudaStream_t st) {
  constexpr int THREADS = 32 * (NB / 8);
  const int smem = (5 * SCANB_SEG * 32 + 2 * SCANB_SEG * NB + SCANB_SUB * 8 * THREADS) * sizeof(float);
  auto kern = selective_scan_bwd_kernel<N, NB>;
  if (smem > 48 * 1024) SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.C + 31) / 32, p.B, N / NB);
  kern<<<grid, THREADS, smem, st>>>(p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// ---------------------------------------------------------------------------- conv1d backward
// dy is the gradient of silu(conv(x)+b) (or of the plain conv when silu == 0).
// Thread = 8 channels x TT steps; block = 32 channel groups x 8 time chunks.
template <int K, bool SILU>
__global__ void __launch_bounds__(256)
conv1d_bwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, const float* __restrict__ bias,
                  const __nv_bfloat16* __restrict__ dy, __nv_bfloat16* __restrict__ dx, float* __restrict__ dw,
                  float* __restrict__ db, int B, int T, int C, long ldx, long lddx, int t_per_thread) {
  const int lane = threadIdx.x & 31, wy = threadIdx.x >> 5;
  const int cg = blockIdx.x * 32 + lane;
  const int c0 = cg * 8;
  const int b = blockIdx.z;
  const int t_begin = (blockIdx.y * 8 + wy) * t_per_thread;
  const bool ok = c0 < C;
  float wk[K][8], bs[8], gw[K][8], gb[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    bs[j] = (ok && bias) ? bias[c0 + j] : 0.f;
    gb[j] = 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) { wk[k][j] = ok ? w[(c0 + j) * K + k] : 0.f; gw[k][j] = 0.f; }
  }
  auto load8 = [&](const __nv_bfloat16* base, long ld, int t, float* o) {
    if (ok && t >= 0 && t < T) {
      const uint4 v = *reinterpret_cast<const uint4*>(base + ((long)b * T + t) * ld + c0);
      o[0] = bf16_lo(v.x); o[1] = bf16_hi(v.x); o[2] = bf16_lo(v.y); o[3] = bf16_hi(v.y);
      o[4] = bf16_lo(v.z); o[5] = bf16_hi(v.z); o[6] = bf16_lo(v.w); o[7] = bf16_hi(v.w);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) o[j] = 0.f;
    }
  };
  // dpre[t] for t in [t_begin, t_begin + tpt + K - 1): needs x[t-K+1 .. t]
  // dx[t] = sum_k w[k] * dpre[t + (K-1-k)];  dw[k] += dpre[t] * x[t-(K-1-k)]
  float xw[2 * K - 1][8];     // x window: xw[i] = x[t - (K-1) + i], i in [0, 2K-1) covers t..t+K-1 lookahead
  float dp[K][8];             // dp[i] = dpre[t + i]
  // initialise windows for t = t_begin
#pragma unroll
  for (int i = 0; i < 2 * K - 1; ++i) load8(x, ldx, t_begin - (K - 1) + i, xw[i]);
  auto dpre_at = [&](int i, int t, float* o) {
    // dpre at time t using x window positions i-(K-1)..i relative to xw index base
    float g[8];
    load8(dy, (long)C, t, g);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = bs[j];
#pragma unroll
      for (int k = 0; k < K; ++k) a = fmaf(wk[k][j], xw[i + k][j], a);
      if (SILU) {
        const float sg = 1.f / (1.f + __expf(-a));
        o[j] = g[j] * sg * (1.f + a * (1.f - sg));
      } else {
        o[j] = g[j];
      }
    }
  };
#pragma unroll
  for (int i = 0; i < K; ++i) dpre_at(i, t_begin + i, dp[i]);
  for (int tt = 0; tt < t_per_thread; ++tt) {
    const int t = t_begin + tt;
    if (t >= T) break;
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = 0.f;
#pragma unroll
      for (int k = 0; k < K; ++k) a = fmaf(wk[k][j], dp[K - 1 - k][j], a);
      o[j] = a;
      gb[j] += dp[0][j];
#pragma unroll
      for (int k = 0; k < K; ++k) gw[k][j] = fmaf(dp[0][j], xw[k][j], gw[k][j]);
    }
    if (ok) {
      uint4 ov;
      ov.x = pack_bf16(o[0], o[1]); ov.y = pack_bf16(o[2], o[3]); ov.z = pack_bf16(o[4], o[5]); ov.w = pack_bf16(o[6], o[7]);
      *reinterpret_cast<uint4*>(dx + ((long)b * T + t) * lddx + c0) = ov;
    }
    // slide both windows by one step
#pragma unroll
    for (int i = 0; i < 2 * K - 2; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) xw[i][j] = xw[i + 1][j];
    load8(x, ldx, t + K, xw[2 * K - 2]);
#pragma unroll
    for (int i = 0; i < K - 1; ++i)
#pragma unroll
      for (int j = 0; j < 8; ++j) dp[i][j] = dp[i + 1][j];
    dpre_at(K - 1, t + K, dp[K - 1]);
  }
  // reduce the parameter gradients over the 8 time-chunk warps, then one atomic per value
  __shared__ float red[8][32][8 * (K + 1) + 1];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    red[wy][lane][j] = gb[j];
#pragma unroll
    for (int k = 0; k < K; ++k) red[wy][lane][8 + k * 8 + j] = gw[k][j];
  }
  __syncthreads();
  if (wy == 0 && ok) {
    for (int v = 0; v < 8 * (K + 1); ++v) {
      float a = 0.f;
#pragma unroll
      for (int r = 0; r < 8; ++r) a += red[r][lane][v];
      if (v < 8) atomicAdd(db + c0 + v, a);
      else { const int k = (v - 8) / 8, j = (v - 8) % 8; atomicAdd(dw + (c0 + j) * K + k, a); }
    }
  }
}

}  // namespace sb

using namespace sb;

// Scan backward. Scratch (fp32): dB_part/dC_part `[ceil(C/32)][B][T][N]`, ddt_part/du_part
// `[max(1, N/64)][B][T][C]`. dA/dD accumulate (zero them first). du/ddelta are bf16
// `[B,T,C]` contiguous; dBm/dCm bf16 `[B,T,N]` with row strides ld_db / ld_dc.
extern "C" int sb_scan_bwd(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm,
                           const float* D, const void* dy, const float* ckpt, const float* dh_out, void* du,
                           void* ddelta, float* dB_part, float* dC_part, float* ddt_part, float* du_part, void* dBm,
                           void* dCm, float* dA, float* dD, float* dh0, int B, int T, int C, int N, long ld_u,
                           long ld_d, long ld_b, long ld_c, long ld_dy, long ld_db, long ld_dc, cudaStream_t st) {
  SB_CHECK_ARG(B > 0 && T > 0 && C > 0);
  ScanBwdParams p;
  p.u = (const __nv_bfloat16*)u; p.delta = (const __nv_bfloat16*)delta; p.Bm = (const __nv_bfloat16*)Bm;
  p.Cm = (const __nv_bfloat16*)Cm; p.dy = (const __nv_bfloat16*)dy; p.A = A; p.ckpt = ckpt;
  p.dh_out = dh_out; p.ddt_part = ddt_part; p.du_part = du_part; p.dB_part = dB_part;
  p.dC_part = dC_part; p.dA = dA; p.dD = dD; p.dh0 = dh0; p.B = B; p.T = T; p.C = C;
  p.ld_u = ld_u; p.ld_d = ld_d; p.ld_b = ld_b; p.ld_c = ld_c; p.ld_dy = ld_dy;
  int rc, ns = 1;
  switch (N) {
    case 8: rc = launch_scan_bwd<8, 8>(p, st); break;
    case 16: rc = launch_scan_bwd<16, 16>(p, st); break;
    case 32: rc = launch_scan_bwd<32, 32>(p, st); break;
    case 64: rc = launch_scan_bwd<64, 64>(p, st); break;
    case 128: rc = launch_scan_bwd<128, 64>(p, st); ns = 2; break;
    case 256: rc = launch_scan_bwd<256, 64>(p, st); ns = 4; break;
    default: return SB_ERR_ARG;
  }
  if (rc) return rc;
  const int tiles = (C + 31) / 32;
  const long per_tile = (long)B * T * N;
  const int cap = num_sms() * 8;
  int blocks = (int)((per_tile + 255) / 256 < cap ? (per_tile + 255) / 256 : cap);
  scan_reduce_parts_kernel<<<blocks, 256, 0, st>>>(dB_part, (__nv_bfloat16*)dBm, tiles, per_tile, N, ld_db);
  scan_reduce_parts_kernel<<<blocks, 256, 0, st>>>(dC_part, (__nv_bfloat16*)dCm, tiles, per_tile, N, ld_dc);
  const long tot = (long)B * T * C;
  blocks = (int)((tot + 255) / 256 < cap ? (tot + 255) / 256 : cap);
  scan_combine_kernel<<<blocks, 256, 0, st>>>(ddt_part, du_part, (const __nv_bfloat16*)delta, (const __nv_bfloat16*)dy,
                                              D, (__nv_bfloat16*)ddelta, (__nv_bfloat16*)du, ns, (long)B * T, C, ld_d,
                                              ld_dy);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// conv1d backward: dx `[B,T,C]` (row stride lddx), dw `[C,K]`, db `[C]` accumulate (fp32).
extern "C" int sb_conv1d_bwd(const void* x, const float* w, const float* bias, const void* dy, void* dx, float* dw,
                             float* db, int B, int T, int C, int K, long ldx, long lddx, int silu, cudaStream_t st) {
  SB_CHECK_ARG(B > 0 && T > 0 && C % 8 == 0 && ldx % 8 == 0 && lddx % 8 == 0 && K >= 2 && K <= 4);
  const int tpt = 32;
  dim3 grid((C / 8 + 31) / 32, (T + 8 * tpt - 1) / (8 * tpt), B);
#define SB_CONVB(KK)                                                                                               \
  if (silu) conv1d_bwd_kernel<KK, true><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, w, bias, (const __nv_bfloat16*)dy, \
                                                              (__nv_bfloat16*)dx, dw, db, B, T, C, ldx, lddx, tpt);  \
  else conv1d_bwd_kernel<KK, false><<<grid, 256, 0, st>>>((const __nv_bfloat16*)x, w, bias, (const __nv_bfloat16*)dy,    \
                                                          (__nv_bfloat16*)dx, dw, db, B, T, C, ldx, lddx, tpt)
  if (K == 4) { SB_CONVB(4); } else if (K == 3) { SB_CONVB(3); } else { SB_CONVB(2); }
#undef SB_CONVB
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
