// Mamba-1 kernels, backward side: segmented selective-scan backward and the depthwise
// conv1d (+SiLU) backward.
//
// Scan backward uses the forward layout (one thread = NPT states of one channel, state
// and its gradient in registers). Segments of 32 steps are visited last to first; each
// starts from the forward pass's checkpoint and rebuilds its states in two levels so that
// nothing but registers is needed: one sweep records the state at every 8th step, then
// each 8-step group is replayed (keeping the 8 pre-step states) and swept in reverse.
// Per step the gradients with respect to delta and u are reduced over the N lanes with
// shuffles; the B_t / C_t gradients (sums over channels) are reduced inside the block
// with shared-memory atomics and written as one partial tile per channel tile, which a
// second kernel sums — no global atomics on the `[B, T, N]` tensors.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int SCANB_SEG = 32;
constexpr int SCANB_SUB = 8;
constexpr int SCANB_THREADS = 256;

__device__ __forceinline__ float softplusb_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }

struct ScanBwdParams {
  const __nv_bfloat16 *u, *delta, *Bm, *Cm, *dy;
  const float *A, *D, *ckpt, *dh_out;      // dh_out: grad wrt final state [B,C,N] or null
  __nv_bfloat16 *du, *ddelta;              // [B,T,C] contiguous
  float *dB_part, *dC_part;                // [tiles][B][T][N]
  float *dA, *dD;                          // [C,N], [C] (atomic accumulate)
  float* dh0;                              // [B,C,N] or null
  int B, T, C;
  long ld_u, ld_d, ld_b, ld_c, ld_dy;
};

template <int N, int NPT>
__global__ void __launch_bounds__(SCANB_THREADS)
selective_scan_bwd_kernel(const ScanBwdParams p) {
  constexpr int LPC = N / NPT;
  constexpr int CH = SCANB_THREADS / LPC;
  constexpr int NSUB = SCANB_SEG / SCANB_SUB;
  extern __shared__ float sm[];
  float* s_dt = sm;                         // [SEG][CH] softplus(delta)
  float* s_sg = s_dt + SCANB_SEG * CH;      // [SEG][CH] sigmoid(delta) = d softplus
  float* s_u = s_sg + SCANB_SEG * CH;
  float* s_dy = s_u + SCANB_SEG * CH;
  float* s_ddt = s_dy + SCANB_SEG * CH;     // outputs
  float* s_duo = s_ddt + SCANB_SEG * CH;
  float* s_B = s_duo + SCANB_SEG * CH;      // [SEG][N]
  float* s_C = s_B + SCANB_SEG * N;
  float* s_dB = s_C + SCANB_SEG * N;
  float* s_dC = s_dB + SCANB_SEG * N;
  const int tid = threadIdx.x;
  const int ch = tid / LPC, ln = tid % LPC;
  const int b = blockIdx.y;
  const int c = blockIdx.x * CH + ch;
  const bool c_ok = c < p.C;
  const int n0 = ln * NPT;
  float A2[NPT], Av[NPT], dh[NPT], dAacc[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    Av[j] = c_ok ? p.A[(long)c * N + n0 + j] : 0.f;
    A2[j] = Av[j] * 1.4426950408889634f;
    dh[j] = (c_ok && p.dh_out) ? p.dh_out[((long)b * p.C + c) * N + n0 + j] : 0.f;
    dAacc[j] = 0.f;
  }
  const float Dc = c_ok ? p.D[c] : 0.f;
  float dDacc = 0.f;
  const int nseg = (p.T + SCANB_SEG - 1) / SCANB_SEG;
  for (int seg = nseg - 1; seg >= 0; --seg) {
    const int t0 = seg * SCANB_SEG;
    const int steps = min(SCANB_SEG, p.T - t0);
    __syncthreads();
    for (int i = tid; i < SCANB_SEG * CH; i += SCANB_THREADS) {
      const int tt = i / CH, cc = i % CH;
      const int cgl = blockIdx.x * CH + cc;
      float dtv = 0.f, sg = 0.f, uv = 0.f, dyv = 0.f;
      if (tt < steps && cgl < p.C) {
        const long row = (long)b * p.T + t0 + tt;
        const float raw = __bfloat162float(p.delta[row * p.ld_d + cgl]);
        dtv = softplusb_(raw);
        sg = 1.f / (1.f + __expf(-raw));
        uv = __bfloat162float(p.u[row * p.ld_u + cgl]);
        dyv = __bfloat162float(p.dy[row * p.ld_dy + cgl]);
      }
      s_dt[i] = dtv; s_sg[i] = sg; s_u[i] = uv; s_dy[i] = dyv;
    }
    for (int i = tid; i < SCANB_SEG * N; i += SCANB_THREADS) {
      const int tt = i / N, n = i % N;
      float bv = 0.f, cv = 0.f;
      if (tt < steps) {
        const long row = (long)b * p.T + t0 + tt;
        bv = __bfloat162float(p.Bm[row * p.ld_b + n]);
        cv = __bfloat162float(p.Cm[row * p.ld_c + n]);
      }
      s_B[i] = bv; s_C[i] = cv; s_dB[i] = 0.f; s_dC[i] = 0.f;
    }
    __syncthreads();
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
#pragma unroll
        for (int k = 0; k < SCANB_SUB; ++k) {
          const int tt = sb_ * SCANB_SUB + k;
          const float dtv = s_dt[tt * CH + ch], duv = dtv * s_u[tt * CH + ch];
#pragma unroll
          for (int j = 0; j < NPT; ++j) h[j] = fmaf(exp2f(dtv * A2[j]), h[j], duv * s_B[tt * N + n0 + j]);
        }
      }
    }
    // ---- level 2: replay each 8-step group, then sweep it in reverse
#pragma unroll
    for (int sb_ = NSUB - 1; sb_ >= 0; --sb_) {
      if (sb_ * SCANB_SUB >= steps) continue;
      float hp[SCANB_SUB][NPT];
#pragma unroll
      for (int j = 0; j < NPT; ++j) hp[0][j] = hs[sb_][j];
#pragma unroll
      for (int k = 0; k < SCANB_SUB - 1; ++k) {
        const int tt = sb_ * SCANB_SUB + k;
        const float dtv = s_dt[tt * CH + ch], duv = dtv * s_u[tt * CH + ch];
#pragma unroll
        for (int j = 0; j < NPT; ++j) hp[k + 1][j] = fmaf(exp2f(dtv * A2[j]), hp[k][j], duv * s_B[tt * N + n0 + j]);
      }
#pragma unroll
      for (int k = SCANB_SUB - 1; k >= 0; --k) {
        const int tt = sb_ * SCANB_SUB + k;
        if (tt >= steps) continue;        // padded tail (dt = u = dy = 0 there anyway)
        const float dtv = s_dt[tt * CH + ch], uv = s_u[tt * CH + ch], dyv = s_dy[tt * CH + ch];
        const float duv = dtv * uv;
        float ddt = 0.f, duacc = 0.f;
#pragma unroll
        for (int j = 0; j < NPT; ++j) {
          const float bv = s_B[tt * N + n0 + j], cv = s_C[tt * N + n0 + j];
          const float dA = exp2f(dtv * A2[j]);
          const float hprev = hp[k][j];
          const float ht = fmaf(dA, hprev, duv * bv);
          const float g = fmaf(cv, dyv, dh[j]);
          if (c_ok) {
            atomicAdd(&s_dC[tt * N + n0 + j], ht * dyv);
            atomicAdd(&s_dB[tt * N + n0 + j], g * duv);
          }
          const float ddA = g * hprev * dA;
          ddt = fmaf(ddA, Av[j], fmaf(g * uv, bv, ddt));
          duacc = fmaf(g * dtv, bv, duacc);
          dAacc[j] = fmaf(ddA, dtv, dAacc[j]);
          dh[j] = g * dA;
        }
#pragma unroll
        for (int o = LPC / 2; o > 0; o >>= 1) {
          ddt += __shfl_xor_sync(0xffffffffu, ddt, o);
          duacc += __shfl_xor_sync(0xffffffffu, duacc, o);
        }
        if (ln == 0) {
          s_ddt[tt * CH + ch] = ddt * s_sg[tt * CH + ch];
          s_duo[tt * CH + ch] = fmaf(Dc, dyv, duacc);
          dDacc = fmaf(dyv, uv, dDacc);
        }
      }
    }
    __syncthreads();
    for (int i = tid; i < steps * CH; i += SCANB_THREADS) {
      const int tt = i / CH, cc = i % CH;
      const int cgl = blockIdx.x * CH + cc;
      if (cgl < p.C) {
        const long o = ((long)b * p.T + t0 + tt) * p.C + cgl;
        p.ddelta[o] = __float2bfloat16(s_ddt[i]);
        p.du[o] = __float2bfloat16(s_duo[i]);
      }
    }
    {
      float* pb = p.dB_part + (((long)blockIdx.x * p.B + b) * p.T + t0) * N;
      float* pc = p.dC_part + (((long)blockIdx.x * p.B + b) * p.T + t0) * N;
      for (int i = tid; i < steps * N; i += SCANB_THREADS) { pb[i] = s_dB[i]; pc[i] = s_dC[i]; }
    }
  }
  if (c_ok) {
#pragma unroll
    for (int j = 0; j < NPT; ++j) {
      atomicAdd(p.dA + (long)c * N + n0 + j, dAacc[j]);
      if (p.dh0) p.dh0[((long)b * p.C + c) * N + n0 + j] = dh[j];
    }
    if (ln == 0) atomicAdd(p.dD + c, dDacc);
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

template <int N, int NPT>
static int launch_scan_bwd(const ScanBwdParams& p, cudaStream_t st) {
  constexpr int LPC = N / NPT, CH = SCANB_THREADS / LPC;
  const int smem = (6 * SCANB_SEG * CH + 4 * SCANB_SEG * N) * sizeof(float);
  auto kern = selective_scan_bwd_kernel<N, NPT>;
  if (smem > 48 * 1024) SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.C + CH - 1) / CH, p.B);
  kern<<<grid, SCANB_THREADS, smem, st>>>(p);
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

// Scan backward. dB_part/dC_part: scratch of tiles*B*T*N floats each, tiles =
// ceil(C / (256 / (N / NPT))) with NPT = 8 for N >= 64 else 4. dA/dD accumulate (zero them
// first). dBm/dCm outputs are bf16 `[B,T,N]` with row strides ld_db / ld_dc.
extern "C" int sb_scan_bwd(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm,
                           const float* D, const void* dy, const float* ckpt, const float* dh_out, void* du,
                           void* ddelta, float* dB_part, float* dC_part, void* dBm, void* dCm, float* dA, float* dD,
                           float* dh0, int B, int T, int C, int N, long ld_u, long ld_d, long ld_b, long ld_c,
                           long ld_dy, long ld_db, long ld_dc, cudaStream_t st) {
  SB_CHECK_ARG(B > 0 && T > 0 && C > 0);
  ScanBwdParams p;
  p.u = (const __nv_bfloat16*)u; p.delta = (const __nv_bfloat16*)delta; p.Bm = (const __nv_bfloat16*)Bm;
  p.Cm = (const __nv_bfloat16*)Cm; p.dy = (const __nv_bfloat16*)dy; p.A = A; p.D = D; p.ckpt = ckpt;
  p.dh_out = dh_out; p.du = (__nv_bfloat16*)du; p.ddelta = (__nv_bfloat16*)ddelta; p.dB_part = dB_part;
  p.dC_part = dC_part; p.dA = dA; p.dD = dD; p.dh0 = dh0; p.B = B; p.T = T; p.C = C;
  p.ld_u = ld_u; p.ld_d = ld_d; p.ld_b = ld_b; p.ld_c = ld_c; p.ld_dy = ld_dy;
  int rc, ch;
  switch (N) {
    case 8: rc = launch_scan_bwd<8, 4>(p, st); ch = 256 / 2; break;
    case 16: rc = launch_scan_bwd<16, 4>(p, st); ch = 256 / 4; break;
    case 32: rc = launch_scan_bwd<32, 4>(p, st); ch = 256 / 8; break;
    case 64: rc = launch_scan_bwd<64, 8>(p, st); ch = 256 / 8; break;
    case 128: rc = launch_scan_bwd<128, 8>(p, st); ch = 256 / 16; break;
    case 256: rc = launch_scan_bwd<256, 8>(p, st); ch = 256 / 32; break;
    default: return SB_ERR_ARG;
  }
  if (rc) return rc;
  const int tiles = (C + ch - 1) / ch;
  const long per_tile = (long)B * T * N;
  const int blocks = (int)((per_tile + 255) / 256 < 148 * 8 ? (per_tile + 255) / 256 : 148 * 8);
  scan_reduce_parts_kernel<<<blocks, 256, 0, st>>>(dB_part, (__nv_bfloat16*)dBm, tiles, per_tile, N, ld_db);
  scan_reduce_parts_kernel<<<blocks, 256, 0, st>>>(dC_part, (__nv_bfloat16*)dCm, tiles, per_tile, N, ld_dc);
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
