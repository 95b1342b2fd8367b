// Mamba-1 kernels, forward side: causal depthwise conv1d (+SiLU), the segmented
// selective scan for training / prefill, and the single-token decode step.
//
// Scan layout: one thread owns 8 consecutive states of one channel and carries them in
// registers for the whole sequence. A block covers 32 channels (one per lane) of one batch
// row with N / 8 warps (one per group of 8 states) and walks the sequence in 32-step
// segments whose inputs (softplus(delta), u, B_t, C_t) are staged in shared memory as
// fp32. At every segment start the state is written to a checkpoint tensor for the
// backward pass. This removes the reference design's N <= 16 limit: N = 8 .. 256 are
// supported (d_state 128 uses 16 warps).
//   dt = softplus(delta); h_t = exp(dt*A) h_{t-1} + dt*u_t*B_t; y_t = <h_t, C_t> + D u_t
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int SCAN_SEG = 32;
constexpr int SCAN_THREADS = 256;

__device__ __forceinline__ float softplusf_(float x) { return x > 20.f ? x : log1pf(__expf(x)); }
__device__ __forceinline__ float silu_f(float x) { return x / (1.f + __expf(-x)); }

// ---------------------------------------------------------------------------- conv1d + SiLU
// x `[B, T, C]` (row stride ldx), w `[C, K]` fp32, bias `[C]` fp32, state `[B, C, K-1]`
// (inputs preceding t = 0, may be null), y `[B, T, C]` contiguous. One thread: 8 channels
// x TT consecutive steps with a sliding window.
template <int K, bool SILU>
__global__ void conv1d_fwd_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w,
                                  const float* __restrict__ bias, const __nv_bfloat16* __restrict__ state,
                                  __nv_bfloat16* __restrict__ y, int B, int T, int C, long ldx) {
  constexpr int TT = 8;
  const int c8 = C / 8;
  const long idx = blockIdx.x * (long)blockDim.x + threadIdx.x;
  const int tchunks = (T + TT - 1) / TT;
  if (idx >= (long)B * tchunks * c8) return;
  const int cg = idx % c8;
  const int tc = (idx / c8) % tchunks;
  const int b = idx / ((long)c8 * tchunks);
  const int c0 = cg * 8, t0 = tc * TT;
  float wk[K][8], bs[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) {
    bs[j] = bias ? bias[c0 + j] : 0.f;
#pragma unroll
    for (int k = 0; k < K; ++k) wk[k][j] = w[(c0 + j) * K + k];
  }
  float win[K][8];   // win[k] = x[t - (K-1) + k]
#pragma unroll
  for (int k = 0; k < K - 1; ++k) {
    const int t = t0 - (K - 1) + k;
    if (t >= 0) {
      const uint4 v = *reinterpret_cast<const uint4*>(x + ((long)b * T + t) * ldx + c0);
      win[k][0] = bf16_lo(v.x); win[k][1] = bf16_hi(v.x); win[k][2] = bf16_lo(v.y); win[k][3] = bf16_hi(v.y);
      win[k][4] = bf16_lo(v.z); win[k][5] = bf16_hi(v.z); win[k][6] = bf16_lo(v.w); win[k][7] = bf16_hi(v.w);
    } else if (state != nullptr) {
      const int si = (K - 1) + t;     // index into the K-1 saved inputs
#pragma unroll
      for (int j = 0; j < 8; ++j) win[k][j] = __bfloat162float(state[((long)b * C + c0 + j) * (K - 1) + si]);
    } else {
#pragma unroll
      for (int j = 0; j < 8; ++j) win[k][j] = 0.f;
    }
  }
  for (int tt = 0; tt < TT && t0 + tt < T; ++tt) {
    const int t = t0 + tt;
    const uint4 v = *reinterpret_cast<const uint4*>(x + ((long)b * T + t) * ldx + c0);
    win[K - 1][0] = bf16_lo(v.x); win[K - 1][1] = bf16_hi(v.x); win[K - 1][2] = bf16_lo(v.y); win[K - 1][3] = bf16_hi(v.y);
    win[K - 1][4] = bf16_lo(v.z); win[K - 1][5] = bf16_hi(v.z); win[K - 1][6] = bf16_lo(v.w); win[K - 1][7] = bf16_hi(v.w);
    float o[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float a = bs[j];
#pragma unroll
      for (int k = 0; k < K; ++k) a = fmaf(wk[k][j], win[k][j], a);
      o[j] = SILU ? silu_f(a) : a;
    }
    uint4 ov;
    ov.x = pack_bf16(o[0], o[1]); ov.y = pack_bf16(o[2], o[3]); ov.z = pack_bf16(o[4], o[5]); ov.w = pack_bf16(o[6], o[7]);
    *reinterpret_cast<uint4*>(y + ((long)b * T + t) * C + c0) = ov;
#pragma unroll
    for (int k = 0; k < K - 1; ++k)
#pragma unroll
      for (int j = 0; j < 8; ++j) win[k][j] = win[k + 1][j];
  }
}

// ---------------------------------------------------------------------------- scan forward
struct ScanFwdParams {
  const __nv_bfloat16* u;      // [B, T, C]   row stride ld_u
  const __nv_bfloat16* delta;  // [B, T, C]   row stride ld_d (pre-softplus)
  const float* A;              // [C, N] (negative)
  const __nv_bfloat16* Bm;     // [B, T, N]   row stride ld_b
  const __nv_bfloat16* Cm;     // [B, T, N]   row stride ld_c
  const float* D;              // [C]
  const float* h0;             // [B, C, N] or null
  __nv_bfloat16* y;            // [B, T, C] contiguous
  float* ckpt;                 // [B, nseg, C, N] or null
  float* h_out;                // [B, C, N] or null
  int B, T, C;
  long ld_u, ld_d, ld_b, ld_c;
};

// Lane = channel (32 channels per block), warp = group of NPT consecutive states, so the
// B_t / C_t reads are warp-wide broadcasts, per-channel inputs are conflict-free, and the
// only cross-thread work per step is one shared-memory add of the partial <h, C_t>.
template <int N, int NPT>
__global__ void __launch_bounds__(32 * (N / NPT))
selective_scan_fwd_kernel(const ScanFwdParams p) {
  constexpr int NW = N / NPT;
  constexpr int THREADS = 32 * NW;
  constexpr int CH = 32;
  extern __shared__ float sm[];
  float* s_dt = sm;                       // [SEG][CH]
  float* s_du = s_dt + SCAN_SEG * CH;     // [SEG][CH]  dt*u
  float* s_u = s_du + SCAN_SEG * CH;      // [SEG][CH]
  float* s_y = s_u + SCAN_SEG * CH;       // [SEG][CH]
  float* s_B = s_y + SCAN_SEG * CH;       // [SEG][N]
  float* s_C = s_B + SCAN_SEG * N;        // [SEG][N]
  const int tid = threadIdx.x;
  const int ch = tid & 31, wn = tid >> 5;
  const int b = blockIdx.y;
  const int c = blockIdx.x * CH + ch;
  const bool c_ok = c < p.C;
  const int n0 = wn * NPT;
  float A2[NPT], h[NPT];
#pragma unroll
  for (int j = 0; j < NPT; ++j) {
    A2[j] = c_ok ? p.A[(long)c * N + n0 + j] * 1.4426950408889634f : 0.f;
    h[j] = (c_ok && p.h0) ? p.h0[((long)b * p.C + c) * N + n0 + j] : 0.f;
  }
  const int nseg = (p.T + SCAN_SEG - 1) / SCAN_SEG;
  for (int seg = 0; seg < nseg; ++seg) {
    const int t0 = seg * SCAN_SEG;
    const int steps = min(SCAN_SEG, p.T - t0);
    __syncthreads();    // previous segment's readers of shared memory are done
    for (int i = tid; i < SCAN_SEG * CH; i += THREADS) {
      const int tt = i >> 5, cc = i & 31;
      const int cgl = blockIdx.x * CH + cc;
      float dtv = 0.f, uv = 0.f;
      if (tt < steps && cgl < p.C) {
        const long row = (long)b * p.T + t0 + tt;
        dtv = softplusf_(__bfloat162float(p.delta[row * p.ld_d + cgl]));
        uv = __bfloat162float(p.u[row * p.ld_u + cgl]);
      }
      s_dt[i] = dtv; s_u[i] = uv; s_du[i] = dtv * uv; s_y[i] = 0.f;
    }
    for (int i = tid; i < SCAN_SEG * N; i += THREADS) {
      const int tt = i / N, n = i % N;
      float bv = 0.f, cv = 0.f;
      if (tt < steps) {
        const long row = (long)b * p.T + t0 + tt;
        bv = __bfloat162float(p.Bm[row * p.ld_b + n]);
        cv = __bfloat162float(p.Cm[row * p.ld_c + n]);
      }
      s_B[i] = bv; s_C[i] = cv;
    }
    if (p.ckpt && c_ok) {
      float* ck = p.ckpt + (((long)b * nseg + seg) * p.C + c) * N + n0;
#pragma unroll
      for (int j = 0; j < NPT; j += 4) *reinterpret_cast<float4*>(ck + j) = make_float4(h[j], h[j + 1], h[j + 2], h[j + 3]);
    }
    __syncthreads();
    for (int tt = 0; tt < steps; ++tt) {
      const float dtv = s_dt[tt * CH + ch], duv = s_du[tt * CH + ch];
      float acc = 0.f;
#pragma unroll
      for (int j = 0; j < NPT; j += 4) {
        const float4 bv = *reinterpret_cast<const float4*>(s_B + tt * N + n0 + j);
        const float4 cv = *reinterpret_cast<const float4*>(s_C + tt * N + n0 + j);
        h[j] = fmaf(exp2f(dtv * A2[j]), h[j], duv * bv.x);             acc = fmaf(h[j], cv.x, acc);
        h[j + 1] = fmaf(exp2f(dtv * A2[j + 1]), h[j + 1], duv * bv.y); acc = fmaf(h[j + 1], cv.y, acc);
        h[j + 2] = fmaf(exp2f(dtv * A2[j + 2]), h[j + 2], duv * bv.z); acc = fmaf(h[j + 2], cv.z, acc);
        h[j + 3] = fmaf(exp2f(dtv * A2[j + 3]), h[j + 3], duv * bv.w); acc = fmaf(h[j + 3], cv.w, acc);
      }
      if (NW == 1) s_y[tt * CH + ch] = acc;
      else atomicAdd(&s_y[tt * CH + ch], acc);
    }
    __syncthreads();
    for (int i = tid; i < steps * CH; i += THREADS) {
      const int tt = i >> 5, cc = i & 31;
      const int cgl = blockIdx.x * CH + cc;
      if (cgl < p.C) p.y[((long)b * p.T + t0 + tt) * p.C + cgl] = __float2bfloat16(fmaf(p.D[cgl], s_u[i], s_y[i]));
    }
  }
  if (p.h_out && c_ok) {
    float* ho = p.h_out + ((long)b * p.C + c) * N + n0;
#pragma unroll
    for (int j = 0; j < NPT; ++j) ho[j] = h[j];
  }
}

template <int N, int NPT>
static int launch_scan_fwd(const ScanFwdParams& p, cudaStream_t st) {
  constexpr int THREADS = 32 * (N / NPT);
  const int smem = (4 * SCAN_SEG * 32 + 2 * SCAN_SEG * N) * sizeof(float);
  auto kern = selective_scan_fwd_kernel<N, NPT>;
  if (smem > 48 * 1024) SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.C + 31) / 32, p.B);
  kern<<<grid, THREADS, smem, st>>>(p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

using namespace sb;

// y = [silu](causal depthwise conv(x) + bias). K in 2..4. C % 8 == 0, ldx % 8 == 0.
extern "C" int sb_conv1d_fwd(const void* x, const float* w, const float* bias, const void* state, void* y, int B, int T,
                             int C, int K, long ldx, int silu, cudaStream_t st) {
  SB_CHECK_ARG(B > 0 && T > 0 && C % 8 == 0 && ldx % 8 == 0 && K >= 2 && K <= 4);
  const long items = (long)B * ((T + 7) / 8) * (C / 8);
  const int blocks = (int)((items + 127) / 128);
#define SB_CONV(KK)                                                                                             \
  if (silu) conv1d_fwd_kernel<KK, true><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias,              \
                                                                (const __nv_bfloat16*)state, (__nv_bfloat16*)y, B, T, C, ldx); \
  else conv1d_fwd_kernel<KK, false><<<blocks, 128, 0, st>>>((const __nv_bfloat16*)x, w, bias,                   \
                                                            (const __nv_bfloat16*)state, (__nv_bfloat16*)y, B, T, C, ldx)
  if (K == 4) { SB_CONV(4); } else if (K == 3) { SB_CONV(3); } else { SB_CONV(2); }
#undef SB_CONV
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Selective scan forward. N in {8,16,32,64,128,256}. ckpt `[B, ceil(T/32), C, N]` fp32 is
// written when non-null (training); h_out `[B,C,N]` receives the final state when non-null.
extern "C" int sb_scan_fwd(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm,
                           const float* D, const float* h0, void* y, float* ckpt, float* h_out, int B, int T, int C,
                           int N, long ld_u, long ld_d, long ld_b, long ld_c, cudaStream_t st) {
  SB_CHECK_ARG(B > 0 && T > 0 && C > 0);
  ScanFwdParams p;
  p.u = (const __nv_bfloat16*)u; p.delta = (const __nv_bfloat16*)delta; p.A = A;
  p.Bm = (const __nv_bfloat16*)Bm; p.Cm = (const __nv_bfloat16*)Cm; p.D = D; p.h0 = h0;
  p.y = (__nv_bfloat16*)y; p.ckpt = ckpt; p.h_out = h_out;
  p.B = B; p.T = T; p.C = C; p.ld_u = ld_u; p.ld_d = ld_d; p.ld_b = ld_b; p.ld_c = ld_c;
  switch (N) {
    case 8: return launch_scan_fwd<8, 8>(p, st);
    case 16: return launch_scan_fwd<16, 8>(p, st);
    case 32: return launch_scan_fwd<32, 8>(p, st);
    case 64: return launch_scan_fwd<64, 8>(p, st);
    case 128: return launch_scan_fwd<128, 8>(p, st);
    case 256: return launch_scan_fwd<256, 8>(p, st);
    default:
      fprintf(stderr, "summa_b200: selective scan supports d_state in {8,16,32,64,128,256}, got %d\n", N);
      return SB_ERR_ARG;
  }
}
