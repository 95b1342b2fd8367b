// Mamba-1 kernels, forward side: causal depthwise conv1d (+SiLU), the segmented
// selective scan for training / prefill, and the single-token decode step.
//
// Scan layout: one thread owns 16 consecutive states of one channel and carries them in
// registers for the whole sequence. A block covers 16 channels of one batch row with N / 16
// state groups (two per warp) and walks the sequence in 16-step segments whose inputs
// (softplus(delta), u, B_t, C_t) are fetched asynchronously one segment ahead and staged in
// shared memory as fp32. At every segment start the state is written to a checkpoint tensor
// for the backward pass. This removes the reference design's N <= 16 limit: N = 8 .. 256
// are supported.
//   dt = softplus(delta); h_t = exp(dt*A) h_{t-1} + dt*u_t*B_t; y_t = <h_t, C_t> + D u_t
#include "host_util.h"
#include "sm100.cuh"
#include "scan_common.cuh"

namespace sb {

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
  int vec;                     // every row of u / delta / B / C starts 16-byte aligned
};

// Thread = one channel x NPT consecutive states, carried in registers as f32x2 pairs for the whole sequence.
// The CH channel lanes of a warp share a state group, so B_t / C_t reads are broadcasts; a block covers CH
// channels x all N states of one batch row (CH = 16 doubles the block count, which is what fills 148 SMs at
// small batch). Per step a thread leaves its partial <h, C_t> in its group's slot of shared memory; the
// segment epilogue adds the N / NPT slots, so the step loop has no atomics and no barrier.
template <int N, int NPT, int CH>
__global__ void __launch_bounds__((N / NPT) * CH)
selective_scan_fwd_kernel(const ScanFwdParams p) {
  constexpr int NG = N / NPT;             // state groups
  constexpr int THREADS = NG * CH;
  constexpr int NP = NPT / 2;
  constexpr int SEG = SCAN_SEG;
  extern __shared__ __align__(16) float sm[];
  float* s_dt = sm;                       // [SEG][CH]
  float* s_du = s_dt + SEG * CH;          // [SEG][CH]  dt*u
  float* s_u = s_du + SEG * CH;           // [SEG][CH]
  float* s_B = s_u + SEG * CH;            // [SEG][N]
  float* s_C = s_B + SEG * N;             // [SEG][N]
  float* s_part = s_C + SEG * N;          // [NG][SEG][CH] partial outputs
  __nv_bfloat16* r_dt = reinterpret_cast<__nv_bfloat16*>(s_part + NG * SEG * CH);   // raw staging, same shapes
  __nv_bfloat16* r_u = r_dt + SEG * CH;
  __nv_bfloat16* r_B = r_u + SEG * CH;
  __nv_bfloat16* r_C = r_B + SEG * N;
  const int tid = threadIdx.x;
  const int ch = tid % CH, grp = tid / CH;
  const int b = blockIdx.y;
  const int c0 = blockIdx.x * CH;
  const int c = c0 + ch;
  const bool c_ok = c < p.C;
  const int n0 = grp * NPT;
  const bool vec = p.vec != 0;
  uint64_t A2[NP], h[NP];
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const float a0 = c_ok ? p.A[(long)c * N + n0 + 2 * j] * 1.4426950408889634f : 0.f;
    const float a1 = c_ok ? p.A[(long)c * N + n0 + 2 * j + 1] * 1.4426950408889634f : 0.f;
    A2[j] = f2_pack(a0, a1);
    const float h0a = (c_ok && p.h0) ? p.h0[((long)b * p.C + c) * N + n0 + 2 * j] : 0.f;
    const float h0b = (c_ok && p.h0) ? p.h0[((long)b * p.C + c) * N + n0 + 2 * j + 1] : 0.f;
    h[j] = f2_pack(h0a, h0b);
  }
  const int nseg = (p.T + SEG - 1) / SEG;
  auto stage = [&](int seg) {
    const long row0 = (long)b * p.T + seg * SEG;
    const int rv = min(SEG, p.T - seg * SEG), cv = p.C - c0;
    scan_stage_rows(smem_u32(r_dt), r_dt, p.delta, p.ld_d, row0, rv, SEG, c0, CH, cv, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_u), r_u, p.u, p.ld_u, row0, rv, SEG, c0, CH, cv, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_B), r_B, p.Bm, p.ld_b, row0, rv, SEG, 0, N, N, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_C), r_C, p.Cm, p.ld_c, row0, rv, SEG, 0, N, N, vec, tid, THREADS);
    cp_async_commit();
  };
  stage(0);
  for (int seg = 0; seg < nseg; ++seg) {
    const int t0 = seg * SEG;
    const int steps = min(SEG, p.T - t0);
    cp_async_wait_all();
    __syncthreads();    // staging complete; the previous segment's epilogue is done with s_u / s_part
    for (int i = tid; i < SEG * CH; i += THREADS) {
      const int tt = i / CH, cc = i - tt * CH;
      const bool ok = tt < steps && c0 + cc < p.C;
      const float dtv = ok ? softplusf_(__bfloat162float(r_dt[i])) : 0.f;
      const float uv = ok ? __bfloat162float(r_u[i]) : 0.f;
      s_dt[i] = dtv; s_u[i] = uv; s_du[i] = dtv * uv;
    }
    for (int i = tid; i < SEG * N / 2; i += THREADS) {
      const uint32_t bb = reinterpret_cast<const uint32_t*>(r_B)[i], cc = reinterpret_cast<const uint32_t*>(r_C)[i];
      reinterpret_cast<float2*>(s_B)[i] = make_float2(bf16_lo(bb), bf16_hi(bb));
      reinterpret_cast<float2*>(s_C)[i] = make_float2(bf16_lo(cc), bf16_hi(cc));
    }
    __syncthreads();
    if (seg + 1 < nseg) stage(seg + 1);       // in flight during this segment's steps
    if (p.ckpt && c_ok) {
      float* ck = p.ckpt + (((long)b * nseg + seg) * p.C + c) * N + n0;
#pragma unroll
      for (int j = 0; j < NP; j += 2) {
        float4 o;
        f2_unpack(h[j], o.x, o.y);
        f2_unpack(h[j + 1], o.z, o.w);
        *reinterpret_cast<float4*>(ck + 2 * j) = o;
      }
    }
#pragma unroll 2
    for (int tt = 0; tt < steps; ++tt) {
      const float dtv = s_dt[tt * CH + ch], duv = s_du[tt * CH + ch];
      const uint64_t dt2 = f2_pack(dtv, dtv), du2 = f2_pack(duv, duv);
      uint64_t acc2 = f2_pack(0.f, 0.f), acc3 = f2_pack(0.f, 0.f);
#pragma unroll
      for (int j = 0; j < NP; j += 2) {
        // 16-byte shared loads: two (B, C) pairs each, broadcast over the channel lanes
        const ulonglong2 bq = *reinterpret_cast<const ulonglong2*>(s_B + tt * N + n0 + 2 * j);
        const ulonglong2 cq = *reinterpret_cast<const ulonglong2*>(s_C + tt * N + n0 + 2 * j);
        const uint64_t x0 = f2_mul(dt2, A2[j]), x1 = f2_mul(dt2, A2[j + 1]);
        const uint64_t e0 = exp2_xu2_packed(x0), e1 = exp2_xu2_packed(x1);
        h[j] = f2_fma(e0, h[j], f2_mul(du2, bq.x));
        h[j + 1] = f2_fma(e1, h[j + 1], f2_mul(du2, bq.y));
        acc2 = f2_fma(h[j], cq.x, acc2);
        acc3 = f2_fma(h[j + 1], cq.y, acc3);
      }
      float a0, a1;
      f2_unpack(f2_add(acc2, acc3), a0, a1);
      s_part[(grp * SEG + tt) * CH + ch] = a0 + a1;
    }
    __syncthreads();
    // y = sum of the group partials + D u, two channels per item
    for (int i = tid; i < steps * (CH / 2); i += THREADS) {
      const int tt = i / (CH / 2), cp = i - tt * (CH / 2);
      const int cgl = c0 + 2 * cp;
      if (cgl < p.C) {       // C is even on this path (the entry point requires it)
        float2 a = make_float2(0.f, 0.f);
#pragma unroll
        for (int g = 0; g < NG; ++g) {
          const float2 v = *reinterpret_cast<const float2*>(s_part + (g * SEG + tt) * CH + 2 * cp);
          a.x += v.x; a.y += v.y;
        }
        const float2 uu = *reinterpret_cast<const float2*>(s_u + tt * CH + 2 * cp);
        const uint32_t o = pack_bf16(fmaf(p.D[cgl], uu.x, a.x), fmaf(p.D[cgl + 1], uu.y, a.y));
        *reinterpret_cast<uint32_t*>(p.y + ((long)b * p.T + t0 + tt) * p.C + cgl) = o;
      }
    }
  }
  if (p.h_out && c_ok) {
    float* ho = p.h_out + ((long)b * p.C + c) * N + n0;
#pragma unroll
    for (int j = 0; j < NP; ++j) f2_unpack(h[j], ho[2 * j], ho[2 * j + 1]);
  }
}

template <int N, int NPT, int CH>
static int launch_scan_fwd(const ScanFwdParams& p, cudaStream_t st) {
  constexpr int NG = N / NPT;
  constexpr int THREADS = NG * CH;
  const int smem = (3 * SCAN_SEG * CH + 2 * SCAN_SEG * N + NG * SCAN_SEG * CH) * sizeof(float) +
                   (2 * SCAN_SEG * CH + 2 * SCAN_SEG * N) * sizeof(__nv_bfloat16);
  auto kern = selective_scan_fwd_kernel<N, NPT, CH>;
  if (smem > 48 * 1024) SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.C + CH - 1) / CH, p.B);
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

// Steps between the state checkpoints that sb_scan_fwd writes and sb_scan_bwd reads.
extern "C" int sb_scan_ckpt_interval() { return SCAN_SEG; }

// Selective scan forward. N in {8,16,32,64,128,256}, C even. ckpt `[B, ceil(T / sb_scan_ckpt_interval()), C, N]` fp32 is
// written when non-null (training); h_out `[B,C,N]` receives the final state when non-null.
extern "C" int sb_scan_fwd(const void* u, const void* delta, const float* A, const void* Bm, const void* Cm,
                           const float* D, const float* h0, void* y, float* ckpt, float* h_out, int B, int T, int C,
                           int N, long ld_u, long ld_d, long ld_b, long ld_c, cudaStream_t st) {
  SB_CHECK_ARG(B > 0 && T > 0 && C > 0 && C % 2 == 0);
  ScanFwdParams p;
  p.u = (const __nv_bfloat16*)u; p.delta = (const __nv_bfloat16*)delta; p.A = A;
  p.Bm = (const __nv_bfloat16*)Bm; p.Cm = (const __nv_bfloat16*)Cm; p.D = D; p.h0 = h0;
  p.y = (__nv_bfloat16*)y; p.ckpt = ckpt; p.h_out = h_out;
  p.B = B; p.T = T; p.C = C; p.ld_u = ld_u; p.ld_d = ld_d; p.ld_b = ld_b; p.ld_c = ld_c;
  p.vec = C % 8 == 0 && ld_u % 8 == 0 && ld_d % 8 == 0 && ld_b % 8 == 0 && ld_c % 8 == 0 &&
          (((uintptr_t)u | (uintptr_t)delta | (uintptr_t)Bm | (uintptr_t)Cm) & 15) == 0;
  switch (N) {
    case 8: return launch_scan_fwd<8, 8, 32>(p, st);
    case 16: return launch_scan_fwd<16, 16, 32>(p, st);
    case 32: return launch_scan_fwd<32, 16, 16>(p, st);
    case 64: return launch_scan_fwd<64, 16, 16>(p, st);
    case 128: return launch_scan_fwd<128, 16, 16>(p, st);
    case 256: return launch_scan_fwd<256, 16, 16>(p, st);
    default:
      fprintf(stderr, "summa_b200: selective scan supports d_state in {8,16,32,64,128,256}, got %d\n", N);
      return SB_ERR_ARG;
  }
}
