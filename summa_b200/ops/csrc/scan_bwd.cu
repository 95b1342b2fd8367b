// Mamba-1 kernels, backward side: segmented selective-scan backward and the depthwise
// conv1d (+SiLU) backward.
//
// Scan backward, N >= 16: the tiled kernel (a thread owns 4 channels x 4 states; see
// selective_scan_bwd_tile_kernel). N = 8 keeps the one-channel-per-lane kernel: lane = channel,
// warp = 8 states, state and its gradient in registers. Both visit the 16-step segments last to
// first; each segment starts from the forward pass's checkpoint and rebuilds its states in two
// levels (sub-group starts in registers, then one sub-group at a time replayed into a per-thread
// column of shared memory and swept in reverse). Per step the B_t / C_t gradients (sums over
// channels) are reduced over lanes by recursive halving and written as one partial tile per
// 32-channel block, which a second kernel sums; the delta / u gradients (sums over states) are
// combined across warps in shared memory. No global atomics touch the `[B, T, N]` or `[B, T, C]`
// tensors.
#include "host_util.h"
#include "sm100.cuh"
#include "scan_common.cuh"

namespace sb {

constexpr int SCANB_SEG = SCAN_SEG;
constexpr int SCANB_SUB = 8;      // replay depth of the one-channel-per-lane kernel (N = 8)
constexpr int SCANB_THREADS = 256;
// 1: the replay also keeps every step's decay factors in shared memory (twice the footprint, one block per
// SM at 64 states per block); 0: the reverse sweep recomputes them.
#ifndef SCANB_STORE_DECAY
#define SCANB_STORE_DECAY 0
#endif

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
  int vec;                                 // every row of u / delta / dy / B / C starts 16-byte aligned
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
  extern __shared__ __align__(16) float sm[];
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
  // Everything per state is carried as f32x2 pairs (two consecutive states): the rebuilds and the reverse
  // sweep run on packed instructions.
  constexpr int NP = NPT / 2;
  uint64_t A2[NP], Av[NP], dh[NP], dAacc[NP];
#pragma unroll
  for (int j = 0; j < NP; ++j) {
    const float a0 = c_ok ? p.A[(long)c * N + n0 + 2 * j] : 0.f, a1 = c_ok ? p.A[(long)c * N + n0 + 2 * j + 1] : 0.f;
    Av[j] = f2_pack(a0, a1);
    A2[j] = f2_pack(a0 * 1.4426950408889634f, a1 * 1.4426950408889634f);
    const float d0 = (c_ok && p.dh_out) ? p.dh_out[((long)b * p.C + c) * N + n0 + 2 * j] : 0.f;
    const float d1 = (c_ok && p.dh_out) ? p.dh_out[((long)b * p.C + c) * N + n0 + 2 * j + 1] : 0.f;
    dh[j] = f2_pack(d0, d1);
    dAacc[j] = f2_pack(0.f, 0.f);
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
    // decay factors of one step for this thread's state pairs
    auto decay = [&](uint64_t dt2, uint64_t (&e)[NP]) {
#pragma unroll
      for (int j = 0; j < NP; j += 2) {
        e[j] = exp2_xu2_packed(f2_mul(dt2, A2[j]));
        e[j + 1] = exp2_xu2_packed(f2_mul(dt2, A2[j + 1]));
      }
    };
    // ---- level 1: states at every 8th step
    uint64_t hs[NSUB][NP];
    {
      uint64_t h[NP];
      const float* ck = p.ckpt + (((long)b * nseg + seg) * p.C + (c_ok ? c : 0)) * N + n0;
#pragma unroll
      for (int j = 0; j < NP; ++j) h[j] = c_ok ? f2_pack(ck[2 * j], ck[2 * j + 1]) : f2_pack(0.f, 0.f);
#pragma unroll
      for (int sb_ = 0; sb_ < NSUB; ++sb_) {
#pragma unroll
        for (int j = 0; j < NP; ++j) hs[sb_][j] = h[j];
        if (sb_ == NSUB - 1) break;
#pragma unroll 1
        for (int k = 0; k < SCANB_SUB; ++k) {
          const int tt = sb_ * SCANB_SUB + k;
          const float dtv = s_dt[tt * CH + ch], duv = dtv * s_u[tt * CH + ch];
          const uint64_t du2 = f2_pack(duv, duv);
          uint64_t e[NP];
          decay(f2_pack(dtv, dtv), e);
#pragma unroll
          for (int j = 0; j < NP; j += 2) {
            const ulonglong2 bq = *reinterpret_cast<const ulonglong2*>(s_B + tt * NB + nl + 2 * j);
            h[j] = f2_fma(e[j], h[j], f2_mul(du2, bq.x));
            h[j + 1] = f2_fma(e[j + 1], h[j + 1], f2_mul(du2, bq.y));
          }
        }
      }
    }
    // ---- level 2: replay each 8-step group (keeping the pre-step states of every step in shared memory,
    // and the decay factors too when SCANB_STORE_DECAY), then sweep it in reverse
    uint64_t* s_hp2 = reinterpret_cast<uint64_t*>(s_hp);                       // [SUB][NP][THREADS] pre-step states
    uint64_t* s_da2 = s_hp2 + SCANB_SUB * NP * THREADS;                        // [SUB][NP][THREADS] decay factors
#pragma unroll
    for (int sb_ = NSUB - 1; sb_ >= 0; --sb_) {
      if (sb_ * SCANB_SUB >= steps) continue;
      {
        uint64_t h[NP];
#pragma unroll
        for (int j = 0; j < NP; ++j) h[j] = hs[sb_][j];
#pragma unroll 1
        for (int k = 0; k < SCANB_SUB; ++k) {
          const int tt = sb_ * SCANB_SUB + k;
          const float dtv = s_dt[tt * CH + ch], duv = dtv * s_u[tt * CH + ch];
          const uint64_t du2 = f2_pack(duv, duv);
          uint64_t e[NP];
          decay(f2_pack(dtv, dtv), e);
#pragma unroll
          for (int j = 0; j < NP; ++j) {
            s_hp2[(k * NP + j) * THREADS + tid] = h[j];
            if (SCANB_STORE_DECAY) s_da2[(k * NP + j) * THREADS + tid] = e[j];
          }
          if (k == SCANB_SUB - 1) break;
#pragma unroll
          for (int j = 0; j < NP; j += 2) {
            const ulonglong2 bq = *reinterpret_cast<const ulonglong2*>(s_B + tt * NB + nl + 2 * j);
            h[j] = f2_fma(e[j], h[j], f2_mul(du2, bq.x));
            h[j + 1] = f2_fma(e[j + 1], h[j + 1], f2_mul(du2, bq.y));
          }
        }
      }
#pragma unroll 1
      for (int k = SCANB_SUB - 1; k >= 0; --k) {
        const int tt = sb_ * SCANB_SUB + k;
        if (tt >= steps) continue;        // uniform across the block
        const float dtv = s_dt[tt * CH + ch], uv = s_u[tt * CH + ch], dyv = s_dy[tt * CH + ch];
        const float duv = dtv * uv;
        const uint64_t dt2 = f2_pack(dtv, dtv), u2 = f2_pack(uv, uv), dy2 = f2_pack(dyv, dyv), du2 = f2_pack(duv, duv);
        uint64_t ddt2 = f2_pack(0.f, 0.f), dua2 = f2_pack(0.f, 0.f);
        float red[2 * NPT];               // [0,NPT): dB contributions, [NPT,2NPT): dC contributions
        uint64_t e[NP];
        if (!SCANB_STORE_DECAY) decay(dt2, e);
#pragma unroll
        for (int j = 0; j < NP; ++j) {
          const uint64_t bv = *reinterpret_cast<const uint64_t*>(s_B + tt * NB + nl + 2 * j);
          const uint64_t cv = *reinterpret_cast<const uint64_t*>(s_C + tt * NB + nl + 2 * j);
          const uint64_t dA = SCANB_STORE_DECAY ? s_da2[(k * NP + j) * THREADS + tid] : e[j];
          const uint64_t hprev = s_hp2[(k * NP + j) * THREADS + tid];
          const uint64_t ht = f2_fma(dA, hprev, f2_mul(du2, bv));
          const uint64_t g = f2_fma(cv, dy2, dh[j]);
          f2_unpack(f2_mul(g, du2), red[2 * j], red[2 * j + 1]);
          f2_unpack(f2_mul(ht, dy2), red[NPT + 2 * j], red[NPT + 2 * j + 1]);
          const uint64_t ddA = f2_mul(f2_mul(g, hprev), dA);
          ddt2 = f2_fma(ddA, Av[j], f2_fma(f2_mul(g, u2), bv, ddt2));
          dua2 = f2_fma(f2_mul(g, dt2), bv, dua2);
          dAacc[j] = f2_fma(ddA, dt2, dAacc[j]);
          dh[j] = f2_mul(g, dA);
        }
        float ddt, ddt_b, duacc, dua_b;
        f2_unpack(ddt2, ddt, ddt_b);
        f2_unpack(dua2, duacc, dua_b);
        ddt += ddt_b;
        duacc += dua_b;
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
    for (int j = 0; j < NP; ++j) {
      float a0, a1, d0, d1;
      f2_unpack(dAacc[j], a0, a1);
      f2_unpack(dh[j], d0, d1);
      atomicAdd(p.dA + (long)c * N + n0 + 2 * j, a0);
      atomicAdd(p.dA + (long)c * N + n0 + 2 * j + 1, a1);
      if (p.dh0) {
        p.dh0[((long)b * p.C + c) * N + n0 + 2 * j] = d0;
        p.dh0[((long)b * p.C + c) * N + n0 + 2 * j + 1] = d1;
      }
    }
    if (wn == 0 && blockIdx.z == 0) atomicAdd(p.dD + c, dDacc);
  }
}

// Sums v[0..V) over the L lanes whose ids differ in bits [SH, SH + log2 L), by recursive halving: each level
// exchanges half of the values still held, so V >= L costs V (1 - 1/L) shuffles and leaves V / L totals per lane
// in v[0..V/L). The lane ends up with the values whose original index is
//   k + sum over levels l of bit(lane, SH + l) * V / 2^(l+1),   k in [0, V/L).
template <int V, int L, int SH>
__device__ __forceinline__ void lane_group_reduce(float (&v)[V], int lane) {
  static_assert(V >= L, "fewer values than lanes");
  int cnt = V;
#pragma unroll
  for (int l = 0; (1 << l) < L; ++l) {
    const bool hi = (lane >> (SH + l)) & 1;
    const int half = cnt / 2;
#pragma unroll
    for (int i = 0; i < V / 2; ++i) {
      if (i < half) {
        const float send = hi ? v[i] : v[i + half];
        const float keep = hi ? v[i + half] : v[i];
        v[i] = keep + __shfl_xor_sync(0xffffffffu, send, 1 << (SH + l));
      }
    }
    cnt = half;
  }
}

constexpr int SCANT_SUB = 4;       // replay depth of the tiled kernel

// Tiled backward, N >= 16. A thread owns a 4-channel x 4-state tile (16 states and their gradients in registers
// as 8 f32x2 pairs); a warp is 8 channel groups x 4 state groups = 32 channels x 16 states; a block is NB / 16
// warps over NB <= 64 states (blockIdx.z picks the slice when N > NB). Compared with one channel per lane this
// puts both kinds of per-step sums partly inside the thread: the B_t / C_t gradients (sums over channels) are
// accumulated over the thread's 4 channels by the fma that computes them and then reduced over 8 lanes
// (7 shuffles for 8 values); the delta / u gradients (sums over states) likewise over 4 lanes (6 shuffles for
// 8 values) and are left in a per-warp slot of shared memory which the segment epilogue adds, so the step loop
// has no atomics. Segments of 16 steps are visited last to first; each is rebuilt from the forward pass's
// checkpoint in two levels: the states at steps 4, 8, 12 stay in registers, then every 4-step group is replayed
// into a per-thread column of shared memory and swept in reverse. The next segment's inputs are fetched
// asynchronously during the sweep.
template <int N, int NB>
__global__ void __launch_bounds__(2 * NB, NB == 64 ? 3 : 4)
selective_scan_bwd_tile_kernel(const ScanBwdParams p) {
  constexpr int NW = NB / 16;
  constexpr int THREADS = 32 * NW;
  constexpr int SEG = SCAN_SEG, SUB = SCANT_SUB, NSUB = SEG / SUB;
  constexpr int CH = 32;
  constexpr int NPR = 8;                   // f32x2 pairs per thread: pair 2 i + q = channel i, states 2 q, 2 q + 1
  constexpr float LN2 = 0.6931471805599453f;
  extern __shared__ __align__(16) float sm[];
  float* s_dt = sm;                        // [SEG][CH] softplus(delta)
  float* s_u = s_dt + SEG * CH;
  float* s_dy = s_u + SEG * CH;
  float* s_B = s_dy + SEG * CH;            // [SEG][NB]
  float* s_C = s_B + SEG * NB;
  float* s_po = s_C + SEG * NB;            // [NW][SEG][2 CH] per-warp sums over the warp's 16 states: ddt | du
  uint64_t* s_hp = reinterpret_cast<uint64_t*>(s_po + NW * SEG * 2 * CH);   // [SUB][NPR][THREADS] pre-step states
  __nv_bfloat16* r_dt = reinterpret_cast<__nv_bfloat16*>(s_hp + SUB * NPR * THREADS);   // raw staging
  __nv_bfloat16* r_u = r_dt + SEG * CH;
  __nv_bfloat16* r_dy = r_u + SEG * CH;
  __nv_bfloat16* r_B = r_dy + SEG * CH;
  __nv_bfloat16* r_C = r_B + SEG * NB;
  const int tid = threadIdx.x, lane = tid & 31, w = tid >> 5;
  const int lc = lane & 7, ln = lane >> 3;
  const int b = blockIdx.y;
  const int c0 = blockIdx.x * CH;
  const int cb = c0 + 4 * lc;              // first channel of this thread
  const int nb0 = blockIdx.z * NB;
  const int nl = 16 * w + 4 * ln;          // first state of this thread inside the block's slice
  const int n0 = nb0 + nl;
  const bool vec = p.vec != 0;
  uint64_t A2[NPR], dh[NPR], dAacc[NPR];
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    const bool ok = cb + i < p.C;
#pragma unroll
    for (int q = 0; q < 2; ++q) {
      const long o = (long)(cb + i) * N + n0 + 2 * q;
      A2[2 * i + q] = ok ? f2_pack(p.A[o] * 1.4426950408889634f, p.A[o + 1] * 1.4426950408889634f) : f2_pack(0.f, 0.f);
      const long od = ((long)b * p.C + cb + i) * N + n0 + 2 * q;
      dh[2 * i + q] = (ok && p.dh_out) ? f2_pack(p.dh_out[od], p.dh_out[od + 1]) : f2_pack(0.f, 0.f);
      dAacc[2 * i + q] = f2_pack(0.f, 0.f);
    }
  }
  float dDacc = 0.f;                        // threads 0..31 of slice 0: channel c0 + tid
  const int nseg = (p.T + SEG - 1) / SEG;
  auto stage = [&](int seg) {
    const long row0 = (long)b * p.T + seg * SEG;
    const int rv = min(SEG, p.T - seg * SEG), cv = p.C - c0;
    scan_stage_rows(smem_u32(r_dt), r_dt, p.delta, p.ld_d, row0, rv, SEG, c0, CH, cv, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_u), r_u, p.u, p.ld_u, row0, rv, SEG, c0, CH, cv, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_dy), r_dy, p.dy, p.ld_dy, row0, rv, SEG, c0, CH, cv, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_B), r_B, p.Bm, p.ld_b, row0, rv, SEG, nb0, NB, NB, vec, tid, THREADS);
    scan_stage_rows(smem_u32(r_C), r_C, p.Cm, p.ld_c, row0, rv, SEG, nb0, NB, NB, vec, tid, THREADS);
    cp_async_commit();
  };
  // the segment's checkpoint: this thread's 4 x 4 tile as 8 pairs
  auto load_ckpt = [&](int seg, uint64_t (&h)[NPR]) {
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
      if (cb + i < p.C) v = *reinterpret_cast<const float4*>(p.ckpt + (((long)b * nseg + seg) * p.C + cb + i) * N + n0);
      h[2 * i] = f2_pack(v.x, v.y);
      h[2 * i + 1] = f2_pack(v.z, v.w);
    }
  };
  // one forward step on all 8 pairs
  auto fwd_step = [&](int tt, uint64_t (&h)[NPR]) {
    const float4 dt4 = *reinterpret_cast<const float4*>(s_dt + tt * CH + 4 * lc);
    const float4 u4 = *reinterpret_cast<const float4*>(s_u + tt * CH + 4 * lc);
    const ulonglong2 bq = *reinterpret_cast<const ulonglong2*>(s_B + tt * NB + nl);
    const float dtv[4] = {dt4.x, dt4.y, dt4.z, dt4.w}, uv[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
      const uint64_t dt2 = f2_pack(dtv[i], dtv[i]);
      const float duv = dtv[i] * uv[i];
      const uint64_t du2 = f2_pack(duv, duv);
      h[2 * i] = f2_fma(exp2_xu2_packed(f2_mul(dt2, A2[2 * i])), h[2 * i], f2_mul(du2, bq.x));
      h[2 * i + 1] = f2_fma(exp2_xu2_packed(f2_mul(dt2, A2[2 * i + 1])), h[2 * i + 1], f2_mul(du2, bq.y));
    }
  };
  stage(nseg - 1);
  for (int seg = nseg - 1; seg >= 0; --seg) {
    const int t0 = seg * SEG;
    const int steps = min(SEG, p.T - t0);
    cp_async_wait_all();
    __syncthreads();      // staging complete; the previous segment's epilogue is done with s_po / s_dy / s_u
    for (int i = tid; i < SEG * CH; i += THREADS) {
      const int tt = i / CH, cc = i - tt * CH;
      const bool ok = tt < steps && c0 + cc < p.C;
      s_dt[i] = ok ? softplusb_(__bfloat162float(r_dt[i])) : 0.f;
      s_u[i] = ok ? __bfloat162float(r_u[i]) : 0.f;
      s_dy[i] = ok ? __bfloat162float(r_dy[i]) : 0.f;
    }
    for (int i = tid; i < SEG * NB / 2; i += THREADS) {
      const uint32_t bb = reinterpret_cast<const uint32_t*>(r_B)[i], cc = reinterpret_cast<const uint32_t*>(r_C)[i];
      reinterpret_cast<float2*>(s_B)[i] = make_float2(bf16_lo(bb), bf16_hi(bb));
      reinterpret_cast<float2*>(s_C)[i] = make_float2(bf16_lo(cc), bf16_hi(cc));
    }
    __syncthreads();
    if (seg > 0) stage(seg - 1);            // in flight during this segment's sweep
    // ---- level 1: states at steps 4, 8, 12 (hs[0] is unused: step 0 is the checkpoint itself)
    uint64_t hs[NSUB][NPR];
    {
      uint64_t h[NPR];
      load_ckpt(seg, h);
#pragma unroll
      for (int sb_ = 0; sb_ < NSUB - 1; ++sb_) {
#pragma unroll 1
        for (int k = 0; k < SUB; ++k) fwd_step(sb_ * SUB + k, h);
#pragma unroll
        for (int j = 0; j < NPR; ++j) hs[sb_ + 1][j] = h[j];
      }
    }
    // ---- level 2: replay each 4-step group into shared memory, then sweep it in reverse
#pragma unroll
    for (int sb_ = NSUB - 1; sb_ >= 0; --sb_) {
      if (sb_ * SUB >= steps) continue;     // uniform across the block
      {
        uint64_t h[NPR];
        if (sb_ == 0) {
          load_ckpt(seg, h);
        } else {
#pragma unroll
          for (int j = 0; j < NPR; ++j) h[j] = hs[sb_][j];
        }
#pragma unroll 1
        for (int k = 0; k < SUB; ++k) {
#pragma unroll
          for (int j = 0; j < NPR; ++j) s_hp[(k * NPR + j) * THREADS + tid] = h[j];
          if (k == SUB - 1) break;
          fwd_step(sb_ * SUB + k, h);
        }
      }
#pragma unroll 1
      for (int k = SUB - 1; k >= 0; --k) {
        const int tt = sb_ * SUB + k;
        if (tt >= steps) continue;          // uniform across the block
        const float4 dt4 = *reinterpret_cast<const float4*>(s_dt + tt * CH + 4 * lc);
        const float4 u4 = *reinterpret_cast<const float4*>(s_u + tt * CH + 4 * lc);
        const float4 dy4 = *reinterpret_cast<const float4*>(s_dy + tt * CH + 4 * lc);
        const ulonglong2 bq = *reinterpret_cast<const ulonglong2*>(s_B + tt * NB + nl);
        const ulonglong2 cq = *reinterpret_cast<const ulonglong2*>(s_C + tt * NB + nl);
        const uint64_t bp[2] = {bq.x, bq.y}, cp[2] = {cq.x, cq.y};
        const float dtv[4] = {dt4.x, dt4.y, dt4.z, dt4.w}, uv[4] = {u4.x, u4.y, u4.z, u4.w};
        const float dyv[4] = {dy4.x, dy4.y, dy4.z, dy4.w};
        uint64_t dBa[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)}, dCa[2] = {f2_pack(0.f, 0.f), f2_pack(0.f, 0.f)};
        float r2[8];                        // [0,4): ddt of the 4 channels, [4,8): du
#pragma unroll
        for (int i = 0; i < 4; ++i) {
          const uint64_t dt2 = f2_pack(dtv[i], dtv[i]), dy2 = f2_pack(dyv[i], dyv[i]);
          const float duv = dtv[i] * uv[i];
          const uint64_t du2 = f2_pack(duv, duv);
          uint64_t sA = f2_pack(0.f, 0.f), sB = f2_pack(0.f, 0.f);
#pragma unroll
          for (int q = 0; q < 2; ++q) {
            const int j = 2 * i + q;
            const uint64_t dA = exp2_xu2_packed(f2_mul(dt2, A2[j]));
            const uint64_t hprev = s_hp[(k * NPR + j) * THREADS + tid];
            const uint64_t ht = f2_fma(dA, hprev, f2_mul(du2, bp[q]));      // h_t
            const uint64_t g = f2_fma(cp[q], dy2, dh[j]);                   // dL/dh_t
            dBa[q] = f2_fma(g, du2, dBa[q]);
            dCa[q] = f2_fma(ht, dy2, dCa[q]);
            const uint64_t ddA = f2_mul(f2_mul(g, hprev), dA);              // dL/d(decay) * decay
            sA = f2_fma(ddA, A2[j], sA);
            sB = f2_fma(g, bp[q], sB);
            dAacc[j] = f2_fma(ddA, dt2, dAacc[j]);
            dh[j] = f2_mul(g, dA);
          }
          float a0, a1, b0, b1;
          f2_unpack(sA, a0, a1);
          f2_unpack(sB, b0, b1);
          const float sb2 = b0 + b1;
          r2[i] = fmaf(LN2, a0 + a1, uv[i] * sb2);
          r2[4 + i] = dtv[i] * sb2;
        }
        float r1[8];                        // [0,4): dB of the 4 states, [4,8): dC
        f2_unpack(dBa[0], r1[0], r1[1]);
        f2_unpack(dBa[1], r1[2], r1[3]);
        f2_unpack(dCa[0], r1[4], r1[5]);
        f2_unpack(dCa[1], r1[6], r1[7]);
        lane_group_reduce<8, 8, 0>(r1, lane);     // over the 8 channel groups: one total per lane
        lane_group_reduce<8, 4, 3>(r2, lane);     // over the 4 state groups: two totals per lane
        {
          const int idx = ((lane & 1) << 2) | (lane & 2) | ((lane >> 2) & 1);
          const long o = (((long)blockIdx.x * p.B + b) * p.T + t0 + tt) * N + n0 + (idx & 3);
          if (idx < 4) p.dB_part[o] = r1[0];
          else p.dC_part[o] = r1[0];
        }
        {
          const int idx = (((lane >> 3) & 1) << 2) | (((lane >> 4) & 1) << 1);     // even: values idx, idx + 1
          float* o = s_po + (w * SEG + tt) * 2 * CH + (idx < 4 ? 0 : CH) + 4 * lc + (idx & 3);
          *reinterpret_cast<float2*>(o) = make_float2(r2[0], r2[1]);
        }
      }
    }
    __syncthreads();
    {
      float* pd = p.ddt_part + ((long)blockIdx.z * p.B + b) * p.T * p.C;
      float* pu = p.du_part + ((long)blockIdx.z * p.B + b) * p.T * p.C;
      for (int i = tid; i < steps * CH; i += THREADS) {
        const int tt = i / CH, cc = i - tt * CH;
        if (c0 + cc < p.C) {
          float a = 0.f, e = 0.f;
#pragma unroll
          for (int ww = 0; ww < NW; ++ww) {
            a += s_po[(ww * SEG + tt) * 2 * CH + cc];
            e += s_po[(ww * SEG + tt) * 2 * CH + CH + cc];
          }
          const long o = ((long)t0 + tt) * p.C + c0 + cc;
          pd[o] = a;
          pu[o] = e;
        }
      }
      if (tid < CH && blockIdx.z == 0) {
        for (int tt = 0; tt < steps; ++tt) dDacc = fmaf(s_dy[tt * CH + tid], s_u[tt * CH + tid], dDacc);
      }
    }
  }
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    if (cb + i < p.C) {
#pragma unroll
      for (int q = 0; q < 2; ++q) {
        float a0, a1, d0, d1;
        f2_unpack(dAacc[2 * i + q], a0, a1);
        f2_unpack(dh[2 * i + q], d0, d1);
        atomicAdd(p.dA + (long)(cb + i) * N + n0 + 2 * q, a0);
        atomicAdd(p.dA + (long)(cb + i) * N + n0 + 2 * q + 1, a1);
        if (p.dh0) {
          p.dh0[((long)b * p.C + cb + i) * N + n0 + 2 * q] = d0;
          p.dh0[((long)b * p.C + cb + i) * N + n0 + 2 * q + 1] = d1;
        }
      }
    }
  }
  if (tid < CH && blockIdx.z == 0 && c0 + tid < p.C) atomicAdd(p.dD + c0 + tid, dDacc);
}

template <int N, int NB>
static int launch_scan_bwd_tile(const ScanBwdParams& p, cudaStream_t st) {
  constexpr int NW = NB / 16, THREADS = 32 * NW;
  const int smem = (3 * SCAN_SEG * 32 + 2 * SCAN_SEG * NB + NW * SCAN_SEG * 64) * sizeof(float) +
                   SCANT_SUB * 8 * THREADS * sizeof(uint64_t) + (3 * SCAN_SEG * 32 + 2 * SCAN_SEG * NB) * sizeof(__nv_bfloat16);
  auto kern = selective_scan_bwd_tile_kernel<N, NB>;
  if (smem > 48 * 1024) SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, smem));
  dim3 grid((p.C + 31) / 32, p.B, N / NB);
  kern<<<grid, THREADS, smem, st>>>(p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
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
  const int smem = (5 * SCANB_SEG * 32 + 2 * SCANB_SEG * NB + (1 + SCANB_STORE_DECAY) * SCANB_SUB * 8 * THREADS) * sizeof(float);
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
  p.vec = C % 8 == 0 && ld_u % 8 == 0 && ld_d % 8 == 0 && ld_b % 8 == 0 && ld_c % 8 == 0 && ld_dy % 8 == 0 &&
          (((uintptr_t)u | (uintptr_t)delta | (uintptr_t)Bm | (uintptr_t)Cm | (uintptr_t)dy) & 15) == 0;
  int rc, ns = 1;
  switch (N) {
    case 8: rc = launch_scan_bwd<8, 8>(p, st); break;
    case 16: rc = launch_scan_bwd_tile<16, 16>(p, st); break;
    case 32: rc = launch_scan_bwd_tile<32, 32>(p, st); break;
    case 64: rc = launch_scan_bwd_tile<64, 64>(p, st); break;
    case 128: rc = launch_scan_bwd_tile<128, 64>(p, st); ns = 2; break;
    case 256: rc = launch_scan_bwd_tile<256, 64>(p, st); ns = 4; break;
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
