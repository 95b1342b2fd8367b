// Flash-style attention backward on tcgen05/TMEM: a delta pre-pass, a dK/dV kernel and a
// dQ kernel (both recompute the probabilities from Q, K and the saved log-sum-exp, so no
// S x S tensor is ever stored and no atomics are needed; results are deterministic).
//
//   delta[b,h,q] = sum_d dO * O
//   dQ kernel   one CTA per (128 queries, head, batch): per 64-key block
//                 S = Q K^T, dP = dO V^T (TMEM) -> dS = P*(dP - delta) (threads, to smem)
//                 dQ += dS K (TMEM accumulate); epilogue scales and stores dQ
//   dKV kernel  one CTA per (128 keys, kv head, batch): per (query head of the group,
//               64-query block)
//                 S^T = K Q^T, dP^T = V dO^T (TMEM) -> P^T, dS^T (threads, to smem)
//                 dV += P^T dO, dK += dS^T Q (TMEM accumulate over the whole loop)
// The same shared-memory tile serves as a K-major operand in one product and as an
// MN-major operand in the other (Q and dO in the dKV kernel, K in the dQ kernel), which
// the UMMA descriptors express without any transposition in memory.
// Roles per CTA: warps 0-7 compute (two groups of 128 threads split the 128 columns of a
// block), warp 8 TMA loader, warp 9 MMA issuer.
#include "host_util.h"
#include "no_alloc.h"
#include "sm100.cuh"

namespace sb {

constexpr int ATTB_THREADS = 320;

struct AttBwdParams {
  int B, Hq, Hkv, Sq, Sk;
  int causal, window, q_offset;
  float scale, scale_log2;
  const float* lse;     // [B, Hq, Sq] natural log
  const float* delta;   // [B, Hq, sq_pad] scratch: sum_d dO*O
  const float* lse2;    // [B, Hq, sq_pad] scratch: lse * log2(e)
  int sq_pad;           // Sq rounded up to 64 (row pitch of the two scratch arrays)
  unsigned int* err;
};

__device__ __forceinline__ bool att_blocked(const AttBwdParams& p, int pos, int kv) {
  bool bl = kv >= p.Sk;
  if (p.causal) bl |= kv > pos;
  if (p.window >= 0) bl |= (pos - kv > p.window) || (kv - pos > p.window);
  return bl;
}

// write 32 bf16 values (one 64-byte quarter of a 256-byte logical row) of row t into a
// [128 x 128] bf16 tile stored as two 64-column halves with the 128-byte swizzle
__device__ __forceinline__ void store_chunk_sw128(uint8_t* tile, int t, int c, const float* val) {
  uint8_t* dst = tile + (c >> 1) * 16384 + t * 128;
#pragma unroll
  for (int g = 0; g < 4; ++g) {
    uint4 w;
    w.x = pack_bf16(val[8 * g + 0], val[8 * g + 1]);
    w.y = pack_bf16(val[8 * g + 2], val[8 * g + 3]);
    w.z = pack_bf16(val[8 * g + 4], val[8 * g + 5]);
    w.w = pack_bf16(val[8 * g + 6], val[8 * g + 7]);
    const int j16 = (c & 1) * 4 + g;
    *reinterpret_cast<uint4*>(dst + ((j16 ^ (t & 7)) << 4)) = w;
  }
}

// ---------------------------------------------------------------------------- delta
// delta[b,h,s] = sum_d dO*O and lse2[b,h,s] = lse*log2(e), both with row pitch sq_pad
// (rows in [Sq, sq_pad) are written as zeros so that bulk copies of 64-row slices are clean).
template <int D>
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                       const float* __restrict__ lse, float* __restrict__ delta,
                                       float* __restrict__ lse2, int B, int Sq, int sq_pad, int Hq, long o_sb, long o_ss,
                                       long o_sh, long d_sb, long d_ss, long d_sh) {
  const long gw = (blockIdx.x * (long)blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  const long total = (long)B * sq_pad * Hq;
  if (gw >= total) return;
  const int h = gw % Hq;
  const long r = gw / Hq;
  const int s = r % sq_pad;
  const int b = r / sq_pad;
  const long oidx = ((long)b * Hq + h) * sq_pad + s;
  if (s >= Sq) {
    if (lane == 0) { delta[oidx] = 0.f; lse2[oidx] = 0.f; }
    return;
  }
  const __nv_bfloat16* po = o + b * o_sb + s * o_ss + h * o_sh;
  const __nv_bfloat16* pd = dout + b * d_sb + s * d_ss + h * d_sh;
  float acc = 0.f;
  constexpr int E = D / 32;
  if (E == 2) {
    const uint32_t a = *reinterpret_cast<const uint32_t*>(po + lane * 2);
    const uint32_t c = *reinterpret_cast<const uint32_t*>(pd + lane * 2);
    acc = bf16_lo(a) * bf16_lo(c) + bf16_hi(a) * bf16_hi(c);
  } else {
    const uint2 a = *reinterpret_cast<const uint2*>(po + lane * 4);
    const uint2 c = *reinterpret_cast<const uint2*>(pd + lane * 4);
    acc = bf16_lo(a.x) * bf16_lo(c.x) + bf16_hi(a.x) * bf16_hi(c.x) + bf16_lo(a.y) * bf16_lo(c.y) +
          bf16_hi(a.y) * bf16_hi(c.y);
  }
  acc = warp_sum(acc);
  if (lane == 0) {
    delta[oidx] = acc;
    lse2[oidx] = lse[((long)b * Hq + h) * Sq + s] * 1.4426950408889634f;
  }
}

// ---------------------------------------------------------------------------- dQ
// Pipelined over 64-key blocks: the score products of block i+1 are issued before the
// accumulate product of block i, into the other half of a double-buffered TMEM region,
// so the tensor core works on one block while the threads turn the other into dS.
template <int D>
struct AttDq {
  static constexpr int TILE = 128 * D * 2;        // Q / dO tile (128 rows)
  static constexpr int KV = 64 * D * 2;           // K / V stage (64 rows)
  static constexpr int OFF_Q = 0, OFF_DO = TILE;
  static constexpr int NS = 4;                    // K / V load stages (the loader runs ahead of the products)
  static constexpr int OFF_K = 2 * TILE;          // NS stages
  static constexpr int OFF_V = OFF_K + NS * KV;   // NS stages
  static constexpr int OFF_DS = OFF_V + NS * KV;  // 2 stages of [128 x 64] bf16 (16 KB)
  static constexpr int OFF_BAR = OFF_DS + 2 * 16384;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int COL_S = 0, COL_DP = 128, COL_DQ = 256;   // S/dP: buffer b at +64*b
};

template <int D>
__global__ void __launch_bounds__(ATTB_THREADS, 1)
attention_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmDQ, const AttBwdParams p) {
  using C = AttDq<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  constexpr int NS = C::NS;
  uint64_t* qdo_full = bars + 0;
  uint64_t* sdp_full = bars + 1;    // [2]
  uint64_t* sdp_free = bars + 3;    // [2] 128 arrivals
  uint64_t* ds_full = bars + 5;     // [2] 128 arrivals
  uint64_t* ds_free = bars + 7;     // [2]
  uint64_t* dq_full = bars + 9;
  uint64_t* kv_full = bars + 10;            // [NS]
  uint64_t* kv_empty = bars + 10 + NS;      // [NS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10 + 2 * NS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;
  const int head = blockIdx.y, b = blockIdx.z;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qblk * 128;
  int j_begin = 0, j_end = (p.Sk + 63) / 64;
  if (p.causal) j_end = min(j_end, (p.q_offset + q0 + 127) / 64 + 1);
  if (p.window >= 0) j_begin = max(0, (p.q_offset + q0 - p.window) / 64);
  const int nblk = max(0, j_end - j_begin);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&sdp_free[s], 128); mbar_init(&ds_full[s], 128); mbar_init(&ds_free[s], 1);
    }
    for (int s = 0; s < NS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    mbar_init(dq_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(qdo_full, 2 * C::TILE);
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        tma_load_4d(smem + C::OFF_Q + h * 16384, &tmQ, qdo_full, h * 64, head, q0, b);
        tma_load_4d(smem + C::OFF_DO + h * 16384, &tmDO, qdo_full, h * 64, head, q0, b);
      }
      for (int i = 0; i < nblk; ++i) {
        const int s = i % NS;
        const int kv0 = (j_begin + i) * 64;
        if (!mbar_wait(&kv_empty[s], ((i / NS) & 1) ^ 1, abort_flag, p.err)) break;
        mbar_expect_tx(&kv_full[s], 2 * C::KV);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          tma_load_4d(smem + C::OFF_K + s * C::KV + h * 8192, &tmK, &kv_full[s], h * 64, kv_head, kv0, b);
          tma_load_4d(smem + C::OFF_V + s * C::KV + h * 8192, &tmV, &kv_full[s], h * 64, kv_head, kv0, b);
        }
      }
      if (*abort_flag) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) {} }
    }
    __syncwarp();
  } else if (warp == 9) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, 0, 1);   // dS (K-major) x K stage (N-major)
      const uint32_t q_base = smem_u32(smem + C::OFF_Q), do_base = smem_u32(smem + C::OFF_DO);
      const uint32_t k_base = smem_u32(smem + C::OFF_K), v_base = smem_u32(smem + C::OFF_V);
      const uint32_t ds_base = smem_u32(smem + C::OFF_DS);
      auto issue_scores = [&](int ls, int tb) {     // ls: K/V ring stage, tb: TMEM buffer
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t boff = ls * C::KV + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + C::COL_S + 64 * tb, make_smem_desc_sw128(q_base + aoff, 16, 1024),
                    make_smem_desc_sw128(k_base + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t boff = ls * C::KV + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + C::COL_DP + 64 * tb, make_smem_desc_sw128(do_base + aoff, 16, 1024),
                    make_smem_desc_sw128(v_base + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[tb]);
      };
      bool ok = mbar_wait(qdo_full, 0, abort_flag, p.err) && mbar_wait(&kv_full[0], 0, abort_flag, p.err);
      if (ok) { tc_fence_after(); issue_scores(0, 0); }
      for (int i = 0; i < nblk && ok; ++i) {
        const int s = i & 1;
        const int ls = i % NS;
        if (i + 1 < nblk) {
          const int s1 = (i + 1) & 1;
          const int ls1 = (i + 1) % NS;
          if (!mbar_wait(&kv_full[ls1], ((i + 1) / NS) & 1, abort_flag, p.err) ||
              !mbar_wait(&sdp_free[s1], (((i + 1) >> 1) & 1) ^ 1, abort_flag, p.err)) {
            ok = false; break;
          }
          tc_fence_after();
          issue_scores(ls1, s1);
        }
        if (!mbar_wait(&ds_full[s], (i >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {      // 64 keys, 16 per instruction
          umma_bf16(tmem_base + C::COL_DQ, make_smem_desc_sw128(ds_base + s * 16384 + kk * 32, 16, 1024),
                    make_smem_desc_sw128(k_base + ls * C::KV + kk * 2048, 8192, 1024), idesc_dq,
                    (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[ls]);
        umma_commit(&ds_free[s]);
      }
      if (ok) umma_commit(dq_full);
    }
    __syncwarp();
  } else {
    const int grp = warp >> 2;                    // compute group: handles key blocks i = grp, grp+2, ...
    const int t = threadIdx.x & 127;
    const int row = q0 + t;
    const int pos = p.q_offset + row;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    float lse2 = 0.f, dl = 0.f;
    if (row < p.Sq) {
      const size_t idx = (static_cast<size_t>(b) * p.Hq + head) * p.Sq + row;
      lse2 = p.lse[idx] * 1.4426950408889634f;
      dl = p.delta[(static_cast<size_t>(b) * p.Hq + head) * p.sq_pad + row];
    }
    uint8_t* ds_tiles = smem + C::OFF_DS;
    bool ok = true;
    const bool row_ok = row < p.Sq;
    // The two groups work on alternate key blocks (stage = group), so one group's TMEM
    // read latency and barrier waits overlap the other group's arithmetic.
    for (int i = grp; i < nblk && ok; i += 2) {
      const int s = grp;
      const uint32_t par = (i >> 1) & 1;
      const int kv0 = (j_begin + i) * 64;
      if (!mbar_wait(&sdp_full[s], par, abort_flag, p.err) || !mbar_wait(&ds_free[s], par ^ 1, abort_flag, p.err)) {
        ok = false; break;
      }
      tc_fence_after();
      const bool need_mask = !row_ok || kv0 + 64 > p.Sk || (p.causal && kv0 + 63 > pos) || p.window >= 0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32b_x32(tmem_base + C::COL_S + 64 * s + lane_sel + c * 32, sv);
        tmem_ld_32x32b_x32(tmem_base + C::COL_DP + 64 * s + lane_sel + c * 32, dp);
        tmem_ld_wait();
        if (c == 1) {
          tc_fence_before();
          mbar_arrive(&sdp_free[s]);
        }
        float ds[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) {
          const float pr = exp2f(fmaf(__uint_as_float(sv[k]), p.scale_log2, -lse2));
          ds[k] = pr * (__uint_as_float(dp[k]) - dl);
        }
        if (need_mask) {
#pragma unroll
          for (int k = 0; k < 32; ++k)
            if (!row_ok || att_blocked(p, pos, kv0 + c * 32 + k)) ds[k] = 0.f;
        }
        // [128 x 64] bf16 tile = one 128-byte swizzled row per query
        uint8_t* dst = ds_tiles + s * 16384 + t * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack_bf16(ds[8 * g + 0], ds[8 * g + 1]);
          w.y = pack_bf16(ds[8 * g + 2], ds[8 * g + 3]);
          w.z = pack_bf16(ds[8 * g + 4], ds[8 * g + 5]);
          w.w = pack_bf16(ds[8 * g + 6], ds[8 * g + 7]);
          const int j16 = c * 4 + g;
          *reinterpret_cast<uint4*>(dst + ((j16 ^ (t & 7)) << 4)) = w;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&ds_full[s]);
    }
    // epilogue: dQ = scale * accumulator; group g stages columns [g*D/2, (g+1)*D/2)
    uint8_t* stage = smem + C::OFF_DS;            // 32 KB, all products are complete
    if (ok && nblk > 0 && mbar_wait(dq_full, 0, abort_flag, p.err)) {
      tc_fence_after();
      constexpr int HALF = D / 2;
#pragma unroll
      for (int c = 0; c < HALF / 32; ++c) {
        const int col = grp * HALF + c * 32;
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + C::COL_DQ + lane_sel + col, v);
        tmem_ld_wait();
        uint8_t* dst = stage + (col >> 6) * 16384 + t * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          uint4 w;
          w.x = pack_bf16(__uint_as_float(v[8 * g + 0]) * p.scale, __uint_as_float(v[8 * g + 1]) * p.scale);
          w.y = pack_bf16(__uint_as_float(v[8 * g + 2]) * p.scale, __uint_as_float(v[8 * g + 3]) * p.scale);
          w.z = pack_bf16(__uint_as_float(v[8 * g + 4]) * p.scale, __uint_as_float(v[8 * g + 5]) * p.scale);
          w.w = pack_bf16(__uint_as_float(v[8 * g + 6]) * p.scale, __uint_as_float(v[8 * g + 7]) * p.scale);
          const int j16 = ((col & 63) >> 3) + g;
          *reinterpret_cast<uint4*>(dst + ((j16 ^ (t & 7)) << 4)) = w;
        }
      }
    }
    fence_proxy_async_smem();
    asm volatile("bar.sync 1, 256;" ::: "memory");
    if (grp == 0 && nblk > 0) {
      const int row0 = q0 + (warp & 3) * 32;
      if (lane == 0 && row0 < p.Sq) {
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_store_4d(&tmDQ, stage + h * 16384 + (warp & 3) * 4096, h * 64, head, row0, b);
        tma_store_commit();
        tma_store_wait_all<0>();
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

// ---------------------------------------------------------------------------- dK / dV
// Pipelined over 64-query blocks with the same double-buffering scheme as the dQ kernel.
template <int D>
struct AttDkv {
  static constexpr int TILE = 128 * D * 2;        // K / V tile (128 rows)
  static constexpr int QS = 64 * D * 2;           // Q / dO stage (64 rows)
  static constexpr int OFF_K = 0, OFF_V = TILE;
  static constexpr int NS = (D == 64) ? 4 : 3;    // Q / dO load stages (the loader runs ahead of the products)
  static constexpr int OFF_Q = 2 * TILE;          // NS stages
  static constexpr int OFF_DO = OFF_Q + NS * QS;  // NS stages
  static constexpr int OFF_PT = OFF_DO + NS * QS; // 2 stages of [128 x 64] bf16
  static constexpr int OFF_DST = OFF_PT + 2 * 16384;
  static constexpr int OFF_STAT = OFF_DST + 2 * 16384;       // [NS][lse2[64], delta[64]]
  static constexpr int OFF_BAR = OFF_STAT + NS * 512;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int COL_ST = 0, COL_DPT = 128, COL_DV = 256, COL_DK = 256 + D;
};

template <int D>
__global__ void __launch_bounds__(ATTB_THREADS, 1)
attention_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                     const AttBwdParams p) {
  using C = AttDkv<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  constexpr int NS = C::NS;
  uint64_t* kv_full = bars + 0;
  uint64_t* sdp_full = bars + 1;    // [2]
  uint64_t* sdp_free = bars + 3;    // [2] 128 arrivals
  uint64_t* pds_full = bars + 5;    // [2] 128 arrivals
  uint64_t* pds_free = bars + 7;    // [2]
  uint64_t* acc_full = bars + 9;
  uint64_t* qdo_full = bars + 10;           // [NS]
  uint64_t* qdo_empty = bars + 10 + NS;     // [NS]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 10 + 2 * NS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stats = reinterpret_cast<float*>(smem + C::OFF_STAT);   // [stage][0:64 lse2, 64:128 delta]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int kblk = blockIdx.x, kv_head = blockIdx.y, b = blockIdx.z;
  const int kv0 = kblk * 128;
  const int group = p.Hq / p.Hkv;
  int qb_begin = 0;
  const int qb_end = (p.Sq + 63) / 64;
  if (p.causal) qb_begin = max(0, (kv0 - p.q_offset) / 64);
  const int nqb = max(0, qb_end - qb_begin);
  const int niter = nqb * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    for (int s = 0; s < 2; ++s) {
      mbar_init(&sdp_full[s], 1);
      mbar_init(&sdp_free[s], 128); mbar_init(&pds_full[s], 128); mbar_init(&pds_free[s], 1);
    }
    for (int s = 0; s < NS; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&qdo_empty[s], 1); }
    mbar_init(acc_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == 9) { tmem_alloc(tmem_slot, 512); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    if (lane == 0 && niter > 0) {
      mbar_expect_tx(kv_full, 2 * C::TILE);
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        tma_load_4d(smem + C::OFF_K + h * 16384, &tmK, kv_full, h * 64, kv_head, kv0, b);
        tma_load_4d(smem + C::OFF_V + h * 16384, &tmV, kv_full, h * 64, kv_head, kv0, b);
      }
      for (int i = 0; i < niter; ++i) {
        const int s = i % NS;
        const int hq = kv_head * group + i / nqb;
        const int q0 = (qb_begin + i % nqb) * 64;
        if (!mbar_wait(&qdo_empty[s], ((i / NS) & 1) ^ 1, abort_flag, p.err)) break;
        mbar_expect_tx(&qdo_full[s], 2 * C::QS + 512);
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          tma_load_4d(smem + C::OFF_Q + s * C::QS + h * 8192, &tmQ, &qdo_full[s], h * 64, hq, q0, b);
          tma_load_4d(smem + C::OFF_DO + s * C::QS + h * 8192, &tmDO, &qdo_full[s], h * 64, hq, q0, b);
        }
        // the 64 queries' log-sum-exp and delta values ride on the same barrier
        const size_t srow = (static_cast<size_t>(b) * p.Hq + hq) * p.sq_pad + q0;
        bulk_load(stats + s * 128, p.lse2 + srow, 256, &qdo_full[s]);
        bulk_load(stats + s * 128 + 64, p.delta + srow, 256, &qdo_full[s]);
      }
      if (*abort_flag) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) {} }
    }
    __syncwarp();
  } else if (warp == 9) {
    if (lane == 0 && niter > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
      const uint32_t k_base = smem_u32(smem + C::OFF_K), v_base = smem_u32(smem + C::OFF_V);
      const uint32_t q_base = smem_u32(smem + C::OFF_Q), do_base = smem_u32(smem + C::OFF_DO);
      const uint32_t pt_base = smem_u32(smem + C::OFF_PT), dst_base = smem_u32(smem + C::OFF_DST);
      auto issue_scores = [&](int ls, int tb) {     // ls: Q/dO ring stage, tb: TMEM buffer
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {      // S^T = K Q^T
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t boff = ls * C::QS + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + C::COL_ST + 64 * tb, make_smem_desc_sw128(k_base + aoff, 16, 1024),
                    make_smem_desc_sw128(q_base + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {      // dP^T = V dO^T
          const uint32_t aoff = (kk >> 2) * 16384 + (kk & 3) * 32;
          const uint32_t boff = ls * C::QS + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16(tmem_base + C::COL_DPT + 64 * tb, make_smem_desc_sw128(v_base + aoff, 16, 1024),
                    make_smem_desc_sw128(do_base + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[tb]);
      };
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err) && mbar_wait(&qdo_full[0], 0, abort_flag, p.err);
      if (ok) { tc_fence_after(); issue_scores(0, 0); }
      for (int i = 0; i < niter && ok; ++i) {
        const int s = i & 1;
        const int ls = i % NS;
        if (i + 1 < niter) {
          const int s1 = (i + 1) & 1;
          const int ls1 = (i + 1) % NS;
          if (!mbar_wait(&qdo_full[ls1], ((i + 1) / NS) & 1, abort_flag, p.err) ||
              !mbar_wait(&sdp_free[s1], (((i + 1) >> 1) & 1) ^ 1, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          issue_scores(ls1, s1);
        }
        if (!mbar_wait(&pds_full[s], (i >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {           // dV += P^T dO (contraction over 64 queries)
          umma_bf16(tmem_base + C::COL_DV, make_smem_desc_sw128(pt_base + s * 16384 + kk * 32, 16, 1024),
                    make_smem_desc_sw128(do_base + ls * C::QS + kk * 2048, 8192, 1024), idesc_acc,
                    (i > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {           // dK += dS^T Q
          umma_bf16(tmem_base + C::COL_DK, make_smem_desc_sw128(dst_base + s * 16384 + kk * 32, 16, 1024),
                    make_smem_desc_sw128(q_base + ls * C::QS + kk * 2048, 8192, 1024), idesc_acc,
                    (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&qdo_empty[ls]);
        umma_commit(&pds_free[s]);
      }
      if (ok) umma_commit(acc_full);
    }
    __syncwarp();
  } else {
    const int grp = warp >> 2;                     // compute group: handles iterations i = grp, grp+2, ...
    const int t = threadIdx.x & 127;               // key row in the block == TMEM lane
    const int kv = kv0 + t;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    uint8_t* pt_tiles = smem + C::OFF_PT;
    uint8_t* dst_tiles = smem + C::OFF_DST;
    bool ok = true;
    for (int i = grp; i < niter && ok; i += 2) {
      const int s = grp;
      const uint32_t par = (i >> 1) & 1;
      const int q0 = (qb_begin + i % nqb) * 64;
      const int ls = i % NS;
      const float4* st4 = reinterpret_cast<const float4*>(stats + ls * 128);
      // qdo_full also covers the statistics copied by the loader
      if (!mbar_wait(&qdo_full[ls], (i / NS) & 1, abort_flag, p.err) || !mbar_wait(&sdp_full[s], par, abort_flag, p.err) ||
          !mbar_wait(&pds_free[s], par ^ 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = q0 + 64 > p.Sq || kv >= p.Sk || (p.causal && kv > p.q_offset + q0) || p.window >= 0;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32b_x32(tmem_base + C::COL_ST + 64 * s + lane_sel + c * 32, sv);
        tmem_ld_32x32b_x32(tmem_base + C::COL_DPT + 64 * s + lane_sel + c * 32, dp);
        tmem_ld_wait();
        if (c == 1) {
          tc_fence_before();
          mbar_arrive(&sdp_free[s]);
        }
        float pr[32], ds[32];
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const float4 l4 = st4[c * 8 + k4];          // lse2 of 4 queries (broadcast read)
          const float4 d4 = st4[16 + c * 8 + k4];     // delta of the same queries
          const float lv[4] = {l4.x, l4.y, l4.z, l4.w};
          const float dv4[4] = {d4.x, d4.y, d4.z, d4.w};
#pragma unroll
          for (int j = 0; j < 4; ++j) {
            const int k = 4 * k4 + j;
            const float pv = exp2f(fmaf(__uint_as_float(sv[k]), p.scale_log2, -lv[j]));
            pr[k] = pv;
            ds[k] = pv * (__uint_as_float(dp[k]) - dv4[j]);
          }
        }
        if (need_mask) {
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const int r = q0 + c * 32 + k;
            if (r >= p.Sq || att_blocked(p, p.q_offset + r, kv)) { pr[k] = 0.f; ds[k] = 0.f; }
          }
        }
        uint8_t* d0 = pt_tiles + s * 16384 + t * 128;
        uint8_t* d1 = dst_tiles + s * 16384 + t * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          const int sw = ((c * 4 + g) ^ (t & 7)) << 4;
          uint4 w;
          w.x = pack_bf16(pr[8 * g + 0], pr[8 * g + 1]);
          w.y = pack_bf16(pr[8 * g + 2], pr[8 * g + 3]);
          w.z = pack_bf16(pr[8 * g + 4], pr[8 * g + 5]);
          w.w = pack_bf16(pr[8 * g + 6], pr[8 * g + 7]);
          *reinterpret_cast<uint4*>(d0 + sw) = w;
          w.x = pack_bf16(ds[8 * g + 0], ds[8 * g + 1]);
          w.y = pack_bf16(ds[8 * g + 2], ds[8 * g + 3]);
          w.z = pack_bf16(ds[8 * g + 4], ds[8 * g + 5]);
          w.w = pack_bf16(ds[8 * g + 6], ds[8 * g + 7]);
          *reinterpret_cast<uint4*>(d1 + sw) = w;
        }
      }
      fence_proxy_async_smem();
      mbar_arrive(&pds_full[s]);
    }
    // both groups must be out of the loop before the staging tiles are reused
    asm volatile("bar.sync 1, 256;" ::: "memory");
    // epilogue: group 0 stores dV, group 1 stores dK (scaled); staging reuses the P^T /
    // dS^T stages (2 x 16 KB = D/64 halves of a [128 x D] tile)
    uint8_t* stage = grp == 0 ? pt_tiles : dst_tiles;
    if (ok && niter > 0 && mbar_wait(acc_full, 0, abort_flag, p.err)) {
      tc_fence_after();
      const float mul = grp == 0 ? 1.f : p.scale;
      const uint32_t col_base = grp == 0 ? C::COL_DV : C::COL_DK;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) {
        uint32_t v[32];
        tmem_ld_32x32b_x32(tmem_base + col_base + lane_sel + c * 32, v);
        tmem_ld_wait();
        float f[32];
#pragma unroll
        for (int k = 0; k < 32; ++k) f[k] = __uint_as_float(v[k]) * mul;
        store_chunk_sw128(stage, t, c, f);
      }
    } else if (niter == 0) {
      float z[32];
#pragma unroll
      for (int k = 0; k < 32; ++k) z[k] = 0.f;
#pragma unroll
      for (int c = 0; c < D / 32; ++c) store_chunk_sw128(stage, t, c, z);
    }
    fence_proxy_async_smem();
    __syncwarp();
    const int row0 = kv0 + (warp & 3) * 32;
    if (lane == 0 && row0 < p.Sk) {
#pragma unroll
      for (int h = 0; h < D / 64; ++h) {
        if (grp == 0) tma_store_4d(&tmDV, stage + h * 16384 + (warp & 3) * 4096, h * 64, kv_head, row0, b);
        else tma_store_4d(&tmDK, stage + h * 16384 + (warp & 3) * 4096, h * 64, kv_head, row0, b);
      }
      tma_store_commit();
      tma_store_wait_all<0>();
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 9) { tc_fence_after(); tmem_dealloc(tmem_base, 512); }
}

static int make_tmap_bshd_b(CUtensorMap* m, const void* base, int B, int S, int H, int D, const long* st, int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)st[2] * 2, (uint64_t)st[1] * 2, (uint64_t)st[0] * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap(m, base, 2, 4, dims, strides, box, true);
}

template <typename K>
static int set_smem(K kern, int bytes, bool* flags) {
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!flags[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes));
    flags[dev & 63] = true;
  }
  return SB_OK;
}

template <int D>
static int launch_att_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout, const float* lse,
                          float* delta, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq, int Sk,
                          const long* qs, const long* ks, const long* vs, const long* os, const long* dos,
                          const long* dqs, const long* dks, const long* dvs, int causal, int window, int q_offset,
                          float scale, cudaStream_t st, unsigned int* err_word_override = nullptr) {
  CUtensorMap tmQ, tmK, tmV, tmDO, tmDQ, tmDK, tmDV, tmQ64, tmDO64, tmK64, tmV64;
  int rc;
  if ((rc = make_tmap_bshd_b(&tmQ64, q, B, Sq, Hq, D, qs, 64))) return rc;
  if ((rc = make_tmap_bshd_b(&tmDO64, dout, B, Sq, Hq, D, dos, 64))) return rc;
  if ((rc = make_tmap_bshd_b(&tmK64, k, B, Sk, Hkv, D, ks, 64))) return rc;
  if ((rc = make_tmap_bshd_b(&tmV64, v, B, Sk, Hkv, D, vs, 64))) return rc;
  if ((rc = make_tmap_bshd_b(&tmQ, q, B, Sq, Hq, D, qs, 128))) return rc;
  if ((rc = make_tmap_bshd_b(&tmK, k, B, Sk, Hkv, D, ks, 128))) return rc;
  if ((rc = make_tmap_bshd_b(&tmV, v, B, Sk, Hkv, D, vs, 128))) return rc;
  if ((rc = make_tmap_bshd_b(&tmDO, dout, B, Sq, Hq, D, dos, 128))) return rc;
  if ((rc = make_tmap_bshd_b(&tmDQ, dq, B, Sq, Hq, D, dqs, 32))) return rc;
  if ((rc = make_tmap_bshd_b(&tmDK, dk, B, Sk, Hkv, D, dks, 32))) return rc;
  if ((rc = make_tmap_bshd_b(&tmDV, dv, B, Sk, Hkv, D, dvs, 32))) return rc;
  AttBwdParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk;
  p.causal = causal; p.window = window; p.q_offset = q_offset;
  p.scale = scale; p.scale_log2 = scale * 1.4426950408889634f;
  const int sq_pad = (Sq + 63) / 64 * 64;
  float* lse2 = delta + (size_t)B * Hq * sq_pad;
  p.lse = lse; p.delta = delta; p.lse2 = lse2; p.sq_pad = sq_pad;
  p.err = err_word_override ? err_word_override : error_word();
  if (!p.err) return SB_ERR_CUDA;

  {
    const long warps = (long)B * sq_pad * Hq;
    const int blocks = (int)((warps + 7) / 8);
    attention_delta_kernel<D><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta,
                                                      lse2, B, Sq, sq_pad, Hq, os[0], os[1], os[2], dos[0], dos[1],
                                                      dos[2]);
  }
  static bool f1[64] = {false}, f2[64] = {false};
  auto kq = attention_dq_kernel<D>;
  auto kkv = attention_dkv_kernel<D>;
  if ((rc = set_smem(kq, AttDq<D>::SMEM_BYTES, f1))) return rc;
  if ((rc = set_smem(kkv, AttDkv<D>::SMEM_BYTES, f2))) return rc;
  kkv<<<dim3((Sk + 127) / 128, Hkv, B), ATTB_THREADS, AttDkv<D>::SMEM_BYTES, st>>>(tmQ64, tmK, tmV, tmDO64, tmDK, tmDV, p);
  kq<<<dim3((Sq + 127) / 128, Hq, B), ATTB_THREADS, AttDq<D>::SMEM_BYTES, st>>>(tmQ, tmK64, tmV64, tmDO, tmDQ, p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

// Backward of sb_attention_fwd. All tensors bf16 `[B,S,H,D]` with element strides
// {batch, seq, head}; lse and the scratch `delta` are fp32 `[B,Hq,Sq]`. dq/dk/dv may be
// strided views (e.g. slices of one packed dqkv buffer). `delta` is scratch of
// 2 * B * Hq * roundup(Sq, 64) floats.
extern "C" int sb_attention_bwd(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                const float* lse, float* delta, void* dq, void* dk, void* dv, int B, int Hq, int Hkv,
                                int Sq, int Sk, int D, const long* qs, const long* ks, const long* vs, const long* os,
                                const long* dos, const long* dqs, const long* dks, const long* dvs, int causal,
                                int window, int q_offset, float scale, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(D == 64 || D == 128);
  SB_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && Sk > 0);
  if (D == 64)
    return launch_att_bwd<64>(q, k, v, o, dout, lse, delta, dq, dk, dv, B, Hq, Hkv, Sq, Sk, qs, ks, vs, os, dos, dqs,
                              dks, dvs, causal, window, q_offset, scale, st);
  return launch_att_bwd<128>(q, k, v, o, dout, lse, delta, dq, dk, dv, B, Hq, Hkv, Sq, Sk, qs, ks, vs, os, dos, dqs, dks,
                             dvs, causal, window, q_offset, scale, st);
}

// ---------------------------------------------------------------------------- allocation-free entry
// See no_alloc.h. The scratch that sb_attention_bwd takes from its caller (the per-row
// `delta` values) lives here in a fixed device array, as does the word the kernels use to
// report a timed-out wait, so this path never asks the CUDA allocator for anything.
namespace {
constexpr long kStaticDeltaFloats = 1L << 21;     // 8 MiB per device that loads the library
static __device__ __align__(256) float g_static_delta[kStaticDeltaFloats];
static __device__ __align__(256) unsigned int g_static_err_word[64];

struct StaticPtrs {
  float* delta;
  unsigned int* err;
  bool ready;
};
StaticPtrs g_static_ptrs[64];
}  // namespace

extern "C" int sb_attention_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                        const float* lse, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                                        int Sk, int D, const long* qs, const long* ks, const long* vs, const long* os,
                                        const long* dos, const long* dqs, const long* dks, const long* dvs, int causal,
                                        int window, int q_offset, float scale, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(D == 64 || D == 128);
  SB_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && Sk > 0);
  const long need = 2L * B * Hq * ((Sq + 63) / 64 * 64);     // two arrays, rows padded to 64
  if (need > kStaticDeltaFloats) {
    fprintf(stderr,
            "summa_b200: sb_attention_bwd_noalloc: 2*batch*heads*roundup(queries,64) = %ld exceeds the built-in "
            "scratch of %ld values; use sb_attention_bwd with caller-provided scratch\n", need, kStaticDeltaFloats);
    return SB_ERR_TOO_LARGE;
  }
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64);
  StaticPtrs& sp = g_static_ptrs[dev];
  if (!sp.ready) {
    // One-time set-up for this device (it is current): the array names above are host-side
    // handles, the kernels need the device addresses behind them.
    void* pd = nullptr;
    void* pe = nullptr;
    SB_CHECK_CUDA(cudaGetSymbolAddress(&pd, g_static_delta));
    SB_CHECK_CUDA(cudaGetSymbolAddress(&pe, g_static_err_word));
    sp.delta = static_cast<float*>(pd);
    sp.err = static_cast<unsigned int*>(pe);
    sp.ready = true;
  }
  if (D == 64)
    return launch_att_bwd<64>(q, k, v, o, dout, lse, sp.delta, dq, dk, dv, B, Hq, Hkv, Sq, Sk, qs, ks, vs, os, dos, dqs,
                              dks, dvs, causal, window, q_offset, scale, st, sp.err);
  return launch_att_bwd<128>(q, k, v, o, dout, lse, sp.delta, dq, dk, dv, B, Hq, Hkv, Sq, Sk, qs, ks, vs, os, dos, dqs,
                             dks, dvs, causal, window, q_offset, scale, st, sp.err);
}
