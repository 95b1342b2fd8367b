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
#include <mutex>

namespace sb {

constexpr int ATTB_DKV_THREADS = 352;   // 8 compute warps, loader, score issuer, accumulate issuer

struct AttBwdParams {
  int B, Hq, Hkv, Sq, Sk;
  int causal, window, q_offset;
  float scale, scale_log2;
  const float* lse;     // [B, Hq, Sq] natural log
  const float* delta;   // [B, Hq, sq_pad] scratch: -sum_d dO*O
  const float* lse2;    // [B, Hq, sq_pad] scratch: -lse * log2(e)
  int sq_pad;           // Sq rounded up to 64 (row pitch of the two scratch arrays)
  unsigned int* err;
};

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
// delta[b,h,s] = -sum_d dO*O and lse2[b,h,s] = -lse*log2(e) (both NEGATED, so that the main
// kernels only need fused multiply-adds), with row pitch sq_pad; rows in [Sq, sq_pad) are
// written as zeros so that bulk copies of 64-row slices are clean.
template <int D>
__global__ void attention_delta_kernel(const __nv_bfloat16* __restrict__ o, const __nv_bfloat16* __restrict__ dout,
                                       const float* __restrict__ lse, float* __restrict__ delta,
                                       float* __restrict__ lse2, int B, int Sq, int sq_pad, int Hq, long o_sb, long o_ss,
                                       long o_sh, long d_sb, long d_ss, long d_sh) {
  // D / 8 threads per (batch, row, head), 16 bytes of O and dO each
  constexpr int TPR = D / 8;
  const long gt = blockIdx.x * (long)blockDim.x + threadIdx.x;
  const long item = gt / TPR;
  const int part = gt % TPR;
  const long total = (long)B * sq_pad * Hq;
  if (item >= total) return;                       // whole sub-groups leave together (blockDim % TPR == 0)
  const int h = item % Hq;
  const long r = item / Hq;
  const int s = r % sq_pad;
  const int b = r / sq_pad;
  const long oidx = ((long)b * Hq + h) * sq_pad + s;
  float acc = 0.f;
  if (s < Sq) {
    const uint4 a = *reinterpret_cast<const uint4*>(o + b * o_sb + s * o_ss + h * o_sh + part * 8);
    const uint4 c = *reinterpret_cast<const uint4*>(dout + b * d_sb + s * d_ss + h * d_sh + part * 8);
    acc = bf16_lo(a.x) * bf16_lo(c.x) + bf16_hi(a.x) * bf16_hi(c.x) + bf16_lo(a.y) * bf16_lo(c.y) +
          bf16_hi(a.y) * bf16_hi(c.y) + bf16_lo(a.z) * bf16_lo(c.z) + bf16_hi(a.z) * bf16_hi(c.z) +
          bf16_lo(a.w) * bf16_lo(c.w) + bf16_hi(a.w) * bf16_hi(c.w);
  }
#pragma unroll
  for (int m = TPR / 2; m > 0; m >>= 1) acc += __shfl_xor_sync(0xffffffffu, acc, m);
  if (part == 0) {
    delta[oidx] = -acc;
    lse2[oidx] = s < Sq ? -lse[((long)b * Hq + h) * Sq + s] * 1.4426950408889634f : 0.f;
  }
}

// ---------------------------------------------------------------------------- dQ
// One CTA per (128 queries, head, batch), pipelined over 64-key blocks. Q and dO (bf16) are
// copied into tensor memory once and serve as the A operands of S = Q K^T and dP = dO V^T; the
// threads overwrite S in place with dS (packed bf16), the A operand of dQ += dS K. Shared
// memory only feeds the B operands (the K / V stage). As in the dK/dV kernel below, the score
// products and the accumulate products are issued by two different warps so that one warp's
// commit stall overlaps the other's products; with head_dim 64 dS has its own TMEM columns
// (the score products of block i + 2 then only wait for the threads to have read block i),
// with head_dim 128 it overwrites S in place.
template <int D>
struct AttDq {
  static constexpr int TILE = 128 * D * 2;        // Q / dO tile (128 rows)
  static constexpr int KV = 64 * D * 2;           // K / V stage (64 rows)
  static constexpr int NS = 4;                    // K / V load stages (the loader runs ahead of the products)
  static constexpr int OFF_Q = 0, OFF_DO = TILE;
  static constexpr int OFF_K = 2 * TILE;          // NS stages
  static constexpr int OFF_V = OFF_K + NS * KV;   // NS stages
  static constexpr int OFF_BAR = OFF_V + NS * KV;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr bool SEP = (D == 64);          // separate TMEM columns for dS
  static constexpr int COL_QT = 0, COL_DOT = D / 2;                 // bf16 tiles: D/2 columns each
  static constexpr int COL_S = D, COL_DP = D + 128, COL_DQ = D + 256;   // S/dP: buffer b at +64*b
  static constexpr int COL_DS = SEP ? D + 256 + D : COL_S;          // + DS_STRIDE * buffer (448 / 512 columns in use)
  static constexpr int DS_STRIDE = SEP ? 32 : 64;
};

template <int D>
__global__ void __launch_bounds__(ATTB_DKV_THREADS, 1)
attention_dq_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                    const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                    const __grid_constant__ CUtensorMap tmDQ, const AttBwdParams p) {
  using C = AttDq<D>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  constexpr int NS = C::NS;
  uint64_t* qdo_full = bars + 0;
  uint64_t* qdot_full = bars + 1;   // 256 arrivals: Q / dO copied into tensor memory
  uint64_t* sdp_full = bars + 2;    // [2] score issuer -> threads
  uint64_t* sdp_free = bars + 4;    // [2] 128 arrivals: threads have read S / dP (SEP only)
  uint64_t* ds_full = bars + 6;     // [2] 128 arrivals: dS written
  uint64_t* dq_full = bars + 8;
  uint64_t* kv_full = bars + 9;             // [NS]
  uint64_t* done = bars + 9 + NS;           // [NS] accumulate product of the block using stage s completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 9 + 2 * NS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (heads, batch, query blocks): blocks are handed out x-fastest, so all the heaviest
  // (latest, under a causal mask) query blocks start first and the tail of the launch is made
  // of the lightest ones
  const int qblk = gridDim.z - 1 - blockIdx.z;
  const int head = blockIdx.x, b = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qblk * 128;
  int j_begin = 0, j_end = (p.Sk + 63) / 64;
  if (p.causal) j_end = min(j_end, (p.q_offset + q0 + 127) / 64 + 1);
  if (p.window >= 0) j_begin = max(0, (p.q_offset + q0 - p.window) / 64);
  const int nblk = max(0, j_end - j_begin);

  if (threadIdx.x == 0) {
    mbar_init(qdo_full, 1);
    mbar_init(qdot_full, 256);
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&sdp_free[s], 128); mbar_init(&ds_full[s], 128); }
    for (int s = 0; s < NS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&done[s], 1); }
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
        if (!mbar_wait(&done[s], ((i / NS) & 1) ^ 1, abort_flag, p.err)) break;
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
    // ------------------------------------------------------------ score issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      const uint32_t k_base = smem_u32(smem + C::OFF_K), v_base = smem_u32(smem + C::OFF_V);
      bool ok = mbar_wait(qdot_full, 0, abort_flag, p.err);
      for (int j = 0; j < nblk && ok; ++j) {
        const int tb = j & 1, ls = j % NS;
        if (!mbar_wait(&kv_full[ls], (j / NS) & 1, abort_flag, p.err)) { ok = false; break; }
        if (j >= 2) {
          const bool got = C::SEP ? mbar_wait(&sdp_free[tb], ((j >> 1) - 1) & 1, abort_flag, p.err)
                                  : mbar_wait(&done[(j - 2) % NS], ((j - 2) / NS) & 1, abort_flag, p.err);
          if (!got) { ok = false; break; }
        }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t boff = ls * C::KV + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16_ta(tmem_base + C::COL_S + 64 * tb, tmem_base + C::COL_QT + 8 * kk,
                       make_smem_desc_sw128(k_base + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t boff = ls * C::KV + (kk >> 2) * 8192 + (kk & 3) * 32;
          umma_bf16_ta(tmem_base + C::COL_DP + 64 * tb, tmem_base + C::COL_DOT + 8 * kk,
                       make_smem_desc_sw128(v_base + boff, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&sdp_full[tb]);
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------------------------ accumulate issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_dq = make_idesc_bf16(128, D, 0, 1);   // dS (TMEM) x K stage (N-major)
      const uint32_t k_base = smem_u32(smem + C::OFF_K);
      bool ok = true;
      for (int i = 0; i < nblk && ok; ++i) {
        const int s = i & 1, ls = i % NS;
        if (!mbar_wait(&ds_full[s], (i >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {      // 64 keys, 16 per instruction
          umma_bf16_ta(tmem_base + C::COL_DQ, tmem_base + C::COL_DS + C::DS_STRIDE * s + 8 * kk,
                       make_smem_desc_sw128(k_base + ls * C::KV + kk * 2048, 8192, 1024), idesc_dq,
                       (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&done[ls]);     // frees the K / V stage and the dS buffer
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
    float nlse2 = 0.f, ndl = 0.f;                  // negated statistics of this query row
    if (row < p.Sq) {
      const size_t idx = (static_cast<size_t>(b) * p.Hq + head) * p.sq_pad + row;
      nlse2 = p.lse2[idx];
      ndl = p.delta[idx];
    }
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
    const uint64_t nl2 = f2_pack(nlse2, nlse2), nd2 = f2_pack(ndl, ndl);
    bool ok = true;
    const bool row_ok = row < p.Sq;
    if (nblk > 0) {
      // copy Q (group 0) / dO (group 1) into tensor memory: thread t owns row t of the tile
      if (mbar_wait(qdo_full, 0, abort_flag, p.err)) {
        const uint8_t* src = smem + (grp == 0 ? C::OFF_Q : C::OFF_DO) + t * 128;
#pragma unroll
        for (int h = 0; h < D / 64; ++h) {
          uint32_t r[32];
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            const uint4 w = *reinterpret_cast<const uint4*>(src + h * 16384 + ((j ^ (t & 7)) << 4));
            r[4 * j + 0] = w.x; r[4 * j + 1] = w.y; r[4 * j + 2] = w.z; r[4 * j + 3] = w.w;
          }
          tmem_st_32x32b_x32(tmem_base + (grp == 0 ? C::COL_QT : C::COL_DOT) + 32 * h + lane_sel, r);
        }
        tmem_st_wait();
        tc_fence_before();
        mbar_arrive(qdot_full);
      } else {
        ok = false;
      }
    }
    // The two groups work on alternate key blocks (TMEM buffer = group), so one group's TMEM
    // latency and barrier waits overlap the other group's arithmetic.
    for (int i = grp; i < nblk && ok; i += 2) {
      const int s = grp;
      const uint32_t par = (i >> 1) & 1;
      const int kv0 = (j_begin + i) * 64;
      if (!mbar_wait(&sdp_full[s], par, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const bool need_mask = !row_ok || kv0 + 64 > p.Sk || (p.causal && kv0 + 63 > pos) || p.window >= 0;
      const uint32_t t_s = tmem_base + C::COL_S + 64 * s + lane_sel;
      const uint32_t t_dp = tmem_base + C::COL_DP + 64 * s + lane_sel;
      const uint32_t t_ds = tmem_base + C::COL_DS + C::DS_STRIDE * s + lane_sel;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32b_x32(t_s + c * 32, sv);
        tmem_ld_32x32b_x32(t_dp + c * 32, dp);
        tmem_ld_wait();
        if (C::SEP && c == 1) {
          tc_fence_before();
          mbar_arrive(&sdp_free[s]);     // scores fully read: the score issuer may refill this buffer
        }
        float ds[32];
#pragma unroll
        for (int k = 0; k < 32; k += 2) {
          float x0, x1;
          f2_unpack(f2_fma(f2_pack_u(sv[k], sv[k + 1]), scale2, nl2), x0, x1);
          const uint64_t pr2 = f2_pack(fast_exp2(x0), fast_exp2(x1));
          f2_unpack(f2_mul(pr2, f2_add(f2_pack_u(dp[k], dp[k + 1]), nd2)), ds[k], ds[k + 1]);
        }
        if (need_mask) {
          // branch-free: this row may see keys [lo, hi] (in units of this chunk's columns)
          int lo = 0, hi = p.Sk - 1;
          if (p.causal) hi = min(hi, pos);
          if (p.window >= 0) { lo = max(lo, pos - p.window); hi = min(hi, pos + p.window); }
          if (!row_ok) hi = -1;
          lo -= kv0 + c * 32;
          hi -= kv0 + c * 32;
#pragma unroll
          for (int k = 0; k < 32; ++k) ds[k] = (k >= lo && k <= hi) ? ds[k] : 0.f;
        }
        // keys [32c, 32c+32) become packed columns [16c, 16c+16); before the first write the
        // accumulate product of block i - 2 (which read this dS buffer) must have completed
        if (C::SEP && c == 0 && i >= 2) {
          if (!mbar_wait(&done[(i - 2) % NS], ((i - 2) / NS) & 1, abort_flag, p.err)) { ok = false; }
          tc_fence_after();
        }
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) pk[j] = pack_bf16(ds[2 * j], ds[2 * j + 1]);
        tmem_st_32x32b_x16(t_ds + c * 16, pk);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&ds_full[s]);
    }
    // epilogue: dQ = scale * accumulator; group g stages columns [g*D/2, (g+1)*D/2) into the
    // Q / dO tiles (their contents already live in tensor memory)
    uint8_t* stage = smem + C::OFF_Q;
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
// One CTA per (128 keys, kv head, batch), looping over (query head of the group, 64-query
// block). Per iteration: S^T = K Q^T and dP^T = V dO^T into tensor memory, the threads turn
// them into P^T and dS^T (packed bf16, written back to tensor memory), then dV += P^T dO and
// dK += dS^T Q with the A operand read from tensor memory.
// Short tcgen05 products (N = 64) cost about 45 cycles each from one issuing thread and every
// commit stalls that thread for a further ~190 cycles, but products issued by two different
// warps overlap in the tensor pipe. So the score products and the accumulate products are
// issued by two separate warps, each with its own commit.
//   head_dim 64 : P^T / dS^T have their own TMEM columns, so the score products of iteration
//                 i + 2 only wait for the threads to have READ the scores of iteration i.
//   head_dim 128: TMEM is full, P^T / dS^T overwrite S^T / dP^T in place and the score products
//                 of iteration i + 2 wait for the accumulate products of iteration i.
template <int D>
struct AttDkv {
  static constexpr bool SEP = (D == 64);          // separate TMEM columns for P^T / dS^T
  static constexpr int TILE = 128 * D * 2;        // K / V tile (128 rows)
  static constexpr int QS = 64 * D * 2;           // Q / dO stage (64 rows)
  static constexpr int NS = (D == 64) ? 6 : 4;    // Q / dO load stages (even, >= 4)
  static constexpr int OFF_K = 0, OFF_V = TILE;
  static constexpr int OFF_Q = 2 * TILE;          // NS stages
  static constexpr int OFF_DO = OFF_Q + NS * QS;  // NS stages
  static constexpr int OFF_STAT = OFF_DO + NS * QS;          // [NS][lse2[64], delta[64]]
  static constexpr int OFF_BAR = OFF_STAT + NS * 512;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  // tensor-memory columns (512 in use for either head_dim)
  static constexpr int COL_ST = 0;                                    // + 64 * buffer
  static constexpr int COL_DPT = 128;                                 // + 64 * buffer
  static constexpr int COL_PT = SEP ? 256 : COL_ST;                   // + (SEP ? 32 : 64) * buffer
  static constexpr int COL_DST = SEP ? 320 : COL_DPT;
  static constexpr int P_STRIDE = SEP ? 32 : 64;
  static constexpr int COL_DV = SEP ? 384 : 256, COL_DK = COL_DV + D;
};

template <int D>
__global__ void __launch_bounds__(ATTB_DKV_THREADS, 1)
attention_dkv_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmDO,
                     const __grid_constant__ CUtensorMap tmDK, const __grid_constant__ CUtensorMap tmDV,
                     const AttBwdParams p) {
  using C = AttDkv<D>;
  constexpr int NS = C::NS;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* kv_full = bars + 0;
  uint64_t* acc_full = bars + 1;
  uint64_t* sdp_full = bars + 2;    // [2] score issuer -> threads
  uint64_t* sdp_free = bars + 4;    // [2] 128 arrivals: threads have read S^T / dP^T (SEP only)
  uint64_t* pds_full = bars + 6;    // [2] 128 arrivals: P^T / dS^T written
  uint64_t* qdo_full = bars + 8;            // [NS]
  uint64_t* done = bars + 8 + NS;           // [NS] accumulate products of the iteration using stage s completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 8 + 2 * NS);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* stats = reinterpret_cast<float*>(smem + C::OFF_STAT);   // [stage][0:64 lse2, 64:128 delta]

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (kv heads, batch, key blocks): the earliest key blocks (most query blocks under a
  // causal mask) start first, see the dQ kernel
  const int kblk = blockIdx.z, kv_head = blockIdx.x, b = blockIdx.y;
  const int kv0 = kblk * 128;
  const int group = p.Hq / p.Hkv;
  int qb_begin = 0;
  const int qb_end = (p.Sq + 63) / 64;
  if (p.causal) qb_begin = max(0, (kv0 - p.q_offset) / 64);
  const int nqb = max(0, qb_end - qb_begin);
  const int niter = nqb * group;

  if (threadIdx.x == 0) {
    mbar_init(kv_full, 1);
    mbar_init(acc_full, 1);
    for (int s = 0; s < 2; ++s) { mbar_init(&sdp_full[s], 1); mbar_init(&sdp_free[s], 128); mbar_init(&pds_full[s], 128); }
    for (int s = 0; s < NS; ++s) { mbar_init(&qdo_full[s], 1); mbar_init(&done[s], 1); }
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
        if (!mbar_wait(&done[s], ((i / NS) & 1) ^ 1, abort_flag, p.err)) break;
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
    // ------------------------------------------------------------ score issuer
    if (lane == 0 && niter > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 64, 0, 0);
      const uint32_t k_base = smem_u32(smem + C::OFF_K), v_base = smem_u32(smem + C::OFF_V);
      const uint32_t q_base = smem_u32(smem + C::OFF_Q), do_base = smem_u32(smem + C::OFF_DO);
      bool ok = mbar_wait(kv_full, 0, abort_flag, p.err);
      for (int j = 0; j < niter && ok; ++j) {
        const int tb = j & 1, ls = j % NS;
        if (!mbar_wait(&qdo_full[ls], (j / NS) & 1, abort_flag, p.err)) { ok = false; break; }
        if (j >= 2) {
          // the TMEM buffer is free once the threads have read iteration j - 2 (SEP) or once the
          // accumulate products that read P^T / dS^T from it have completed (in place)
          const bool got = C::SEP ? mbar_wait(&sdp_free[tb], ((j >> 1) - 1) & 1, abort_flag, p.err)
                                  : mbar_wait(&done[(j - 2) % NS], ((j - 2) / NS) & 1, abort_flag, p.err);
          if (!got) { ok = false; break; }
        }
        tc_fence_after();
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
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ------------------------------------------------------------ accumulate issuer
    if (lane == 0 && niter > 0) {
      constexpr uint32_t idesc_acc = make_idesc_bf16(128, D, 0, 1);
      const uint32_t q_base = smem_u32(smem + C::OFF_Q), do_base = smem_u32(smem + C::OFF_DO);
      bool ok = true;
      for (int i = 0; i < niter && ok; ++i) {
        const int s = i & 1, ls = i % NS;
        if (!mbar_wait(&pds_full[s], (i >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {           // dV += P^T dO (contraction over 64 queries)
          umma_bf16_ta(tmem_base + C::COL_DV, tmem_base + C::COL_PT + C::P_STRIDE * s + 8 * kk,
                       make_smem_desc_sw128(do_base + ls * C::QS + kk * 2048, 8192, 1024), idesc_acc,
                       (i > 0 || kk > 0) ? 1u : 0u);
        }
#pragma unroll
        for (int kk = 0; kk < 4; ++kk) {           // dK += dS^T Q
          umma_bf16_ta(tmem_base + C::COL_DK, tmem_base + C::COL_DST + C::P_STRIDE * s + 8 * kk,
                       make_smem_desc_sw128(q_base + ls * C::QS + kk * 2048, 8192, 1024), idesc_acc,
                       (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&done[ls]);     // frees the Q / dO stage and the P^T / dS^T buffer
      }
      if (ok) umma_commit(acc_full);
    }
    __syncwarp();
  } else {
    const int grp = warp >> 2;                     // compute group: handles iterations i = grp, grp+2, ...
    const int t = threadIdx.x & 127;               // key row in the block == TMEM lane
    const int kv = kv0 + t;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    bool ok = true;
    for (int i = grp; i < niter && ok; i += 2) {
      const int s = grp;
      const uint32_t par = (i >> 1) & 1;
      const int q0 = (qb_begin + i % nqb) * 64;
      const int ls = i % NS;
      const float4* st4 = reinterpret_cast<const float4*>(stats + ls * 128);
      // qdo_full also covers the statistics copied by the loader
      if (!mbar_wait(&qdo_full[ls], (i / NS) & 1, abort_flag, p.err) || !mbar_wait(&sdp_full[s], par, abort_flag, p.err)) {
        ok = false; break;
      }
      tc_fence_after();
      const bool need_mask = q0 + 64 > p.Sq || kv >= p.Sk || (p.causal && kv > p.q_offset + q0) || p.window >= 0;
      const uint32_t t_st = tmem_base + C::COL_ST + 64 * s + lane_sel;
      const uint32_t t_dp = tmem_base + C::COL_DPT + 64 * s + lane_sel;
      const uint32_t t_p = tmem_base + C::COL_PT + C::P_STRIDE * s + lane_sel;
      const uint32_t t_ds = tmem_base + C::COL_DST + C::P_STRIDE * s + lane_sel;
#pragma unroll
      for (int c = 0; c < 2; ++c) {
        uint32_t sv[32], dp[32];
        tmem_ld_32x32b_x32(t_st + c * 32, sv);
        tmem_ld_32x32b_x32(t_dp + c * 32, dp);
        tmem_ld_wait();
        if (C::SEP && c == 1) {
          // scores fully read: the score issuer may refill this buffer; before writing P^T / dS^T
          // the accumulate products of iteration i - 2 (which read them) must have completed
          tc_fence_before();
          mbar_arrive(&sdp_free[s]);
        }
        // two queries per instruction: x = s * scale - lse2, p = 2^x, ds = p * (dp - delta)
        float pr[32], ds[32];
        const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);
#pragma unroll
        for (int k4 = 0; k4 < 8; ++k4) {
          const float4 l4 = st4[c * 8 + k4];          // -lse2 of 4 queries (broadcast read)
          const float4 d4 = st4[16 + c * 8 + k4];     // -delta of the same queries
#pragma unroll
          for (int h2 = 0; h2 < 2; ++h2) {
            const int k = 4 * k4 + 2 * h2;
            const uint64_t nl = h2 == 0 ? f2_pack(l4.x, l4.y) : f2_pack(l4.z, l4.w);
            const uint64_t nd = h2 == 0 ? f2_pack(d4.x, d4.y) : f2_pack(d4.z, d4.w);
            float x0, x1;
            f2_unpack(f2_fma(f2_pack_u(sv[k], sv[k + 1]), scale2, nl), x0, x1);
            pr[k] = fast_exp2(x0);
            pr[k + 1] = fast_exp2(x1);
            f2_unpack(f2_mul(f2_pack(pr[k], pr[k + 1]), f2_add(f2_pack_u(dp[k], dp[k + 1]), nd)), ds[k], ds[k + 1]);
          }
        }
        if (need_mask) {
          // branch-free: this key may be seen by queries [lo, hi] (in units of this chunk's columns)
          int lo = 0, hi = p.Sq - 1;
          if (p.causal) lo = max(lo, kv - p.q_offset);
          if (p.window >= 0) { lo = max(lo, kv - p.q_offset - p.window); hi = min(hi, kv - p.q_offset + p.window); }
          if (kv >= p.Sk) hi = -1;
          lo -= q0 + c * 32;
          hi -= q0 + c * 32;
#pragma unroll
          for (int k = 0; k < 32; ++k) {
            const bool keep = k >= lo && k <= hi;
            pr[k] = keep ? pr[k] : 0.f;
            ds[k] = keep ? ds[k] : 0.f;
          }
        }
        // queries [32c, 32c+32) become packed columns [16c, 16c+16); in the in-place layout these
        // only cover score columns this thread has already read
        if (C::SEP && c == 0 && i >= 2) {
          if (!mbar_wait(&done[(i - 2) % NS], ((i - 2) / NS) & 1, abort_flag, p.err)) { ok = false; }
          tc_fence_after();
        }
        uint32_t pk[16], dk_[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          pk[j] = pack_bf16(pr[2 * j], pr[2 * j + 1]);
          dk_[j] = pack_bf16(ds[2 * j], ds[2 * j + 1]);
        }
        tmem_st_32x32b_x16(t_p + c * 16, pk);
        tmem_st_32x32b_x16(t_ds + c * 16, dk_);
      }
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&pds_full[s]);
    }
    // epilogue: group 0 stores dV, group 1 stores dK (scaled); staging reuses the K / V tiles
    // (every product that read them has completed once acc_full fires)
    uint8_t* stage = smem + (grp == 0 ? C::OFF_K : C::OFF_V);
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
    const long threads = (long)B * sq_pad * Hq * (D / 8);
    const int blocks = (int)((threads + 255) / 256);
    attention_delta_kernel<D><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)o, (const __nv_bfloat16*)dout, lse, delta,
                                                      lse2, B, Sq, sq_pad, Hq, os[0], os[1], os[2], dos[0], dos[1],
                                                      dos[2]);
  }
  static bool f1[64] = {false}, f2[64] = {false};
  auto kq = attention_dq_kernel<D>;
  auto kkv = attention_dkv_kernel<D>;
  if ((rc = set_smem(kq, AttDq<D>::SMEM_BYTES, f1))) return rc;
  if ((rc = set_smem(kkv, AttDkv<D>::SMEM_BYTES, f2))) return rc;
  kkv<<<dim3(Hkv, B, (Sk + 127) / 128), ATTB_DKV_THREADS, AttDkv<D>::SMEM_BYTES, st>>>(tmQ64, tmK, tmV, tmDO64, tmDK, tmDV, p);
  kq<<<dim3(Hq, B, (Sq + 127) / 128), ATTB_DKV_THREADS, AttDq<D>::SMEM_BYTES, st>>>(tmQ, tmK64, tmV64, tmDO, tmDQ, p);
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
  SB_CHECK_ARG(B <= 65535 && Sq / 128 < 65535 && Sk / 128 < 65535);   // grid y / z limits
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
  float* delta = nullptr;
  unsigned int* err = nullptr;
  cudaError_t status = cudaSuccess;
  std::once_flag once;
};
StaticPtrs g_static_ptrs[64];

// Device addresses of the built-in arrays for `dev` (which must be current). The look-up runs
// once per device; std::call_once orders it against every other host thread.
StaticPtrs* static_ptrs(int dev) {
  StaticPtrs& sp = g_static_ptrs[dev];
  std::call_once(sp.once, [&sp] {
    // The array names are host-side handles; the kernels need the device addresses behind them.
    void* pd = nullptr;
    void* pe = nullptr;
    cudaError_t e = cudaGetSymbolAddress(&pd, g_static_delta);
    if (e == cudaSuccess) e = cudaGetSymbolAddress(&pe, g_static_err_word);
    sp.delta = static_cast<float*>(pd);
    sp.err = static_cast<unsigned int*>(pe);
    sp.status = e;
  });
  return sp.status == cudaSuccess ? &sp : nullptr;
}
}  // namespace

extern "C" int sb_attention_bwd_noalloc(const void* q, const void* k, const void* v, const void* o, const void* dout,
                                        const float* lse, void* dq, void* dk, void* dv, int B, int Hq, int Hkv, int Sq,
                                        int Sk, int D, const long* qs, const long* ks, const long* vs, const long* os,
                                        const long* dos, const long* dqs, const long* dks, const long* dvs, int causal,
                                        int window, int q_offset, float scale, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(D == 64 || D == 128);
  SB_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && Sk > 0);
  SB_CHECK_ARG(B <= 65535 && Sq / 128 < 65535 && Sk / 128 < 65535);   // grid y / z limits
  // two arrays of batch * heads * roundup(queries, 64) floats; checked factor by factor so that no
  // product can wrap around before it is compared with the capacity
  const long sq_pad = ((long)Sq + 63) / 64 * 64;
  const long per_array = kStaticDeltaFloats / 2;
  const bool fits = sq_pad <= per_array && (long)Hq <= per_array / sq_pad && (long)B <= per_array / (sq_pad * Hq);
  if (!fits) {
    fprintf(stderr,
            "summa_b200: sb_attention_bwd_noalloc: batch (%d) * heads (%d) * roundup(queries, 64) (%ld) exceeds the "
            "built-in scratch of %ld values per array; use sb_attention_bwd with caller-provided scratch\n",
            B, Hq, sq_pad, per_array);
    return SB_ERR_TOO_LARGE;
  }
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64);
  StaticPtrs* spp = static_ptrs(dev);
  if (!spp) {
    fprintf(stderr, "summa_b200: sb_attention_bwd_noalloc: cudaGetSymbolAddress failed on device %d\n", dev);
    return SB_ERR_CUDA;
  }
  StaticPtrs& sp = *spp;
  if (D == 64)
    return launch_att_bwd<64>(q, k, v, o, dout, lse, sp.delta, dq, dk, dv, B, Hq, Hkv, Sq, Sk, qs, ks, vs, os, dos, dqs,
                              dks, dvs, causal, window, q_offset, scale, st, sp.err);
  return launch_att_bwd<128>(q, k, v, o, dout, lse, sp.delta, dq, dk, dv, B, Hq, Hkv, Sq, Sk, qs, ks, vs, os, dos, dqs,
                             dks, dvs, causal, window, q_offset, scale, st, sp.err);
}

// Reads and clears the status word of the allocation-free path on the current device (same bits as
// sb_read_error_flag: 1 = an mbarrier wait timed out, so dq / dk / dv of that call are not valid).
// Synchronises the device; allocates nothing (the word is a static device word, copied through the
// address cached by the first sb_attention_bwd_noalloc call, or looked up here).
extern "C" int sb_attention_bwd_noalloc_status(unsigned int* out) {
  using namespace sb;
  SB_CHECK_ARG(out != nullptr);
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64);
  StaticPtrs* sp = static_ptrs(dev);
  if (!sp) return SB_ERR_CUDA;
  unsigned int v = 0;
  SB_CHECK_CUDA(cudaDeviceSynchronize());
  SB_CHECK_CUDA(cudaMemcpy(&v, sp->err, sizeof(v), cudaMemcpyDeviceToHost));
  if (v != 0) SB_CHECK_CUDA(cudaMemset(sp->err, 0, sizeof(v)));
  *out = v;
  return SB_OK;
}
