// Flash-style attention forward on tcgen05/TMEM (causal, sliding window, native GQA,
// head_dim 64 or 128), emitting O (bf16) and the log-sum-exp (fp32).
//
// One CTA handles 256 query rows of one (batch, head) as two 128-row tiles that
// ping-pong on the tensor core:
//   warps 0-3 / 4-7  softmax group for tile 0 / 1: thread t owns query row t, reads its
//                    score row from TMEM (tcgen05.ld), does the online softmax in registers
//                    (packed f32x2 arithmetic) and writes P as packed bf16 back into TMEM,
//                    where it is the A operand of the P V product; the fp32 output accumulates
//                    in TMEM and is rescaled lazily (only when the row maximum grows by more
//                    than 2^8)
//   warp 8           TMA loader: Q once, then K_j / V_j per 128-key block through multi-stage
//                    rings (4-D tensor maps straight over the packed qkv activation or the KV
//                    cache; rows past the sequence end are zero-filled by TMA and masked)
//   warp 9           issues S_a = Q_a K_j^T
//   warp 10          issues O_a += P_a V_j
// Two issuing warps because a commit stalls its issuing thread for ~190 cycles while
// products issued by another warp keep the tensor pipe busy.
// TMEM: S0,S1 (128 fp32 columns each), O0,O1 (D columns each) and, for head_dim 64, separate
// P0,P1 (64 columns each) so that S_a(j+1) can be computed while the threads still work on
// block j; with head_dim 128 TMEM is full and P overwrites S in place.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int ATT_THREADS = 352;
#ifndef ATT_POLY_EVERY
#define ATT_POLY_EVERY 4      // 1 of 4 score pairs: measured best split between the XU and the FMA pipe
#endif

template <int D>
struct AttFwd {
  static constexpr bool SEP = (D == 64);                         // separate TMEM columns for P
  static constexpr int TILE_BYTES = 128 * D * 2;                 // one 128-row Q/K/V tile
  static constexpr int NSK = (D == 64) ? 3 : 2;                  // K load stages
  static constexpr int NSV = (D == 64) ? 3 : 2;                  // V load stages
  static constexpr int OFF_Q = 0;                                // two tiles (reused to stage O)
  static constexpr int OFF_K = 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NSK * TILE_BYTES;
  static constexpr int OFF_BAR = OFF_V + NSV * TILE_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S = 0;                                // S_a at COL_S + a*128
  static constexpr int COL_O = 256;                              // O_a at COL_O + a*D
  static constexpr int COL_P = SEP ? 384 : COL_S;                // P_a at COL_P + a*P_STRIDE (64 packed columns)
  static constexpr int P_STRIDE = SEP ? 64 : 128;
};

struct AttFwdParams {
  int B, Hq, Hkv, Sq, Sk;
  int causal, window, q_offset;    // window < 0: none
  float scale_log2;                // softmax scale * log2(e)
  float* lse;                      // [B, Hq, Sq] natural-log LSE (may be null)
  unsigned int* err;
};

template <int D>
__global__ void __launch_bounds__(ATT_THREADS, 1)
attention_fwd_kernel(const __grid_constant__ CUtensorMap tmQ, const __grid_constant__ CUtensorMap tmK,
                     const __grid_constant__ CUtensorMap tmV, const __grid_constant__ CUtensorMap tmO,
                     const AttFwdParams p) {
  using C = AttFwd<D>;
  constexpr int NSK = C::NSK, NSV = C::NSV;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  uint64_t* q_full = bars + 0;
  uint64_t* s_full = bars + 1;    // [2]
  uint64_t* s_free = bars + 3;    // [2], 128 arrivals: the group has read S_a (SEP only)
  uint64_t* p_full = bars + 5;    // [2], 128 arrivals
  uint64_t* o_full = bars + 7;    // [2] P_a V product of a block completed
  uint64_t* k_full = bars + 9;    // [NSK]
  uint64_t* k_empty = bars + 12;  // [NSK]
  uint64_t* v_full = bars + 15;   // [NSV]
  uint64_t* v_empty = bars + 18;  // [NSV]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 21);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  // grid (heads, batch, query blocks), handed out x-fastest: every heavy (late, under a causal
  // mask) query block starts before any light one, so the tail of the launch is short
  const int qblk = gridDim.z - 1 - blockIdx.z;
  const int head = blockIdx.x, b = blockIdx.y;
  const int kv_head = head / (p.Hq / p.Hkv);
  const int q0 = qblk * 256;

  // key-block range for this CTA
  int j_begin = 0, j_end = (p.Sk + 127) / 128;
  if (p.causal) j_end = min(j_end, (p.q_offset + q0 + 255) / 128 + 1);
  if (p.window >= 0) {
    j_begin = max(0, (p.q_offset + q0 - p.window) / 128);
    if (!p.causal) j_end = min(j_end, (p.q_offset + q0 + 255 + p.window) / 128 + 1);
  }
  const int nblk = max(0, j_end - j_begin);

  if (threadIdx.x == 0) {
    mbar_init(q_full, 1);
    for (int a = 0; a < 2; ++a) {
      mbar_init(&s_full[a], 1); mbar_init(&s_free[a], 128); mbar_init(&p_full[a], 128); mbar_init(&o_full[a], 1);
    }
    for (int s = 0; s < 3; ++s) {
      mbar_init(&k_full[s], 1); mbar_init(&k_empty[s], 1); mbar_init(&v_full[s], 1); mbar_init(&v_empty[s], 1);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmQ); tma_prefetch_desc(&tmK); tma_prefetch_desc(&tmV); tma_prefetch_desc(&tmO);
  }
  if (warp == 9) { tmem_alloc(tmem_slot, C::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;

  if (warp == 8) {
    // ---------------------------------------------------------------- TMA loader
    if (lane == 0 && nblk > 0) {
      mbar_expect_tx(q_full, 2 * C::TILE_BYTES);
#pragma unroll
      for (int a = 0; a < 2; ++a)
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(smem + C::OFF_Q + a * C::TILE_BYTES + h * 16384, &tmQ, q_full, h * 64, head, q0 + a * 128, b);
      for (int i = 0; i < nblk; ++i) {
        const int kv0 = (j_begin + i) * 128;
        const int ks = i % NSK, vs = i % NSV;
        if (!mbar_wait(&k_empty[ks], ((i / NSK) & 1) ^ 1, abort_flag, p.err)) break;
        mbar_expect_tx(&k_full[ks], C::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(smem + C::OFF_K + ks * C::TILE_BYTES + h * 16384, &tmK, &k_full[ks], h * 64, kv_head, kv0, b);
        if (!mbar_wait(&v_empty[vs], ((i / NSV) & 1) ^ 1, abort_flag, p.err)) break;
        mbar_expect_tx(&v_full[vs], C::TILE_BYTES);
#pragma unroll
        for (int h = 0; h < D / 64; ++h)
          tma_load_4d(smem + C::OFF_V + vs * C::TILE_BYTES + h * 16384, &tmV, &v_full[vs], h * 64, kv_head, kv0, b);
      }
      if (*abort_flag) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) {} }
    }
    __syncwarp();
  } else if (warp == 9) {
    // ---------------------------------------------------------------- S issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S = Q K^T, both K-major
      const uint32_t q_base = smem_u32(smem + C::OFF_Q), k_base = smem_u32(smem + C::OFF_K);
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err);
      for (int i = 0; i < nblk && ok; ++i) {
        const int ks = i % NSK;
        if (!mbar_wait(&k_full[ks], (i / NSK) & 1, abort_flag, p.err)) { ok = false; break; }
        for (int a = 0; a < 2 && ok; ++a) {
          if (i > 0) {
            // S_a may be overwritten once the group has read block i-1 (SEP) or once the
            // product that read P_a(i-1) from the same columns has completed (in place)
            ok = C::SEP ? mbar_wait(&s_free[a], (i - 1) & 1, abort_flag, p.err)
                        : mbar_wait(&o_full[a], (i - 1) & 1, abort_flag, p.err);
            if (!ok) break;
          }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < D / 16; ++kk) {
            const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
            umma_bf16(tmem_base + C::COL_S + a * 128, make_smem_desc_sw128(q_base + a * C::TILE_BYTES + off, 16, 1024),
                      make_smem_desc_sw128(k_base + ks * C::TILE_BYTES + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
          }
          umma_commit(&s_full[a]);
        }
        if (ok) umma_commit(&k_empty[ks]);
      }
    }
    __syncwarp();
  } else if (warp == 10) {
    // ---------------------------------------------------------------- P V issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);     // O += P V, P in TMEM, V N-major
      const uint32_t v_base = smem_u32(smem + C::OFF_V);
      bool ok = true;
      for (int i = 0; i < nblk && ok; ++i) {
        const int vs = i % NSV;
        if (!mbar_wait(&v_full[vs], (i / NSV) & 1, abort_flag, p.err)) { ok = false; break; }
        for (int a = 0; a < 2 && ok; ++a) {
          if (!mbar_wait(&p_full[a], i & 1, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
#pragma unroll
          for (int kk = 0; kk < 8; ++kk) {   // 128 keys, 16 per instruction; O accumulates in TMEM over blocks
            umma_bf16_ta(tmem_base + C::COL_O + a * D, tmem_base + C::COL_P + a * C::P_STRIDE + 8 * kk,
                         make_smem_desc_sw128(v_base + vs * C::TILE_BYTES + kk * 2048, 16384, 1024), idesc_o,
                         (i > 0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&o_full[a]);
        }
        if (ok) umma_commit(&v_empty[vs]);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax groups
    const int a = warp >> 2;                       // tile index
    const int t = threadIdx.x & 127;               // row in tile == TMEM lane
    const int row = q0 + a * 128 + t;
    const int pos = p.q_offset + row;
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const uint32_t t_s = tmem_base + C::COL_S + a * 128 + lane_sel;
    const uint32_t t_o = tmem_base + C::COL_O + a * D + lane_sel;
    const uint32_t t_p = tmem_base + C::COL_P + a * C::P_STRIDE + lane_sel;
    uint8_t* o_tile = smem + C::OFF_Q + a * C::TILE_BYTES;     // Q_a is dead by the time O is staged

    // The output accumulates in TMEM across key blocks. `m_ref` is the maximum the
    // probabilities are currently expressed against; it is only advanced (and the TMEM
    // accumulator rescaled) when the running maximum has grown by more than 2^8, so in the
    // steady state a block costs one TMEM read of the scores and no touch of O.
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;
    const uint64_t scale2 = f2_pack(p.scale_log2, p.scale_log2);

    for (int i = 0; i < nblk && ok; ++i) {
      const int kv0 = (j_begin + i) * 128;
      if (!mbar_wait(&s_full[a], i & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[128];
      tmem_ld_32x32b_x32(t_s, v);
      tmem_ld_32x32b_x32(t_s + 32, v + 32);
      tmem_ld_32x32b_x32(t_s + 64, v + 64);
      tmem_ld_32x32b_x32(t_s + 96, v + 96);
      tmem_ld_wait();
      if (C::SEP) {
        tc_fence_before();
        mbar_arrive(&s_free[a]);                    // the S issuer may start on block i+1
      }
      bool mask = kv0 + 128 > p.Sk;
      if (p.causal) mask |= kv0 + 127 > pos;
      if (p.window >= 0) mask |= (pos - kv0 > p.window) || (kv0 + 127 - pos > p.window);
      if (mask) {
        // branch-free: this row may see keys [lo, hi] (in units of this block's columns)
        int lo = 0, hi = p.Sk - 1;
        if (p.causal) hi = min(hi, pos);
        if (p.window >= 0) { lo = max(lo, pos - p.window); hi = min(hi, pos + p.window); }
        lo -= kv0;
        hi -= kv0;
#pragma unroll
        for (int k = 0; k < 128; ++k) v[k] = (k >= lo && k <= hi) ? v[k] : 0xff800000u;   // -inf
      }
      float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
      for (int k = 0; k < 128; k += 4) {
        mx0 = fmaxf(mx0, fmaxf(__uint_as_float(v[k]), __uint_as_float(v[k + 1])));
        mx1 = fmaxf(mx1, fmaxf(__uint_as_float(v[k + 2]), __uint_as_float(v[k + 3])));
      }
      const float m_blk = fmaxf(mx0, mx1) * p.scale_log2;
      const bool grow = m_blk > m_ref + 8.f;        // also true for the first finite block (m_ref = -inf)
      // P_a(i-1) must have been consumed (and O_a be quiescent) before P or O are touched
      if (i > 0 && !mbar_wait(&o_full[a], (i - 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? m_blk : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : fast_exp2(m_ref - m_new);
        if (i > 0) {
          // rescale this warp's 32 rows of the TMEM accumulator (rows that did not grow use 1)
#pragma unroll
          for (int c = 0; c < D / 16; ++c) {
            uint32_t o16[16];
            tmem_ld_32x32b_x16(t_o + c * 16, o16);
            tmem_ld_wait();
#pragma unroll
            for (int k = 0; k < 16; ++k) o16[k] = __float_as_uint(__uint_as_float(o16[k]) * (grow ? alpha : 1.f));
            tmem_st_32x32b_x16(t_o + c * 16, o16);
          }
        }
        if (grow) { l *= alpha; m_ref = m_new; }
      }
      const float m_eff = (m_ref == -INFINITY) ? 0.f : m_ref;
      const uint64_t nm2 = f2_pack(-m_eff, -m_eff);
      uint64_t sum2 = f2_pack(0.f, 0.f);
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint32_t pk[16];
#pragma unroll
        for (int j = 0; j < 16; ++j) {
          const int k = c * 32 + 2 * j;
          float x0, x1;
          f2_unpack(f2_fma(f2_pack_u(v[k], v[k + 1]), scale2, nm2), x0, x1);
          float e0, e1;
          // every ATT_POLY_EVERY-th pair takes the FMA-pipe exponential (see exp2_poly2)
          if (ATT_POLY_EVERY > 0 && (j % ATT_POLY_EVERY) == ATT_POLY_EVERY - 1) {
            exp2_poly2(x0, x1, e0, e1);
          } else {
            e0 = fast_exp2(x0);
            e1 = fast_exp2(x1);
          }
          sum2 = f2_add(sum2, f2_pack(e0, e1));
          pk[j] = pack_bf16(e0, e1);
        }
        tmem_st_32x32b_x16(t_p + c * 16, pk);
      }
      float s0, s1;
      f2_unpack(sum2, s0, s1);
      l += s0 + s1;
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&p_full[a]);
    }
    // epilogue: O = accumulator / l
    const float inv_l = l > 0.f ? 1.f / l : 0.f;
    if (p.lse != nullptr && row < p.Sq) {
      const float lse = l > 0.f ? (m_ref + log2f(l)) * 0.6931471805599453f : -INFINITY;
      p.lse[(static_cast<size_t>(b) * p.Hq + head) * p.Sq + row] = lse;
    }
    const bool have = ok && nblk > 0 && mbar_wait(&o_full[a], (nblk - 1) & 1, abort_flag, p.err);
    if (have) tc_fence_after();
#pragma unroll
    for (int c = 0; c < D / 32; ++c) {
      uint32_t o32[32];
      if (have) {
        tmem_ld_32x32b_x32(t_o + c * 32, o32);
        tmem_ld_wait();
      } else {
#pragma unroll
        for (int k = 0; k < 32; ++k) o32[k] = 0u;
      }
      uint8_t* dst = o_tile + (c >> 1) * 16384 + t * 128;
#pragma unroll
      for (int g = 0; g < 4; ++g) {
        uint4 w;
        w.x = pack_bf16(__uint_as_float(o32[8 * g + 0]) * inv_l, __uint_as_float(o32[8 * g + 1]) * inv_l);
        w.y = pack_bf16(__uint_as_float(o32[8 * g + 2]) * inv_l, __uint_as_float(o32[8 * g + 3]) * inv_l);
        w.z = pack_bf16(__uint_as_float(o32[8 * g + 4]) * inv_l, __uint_as_float(o32[8 * g + 5]) * inv_l);
        w.w = pack_bf16(__uint_as_float(o32[8 * g + 6]) * inv_l, __uint_as_float(o32[8 * g + 7]) * inv_l);
        const int j16 = (c & 1) * 4 + g;
        *reinterpret_cast<uint4*>(dst + ((j16 ^ (t & 7)) << 4)) = w;
      }
    }
    fence_proxy_async_smem();
    __syncwarp();
    const int row0 = q0 + a * 128 + (warp & 3) * 32;
    if (lane == 0 && row0 < p.Sq) {
#pragma unroll
      for (int h = 0; h < D / 64; ++h)
        tma_store_4d(&tmO, o_tile + h * 16384 + (warp & 3) * 4096, h * 64, head, row0, b);
      tma_store_commit();
      tma_store_wait_all<0>();
    }
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 9) {
    tc_fence_after();
    tmem_dealloc(tmem_base, C::TMEM_COLS);
  }
}

// 4-D map over a `[B, S, H, D]` tensor with element strides (batch, seq, head); inner D contiguous.
static int make_tmap_bshd(CUtensorMap* m, const void* base, int B, int S, int H, int D, long sb_, long ss, long sh,
                          int box_rows) {
  uint64_t dims[4] = {(uint64_t)D, (uint64_t)H, (uint64_t)S, (uint64_t)B};
  uint64_t strides[3] = {(uint64_t)sh * 2, (uint64_t)ss * 2, (uint64_t)sb_ * 2};
  uint32_t box[4] = {64, 1, (uint32_t)box_rows, 1};
  return make_tmap(m, base, 2, 4, dims, strides, box, true);
}

template <int D>
static int launch_att_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq, int Hkv, int Sq,
                          int Sk, const long* qs, const long* ks, const long* vs, const long* os, int causal, int window,
                          int q_offset, float scale, cudaStream_t st) {
  using C = AttFwd<D>;
  CUtensorMap tmQ, tmK, tmV, tmO;
  int rc;
  if ((rc = make_tmap_bshd(&tmQ, q, B, Sq, Hq, D, qs[0], qs[1], qs[2], 128))) return rc;
  if ((rc = make_tmap_bshd(&tmK, k, B, Sk, Hkv, D, ks[0], ks[1], ks[2], 128))) return rc;
  if ((rc = make_tmap_bshd(&tmV, v, B, Sk, Hkv, D, vs[0], vs[1], vs[2], 128))) return rc;
  if ((rc = make_tmap_bshd(&tmO, o, B, Sq, Hq, D, os[0], os[1], os[2], 32))) return rc;
  AttFwdParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sq = Sq; p.Sk = Sk;
  p.causal = causal; p.window = window; p.q_offset = q_offset;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.lse = lse;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  auto kern = attention_fwd_kernel<D>;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, C::SMEM_BYTES));
    attr_set[dev & 63] = true;
  }
  dim3 grid(Hq, B, (Sq + 255) / 256);
  kern<<<grid, ATT_THREADS, C::SMEM_BYTES, st>>>(tmQ, tmK, tmV, tmO, p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

// q `[B,Sq,Hq,D]`, k/v `[B,Sk,Hkv,D]`, o `[B,Sq,Hq,D]` bf16 with element strides
// {batch, seq, head} each (inner D contiguous); lse `[B,Hq,Sq]` fp32 or null.
// window < 0 disables the sliding window; q_offset is the absolute position of query 0.
extern "C" int sb_attention_fwd(const void* q, const void* k, const void* v, void* o, float* lse, int B, int Hq, int Hkv,
                                int Sq, int Sk, int D, const long* q_strides, const long* k_strides,
                                const long* v_strides, const long* o_strides, int causal, int window, int q_offset,
                                float scale, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(D == 64 || D == 128);
  SB_CHECK_ARG(B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Sq > 0 && Sk > 0);
  SB_CHECK_ARG(B <= 65535 && Sq / 128 < 65535 && Sk / 128 < 65535);   // grid y / z limits
  if (D == 64)
    return launch_att_fwd<64>(q, k, v, o, lse, B, Hq, Hkv, Sq, Sk, q_strides, k_strides, v_strides, o_strides, causal,
                              window, q_offset, scale, st);
  return launch_att_fwd<128>(q, k, v, o, lse, B, Hq, Hkv, Sq, Sk, q_strides, k_strides, v_strides, o_strides, causal,
                             window, q_offset, scale, st);
}
