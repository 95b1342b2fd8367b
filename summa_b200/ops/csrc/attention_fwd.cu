// Flash-style attention forward on tcgen05/TMEM (causal, sliding window, native GQA,
// head_dim 64 or 128), emitting O (bf16) and the log-sum-exp (fp32).
//
// One CTA handles 256 query rows of one (batch, head) as two 128-row tiles that
// ping-pong on the tensor core:
//   warps 0-3 / 4-7  softmax group for tile 0 / 1: thread t owns query row t, reads its
//                    score row from TMEM (tcgen05.ld), does the online softmax in
//                    registers and writes P (bf16) into swizzled shared memory; the fp32
//                    output accumulates in TMEM and is rescaled lazily (only when the row
//                    maximum grows by more than 2^8)
//   warp 8           TMA loader: Q once, then K_j / V_j per 128-key block (4-D tensor maps
//                    straight over the packed qkv activation or the KV cache; rows past
//                    the sequence end are zero-filled by TMA and masked)
//   warp 9           MMA issuer: S_a = Q_a K_j^T and Opart_a = P_a V_j into TMEM; issues
//                    S_a(j+1) right after PV_a(j) so one tile's softmax overlaps the other
//                    tile's matrix work
// TMEM: S0,S1 (128 fp32 columns each) + O0,O1 accumulators (D columns each).
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int ATT_THREADS = 320;

template <int D>
struct AttFwd {
  static constexpr int TILE_BYTES = 128 * D * 2;                 // one 128-row Q/K/V tile
  static constexpr int P_BYTES = 128 * 128 * 2;                  // one P tile
  static constexpr int OFF_Q = 0;                                // two tiles
  static constexpr int NSK = 2;                                  // K load stages
  static constexpr int NSV = (D == 64) ? 2 : 1;                  // V load stages (what fits beside Q and P)
  static constexpr int OFF_K = 2 * TILE_BYTES;
  static constexpr int OFF_V = OFF_K + NSK * TILE_BYTES;
  static constexpr int OFF_P = OFF_V + NSV * TILE_BYTES;         // two tiles
  static constexpr int OFF_BAR = OFF_P + 2 * P_BYTES;
  static constexpr int SMEM_BYTES = OFF_BAR + 256 + 1024;
  static constexpr int TMEM_COLS = 512;
  static constexpr int COL_S = 0;                                // S_a at COL_S + a*128
  static constexpr int COL_O = 256;                              // Opart_a at COL_O + a*D
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
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + C::OFF_BAR);
  constexpr int NSK = C::NSK, NSV = C::NSV;
  uint64_t* q_full = bars + 0;
  uint64_t* s_full = bars + 1;    // [2]
  uint64_t* p_full = bars + 3;    // [2], 128 arrivals
  uint64_t* o_full = bars + 5;    // [2]
  uint64_t* k_full = bars + 7;    // [2]
  uint64_t* k_empty = bars + 9;   // [2]
  uint64_t* v_full = bars + 11;   // [2]
  uint64_t* v_empty = bars + 13;  // [2]
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 15);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int qblk = gridDim.x - 1 - blockIdx.x;      // heavy (late) causal blocks first
  const int head = blockIdx.y, b = blockIdx.z;
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
      mbar_init(&s_full[a], 1); mbar_init(&p_full[a], 128); mbar_init(&o_full[a], 1);
      mbar_init(&k_full[a], 1); mbar_init(&k_empty[a], 1); mbar_init(&v_full[a], 1); mbar_init(&v_empty[a], 1);
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
    // ---------------------------------------------------------------- MMA issuer
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, 128, 0, 0);   // S = Q K^T, both K-major
      constexpr uint32_t idesc_o = make_idesc_bf16(128, D, 0, 1);     // O = P V, V is N-major
      const uint32_t q_base = smem_u32(smem + C::OFF_Q), k_base = smem_u32(smem + C::OFF_K);
      const uint32_t v_base = smem_u32(smem + C::OFF_V), p_base = smem_u32(smem + C::OFF_P);
      auto issue_s = [&](int a, int ks) {
#pragma unroll
        for (int kk = 0; kk < D / 16; ++kk) {
          const uint32_t off = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + C::COL_S + a * 128, make_smem_desc_sw128(q_base + a * C::TILE_BYTES + off, 16, 1024),
                    make_smem_desc_sw128(k_base + ks * C::TILE_BYTES + off, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[a]);
      };
      auto issue_pv = [&](int a, int vs, bool first_block) {
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {   // 128 keys, 16 per instruction; O accumulates in TMEM over blocks
          const uint32_t poff = (kk >> 2) * 16384 + (kk & 3) * 32;
          umma_bf16(tmem_base + C::COL_O + a * D, make_smem_desc_sw128(p_base + a * C::P_BYTES + poff, 16, 1024),
                    make_smem_desc_sw128(v_base + vs * C::TILE_BYTES + kk * 2048, 16384, 1024), idesc_o,
                    (!first_block || kk > 0) ? 1u : 0u);
        }
        umma_commit(&o_full[a]);
      };
      bool ok = mbar_wait(q_full, 0, abort_flag, p.err) && mbar_wait(&k_full[0], 0, abort_flag, p.err);
      if (ok) {
        tc_fence_after();
        issue_s(0, 0);
        issue_s(1, 0);
        umma_commit(&k_empty[0]);
      }
      for (int i = 0; i < nblk && ok; ++i) {
        const int vs = i % NSV, ks1 = (i + 1) % NSK;
        if (!mbar_wait(&v_full[vs], (i / NSV) & 1, abort_flag, p.err)) { ok = false; break; }
        const bool more = i + 1 < nblk;
        if (more && !mbar_wait(&k_full[ks1], ((i + 1) / NSK) & 1, abort_flag, p.err)) { ok = false; break; }
        for (int a = 0; a < 2; ++a) {
          if (!mbar_wait(&p_full[a], i & 1, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          issue_pv(a, vs, i == 0);
          if (a == 1) umma_commit(&v_empty[vs]);
          if (more) {
            issue_s(a, ks1);
            if (a == 1) umma_commit(&k_empty[ks1]);
          }
        }
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
    uint8_t* p_tile = smem + C::OFF_P + a * C::P_BYTES;

    // The output accumulates in TMEM across key blocks. `m_ref` is the maximum the
    // probabilities are currently expressed against; it is only advanced (and the TMEM
    // accumulator rescaled) when the running maximum has grown by more than 2^8, so in the
    // steady state a block costs one TMEM read of the scores and no touch of O.
    float m_ref = -INFINITY, l = 0.f;
    bool ok = true;

    for (int i = 0; i < nblk && ok; ++i) {
      const int kv0 = (j_begin + i) * 128;
      if (!mbar_wait(&s_full[a], i & 1, abort_flag, p.err)) { ok = false; break; }
      // P(i-1) has been consumed once PV(i-1) is complete; S(i) was issued after it
      if (i > 0 && !mbar_wait(&o_full[a], (i - 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      uint32_t v[128];
      tmem_ld_32x32b_x32(t_s, v);
      tmem_ld_32x32b_x32(t_s + 32, v + 32);
      tmem_ld_32x32b_x32(t_s + 64, v + 64);
      tmem_ld_32x32b_x32(t_s + 96, v + 96);
      tmem_ld_wait();
      bool mask = kv0 + 128 > p.Sk;
      if (p.causal) mask |= kv0 + 127 > pos;
      if (p.window >= 0) mask |= (pos - kv0 > p.window) || (kv0 + 127 - pos > p.window);
      if (mask) {
#pragma unroll
        for (int k = 0; k < 128; ++k) {
          const int kv = kv0 + k;
          bool bl = kv >= p.Sk;
          if (p.causal) bl |= kv > pos;
          if (p.window >= 0) bl |= (pos - kv > p.window) || (kv - pos > p.window);
          if (bl) v[k] = 0xff800000u;               // -inf
        }
      }
      float mx = -INFINITY;
#pragma unroll
      for (int k = 0; k < 128; ++k) mx = fmaxf(mx, __uint_as_float(v[k]));
      const float m_blk = mx * p.scale_log2;
      const bool grow = m_blk > m_ref + 8.f;        // also true for the first finite block (m_ref = -inf)
      if (__any_sync(0xffffffffu, grow)) {
        const float m_new = grow ? m_blk : m_ref;
        const float alpha = (m_ref == -INFINITY) ? 0.f : exp2f(m_ref - m_new);
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
          tmem_st_wait();
        }
        if (grow) { l *= alpha; m_ref = m_new; }
      }
      const float m_eff = (m_ref == -INFINITY) ? 0.f : m_ref;
      float lsum = 0.f;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        uint8_t* dst = p_tile + (c >> 1) * 16384 + t * 128;
#pragma unroll
        for (int g = 0; g < 4; ++g) {
          float e[8];
#pragma unroll
          for (int k = 0; k < 8; ++k) {
            e[k] = exp2f(fmaf(__uint_as_float(v[c * 32 + g * 8 + k]), p.scale_log2, -m_eff));
            lsum += e[k];
          }
          uint4 w;
          w.x = pack_bf16(e[0], e[1]); w.y = pack_bf16(e[2], e[3]); w.z = pack_bf16(e[4], e[5]); w.w = pack_bf16(e[6], e[7]);
          const int j16 = (c & 1) * 4 + g;
          *reinterpret_cast<uint4*>(dst + ((j16 ^ (t & 7)) << 4)) = w;
        }
      }
      l += lsum;
      tc_fence_before();
      fence_proxy_async_smem();
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
      uint8_t* dst = p_tile + (c >> 1) * 16384 + t * 128;
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
        tma_store_4d(&tmO, p_tile + h * 16384 + (warp & 3) * 4096, h * 64, head, row0, b);
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
  dim3 grid((Sq + 255) / 256, Hq, B);
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
  if (D == 64)
    return launch_att_fwd<64>(q, k, v, o, lse, B, Hq, Hkv, Sq, Sk, q_strides, k_strides, v_strides, o_strides, causal,
                              window, q_offset, scale, st);
  return launch_att_fwd<128>(q, k, v, o, lse, B, Hq, Hkv, Sq, Sk, q_strides, k_strides, v_strides, o_strides, causal,
                             window, q_offset, scale, st);
}
