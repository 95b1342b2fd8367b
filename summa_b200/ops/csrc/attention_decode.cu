// Decode attention (one new token per sequence) over a bf16 KV cache, head_dim 128, split
// over the keys ("flash decoding") and written for tcgen05 so that the cache streams through
// TMA at memory speed while the threads only touch one score per key.
//
// One CTA handles (key split, kv head, batch) and the G = Hq / Hkv query heads that share the
// kv head (grouped-query packing: the cache is read once for all of them). Per 128-key block:
//   S^T[128 keys x 8]  = K_blk[128 x 128] * Q^T            (A = K tile, B = 8 padded query rows)
//   threads (lane = key): scale, mask, block max per head (shuffles + one smem exchange),
//                         p = 2^(s - m), write P (bf16) into an 8 x 128 swizzled smem tile
//   O^T[128 d x 8]    += V_blk^T[128 d x 128 keys] * P^T   (A = V tile read MN-major, B = P)
// O^T accumulates in tensor memory and is rescaled lazily (only when a head's maximum grows by
// more than 2^8). Each split writes an unnormalised partial (O, m, l); a second kernel merges
// the splits. Roles: warps 0-3 softmax, warp 4 TMA loader (3-stage K/V ring), warp 5 MMA issuer.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

__device__ __forceinline__ void tmem_ld_32x32b_x8(uint32_t taddr, uint32_t* r) {
  asm volatile("tcgen05.ld.sync.aligned.32x32b.x8.b32 {%0, %1, %2, %3, %4, %5, %6, %7}, [%8];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7])
               : "r"(taddr)
               : "memory");
}

constexpr int DEC_D = 128;
constexpr int DEC_N = 8;                           // padded query heads per kv head
constexpr int DEC_THREADS = 192;
constexpr int DEC_TILE = 128 * DEC_D * 2;          // 32 KB
constexpr int DEC_NS = 3;
constexpr int DEC_OFF_K = 0;
constexpr int DEC_OFF_V = DEC_NS * DEC_TILE;
constexpr int DEC_OFF_Q = 2 * DEC_NS * DEC_TILE;   // 8 rows x 256 B (two swizzle atoms)
constexpr int DEC_OFF_P = DEC_OFF_Q + 2048;        // 2 buffers x 2 KB
constexpr int DEC_OFF_RED = DEC_OFF_P + 4096;      // [2][4 warps][8] floats
constexpr int DEC_OFF_BAR = DEC_OFF_RED + 256;
constexpr int DEC_SMEM = DEC_OFF_BAR + 256 + 1024;

struct DecParams {
  int B, Hq, Hkv, Sk, splits, blocks_per_split;
  const int* sk_ptr;          // when set, the live length is *sk_ptr + sk_add (graph-capturable decode)
  int sk_add;
  float scale_log2;
  const __nv_bfloat16* q;     // [B, Hq, D] (token stride folded into q_sb)
  long q_sb, q_sh;
  float* part_o;              // [B, Hkv, splits, 8, D]
  float* part_m;              // [B, Hkv, splits, 8]  (log2 domain)
  float* part_l;              // [B, Hkv, splits, 8]
  unsigned int* err;
};

__global__ void __launch_bounds__(DEC_THREADS, 1)
attention_decode_kernel(const __grid_constant__ CUtensorMap tmK, const __grid_constant__ CUtensorMap tmV, const DecParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + DEC_OFF_BAR);
  uint64_t* kv_full = bars + 0;    // [3]
  uint64_t* kv_empty = bars + 3;   // [3]
  uint64_t* s_full = bars + 6;     // [2]
  uint64_t* p_full = bars + 8;     // [2] 128 arrivals
  uint64_t* o_done = bars + 10;    // PV product of a block completed
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(bars + 11);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  float* red = reinterpret_cast<float*>(smem + DEC_OFF_RED);

  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int split = blockIdx.x, kv_head = blockIdx.y, b = blockIdx.z;
  const int G = p.Hq / p.Hkv;
  const int Sk = p.sk_ptr != nullptr ? min(*p.sk_ptr + p.sk_add, p.Sk) : p.Sk;     // p.Sk bounds it (capacity)
  const int nblocks_total = (Sk + 127) / 128;
  const int blk0 = split * p.blocks_per_split;
  const int nblk = max(0, min(p.blocks_per_split, nblocks_total - blk0));

  if (threadIdx.x == 0) {
    for (int s = 0; s < DEC_NS; ++s) { mbar_init(&kv_full[s], 1); mbar_init(&kv_empty[s], 1); }
    for (int s = 0; s < 2; ++s) { mbar_init(&s_full[s], 1); mbar_init(&p_full[s], 128); }
    mbar_init(o_done, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  // query rows -> swizzled B operand tile (rows >= G are zero)
  for (int i = threadIdx.x; i < DEC_N * 16; i += DEC_THREADS) {
    const int g = i >> 4, j = i & 15;               // row, 16-byte chunk (8 bf16) of the 256-byte row
    uint4 w = make_uint4(0, 0, 0, 0);
    if (g < G) w = *reinterpret_cast<const uint4*>(p.q + b * p.q_sb + (long)(kv_head * G + g) * p.q_sh + j * 8);
    *reinterpret_cast<uint4*>(smem + DEC_OFF_Q + (j >> 3) * 1024 + g * 128 + (((j & 7) ^ (g & 7)) << 4)) = w;
  }
  fence_proxy_async_smem();
  if (warp == 5) { tmem_alloc(tmem_slot, 32); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t COL_O = 0, COL_S = 8;          // S^T buffers at 8, 16

  if (warp == 4) {
    if (lane == 0) {
      for (int i = 0; i < nblk; ++i) {
        const int s = i % DEC_NS;
        const int kv0 = (blk0 + i) * 128;
        if (!mbar_wait(&kv_empty[s], ((i / DEC_NS) & 1) ^ 1, abort_flag, p.err)) break;
        mbar_expect_tx(&kv_full[s], 2 * DEC_TILE);
#pragma unroll
        for (int h = 0; h < 2; ++h) {
          tma_load_4d(smem + DEC_OFF_K + s * DEC_TILE + h * 16384, &tmK, &kv_full[s], h * 64, kv_head, kv0, b);
          tma_load_4d(smem + DEC_OFF_V + s * DEC_TILE + h * 16384, &tmV, &kv_full[s], h * 64, kv_head, kv0, b);
        }
      }
      if (*abort_flag) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) {} }
    }
    __syncwarp();
  } else if (warp == 5) {
    if (lane == 0 && nblk > 0) {
      constexpr uint32_t idesc_s = make_idesc_bf16(128, DEC_N, 0, 0);
      constexpr uint32_t idesc_o = make_idesc_bf16(128, DEC_N, 1, 0);    // A = V tile read MN-major
      const uint32_t k_base = smem_u32(smem + DEC_OFF_K), v_base = smem_u32(smem + DEC_OFF_V);
      const uint32_t q_base = smem_u32(smem + DEC_OFF_Q), p_base = smem_u32(smem + DEC_OFF_P);
      auto issue_s = [&](int i) {
        const int s = i % DEC_NS;
#pragma unroll
        for (int kk = 0; kk < DEC_D / 16; ++kk) {
          umma_bf16(tmem_base + COL_S + 8 * (i & 1),
                    make_smem_desc_sw128(k_base + s * DEC_TILE + (kk >> 2) * 16384 + (kk & 3) * 32, 16, 1024),
                    make_smem_desc_sw128(q_base + (kk >> 2) * 1024 + (kk & 3) * 32, 16, 1024), idesc_s, kk > 0 ? 1u : 0u);
        }
        umma_commit(&s_full[i & 1]);
      };
      bool ok = mbar_wait(&kv_full[0], 0, abort_flag, p.err);
      if (ok) { tc_fence_after(); issue_s(0); }
      for (int i = 0; i < nblk && ok; ++i) {
        if (i + 1 < nblk) {
          // S^T buffer (i+1)&1 was read by the threads in block i-1, before their p_full(i-1)
          if (!mbar_wait(&kv_full[(i + 1) % DEC_NS], ((i + 1) / DEC_NS) & 1, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          issue_s(i + 1);
        }
        if (!mbar_wait(&p_full[i & 1], (i >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const int s = i % DEC_NS;
#pragma unroll
        for (int kk = 0; kk < 8; ++kk) {             // 128 keys, 16 per instruction
          umma_bf16(tmem_base + COL_O, make_smem_desc_sw128(v_base + s * DEC_TILE + kk * 2048, 16384, 1024),
                    make_smem_desc_sw128(p_base + (i & 1) * 2048 + (kk >> 2) * 1024 + (kk & 3) * 32, 16, 1024), idesc_o,
                    (i > 0 || kk > 0) ? 1u : 0u);
        }
        umma_commit(&kv_empty[s]);
        umma_commit(o_done);
      }
    }
    __syncwarp();
  } else {
    // ---------------------------------------------------------------- softmax (thread = key of the block)
    const int t = threadIdx.x;
    const uint32_t lane_sel = static_cast<uint32_t>(warp * 32) << 16;
    float m_run[DEC_N], l_part[DEC_N];
#pragma unroll
    for (int g = 0; g < DEC_N; ++g) { m_run[g] = -INFINITY; l_part[g] = 0.f; }
    bool ok = true;
    for (int i = 0; i < nblk && ok; ++i) {
      const int kv = (blk0 + i) * 128 + t;
      if (!mbar_wait(&s_full[i & 1], (i >> 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      uint32_t sv[8];
      tmem_ld_32x32b_x8(tmem_base + COL_S + 8 * (i & 1) + lane_sel, sv);
      tmem_ld_wait();
      float s[DEC_N], bm[DEC_N];
#pragma unroll
      for (int g = 0; g < DEC_N; ++g) {
        s[g] = (kv < Sk && g < G) ? __uint_as_float(sv[g]) * p.scale_log2 : -INFINITY;
        bm[g] = warp_max(s[g]);
      }
      float* rbuf = red + (i & 1) * 32;
      if (lane == 0) {
#pragma unroll
        for (int g = 0; g < DEC_N; ++g) rbuf[warp * 8 + g] = bm[g];
      }
      asm volatile("bar.sync 1, 128;" ::: "memory");
      bool grow_any = false;
      float alpha[DEC_N];
#pragma unroll
      for (int g = 0; g < DEC_N; ++g) {
        const float mb = fmaxf(fmaxf(rbuf[g], rbuf[8 + g]), fmaxf(rbuf[16 + g], rbuf[24 + g]));
        alpha[g] = 1.f;
        if (mb > m_run[g] + 8.f) {                    // uniform over the CTA (same inputs everywhere)
          alpha[g] = (m_run[g] == -INFINITY) ? 0.f : fast_exp2(m_run[g] - mb);
          m_run[g] = mb;
          grow_any = true;
        }
      }
      // the previous block's P V product must be complete before O is rescaled or P reused
      if (i > 0 && !mbar_wait(o_done, (i - 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      if (grow_any && i > 0) {
        uint32_t o16[8];
        tmem_ld_32x32b_x8(tmem_base + COL_O + lane_sel, o16);                // row d = t, 8 heads
        tmem_ld_wait();
        uint32_t o8[8];
#pragma unroll
        for (int g = 0; g < DEC_N; ++g) o8[g] = __float_as_uint(__uint_as_float(o16[g]) * alpha[g]);
        asm volatile("tcgen05.st.sync.aligned.32x32b.x8.b32 [%0], {%1, %2, %3, %4, %5, %6, %7, %8};"
                     ::"r"(tmem_base + COL_O + lane_sel), "r"(o8[0]), "r"(o8[1]), "r"(o8[2]), "r"(o8[3]), "r"(o8[4]),
                       "r"(o8[5]), "r"(o8[6]), "r"(o8[7]) : "memory");
        tmem_st_wait();
      }
      uint8_t* pt = smem + DEC_OFF_P + (i & 1) * 2048 + (t >> 6) * 1024;
      const int tc = t & 63;
#pragma unroll
      for (int g = 0; g < DEC_N; ++g) {
        l_part[g] *= alpha[g];
        const float e = (s[g] == -INFINITY) ? 0.f : fast_exp2(s[g] - m_run[g]);
        l_part[g] += e;
        *reinterpret_cast<__nv_bfloat16*>(pt + g * 128 + ((((tc >> 3) ^ (g & 7)) << 4) | ((tc & 7) << 1))) = __float2bfloat16(e);
      }
      tc_fence_before();
      fence_proxy_async_smem();
      mbar_arrive(&p_full[i & 1]);
    }
    // partial results of this split
    float l_tot[DEC_N];
#pragma unroll
    for (int g = 0; g < DEC_N; ++g) l_tot[g] = warp_sum(l_part[g]);
    asm volatile("bar.sync 1, 128;" ::: "memory");
    if (lane == 0) {
#pragma unroll
      for (int g = 0; g < DEC_N; ++g) red[warp * 8 + g] = l_tot[g];
    }
    asm volatile("bar.sync 1, 128;" ::: "memory");
    const size_t pbase = ((static_cast<size_t>(b) * p.Hkv + kv_head) * p.splits + split) * DEC_N;
    if (t < DEC_N) {
      p.part_l[pbase + t] = red[t] + red[8 + t] + red[16 + t] + red[24 + t];
      float mr = -INFINITY;
#pragma unroll
      for (int g = 0; g < DEC_N; ++g) if (g == t) mr = m_run[g];
      p.part_m[pbase + t] = mr;
    }
    const bool have = ok && nblk > 0 && mbar_wait(o_done, (nblk - 1) & 1, abort_flag, p.err);
    uint32_t o16[8];
    if (have) {
      tc_fence_after();
      tmem_ld_32x32b_x8(tmem_base + COL_O + lane_sel, o16);
      tmem_ld_wait();
    }
#pragma unroll
    for (int g = 0; g < DEC_N; ++g) p.part_o[(pbase + g) * DEC_D + t] = have ? __uint_as_float(o16[g]) : 0.f;
  }
  tc_fence_before();
  __syncthreads();
  if (warp == 5) { tc_fence_after(); tmem_dealloc(tmem_base, 32); }
}

// merge the splits: one block per (batch, query head), thread = d
__global__ void __launch_bounds__(DEC_D)
attention_decode_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_m,
                              const float* __restrict__ part_l, __nv_bfloat16* __restrict__ o, long o_sb, long o_sh,
                              int Hq, int Hkv, int splits) {
  // a following kernel launched with programmatic stream serialization (the output projection's GEMV)
  // may start its input-independent prologue now; it still waits for this grid before reading `o`
  asm volatile("griddepcontrol.launch_dependents;");
  const int hq = blockIdx.x, b = blockIdx.y, d = threadIdx.x;
  const int G = Hq / Hkv, kvh = hq / G, g = hq % G;
  const size_t base = (static_cast<size_t>(b) * Hkv + kvh) * splits;
  float M = -INFINITY;
  for (int s = 0; s < splits; ++s) M = fmaxf(M, part_m[(base + s) * DEC_N + g]);
  float acc = 0.f, l = 0.f;
  for (int s = 0; s < splits; ++s) {
    const float ms = part_m[(base + s) * DEC_N + g];
    const float w = (ms == -INFINITY) ? 0.f : exp2f(ms - M);
    l += part_l[(base + s) * DEC_N + g] * w;
    acc += part_o[((base + s) * DEC_N + g) * DEC_D + d] * w;
  }
  o[b * o_sb + (long)hq * o_sh + d] = __float2bfloat16(l > 0.f ? acc / l : 0.f);
}

}  // namespace sb

// Decode attention for ONE query token per sequence. q / o: bf16 `[B, Hq, 128]` with element
// strides (batch, head); k / v cache: bf16 `[B, cap, Hkv, 128]` with element strides (batch,
// seq, head); the first Sk cache rows of every sequence are attended (no mask beyond that).
// work: fp32 scratch of sb_attention_decode_workspace(B, Hkv, splits) floats. splits <= 0 picks a
// split count that fills the GPU. Requires Hq / Hkv <= 8.
extern "C" long sb_attention_decode_workspace(int B, int Hkv, int splits) {
  return (long)B * Hkv * splits * sb::DEC_N * (sb::DEC_D + 2);
}

extern "C" int sb_attention_decode_splits(int B, int Hkv, int Sk) {
  const int nblocks = (Sk + 127) / 128;
  int want = (2 * sb::num_sms() + B * Hkv - 1) / (B * Hkv);     // about two waves of CTAs
  if (want > nblocks) want = nblocks;
  if (want < 1) want = 1;
  if (want > 64) want = 64;
  return want;
}

static int decode_launch(const void* q, const void* k, const void* v, void* o, float* work, int B, int Hq, int Hkv,
                         int Sk, const int* sk_ptr, int sk_add, int cap, int D, const long* q_strides,
                         const long* k_strides, const long* v_strides, const long* o_strides, float scale, int splits,
                         cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(D == DEC_D && B > 0 && Hq > 0 && Hkv > 0 && Hq % Hkv == 0 && Hq / Hkv <= DEC_N);
  SB_CHECK_ARG(Sk > 0 && Sk <= cap && B <= 65535 && Hkv <= 65535);
  if (splits <= 0) splits = sb_attention_decode_splits(B, Hkv, Sk);
  const int nblocks = (Sk + 127) / 128;
  if (splits > nblocks) splits = nblocks;
  CUtensorMap tmK, tmV;
  int rc;
  {
    uint64_t dims[4] = {(uint64_t)D, (uint64_t)Hkv, (uint64_t)cap, (uint64_t)B};
    uint32_t box[4] = {64, 1, 128, 1};
    uint64_t ks[3] = {(uint64_t)k_strides[2] * 2, (uint64_t)k_strides[1] * 2, (uint64_t)k_strides[0] * 2};
    uint64_t vs[3] = {(uint64_t)v_strides[2] * 2, (uint64_t)v_strides[1] * 2, (uint64_t)v_strides[0] * 2};
    if ((rc = make_tmap(&tmK, k, 2, 4, dims, ks, box, true))) return rc;
    if ((rc = make_tmap(&tmV, v, 2, 4, dims, vs, box, true))) return rc;
  }
  DecParams p;
  p.B = B; p.Hq = Hq; p.Hkv = Hkv; p.Sk = Sk; p.splits = splits;
  p.sk_ptr = sk_ptr; p.sk_add = sk_add;
  p.blocks_per_split = (nblocks + splits - 1) / splits;
  p.scale_log2 = scale * 1.4426950408889634f;
  p.q = (const __nv_bfloat16*)q; p.q_sb = q_strides[0]; p.q_sh = q_strides[1];
  const size_t n8 = (size_t)B * Hkv * splits * DEC_N;
  p.part_o = work; p.part_m = work + n8 * DEC_D; p.part_l = p.part_m + n8;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(attention_decode_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, DEC_SMEM));
    attr_set[dev & 63] = true;
  }
  attention_decode_kernel<<<dim3(splits, Hkv, B), DEC_THREADS, DEC_SMEM, st>>>(tmK, tmV, p);
  attention_decode_merge_kernel<<<dim3(Hq, B), DEC_D, 0, st>>>(p.part_o, p.part_m, p.part_l, (__nv_bfloat16*)o,
                                                               o_strides[0], o_strides[1], Hq, Hkv, splits);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_attention_decode(const void* q, const void* k, const void* v, void* o, float* work, int B, int Hq, int Hkv,
                                   int Sk, int cap, int D, const long* q_strides, const long* k_strides,
                                   const long* v_strides, const long* o_strides, float scale, int splits, cudaStream_t st) {
  return decode_launch(q, k, v, o, work, B, Hq, Hkv, Sk, nullptr, 0, cap, D, q_strides, k_strides, v_strides, o_strides,
                       scale, splits, st);
}

// Same, with the live length read on the device: Sk = min(*sk_ptr + sk_add, cap). The grid is
// sized for `cap`, so the launch does not depend on the position and can sit in a CUDA graph.
extern "C" int sb_attention_decode_dyn(const void* q, const void* k, const void* v, void* o, float* work, int B, int Hq,
                                       int Hkv, const int* sk_ptr, int sk_add, int cap, int D, const long* q_strides,
                                       const long* k_strides, const long* v_strides, const long* o_strides, float scale,
                                       int splits, cudaStream_t st) {
  SB_CHECK_ARG(sk_ptr != nullptr);
  return decode_launch(q, k, v, o, work, B, Hq, Hkv, cap, sk_ptr, sk_add, cap, D, q_strides, k_strides, v_strides,
                       o_strides, scale, splits, st);
}

// One decode step's RoPE + KV-cache append with the position read on the device:
//   q heads of qkv `[B, (Hq + 2 Hkv) * D]` (row stride ld) are rotated in place, k heads are rotated
//   and written to k_cache[b, *pos], v heads are copied to v_cache[b, *pos]. cos / sin `[max_pos, D/2]`.
namespace sb {
__global__ void decode_rope_append_kernel(__nv_bfloat16* __restrict__ qkv, const float* __restrict__ cos_t,
                                          const float* __restrict__ sin_t, __nv_bfloat16* __restrict__ kc,
                                          __nv_bfloat16* __restrict__ vc, const int* __restrict__ pos_ptr, int B, int Hq,
                                          int Hkv, int D, long ld, long c_sb, long c_ss, long c_sh, int cap) {
  const int pos = min(*pos_ptr, cap - 1);
  const int tph = D / 8, heads = Hq + 2 * Hkv;
  const long total = (long)B * heads * tph;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int part = i % tph;
    const int h = (i / tph) % heads;
    const int b = i / ((long)tph * heads);
    __nv_bfloat16* src = qkv + b * ld + (long)h * D + part * 8;
    uint4 w = *reinterpret_cast<const uint4*>(src);
    if (h < Hq + Hkv) {
      const float4 c = *reinterpret_cast<const float4*>(cos_t + (long)pos * (D / 2) + part * 4);
      const float4 sn = *reinterpret_cast<const float4*>(sin_t + (long)pos * (D / 2) + part * 4);
      uint4 r;
      r.x = pack_bf16(bf16_lo(w.x) * c.x - bf16_hi(w.x) * sn.x, bf16_lo(w.x) * sn.x + bf16_hi(w.x) * c.x);
      r.y = pack_bf16(bf16_lo(w.y) * c.y - bf16_hi(w.y) * sn.y, bf16_lo(w.y) * sn.y + bf16_hi(w.y) * c.y);
      r.z = pack_bf16(bf16_lo(w.z) * c.z - bf16_hi(w.z) * sn.z, bf16_lo(w.z) * sn.z + bf16_hi(w.z) * c.z);
      r.w = pack_bf16(bf16_lo(w.w) * c.w - bf16_hi(w.w) * sn.w, bf16_lo(w.w) * sn.w + bf16_hi(w.w) * c.w);
      w = r;
    }
    if (h < Hq) {
      *reinterpret_cast<uint4*>(src) = w;
    } else {
      const int hk = h < Hq + Hkv ? h - Hq : h - Hq - Hkv;
      __nv_bfloat16* dst = (h < Hq + Hkv ? kc : vc) + b * c_sb + (long)pos * c_ss + (long)hk * c_sh + part * 8;
      *reinterpret_cast<uint4*>(dst) = w;
    }
  }
}
}  // namespace sb

extern "C" int sb_decode_rope_append(void* qkv, const float* cos_t, const float* sin_t, void* k_cache, void* v_cache,
                                     const int* pos_ptr, int B, int Hq, int Hkv, int D, long ld, const long* cache_strides,
                                     int cap, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(D % 8 == 0 && ld % 8 == 0 && B > 0 && cap > 0);
  const long total = (long)B * (Hq + 2 * Hkv) * (D / 8);
  long blocks = (total + 255) / 256;
  if (blocks > 8L * num_sms()) blocks = 8L * num_sms();
  decode_rope_append_kernel<<<(int)blocks, 256, 0, st>>>((__nv_bfloat16*)qkv, cos_t, sin_t, (__nv_bfloat16*)k_cache,
                                                         (__nv_bfloat16*)v_cache, pos_ptr, B, Hq, Hkv, D, ld,
                                                         cache_strides[0], cache_strides[1], cache_strides[2], cap);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
