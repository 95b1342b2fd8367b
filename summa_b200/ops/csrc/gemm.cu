// BF16 GEMM on the 5th-generation tensor cores: C[M,N] = A * B (+ bias), fp32 accumulate.
//
// Design (one persistent CTA per SM, 192 threads):
//   warp 0      TMA producer: cp.async.bulk.tensor loads of A and B tiles into a
//               multi-stage 128B-swizzled shared-memory ring (full/empty mbarriers)
//   warp 1      MMA issuer: one thread issues tcgen05.mma (128 x BN x 16) reading the
//               ring through shared-memory descriptors, accumulating in TMEM; commits
//               free ring slots and publish finished accumulators
//   warps 2..5  epilogue: tcgen05.ld the accumulator (one row per thread), add bias,
//               convert, stage through swizzled shared memory and write with TMA stores
//               (or TMA reduce-add for fp32 accumulation into an existing C)
// The accumulator is double-buffered in TMEM (2 x BN columns), so the epilogue of tile i
// overlaps the main loop of tile i+1.
//
// Operand layouts (all row-major in memory, leading dimension in elements):
//   A "K-major":  memory [M, K]        A "MN-major": memory [K, M]
//   B "K-major":  memory [N, K]        B "MN-major": memory [K, N]
// so x @ W with W [K,N] is (A K-major, B MN-major); dY @ W^T is (K-major, K-major);
// X^T @ dY is (MN-major, MN-major). No operand is ever transposed in memory.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int GEMM_BM = 128;
constexpr int GEMM_BK = 64;
constexpr int GEMM_THREADS = 192;
constexpr int GEMM_A_BYTES = GEMM_BM * GEMM_BK * 2;      // 16 KB
constexpr int GEMM_EPI_BYTES = 4 * 2 * 4096;             // 4 warps x 2 buffers x (32 rows x 128 B)
constexpr int GEMM_GROUP_M = 8;

template <int BN>
struct GemmShape {
  static constexpr int B_BYTES = BN * GEMM_BK * 2;
  static constexpr int STAGE_BYTES = GEMM_A_BYTES + B_BYTES;
  static constexpr int STAGES = (BN == 256) ? 4 : 6;
  static constexpr int TMEM_COLS = 2 * BN;
  static constexpr int SMEM_BYTES = STAGES * STAGE_BYTES + GEMM_EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
};

struct GemmParams {
  int M, N, K;
  int tiles_m, tiles_n, num_tiles, k_blocks;
  int splits, kb_per_split, num_units;   // split-K (fp32 reduce-add output only)
  // grouped (mixture-of-experts) modes, see GROUP below
  const int* tile_expert;   // [m tiles] expert of every 128-row tile of the padded routed layout
  const int* num_m_tiles;   // device scalar: live 128-row tiles
  const int* poff;          // [E+1] padded row offset of every expert (multiples of 128)
  int E;
  const void* bias;      // [N] or null
  int bias_is_bf16;
  unsigned int* err;
};

enum { OUT_BF16 = 0, OUT_F32 = 1, OUT_F32_ADD = 2 };

__device__ __forceinline__ void tile_coords(int t, int tiles_m, int tiles_n, int& tm, int& tn) {
  const int group = GEMM_GROUP_M * tiles_n;
  const int g = t / group;
  const int first_m = g * GEMM_GROUP_M;
  const int gm = min(tiles_m - first_m, GEMM_GROUP_M);
  const int r = t - g * group;
  tm = first_m + r % gm;
  tn = r / gm;
}

// GROUP 0: one dense problem.
// GROUP 1: rows of A / C are the expert-sorted, 128-row-padded routed tokens; B is `[E, ...]`
//          and the expert of a row tile comes from `tile_expert` (device memory); the number
//          of live row tiles is read from `num_m_tiles`, so no count ever visits the host.
// GROUP 2: per-expert weight gradient: C is `[E, M, N]`, the contraction runs over the
//          expert's padded rows [poff[e], poff[e+1]).
template <int GROUP>
__device__ __forceinline__ void decode_unit(const GemmParams& p, int u, int tiles_m, int& tm, int& tn, int& e,
                                            int& kb0, int& kb1) {
  if (GROUP == 0) {
    const int t = u / p.splits, sp = u - t * p.splits;
    tile_coords(t, tiles_m, p.tiles_n, tm, tn);
    e = 0;
    kb0 = sp * p.kb_per_split;
    kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
  } else if (GROUP == 1) {
    tile_coords(u, tiles_m, p.tiles_n, tm, tn);
    e = p.tile_expert[tm];
    kb0 = 0;
    kb1 = p.k_blocks;
  } else {
    const int per = tiles_m * p.tiles_n;
    e = u / per;
    tile_coords(u - e * per, tiles_m, p.tiles_n, tm, tn);
    kb0 = p.poff[e] / GEMM_BK;
    kb1 = p.poff[e + 1] / GEMM_BK;
  }
}

template <int BN, bool A_MN, bool B_MN, int OUT, int GROUP>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  using S = GemmShape<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* epi = smem + S::STAGES * S::STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + GEMM_EPI_BYTES);
  uint64_t* full = bars;
  uint64_t* empty = bars + S::STAGES;
  uint64_t* tfull = bars + 2 * S::STAGES;
  uint64_t* tempty = tfull + 2;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;

  if (threadIdx.x == 0) {
    for (int s = 0; s < S::STAGES; ++s) {
      mbar_init(&full[s], 1);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 4);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc(tmem_slot, S::TMEM_COLS);
    tmem_relinquish();
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int tiles_m = GROUP == 1 ? *p.num_m_tiles : p.tiles_m;
  const int num_units = GROUP == 1 ? tiles_m * p.tiles_n : p.num_units;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x) {
        int tm, tn, e, kb0, kb1;
        decode_unit<GROUP>(p, u, tiles_m, tm, tn, e, kb0, kb1);
        const int m0 = tm * GEMM_BM, n0 = tn * BN;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % S::STAGES;
          const uint32_t ph = (it / S::STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.err)) { ok = false; break; }
          uint8_t* sa = ring + s * S::STAGE_BYTES;
          uint8_t* sb_ = sa + GEMM_A_BYTES;
          mbar_expect_tx(&full[s], S::STAGE_BYTES);
          const int k0 = kb * GEMM_BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < GEMM_BM / 64; ++i) tma_load_2d(sa + i * 8192, &tmA, &full[s], m0 + 64 * i, k0);
          } else {
            tma_load_2d(sa, &tmA, &full[s], k0, m0);
          }
          if (GROUP == 1) {
            if (B_MN) {
#pragma unroll
              for (int i = 0; i < BN / 64; ++i) tma_load_3d(sb_ + i * 8192, &tmB, &full[s], n0 + 64 * i, k0, e);
            } else {
              tma_load_3d(sb_, &tmB, &full[s], k0, n0, e);
            }
          } else if (B_MN) {
#pragma unroll
            for (int i = 0; i < BN / 64; ++i) tma_load_2d(sb_ + i * 8192, &tmB, &full[s], n0 + 64 * i, k0);
          } else {
            tma_load_2d(sb_, &tmB, &full[s], k0, n0);
          }
        }
      }
      if (!ok) {
        // give loads already in flight time to land before the CTA can exit
        const long long t0 = clock64();
        while (clock64() - t0 < 2000000) {}
      }
    }
    __syncwarp();
  } else if (warp == 1) {
    // ------------------------------------------------------------ MMA issuer
    if (lane == 0) {
      constexpr uint32_t idesc = make_idesc_bf16(GEMM_BM, BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int tm_, tn_, e_, kb0, kb1;
        decode_unit<GROUP>(p, u, tiles_m, tm_, tn_, e_, kb0, kb1);
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % S::STAGES;
          const uint32_t ph = (it / S::STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(ring + s * S::STAGE_BYTES);
          const uint32_t b_base = a_base + GEMM_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < GEMM_BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_base + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_base + kk * 32, 16, 1024);
            umma_bf16(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit(&empty[s]);
        }
        // an expert without rows contributes nothing: publish an accumulator the epilogue skips
        if (ok) umma_commit(&tfull[acc]);
      }
    }
    __syncwarp();
  } else {
    // ------------------------------------------------------------ epilogue (warps 2..5)
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    uint8_t* stage_buf = epi + q * 8192;
    uint32_t tile_iter = 0;
    uint32_t buf = 0;
    bool ok = true;
    constexpr int CHUNK_COLS = (OUT == OUT_BF16) ? 64 : 32;   // 128 bytes per row per chunk
    for (int u = blockIdx.x; u < num_units && ok; u += gridDim.x, ++tile_iter) {
      int tm, tn, e, kb0, kb1;
      decode_unit<GROUP>(p, u, tiles_m, tm, tn, e, kb0, kb1);
      const int m0 = tm * GEMM_BM, n0 = tn * BN;
      const bool empty_unit = GROUP == 2 && kb1 <= kb0;   // nothing was accumulated
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * BN + (static_cast<uint32_t>(q * 32) << 16);
      for (int c = 0; c < BN / CHUNK_COLS; ++c) {
        const int col0 = n0 + c * CHUNK_COLS;
        if (col0 >= p.N || empty_unit) break;      // nothing to store
        uint32_t v[64];
        tmem_ld_32x32b_x32(t_row + c * CHUNK_COLS, v);
        if (CHUNK_COLS == 64) tmem_ld_32x32b_x32(t_row + c * CHUNK_COLS + 32, v + 32);
        tmem_ld_wait();
        if (p.bias != nullptr) {
#pragma unroll
          for (int j = 0; j < CHUNK_COLS; ++j) {
            const int col = col0 + j;
            float b = 0.f;
            if (col < p.N) {
              b = p.bias_is_bf16 ? __bfloat162float(reinterpret_cast<const __nv_bfloat16*>(p.bias)[col])
                                 : reinterpret_cast<const float*>(p.bias)[col];
            }
            v[j] = __float_as_uint(__uint_as_float(v[j]) + b);
          }
        }
        // the buffer we are about to overwrite must have been drained by its TMA store
        if (lane == 0) tma_store_wait_read<1>();
        __syncwarp();
        uint8_t* dst = stage_buf + buf * 4096 + lane * 128;
        if (OUT == OUT_BF16) {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 w;
            w.x = pack_bf16(__uint_as_float(v[8 * j + 0]), __uint_as_float(v[8 * j + 1]));
            w.y = pack_bf16(__uint_as_float(v[8 * j + 2]), __uint_as_float(v[8 * j + 3]));
            w.z = pack_bf16(__uint_as_float(v[8 * j + 4]), __uint_as_float(v[8 * j + 5]));
            w.w = pack_bf16(__uint_as_float(v[8 * j + 6]), __uint_as_float(v[8 * j + 7]));
            *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = w;
          }
        } else {
#pragma unroll
          for (int j = 0; j < 8; ++j) {
            uint4 w = make_uint4(v[4 * j], v[4 * j + 1], v[4 * j + 2], v[4 * j + 3]);
            *reinterpret_cast<uint4*>(dst + ((j ^ (lane & 7)) << 4)) = w;
          }
        }
        fence_proxy_async_smem();
        __syncwarp();
        if (lane == 0) {
          if (GROUP == 2) tma_reduce_add_3d(&tmC, stage_buf + buf * 4096, col0, m0 + q * 32, e);
          else if (OUT == OUT_F32_ADD) tma_reduce_add_2d(&tmC, stage_buf + buf * 4096, col0, m0 + q * 32);
          else tma_store_2d(&tmC, stage_buf + buf * 4096, col0, m0 + q * 32);
          tma_store_commit();
        }
        buf ^= 1;
      }
      // accumulator fully read: hand the TMEM buffer back to the MMA warp
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive(&tempty[acc]);
    }
    if (lane == 0) tma_store_wait_all<0>();
  }

  tc_fence_before();
  __syncthreads();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc(tmem_base, S::TMEM_COLS);
  }
}

template <int BN, bool A_MN, bool B_MN, int OUT>
static int launch_gemm(const void* A, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N, int K,
                       int lda, int ldb, int ldc, cudaStream_t stream) {
  using S = GemmShape<BN>;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if (A_MN) rc = make_tmap_2d(&tmA, A, 2, M, K, (uint64_t)lda * 2, 64, 64, true);
  else      rc = make_tmap_2d(&tmA, A, 2, K, M, (uint64_t)lda * 2, 64, GEMM_BM, true);
  if (rc) return rc;
  if (B_MN) rc = make_tmap_2d(&tmB, B, 2, N, K, (uint64_t)ldb * 2, 64, 64, true);
  else      rc = make_tmap_2d(&tmB, B, 2, K, N, (uint64_t)ldb * 2, 64, BN, true);
  if (rc) return rc;
  if (OUT == OUT_BF16) rc = make_tmap_2d(&tmC, C, 2, N, M, (uint64_t)ldc * 2, 64, 32, true);
  else                 rc = make_tmap_2d(&tmC, C, 4, N, M, (uint64_t)ldc * 4, 32, 32, true, true);
  if (rc) return rc;

  GemmParams p;
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.splits = 1;
  if (OUT == OUT_F32_ADD && p.num_tiles < num_sms() && bias == nullptr) {
    int want = num_sms() / p.num_tiles;
    int max_by_k = p.k_blocks / 4;          // keep at least 4 k-blocks per unit
    p.splits = want < max_by_k ? want : max_by_k;
    if (p.splits < 1) p.splits = 1;
  }
  p.kb_per_split = (p.k_blocks + p.splits - 1) / p.splits;
  p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;   // no empty split
  p.num_units = p.num_tiles * p.splits;
  p.bias = bias;
  p.bias_is_bf16 = bias_is_bf16;
  p.tile_expert = nullptr; p.num_m_tiles = nullptr; p.poff = nullptr; p.E = 1;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;

  auto kern = gemm_bf16_kernel<BN, A_MN, B_MN, OUT, 0>;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
    attr_set[dev & 63] = true;
  }
  const int grid = p.num_units < num_sms() ? p.num_units : num_sms();
  kern<<<grid, GEMM_THREADS, S::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

template <int BN, int OUT>
static int dispatch_major(int a_mn, int b_mn, const void* A, const void* B, void* C, const void* bias, int bias_is_bf16,
                          int M, int N, int K, int lda, int ldb, int ldc, cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_gemm<BN, false, false, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, st);
  if (!a_mn && b_mn) return launch_gemm<BN, false, true, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, st);
  if (a_mn && !b_mn) return launch_gemm<BN, true, false, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, st);
  return launch_gemm<BN, true, true, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, st);
}


// ---------------------------------------------------------------------------- grouped launchers
static int make_tmap_3d(CUtensorMap* m, const void* base, int elem, uint64_t d0, uint64_t d1, uint64_t d2,
                        uint64_t s1_bytes, uint64_t s2_bytes, uint32_t b0, uint32_t b1, bool f32) {
  uint64_t dims[3] = {d0, d1, d2};
  uint64_t strides[2] = {s1_bytes, s2_bytes};
  uint32_t box[3] = {b0, b1, 1};
  return make_tmap(m, base, elem, 3, dims, strides, box, true, f32);
}

// GROUP 1: C[rows, N] = A[rows, K] * B[expert(row tile)]; rows = padded routed layout.
template <int BN, bool B_MN>
static int launch_grouped_rows(const void* A, const void* B, void* C, int max_rows, int N, int K, int E, int lda, int ldc,
                               const int* tile_expert, const int* num_m_tiles, cudaStream_t stream) {
  using S = GemmShape<BN>;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_tmap_2d(&tmA, A, 2, K, max_rows, (uint64_t)lda * 2, 64, GEMM_BM, true))) return rc;
  if (B_MN) rc = make_tmap_3d(&tmB, B, 2, N, K, E, (uint64_t)N * 2, (uint64_t)N * K * 2, 64, 64, false);    // [E,K,N]
  else      rc = make_tmap_3d(&tmB, B, 2, K, N, E, (uint64_t)K * 2, (uint64_t)N * K * 2, 64, BN, false);    // [E,N,K]
  if (rc) return rc;
  if ((rc = make_tmap_2d(&tmC, C, 2, N, max_rows, (uint64_t)ldc * 2, 64, 32, true))) return rc;
  GemmParams p;
  p.M = max_rows; p.N = N; p.K = K;
  p.tiles_m = (max_rows + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.splits = 1; p.kb_per_split = p.k_blocks; p.num_units = p.num_tiles;
  p.bias = nullptr; p.bias_is_bf16 = 0;
  p.tile_expert = tile_expert; p.num_m_tiles = num_m_tiles; p.poff = nullptr; p.E = E;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  auto kern = gemm_bf16_kernel<BN, false, B_MN, OUT_BF16, 1>;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
    attr_set[dev & 63] = true;
  }
  const int grid = p.num_tiles < num_sms() ? p.num_tiles : num_sms();
  kern<<<grid, GEMM_THREADS, S::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// GROUP 2: dW[e] (+)= X[rows of e]^T * dY[rows of e], fp32 `[E, M, N]` accumulate.
template <int BN>
static int launch_grouped_wgrad(const void* X, const void* dY, float* dW, int max_rows, int M, int N, int E, int ldx,
                                int ldy, const int* poff, cudaStream_t stream) {
  using S = GemmShape<BN>;
  CUtensorMap tmA, tmB, tmC;
  int rc;
  if ((rc = make_tmap_2d(&tmA, X, 2, M, max_rows, (uint64_t)ldx * 2, 64, 64, true))) return rc;
  if ((rc = make_tmap_2d(&tmB, dY, 2, N, max_rows, (uint64_t)ldy * 2, 64, 64, true))) return rc;
  if ((rc = make_tmap_3d(&tmC, dW, 4, N, M, E, (uint64_t)N * 4, (uint64_t)N * M * 4, 32, 32, true))) return rc;
  GemmParams p;
  p.M = M; p.N = N; p.K = max_rows;
  p.tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = 0;
  p.splits = 1; p.kb_per_split = 0; p.num_units = p.num_tiles * E;
  p.bias = nullptr; p.bias_is_bf16 = 0;
  p.tile_expert = nullptr; p.num_m_tiles = nullptr; p.poff = poff; p.E = E;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  auto kern = gemm_bf16_kernel<BN, true, true, OUT_F32_ADD, 2>;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
    attr_set[dev & 63] = true;
  }
  const int grid = p.num_units < num_sms() ? p.num_units : num_sms();
  kern<<<grid, GEMM_THREADS, S::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

// C[M,N] = A*B (+bias). out_mode: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (C += A*B).
// a_mn / b_mn select the operand memory layout (see the file header). Leading
// dimensions are in elements; every base pointer must be 16-byte aligned and every
// leading dimension a multiple of 8 (bf16) / 4 (fp32) elements. tile_n: 0 = choose.
extern "C" int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N,
                            int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode, int tile_n,
                            cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(M > 0 && N > 0 && K > 0);
  SB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0);
  SB_CHECK_ARG(out_mode >= 0 && out_mode <= 2);
  SB_CHECK_ARG(out_mode == OUT_BF16 ? (ldc % 8 == 0) : (ldc % 4 == 0));
  if (tile_n == 0) {
    // fewer, fatter tiles unless that leaves the last wave mostly idle
    const int sms = num_sms();
    auto waves_cost = [&](int bn) {
      const long tiles = (long)((M + 127) / 128) * ((N + bn - 1) / bn);
      const long waves = (tiles + sms - 1) / sms;
      return (double)waves * bn * (bn == 256 ? 1.0 : 1.35);
    };
    tile_n = (N > 128 && waves_cost(256) <= waves_cost(128)) ? 256 : 128;
  }
  SB_CHECK_ARG(tile_n == 128 || tile_n == 256);
#define SB_GEMM_CASE(BN, OUT) \
  return dispatch_major<BN, OUT>(a_mn, b_mn, A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, stream)
  if (tile_n == 256) {
    if (out_mode == OUT_BF16) SB_GEMM_CASE(256, OUT_BF16);
    if (out_mode == OUT_F32) SB_GEMM_CASE(256, OUT_F32);
    SB_GEMM_CASE(256, OUT_F32_ADD);
  } else {
    if (out_mode == OUT_BF16) SB_GEMM_CASE(128, OUT_BF16);
    if (out_mode == OUT_F32) SB_GEMM_CASE(128, OUT_F32);
    SB_GEMM_CASE(128, OUT_F32_ADD);
  }
#undef SB_GEMM_CASE
}

// Grouped expert GEMM over the padded routed layout (see csrc/moe.cu for the layout):
//   C[rows, N] = A[rows, K] * W[expert of row tile]; W is `[E, K, N]` (w_kmajor = 0) or
//   `[E, N, K]` (w_kmajor = 1, i.e. multiply by the transpose of an `[E, N, K]` bank).
// tile_expert / num_m_tiles live in device memory; max_rows bounds the routed buffer.
extern "C" int sb_grouped_gemm_rows(const void* A, const void* W, void* C, int max_rows, int N, int K, int E, int lda,
                                    int ldc, int w_kmajor, const int* tile_expert, const int* num_m_tiles,
                                    cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(max_rows > 0 && max_rows % 128 == 0 && N % 8 == 0 && K % 8 == 0 && lda % 8 == 0 && ldc % 8 == 0);
  if (N >= 256) {
    if (w_kmajor) return launch_grouped_rows<256, false>(A, W, C, max_rows, N, K, E, lda, ldc, tile_expert, num_m_tiles, stream);
    return launch_grouped_rows<256, true>(A, W, C, max_rows, N, K, E, lda, ldc, tile_expert, num_m_tiles, stream);
  }
  if (w_kmajor) return launch_grouped_rows<128, false>(A, W, C, max_rows, N, K, E, lda, ldc, tile_expert, num_m_tiles, stream);
  return launch_grouped_rows<128, true>(A, W, C, max_rows, N, K, E, lda, ldc, tile_expert, num_m_tiles, stream);
}

// dW[e, M, N] += X[rows of e, M]^T * dY[rows of e, N] (fp32, accumulating). poff `[E+1]`
// device array of padded row offsets (multiples of 128).
extern "C" int sb_grouped_gemm_wgrad(const void* X, const void* dY, float* dW, int max_rows, int M, int N, int E, int ldx,
                                     int ldy, const int* poff, cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(max_rows > 0 && max_rows % 128 == 0 && N % 8 == 0 && M % 8 == 0 && ldx % 8 == 0 && ldy % 8 == 0);
  if (N >= 256) return launch_grouped_wgrad<256>(X, dY, dW, max_rows, M, N, E, ldx, ldy, poff, stream);
  return launch_grouped_wgrad<128>(X, dY, dW, max_rows, M, N, E, ldx, ldy, poff, stream);
}
