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
#include "gemm_pair.h"
#include "host_util.h"
#include "sm100.cuh"
#include <stdlib.h>
#include <string.h>

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

// Tensor-parallel fusion (COMM template parameter of the kernel body):
//   COMM_AG  all-gather -> GEMM: every rank owns M/P rows of the activation, stored in place in
//            its own full-size symmetric buffer; a few trailing "copier" CTAs pull the peers'
//            row blocks over NVLink with bulk copies (exactly once per byte) into the local
//            buffer and publish one counter per 128-row tile; the GEMM CTAs start with the
//            local rows and wait per tile for the counter before loading a peer's rows.
//   COMM_RS  GEMM -> reduce-scatter: the epilogue stores each partial output tile straight into
//            the owning rank's inbox slot (TMA store to peer memory); after its last tile every
//            CTA joins an arrival protocol and the kernel ends with the owner summing the P
//            slots of its rows (+ residual) into the bf16 output.
enum { COMM_NONE = 0, COMM_AG = 1, COMM_RS = 2 };
constexpr int TP_MAX = 8;
constexpr int SIG_RS_ARRIVE = 16, SIG_AG_READY = 32, SIG_AG_DONE = 48;   // words of the signal pad
constexpr uint32_t AG_CHUNK = 16384;

struct alignas(64) TpArgs {
  CUtensorMap tmC[TP_MAX];          // RS: slot of this rank inside every owner's inbox
  uint32_t* sig[TP_MAX];            // every rank's signal pad
  const uint8_t* xfull[TP_MAX];     // AG: every rank's full-size activation buffer
  uint8_t* xlocal;                  // AG: this rank's buffer (writable alias of xfull[rank])
  const __nv_bfloat16* slots;       // RS: this rank's inbox for this call, [P][rows_per * N]
  const __nv_bfloat16* residual;    // RS: optional [rows_per, N]
  __nv_bfloat16* out;               // RS: [rows_per, N]
  uint32_t* ag_flags;               // AG: per row tile, chunks landed (zeroed before launch)
  unsigned int* cta_counter;        // local arrival counter (self-resetting)
  long slot_elems;                  // RS: rows_per * N
  long slot_pitch;                  // RS: elements between two sources' slots in an inbox
  int rank, world, tiles_per_rank, n_copiers;
  uint32_t epoch, chunks_per_tile;
};

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
template <int GROUP, int COMM = COMM_NONE>
__device__ __forceinline__ void decode_unit(const GemmParams& p, int u, int tiles_m, int& tm, int& tn, int& e,
                                            int& kb0, int& kb1, const TpArgs* tp = nullptr) {
  if (COMM != COMM_NONE) {
    // row tiles in ownership order: AG starts with this rank's rows (no wait), RS ends with
    // them (the stores that cross NVLink leave first); column tiles fastest
    const int lin = u / p.tiles_n;
    tn = u - lin * p.tiles_n;
    const int rot = (COMM == COMM_AG ? tp->rank : tp->rank + 1) * tp->tiles_per_rank;
    tm = (lin + rot) % tiles_m;
    e = 0;
    kb0 = 0;
    kb1 = p.k_blocks;
  } else if (GROUP == 0) {
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

// Copier role of the all-gather GEMM (one thread per copier CTA drives a ring of bulk copies:
// peer memory -> shared memory -> local buffer). NST ring slots of AG_CHUNK bytes; a slot is
// refilled once its store has completed, which is also when its row tile's counter is bumped.
template <int NST, int LAG>
__device__ void ag_copier(const GemmParams& p, const TpArgs& tp, uint8_t* smem, int c) {
  uint64_t* full = reinterpret_cast<uint64_t*>(smem + NST * AG_CHUNK);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(full + NST);
  if (threadIdx.x == 0) {
    for (int s = 0; s < NST; ++s) mbar_init(&full[s], 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  __syncthreads();
  if (threadIdx.x != 0) return;
  const int P = tp.world, rank = tp.rank, nc = tp.n_copiers;
  if (c == 0) {
    // everything this rank wrote into its own rows is complete (stream order): tell the peers
    __threadfence_system();
    for (int pr = 0; pr < P; ++pr)
      if (pr != rank) st_release_sys_u32(tp.sig[pr] + SIG_AG_READY + rank, tp.epoch);
  }
  const long cpt = tp.chunks_per_tile;
  const long per_peer = (long)tp.tiles_per_rank * cpt;
  const long total = (long)(P - 1) * per_peer;
  const long n_my = total > c ? (total - c + nc - 1) / nc : 0;
  int ready_s = 0;
  bool ok = true;
  auto locate = [&](long i, int& s, int& src, int& tile, long& off) {
    const long g = c + i * nc;
    s = (int)(g / per_peer) + 1;
    const long w = g - (long)(s - 1) * per_peer;
    src = rank + s;
    if (src >= P) src -= P;
    tile = src * tp.tiles_per_rank + (int)(w / cpt);
    off = ((long)src * per_peer + w) * AG_CHUNK;
  };
  auto issue_load = [&](long i) -> bool {
    int s, src, tile; long off;
    locate(i, s, src, tile, off);
    if (s > ready_s) {
      if (!wait_flag_sys(tp.sig[rank] + SIG_AG_READY + src, tp.epoch)) { atomicOr(p.err, 4u); return false; }
      ready_s = s;
    }
    const int st = (int)(i % NST);
    mbar_expect_tx(&full[st], AG_CHUNK);
    bulk_load(smem + st * AG_CHUNK, tp.xfull[src] + off, AG_CHUNK, &full[st]);
    return true;
  };
  auto signal = [&](long i) {
    int s, src, tile; long off;
    locate(i, s, src, tile, off);
    fence_proxy_async_global();
    red_release_gpu_add_u32(tp.ag_flags + tile, 1u);
  };
  long issued = 0, signalled = 0;
  for (; issued < n_my && issued < NST && ok; ++issued) ok = issue_load(issued);
  long i = 0;
  for (; i < n_my && ok; ++i) {
    if (!mbar_wait(&full[i % NST], (uint32_t)((i / NST) & 1), abort_flag, p.err)) { ok = false; break; }
    int s, src, tile; long off;
    locate(i, s, src, tile, off);
    bulk_store(tp.xlocal + off, smem + (i % NST) * AG_CHUNK, AG_CHUNK);
    tma_store_commit();
    if (i >= LAG) {
      tma_store_wait_all<LAG>();          // the store of chunk i - LAG has completed
      signal(i - LAG);
      signalled = i - LAG + 1;
      if (issued < n_my) { ok = issue_load(issued); ++issued; }
    }
  }
  tma_store_wait_all<0>();
  if (ok) for (; signalled < n_my; ++signalled) signal(signalled);
  if (!ok) { const long long t0 = clock64(); while (clock64() - t0 < 4000000) {} }   // loads in flight
  // Last copier CTA: tell the peers this rank has finished reading their rows, then hold the
  // kernel until every peer has finished reading ours, so that the end of this kernel means
  // "my rows may be overwritten".
  __threadfence();
  if (atomicAdd(tp.cta_counter, 1u) == (unsigned)nc - 1) {
    *tp.cta_counter = 0;
    __threadfence_system();
    for (int pr = 0; pr < P; ++pr)
      if (pr != rank) st_release_sys_u32(tp.sig[pr] + SIG_AG_DONE + rank, tp.epoch);
    for (int pr = 0; pr < P && ok; ++pr)
      if (pr != rank && !wait_flag_sys(tp.sig[rank] + SIG_AG_DONE + pr, tp.epoch)) { atomicOr(p.err, 4u); ok = false; }
  }
}

template <int BN, bool A_MN, bool B_MN, int OUT, int GROUP, int COMM>
__device__ __forceinline__ void gemm_body(const CUtensorMap& tmA, const CUtensorMap& tmB, const CUtensorMap& tmC,
                                          const GemmParams& p, const TpArgs* tp) {
  using S = GemmShape<BN>;
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  const int ncta = COMM == COMM_AG ? (int)gridDim.x - tp->n_copiers : (int)gridDim.x;
  if (COMM == COMM_AG && (int)blockIdx.x >= ncta) {
    ag_copier<12, 4>(p, *tp, smem, (int)blockIdx.x - ncta);
    return;
  }
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
      for (int u = blockIdx.x; u < num_units && ok; u += ncta) {
        int tm, tn, e, kb0, kb1;
        decode_unit<GROUP, COMM>(p, u, tiles_m, tm, tn, e, kb0, kb1, tp);
        const int m0 = tm * GEMM_BM, n0 = tn * BN;
        if (COMM == COMM_AG && tm / tp->tiles_per_rank != tp->rank) {
          // a peer's rows: wait until the copiers have landed the whole 128-row tile
          if (!wait_flag_gpu(tp->ag_flags + tm, tp->chunks_per_tile)) {
            *abort_flag = 1;
            atomicOr(p.err, 4u);
            ok = false;
            break;
          }
          fence_proxy_async_global();
        }
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
      for (int u = blockIdx.x; u < num_units && ok; u += ncta, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * BN;
        int tm_, tn_, e_, kb0, kb1;
        decode_unit<GROUP, COMM>(p, u, tiles_m, tm_, tn_, e_, kb0, kb1, tp);
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
    for (int u = blockIdx.x; u < num_units && ok; u += ncta, ++tile_iter) {
      int tm, tn, e, kb0, kb1;
      decode_unit<GROUP, COMM>(p, u, tiles_m, tm, tn, e, kb0, kb1, tp);
      const int m0 = tm * GEMM_BM, n0 = tn * BN;
      // RS: the tile goes to the rank that owns these rows, at its row offset inside the slot
      const int owner = COMM == COMM_RS ? tm / tp->tiles_per_rank : 0;
      const CUtensorMap* tmc = COMM == COMM_RS ? &tp->tmC[owner] : &tmC;
      const int c_row0 = COMM == COMM_RS ? m0 - owner * tp->tiles_per_rank * GEMM_BM : m0;
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
          else tma_store_2d(tmc, stage_buf + buf * 4096, col0, c_row0 + q * 32);
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
  if (COMM == COMM_RS) {
    // Every store of this CTA has completed (the epilogue warps drained their bulk groups
    // before the barrier above). The last CTA to get here publishes this rank's arrival to
    // every owner; then all CTAs wait for all sources and sum the slots of this rank's rows.
    __shared__ int rs_ok;
    if (threadIdx.x == 0) {
      rs_ok = *abort_flag ? 0 : 1;
      __threadfence_system();
      if (atomicAdd(tp->cta_counter, 1u) == gridDim.x - 1) {
        *tp->cta_counter = 0;
        __threadfence_system();
        for (int pr = 0; pr < tp->world; ++pr) st_release_sys_u32(tp->sig[pr] + SIG_RS_ARRIVE + tp->rank, tp->epoch);
      }
    }
    __syncthreads();
    if ((int)threadIdx.x < tp->world) {
      if (!wait_flag_sys(tp->sig[tp->rank] + SIG_RS_ARRIVE + threadIdx.x, tp->epoch)) {
        atomicOr(p.err, 8u);
        rs_ok = 0;
      }
    }
    __syncthreads();
    if (rs_ok) {
      const long n8 = tp->slot_elems >> 3;
      const int P = tp->world;
      for (long i = blockIdx.x * (long)GEMM_THREADS + threadIdx.x; i < n8; i += (long)gridDim.x * GEMM_THREADS) {
        float a[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
        if (tp->residual != nullptr) {
          const uint4 r = reinterpret_cast<const uint4*>(tp->residual)[i];
          a[0] = bf16_lo(r.x); a[1] = bf16_hi(r.x); a[2] = bf16_lo(r.y); a[3] = bf16_hi(r.y);
          a[4] = bf16_lo(r.z); a[5] = bf16_hi(r.z); a[6] = bf16_lo(r.w); a[7] = bf16_hi(r.w);
        }
        for (int s2 = 0; s2 < P; ++s2) {
          const uint4 v = __ldcg(reinterpret_cast<const uint4*>(tp->slots + (long)s2 * tp->slot_pitch) + i);
          a[0] += bf16_lo(v.x); a[1] += bf16_hi(v.x); a[2] += bf16_lo(v.y); a[3] += bf16_hi(v.y);
          a[4] += bf16_lo(v.z); a[5] += bf16_hi(v.z); a[6] += bf16_lo(v.w); a[7] += bf16_hi(v.w);
        }
        uint4 o;
        o.x = pack_bf16(a[0], a[1]); o.y = pack_bf16(a[2], a[3]); o.z = pack_bf16(a[4], a[5]); o.w = pack_bf16(a[6], a[7]);
        reinterpret_cast<uint4*>(tp->out)[i] = o;
      }
    }
  }
}

template <int BN, bool A_MN, bool B_MN, int OUT, int GROUP>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_bf16_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmC, const GemmParams p) {
  gemm_body<BN, A_MN, B_MN, OUT, GROUP, COMM_NONE>(tmA, tmB, tmC, p, nullptr);
}

// Tensor-parallel variants (A K-major, bf16 output): see COMM_AG / COMM_RS above.
template <int BN, bool B_MN, int COMM>
__global__ void __launch_bounds__(GEMM_THREADS, 1)
gemm_tp_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
               const __grid_constant__ CUtensorMap tmC, const GemmParams p, const __grid_constant__ TpArgs tp) {
  gemm_body<BN, false, B_MN, OUT_BF16, 0, COMM>(tmA, tmB, tmC, p, &tp);
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
  if (OUT == OUT_F32_ADD && bias == nullptr) {
    // The output is accumulated with TMA reduce-adds, so the contraction can be cut into any
    // number of pieces: pick the split count whose unit count fills whole waves of the
    // persistent grid best (each extra split costs one more fp32 read-modify-write of C).
    const int sms = num_sms();
    const int max_by_k = p.k_blocks / 8 > 0 ? p.k_blocks / 8 : 1;      // at least 8 k-blocks per unit
    double best_cost = 1e30;
    for (int s = 1; s <= max_by_k && s <= 32; ++s) {
      const long units = (long)p.num_tiles * s;
      const long waves = (units + sms - 1) / sms;
      const double kb = (double)((p.k_blocks + s - 1) / s);
      const double cost = waves * (kb + 6.0);                          // +6 k-blocks ~ per-unit prologue/epilogue
      if (cost < best_cost * 0.97) { best_cost = cost; p.splits = s; }
    }
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


// ---------------------------------------------------------------------------- tensor-parallel launchers
struct TpLocal {
  uint32_t* ag_flags;          // [4096] per row tile counters
  unsigned int* counter_ag;    // arrival counters (self-resetting)
  unsigned int* counter_rs;
};
static int tp_local(TpLocal** out) {
  static TpLocal locals[64];
  static bool ready[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64);
  if (!ready[dev]) {
    uint32_t* base = nullptr;
    SB_CHECK_CUDA(cudaMalloc(&base, (4096 + 64) * sizeof(uint32_t)));
    SB_CHECK_CUDA(cudaMemset(base, 0, (4096 + 64) * sizeof(uint32_t)));
    locals[dev].ag_flags = base;
    locals[dev].counter_ag = base + 4096;
    locals[dev].counter_rs = base + 4096 + 32;
    ready[dev] = true;
  }
  *out = &locals[dev];
  return SB_OK;
}

static void fill_params(GemmParams& p, int M, int N, int K, int BN) {
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + GEMM_BM - 1) / GEMM_BM;
  p.tiles_n = (N + BN - 1) / BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = (K + GEMM_BK - 1) / GEMM_BK;
  p.splits = 1; p.kb_per_split = p.k_blocks; p.num_units = p.num_tiles;
  p.bias = nullptr; p.bias_is_bf16 = 0;
  p.tile_expert = nullptr; p.num_m_tiles = nullptr; p.poff = nullptr; p.E = 1;
}

template <int BN, bool B_MN>
static int launch_ag_gemm(const void* const* xfull, const void* B, void* C, const void* bias, int bias_is_bf16,
                          const void* const* sig, int M, int N, int K, int ldb, int ldc, int rank, int world,
                          unsigned int epoch, int n_copiers, cudaStream_t stream) {
  using S = GemmShape<BN>;
  TpLocal* loc;
  int rc;
  if ((rc = tp_local(&loc))) return rc;
  CUtensorMap tmA, tmB, tmC;
  if ((rc = make_tmap_2d(&tmA, xfull[rank], 2, K, M, (uint64_t)K * 2, 64, GEMM_BM, true))) return rc;
  if (B_MN) rc = make_tmap_2d(&tmB, B, 2, N, K, (uint64_t)ldb * 2, 64, 64, true);
  else      rc = make_tmap_2d(&tmB, B, 2, K, N, (uint64_t)ldb * 2, 64, BN, true);
  if (rc) return rc;
  if ((rc = make_tmap_2d(&tmC, C, 2, N, M, (uint64_t)ldc * 2, 64, 32, true))) return rc;
  GemmParams p;
  fill_params(p, M, N, K, BN);
  p.bias = bias; p.bias_is_bf16 = bias_is_bf16;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  TpArgs tp;
  memset(&tp, 0, sizeof(tp));
  for (int i = 0; i < world; ++i) { tp.sig[i] = (uint32_t*)sig[i]; tp.xfull[i] = (const uint8_t*)xfull[i]; }
  tp.xlocal = (uint8_t*)xfull[rank];
  tp.ag_flags = loc->ag_flags;
  tp.cta_counter = loc->counter_ag;
  tp.rank = rank; tp.world = world;
  tp.tiles_per_rank = p.tiles_m / world;
  tp.n_copiers = n_copiers;
  tp.epoch = epoch;
  tp.chunks_per_tile = (uint32_t)((size_t)GEMM_BM * K * 2 / AG_CHUNK);
  SB_CHECK_CUDA(cudaMemsetAsync(loc->ag_flags, 0, sizeof(uint32_t) * p.tiles_m, stream));
  auto kern = gemm_tp_kernel<BN, B_MN, COMM_AG>;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
    attr_set[dev & 63] = true;
  }
  // all CTAs must be co-resident (GEMM CTAs wait on the copiers): one CTA per SM at most
  int gemm_ctas = num_sms() - n_copiers;
  if (gemm_ctas > p.num_units) gemm_ctas = p.num_units;
  kern<<<gemm_ctas + n_copiers, GEMM_THREADS, S::SMEM_BYTES, stream>>>(tmA, tmB, tmC, p, tp);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

template <int BN, bool B_MN>
static int launch_gemm_rs(const void* A, const void* B, const void* const* inbox, const void* const* sig, void* out,
                          const void* residual, int M, int N, int K, int lda, int ldb, long slot_pitch, int rank,
                          int world, unsigned int epoch, cudaStream_t stream) {
  using S = GemmShape<BN>;
  TpLocal* loc;
  int rc;
  if ((rc = tp_local(&loc))) return rc;
  CUtensorMap tmA, tmB;
  if ((rc = make_tmap_2d(&tmA, A, 2, K, M, (uint64_t)lda * 2, 64, GEMM_BM, true))) return rc;
  if (B_MN) rc = make_tmap_2d(&tmB, B, 2, N, K, (uint64_t)ldb * 2, 64, 64, true);
  else      rc = make_tmap_2d(&tmB, B, 2, K, N, (uint64_t)ldb * 2, 64, BN, true);
  if (rc) return rc;
  GemmParams p;
  fill_params(p, M, N, K, BN);
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  const int rows_per = M / world;
  const size_t parity_off = (size_t)(epoch & 1u) * world * slot_pitch;     // elements
  TpArgs tp;
  memset(&tp, 0, sizeof(tp));
  for (int i = 0; i < world; ++i) {
    tp.sig[i] = (uint32_t*)sig[i];
    const __nv_bfloat16* slot = (const __nv_bfloat16*)inbox[i] + parity_off + (size_t)rank * slot_pitch;
    if ((rc = make_tmap_2d(&tp.tmC[i], slot, 2, N, rows_per, (uint64_t)N * 2, 64, 32, true))) return rc;
  }
  tp.slots = (const __nv_bfloat16*)inbox[rank] + parity_off;
  tp.residual = (const __nv_bfloat16*)residual;
  tp.out = (__nv_bfloat16*)out;
  tp.cta_counter = loc->counter_rs;
  tp.slot_elems = (long)rows_per * N;
  tp.slot_pitch = slot_pitch;
  tp.rank = rank; tp.world = world;
  tp.tiles_per_rank = p.tiles_m / world;
  tp.epoch = epoch;
  auto kern = gemm_tp_kernel<BN, B_MN, COMM_RS>;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, S::SMEM_BYTES));
    attr_set[dev & 63] = true;
  }
  const int grid = p.num_units < num_sms() ? p.num_units : num_sms();
  kern<<<grid, GEMM_THREADS, S::SMEM_BYTES, stream>>>(tmA, tmB, tmA /*C comes from tp.tmC*/, p, tp);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

}  // namespace sb

// Whether the automatic tile choice takes the paired-CTA kernel (256 x 256 tiles over two SMs) for this
// shape. Measured on the llama-350m training shapes it is 8-12 % ahead of the single-CTA 128 x 256 kernel
// and level with cuBLAS; it needs enough 256 x 256 tiles to occupy the 74 pairs, unless the output is an
// fp32 accumulation, whose contraction is cut to fill the grid. SUMMA_GEMM_PAIR=0 turns it off.
static bool pair_gemm_preferred(int M, int N, int K, int out_mode) {
  static int mode = -1;
  if (mode < 0) {
    const char* e = getenv("SUMMA_GEMM_PAIR");
    mode = e ? atoi(e) : 1;
  }
  if (mode == 0 || M < 256 || N < 256) return false;
  const long tiles = (long)((M + 255) / 256) * ((N + 255) / 256);
  const int pairs = sb::num_sms() / 2;
  if (out_mode == sb::OUT_F32_ADD) return tiles * (K / 512 > 0 ? K / 512 : 1) >= pairs / 2;
  return tiles >= pairs / 2;
}

// C[M,N] = A*B (+bias). out_mode: 0 bf16 store, 1 fp32 store, 2 fp32 accumulate (C += A*B).
// a_mn / b_mn select the operand memory layout (see the file header). Leading
// dimensions are in elements; every base pointer must be 16-byte aligned and every
// leading dimension a multiple of 8 (bf16) / 4 (fp32) elements. tile_n: 0 = choose, 128 / 256 =
// single-CTA tiles of that width, 512 = the paired-CTA kernel (256 x 256 tile over two SMs).
extern "C" int sb_gemm_bf16(const void* A, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N,
                            int K, int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode, int tile_n,
                            cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(M > 0 && N > 0 && K > 0);
  SB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0);
  SB_CHECK_ARG(out_mode >= 0 && out_mode <= 2);
  SB_CHECK_ARG(out_mode == OUT_BF16 ? (ldc % 8 == 0) : (ldc % 4 == 0));
  if (tile_n == 0 && pair_gemm_preferred(M, N, K, out_mode)) tile_n = 512;
  if (tile_n == 512) return gemm_pair_bf16(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, stream);
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

// All-gather -> GEMM over `world` ranks of one NVSwitch domain (see COMM_AG in this file).
//   xfull[r]  rank r's full-size activation buffer `[M, K]` bf16 (row pitch K) in symmetric
//             memory; before the call every rank has written ITS rows [r*M/P, (r+1)*M/P) in place.
//   C[M, N] = gather(X) * B (+ bias); B is `[K, N]` (b_mn = 1) or `[N, K]` (b_mn = 0), local.
//   sig[r]    rank r's signal pad (>= 64 words, zero at start); epoch grows by one per call on
//             every rank. When the kernel has finished, this rank's rows may be overwritten.
// Requires M % (128 * world) == 0, K % 64 == 0, world <= 8.
extern "C" int sb_tp_ag_gemm(const void* const* xfull, const void* B, void* C, const void* bias, int bias_is_bf16,
                             const void* const* sig, int M, int N, int K, int ldb, int ldc, int b_mn, int rank,
                             int world, unsigned int epoch, int n_copiers, cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(world >= 2 && world <= TP_MAX && rank >= 0 && rank < world);
  SB_CHECK_ARG(M > 0 && M % (GEMM_BM * world) == 0 && K % 64 == 0 && N % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0);
  SB_CHECK_ARG(M / GEMM_BM <= 4096);
  // copier CTAs: 12 cover one peer; with more peers the copy phase was exposed (4 ranks, 8192 x 4096 x 7168:
  // 0.667 ms with 12, 0.438 ms with 24, 0.470 ms with 40 copiers; NCCL all-gather + GEMM 0.455 ms)
  if (n_copiers <= 0) n_copiers = world > 2 ? 24 : 12;
  SB_CHECK_ARG(n_copiers < num_sms() - 8);
  if (N >= 256) {
    if (b_mn) return launch_ag_gemm<256, true>(xfull, B, C, bias, bias_is_bf16, sig, M, N, K, ldb, ldc, rank, world, epoch, n_copiers, stream);
    return launch_ag_gemm<256, false>(xfull, B, C, bias, bias_is_bf16, sig, M, N, K, ldb, ldc, rank, world, epoch, n_copiers, stream);
  }
  if (b_mn) return launch_ag_gemm<128, true>(xfull, B, C, bias, bias_is_bf16, sig, M, N, K, ldb, ldc, rank, world, epoch, n_copiers, stream);
  return launch_ag_gemm<128, false>(xfull, B, C, bias, bias_is_bf16, sig, M, N, K, ldb, ldc, rank, world, epoch, n_copiers, stream);
}

// GEMM -> reduce-scatter (see COMM_RS in this file): every rank multiplies its K-shard,
// partial = A[M, K] * B, and rank r ends with out[M/P, N] = sum over ranks of the partial rows
// [r*M/P, (r+1)*M/P) (+ residual[M/P, N]).
//   inbox[r]  rank r's inbox in symmetric memory: 2 (epoch parity) * world * slot_capacity bf16
//             (slot_capacity >= (M/P) * N and a multiple of 8; it is the pitch between slots, so
//             calls of different shapes can share one inbox).
//   sig[r]    signal pads as above; epoch grows by one per call on every rank.
// Requires M % (128 * world) == 0, N % 8 == 0, world <= 8.
extern "C" int sb_tp_gemm_rs(const void* A, const void* B, const void* const* inbox, const void* const* sig, void* out,
                             const void* residual, int M, int N, int K, int lda, int ldb, int b_mn, long slot_capacity,
                             int rank, int world, unsigned int epoch, cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(world >= 2 && world <= TP_MAX && rank >= 0 && rank < world);
  SB_CHECK_ARG(M > 0 && M % (GEMM_BM * world) == 0 && K % 8 == 0 && N % 8 == 0 && lda % 8 == 0 && ldb % 8 == 0);
  const long slot_elems = (long)(M / world) * N;
  if (slot_elems > slot_capacity) return SB_ERR_TOO_LARGE;
  SB_CHECK_ARG(slot_capacity % 8 == 0);
  if (N >= 256) {
    if (b_mn) return launch_gemm_rs<256, true>(A, B, inbox, sig, out, residual, M, N, K, lda, ldb, slot_capacity, rank, world, epoch, stream);
    return launch_gemm_rs<256, false>(A, B, inbox, sig, out, residual, M, N, K, lda, ldb, slot_capacity, rank, world, epoch, stream);
  }
  if (b_mn) return launch_gemm_rs<128, true>(A, B, inbox, sig, out, residual, M, N, K, lda, ldb, slot_capacity, rank, world, epoch, stream);
  return launch_gemm_rs<128, false>(A, B, inbox, sig, out, residual, M, N, K, lda, ldb, slot_capacity, rank, world, epoch, stream);
}
