// BF16 GEMM on CTA pairs: C[M,N] = A * B (+ bias), fp32 accumulate, tcgen05.mma.cta_group::2.
//
// Why a second GEMM kernel: a single-CTA 128 x 256 x 16 product reads 12 KB of operands from
// shared memory per 128 tensor-core cycles (96 B/clk of a 128 B/clk port), and every stall of
// that port is a stall of the tensor pipe. In the paired form two SMs of one TPC compute a
// 256 x 256 tile together: each CTA stages its own 128 rows of A and only ITS HALF (128
// columns) of B, the hardware exchanges the halves, so the port carries 8 KB per 128 cycles.
//
// Roles per CTA (192 threads), both CTAs of the pair run all three:
//   warp 0      TMA producer: loads this CTA's A rows and B half into a 6-stage ring; the
//               byte counts of both CTAs are credited to the LEADER's `full` barrier
//   warp 1      leader only: one thread issues the M = 256 products and commits; a commit
//               arrives on the `empty` (ring slot free) or `tfull` (accumulator ready)
//               barrier at the same offset in BOTH CTAs
//   warps 2..5  epilogue: tcgen05.ld of this CTA's 128 accumulator rows, bias, convert,
//               swizzled staging, TMA store / reduce-add; then arrive on the leader's
//               `tempty` barrier (remote arrive from the second CTA)
// Accumulators are double-buffered in tensor memory (2 x 256 columns in each SM).
//
// Wave-aware tail: a persistent grid of 74 pairs leaves the last wave of a 3.46-wave problem
// mostly idle. When the remainder of the tile count fits twice into one wave, the last tiles
// are cut into 256 x 128 halves (same kernel, N = 128 products), so the tail costs half a
// wave instead of a whole one.
//
// Every wait is bounded (see sm100.cuh); the cluster barriers at the start and the end are
// hardware barriers that all threads reach because the bounded waits always return.
#include "gemm_pair.h"
#include "sm100.cuh"
#include <stdlib.h>
#include <string.h>

namespace sb {

constexpr int PG_BM = 128;                 // rows per CTA (the pair covers 256)
constexpr int PG_BN = 256;                 // columns per pair
constexpr int PG_BK = 64;
constexpr int PG_THREADS = 192;
constexpr int PG_A_BYTES = PG_BM * PG_BK * 2;            // 16 KB
constexpr int PG_B_BYTES = (PG_BN / 2) * PG_BK * 2;      // 16 KB: this CTA's half of B
constexpr int PG_STAGE_BYTES = PG_A_BYTES + PG_B_BYTES;
constexpr int PG_STAGES = 6;
constexpr int PG_EPI_BYTES = 4 * 2 * 4096;               // 4 warps x 2 buffers x (32 rows x 128 B)
constexpr int PG_TMEM_COLS = 2 * PG_BN;
constexpr int PG_SMEM_BYTES = PG_STAGES * PG_STAGE_BYTES + PG_EPI_BYTES + 1024 /*align*/ + 256 /*barriers*/;
constexpr int PG_GROUP_M = 8;

// All-gather role (world > 1): A is this rank's full-size activation buffer in symmetric memory, of which
// only the rank's own row block is valid at launch. The kernel first pushes that block into every peer's
// buffer (one `multimem.st` per 16 bytes through the switch when the allocation has a multicast address,
// otherwise one plain store per peer), 128-row chunk by chunk, raising one flag per (source, chunk) on every
// peer; the tile loop starts with the own rows and the TMA producer waits (bounded) on the chunk flag before it
// loads another rank's rows from LOCAL memory. No load of any kind touches peer memory.
constexpr int PG_AG_MAX = 8;
constexpr int PG_AG_DONE = 0;              // flag words [0, 8): rank r has finished reading its buffer (per call)
constexpr int PG_AG_CHUNK = 8;             // flag words [8, 8 + M / 128): chunk of 128 rows has arrived
struct PairAg {
  int world, rank;
  unsigned int epoch;                      // call number of this role (1, 2, ...), equal on all ranks
  int chunks_per_rank;                     // M / world / 128
  long chunk_bytes;                        // 128 * K * 2
  uint8_t* xfull[PG_AG_MAX];               // every rank's activation buffer
  uint8_t* xmc;                            // multicast address of the buffers, or null
  uint32_t* flags[PG_AG_MAX];              // every rank's flag array
  unsigned int* counters;                  // local, zero at first use: [chunks_per_rank] chunk counters, [+0] exit counter after them
};

struct PairParams {
  int group_m;                           // tile rows per raster group
  PairAg ag;
  int M, N, K;
  int tiles_m, tiles_n, num_tiles;       // 256 x 256 tiles
  int k_blocks, splits, kb_per_split;
  int first_half_tile;                   // tiles [first_half_tile, num_tiles) run as two 256 x 128 halves
  int num_full_units;                    // first_half_tile * splits
  int num_units;                         // + 2 per halved tile (per batch entry)
  int batch;                             // independent problems of the same shape (z coordinate of every tensor map)
  const void* bias;
  int bias_is_bf16;
  unsigned int* err;
};

// ag_world > 1 (all-gather role): tile rows are visited own rows first, then row j of every other source
// (ring order from this rank) for j = 0, 1, ...: the order in which pushed chunks arrive.
__device__ __forceinline__ void pair_tile_coords(int t, int tiles_m, int tiles_n, int group_m, int ag_world, int ag_rank,
                                                 int& tm, int& tn) {
  const int group = group_m * tiles_n;
  const int g = t / group;
  const int first_m = g * group_m;
  const int gm = min(tiles_m - first_m, group_m);
  const int r = t - g * group;
  int i = first_m + r % gm;
  tn = r / gm;
  if (ag_world > 1) {
    const int tpr = tiles_m / ag_world;            // tile rows per rank
    if (i < tpr) {
      i += ag_rank * tpr;
    } else {
      const int k = i - tpr;
      const int j = k / (ag_world - 1);
      int src = ag_rank + 1 + k % (ag_world - 1);
      if (src >= ag_world) src -= ag_world;
      i = src * tpr + j;
    }
  }
  tm = i;
}

// unit -> tile, column offset inside the tile, tile width, k-block range
__device__ __forceinline__ void pair_decode(const PairParams& p, int u, int& tm, int& tn, int& ncol0, int& width,
                                            int& kb0, int& kb1, int& bz) {
  int t;
  bz = u / p.num_units;
  u -= bz * p.num_units;
  if (u < p.num_full_units) {
    t = u / p.splits;
    const int sp = u - t * p.splits;
    kb0 = sp * p.kb_per_split;
    kb1 = min(p.k_blocks, kb0 + p.kb_per_split);
    ncol0 = 0;
    width = PG_BN;
  } else {
    const int h = u - p.num_full_units;
    t = p.first_half_tile + (h >> 1);
    kb0 = 0;
    kb1 = p.k_blocks;
    ncol0 = (h & 1) * (PG_BN / 2);
    width = PG_BN / 2;
  }
  pair_tile_coords(t, p.tiles_m, p.tiles_n, p.group_m, p.ag.world, p.ag.rank, tm, tn);
}

template <bool A_MN, bool B_MN, int OUT>
__global__ void __cluster_dims__(2, 1, 1) __launch_bounds__(PG_THREADS + 32, 1)
gemm_pair_kernel(const __grid_constant__ CUtensorMap tmA, const __grid_constant__ CUtensorMap tmB,
                 const __grid_constant__ CUtensorMap tmBh, const __grid_constant__ CUtensorMap tmC,
                 const PairParams p) {
  extern __shared__ uint8_t smem_raw[];
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint8_t* ring = smem;
  uint8_t* epi = smem + PG_STAGES * PG_STAGE_BYTES;
  uint64_t* bars = reinterpret_cast<uint64_t*>(epi + PG_EPI_BYTES);
  uint64_t* full = bars;                       // used in the leader only (count 2: both producers)
  uint64_t* empty = bars + PG_STAGES;          // one set per CTA, signalled by the leader's commits
  uint64_t* tfull = bars + 2 * PG_STAGES;      // one set per CTA
  uint64_t* tempty = tfull + 2;                // used in the leader only (count 8: 4 warps x 2 CTAs)
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(tempty + 2);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);

  const int warp = threadIdx.x >> 5;
  const int lane = threadIdx.x & 31;
  const uint32_t rank = cluster_ctarank();
  const int pair = (int)cluster_id_x();
  const int npairs = (int)cluster_count_x();

  // both CTAs are resident before anything touches the peer
  cluster_sync_all();
  if (threadIdx.x == 0) {
    for (int s = 0; s < PG_STAGES; ++s) {
      mbar_init(&full[s], 2);
      mbar_init(&empty[s], 1);
    }
    for (int i = 0; i < 2; ++i) {
      mbar_init(&tfull[i], 1);
      mbar_init(&tempty[i], 8);
    }
    *abort_flag = 0;
    fence_barrier_init();
    tma_prefetch_desc(&tmA);
    tma_prefetch_desc(&tmB);
    tma_prefetch_desc(&tmBh);
    tma_prefetch_desc(&tmC);
  }
  if (warp == 1) {
    tmem_alloc_pair(tmem_slot, PG_TMEM_COLS);
    tmem_relinquish_pair();
  }
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();      // the peer's barriers are initialised, its tensor memory is reserved
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  const int num_units = p.num_units * p.batch;

  if (warp == 0) {
    // ------------------------------------------------------------ TMA producer (both CTAs)
    if (lane == 0) {
      uint32_t it = 0;
      bool ok = true;
      for (int u = pair; u < num_units && ok; u += npairs) {
        int tm, tn, ncol0, width, kb0, kb1, bz;
        pair_decode(p, u, tm, tn, ncol0, width, kb0, kb1, bz);
        const int m0 = tm * (2 * PG_BM) + (int)rank * PG_BM;
        if (p.ag.world > 1) {
          // another rank's rows: present in local memory once their source has raised the chunk's flag
          const int chunk = m0 / PG_BM;
          if (chunk / p.ag.chunks_per_rank != p.ag.rank) {
            if (!wait_flag_sys(p.ag.flags[p.ag.rank] + PG_AG_CHUNK + chunk, p.ag.epoch)) { atomicOr(p.err, 4u); }
            asm volatile("fence.proxy.async;" ::: "memory");         // peer stores (generic proxy) before my TMA reads
          }
        }
        const int bcols = width / 2;                                  // B columns this CTA stages
        const int n0 = tn * PG_BN + ncol0 + (int)rank * bcols;
        const uint32_t my_bytes = PG_A_BYTES + (uint32_t)bcols * PG_BK * 2;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % PG_STAGES;
          const uint32_t ph = (it / PG_STAGES) & 1;
          if (!mbar_wait(&empty[s], ph ^ 1, abort_flag, p.err)) { ok = false; break; }
          uint8_t* sa = ring + s * PG_STAGE_BYTES;
          uint8_t* sb_ = sa + PG_A_BYTES;
          const uint32_t lead_full = map_to_cta(smem_u32(&full[s]), 0);
          const int k0 = kb * PG_BK;
          if (A_MN) {
#pragma unroll
            for (int i = 0; i < PG_BM / 64; ++i) tma_load_3d_pair(sa + i * 8192, &tmA, lead_full, m0 + 64 * i, k0, bz);
          } else {
            tma_load_3d_pair(sa, &tmA, lead_full, k0, m0, bz);
          }
          if (B_MN) {
            for (int i = 0; i < bcols / 64; ++i) tma_load_3d_pair(sb_ + i * 8192, &tmB, lead_full, n0 + 64 * i, k0, bz);
          } else {
            tma_load_3d_pair(sb_, width == PG_BN ? &tmB : &tmBh, lead_full, k0, n0, bz);
          }
          if (rank == 0) mbar_expect_tx(&full[s], 2 * my_bytes);     // arrive + the bytes of both CTAs
          else mbar_arrive_cluster(lead_full);
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
    // ------------------------------------------------------------ MMA issuer (leader CTA only)
    if (lane == 0 && rank == 0) {
      constexpr uint32_t idesc_full = make_idesc_bf16(2 * PG_BM, PG_BN, A_MN ? 1 : 0, B_MN ? 1 : 0);
      constexpr uint32_t idesc_half = make_idesc_bf16(2 * PG_BM, PG_BN / 2, A_MN ? 1 : 0, B_MN ? 1 : 0);
      uint32_t it = 0;
      uint32_t tile_iter = 0;
      bool ok = true;
      for (int u = pair; u < num_units && ok; u += npairs, ++tile_iter) {
        const uint32_t acc = tile_iter & 1;
        const uint32_t acc_ph = (tile_iter >> 1) & 1;
        if (!mbar_wait(&tempty[acc], acc_ph ^ 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t d_tmem = tmem_base + acc * PG_BN;
        int tm_, tn_, ncol0, width, kb0, kb1, bz_;
        pair_decode(p, u, tm_, tn_, ncol0, width, kb0, kb1, bz_);
        const uint32_t idesc = width == PG_BN ? idesc_full : idesc_half;
        for (int kb = kb0; kb < kb1; ++kb, ++it) {
          const int s = it % PG_STAGES;
          const uint32_t ph = (it / PG_STAGES) & 1;
          if (!mbar_wait(&full[s], ph, abort_flag, p.err)) { ok = false; break; }
          tc_fence_after();
          const uint32_t a_base = smem_u32(ring + s * PG_STAGE_BYTES);
          const uint32_t b_base = a_base + PG_A_BYTES;
#pragma unroll
          for (int kk = 0; kk < PG_BK / 16; ++kk) {
            const uint64_t da = A_MN ? make_smem_desc_sw128(a_base + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(a_base + kk * 32, 16, 1024);
            const uint64_t db = B_MN ? make_smem_desc_sw128(b_base + kk * 2048, 8192, 1024)
                                     : make_smem_desc_sw128(b_base + kk * 32, 16, 1024);
            umma_bf16_pair(d_tmem, da, db, idesc, (kb > kb0 || kk > 0) ? 1u : 0u);
          }
          umma_commit_pair(&empty[s], 3);
        }
        if (ok) umma_commit_pair(&tfull[acc], 3);
      }
    }
    __syncwarp();
  } else if (warp < 6) {
    // ------------------------------------------------------------ epilogue (warps 2..5, both CTAs)
    const int q = warp & 3;                       // TMEM lane quadrant this warp may read
    uint8_t* stage_buf = epi + q * 8192;
    uint32_t tile_iter = 0;
    uint32_t buf = 0;
    bool ok = true;
    constexpr int CHUNK_COLS = (OUT == 0) ? 64 : 32;   // 128 bytes per row per chunk
    for (int u = pair; u < num_units && ok; u += npairs, ++tile_iter) {
      int tm, tn, ncol0, width, kb0, kb1, bz;
      pair_decode(p, u, tm, tn, ncol0, width, kb0, kb1, bz);
      const int m0 = tm * (2 * PG_BM) + (int)rank * PG_BM;
      const int n0 = tn * PG_BN + ncol0;
      const uint32_t acc = tile_iter & 1;
      const uint32_t acc_ph = (tile_iter >> 1) & 1;
      if (!mbar_wait(&tfull[acc], acc_ph, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      const uint32_t t_row = tmem_base + acc * PG_BN + (static_cast<uint32_t>(q * 32) << 16);
      const int nchunks = width / CHUNK_COLS;
      for (int c = 0; c < nchunks; ++c) {
        const int col0 = n0 + c * CHUNK_COLS;
        if (col0 >= p.N || m0 >= p.M) break;      // nothing to store
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
        if (OUT == 0) {
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
          if (OUT == 2) tma_reduce_add_3d(&tmC, stage_buf + buf * 4096, col0, m0 + q * 32, bz);
          else tma_store_3d(&tmC, stage_buf + buf * 4096, col0, m0 + q * 32, bz);
          tma_store_commit();
        }
        buf ^= 1;
      }
      // accumulator fully read: hand the buffer back to the leader's MMA thread
      tc_fence_before();
      __syncwarp();
      if (lane == 0) mbar_arrive_cluster(map_to_cta(smem_u32(&tempty[acc]), 0));
    }
    if (lane == 0) tma_store_wait_all<0>();
  } else if (p.ag.world > 1) {
    // ------------------------------------------------------------ all-gather role: warp 6 pushes this rank's rows
    // while the other warps already compute the own tile rows; its fences stall nobody but itself
    const PairAg& ag = p.ag;
    // a peer's buffer may be overwritten only after that peer has finished reading it in the previous call
    if (lane < ag.world && lane != ag.rank && !wait_flag_sys(ag.flags[ag.rank] + PG_AG_DONE + lane, ag.epoch - 1))
      atomicOr(p.err, 4u);
    __syncwarp();
    // Up to four rounds: in round r the CTAs, split into teams, push chunks r T .. r T + T - 1 (one per team).
    // The chunks of every source then reach a destination roughly in chunk order (its ingress is shared by all
    // sources), which is the order in which the tile loop asks for them, at the price of one system-scope
    // fence per round instead of one per kernel.
    const long nvec = ag.chunk_bytes >> 4;
    const int rounds = ag.world <= 2 ? 1 : (ag.chunks_per_rank < 4 ? ag.chunks_per_rank : 4);   // one source: nothing to order
    const int teams = (ag.chunks_per_rank + rounds - 1) / rounds;
    const int team = blockIdx.x % teams, ci = blockIdx.x / teams;
    const int gsz = ((int)gridDim.x - team + teams - 1) / teams;          // CTAs of my team
    for (int r = 0; r < rounds; ++r) {
      const int c = r * teams + team;
      if (c >= ag.chunks_per_rank) break;
      const long off0 = ((long)ag.rank * ag.chunks_per_rank + c) * ag.chunk_bytes;
      const uint4* src = reinterpret_cast<const uint4*>(ag.xfull[ag.rank] + off0);
      const long stride = (long)gsz * 32;
      for (long v0 = (long)ci * 32 + lane; v0 < nvec; v0 += 8 * stride) {
        uint4 w[8];                                  // eight loads in flight per lane
#pragma unroll
        for (int i = 0; i < 8; ++i)
          if (v0 + i * stride < nvec) w[i] = src[v0 + i * stride];
#pragma unroll
        for (int i = 0; i < 8; ++i) {
          const long v = v0 + i * stride;
          if (v >= nvec) break;
          if (ag.xmc != nullptr) {
            asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                             reinterpret_cast<uint4*>(ag.xmc + off0) + v),
                         "f"(__uint_as_float(w[i].x)), "f"(__uint_as_float(w[i].y)), "f"(__uint_as_float(w[i].z)),
                         "f"(__uint_as_float(w[i].w))
                         : "memory");
          } else {
            for (int s = 1; s < ag.world; ++s) {
              int dst = ag.rank + s;
              if (dst >= ag.world) dst -= ag.world;
              reinterpret_cast<uint4*>(ag.xfull[dst] + off0)[v] = w[i];
            }
          }
        }
      }
      __syncwarp();
      __threadfence_system();                        // every lane's stores have been performed at the peers
      __syncwarp();
      if (lane == 0) {
        if (atomicAdd(ag.counters + c, 1u) == (unsigned)gsz - 1) {        // the chunk's last CTA tells every peer
          ag.counters[c] = 0;
          for (int pr = 0; pr < ag.world; ++pr)
            if (pr != ag.rank) st_release_sys_u32(ag.flags[pr] + PG_AG_CHUNK + ag.rank * ag.chunks_per_rank + c, ag.epoch);
        }
      }
    }
  }

  // No CTA may leave while its peer can still signal its barriers or write its tensor memory.
  tc_fence_before();
  __syncthreads();
  cluster_sync_all();
  if (warp == 1) {
    tc_fence_after();
    tmem_dealloc_pair(tmem_base, PG_TMEM_COLS);
  }
  if (p.ag.world > 1 && threadIdx.x == 0) {
    // the last CTA of the grid: every read of this rank's buffer has completed, peers may overwrite it
    __threadfence();
    unsigned int* exit_counter = p.ag.counters + p.ag.chunks_per_rank;
    if (atomicAdd(exit_counter, 1u) == gridDim.x - 1) {
      *exit_counter = 0;
      for (int pr = 0; pr < p.ag.world; ++pr)
        if (pr != p.ag.rank) st_release_sys_u32(p.ag.flags[pr] + PG_AG_DONE + p.ag.rank, p.ag.epoch);
    }
  }
}

static int pair_tmap(CUtensorMap* m, const void* base, int elem, uint64_t inner, uint64_t outer, uint64_t batch,
                     uint64_t pitch_bytes, uint64_t batch_stride_bytes, uint32_t box_inner, uint32_t box_outer, bool f32) {
  uint64_t dims[3] = {inner, outer, batch};
  uint64_t strides[2] = {pitch_bytes, batch > 1 ? batch_stride_bytes : pitch_bytes * outer};
  uint32_t box[3] = {box_inner, box_outer, 1};
  return make_tmap(m, base, elem, 3, dims, strides, box, true, f32);
}

template <bool A_MN, bool B_MN, int OUT>
static int launch_pair(const void* A, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N, int K,
                       int lda, int ldb, int ldc, int batch, long sa, long sb_, long sc, cudaStream_t stream,
                       const PairAg* ag = nullptr) {
  CUtensorMap tmA, tmB, tmBh, tmC;
  int rc;
  const uint64_t nb = (uint64_t)batch;
  if (A_MN) rc = pair_tmap(&tmA, A, 2, M, K, nb, (uint64_t)lda * 2, (uint64_t)sa * 2, 64, 64, false);
  else      rc = pair_tmap(&tmA, A, 2, K, M, nb, (uint64_t)lda * 2, (uint64_t)sa * 2, 64, PG_BM, false);
  if (rc) return rc;
  if (B_MN) {
    rc = pair_tmap(&tmB, B, 2, N, K, nb, (uint64_t)ldb * 2, (uint64_t)sb_ * 2, 64, 64, false);
    tmBh = tmB;
  } else {
    rc = pair_tmap(&tmB, B, 2, K, N, nb, (uint64_t)ldb * 2, (uint64_t)sb_ * 2, 64, PG_BN / 2, false);
    if (rc) return rc;
    rc = pair_tmap(&tmBh, B, 2, K, N, nb, (uint64_t)ldb * 2, (uint64_t)sb_ * 2, 64, PG_BN / 4, false);
  }
  if (rc) return rc;
  if (OUT == 0) rc = pair_tmap(&tmC, C, 2, N, M, nb, (uint64_t)ldc * 2, (uint64_t)sc * 2, 64, 32, false);
  else          rc = pair_tmap(&tmC, C, 4, N, M, nb, (uint64_t)ldc * 4, (uint64_t)sc * 4, 32, 32, true);
  if (rc) return rc;

  auto kern = gemm_pair_kernel<A_MN, B_MN, OUT>;
  static int max_pairs[64] = {0};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  SB_CHECK_ARG(dev >= 0 && dev < 64);
  if (max_pairs[dev] == 0) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, PG_SMEM_BYTES));
    // how many pairs the device can hold at once (a persistent grid must not be larger)
    cudaLaunchConfig_t cfg;
    memset(&cfg, 0, sizeof(cfg));
    cfg.gridDim = dim3((unsigned)num_sms() & ~1u);
    cfg.blockDim = dim3(PG_THREADS);
    cfg.dynamicSmemBytes = PG_SMEM_BYTES;
    cudaLaunchAttribute attr;
    attr.id = cudaLaunchAttributeClusterDimension;
    attr.val.clusterDim.x = 2; attr.val.clusterDim.y = 1; attr.val.clusterDim.z = 1;
    cfg.attrs = &attr;
    cfg.numAttrs = 1;
    int n = 0;
    if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess || n <= 0) {
      cudaGetLastError();
      n = num_sms() / 2;
    }
    if (n > num_sms() / 2) n = num_sms() / 2;
    if (const char* lim = getenv("SUMMA_PAIR_LIMIT")) { const int l = atoi(lim); if (l > 0 && l < n) n = l; }
    if (getenv("SUMMA_PAIR_DEBUG")) fprintf(stderr, "summa_b200: gemm_pair: %d resident pairs on %d SMs\n", n, num_sms());
    max_pairs[dev] = n;
  }
  const int pairs = max_pairs[dev];

  PairParams p;
  p.group_m = PG_GROUP_M;
  memset(&p.ag, 0, sizeof(p.ag));
  if (ag != nullptr) {
    p.ag = *ag;
    // raster groups never straddle the boundary between the own tile rows and the others
    const int tpr = ag->chunks_per_rank / 2;
    p.group_m = (tpr >= PG_GROUP_M && tpr % PG_GROUP_M == 0) ? PG_GROUP_M : tpr;
  }
  p.M = M; p.N = N; p.K = K;
  p.tiles_m = (M + 2 * PG_BM - 1) / (2 * PG_BM);
  p.tiles_n = (N + PG_BN - 1) / PG_BN;
  p.num_tiles = p.tiles_m * p.tiles_n;
  p.k_blocks = (K + PG_BK - 1) / PG_BK;
  p.splits = 1;
  p.batch = batch;
  if (OUT == 2 && bias == nullptr && batch == 1) {
    // fp32 reduce-add output: the contraction may be cut anywhere; pick the split count that
    // fills whole waves of the persistent grid best (each split costs one more pass over C)
    const int max_by_k = p.k_blocks / 8 > 0 ? p.k_blocks / 8 : 1;
    double best_cost = 1e30;
    for (int s = 1; s <= max_by_k && s <= 32; ++s) {
      const long units = (long)p.num_tiles * s;
      const long waves = (units + pairs - 1) / pairs;
      const double kb = (double)((p.k_blocks + s - 1) / s);
      const double cost = waves * (kb + 4.0);
      if (cost < best_cost * 0.97) { best_cost = cost; p.splits = s; }
    }
  }
  p.kb_per_split = (p.k_blocks + p.splits - 1) / p.splits;
  p.splits = (p.k_blocks + p.kb_per_split - 1) / p.kb_per_split;
  p.first_half_tile = p.num_tiles;
  if (p.splits == 1 && N % PG_BN == 0 && batch == 1) {
    const int rem = p.num_tiles % pairs;
    if (rem != 0 && 2 * rem <= pairs) p.first_half_tile = p.num_tiles - rem;
  }
  p.num_full_units = p.first_half_tile * p.splits;
  p.num_units = p.num_full_units + 2 * (p.num_tiles - p.first_half_tile);
  p.bias = bias;
  p.bias_is_bf16 = bias_is_bf16;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  const long all_units = (long)p.num_units * batch;
  const int grid_pairs = all_units < pairs ? (int)all_units : pairs;
  // the all-gather role adds a seventh warp (the pusher)
  kern<<<2 * grid_pairs, PG_THREADS + (ag != nullptr ? 32 : 0), PG_SMEM_BYTES, stream>>>(tmA, tmB, tmBh, tmC, p);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

template <int OUT>
static int pair_dispatch_major(int a_mn, int b_mn, const void* A, const void* B, void* C, const void* bias,
                               int bias_is_bf16, int M, int N, int K, int lda, int ldb, int ldc, int batch, long sa,
                               long sb_, long sc, cudaStream_t st) {
  if (!a_mn && !b_mn) return launch_pair<false, false, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, sa, sb_, sc, st);
  if (!a_mn && b_mn) return launch_pair<false, true, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, sa, sb_, sc, st);
  if (a_mn && !b_mn) return launch_pair<true, false, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, sa, sb_, sc, st);
  return launch_pair<true, true, OUT>(A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, sa, sb_, sc, st);
}

int gemm_pair_bf16(const void* A, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N, int K,
                   int lda, int ldb, int ldc, int a_mn, int b_mn, int out_mode, cudaStream_t stream, int batch,
                   long stride_a, long stride_b, long stride_c) {
  if (out_mode == 0) return pair_dispatch_major<0>(a_mn, b_mn, A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, stride_a, stride_b, stride_c, stream);
  if (out_mode == 1) return pair_dispatch_major<1>(a_mn, b_mn, A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, stride_a, stride_b, stride_c, stream);
  return pair_dispatch_major<2>(a_mn, b_mn, A, B, C, bias, bias_is_bf16, M, N, K, lda, ldb, ldc, batch, stride_a, stride_b, stride_c, stream);
}

int gemm_pair_ag(const PairAg& ag, const void* B, void* C, const void* bias, int bias_is_bf16, int M, int N, int K,
                 int ldb, int ldc, int b_mn, cudaStream_t stream) {
  if (b_mn) return launch_pair<false, true, 0>(ag.xfull[ag.rank], B, C, bias, bias_is_bf16, M, N, K, K, ldb, ldc, 1, 0, 0, 0, stream, &ag);
  return launch_pair<false, false, 0>(ag.xfull[ag.rank], B, C, bias, bias_is_bf16, M, N, K, K, ldb, ldc, 1, 0, 0, 0, stream, &ag);
}

}  // namespace sb

// All-gather -> GEMM on the paired-CTA kernel. xfull[r]: rank r's `[M, K]` bf16 activation buffer (row pitch K)
// in symmetric memory, of which rank r has written ITS rows [r M / P, (r + 1) M / P) before the call; xmc: the
// buffers' multicast address or null; flags[r]: rank r's flag array in symmetric memory (8 + M / 128 words, zero
// at start); counters: local, M / P / 128 + 1 words, zero at start; epoch: 1, 2, ... per call of this entry on
// every rank. C[M, N] = gather(X) * B (+ bias), B `[K, N]` (b_mn = 1) or `[N, K]` (b_mn = 0), local.
// Requires M % (256 * world) == 0, K % 64 == 0, N % 8 == 0, world <= 8.
extern "C" int sb_tp_ag_gemm_pair(const void* const* xfull, const void* xmc, const void* B, void* C, const void* bias,
                                  int bias_is_bf16, const void* const* flags, void* counters, int M, int N, int K,
                                  int ldb, int ldc, int b_mn, int rank, int world, unsigned int epoch,
                                  cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(world >= 2 && world <= PG_AG_MAX && rank >= 0 && rank < world && epoch >= 1);
  SB_CHECK_ARG(M > 0 && M % (2 * PG_BM * world) == 0 && K % 64 == 0 && N % 8 == 0 && ldb % 8 == 0 && ldc % 8 == 0);
  PairAg ag;
  memset(&ag, 0, sizeof(ag));
  ag.world = world; ag.rank = rank; ag.epoch = epoch;
  ag.chunks_per_rank = M / world / PG_BM;
  ag.chunk_bytes = (long)PG_BM * K * 2;
  for (int i = 0; i < world; ++i) { ag.xfull[i] = (uint8_t*)xfull[i]; ag.flags[i] = (uint32_t*)flags[i]; }
  ag.xmc = (uint8_t*)xmc;
  ag.counters = (unsigned int*)counters;
  return gemm_pair_ag(ag, B, C, bias, bias_is_bf16, M, N, K, ldb, ldc, b_mn, stream);
}

// Batched GEMM on the paired-CTA kernel: `batch` independent problems of one shape, problem i at
// A + i * stride_a, B + i * stride_b, C + i * stride_c (strides in elements, positive multiples of 8). Layout flags, leading dimensions and out_mode as in sb_gemm_bf16.
extern "C" int sb_gemm_bf16_batched(const void* A, const void* B, void* C, int batch, long stride_a, long stride_b,
                                    long stride_c, int M, int N, int K, int lda, int ldb, int ldc, int a_mn, int b_mn,
                                    int out_mode, cudaStream_t stream) {
  using namespace sb;
  SB_CHECK_ARG(batch >= 1 && batch <= 65535 && M > 0 && N > 0 && K > 0);
  SB_CHECK_ARG(lda % 8 == 0 && ldb % 8 == 0 && out_mode >= 0 && out_mode <= 2);
  SB_CHECK_ARG(out_mode == 0 ? (ldc % 8 == 0) : (ldc % 4 == 0));
  SB_CHECK_ARG(stride_a % 8 == 0 && stride_b % 8 == 0 && stride_c % 8 == 0 && stride_a > 0 && stride_b > 0 && stride_c > 0);
  return gemm_pair_bf16(A, B, C, nullptr, 0, M, N, K, lda, ldb, ldc, a_mn, b_mn, out_mode, stream, batch, stride_a,
                        stride_b, stride_c);
}
