// Expert-parallel dispatch / return over NVLink peer memory (symmetric buffers, flags with
// bounded waits). Experts are sharded by contiguous blocks: rank o owns experts
// [o*El, (o+1)*El). Every rank routes its own tokens over ALL experts (the local plan of
// moe.cu: routes sorted by expert, each expert's rows padded to 128 = the "source layout").
//
//   ep_counts    every rank publishes its per-expert route counts to all peers (P x E ints)
//   ep_dispatch  waits for the count matrix, then pushes each routed row straight from the
//                token activation (gather fused with the send) or from a source-layout buffer
//                (backward) into its final row of the owner's compact buffer:
//                   owner row = opoff[el] + sum_{s < src} count_s[e] + j
//                where opoff pads every local expert to 128 rows. Nothing is staged.
//   ep_meta      on the owner: waits for all sources' data flags, builds the grouped-GEMM
//                metadata of the compact layout (tile -> expert, live tiles, padded offsets)
//                and zeroes the padding rows
//   ep_return    pushes every compact output row back into the source-layout buffer of the rank
//                it came from (row = spoff_src[e] + j), then flags
//   ep_wait      on the source: waits for all owners' return flags
// All layouts derive from the same count matrix, so no per-row metadata crosses the link.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int EP_MAX_RANKS = 8;
constexpr int EP_MAX_EXPERTS = 256;
constexpr int SIG_EP_COUNT = 0, SIG_EP_DATA = 8, SIG_EP_RET = 16;     // words of the EP signal pad

struct EpPeers {
  uint8_t* recv[EP_MAX_RANKS];      // compact buffer of every rank (dispatch destination)
  uint8_t* ret[EP_MAX_RANKS];       // source-layout buffer of every rank (return destination)
  int* count_mat[EP_MAX_RANKS];     // [P][E] on every rank
  uint32_t* sig[EP_MAX_RANKS];
};

__device__ __forceinline__ int pad128(int n) { return (n + 127) & ~127; }

__global__ void ep_counts_kernel(EpPeers peers, const int* __restrict__ counts, int E, int rank, int world, uint32_t epoch) {
  for (int pr = 0; pr < world; ++pr)
    for (int e = threadIdx.x; e < E; e += blockDim.x) peers.count_mat[pr][rank * E + e] = counts[e];
  __threadfence_system();
  __syncthreads();
  if (threadIdx.x < world) st_release_sys_u32(peers.sig[threadIdx.x] + SIG_EP_COUNT + rank, epoch);
}

// Shared tables built by every CTA of the dispatch / return kernels from the count matrix.
struct EpTables {
  int before[EP_MAX_EXPERTS];       // rows of ranks < me for expert e
  int total[EP_MAX_EXPERTS];        // rows of all ranks for expert e
  int opoff[EP_MAX_EXPERTS];        // padded offset of expert e inside ITS OWNER's compact layout
  int over[EP_MAX_RANKS];           // owner o's padded rows exceed its compact buffer: nothing may be sent to it
};

__device__ __forceinline__ bool ep_wait_flags(const uint32_t* sig, int base, int world, uint32_t epoch, unsigned int* err) {
  __shared__ int ok_s;
  __syncthreads();            // a previous call's result has been read by every thread before it is reset
  if (threadIdx.x == 0) ok_s = 1;
  __syncthreads();
  if ((int)threadIdx.x < world) {
    if (!wait_flag_sys(sig + base + threadIdx.x, epoch)) { atomicOr(err, 16u); ok_s = 0; }
  }
  __syncthreads();
  return ok_s != 0;
}

__device__ __forceinline__ void ep_build_tables(EpTables& tb, const int* count_mat, int E, int El, int rank, int world,
                                                int owner_rows = 0x7fffffff) {
  for (int e = threadIdx.x; e < E; e += blockDim.x) {
    int before = 0, total = 0;
    for (int s = 0; s < world; ++s) {
      const int c = count_mat[s * E + e];
      if (s < rank) before += c;
      total += c;
    }
    tb.before[e] = before;
    tb.total[e] = total;
  }
  __syncthreads();
  if ((int)threadIdx.x < world) {          // one thread per owner: prefix over its local experts
    int off = 0;
    for (int el = 0; el < El; ++el) {
      const int e = threadIdx.x * El + el;
      tb.opoff[e] = off;
      off += pad128(tb.total[e]);
    }
    tb.over[threadIdx.x] = off > owner_rows ? 1 : 0;
  }
  __syncthreads();
}

// One warp per source-layout row. src_tokens != null: row data = x[token(row)] (row_route holds
// token * k + slot); otherwise row data = src_rows[row] (a buffer already in source layout).
__global__ void __launch_bounds__(256)
ep_dispatch_kernel(EpPeers peers, const __nv_bfloat16* __restrict__ x, long ldx, const __nv_bfloat16* __restrict__ src_rows,
                   const int* __restrict__ row_route, const int* __restrict__ meta, const int* __restrict__ tile_expert,
                   const int* __restrict__ counts, int E, int El, int H, int k, int rank, int world, uint32_t epoch,
                   unsigned int* counter, unsigned int* err, int owner_rows) {
  __shared__ EpTables tb;
  const bool ok = ep_wait_flags(peers.sig[rank], SIG_EP_COUNT, world, epoch, err);
  if (ok) {
    // Every rank derives every owner's layout from the same count matrix. An owner whose padded rows do
    // not fit its compact buffer (`owner_rows`) receives NOTHING (it exposes no rows either, see ep_meta):
    // a peer store must never leave the buffer it was sized for.
    ep_build_tables(tb, peers.count_mat[rank], E, El, rank, world, owner_rows);
    if (blockIdx.x == 0 && (int)threadIdx.x < world && tb.over[threadIdx.x]) atomicOr(err, 32u);
    const int live_rows = meta[E];
    const int lane = threadIdx.x & 31;
    const int warps = (gridDim.x * blockDim.x) >> 5;
    for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < live_rows; row += warps) {
      const int e = tile_expert[row >> 7];
      const int j = row - meta[e];
      if (j >= counts[e]) continue;                                   // padding of the source layout
      const int owner = e / El;
      if (tb.over[owner]) continue;
      const long dst_row = tb.opoff[e] + tb.before[e] + j;
      const uint4* src = x != nullptr ? reinterpret_cast<const uint4*>(x + (long)(row_route[row] / k) * ldx)
                                      : reinterpret_cast<const uint4*>(src_rows + (long)row * H);
      uint4* dst = reinterpret_cast<uint4*>(peers.recv[owner] + dst_row * H * 2);
      for (int c = lane; c < H / 8; c += 32) dst[c] = src[c];
    }
  }
  // arrival: the last CTA tells every owner that this rank's rows are in place
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      *counter = 0;
      __threadfence_system();
      for (int pr = 0; pr < world; ++pr) st_release_sys_u32(peers.sig[pr] + SIG_EP_DATA + rank, epoch);
    }
  }
}

// Owner side, one CTA. out_meta has the layout of the local plan's meta for El experts:
// [0..El] padded offsets, [El+1] live 128-row tiles; out_counts[el] = rows of local expert el.
__global__ void __launch_bounds__(256)
ep_meta_kernel(EpPeers peers, int* __restrict__ out_meta, int* __restrict__ out_tile_expert, int* __restrict__ out_counts,
               __nv_bfloat16* __restrict__ recv, int E, int El, int H, int max_tiles, int rank, int world, uint32_t epoch,
               unsigned int* err) {
  __shared__ EpTables tb;
  bool ok = ep_wait_flags(peers.sig[rank], SIG_EP_COUNT, world, epoch, err);
  ok = ep_wait_flags(peers.sig[rank], SIG_EP_DATA, world, epoch, err) && ok;
  ep_build_tables(tb, peers.count_mat[rank], E, El, rank, world);
  __shared__ int end_s;
  if (threadIdx.x == 0) {
    int off = 0;
    for (int el = 0; el < El; ++el) {
      const int e = rank * El + el;
      out_meta[el] = off;
      out_counts[el] = ok ? tb.total[e] : 0;
      off += ok ? pad128(tb.total[e]) : 0;
    }
    if (off > max_tiles * 128) {        // capacity exceeded: expose nothing, and say so consistently
      off = 0;
      atomicOr(err, 32u);
      for (int el = 0; el < El; ++el) { out_meta[el] = 0; out_counts[el] = 0; }
    }
    out_meta[El] = off;
    out_meta[El + 1] = off / 128;
    end_s = off;
  }
  __syncthreads();
  const int end = end_s;
  for (int t = threadIdx.x; t < max_tiles; t += blockDim.x) {
    int ex = 0;
    if (t * 128 < end) {
      for (int el = 0; el < El; ++el)
        if (t * 128 >= out_meta[el]) ex = el;
    }
    out_tile_expert[t] = ex;
  }
  // zero the padding rows (fewer than 128 per expert) so that contractions over padded ranges stay exact
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int el = 0; el < El && end > 0; ++el) {
    const int e = rank * El + el;
    const int r0 = out_meta[el] + tb.total[e], r1 = out_meta[el] + pad128(tb.total[e]);
    for (int r = r0 + warp; r < r1; r += 8) {
      uint4* dst = reinterpret_cast<uint4*>(recv + (long)r * H);
      for (int c = lane; c < H / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    }
  }
}

// One warp per compact row: y[row] -> ret buffer of the rank the row came from.
__global__ void __launch_bounds__(256)
ep_return_kernel(EpPeers peers, const __nv_bfloat16* __restrict__ y, const int* __restrict__ meta,
                 const int* __restrict__ tile_expert, int E, int El, int H, int rank, int world, uint32_t epoch,
                 unsigned int* counter) {
  __shared__ int cnt[EP_MAX_RANKS][64];            // count_s[e] for my experts (El <= 64)
  __shared__ int spoff[EP_MAX_RANKS][64];          // source-layout padded offset of my experts on rank s
  const int* cm = peers.count_mat[rank];
  if ((int)threadIdx.x < world) {
    const int s = threadIdx.x;
    int off = 0;
    for (int e = 0; e < E; ++e) {
      const int c = cm[s * E + e];
      if (e / El == rank) { cnt[s][e - rank * El] = c; spoff[s][e - rank * El] = off; }
      off += pad128(c);
    }
  }
  __syncthreads();
  const int live_rows = meta[El];
  const int lane = threadIdx.x & 31;
  const int warps = (gridDim.x * blockDim.x) >> 5;
  for (int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5; row < live_rows; row += warps) {
    const int el = tile_expert[row >> 7];
    int q = row - meta[el];
    int s = 0;
    while (s < world && q >= cnt[s][el]) { q -= cnt[s][el]; ++s; }
    if (s >= world) continue;                                         // padding row
    const long dst_row = spoff[s][el] + q;
    const uint4* src = reinterpret_cast<const uint4*>(y + (long)row * H);
    uint4* dst = reinterpret_cast<uint4*>(peers.ret[s] + dst_row * H * 2);
    for (int c = lane; c < H / 8; c += 32) dst[c] = src[c];
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    if (atomicAdd(counter, 1u) == gridDim.x - 1) {
      *counter = 0;
      __threadfence_system();
      for (int pr = 0; pr < world; ++pr) st_release_sys_u32(peers.sig[pr] + SIG_EP_RET + rank, epoch);
    }
  }
}

__global__ void ep_wait_kernel(EpPeers peers, int rank, int world, uint32_t epoch, unsigned int* err) {
  ep_wait_flags(peers.sig[rank], SIG_EP_RET, world, epoch, err);
}

static int ep_fill(EpPeers& p, const void* const* recv, const void* const* ret, const void* const* count_mat,
                   const void* const* sig, int world) {
  for (int i = 0; i < EP_MAX_RANKS; ++i) { p.recv[i] = nullptr; p.ret[i] = nullptr; p.count_mat[i] = nullptr; p.sig[i] = nullptr; }
  for (int i = 0; i < world; ++i) {
    p.recv[i] = (uint8_t*)recv[i]; p.ret[i] = (uint8_t*)ret[i]; p.count_mat[i] = (int*)count_mat[i]; p.sig[i] = (uint32_t*)sig[i];
  }
  return SB_OK;
}

static unsigned int* ep_counter(int which) {
  static unsigned int* counters[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
  if (!counters[dev]) {
    if (cudaMalloc(&counters[dev], 16 * sizeof(unsigned int)) != cudaSuccess) return nullptr;
    cudaMemset(counters[dev], 0, 16 * sizeof(unsigned int));
  }
  return counters[dev] + which;
}

}  // namespace sb

using namespace sb;

#define EP_COMMON_ARGS const void* const* recv, const void* const* ret, const void* const* count_mat, const void* const* sig
#define EP_CHECK_COMMON                                                                                   \
  SB_CHECK_ARG(world >= 1 && world <= EP_MAX_RANKS && rank >= 0 && rank < world);                         \
  SB_CHECK_ARG(E > 0 && E <= EP_MAX_EXPERTS && E % world == 0 && E / world <= 64);                        \
  EpPeers peers;                                                                                          \
  ep_fill(peers, recv, ret, count_mat, sig, world);                                                       \
  unsigned int* err = error_word();                                                                       \
  if (!err) return SB_ERR_CUDA

// counts: this rank's per-expert route counts (device, from the local plan).
extern "C" int sb_ep_counts(EP_COMMON_ARGS, const int* counts, int E, int rank, int world, unsigned int epoch,
                            cudaStream_t st) {
  EP_CHECK_COMMON;
  ep_counts_kernel<<<1, 256, 0, st>>>(peers, counts, E, rank, world, epoch);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Push this rank's routed rows to their owners. x != null: gather from the token activation
// `[T, H]` (row stride ldx); else copy from src_rows (source layout `[rows, H]`). owner_rows: rows of
// every rank's compact buffer (the same on all ranks); an owner that would overflow is sent nothing.
extern "C" int sb_ep_dispatch(EP_COMMON_ARGS, const void* x, long ldx, const void* src_rows, const int* row_route,
                              const int* meta, const int* tile_expert, const int* counts, int max_rows, int E, int H, int k,
                              int rank, int world, unsigned int epoch, int owner_rows, cudaStream_t st) {
  EP_CHECK_COMMON;
  SB_CHECK_ARG(H % 8 == 0 && max_rows > 0 && owner_rows > 0 && (x != nullptr || src_rows != nullptr));
  unsigned int* counter = ep_counter(0);
  if (!counter) return SB_ERR_CUDA;
  long blocks = ((long)max_rows + 7) / 8;
  if (blocks > 4L * num_sms()) blocks = 4L * num_sms();
  ep_dispatch_kernel<<<(int)blocks, 256, 0, st>>>(peers, (const __nv_bfloat16*)x, ldx, (const __nv_bfloat16*)src_rows,
                                                  row_route, meta, tile_expert, counts, E, E / world, H, k, rank, world,
                                                  epoch, counter, err, owner_rows);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Owner: wait for every source's rows and build the compact layout's metadata (out_meta:
// El + 2 ints, out_tile_expert: max_tiles ints, out_counts: El ints). recv_local is this
// rank's compact buffer `[max_tiles * 128, H]`.
extern "C" int sb_ep_meta(EP_COMMON_ARGS, int* out_meta, int* out_tile_expert, int* out_counts, void* recv_local, int E,
                          int H, int max_tiles, int rank, int world, unsigned int epoch, cudaStream_t st) {
  EP_CHECK_COMMON;
  ep_meta_kernel<<<1, 256, 0, st>>>(peers, out_meta, out_tile_expert, out_counts, (__nv_bfloat16*)recv_local, E, E / world,
                                    H, max_tiles, rank, world, epoch, err);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Owner: push the compact rows of y `[rows, H]` back to the ranks they came from.
extern "C" int sb_ep_return(EP_COMMON_ARGS, const void* y, const int* meta, const int* tile_expert, int max_rows, int E,
                            int H, int rank, int world, unsigned int epoch, cudaStream_t st) {
  EP_CHECK_COMMON;
  SB_CHECK_ARG(H % 8 == 0 && max_rows > 0);
  unsigned int* counter = ep_counter(1);
  if (!counter) return SB_ERR_CUDA;
  long blocks = ((long)max_rows + 7) / 8;
  if (blocks > 4L * num_sms()) blocks = 4L * num_sms();
  ep_return_kernel<<<(int)blocks, 256, 0, st>>>(peers, (const __nv_bfloat16*)y, meta, tile_expert, E, E / world, H, rank,
                                                world, epoch, counter);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Source: wait until every owner has returned this rank's rows.
extern "C" int sb_ep_wait_return(EP_COMMON_ARGS, int E, int rank, int world, unsigned int epoch, cudaStream_t st) {
  EP_CHECK_COMMON;
  ep_wait_kernel<<<1, 32, 0, st>>>(peers, rank, world, epoch, err);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
