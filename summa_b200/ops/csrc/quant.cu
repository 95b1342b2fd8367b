// Group-quantised 4-bit weights (group 128 along the input dimension, bf16 scales).
//   packed `[K/2, N]` uint8: byte (k2, n) holds k = 2*k2 in the low nibble and k = 2*k2+1
//   in the high nibble, code q in [0, 15] meaning (q - 8) * scale[k / 128, n].
// Kernels:
//   int4_gemv      y[M,N] (+)= x[M,K] @ dequant(W) for decode-sized M (<= 8 rows per pass),
//                  split over K across blocks (fp32 atomics into a zeroed accumulator) so
//                  that even a tensor-parallel weight shard fills the GPU; the weight is
//                  read exactly once per pass in 4-byte lanes (coalesced along N)
//   w4a16_gemm     the same product for M <= 64 on the tensor cores, over the REPACKED weight
//                  (`[K/8, N]` uint32: the 8 codes of 8 consecutive k for one column, even k in the
//                  low half-word and odd k in the high half-word, nibble i of each half = pair i, so
//                  `(w >> 4i) & 0x000F000F | 0x43004300` is the bf16 pair (128+q_2i, 128+q_2i+1)): the
//                  tile streams in through TMA, the threads expand it to bf16 in registers and hand
//                  it to tcgen05.mma as the A operand through TENSOR MEMORY (no swizzled smem
//                  round trip); x is the B operand (N = M padded to 16/32/64); split over K,
//                  fp32 atomics into the accumulator. One weight pass serves the whole batch.
//   int4_finish    accumulator -> bf16 (+ optional residual)
//   int4_dequant   packed -> bf16 `[K, N]` for the prefill path (tensor-core GEMM)
//   argmax_rows    greedy sampling: argmax over the vocabulary per row
#include <cooperative_groups.h>

#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int GV_KSLICE = 512;     // k range per block (4 groups)
constexpr int GV_MAXM = 8;

// grid: (ceil(N / 512), K / GV_KSLICE, ceil(M / 8)); block 128 threads, thread = 4 columns
__global__ void __launch_bounds__(128)
int4_gemv_kernel(const __nv_bfloat16* __restrict__ x, const uint8_t* __restrict__ packed,
                 const __nv_bfloat16* __restrict__ scales, float* __restrict__ acc_out, int M, int N, int K, long ldx) {
  __shared__ float xs[GV_MAXM][GV_KSLICE];
  const int n0 = (blockIdx.x * 128 + threadIdx.x) * 4;
  const int k0 = blockIdx.y * GV_KSLICE;
  const int m0 = blockIdx.z * GV_MAXM;
  const int mrows = min(GV_MAXM, M - m0);
  for (int i = threadIdx.x; i < GV_MAXM * GV_KSLICE; i += 128) {
    const int m = i / GV_KSLICE, k = i % GV_KSLICE;
    xs[m][k] = (m < mrows && k0 + k < K) ? __bfloat162float(x[(long)(m0 + m) * ldx + k0 + k]) : 0.f;
  }
  __syncthreads();
  if (n0 >= N) return;
  float acc[GV_MAXM][4];
#pragma unroll
  for (int m = 0; m < GV_MAXM; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) acc[m][c] = 0.f;
  const int kend = min(GV_KSLICE, K - k0);
  for (int g0 = 0; g0 < kend; g0 += 128) {
    float part[GV_MAXM][4];
#pragma unroll
    for (int m = 0; m < GV_MAXM; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) part[m][c] = 0.f;
    const uint8_t* wp = packed + (long)((k0 + g0) >> 1) * N + n0;
#pragma unroll 4
    for (int k2 = 0; k2 < 64; ++k2) {
      const uint32_t w = *reinterpret_cast<const uint32_t*>(wp + (long)k2 * N);
      const int kk = g0 + 2 * k2;
#pragma unroll
      for (int c = 0; c < 4; ++c) {
        const uint32_t byte = (w >> (8 * c)) & 0xffu;
        const float lo = static_cast<float>(static_cast<int>(byte & 15u) - 8);
        const float hi = static_cast<float>(static_cast<int>(byte >> 4) - 8);
#pragma unroll
        for (int m = 0; m < GV_MAXM; ++m) part[m][c] = fmaf(xs[m][kk], lo, fmaf(xs[m][kk + 1], hi, part[m][c]));
      }
    }
    const uint2 sv = *reinterpret_cast<const uint2*>(scales + (long)((k0 + g0) >> 7) * N + n0);
    const float sc[4] = {bf16_lo(sv.x), bf16_hi(sv.x), bf16_lo(sv.y), bf16_hi(sv.y)};
#pragma unroll
    for (int m = 0; m < GV_MAXM; ++m)
#pragma unroll
      for (int c = 0; c < 4; ++c) acc[m][c] = fmaf(part[m][c], sc[c], acc[m][c]);
  }
  for (int m = 0; m < mrows; ++m)
#pragma unroll
    for (int c = 0; c < 4; ++c) atomicAdd(acc_out + (long)(m0 + m) * N + n0 + c, acc[m][c]);
}

// ---------------------------------------------------------------------------- W4A16 on tcgen05
// CTA = (128 output columns n, one K split). Warps 0-3: dequant (thread = n), warp 4: TMA
// loader, warp 5: MMA issuer. Per 64-k block: W words [8 k8 x 128 n] + x tile [MP x 64 k].
// The K splits of a column tile form a thread-block cluster: every CTA parks its fp32 tile
// (`[128 n][MP]`, read back from tensor memory) in shared memory, the cluster's first CTA sums the
// tiles through distributed shared memory, adds the residual and stores bf16 `y[m][n]`: one launch,
// no global accumulator, no atomics. Launched with programmatic stream serialization: barrier set-up,
// tensor-memory allocation and descriptor prefetch overlap the tail of the preceding kernel.
//
// Two instances. Decode (M <= 64): 8 ring stages, x tile of up to 64 rows, 128 tensor-memory columns, two CTAs
// per SM, K split over the cluster. Prefill (M > 64): grid.z walks the rows in tiles of MP = 128 or 256, 6 ring
// stages with a 256-row x tile, 512 tensor-memory columns (128 for four weight buffers + up to 256 for D),
// one CTA per SM, no K split: the weight tile is expanded once per 128 x MP output tile, in registers, on its
// way into tensor memory, and never exists in global memory.
constexpr int WQ_WBYTES = 8 * 128 * 4;           // repacked weight tile
// decode rows with three groups (SUMMA_W4A16_DECODE_GROUPS=3): 12 % faster on the 28672-wide projection, 20 % slower at
// 64 rows x 4096 columns, level elsewhere (all 20-60 us launches): one group stays the default
constexpr int W4A16_DECODE_GROUPS_DEFAULT = 1;
template <int MPMAX, int G> struct WqCfg {
  static constexpr int NS = MPMAX <= 64 ? 8 : 6;                 // ring stages
  static constexpr int XBYTES = MPMAX * 128;                     // x tile at MP = MPMAX
  static constexpr int STAGE = WQ_WBYTES + XBYTES;
  static constexpr int SMEM = NS * STAGE + 256 + 1024;
  static constexpr int TMEM_COLS = MPMAX <= 64 ? (G == 1 ? 128 : 256) : 512;
  static constexpr int MIN_CTAS = MPMAX <= 64 ? 2 : 1;
  // dequant warps = 4 * DQ, in DQ groups of 128 threads (thread = output column; every group reaches every
  // tensor-memory lane). With one CTA per SM one group cannot expand a weight tile within the 512 cycles its four
  // 128 x 256 x 16 MMAs take: per 64-k block a warp pays a barrier wake-up, the shared-memory load latency, ~130
  // dependent ALU / bf16x2 instructions and a tensor-memory store + wait, about 1,200 cycles (one group: 0.38-0.52
  // of the GEMM peak; two groups splitting each block's k range: 0.61, tensor pipe 41 % in the profile, because the
  // fixed latencies are paid per block by everyone). So the prefill instance hands WHOLE 64-k blocks to its three
  // groups in turn: each group has three block times to expand one block.
  static constexpr int DQ = G;
  static constexpr int THREADS = 128 * DQ + 64;
  static constexpr int NA = G == 1 ? 2 : 4;                 // expanded weight buffers in tensor memory (32 columns each)
  // a group skips blocks, so it does not see every phase of a buffer's `free` barrier; a parity wait stays
  // unambiguous because the ring bounds how far the MMA can lag: block i is only loaded once block i - NS has been
  // consumed, and i - NS >= i - 2 NA
  static_assert(DQ == 1 || NS <= 2 * NA, "ring deeper than two rounds of weight buffers: free-barrier parity would alias");
};

struct W4Params {
  int M, N, K, MP, kb_per_split;
  const __nv_bfloat16* scales;    // [K / 128, N]
  const __nv_bfloat16* residual;  // [M, N] or null
  __nv_bfloat16* y;               // [M, N]
  unsigned int* err;
};

template <int MPMAX, int G>
__global__ void __launch_bounds__(WqCfg<MPMAX, G>::THREADS, WqCfg<MPMAX, G>::MIN_CTAS)
w4a16_gemm_kernel(const __grid_constant__ CUtensorMap tmW, const __grid_constant__ CUtensorMap tmX, const W4Params p) {
  constexpr int WQ_NS = WqCfg<MPMAX, G>::NS, WQ_STAGE = WqCfg<MPMAX, G>::STAGE, DQ = WqCfg<MPMAX, G>::DQ;
  constexpr int TMA_WARP = 4 * DQ, MMA_WARP = 4 * DQ + 1, NA = WqCfg<MPMAX, G>::NA;
  extern __shared__ uint8_t smem_raw[];
  asm volatile("griddepcontrol.launch_dependents;");
  namespace cg = cooperative_groups;
  cg::cluster_group cluster = cg::this_cluster();
  uint8_t* smem = reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(smem_raw) + 1023) & ~uintptr_t(1023));
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + WQ_NS * WQ_STAGE);
  uint64_t* full = bars;                 // [NS]
  uint64_t* empty = bars + WQ_NS;        // [NS]
  uint64_t* a_full = bars + 2 * WQ_NS;   // [NA] one arrival per dequant thread
  uint64_t* a_free = a_full + NA;        // [NA]
  uint64_t* d_full = a_free + NA;
  uint32_t* tmem_slot = reinterpret_cast<uint32_t*>(d_full + 1);
  volatile int* abort_flag = reinterpret_cast<volatile int*>(tmem_slot + 1);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n0 = blockIdx.x * 128;
  const int kblocks = p.K / 64;
  const int kb0 = blockIdx.y * p.kb_per_split;
  const int nkb = max(0, min(p.kb_per_split, kblocks - kb0));
  if (threadIdx.x == 0) {
    for (int s = 0; s < WQ_NS; ++s) { mbar_init(&full[s], 1); mbar_init(&empty[s], 1); }
    for (int s = 0; s < NA; ++s) { mbar_init(&a_full[s], 128); mbar_init(&a_free[s], 1); }
    mbar_init(d_full, 1);
    *abort_flag = 0;
    fence_barrier_init();
  }
  if (warp == MMA_WARP) { tmem_alloc(tmem_slot, WqCfg<MPMAX, G>::TMEM_COLS); tmem_relinquish(); }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tmem_base = *tmem_slot;
  constexpr uint32_t COL_A = 0, COL_D = 32 * NA;  // A: NA buffers x 32 columns, D: MP columns
  const int m0 = blockIdx.z * p.MP;               // first row of this CTA's row tile (decode: one tile)
  asm volatile("griddepcontrol.wait;" ::: "memory");   // x and the residual come from the preceding kernel
  float* tile = reinterpret_cast<float*>(smem);   // [128][MP + 1], reuses the ring once the products are done
  const int tpitch = p.MP + 1;
  // one K split, whole 128-column tile, 16-byte aligned rows of y: the tile is parked as bf16 `[m][128 n]` and
  // leaves in 16-byte row segments; otherwise as fp32 `[n][m]` for the cluster's reduction and scalar stores
  __nv_bfloat16* tileb = reinterpret_cast<__nv_bfloat16*>(smem);
  const bool fast_out = gridDim.y == 1 && (p.N & 7) == 0 && n0 + 128 <= p.N;

  if (warp == TMA_WARP) {
    if (lane == 0) {
      for (int i = 0; i < nkb; ++i) {
        const int s = i % WQ_NS;
        if (!mbar_wait(&empty[s], ((i / WQ_NS) & 1) ^ 1, abort_flag, p.err)) break;
        mbar_expect_tx(&full[s], WQ_WBYTES + p.MP * 128);
        tma_load_2d(smem + s * WQ_STAGE, &tmW, &full[s], n0, (kb0 + i) * 8);
        tma_load_2d(smem + s * WQ_STAGE + WQ_WBYTES, &tmX, &full[s], (kb0 + i) * 64, m0);
      }
      if (*abort_flag) { const long long t0 = clock64(); while (clock64() - t0 < 2000000) {} }
    }
    __syncwarp();
  } else if (warp == MMA_WARP) {
    if (lane == 0 && nkb > 0) {
      const uint32_t idesc = make_idesc_bf16(128, p.MP, 0, 0);
      bool ok = true;
      for (int i = 0; i < nkb && ok; ++i) {
        const int s = i % WQ_NS, b = i % NA;
        if (!mbar_wait(&full[s], (i / WQ_NS) & 1, abort_flag, p.err) ||       // the x tile of this stage
            !mbar_wait(&a_full[b], (i / NA) & 1, abort_flag, p.err)) { ok = false; break; }
        tc_fence_after();
        const uint32_t x_base = smem_u32(smem + s * WQ_STAGE + WQ_WBYTES);
#pragma unroll
        for (int kk = 0; kk < 4; ++kk)
          umma_bf16_ta(tmem_base + COL_D, tmem_base + COL_A + 32 * b + 8 * kk,
                       make_smem_desc_sw128(x_base + kk * 32, 16, 1024), idesc, (i > 0 || kk > 0) ? 1u : 0u);
        umma_commit(&a_free[b]);
        umma_commit(&empty[s]);
      }
      if (ok) umma_commit(d_full);
    }
    __syncwarp();
  } else {
    const int t = threadIdx.x & 127;              // output column n0 + t == TMEM lane
    const int h = threadIdx.x >> 7;               // group: expands the 64-k blocks i with i % DQ == h, and 1/DQ of D's columns
    const uint32_t lane_sel = static_cast<uint32_t>((warp & 3) * 32) << 16;
    const int n = n0 + t;
    bool ok = true;
    __nv_bfloat162 s2 = __float2bfloat162_rn(0.f);
    const __nv_bfloat162 off2 = __float2bfloat162_rn(136.f);
    int scale_row = -1;
    for (int i = 0; i < nkb && ok; ++i) {
      const int s = i % WQ_NS, b = i % NA, kb = kb0 + i;
      // every group waits for every block's load in order (a group that skipped phases of `full` could otherwise
      // take an older phase of the same parity for the one it needs)
      if (!mbar_wait(&full[s], (i / WQ_NS) & 1, abort_flag, p.err)) { ok = false; break; }
      if (DQ > 1 && i % DQ != h) continue;
      if ((kb >> 1) != scale_row) {
        scale_row = kb >> 1;
        const __nv_bfloat16 sc = n < p.N ? p.scales[(long)scale_row * p.N + n] : __float2bfloat16(0.f);
        s2 = __halves2bfloat162(sc, sc);
      }
      const uint32_t* wt = reinterpret_cast<const uint32_t*>(smem + s * WQ_STAGE) + t;
      uint32_t r[32];
#pragma unroll
      for (int jj = 0; jj < 8; ++jj) {
        const int j = jj;
        const uint32_t w = wt[j * 128];            // codes of k = 8j .. 8j+7 for this column
#pragma unroll
        for (int q = 0; q < 4; ++q) {
          // (128 + q_even, 128 + q_odd) as two bf16, minus 136 (exact), times the group scale
          uint32_t pr = ((w >> (4 * q)) & 0x000F000Fu) | 0x43004300u;
          __nv_bfloat162 v = *reinterpret_cast<__nv_bfloat162*>(&pr);
          v = __hmul2(__hsub2(v, off2), s2);
          r[4 * jj + q] = *reinterpret_cast<uint32_t*>(&v);
        }
      }
      if (i >= NA && !mbar_wait(&a_free[b], ((i / NA) - 1) & 1, abort_flag, p.err)) { ok = false; break; }
      tc_fence_after();
      tmem_st_32x32b_x32(tmem_base + COL_A + 32 * b + lane_sel, r);
      tmem_st_wait();
      tc_fence_before();
      mbar_arrive(&a_full[b]);
    }
    if (ok && nkb > 0 && mbar_wait(d_full, 0, abort_flag, p.err)) {
      tc_fence_after();
      // every product has completed, so the ring is free: park this thread's row of the tile there
      for (int c = 16 * h; c < p.MP; c += 16 * DQ) {
        uint32_t v[16];
        tmem_ld_32x32b_x16(tmem_base + COL_D + c + lane_sel, v);
        tmem_ld_wait();
        if (fast_out) {
#pragma unroll
          for (int j = 0; j < 16; ++j) tileb[(c + j) * 128 + t] = __float2bfloat16(__uint_as_float(v[j]));
        } else {
#pragma unroll
          for (int j = 0; j < 16; ++j) tile[t * tpitch + c + j] = __uint_as_float(v[j]);
        }
      }
    } else if (nkb == 0) {
      for (int c = h; c < p.MP; c += DQ) {
        if (fast_out) tileb[c * 128 + t] = __float2bfloat16(0.f);
        else tile[t * tpitch + c] = 0.f;
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  if (warp == MMA_WARP) { tc_fence_after(); tmem_dealloc(tmem_base, WqCfg<MPMAX, G>::TMEM_COLS); }
  // ---- split-K reduction over the cluster, residual, bf16 store (thread = column, coalesced along n)
  cluster.sync();
  if (fast_out) {
    if (threadIdx.x < 128 * DQ) {
      const int rows = min(p.MP, p.M - m0);
      for (int idx = threadIdx.x; idx < rows * 16; idx += 128 * DQ) {
        const int m = idx >> 4, ch = idx & 15;
        uint4 v = *reinterpret_cast<const uint4*>(tileb + m * 128 + ch * 8);
        const long off = (long)(m0 + m) * p.N + n0 + ch * 8;
        if (p.residual) {
          const uint4 rv = *reinterpret_cast<const uint4*>(p.residual + off);
          const uint32_t* a = reinterpret_cast<const uint32_t*>(&v);
          const uint32_t* b = reinterpret_cast<const uint32_t*>(&rv);
          uint32_t o[4];
#pragma unroll
          for (int q = 0; q < 4; ++q) {
            const float2 fa = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&a[q]));
            const float2 fb = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&b[q]));
            const __nv_bfloat162 r2 = __floats2bfloat162_rn(fa.x + fb.x, fa.y + fb.y);
            o[q] = *reinterpret_cast<const uint32_t*>(&r2);
          }
          v = make_uint4(o[0], o[1], o[2], o[3]);
        }
        *reinterpret_cast<uint4*>(p.y + off) = v;
      }
    }
  } else if (threadIdx.x < 128 * DQ) {
    // every CTA of the cluster reduces its share of the rows (m = rank, rank + S, ...), so the
    // distributed-shared-memory reads are spread over the cluster instead of serialised in one CTA
    const int t = threadIdx.x & 127, n = n0 + t, h = threadIdx.x >> 7;
    const int S = (int)cluster.num_blocks(), r0 = (int)cluster.block_rank();
    const int rows = min(p.MP, p.M - m0);
    if (n < p.N) {
      for (int m = r0 + S * h; m < rows; m += S * DQ) {
        float v = 0.f;
#pragma unroll 8
        for (int r = 0; r < S; ++r) v += cluster.map_shared_rank(tile, r)[t * tpitch + m];
        if (p.residual) v += __bfloat162float(p.residual[(long)(m0 + m) * p.N + n]);
        p.y[(long)(m0 + m) * p.N + n] = __float2bfloat16(v);
      }
    }
  }
  cluster.sync();                                 // nobody leaves while a peer still reads its tile
}

__global__ void int4_finish_kernel(const float* __restrict__ acc, const __nv_bfloat16* __restrict__ residual,
                                   __nv_bfloat16* __restrict__ y, long n) {
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n; i += (long)gridDim.x * blockDim.x) {
    float v = acc[i];
    if (residual) v += __bfloat162float(residual[i]);
    y[i] = __float2bfloat16(v);
  }
}

// y[m, n] = accT[n, m] (+ residual[m, n]); 32 x 32 tiles through shared memory
__global__ void __launch_bounds__(256)
int4_finish_t_kernel(const float* __restrict__ accT, const __nv_bfloat16* __restrict__ residual,
                     __nv_bfloat16* __restrict__ y, int M, int N, int MP) {
  __shared__ float tile[32][33];
  const int n0 = blockIdx.x * 32, m0 = blockIdx.y * 32;
  const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
  for (int r = ty; r < 32; r += 8) {               // r: n within the tile, tx: m within the tile
    const int n = n0 + r, m = m0 + tx;
    tile[r][tx] = (n < N && m < MP) ? accT[(long)n * MP + m] : 0.f;
  }
  __syncthreads();
  for (int r = ty; r < 32; r += 8) {               // r: m within the tile, tx: n within the tile
    const int m = m0 + r, n = n0 + tx;
    if (m < M && n < N) {
      float v = tile[tx][r];
      if (residual) v += __bfloat162float(residual[(long)m * N + n]);
      y[(long)m * N + n] = __float2bfloat16(v);
    }
  }
}

// thread = 4 columns x 2 rows (one packed word)
__global__ void int4_dequant_kernel(const uint8_t* __restrict__ packed, const __nv_bfloat16* __restrict__ scales,
                                    __nv_bfloat16* __restrict__ out, int K, int N) {
  const long total = (long)(K / 2) * (N / 4);
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < total; i += (long)gridDim.x * blockDim.x) {
    const int k2 = i / (N / 4);
    const int n0 = (i - (long)k2 * (N / 4)) * 4;
    const uint32_t w = *reinterpret_cast<const uint32_t*>(packed + (long)k2 * N + n0);
    const uint2 sv = *reinterpret_cast<const uint2*>(scales + (long)((2 * k2) >> 7) * N + n0);
    const float sc[4] = {bf16_lo(sv.x), bf16_hi(sv.x), bf16_lo(sv.y), bf16_hi(sv.y)};
    float lo[4], hi[4];
#pragma unroll
    for (int c = 0; c < 4; ++c) {
      const uint32_t byte = (w >> (8 * c)) & 0xffu;
      lo[c] = static_cast<float>(static_cast<int>(byte & 15u) - 8) * sc[c];
      hi[c] = static_cast<float>(static_cast<int>(byte >> 4) - 8) * sc[c];
    }
    *reinterpret_cast<uint2*>(out + (long)(2 * k2) * N + n0) = make_uint2(pack_bf16(lo[0], lo[1]), pack_bf16(lo[2], lo[3]));
    *reinterpret_cast<uint2*>(out + (long)(2 * k2 + 1) * N + n0) = make_uint2(pack_bf16(hi[0], hi[1]), pack_bf16(hi[2], hi[3]));
  }
}

// one block per row: argmax over `vocab` logits (fp32 or bf16), lowest index wins ties
template <typename T>
__global__ void __launch_bounds__(256)
argmax_rows_kernel(const T* __restrict__ logits, long* __restrict__ out, int vocab, long ld) {
  const T* row = logits + (long)blockIdx.x * ld;
  float best = -INFINITY;
  int bi = 0x7fffffff;
  for (int i = threadIdx.x; i < vocab; i += 256) {
    const float v = static_cast<float>(row[i]);
    if (v > best || (v == best && i < bi)) { best = v; bi = i; }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
    const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
    if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
  }
  __shared__ float sb_[8];
  __shared__ int si[8];
  if ((threadIdx.x & 31) == 0) { sb_[threadIdx.x >> 5] = best; si[threadIdx.x >> 5] = bi; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int w = 1; w < 8; ++w)
      if (sb_[w] > best || (sb_[w] == best && si[w] < bi)) { best = sb_[w]; bi = si[w]; }
    out[blockIdx.x] = bi;
  }
}

}  // namespace sb

using namespace sb;

// y[M,N] = x[M,K] @ dequant(packed, scales) (+ residual). acc: fp32 scratch of max(M, 64) * N floats.
// M <= 64, K % 128 == 0, N % 4 == 0.
extern "C" int sb_int4_gemv(const void* x, const void* packed, const void* scales, float* acc, const void* residual,
                            void* y, int M, int N, int K, long ldx, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && M <= 64 && K % 128 == 0 && N % 4 == 0 && N > 0);
  SB_CHECK_CUDA(cudaMemsetAsync(acc, 0, sizeof(float) * (size_t)M * N, st));
  {
    dim3 grid((N + 511) / 512, (K + GV_KSLICE - 1) / GV_KSLICE, (M + GV_MAXM - 1) / GV_MAXM);
    int4_gemv_kernel<<<grid, 128, 0, st>>>((const __nv_bfloat16*)x, (const uint8_t*)packed,
                                           (const __nv_bfloat16*)scales, acc, M, N, K, ldx);
  }
  const long n = (long)M * N;
  int4_finish_kernel<<<(int)((n + 255) / 256), 256, 0, st>>>(acc, (const __nv_bfloat16*)residual, (__nv_bfloat16*)y, n);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_int4_dequant(const void* packed, const void* scales, void* out, int K, int N, cudaStream_t st) {
  SB_CHECK_ARG(K % 128 == 0 && N % 4 == 0);
  const long total = (long)(K / 2) * (N / 4);
  long blocks = (total + 255) / 256;
  if (blocks > num_sms() * 16L) blocks = num_sms() * 16L;
  int4_dequant_kernel<<<(int)blocks, 256, 0, st>>>((const uint8_t*)packed, (const __nv_bfloat16*)scales,
                                                   (__nv_bfloat16*)out, K, N);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_argmax_rows(const void* logits, long* out, int rows, int vocab, long ld, int is_bf16, cudaStream_t st) {
  SB_CHECK_ARG(rows > 0 && vocab > 0);
  if (is_bf16) argmax_rows_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((const __nv_bfloat16*)logits, out, vocab, ld);
  else argmax_rows_kernel<float><<<rows, 256, 0, st>>>((const float*)logits, out, vocab, ld);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// ---------------------------------------------------------------------------- sampling
// One block per row: repetition penalty over the tokens already seen (a V-bit map, so each
// distinct token is penalised once), then greedy / top-k / full-distribution sampling at a
// temperature, driven by one uniform number per row. The chosen token is written out and its
// bit is set, so consecutive decode steps need no host involvement.
namespace sb {

template <typename T>
__device__ __forceinline__ float sample_logit(const T* row, const uint32_t* seen, int i, float penalty) {
  float v = static_cast<float>(row[i]);
  if (seen != nullptr && ((seen[i >> 5] >> (i & 31)) & 1u)) v = v > 0.f ? v / penalty : v * penalty;
  return v;
}

// block-wide argmax of (value desc, index asc); result broadcast to all threads
__device__ __forceinline__ void block_best(float& v, int& idx, float* sv, int* si) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float ov = __shfl_xor_sync(0xffffffffu, v, o);
    const int oi = __shfl_xor_sync(0xffffffffu, idx, o);
    if (ov > v || (ov == v && oi < idx)) { v = ov; idx = oi; }
  }
  __syncthreads();
  if ((threadIdx.x & 31) == 0) { sv[threadIdx.x >> 5] = v; si[threadIdx.x >> 5] = idx; }
  __syncthreads();
  v = sv[0]; idx = si[0];
  for (int w = 1; w < (int)(blockDim.x >> 5); ++w)
    if (sv[w] > v || (sv[w] == v && si[w] < idx)) { v = sv[w]; idx = si[w]; }
}

constexpr int SAMPLE_MAX_K = 64;

template <typename T>
__global__ void __launch_bounds__(256)
sample_rows_kernel(const T* __restrict__ logits, long ld, uint32_t* __restrict__ seen, int seen_words,
                   const float* __restrict__ uniform, long* __restrict__ out, int vocab, float penalty, float temperature,
                   int top_k) {
  __shared__ float sv[8];
  __shared__ int si[8];
  __shared__ float kv[SAMPLE_MAX_K];
  __shared__ int ki[SAMPLE_MAX_K];
  __shared__ float part[256];
  const T* row = logits + (long)blockIdx.x * ld;
  uint32_t* sn = seen != nullptr ? seen + (long)blockIdx.x * seen_words : nullptr;
  const uint32_t* snc = (penalty != 1.f) ? sn : nullptr;
  int chosen = 0;
  if (temperature <= 0.f || top_k == 1) {
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += 256) {
      const float v = sample_logit(row, snc, i, penalty);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    block_best(best, bi, sv, si);
    chosen = bi;
  } else if (top_k > 0 && top_k < vocab) {
    const int k = min(top_k, SAMPLE_MAX_K);
    float pv = INFINITY; int pi = -1;                 // previous pick in (value desc, index asc) order
    for (int r = 0; r < k; ++r) {
      float best = -INFINITY; int bi = 0x7fffffff;
      for (int i = threadIdx.x; i < vocab; i += 256) {
        const float v = sample_logit(row, snc, i, penalty);
        const bool after = v < pv || (v == pv && i > pi);
        if (after && (v > best || (v == best && i < bi))) { best = v; bi = i; }
      }
      block_best(best, bi, sv, si);
      if (threadIdx.x == 0) { kv[r] = best; ki[r] = bi; }
      pv = best; pi = bi;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      const float inv_t = 1.f / temperature;
      float tot = 0.f;
      for (int r = 0; r < k; ++r) tot += __expf((kv[r] - kv[0]) * inv_t);
      const float target = uniform[blockIdx.x] * tot;
      float acc = 0.f;
      int pick = k - 1;
      for (int r = 0; r < k; ++r) {
        acc += __expf((kv[r] - kv[0]) * inv_t);
        if (acc >= target) { pick = r; break; }
      }
      si[0] = ki[pick];
    }
    __syncthreads();
    chosen = si[0];
  } else {
    // full distribution: max, per-thread chunk sums (contiguous chunks), then the owning thread walks its chunk
    const float inv_t = 1.f / temperature;
    float best = -INFINITY; int bi = 0x7fffffff;
    for (int i = threadIdx.x; i < vocab; i += 256) {
      const float v = sample_logit(row, snc, i, penalty);
      if (v > best || (v == best && i < bi)) { best = v; bi = i; }
    }
    block_best(best, bi, sv, si);
    const int chunk = (vocab + 255) / 256;
    const int lo = threadIdx.x * chunk, hi = min(vocab, lo + chunk);
    float s = 0.f;
    for (int i = lo; i < hi; ++i) s += __expf((sample_logit(row, snc, i, penalty) - best) * inv_t);
    part[threadIdx.x] = s;
    __syncthreads();
    if (threadIdx.x == 0) {
      float tot = 0.f;
      for (int t = 0; t < 256; ++t) tot += part[t];
      const float target = uniform[blockIdx.x] * tot;
      float acc = 0.f;
      int owner = 255;
      for (int t = 0; t < 256; ++t) {
        if (acc + part[t] >= target) { owner = t; break; }
        acc += part[t];
      }
      sv[0] = target - acc;
      si[0] = owner;
    }
    __syncthreads();
    if ((int)threadIdx.x == si[0]) {
      float acc = 0.f;
      int pick = max(lo, hi - 1);
      for (int i = lo; i < hi; ++i) {
        acc += __expf((sample_logit(row, snc, i, penalty) - best) * inv_t);
        if (acc >= sv[0]) { pick = i; break; }
      }
      si[1] = pick;
    }
    __syncthreads();
    chosen = si[1];
  }
  if (threadIdx.x == 0) {
    out[blockIdx.x] = chosen;
    if (sn != nullptr) atomicOr(&sn[chosen >> 5], 1u << (chosen & 31));
  }
}

}  // namespace sb

// Sample one token per row. logits `[rows, vocab]` (row stride ld, fp32 or bf16); seen: optional
// `[rows, ceil(vocab / 32)]` bit map of tokens already produced (read for the penalty, updated with
// the pick); uniform: `[rows]` numbers in [0, 1) (unused for greedy). temperature <= 0 = greedy.
// top_k in [2, 64] restricts to the k best, 0 samples the full distribution.
extern "C" int sb_sample_rows(const void* logits, long ld, int is_bf16, unsigned int* seen, const float* uniform, long* out,
                              int rows, int vocab, float penalty, float temperature, int top_k, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(rows > 0 && vocab > 0 && penalty > 0.f && top_k >= 0 && top_k <= SAMPLE_MAX_K);
  SB_CHECK_ARG(temperature <= 0.f || uniform != nullptr);
  const int words = (vocab + 31) / 32;
  if (is_bf16)
    sample_rows_kernel<__nv_bfloat16><<<rows, 256, 0, st>>>((const __nv_bfloat16*)logits, ld, seen, words, uniform, out,
                                                            vocab, penalty, temperature, top_k);
  else
    sample_rows_kernel<float><<<rows, 256, 0, st>>>((const float*)logits, ld, seen, words, uniform, out, vocab, penalty,
                                                    temperature, top_k);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// The same product on the tensor cores (see w4a16_gemm above). packed_k8: `[K/8, N]` uint32 repacked
// weight. K % 128 == 0, N % 4 == 0, x 16-byte aligned with ldx % 8 == 0. M <= 64 runs the decode instance
// (K split over a cluster), larger M the prefill instance over row tiles of 128 or 256.
template <int MPMAX, int G>
static int launch_w4a16(const void* x, const void* packed_k8, const void* scales, const void* residual, void* y, int M, int N,
                        int K, long ldx, cudaStream_t st) {
  using Cfg = WqCfg<MPMAX, G>;
  W4Params p;
  p.M = M; p.N = N; p.K = K;
  const int n_tiles = (N + 127) / 128, kblocks = K / 64;
  int splits = 1, m_tiles = 1;
  if (MPMAX <= 64) {
    p.MP = M <= 16 ? 16 : (M <= 32 ? 32 : 64);
    // K splits = cluster size (1, 2, 4 or 8): about one round of two-per-SM CTAs, at least 4 k-blocks each
    // (twice as many splits measured slower: 5,539 against 6,494 decode tokens/s at batch 64)
    while (splits < 8 && n_tiles * 2 * splits <= 2 * num_sms() && kblocks / (2 * splits) >= 4) splits *= 2;
  } else {
    p.MP = M <= 128 ? 128 : 256;
    m_tiles = (M + p.MP - 1) / p.MP;
    SB_CHECK_ARG(m_tiles <= 65535);
    // few output tiles: split K over a cluster until the grid fills the GPU once
    while (splits < 8 && (long)n_tiles * m_tiles * splits * 2 <= num_sms() && kblocks / (2 * splits) >= 4) splits *= 2;
  }
  p.kb_per_split = (kblocks + splits - 1) / splits;
  p.scales = (const __nv_bfloat16*)scales;
  p.residual = (const __nv_bfloat16*)residual;
  p.y = (__nv_bfloat16*)y;
  p.err = error_word();
  if (!p.err) return SB_ERR_CUDA;
  CUtensorMap tmW, tmX;
  int rc;
  if ((rc = make_tmap_2d(&tmW, packed_k8, 4, (uint64_t)N, (uint64_t)K / 8, (uint64_t)N * 4, 128, 8, false))) return rc;
  if ((rc = make_tmap_2d(&tmX, x, 2, (uint64_t)K, (uint64_t)M, (uint64_t)ldx * 2, 64, (uint32_t)p.MP, true))) return rc;
  static bool attr_set[64] = {false};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!attr_set[dev & 63]) {
    SB_CHECK_CUDA(cudaFuncSetAttribute(w4a16_gemm_kernel<MPMAX, G>, cudaFuncAttributeMaxDynamicSharedMemorySize, Cfg::SMEM));
    attr_set[dev & 63] = true;
  }
  cudaLaunchConfig_t cfg = {};
  cfg.gridDim = dim3(n_tiles, splits, m_tiles);
  cfg.blockDim = dim3(Cfg::THREADS, 1, 1);
  cfg.dynamicSmemBytes = Cfg::SMEM;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = 1;
  attr[0].val.clusterDim.y = splits;
  attr[0].val.clusterDim.z = 1;
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = 2;
  SB_CHECK_CUDA(cudaLaunchKernelEx(&cfg, w4a16_gemm_kernel<MPMAX, G>, tmW, tmX, p));
  return SB_OK;
}

extern "C" int sb_w4a16_gemm(const void* x, const void* packed_k8, const void* scales, float* acc, const void* residual,
                             void* y, int M, int N, int K, long ldx, cudaStream_t st) {
  SB_CHECK_ARG(M >= 1 && K % 128 == 0 && N % 4 == 0 && N > 0 && ldx % 8 == 0);
  SB_CHECK_ARG((reinterpret_cast<uintptr_t>(x) & 15) == 0 && (reinterpret_cast<uintptr_t>(packed_k8) & 15) == 0);
  (void)acc;
  if (M <= 64) {
    // decode rows: one expanding group per CTA, or three (whole 64-k blocks in turn, like the prefill instance)
    static const int groups = [] { const char* e = getenv("SUMMA_W4A16_DECODE_GROUPS"); return e ? atoi(e) : W4A16_DECODE_GROUPS_DEFAULT; }();
    if (groups == 3) return launch_w4a16<64, 3>(x, packed_k8, scales, residual, y, M, N, K, ldx, st);
    return launch_w4a16<64, 1>(x, packed_k8, scales, residual, y, M, N, K, ldx, st);
  }
  return launch_w4a16<256, 3>(x, packed_k8, scales, residual, y, M, N, K, ldx, st);
}
