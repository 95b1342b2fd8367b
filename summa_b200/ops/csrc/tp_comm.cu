// One-shot all-reduce over NVLink peer memory for tensor-parallel inference.
//
// Each rank owns an "inbox" in symmetric memory with one slot per source rank (double
// buffered by epoch parity). A single kernel (a) stores this rank's partial activation
// into its slot of EVERY peer's inbox with 16-byte peer stores, (b) publishes an arrival
// flag once all of its CTAs have stored, (c) waits (bounded) for every peer's arrival flag
// and (d) sums the `world` slots of its own inbox into the output. For decode-sized
// activations this replaces a ring all-reduce (2(P-1) latency steps) by one store wave and
// one flag wait. The grid never exceeds the SM count, so all CTAs are co-resident and the
// in-kernel wait cannot starve its own producers.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int TP_MAX_RANKS = 16;
constexpr int TPSIG_ARRIVE = 0;    // [src] epoch of the last complete store wave from src

struct TpPeers {
  __nv_bfloat16* inbox[TP_MAX_RANKS];
  uint32_t* sig[TP_MAX_RANKS];
};

__device__ __forceinline__ void tp_st_release(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t tp_ld_acquire(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

__global__ void __launch_bounds__(256)
tp_allreduce_kernel(TpPeers peers, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out, long n,
                    long slot_elems, int rank, int world, unsigned int* epoch_word, unsigned int* counter,
                    unsigned int* err, const __nv_bfloat16* __restrict__ residual) {
  // The call number lives in device memory (bumped by the last CTA of every launch, after all
  // CTAs have read it), so a captured CUDA graph can replay this kernel any number of times.
  const uint32_t epoch = *reinterpret_cast<volatile unsigned int*>(epoch_word) + 1u;
  const long buf_off = (long)(epoch & 1u) * world * slot_elems;
  const long n8 = n >> 3;
  const long tid = blockIdx.x * (long)blockDim.x + threadIdx.x;
  const long stride = (long)gridDim.x * blockDim.x;
  // (a) scatter my partial into every inbox
  for (long i = tid; i < n8; i += stride) {
    const uint4 v = reinterpret_cast<const uint4*>(x)[i];
#pragma unroll 4
    for (int s = 0; s < world; ++s) {
      int dst = rank + s;
      if (dst >= world) dst -= world;
      reinterpret_cast<uint4*>(peers.inbox[dst] + buf_off + (long)rank * slot_elems)[i] = v;
    }
  }
  // (b) arrival: last CTA of this rank tells every peer
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;
      *epoch_word = epoch;
      for (int pr = 0; pr < world; ++pr) tp_st_release(peers.sig[pr] + TPSIG_ARRIVE + rank, epoch);
    }
  }
  // (c) wait for all sources
  if (threadIdx.x < world) {
    const uint32_t* f = peers.sig[rank] + TPSIG_ARRIVE + threadIdx.x;
    const long long t0 = clock64();
    while (static_cast<int32_t>(tp_ld_acquire(f) - epoch) < 0) {
      if (clock64() - t0 > SB_WAIT_CYCLES) { atomicOr(err, 2u); break; }
      __nanosleep(32);
    }
  }
  __syncthreads();
  // (d) reduce my inbox
  const __nv_bfloat16* mine = peers.inbox[rank] + buf_off;
  for (long i = tid; i < n8; i += stride) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    if (residual != nullptr) {           // the residual stream is added once, after the sum
      const uint4 r = reinterpret_cast<const uint4*>(residual)[i];
      acc[0] = bf16_lo(r.x); acc[1] = bf16_hi(r.x); acc[2] = bf16_lo(r.y); acc[3] = bf16_hi(r.y);
      acc[4] = bf16_lo(r.z); acc[5] = bf16_hi(r.z); acc[6] = bf16_lo(r.w); acc[7] = bf16_hi(r.w);
    }
    for (int s = 0; s < world; ++s) {
      const uint4 v = __ldcg(reinterpret_cast<const uint4*>(mine + (long)s * slot_elems) + i);
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]); o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out)[i] = o;
  }
}

// ---------------------------------------------------------------------------- NVLS variant
// The same all-reduce through the NVSwitch multicast object of the symmetric buffer: every rank
// copies its partial into ITS OWN slot-less staging buffer (local stores only), publishes an
// arrival flag, waits for all peers and then issues `multimem.ld_reduce` on the multicast
// address: the switch fetches the word from every rank's buffer, adds in fp32 and returns one
// 16-byte result, so each rank receives n * 2 bytes instead of world * n * 2.
constexpr int TPSIG_MM_ARRIVE = 0;     // in its OWN signal pad: the pad of the peer-store kernels is shared with the fused GEMMs

__global__ void __launch_bounds__(256)
tp_allreduce_mm_kernel(TpPeers peers, const __nv_bfloat16* __restrict__ x, __nv_bfloat16* __restrict__ out,
                       __nv_bfloat16* stage_local, const __nv_bfloat16* stage_mc, long n, long slot_elems, int rank,
                       int world, unsigned int* epoch_word, unsigned int* counter, unsigned int* err,
                       const __nv_bfloat16* __restrict__ residual) {
  const uint32_t epoch = *reinterpret_cast<volatile unsigned int*>(epoch_word) + 1u;
  const long buf_off = (long)(epoch & 1u) * slot_elems;
  const long n8 = n >> 3;
  const long tid = blockIdx.x * (long)blockDim.x + threadIdx.x;
  const long stride = (long)gridDim.x * blockDim.x;
  for (long i = tid; i < n8; i += stride)
    reinterpret_cast<uint4*>(stage_local + buf_off)[i] = reinterpret_cast<const uint4*>(x)[i];
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;
      *epoch_word = epoch;
      for (int pr = 0; pr < world; ++pr) tp_st_release(peers.sig[pr] + TPSIG_MM_ARRIVE + rank, epoch);
    }
  }
  if (threadIdx.x < world) {
    const uint32_t* f = peers.sig[rank] + TPSIG_MM_ARRIVE + threadIdx.x;
    const long long t0 = clock64();
    while (static_cast<int32_t>(tp_ld_acquire(f) - epoch) < 0) {
      if (clock64() - t0 > SB_WAIT_CYCLES) { atomicOr(err, 2u); break; }
      __nanosleep(32);
    }
  }
  __syncthreads();
  for (long i = tid; i < n8; i += stride) {
    uint4 v;
    asm volatile("multimem.ld_reduce.relaxed.sys.global.add.acc::f32.v4.bf16x2 {%0, %1, %2, %3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(reinterpret_cast<const uint4*>(stage_mc + buf_off) + i)
                 : "memory");
    if (residual != nullptr) {
      const uint4 r = reinterpret_cast<const uint4*>(residual)[i];
      v.x = pack_bf16(bf16_lo(v.x) + bf16_lo(r.x), bf16_hi(v.x) + bf16_hi(r.x));
      v.y = pack_bf16(bf16_lo(v.y) + bf16_lo(r.y), bf16_hi(v.y) + bf16_hi(r.y));
      v.z = pack_bf16(bf16_lo(v.z) + bf16_lo(r.z), bf16_hi(v.z) + bf16_hi(r.z));
      v.w = pack_bf16(bf16_lo(v.w) + bf16_lo(r.w), bf16_hi(v.w) + bf16_hi(r.w));
    }
    reinterpret_cast<uint4*>(out)[i] = v;
  }
}

}  // namespace sb

using namespace sb;

static unsigned int* tp_counter() {
  static unsigned int* counters[64] = {nullptr};
  int dev = 0;
  if (cudaGetDevice(&dev) != cudaSuccess) return nullptr;
  if (!counters[dev & 63]) {
    if (cudaMalloc(&counters[dev & 63], sizeof(unsigned int)) != cudaSuccess) return nullptr;
    if (cudaMemset(counters[dev & 63], 0, sizeof(unsigned int)) != cudaSuccess) return nullptr;
  }
  return counters[dev & 63];
}

// NVLS form: stage_local = this rank's symmetric staging buffer (2 * slot_elems bf16), stage_mc =
// the multicast address of the same symmetric allocation; sig = peer pointers of a signal pad used by
// this kernel only.
extern "C" int sb_tp_allreduce_mm(const void* x, void* out, void* stage_local, const void* stage_mc,
                                  const void* const* sig, long n, long slot_elems, int rank, int world,
                                  unsigned int* epoch_word, const void* residual, cudaStream_t st) {
  SB_CHECK_ARG(world >= 1 && world <= TP_MAX_RANKS && rank >= 0 && rank < world);
  SB_CHECK_ARG(n > 0 && n % 8 == 0 && n <= slot_elems && slot_elems % 8 == 0 && stage_local && stage_mc);
  TpPeers p;
  for (int i = 0; i < TP_MAX_RANKS; ++i) { p.inbox[i] = nullptr; p.sig[i] = nullptr; }
  for (int i = 0; i < world; ++i) p.sig[i] = (uint32_t*)sig[i];
  unsigned int* err = error_word();
  unsigned int* counter = tp_counter();
  if (!err || !counter) return SB_ERR_CUDA;
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > num_sms()) blocks = num_sms();
  if (blocks < 1) blocks = 1;
  tp_allreduce_mm_kernel<<<(int)blocks, 256, 0, st>>>(p, (const __nv_bfloat16*)x, (__nv_bfloat16*)out,
                                                      (__nv_bfloat16*)stage_local, (const __nv_bfloat16*)stage_mc, n,
                                                      slot_elems, rank, world, epoch_word, counter, err,
                                                      (const __nv_bfloat16*)residual);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// out = sum over ranks of x (bf16, n % 8 == 0, n <= slot_elems). inbox / sig: host arrays of
// `world` peer-mapped device pointers; each inbox holds 2 * world * slot_elems bf16, each
// signal pad at least 64 words. epoch_word: one device word per group (zero at start, owned by
// the kernel): the call number, kept on the device so that the launch is graph-capturable.
// residual (bf16 [n], local, or null) is added to the sum. Every rank must make the same sequence of calls.
extern "C" int sb_tp_allreduce(const void* x, void* out, const void* const* inbox, const void* const* sig, long n,
                               long slot_elems, int rank, int world, unsigned int* epoch_word, const void* residual,
                               cudaStream_t st) {
  SB_CHECK_ARG(world >= 1 && world <= TP_MAX_RANKS && rank >= 0 && rank < world);
  SB_CHECK_ARG(n > 0 && n % 8 == 0 && n <= slot_elems && slot_elems % 8 == 0);
  TpPeers p;
  for (int i = 0; i < TP_MAX_RANKS; ++i) { p.inbox[i] = nullptr; p.sig[i] = nullptr; }
  for (int i = 0; i < world; ++i) { p.inbox[i] = (__nv_bfloat16*)inbox[i]; p.sig[i] = (uint32_t*)sig[i]; }
  unsigned int* err = error_word();
  if (!err) return SB_ERR_CUDA;
  // per-device counter lives right after the error word's allocation: use a static one
  static unsigned int* counters[64] = {nullptr};
  int dev = 0;
  SB_CHECK_CUDA(cudaGetDevice(&dev));
  if (!counters[dev & 63]) {
    SB_CHECK_CUDA(cudaMalloc(&counters[dev & 63], sizeof(unsigned int)));
    SB_CHECK_CUDA(cudaMemset(counters[dev & 63], 0, sizeof(unsigned int)));
  }
  long blocks = ((n >> 3) + 255) / 256;
  if (blocks > num_sms()) blocks = num_sms();
  if (blocks < 1) blocks = 1;
  tp_allreduce_kernel<<<(int)blocks, 256, 0, st>>>(p, (const __nv_bfloat16*)x, (__nv_bfloat16*)out, n, slot_elems, rank,
                                                   world, epoch_word, counters[dev & 63], err,
                                                   (const __nv_bfloat16*)residual);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
