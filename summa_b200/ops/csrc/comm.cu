// Data-parallel optimizer step fused with its collectives over NVLink peer memory.
//
// Every rank owns one contiguous shard of the flat parameter range. Two kernels, each of
// which does its arithmetic and its communication in the same launch with plain peer
// loads/stores (no copy engine, no library collective):
//
//   dp_reduce_scatter_kernel   waits until every peer has published "gradients final",
//       then reads this rank's shard of the fp32 gradient buffer from all peers, sums,
//       keeps the reduced shard locally and accumulates its sum of squares; the last CTA
//       publishes the partial sum of squares to every peer.
//   dp_adamw_allgather_kernel  collects all partial sums (global gradient norm -> clip
//       coefficient), applies AdamW to the fp32 master shard and writes the new bf16
//       weights directly into EVERY peer's parameter buffer; the last CTA publishes "done"
//       and waits for all peers' "done", so the next kernel on the stream sees complete
//       parameters.
//
// Flags are monotonically increasing epochs in a symmetric signal pad (no resets, no ABA).
// Every spin is bounded by a clock limit; on expiry the kernel records bit 2 in the device
// error word, so a missing peer can never hang the GPU. A failed "gradients final" or "norm
// valid" wait also stamps the step's epoch into an abort word in the scratch area: the update
// kernel then applies nothing and stores nothing (masters, moments and every peer's
// parameters keep their values of the previous step), and the host, which reads the error
// word after each step, raises before anything can be checkpointed.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

constexpr int DP_MAX_RANKS = 16;
// signal pad layout (uint32 words)
constexpr int SIG_READY = 0;       // [src] gradients of src are final for epoch
constexpr int SIG_NORMFLAG = 16;   // [src] partial sum of squares of src is valid for epoch
constexpr int SIG_DONE = 32;       // [src] src has written its parameter shard everywhere
constexpr int SIG_NORMVAL = 48;    // [src] float bits
constexpr int SIG_BUCKET = 64;     // [bucket][src] gradients of src inside the bucket's range are final for epoch
constexpr int DP_MAX_BUCKETS = 64;
constexpr int SIG_WORDS = SIG_BUCKET + DP_MAX_BUCKETS * DP_MAX_RANKS;

struct DpPeers {
  float* grads[DP_MAX_RANKS];
  __nv_bfloat16* params[DP_MAX_RANKS];
  uint32_t* sig[DP_MAX_RANKS];
};

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}
// bounded wait for *p >= epoch (wrap-safe signed difference)
__device__ __forceinline__ bool wait_epoch(const uint32_t* p, uint32_t epoch, unsigned int* err) {
  const long long t0 = clock64();
  while (static_cast<int32_t>(ld_acquire_sys(p) - epoch) < 0) {
    if (clock64() - t0 > SB_WAIT_CYCLES) {
      atomicOr(err, 2u);
      return false;
    }
    __nanosleep(64);
  }
  return true;
}

__global__ void __launch_bounds__(512)
dp_reduce_scatter_kernel(DpPeers peers, float* __restrict__ reduced, long shard_off, long shard_len, int rank,
                         int world, uint32_t epoch, unsigned int* counter, float* local_sumsq, unsigned int* err,
                         const float* __restrict__ mc_grads, uint32_t* abort_word) {
  // ---- start barrier: all peers' backward passes are complete
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(peers.sig[threadIdx.x] + SIG_READY + rank, epoch);
  }
  if (threadIdx.x < world && !wait_epoch(peers.sig[rank] + SIG_READY + threadIdx.x, epoch, err))
    atomicExch(abort_word, epoch);          // a peer's gradients are not final: this step applies nothing
  __syncthreads();

  // ---- reduce this rank's shard over all peers (16-byte peer loads, staggered start)
  const long n4 = shard_len >> 2;
  float sq = 0.f;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n4; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mc_grads != nullptr) {
      // NVLS: one load on the multicast address, the switch sums the word over all ranks
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                   : "l"(reinterpret_cast<const float4*>(mc_grads + shard_off) + i)
                   : "memory");
    } else {
#pragma unroll 4
      for (int s = 0; s < world; ++s) {
        int src = rank + s;
        if (src >= world) src -= world;
        const float4 v = __ldcg(reinterpret_cast<const float4*>(peers.grads[src] + shard_off) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    reinterpret_cast<float4*>(reduced)[i] = acc;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  sq = warp_sum(sq);
  __shared__ float red[16];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = sq;
  __syncthreads();
  if (w == 0) {
    sq = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    sq = warp_sum(sq);
    if (lane == 0) {
      atomicAdd(local_sumsq, sq);
      __threadfence();
      const unsigned int prev = atomicAdd(counter, 1u);
      if (prev == gridDim.x - 1) {
        // last CTA: publish this rank's partial sum of squares to every peer
        const float total = atomicExch(local_sumsq, 0.f);
        *counter = 0;
        for (int pr = 0; pr < world; ++pr) {
          peers.sig[pr][SIG_NORMVAL + rank] = __float_as_uint(total);
        }
        __threadfence_system();
        for (int pr = 0; pr < world; ++pr) st_release_sys(peers.sig[pr] + SIG_NORMFLAG + rank, epoch);
      }
    }
  }
}

// One bucket of the reduce-scatter, launched while the backward pass is still running: [lo, hi) is the part of
// the bucket's flat range that lies in this rank's shard (shard-relative, multiples of 4; empty for most ranks,
// since shards are contiguous). Every rank tells every peer "my gradients inside this bucket are final"; a rank
// that owns a part waits (bounded) for all peers' flags, sums the part over the ranks into its reduced shard and
// adds the part's sum of squares to the running total. With `publish` (the last bucket of the step) the last
// CTA hands the total to every peer exactly as dp_reduce_scatter_kernel does.
__global__ void __launch_bounds__(512)
dp_bucket_reduce_kernel(DpPeers peers, float* __restrict__ reduced, long shard_off, long lo, long hi, int rank, int world,
                        uint32_t epoch, int bucket, int publish, unsigned int* counter, float* local_sumsq,
                        unsigned int* err, const float* __restrict__ mc_grads, uint32_t* abort_word) {
  const int flag0 = SIG_BUCKET + bucket * DP_MAX_RANKS;
  if (blockIdx.x == 0 && threadIdx.x < world) {
    __threadfence_system();
    st_release_sys(peers.sig[threadIdx.x] + flag0 + rank, epoch);
  }
  if (hi > lo && threadIdx.x < world && !wait_epoch(peers.sig[rank] + flag0 + threadIdx.x, epoch, err))
    atomicExch(abort_word, epoch);          // a peer's gradients are not final: this step applies nothing
  __syncthreads();
  float sq = 0.f;
  const long i0 = lo >> 2, i1 = hi >> 2;
  for (long i = i0 + blockIdx.x * (long)blockDim.x + threadIdx.x; i < i1; i += (long)gridDim.x * blockDim.x) {
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (mc_grads != nullptr) {
      asm volatile("multimem.ld_reduce.relaxed.sys.global.add.v4.f32 {%0, %1, %2, %3}, [%4];"
                   : "=f"(acc.x), "=f"(acc.y), "=f"(acc.z), "=f"(acc.w)
                   : "l"(reinterpret_cast<const float4*>(mc_grads + shard_off) + i)
                   : "memory");
    } else {
#pragma unroll 4
      for (int s = 0; s < world; ++s) {
        int src = rank + s;
        if (src >= world) src -= world;
        const float4 v = __ldcg(reinterpret_cast<const float4*>(peers.grads[src] + shard_off) + i);
        acc.x += v.x; acc.y += v.y; acc.z += v.z; acc.w += v.w;
      }
    }
    reinterpret_cast<float4*>(reduced)[i] = acc;
    sq += acc.x * acc.x + acc.y * acc.y + acc.z * acc.z + acc.w * acc.w;
  }
  sq = warp_sum(sq);
  __shared__ float red[16];
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  if (lane == 0) red[w] = sq;
  __syncthreads();
  if (w == 0) {
    sq = lane < (blockDim.x >> 5) ? red[lane] : 0.f;
    sq = warp_sum(sq);
    if (lane == 0) {
      if (sq != 0.f) atomicAdd(local_sumsq, sq);
      if (publish) {
        __threadfence();
        const unsigned int prev = atomicAdd(counter, 1u);
        if (prev == gridDim.x - 1) {
          const float total = atomicExch(local_sumsq, 0.f);
          *counter = 0;
          for (int pr = 0; pr < world; ++pr) peers.sig[pr][SIG_NORMVAL + rank] = __float_as_uint(total);
          __threadfence_system();
          for (int pr = 0; pr < world; ++pr) st_release_sys(peers.sig[pr] + SIG_NORMFLAG + rank, epoch);
        }
      }
    }
  }
}

__global__ void __launch_bounds__(512)
dp_adamw_allgather_kernel(DpPeers peers, const float* __restrict__ reduced, float* __restrict__ master,
                          float* __restrict__ m, float* __restrict__ v, long shard_off, long shard_len, int rank,
                          int world, uint32_t epoch, float grad_scale, float max_norm, float lr, float beta1,
                          float beta2, float eps, float wd, float bc1, float bc2, unsigned int* counter,
                          float* norm_out, const float* extra_sumsq, long adamw_limit, unsigned int* err,
                          __nv_bfloat16* mc_params, uint32_t* abort_word) {
  __shared__ float parts[DP_MAX_RANKS];
  __shared__ float coef_sh;
  __shared__ int skip_sh;
  if (threadIdx.x == 0) skip_sh = 0;
  __syncthreads();
  if (threadIdx.x < world) {
    if (!wait_epoch(peers.sig[rank] + SIG_NORMFLAG + threadIdx.x, epoch, err)) {
      atomicExch(abort_word, epoch);
      skip_sh = 1;
    }
    parts[threadIdx.x] = __uint_as_float(*reinterpret_cast<volatile uint32_t*>(peers.sig[rank] + SIG_NORMVAL + threadIdx.x));
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    // extra_sumsq: squared norm of gradients that live outside the sharded range
    float tot = extra_sumsq ? *extra_sumsq : 0.f;
    for (int i = 0; i < world; ++i) tot += parts[i];
    const float norm = sqrtf(tot) * grad_scale;
    float coef = grad_scale;
    if (max_norm > 0.f) coef *= fminf(1.f, max_norm / (norm + 1e-6f));
    coef_sh = coef;
    if (blockIdx.x == 0) { norm_out[0] = norm; norm_out[1] = coef; }
    if (*reinterpret_cast<volatile uint32_t*>(abort_word) == epoch) skip_sh = 1;
  }
  __syncthreads();
  const float coef = coef_sh;
  const bool skip = skip_sh != 0;

  // 8 elements per thread-iteration: one 16-byte bf16 store per peer
  const long n8 = shard_len >> 3;
  for (long i = blockIdx.x * (long)blockDim.x + threadIdx.x; i < n8 && !skip; i += (long)gridDim.x * blockDim.x) {
    // elements at or past adamw_limit (flat index) belong to another optimizer (Muon): reduced and
    // counted in the norm, but neither updated nor redistributed here
    if (adamw_limit >= 0 && shard_off + 8 * i >= adamw_limit) continue;
    float p[8], g[8], mm[8], vv[8];
    *reinterpret_cast<float4*>(g) = reinterpret_cast<const float4*>(reduced)[2 * i];
    *reinterpret_cast<float4*>(g + 4) = reinterpret_cast<const float4*>(reduced)[2 * i + 1];
    *reinterpret_cast<float4*>(p) = reinterpret_cast<const float4*>(master)[2 * i];
    *reinterpret_cast<float4*>(p + 4) = reinterpret_cast<const float4*>(master)[2 * i + 1];
    *reinterpret_cast<float4*>(mm) = reinterpret_cast<const float4*>(m)[2 * i];
    *reinterpret_cast<float4*>(mm + 4) = reinterpret_cast<const float4*>(m)[2 * i + 1];
    *reinterpret_cast<float4*>(vv) = reinterpret_cast<const float4*>(v)[2 * i];
    *reinterpret_cast<float4*>(vv + 4) = reinterpret_cast<const float4*>(v)[2 * i + 1];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const float gk = g[k] * coef;
      mm[k] = beta1 * mm[k] + (1.f - beta1) * gk;
      vv[k] = beta2 * vv[k] + (1.f - beta2) * gk * gk;
      p[k] = p[k] - lr * wd * p[k] - lr * (mm[k] / bc1) / (sqrtf(vv[k] / bc2) + eps);
    }
    reinterpret_cast<float4*>(master)[2 * i] = *reinterpret_cast<float4*>(p);
    reinterpret_cast<float4*>(master)[2 * i + 1] = *reinterpret_cast<float4*>(p + 4);
    reinterpret_cast<float4*>(m)[2 * i] = *reinterpret_cast<float4*>(mm);
    reinterpret_cast<float4*>(m)[2 * i + 1] = *reinterpret_cast<float4*>(mm + 4);
    reinterpret_cast<float4*>(v)[2 * i] = *reinterpret_cast<float4*>(vv);
    reinterpret_cast<float4*>(v)[2 * i + 1] = *reinterpret_cast<float4*>(vv + 4);
    uint4 o;
    o.x = pack_bf16(p[0], p[1]); o.y = pack_bf16(p[2], p[3]); o.z = pack_bf16(p[4], p[5]); o.w = pack_bf16(p[6], p[7]);
    if (mc_params != nullptr) {
      // NVLS: one store on the multicast address lands in every rank's parameter buffer
      asm volatile("multimem.st.relaxed.sys.global.v4.f32 [%0], {%1, %2, %3, %4};" ::"l"(
                       reinterpret_cast<uint4*>(mc_params + shard_off) + i),
                   "f"(__uint_as_float(o.x)), "f"(__uint_as_float(o.y)), "f"(__uint_as_float(o.z)),
                   "f"(__uint_as_float(o.w))
                   : "memory");
    } else {
#pragma unroll 4
      for (int s = 0; s < world; ++s) {
        int dst = rank + s;
        if (dst >= world) dst -= world;
        reinterpret_cast<uint4*>(peers.params[dst] + shard_off)[i] = o;
      }
    }
  }
  // ---- completion: all of this rank's stores are out; tell peers and wait for theirs
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();
    const unsigned int prev = atomicAdd(counter, 1u);
    if (prev == gridDim.x - 1) {
      *counter = 0;
      for (int pr = 0; pr < world; ++pr) st_release_sys(peers.sig[pr] + SIG_DONE + rank, epoch);
      for (int pr = 0; pr < world; ++pr) wait_epoch(peers.sig[rank] + SIG_DONE + pr, epoch, err);
    }
  }
}

// One thread waits for *flag >= expected for at most `limit_cycles` SM clocks, exactly like the
// peer-flag waits of the fused kernels; on expiry it records bit 2 in the error word and returns.
__global__ void wait_probe_kernel(const uint32_t* flag, uint32_t expected, long long limit_cycles, unsigned int* err,
                                  unsigned int* waited_out) {
  const long long t0 = clock64();
  bool ok = true;
  while (static_cast<int32_t>(ld_acquire_sys(flag) - expected) < 0) {
    if (clock64() - t0 > limit_cycles) {
      atomicOr(err, 2u);
      ok = false;
      break;
    }
    __nanosleep(64);
  }
  if (waited_out) *waited_out = ok ? 0u : 1u;
}

}  // namespace sb

using namespace sb;

// Failure-detection self-test of the bounded peer-flag wait: returns immediately when the flag
// already holds `expected`, otherwise gives up after `limit_cycles` (capped at SB_WAIT_CYCLES)
// with the error word's bit 2 set and `gave_up[0] = 1`. The context stays usable either way.
extern "C" int sb_wait_probe(const void* flag, unsigned int expected, long long limit_cycles, void* gave_up,
                             cudaStream_t st) {
  SB_CHECK_ARG(flag != nullptr && limit_cycles > 0);
  if (limit_cycles > SB_WAIT_CYCLES) limit_cycles = SB_WAIT_CYCLES;
  unsigned int* err = error_word();
  if (!err) return SB_ERR_CUDA;
  wait_probe_kernel<<<1, 1, 0, st>>>((const uint32_t*)flag, expected, limit_cycles, err, (unsigned int*)gave_up);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

static int fill_peers(DpPeers& pr, const void* const* grads, const void* const* params, const void* const* sig, int world) {
  for (int i = 0; i < DP_MAX_RANKS; ++i) { pr.grads[i] = nullptr; pr.params[i] = nullptr; pr.sig[i] = nullptr; }
  for (int i = 0; i < world; ++i) {
    pr.grads[i] = (float*)grads[i];
    pr.params[i] = (__nv_bfloat16*)params[i];
    pr.sig[i] = (uint32_t*)sig[i];
  }
  return 0;
}

// Fused data-parallel step. grads/params/sig: host arrays of `world` device pointers (this
// rank's own buffer included, at index `rank`), all in peer-mapped symmetric memory.
// reduced/master/m/v: local fp32 buffers of shard_len elements; scratch: 8 words, zero before the
// first call (uint32 counter, uint32 counter, float sumsq, float norm_out, float coef_out, uint32 abort
// epoch: equals `epoch` after a step whose peer waits failed and which therefore applied nothing).
// extra_sumsq (device scalar or null) is added to the squared gradient norm. shard_len % 8 == 0.
// adamw_limit >= 0: flat elements at or past it are left to another optimizer (multiple of 8); -1: none.
// mc_grads / mc_params: multicast (NVLS) addresses of the symmetric gradient / parameter buffers, or
// null for plain peer loads and stores.
// Signal-pad size (32-bit words) the data-parallel kernels expect.
extern "C" int sb_dp_sig_words() { return SIG_WORDS; }

// One bucket of the overlapped reduce-scatter: [lo_flat, hi_flat) is the bucket's range of the flat gradient
// buffer (multiples of 4); the part inside this rank's shard is reduced over all ranks into `reduced` and its
// sum of squares joins the step's running total in `scratch`. Every rank of the group launches it for every
// bucket of a step, in the same order, each bucket id (< 64) once per epoch; `publish` != 0 on the step's last
// bucket. Safe on a side stream next to the backward pass: it reads gradients only inside the bucket.
extern "C" int sb_dp_bucket_reduce(const void* const* grads, const void* const* sig, float* reduced, void* scratch,
                                   long shard_off, long shard_len, long lo_flat, long hi_flat, int bucket, int publish,
                                   int rank, int world, unsigned int epoch, const void* mc_grads, int ctas,
                                   cudaStream_t st) {
  SB_CHECK_ARG(world >= 1 && world <= DP_MAX_RANKS && rank >= 0 && rank < world && bucket >= 0 && bucket < DP_MAX_BUCKETS);
  SB_CHECK_ARG(shard_len > 0 && shard_len % 8 == 0 && shard_off % 8 == 0 && lo_flat % 4 == 0 && hi_flat % 4 == 0 &&
               lo_flat <= hi_flat);
  DpPeers pr;
  for (int i = 0; i < DP_MAX_RANKS; ++i) { pr.grads[i] = nullptr; pr.params[i] = nullptr; pr.sig[i] = nullptr; }
  for (int i = 0; i < world; ++i) { pr.grads[i] = (float*)grads[i]; pr.sig[i] = (uint32_t*)sig[i]; }
  unsigned int* err = error_word();
  if (!err) return SB_ERR_CUDA;
  long lo = lo_flat - shard_off, hi = hi_flat - shard_off;
  if (lo < 0) lo = 0;
  if (hi > shard_len) hi = shard_len;
  if (hi < lo) hi = lo;
  unsigned int* counters = (unsigned int*)scratch;
  float* fs = (float*)scratch;
  const int grid = ctas > 0 ? ctas : num_sms();
  dp_bucket_reduce_kernel<<<grid, 512, 0, st>>>(pr, reduced, shard_off, lo, hi, rank, world, epoch, bucket, publish,
                                                counters, fs + 2, err, (const float*)mc_grads, counters + 5);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// The second half of sb_dp_fused_step alone (norm -> clip -> AdamW -> all-gather), for a step whose
// reduce-scatter was done bucket by bucket with sb_dp_bucket_reduce. Same arguments as sb_dp_fused_step.
extern "C" int sb_dp_update_step(const void* const* grads, const void* const* params, const void* const* sig,
                                 float* reduced, float* master, float* m, float* v, void* scratch, long shard_off,
                                 long shard_len, int rank, int world, unsigned int epoch, float grad_scale,
                                 float max_norm, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                 float bc2, const float* extra_sumsq, long adamw_limit, const void* mc_grads,
                                 void* mc_params, cudaStream_t st);

extern "C" int sb_dp_fused_step(const void* const* grads, const void* const* params, const void* const* sig,
                                float* reduced, float* master, float* m, float* v, void* scratch, long shard_off,
                                long shard_len, int rank, int world, unsigned int epoch, float grad_scale,
                                float max_norm, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                float bc2, const float* extra_sumsq, long adamw_limit, const void* mc_grads, void* mc_params,
                                cudaStream_t st) {
  SB_CHECK_ARG(adamw_limit < 0 || adamw_limit % 8 == 0);
  SB_CHECK_ARG(world >= 1 && world <= DP_MAX_RANKS && rank >= 0 && rank < world);
  SB_CHECK_ARG(shard_len > 0 && shard_len % 8 == 0 && shard_off % 8 == 0);
  DpPeers pr;
  fill_peers(pr, grads, params, sig, world);
  unsigned int* err = error_word();
  if (!err) return SB_ERR_CUDA;
  unsigned int* counters = (unsigned int*)scratch;
  float* fs = (float*)scratch;
  const int grid = num_sms();
  dp_reduce_scatter_kernel<<<grid, 512, 0, st>>>(pr, reduced, shard_off, shard_len, rank, world, epoch, counters,
                                                 fs + 2, err, (const float*)mc_grads, counters + 5);
  dp_adamw_allgather_kernel<<<grid, 512, 0, st>>>(pr, reduced, master, m, v, shard_off, shard_len, rank, world, epoch,
                                                  grad_scale, max_norm, lr, beta1, beta2, eps, wd, bc1, bc2,
                                                  counters + 1, fs + 3, extra_sumsq, adamw_limit, err,
                                                  (__nv_bfloat16*)mc_params, counters + 5);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_dp_update_step(const void* const* grads, const void* const* params, const void* const* sig,
                                 float* reduced, float* master, float* m, float* v, void* scratch, long shard_off,
                                 long shard_len, int rank, int world, unsigned int epoch, float grad_scale,
                                 float max_norm, float lr, float beta1, float beta2, float eps, float wd, float bc1,
                                 float bc2, const float* extra_sumsq, long adamw_limit, const void* mc_grads,
                                 void* mc_params, cudaStream_t st) {
  (void)mc_grads;
  SB_CHECK_ARG(adamw_limit < 0 || adamw_limit % 8 == 0);
  SB_CHECK_ARG(world >= 1 && world <= DP_MAX_RANKS && rank >= 0 && rank < world);
  SB_CHECK_ARG(shard_len > 0 && shard_len % 8 == 0 && shard_off % 8 == 0);
  DpPeers pr;
  fill_peers(pr, grads, params, sig, world);
  unsigned int* err = error_word();
  if (!err) return SB_ERR_CUDA;
  unsigned int* counters = (unsigned int*)scratch;
  float* fs = (float*)scratch;
  dp_adamw_allgather_kernel<<<num_sms(), 512, 0, st>>>(pr, reduced, master, m, v, shard_off, shard_len, rank, world, epoch,
                                                       grad_scale, max_norm, lr, beta1, beta2, eps, wd, bc1, bc2,
                                                       counters + 1, fs + 3, extra_sumsq, adamw_limit, err,
                                                       (__nv_bfloat16*)mc_params, counters + 5);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
