// Mixture-of-experts routing and dispatch kernels. Everything stays on the device: the
// per-expert counts are never read by the host.
//
// Padded routed layout: the (token, slot) routes are sorted stably by expert and each
// expert's rows start at a multiple of 128, so every 128-row GEMM tile belongs to exactly
// one expert (`tile_expert`) and the grouped GEMM can use plain TMA loads and stores.
//   router_logits   fp32 logits = x(bf16) @ W(fp32), SIMT (the router stays in fp32)
//   topk            per token: top-k on logits (k <= 8), ties to the lower index
//   plan            histogram -> padded offsets -> stable destination row of every route,
//                   row -> (token, slot) map, tile -> expert map, live tile count
//   gather          routed[row] = x[token(row)] (zero rows in the padding)
//   combine         out[t] = sum_slot gate[t,slot] * y[dest[t,slot]]
//   and the matching backward kernels.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

// ---------------------------------------------------------------------------- router GEMM
// logits[T, E] = x[T, H] (bf16, row stride ldx) @ W[H, E] (fp32). 64 tokens per block,
// each thread computes one token row for a strip of 16 experts? Simple register tiling:
// block = 256 threads = 64 tokens x 4 expert groups; E <= 256.
__global__ void __launch_bounds__(256)
router_logits_kernel(const __nv_bfloat16* __restrict__ x, const float* __restrict__ w, float* __restrict__ logits,
                     int T, int H, int E, long ldx) {
  __shared__ float xs[64][33];
  __shared__ float ws[32][257];
  const int tid = threadIdx.x;
  const int tok = tid & 63, eg = tid >> 6;          // expert group: experts eg, eg+4, eg+8, ...
  const int t0 = blockIdx.x * 64;
  float acc[64];
#pragma unroll
  for (int i = 0; i < 64; ++i) acc[i] = 0.f;
  const int ne = (E + 3) / 4;                        // experts per thread (<= 64)
  for (int k0 = 0; k0 < H; k0 += 32) {
    for (int i = tid; i < 64 * 32; i += 256) {
      const int r = i >> 5, c = i & 31;
      const int t = t0 + r;
      xs[r][c] = (t < T && k0 + c < H) ? __bfloat162float(x[(long)t * ldx + k0 + c]) : 0.f;
    }
    for (int i = tid; i < 32 * E; i += 256) {
      const int r = i / E, c = i % E;
      ws[r][c] = (k0 + r < H) ? w[(long)(k0 + r) * E + c] : 0.f;
    }
    __syncthreads();
#pragma unroll 4
    for (int kk = 0; kk < 32; ++kk) {
      const float xv = xs[tok][kk];
#pragma unroll
      for (int i = 0; i < 64; ++i)
        if (i < ne) acc[i] = fmaf(xv, ws[kk][eg + 4 * i], acc[i]);
    }
    __syncthreads();
  }
  const int t = t0 + tok;
  if (t < T) {
#pragma unroll
    for (int i = 0; i < 64; ++i) {
      const int e = eg + 4 * i;
      if (i < ne && e < E) logits[(long)t * E + e] = acc[i];
    }
  }
}

// ---------------------------------------------------------------------------- top-k
// One warp per token; lane l holds experts l, l+32, ... (E <= 256). Emits indices in
// descending-logit order and bumps the per-expert histogram.
template <int EPL>
__global__ void moe_topk_kernel(const float* __restrict__ logits, int* __restrict__ idx, int* __restrict__ counts,
                                int T, int E, int k) {
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (gw >= T) return;
  float v[EPL];
#pragma unroll
  for (int i = 0; i < EPL; ++i) {
    const int e = lane + 32 * i;
    v[i] = e < E ? logits[(long)gw * E + e] : -INFINITY;
  }
  for (int s = 0; s < k; ++s) {
    float best = -INFINITY;
    int bi = 0x7fffffff;
#pragma unroll
    for (int i = 0; i < EPL; ++i) {
      const int e = lane + 32 * i;
      if (v[i] > best || (v[i] == best && e < bi)) { best = v[i]; bi = e; }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float ob = __shfl_xor_sync(0xffffffffu, best, o);
      const int oi = __shfl_xor_sync(0xffffffffu, bi, o);
      if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
    }
    if (lane == 0) {
      idx[(long)gw * k + s] = bi;
      atomicAdd(counts + bi, 1);
    }
#pragma unroll
    for (int i = 0; i < EPL; ++i)
      if (lane + 32 * i == bi) v[i] = -INFINITY;
  }
}

// ---------------------------------------------------------------------------- route plan
// meta layout (int32): [0, E] poff (padded offsets, poff[E] = total padded rows),
// [E+1] live 128-row tiles. One block.
__global__ void moe_offsets_kernel(const int* __restrict__ counts, int* __restrict__ meta, int* __restrict__ tile_expert,
                                   int E, int max_tiles) {
  __shared__ int off[257];
  if (threadIdx.x == 0) {
    int a = 0;
    for (int e = 0; e < E; ++e) {
      off[e] = a;
      a += (counts[e] + 127) / 128 * 128;
    }
    off[E] = a;
  }
  __syncthreads();
  for (int e = threadIdx.x; e <= E; e += blockDim.x) meta[e] = off[e];
  if (threadIdx.x == 0) meta[E + 1] = off[E] / 128;
  for (int e = threadIdx.x; e < E; e += blockDim.x)
    for (int t = off[e] / 128; t < off[e + 1] / 128 && t < max_tiles; ++t) tile_expert[t] = e;
}

// One block per expert: stable compaction of the routes that chose it. dest[route] =
// padded row; row_route[row] = route id (token * k + slot) or -1 for padding.
__global__ void __launch_bounds__(256)
moe_pack_kernel(const int* __restrict__ idx, const int* __restrict__ meta, int* __restrict__ dest,
                int* __restrict__ row_route, int routes) {
  const int e = blockIdx.x;
  const int base = meta[e], end = meta[e + 1];
  __shared__ int warp_tot[8];
  __shared__ int running;
  if (threadIdx.x == 0) running = 0;
  __syncthreads();
  const int lane = threadIdx.x & 31, w = threadIdx.x >> 5;
  for (int r0 = 0; r0 < routes; r0 += 256) {
    const int r = r0 + threadIdx.x;
    const bool hit = r < routes && idx[r] == e;
    const unsigned m = __ballot_sync(0xffffffffu, hit);
    const int before = __popc(m & ((1u << lane) - 1));
    if (lane == 0) warp_tot[w] = __popc(m);
    __syncthreads();
    int woff = 0;
    for (int i = 0; i < w; ++i) woff += warp_tot[i];
    const int start = running;
    if (hit) {
      const int row = base + start + woff + before;
      dest[r] = row;
      row_route[row] = r;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
      int tot = 0;
      for (int i = 0; i < 8; ++i) tot += warp_tot[i];
      running = start + tot;
    }
    __syncthreads();
  }
  // padding rows of this expert
  for (int row = base + running + threadIdx.x; row < end; row += 256) row_route[row] = -1;
}

// ---------------------------------------------------------------------------- gather / combine
// routed[row, :] = x[token(row), :] for live rows, 0 for padding. One warp per row.
__global__ void moe_gather_kernel(const __nv_bfloat16* __restrict__ x, const int* __restrict__ row_route,
                                  const int* __restrict__ meta, __nv_bfloat16* __restrict__ routed, int E, int H, int k,
                                  long ldx, int max_rows) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= max_rows || row >= meta[E]) return;
  const int r = row_route[row];
  uint4* dst = reinterpret_cast<uint4*>(routed + (long)row * H);
  if (r < 0) {
    for (int c = lane; c < H / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
  } else {
    const uint4* src = reinterpret_cast<const uint4*>(x + (long)(r / k) * ldx);
    for (int c = lane; c < H / 8; c += 32) dst[c] = src[c];
  }
}

// out[t, :] = sum_slot gates[t, slot] * y[dest[t*k+slot], :]. One warp per token.
__global__ void moe_combine_kernel(const __nv_bfloat16* __restrict__ y, const int* __restrict__ dest,
                                   const float* __restrict__ gates, __nv_bfloat16* __restrict__ out, int T, int H, int k) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane; c < H / 8; c += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < k; ++s) {
      const float g = gates[(long)t * k + s];
      const uint4 v = reinterpret_cast<const uint4*>(y + (long)dest[(long)t * k + s] * H)[c];
      acc[0] = fmaf(g, bf16_lo(v.x), acc[0]); acc[1] = fmaf(g, bf16_hi(v.x), acc[1]);
      acc[2] = fmaf(g, bf16_lo(v.y), acc[2]); acc[3] = fmaf(g, bf16_hi(v.y), acc[3]);
      acc[4] = fmaf(g, bf16_lo(v.z), acc[4]); acc[5] = fmaf(g, bf16_hi(v.z), acc[5]);
      acc[6] = fmaf(g, bf16_lo(v.w), acc[6]); acc[7] = fmaf(g, bf16_hi(v.w), acc[7]);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]); o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(out + (long)t * H)[c] = o;
  }
}

// Backward of combine. One warp per padded row:
//   dy[row, :] = gate(route) * dout[token, :]   (0 for padding)
//   dgate[route] = <dout[token, :], y[row, :]>
__global__ void moe_combine_bwd_kernel(const __nv_bfloat16* __restrict__ dout, const __nv_bfloat16* __restrict__ y,
                                       const int* __restrict__ row_route, const float* __restrict__ gates,
                                       const int* __restrict__ meta, __nv_bfloat16* __restrict__ dy,
                                       float* __restrict__ dgates, int E, int H, int k, int max_rows) {
  const int row = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (row >= max_rows || row >= meta[E]) return;
  const int r = row_route[row];
  uint4* dst = reinterpret_cast<uint4*>(dy + (long)row * H);
  if (r < 0) {
    for (int c = lane; c < H / 8; c += 32) dst[c] = make_uint4(0, 0, 0, 0);
    return;
  }
  const float g = gates[r];
  const uint4* src = reinterpret_cast<const uint4*>(dout + (long)(r / k) * H);
  const uint4* ys = reinterpret_cast<const uint4*>(y + (long)row * H);
  float dot = 0.f;
  for (int c = lane; c < H / 8; c += 32) {
    const uint4 v = src[c], yv = ys[c];
    const float d[8] = {bf16_lo(v.x), bf16_hi(v.x), bf16_lo(v.y), bf16_hi(v.y), bf16_lo(v.z), bf16_hi(v.z), bf16_lo(v.w), bf16_hi(v.w)};
    const float q[8] = {bf16_lo(yv.x), bf16_hi(yv.x), bf16_lo(yv.y), bf16_hi(yv.y), bf16_lo(yv.z), bf16_hi(yv.z), bf16_lo(yv.w), bf16_hi(yv.w)};
#pragma unroll
    for (int j = 0; j < 8; ++j) dot = fmaf(d[j], q[j], dot);
    uint4 o;
    o.x = pack_bf16(g * d[0], g * d[1]); o.y = pack_bf16(g * d[2], g * d[3]);
    o.z = pack_bf16(g * d[4], g * d[5]); o.w = pack_bf16(g * d[6], g * d[7]);
    dst[c] = o;
  }
  dot = warp_sum(dot);
  if (lane == 0) dgates[r] = dot;
}

// Backward of gather: dx[t, :] = sum_slot drouted[dest[t*k+slot], :]. One warp per token.
__global__ void moe_gather_bwd_kernel(const __nv_bfloat16* __restrict__ drouted, const int* __restrict__ dest,
                                      __nv_bfloat16* __restrict__ dx, int T, int H, int k) {
  const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5;
  const int lane = threadIdx.x & 31;
  if (t >= T) return;
  for (int c = lane; c < H / 8; c += 32) {
    float acc[8] = {0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f, 0.f};
    for (int s = 0; s < k; ++s) {
      const uint4 v = reinterpret_cast<const uint4*>(drouted + (long)dest[(long)t * k + s] * H)[c];
      acc[0] += bf16_lo(v.x); acc[1] += bf16_hi(v.x); acc[2] += bf16_lo(v.y); acc[3] += bf16_hi(v.y);
      acc[4] += bf16_lo(v.z); acc[5] += bf16_hi(v.z); acc[6] += bf16_lo(v.w); acc[7] += bf16_hi(v.w);
    }
    uint4 o;
    o.x = pack_bf16(acc[0], acc[1]); o.y = pack_bf16(acc[2], acc[3]); o.z = pack_bf16(acc[4], acc[5]); o.w = pack_bf16(acc[6], acc[7]);
    reinterpret_cast<uint4*>(dx + (long)t * H)[c] = o;
  }
}


// ---------------------------------------------------------------------------- router auxiliary loss
// aux = lb_w * E * sum_e mean_t(p[t,e]) * frac_e + z_w * mean_t(lse_t^2), p = softmax over all experts of the fp32
// router logits, frac_e = routes to expert e / (T k) (a constant for the gradient). One warp per row, lane l owns
// experts l, l + 32, ... (E <= 256). Forward: per-CTA partial sums of p and of lse^2 go to `partial[cta][E + 1]`
// (no atomics: the finish kernel adds them in a fixed order, so the loss is bit-reproducible), lse is kept per row.
constexpr int AUX_ROWS = 64;       // rows per CTA (8 warps x 8 rows)

__global__ void __launch_bounds__(256)
moe_aux_fwd_kernel(const float* __restrict__ logits, float* __restrict__ lse_out, float* __restrict__ partial, int T, int E) {
  __shared__ float s_p[8][256];
  __shared__ float s_z[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  float psum[8], z = 0.f;
#pragma unroll
  for (int j = 0; j < 8; ++j) psum[j] = 0.f;
  for (int r = warp; r < AUX_ROWS; r += 8) {
    const int t = blockIdx.x * AUX_ROWS + r;
    if (t >= T) break;
    const float* row = logits + (long)t * E;
    float v[8], mx = -INFINITY;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      v[j] = e < E ? row[e] : -INFINITY;
      mx = fmaxf(mx, v[j]);
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
    float sum = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) { v[j] = lane + 32 * j < E ? __expf(v[j] - mx) : 0.f; sum += v[j]; }
#pragma unroll
    for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const float inv = 1.f / sum, lse = mx + __logf(sum);
#pragma unroll
    for (int j = 0; j < 8; ++j) psum[j] += v[j] * inv;
    if (lane == 0) { lse_out[t] = lse; z += lse * lse; }
  }
#pragma unroll
  for (int j = 0; j < 8; ++j) s_p[warp][lane + 32 * j] = psum[j];
  if (lane == 0) s_z[warp] = z;
  __syncthreads();
  float* out = partial + (long)blockIdx.x * (E + 1);
  if ((int)threadIdx.x < E) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += s_p[w][threadIdx.x];
    out[threadIdx.x] = a;
  }
  if (threadIdx.x == 0) {
    float a = 0.f;
#pragma unroll
    for (int w = 0; w < 8; ++w) a += s_z[w];
    out[E] = a;
  }
}

// One CTA: aux and the per-expert gradient coefficients coef[e] = lb_w * E * frac_e / T.
__global__ void __launch_bounds__(256)
moe_aux_finish_kernel(const float* __restrict__ partial, const int* __restrict__ counts, float* __restrict__ coef,
                      float* __restrict__ aux, int n_cta, int T, int E, int k, float lb_w, float z_w) {
  __shared__ float s_red[256];
  const int e = threadIdx.x;
  float term = 0.f;
  if (e < E) {
    float p = 0.f;
    for (int c = 0; c < n_cta; ++c) p += partial[(long)c * (E + 1) + e];
    const float frac = (float)counts[e] / ((float)T * (float)k);
    const float ce = lb_w * (float)E * frac / (float)T;
    coef[e] = ce;
    term = ce * p;
  }
  s_red[threadIdx.x] = term;
  __syncthreads();
  for (int o = 128; o; o >>= 1) {
    if ((int)threadIdx.x < o) s_red[threadIdx.x] += s_red[threadIdx.x + o];
    __syncthreads();
  }
  if (threadIdx.x == 0) {
    float z = 0.f;
    for (int c = 0; c < n_cta; ++c) z += partial[(long)c * (E + 1) + E];
    aux[0] = s_red[0] + z_w * z / (float)T;
  }
}

// d aux / d logits[t, j] = gout * p_j * (coef_j - sum_e coef_e p_e + 2 z_w lse_t / T)
__global__ void __launch_bounds__(256)
moe_aux_bwd_kernel(const float* __restrict__ logits, const float* __restrict__ lse, const float* __restrict__ coef,
                   const float* __restrict__ gout, float* __restrict__ grad, int T, int E, float z_w) {
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const float g = gout[0];
  float cf[8];
#pragma unroll
  for (int j = 0; j < 8; ++j) cf[j] = lane + 32 * j < E ? coef[lane + 32 * j] : 0.f;
  for (int r = warp; r < AUX_ROWS; r += 8) {
    const int t = blockIdx.x * AUX_ROWS + r;
    if (t >= T) break;
    const float* row = logits + (long)t * E;
    const float l = lse[t];
    float pv[8], dot = 0.f;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      pv[j] = e < E ? __expf(row[e] - l) : 0.f;
      dot += cf[j] * pv[j];
    }
#pragma unroll
    for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
    const float zc = 2.f * z_w * l / (float)T;
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const int e = lane + 32 * j;
      if (e < E) grad[(long)t * E + e] = g * pv[j] * (cf[j] - dot + zc);
    }
  }
}

}  // namespace sb

using namespace sb;

extern "C" int sb_router_logits(const void* x, const float* w, float* logits, int T, int H, int E, long ldx,
                                cudaStream_t st) {
  SB_CHECK_ARG(T > 0 && H > 0 && E >= 1 && E <= 256);
  router_logits_kernel<<<(T + 63) / 64, 256, 0, st>>>((const __nv_bfloat16*)x, w, logits, T, H, E, ldx);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Routing plan for `T` tokens with top-k over `E` experts (k <= 8, E <= 256).
//   idx[T,k] int32 out; counts[E] scratch (zeroed here); meta[E+2] = padded offsets + live
//   tile count; tile_expert[max_rows/128]; dest[T*k]; row_route[max_rows].
// max_rows must be >= T*k + E*128 rounded to 128 (the padded layout's worst case).
extern "C" int sb_moe_plan(const float* logits, int* idx, int* counts, int* meta, int* tile_expert, int* dest,
                           int* row_route, int T, int E, int k, int max_rows, cudaStream_t st) {
  SB_CHECK_ARG(T > 0 && E >= 2 && E <= 256 && k >= 1 && k <= 8 && k <= E);
  SB_CHECK_ARG(max_rows % 128 == 0 && (long)max_rows >= (long)T * k + (long)E * 127);
  SB_CHECK_CUDA(cudaMemsetAsync(counts, 0, sizeof(int) * E, st));
  const int blocks = (T + 7) / 8;
  if (E <= 32) moe_topk_kernel<1><<<blocks, 256, 0, st>>>(logits, idx, counts, T, E, k);
  else if (E <= 64) moe_topk_kernel<2><<<blocks, 256, 0, st>>>(logits, idx, counts, T, E, k);
  else if (E <= 128) moe_topk_kernel<4><<<blocks, 256, 0, st>>>(logits, idx, counts, T, E, k);
  else moe_topk_kernel<8><<<blocks, 256, 0, st>>>(logits, idx, counts, T, E, k);
  moe_offsets_kernel<<<1, 256, 0, st>>>(counts, meta, tile_expert, E, max_rows / 128);
  moe_pack_kernel<<<E, 256, 0, st>>>(idx, meta, dest, row_route, T * k);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_moe_gather(const void* x, const int* row_route, const int* meta, void* routed, int E, int H, int k,
                             long ldx, int max_rows, cudaStream_t st) {
  SB_CHECK_ARG(H % 8 == 0 && ldx % 8 == 0);
  moe_gather_kernel<<<(max_rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)x, row_route, meta, (__nv_bfloat16*)routed,
                                                        E, H, k, ldx, max_rows);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_moe_combine(const void* y, const int* dest, const float* gates, void* out, int T, int H, int k,
                              cudaStream_t st) {
  SB_CHECK_ARG(H % 8 == 0);
  moe_combine_kernel<<<(T + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)y, dest, gates, (__nv_bfloat16*)out, T, H, k);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_moe_combine_bwd(const void* dout, const void* y, const int* row_route, const float* gates,
                                  const int* meta, void* dy, float* dgates, int E, int H, int k, int max_rows,
                                  cudaStream_t st) {
  SB_CHECK_ARG(H % 8 == 0);
  moe_combine_bwd_kernel<<<(max_rows + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)dout, (const __nv_bfloat16*)y,
                                                            row_route, gates, meta, (__nv_bfloat16*)dy, dgates, E, H, k,
                                                            max_rows);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_moe_gather_bwd(const void* drouted, const int* dest, void* dx, int T, int H, int k, cudaStream_t st) {
  SB_CHECK_ARG(H % 8 == 0);
  moe_gather_bwd_kernel<<<(T + 7) / 8, 256, 0, st>>>((const __nv_bfloat16*)drouted, dest, (__nv_bfloat16*)dx, T, H, k);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

// Router auxiliary loss (load balance + z) of fp32 logits `[T, E]` (contiguous, E <= 256). `counts[E]`: routes per
// expert (the plan's histogram); `lse[T]`, `coef[E]`, `partial[ceil(T / 64) * (E + 1)]`: scratch kept for backward;
// `aux[1]`: the loss.
extern "C" int sb_moe_aux_fwd(const float* logits, const int* counts, float* lse, float* coef, float* partial, float* aux,
                              int T, int E, int k, float lb_w, float z_w, cudaStream_t st) {
  SB_CHECK_ARG(T > 0 && E >= 1 && E <= 256 && k >= 1);
  const int n_cta = (T + AUX_ROWS - 1) / AUX_ROWS;
  moe_aux_fwd_kernel<<<n_cta, 256, 0, st>>>(logits, lse, partial, T, E);
  moe_aux_finish_kernel<<<1, 256, 0, st>>>(partial, counts, coef, aux, n_cta, T, E, k, lb_w, z_w);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}

extern "C" int sb_moe_aux_bwd(const float* logits, const float* lse, const float* coef, const float* gout, float* grad,
                              int T, int E, float z_w, cudaStream_t st) {
  SB_CHECK_ARG(T > 0 && E >= 1 && E <= 256);
  moe_aux_bwd_kernel<<<(T + AUX_ROWS - 1) / AUX_ROWS, 256, 0, st>>>(logits, lse, coef, gout, grad, T, E, z_w);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
