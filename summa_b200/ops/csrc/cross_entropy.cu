// Row kernels of the fused (chunked) linear cross-entropy: given a chunk of fp32 logits
// `[rows, Vpad]` produced by the tcgen05 GEMM, one block per row computes the online
// (max, sum-exp) over the LOGICAL vocabulary, the row loss, and — in the same launch, while
// the row is still in L2 — the gradient (softmax - onehot) * scale as bf16 with exact
// zeros in the padded columns. The surrounding GEMMs (logits, dH = G W^T, dW += H^T G) run
// on the tensor-core GEMM, so full-vocabulary logits exist only one chunk at a time.
#include "host_util.h"
#include "sm100.cuh"

namespace sb {

__global__ void __launch_bounds__(256)
ce_row_kernel(const float* __restrict__ logits, const long* __restrict__ targets, float* __restrict__ row_loss,
              __nv_bfloat16* __restrict__ grad, int vocab, int vpad, long ld_logits, long ld_grad, float grad_scale) {
  const int row = blockIdx.x;
  const float* lr = logits + static_cast<size_t>(row) * ld_logits;
  const int tid = threadIdx.x;
  // pass 1: online max / sum over float4 lanes
  float m = -INFINITY, s = 0.f;
  const int v4 = vocab >> 2;
  for (int i = tid; i < v4; i += 256) {
    const float4 x = *reinterpret_cast<const float4*>(lr + 4 * i);
    const float mx = fmaxf(fmaxf(x.x, x.y), fmaxf(x.z, x.w));
    if (mx > m) { s *= __expf(m - mx); m = mx; }
    s += __expf(x.x - m) + __expf(x.y - m) + __expf(x.z - m) + __expf(x.w - m);
  }
  for (int i = (v4 << 2) + tid; i < vocab; i += 256) {
    const float x = lr[i];
    if (x > m) { s *= __expf(m - x); m = x; }
    s += __expf(x - m);
  }
  __shared__ float sm[8], ss[8];
  __shared__ float lse_sh;
  // warp then block combine of (m, s)
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    const float om = __shfl_xor_sync(0xffffffffu, m, o);
    const float os = __shfl_xor_sync(0xffffffffu, s, o);
    const float nm = fmaxf(m, om);
    s = (m == -INFINITY ? 0.f : s * __expf(m - nm)) + (om == -INFINITY ? 0.f : os * __expf(om - nm));
    m = nm;
  }
  if ((tid & 31) == 0) { sm[tid >> 5] = m; ss[tid >> 5] = s; }
  __syncthreads();
  if (tid == 0) {
    float M = sm[0], S = ss[0];
    for (int w = 1; w < 8; ++w) {
      const float nm = fmaxf(M, sm[w]);
      S = (M == -INFINITY ? 0.f : S * __expf(M - nm)) + (sm[w] == -INFINITY ? 0.f : ss[w] * __expf(sm[w] - nm));
      M = nm;
    }
    const float lse = M + __logf(S);
    lse_sh = lse;
    const long tgt = targets[row];
    row_loss[row] = (tgt >= 0 && tgt < vocab) ? lse - lr[tgt] : 0.f;
  }
  __syncthreads();
  if (grad == nullptr) return;
  const float lse = lse_sh;
  const long tgt = targets[row];
  __nv_bfloat16* gr = grad + static_cast<size_t>(row) * ld_grad;
  const bool live = tgt >= 0 && tgt < vocab;
  for (int c = tid * 8; c < vpad; c += 256 * 8) {
    float g[8];
#pragma unroll
    for (int k = 0; k < 8; ++k) {
      const int col = c + k;
      float v = 0.f;
      if (col < vocab && live) {
        v = __expf(lr[col] - lse);
        if (col == tgt) v -= 1.f;
        v *= grad_scale;
      }
      g[k] = v;
    }
    uint4 w;
    w.x = pack_bf16(g[0], g[1]); w.y = pack_bf16(g[2], g[3]); w.z = pack_bf16(g[4], g[5]); w.w = pack_bf16(g[6], g[7]);
    *reinterpret_cast<uint4*>(gr + c) = w;
  }
}

}  // namespace sb

// logits `[rows, >=vocab]` fp32 (row stride ld_logits, multiple of 4), targets int64
// (negative = ignored row), row_loss `[rows]`, grad `[rows, vpad]` bf16 or null
// (row stride ld_grad, multiple of 8; vpad % 8 == 0).
extern "C" int sb_ce_rows(const float* logits, const long* targets, float* row_loss, void* grad, int rows, int vocab,
                          int vpad, long ld_logits, long ld_grad, float grad_scale, cudaStream_t st) {
  using namespace sb;
  SB_CHECK_ARG(rows > 0 && vocab > 0 && vpad >= vocab && vpad % 8 == 0 && ld_logits % 4 == 0 && ld_grad % 8 == 0);
  ce_row_kernel<<<rows, 256, 0, st>>>(logits, targets, row_loss, (__nv_bfloat16*)grad, vocab, vpad, ld_logits, ld_grad,
                                      grad_scale);
  SB_CHECK_CUDA(cudaGetLastError());
  return SB_OK;
}
