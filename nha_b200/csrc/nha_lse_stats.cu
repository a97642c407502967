// Layer-side consumers of the operator's two log-sum-exps, fused.
//
// In training the layer turns lse_swa and lse_gsa [T, HQ] into two scalars with a chain of a dozen element-wise and
// reduction kernels (nha_fla/layers/nha.py:255-264, 288-323):
//     delta      = lse_gsa - lse_swa
//     gsa_ratio  = mean(w_gsa / (w_swa + w_gsa)),  w_x = exp(lse_x - max(lse_swa, lse_gsa))   = mean(sigmoid(delta))
//     aux_loss   = mean(binary_cross_entropy_with_logits(delta, target))
//                = mean(max(delta, 0) - delta * target + log1p(exp(-|delta|)))
// and autograd sends  d aux_loss / d lse_gsa = (sigmoid(delta) - target) / n  back into the operator (lse_swa is
// detached there).  Here: one launch for both means (every CTA sums a slice in a fixed order and writes its two
// partial sums; the last CTA to arrive, told by a ticket it resets, adds the partials in index order, so the
// result does not depend on the order in which CTAs finish), one element-wise launch for the gradient.
#include "nha_common.cuh"

namespace nha {

constexpr int kLseThreads = 256;
constexpr int kLseMaxCtas = 256;

__device__ __forceinline__ float block_sum(float v, float* red) {
  v = warp_sum(v);
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  __syncthreads();
  if (lane == 0) red[warp] = v;
  __syncthreads();
  float t = 0.f;
  if (warp == 0) {
    t = lane < kLseThreads / 32 ? red[lane] : 0.f;
    t = warp_sum(t);
  }
  return t;                                                        // valid in warp 0
}

// scratch: [0] ticket (as int), [1 .. 2*kLseMaxCtas] partial sums; out: [0] aux loss, [1] gsa ratio
__global__ void __launch_bounds__(kLseThreads) nha_lse_stats_kernel(const float* __restrict__ lse_swa,
                                                                    const float* __restrict__ lse_gsa, int64_t n, float target,
                                                                    float* __restrict__ out, float* __restrict__ scratch) {
  __shared__ float red[kLseThreads / 32];
  __shared__ int last;
  float loss = 0.f, ratio = 0.f;
  for (int64_t i = (int64_t)blockIdx.x * kLseThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLseThreads) {
    const float d = lse_gsa[i] - lse_swa[i];
    const float e = __expf(-fabsf(d));
    const float sp = e < 1e-3f ? e * (1.0f - e * (0.5f - e * (1.0f / 3.0f))) : __logf(1.0f + e);      // log1p(e)
    loss += fmaxf(d, 0.f) - d * target + sp;
    ratio += d >= 0.f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);                          // sigmoid(d)
  }
  const float bl = block_sum(loss, red);
  const float br = block_sum(ratio, red);
  if (threadIdx.x == 0) {
    scratch[1 + 2 * blockIdx.x] = bl;
    scratch[2 + 2 * blockIdx.x] = br;
    __threadfence();
    const int t = atomicAdd(reinterpret_cast<int*>(scratch), 1);
    last = t == (int)gridDim.x - 1;
  }
  __syncthreads();
  if (!last) return;
  __threadfence();
  float tl = 0.f, tr = 0.f;
  if (threadIdx.x < 32) {
    // 32 lanes, each over its own partials in index order, then a fixed shuffle tree
    for (int c = threadIdx.x; c < (int)gridDim.x; c += 32) {
      tl += __ldcg(scratch + 1 + 2 * c);
      tr += __ldcg(scratch + 2 + 2 * c);
    }
    tl = warp_sum(tl);
    tr = warp_sum(tr);
    if (threadIdx.x == 0) {
      out[0] = tl / (float)n;
      out[1] = tr / (float)n;
      *reinterpret_cast<int*>(scratch) = 0;                        // the next call starts from a clear ticket
    }
  }
}

// d_lse_gsa[i] = dloss * (sigmoid(delta_i) - target) / n
__global__ void __launch_bounds__(kLseThreads) nha_lse_aux_grad_kernel(const float* __restrict__ lse_swa,
                                                                       const float* __restrict__ lse_gsa,
                                                                       const float* __restrict__ dloss, int64_t n, float target,
                                                                       float* __restrict__ d_lse_gsa) {
  const float c = dloss[0] / (float)n;
  for (int64_t i = (int64_t)blockIdx.x * kLseThreads + threadIdx.x; i < n; i += (int64_t)gridDim.x * kLseThreads) {
    const float d = lse_gsa[i] - lse_swa[i];
    const float e = __expf(-fabsf(d));
    const float sig = d >= 0.f ? __fdividef(1.0f, 1.0f + e) : __fdividef(e, 1.0f + e);
    d_lse_gsa[i] = c * (sig - target);
  }
}

static int lse_grid(int64_t n) {
  const int64_t want = (n + kLseThreads * 8 - 1) / (kLseThreads * 8);
  return (int)(want < 1 ? 1 : (want < kLseMaxCtas ? want : kLseMaxCtas));
}

}  // namespace nha

using namespace nha;

extern "C" int64_t nha_lse_stats_scratch_bytes(void) { return (1 + 2 * kLseMaxCtas) * (int64_t)sizeof(float); }

extern "C" int nha_lse_stats(const float* lse_swa, const float* lse_gsa, int64_t n, float target, float* out, void* scratch,
                             void* stream) {
  if (!lse_swa || !lse_gsa || !out || !scratch || n <= 0) return NHA_ERR_BAD_ARG;
  nha_lse_stats_kernel<<<lse_grid(n), kLseThreads, 0, (cudaStream_t)stream>>>(lse_swa, lse_gsa, n, target, out,
                                                                             (float*)scratch);
  return check_launch();
}

extern "C" int nha_lse_aux_grad(const float* lse_swa, const float* lse_gsa, const float* dloss, int64_t n, float target,
                                float* d_lse_gsa, void* stream) {
  if (!lse_swa || !lse_gsa || !dloss || !d_lse_gsa || n <= 0) return NHA_ERR_BAD_ARG;
  const int64_t want = (n + kLseThreads * 4 - 1) / (kLseThreads * 4);
  const int grid = (int)(want < 1 ? 1 : (want < 148 * 8 ? want : 148 * 8));
  nha_lse_aux_grad_kernel<<<grid, kLseThreads, 0, (cudaStream_t)stream>>>(lse_swa, lse_gsa, dloss, n, target, d_lse_gsa);
  return check_launch();
}
