// Slot gates of the callers, fused into one pass over the gate logits.
//
// The layers that call the operator turn the gate projection f [.., H, M] into the two gate tensors the operator
// takes, with a chain of element-wise torch kernels (nha_fla/layers/nha.py:229-231: logsigmoid, division by
// gate_logit_normalizer, exp, 1 - x, cast; the hybrid models compute s the same way,
// nha_fla/models/qwen3_nha/qwennha.py:116):
//     g = logsigmoid(f) / normalizer          log forget gate, <= 0
//     s = 1 - exp(g)                          slot write weight
// Here: one kernel reads f once and writes g and s (6 bytes per element instead of the chain's 18), one kernel
// for the backward (df from dg and ds).  fp32 arithmetic, one rounding to bf16 per output; s is computed from the
// ROUNDED g, as the reference computes it from its bf16 g, so that s and g stay consistent to the last bit the
// operator sees.  HBM-bound: 16-byte loads and stores, grid sized to the SM count.
#include "nha_common.cuh"

namespace nha {

constexpr int kGateThreads = 256;
constexpr int kGateVecPerThread = 4;       // 16-byte vectors in flight per thread

// log(1 + e) for e in (0, 1]: three series terms below 1e-3 (error < 3e-7 relative), the fast logarithm above (the
// rounding of 1 + e costs at most 6e-5 relative there); both far inside the bf16 rounding of the result.  The
// library's log1pf / expm1f made the forward compute-bound.
__device__ __forceinline__ float log1p_unit(float e) {
  return e < 1e-3f ? e * (1.0f - e * (0.5f - e * (1.0f / 3.0f))) : __logf(1.0f + e);
}
__device__ __forceinline__ float log_sigmoid(float x) {
  // min(x, 0) - log1p(exp(-|x|)); accurate for both tails
  return fminf(x, 0.0f) - log1p_unit(__expf(-fabsf(x)));
}
// 1 - exp(g) for g <= 0 without cancellation near 0
__device__ __forceinline__ float one_minus_exp(float g) {
  return g > -1e-2f ? -g * (1.0f + g * (0.5f + g * (1.0f / 6.0f))) : 1.0f - __expf(g);
}

__device__ __forceinline__ void gate_of(float f, float inv_norm, bf16& g_out, bf16& s_out) {
  const bf16 gb = f2bf(log_sigmoid(f) * inv_norm);
  g_out = gb;
  s_out = f2bf(one_minus_exp(bf2f(gb)));
}

__global__ void __launch_bounds__(kGateThreads) nha_slot_gates_fwd_kernel(const bf16* __restrict__ f, bf16* __restrict__ g,
                                                                          bf16* __restrict__ s, int64_t n, float inv_norm) {
  const int64_t nvec = n >> 3;
  const int64_t stride = (int64_t)gridDim.x * kGateThreads;
  const uint4* f4 = reinterpret_cast<const uint4*>(f);
  uint4* g4 = reinterpret_cast<uint4*>(g);
  uint4* s4 = reinterpret_cast<uint4*>(s);
  for (int64_t i0 = (int64_t)blockIdx.x * kGateThreads + threadIdx.x; i0 < nvec; i0 += stride * kGateVecPerThread) {
    uint4 in[kGateVecPerThread];
#pragma unroll
    for (int u = 0; u < kGateVecPerThread; ++u) {
      const int64_t i = i0 + u * stride;
      if (i < nvec) in[u] = __ldcs(f4 + i);
    }
#pragma unroll
    for (int u = 0; u < kGateVecPerThread; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= nvec) continue;
      const bf16* x = reinterpret_cast<const bf16*>(&in[u]);
      uint4 go, so;
      bf16* gp = reinterpret_cast<bf16*>(&go);
      bf16* sp = reinterpret_cast<bf16*>(&so);
#pragma unroll
      for (int e = 0; e < 8; ++e) gate_of(bf2f(x[e]), inv_norm, gp[e], sp[e]);
      g4[i] = go;
      if (s) s4[i] = so;
    }
  }
  // ragged tail (n not a multiple of 8)
  if (blockIdx.x == 0) {
    for (int64_t i = (nvec << 3) + threadIdx.x; i < n; i += kGateThreads) {
      bf16 gb, sb;
      gate_of(bf2f(f[i]), inv_norm, gb, sb);
      g[i] = gb;
      if (s) s[i] = sb;
    }
  }
}

// d f = (dg - ds * exp(g)) * sigmoid(-f) / normalizer      (d logsigmoid(f) / d f = sigmoid(-f); d s / d g = -exp(g))
__device__ __forceinline__ float gate_grad(float f, float dg, float ds, float inv_norm) {
  const float g = log_sigmoid(f) * inv_norm;
  const float sig = __fdividef(1.0f, 1.0f + __expf(fminf(f, 80.0f)));   // sigmoid(-f); the clamp keeps the divisor finite
  return (dg - ds * __expf(g)) * sig * inv_norm;
}

__global__ void __launch_bounds__(kGateThreads) nha_slot_gates_bwd_kernel(const bf16* __restrict__ f, const bf16* __restrict__ dg,
                                                                          const bf16* __restrict__ ds, bf16* __restrict__ df,
                                                                          int64_t n, float inv_norm) {
  const int64_t nvec = n >> 3;
  const int64_t stride = (int64_t)gridDim.x * kGateThreads;
  const uint4* f4 = reinterpret_cast<const uint4*>(f);
  const uint4* dg4 = reinterpret_cast<const uint4*>(dg);
  const uint4* ds4 = reinterpret_cast<const uint4*>(ds);
  uint4* df4 = reinterpret_cast<uint4*>(df);
  const uint4 zero = make_uint4(0u, 0u, 0u, 0u);
  for (int64_t i0 = (int64_t)blockIdx.x * kGateThreads + threadIdx.x; i0 < nvec; i0 += stride * 2) {
    uint4 fin[2], gin[2], sin_[2];
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t i = i0 + u * stride;
      fin[u] = gin[u] = sin_[u] = zero;
      if (i < nvec) {
        fin[u] = __ldcs(f4 + i);
        if (dg) gin[u] = __ldcs(dg4 + i);
        if (ds) sin_[u] = __ldcs(ds4 + i);
      }
    }
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int64_t i = i0 + u * stride;
      if (i >= nvec) continue;
      const bf16* x = reinterpret_cast<const bf16*>(&fin[u]);
      const bf16* a = reinterpret_cast<const bf16*>(&gin[u]);
      const bf16* b = reinterpret_cast<const bf16*>(&sin_[u]);
      uint4 out;
      bf16* op = reinterpret_cast<bf16*>(&out);
#pragma unroll
      for (int e = 0; e < 8; ++e) op[e] = f2bf(gate_grad(bf2f(x[e]), bf2f(a[e]), bf2f(b[e]), inv_norm));
      df4[i] = out;
    }
  }
  if (blockIdx.x == 0) {
    for (int64_t i = (nvec << 3) + threadIdx.x; i < n; i += kGateThreads)
      df[i] = f2bf(gate_grad(bf2f(f[i]), dg ? bf2f(dg[i]) : 0.0f, ds ? bf2f(ds[i]) : 0.0f, inv_norm));
  }
}

static int gate_grid(int64_t n, int vec_per_thread) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t per_cta = (int64_t)kGateThreads * 8 * vec_per_thread;
  const int64_t want = (n + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)sms * 8;                       // eight 256-thread CTAs per SM, whole waves
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}

static bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

}  // namespace nha

using namespace nha;

extern "C" int nha_slot_gates_fwd(const void* f, void* g, void* s, int64_t n, float normalizer, void* stream) {
  if (!f || !g || n < 0 || !(normalizer > 0.0f)) return NHA_ERR_BAD_ARG;
  if (!aligned16(f) || !aligned16(g) || !aligned16(s)) return NHA_ERR_BAD_ARG;
  if (n == 0) return NHA_OK;
  nha_slot_gates_fwd_kernel<<<gate_grid(n, kGateVecPerThread), kGateThreads, 0, (cudaStream_t)stream>>>(
      (const bf16*)f, (bf16*)g, (bf16*)s, n, 1.0f / normalizer);
  return check_launch();
}

extern "C" int nha_slot_gates_bwd(const void* f, const void* dg, const void* ds, void* df, int64_t n, float normalizer,
                                  void* stream) {
  if (!f || !df || (!dg && !ds) || n < 0 || !(normalizer > 0.0f)) return NHA_ERR_BAD_ARG;
  if (!aligned16(f) || !aligned16(dg) || !aligned16(ds) || !aligned16(df)) return NHA_ERR_BAD_ARG;
  if (n == 0) return NHA_OK;
  nha_slot_gates_bwd_kernel<<<gate_grid(n, 2), kGateThreads, 0, (cudaStream_t)stream>>>(
      (const bf16*)f, (const bf16*)dg, (const bf16*)ds, (bf16*)df, n, 1.0f / normalizer);
  return check_launch();
}
