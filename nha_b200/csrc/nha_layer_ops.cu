// Element-wise work of the calling layer on either side of the operator, one pass each (sm_100a, HBM-bound).
//
//   * Feature map and value activation (nha_fla/layers/nha.py:219-223): q_gsa = swish(q), k_gsa = swish(k),
//     v = silu(v) - the layer launches three element-wise torch kernels (SwishFeatureMap is x * sigmoid(x), the
//     same function as silu; feature_map='relu' is max(x, 0)).  nha_act3_fwd / nha_act3_bwd take up to three tensors
//     in ONE launch.
//   * Output side (nha_fla/layers/nha.py:277-278): o = rms_norm_linear(silu(o), g_norm.weight, g_norm.bias,
//     o_proj.weight, o_proj.bias).  nha_silu_rmsnorm_fwd / _bwd fuse silu, the RMS normalisation and its affine part
//     into one pass over the rows (one warp per row, the row held in registers), leaving the projection itself to the
//     GEMM library.  The backward also produces the gradients of the norm's weight and bias: per-CTA column sums in
//     registers, written as partial rows that the host side adds up.
//
// fp32 arithmetic, one rounding to bf16 per output, 16-byte accesses, grids sized to whole waves of the SM count.
#include "nha_common.cuh"

namespace nha {

constexpr int kActThreads = 256;

struct Act3 {
  const bf16* x[3];
  const bf16* dy[3];
  bf16* y[3];
  int64_t n[3];
  int relu[3];       // 1: max(x, 0) instead of x * sigmoid(x)
};

__device__ __forceinline__ float sigmoid_fast(float x) { return __fdividef(1.0f, 1.0f + __expf(-x)); }
__device__ __forceinline__ float act_fwd(float x, int relu) { return relu ? fmaxf(x, 0.0f) : x * sigmoid_fast(x); }
// d/dx x sigmoid(x) = sigmoid(x) (1 + x (1 - sigmoid(x)))
__device__ __forceinline__ float act_grad(float x, float dy, int relu) {
  if (relu) return x > 0.0f ? dy : 0.0f;
  const float s = sigmoid_fast(x);
  return dy * s * (1.0f + x * (1.0f - s));
}

template <bool BWD>
__global__ void __launch_bounds__(kActThreads) nha_act3_kernel(const Act3 a) {
#pragma unroll 1
  for (int t = 0; t < 3; ++t) {
    const int64_t n = a.n[t];
    if (n <= 0) continue;
    const int relu = a.relu[t];
    const int64_t nvec = n >> 3;
    const int64_t stride = (int64_t)gridDim.x * kActThreads;
    const uint4* x4 = reinterpret_cast<const uint4*>(a.x[t]);
    const uint4* d4 = reinterpret_cast<const uint4*>(a.dy[t]);
    uint4* y4 = reinterpret_cast<uint4*>(a.y[t]);
    for (int64_t i0 = (int64_t)blockIdx.x * kActThreads + threadIdx.x; i0 < nvec; i0 += stride * 4) {
      uint4 xin[4], din[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = i0 + u * stride;
        if (i < nvec) {
          xin[u] = __ldcs(x4 + i);
          if (BWD) din[u] = __ldcs(d4 + i);
        }
      }
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int64_t i = i0 + u * stride;
        if (i >= nvec) continue;
        float xv[8], dv[8], out[8];
        unpack8(xin[u], xv);
        if (BWD) unpack8(din[u], dv);
#pragma unroll
        for (int e = 0; e < 8; ++e) out[e] = BWD ? act_grad(xv[e], dv[e], relu) : act_fwd(xv[e], relu);
        y4[i] = pack8(out);
      }
    }
    if (blockIdx.x == 0) {                      // ragged tail (n not a multiple of 8)
      for (int64_t i = (nvec << 3) + threadIdx.x; i < n; i += kActThreads) {
        const float xv = bf2f(a.x[t][i]);
        a.y[t][i] = f2bf(BWD ? act_grad(xv, bf2f(a.dy[t][i]), relu) : act_fwd(xv, relu));
      }
    }
  }
}

static int wave_grid(int64_t work_items, int64_t per_cta, int ctas_per_sm) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t want = (work_items + per_cta - 1) / per_cta;
  const int64_t cap = (int64_t)sms * ctas_per_sm;
  return (int)(want < 1 ? 1 : (want < cap ? want : cap));
}
static bool aligned16(const void* p) { return ((uintptr_t)p & 15u) == 0; }

// ---------------------------------------------------------------------------------------------
// y = rmsnorm(silu(o)) * w + b, one warp per row.  PIECES = cols / 256: 16-byte pieces of the row per lane.
constexpr int kNormThreads = 256;
constexpr int kNormWarps = kNormThreads / 32;

template <int PIECES>
__global__ void __launch_bounds__(kNormThreads) nha_silu_rmsnorm_fwd_kernel(const bf16* __restrict__ o, const float* __restrict__ w,
                                                                            const float* __restrict__ b, bf16* __restrict__ y,
                                                                            float* __restrict__ rstd, int64_t rows, int cols,
                                                                            float eps) {
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wstride = (int64_t)gridDim.x * kNormWarps;
  for (int64_t r = (int64_t)blockIdx.x * kNormWarps + warp; r < rows; r += wstride) {
    const uint4* src = reinterpret_cast<const uint4*>(o + r * cols);
    uint4 in[PIECES];
#pragma unroll
    for (int p = 0; p < PIECES; ++p) in[p] = __ldcs(src + lane + 32 * p);
    float x[PIECES][8];
    float ss = 0.f;
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      unpack8(in[p], x[p]);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        x[p][e] = x[p][e] * sigmoid_fast(x[p][e]);
        ss += x[p][e] * x[p][e];
      }
    }
    ss = warp_sum(ss);
    const float rs = rsqrtf(ss / (float)cols + eps);
    if (lane == 0 && rstd) rstd[r] = rs;
    uint4* dst = reinterpret_cast<uint4*>(y + r * cols);
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int c = 8 * (lane + 32 * p);
      const float4 w0 = *reinterpret_cast<const float4*>(w + c), w1 = *reinterpret_cast<const float4*>(w + c + 4);
      float4 b0 = make_float4(0.f, 0.f, 0.f, 0.f), b1 = b0;
      if (b) {
        b0 = *reinterpret_cast<const float4*>(b + c);
        b1 = *reinterpret_cast<const float4*>(b + c + 4);
      }
      float out[8];
      out[0] = x[p][0] * rs * w0.x + b0.x; out[1] = x[p][1] * rs * w0.y + b0.y;
      out[2] = x[p][2] * rs * w0.z + b0.z; out[3] = x[p][3] * rs * w0.w + b0.w;
      out[4] = x[p][4] * rs * w1.x + b1.x; out[5] = x[p][5] * rs * w1.y + b1.y;
      out[6] = x[p][6] * rs * w1.z + b1.z; out[7] = x[p][7] * rs * w1.w + b1.w;
      dst[lane + 32 * p] = pack8(out);
    }
  }
}

// Backward of the above for dy (gradient of y).  With x = silu(o), xh = x rstd, dyh = dy w, c = mean(dyh xh):
//     dx = (dyh - xh c) rstd,  do = dx silu'(o),  dw[j] += dy xh,  db[j] += dy.
// dw / db: per-thread sums over the rows of this CTA's warps (in registers up to 1024 columns, beyond that in the
// warp's own row of shared memory: a lane owns its columns, so plain read-modify-writes suffice), combined across the
// CTA's warps in shared memory and written as one partial row per CTA (part_w, part_b [gridDim.x][cols] fp32).
template <int PIECES, bool SMEM_ACC = (PIECES > 4)>
__global__ void __launch_bounds__(kNormThreads) nha_silu_rmsnorm_bwd_kernel(const bf16* __restrict__ o, const float* __restrict__ w,
                                                                            const float* __restrict__ rstd,
                                                                            const bf16* __restrict__ dy, bf16* __restrict__ d_o,
                                                                            float* __restrict__ part_w, float* __restrict__ part_b,
                                                                            int64_t rows, int cols) {
  extern __shared__ float red[];                       // [kNormWarps][cols] twice
  const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
  const int64_t wstride = (int64_t)gridDim.x * kNormWarps;
  constexpr int ACC = SMEM_ACC ? 1 : PIECES;
  float aw[ACC][8], ab[ACC][8];
  float* rw = red;
  float* rb = red + kNormWarps * cols;
#pragma unroll
  for (int p = 0; p < PIECES; ++p)
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      if (SMEM_ACC) {
        rw[warp * cols + 8 * (lane + 32 * p) + e] = 0.f;
        rb[warp * cols + 8 * (lane + 32 * p) + e] = 0.f;
      } else {
        aw[p % ACC][e] = ab[p % ACC][e] = 0.f;
      }
    }
  for (int64_t r = (int64_t)blockIdx.x * kNormWarps + warp; r < rows; r += wstride) {
    const uint4* so = reinterpret_cast<const uint4*>(o + r * cols);
    const uint4* sd = reinterpret_cast<const uint4*>(dy + r * cols);
    uint4 oin[PIECES], din[PIECES];
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      oin[p] = __ldcs(so + lane + 32 * p);
      din[p] = __ldcs(sd + lane + 32 * p);
    }
    const float rs = rstd[r];
    float cs = 0.f;
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int c = 8 * (lane + 32 * p);
      const float4 w0 = *reinterpret_cast<const float4*>(w + c), w1 = *reinterpret_cast<const float4*>(w + c + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float ov[8], dv[8];
      unpack8(oin[p], ov);
      unpack8(din[p], dv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = ov[e] * sigmoid_fast(ov[e]) * rs;
        cs += dv[e] * wv[e] * xh;
        if (SMEM_ACC) {
          rw[warp * cols + c + e] += dv[e] * xh;
          rb[warp * cols + c + e] += dv[e];
        } else {
          aw[p % ACC][e] += dv[e] * xh;
          ab[p % ACC][e] += dv[e];
        }
      }
    }
    cs = warp_sum(cs) / (float)cols;
    // second sweep over the row in registers: xh and dyh are recomputed rather than kept (registers)
    uint4* dst = reinterpret_cast<uint4*>(d_o + r * cols);
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int c = 8 * (lane + 32 * p);
      const float4 w0 = *reinterpret_cast<const float4*>(w + c), w1 = *reinterpret_cast<const float4*>(w + c + 4);
      const float wv[8] = {w0.x, w0.y, w0.z, w0.w, w1.x, w1.y, w1.z, w1.w};
      float ov[8], dv[8], out[8];
      unpack8(oin[p], ov);
      unpack8(din[p], dv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const float xh = ov[e] * sigmoid_fast(ov[e]) * rs;
        out[e] = act_grad(ov[e], (dv[e] * wv[e] - xh * cs) * rs, 0);
      }
      dst[lane + 32 * p] = pack8(out);
    }
  }
  if (!SMEM_ACC) {
#pragma unroll
    for (int p = 0; p < PIECES; ++p) {
      const int c = 8 * (lane + 32 * p);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        rw[warp * cols + c + e] = aw[p % ACC][e];
        rb[warp * cols + c + e] = ab[p % ACC][e];
      }
    }
  }
  __syncthreads();
  for (int c = threadIdx.x; c < cols; c += kNormThreads) {
    float sw = 0.f, sb = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < kNormWarps; ++w8) {
      sw += rw[w8 * cols + c];
      sb += rb[w8 * cols + c];
    }
    part_w[(size_t)blockIdx.x * cols + c] = sw;
    if (part_b) part_b[(size_t)blockIdx.x * cols + c] = sb;
  }
}

static int norm_grid(int64_t rows, int ctas_per_sm) { return wave_grid(rows, kNormWarps, ctas_per_sm); }

}  // namespace nha

using namespace nha;

static int act3_launch(bool bwd, const void* const* x, const void* const* dy, void* const* y, const int64_t* n, const int* relu,
                       int count, void* stream) {
  if (count < 1 || count > 3 || !x || !y || !n) return NHA_ERR_BAD_ARG;
  Act3 a;
  int64_t total = 0;
  for (int t = 0; t < 3; ++t) {
    a.x[t] = nullptr; a.dy[t] = nullptr; a.y[t] = nullptr; a.n[t] = 0; a.relu[t] = 0;
    if (t >= count) continue;
    if (n[t] < 0) return NHA_ERR_BAD_ARG;
    if (n[t] == 0) continue;
    if (!x[t] || !y[t] || (bwd && (!dy || !dy[t]))) return NHA_ERR_BAD_ARG;
    if (!aligned16(x[t]) || !aligned16(y[t]) || (bwd && !aligned16(dy[t]))) return NHA_ERR_BAD_ARG;
    a.x[t] = (const bf16*)x[t]; a.y[t] = (bf16*)y[t]; a.n[t] = n[t];
    if (bwd) a.dy[t] = (const bf16*)dy[t];
    a.relu[t] = relu ? relu[t] : 0;
    total = total > n[t] ? total : n[t];
  }
  if (total == 0) return NHA_OK;
  const int grid = wave_grid(total, (int64_t)kActThreads * 8 * 4, 8);
  if (bwd) nha_act3_kernel<true><<<grid, kActThreads, 0, (cudaStream_t)stream>>>(a);
  else nha_act3_kernel<false><<<grid, kActThreads, 0, (cudaStream_t)stream>>>(a);
  return check_launch();
}

extern "C" int nha_act3_fwd(const void* const* x, void* const* y, const int64_t* n, const int* relu, int count, void* stream) {
  return act3_launch(false, x, nullptr, y, n, relu, count, stream);
}
extern "C" int nha_act3_bwd(const void* const* x, const void* const* dy, void* const* dx, const int64_t* n, const int* relu,
                            int count, void* stream) {
  return act3_launch(true, x, dy, dx, n, relu, count, stream);
}

extern "C" int nha_silu_rmsnorm_fwd(const void* o, const float* weight, const float* bias, void* y, float* rstd, int64_t rows,
                                    int cols, float eps, void* stream) {
  if (!o || !weight || !y || rows < 0 || cols <= 0 || !(eps >= 0.0f)) return NHA_ERR_BAD_ARG;
  if (cols % 256 || cols > 2048) return NHA_ERR_UNSUPPORTED;
  if (!aligned16(o) || !aligned16(y) || !aligned16(weight) || !aligned16(bias)) return NHA_ERR_BAD_ARG;
  if (rows == 0) return NHA_OK;
  const int grid = norm_grid(rows, 8);
  cudaStream_t cs = (cudaStream_t)stream;
#define NHA_NORM_FWD(P)                                                                                                  \
  case P:                                                                                                                \
    nha_silu_rmsnorm_fwd_kernel<P><<<grid, kNormThreads, 0, cs>>>((const bf16*)o, weight, bias, (bf16*)y, rstd, rows, cols, eps); \
    break;
  switch (cols / 256) {
    NHA_NORM_FWD(1) NHA_NORM_FWD(2) NHA_NORM_FWD(3) NHA_NORM_FWD(4) NHA_NORM_FWD(5) NHA_NORM_FWD(6) NHA_NORM_FWD(7) NHA_NORM_FWD(8)
    default: return NHA_ERR_UNSUPPORTED;
  }
#undef NHA_NORM_FWD
  return check_launch();
}

extern "C" int nha_silu_rmsnorm_bwd_ctas(int64_t rows) { return rows <= 0 ? 0 : norm_grid(rows, 2); }

extern "C" int nha_silu_rmsnorm_bwd(const void* o, const float* weight, const float* rstd, const void* dy, void* d_o,
                                    float* part_w, float* part_b, int64_t rows, int cols, void* stream) {
  if (!o || !weight || !rstd || !dy || !d_o || !part_w || rows < 0 || cols <= 0) return NHA_ERR_BAD_ARG;
  if (cols % 256 || cols > 2048) return NHA_ERR_UNSUPPORTED;
  if (!aligned16(o) || !aligned16(dy) || !aligned16(d_o) || !aligned16(weight)) return NHA_ERR_BAD_ARG;
  if (rows == 0) return NHA_OK;
  const int grid = norm_grid(rows, 2);
  const int smem = 2 * kNormWarps * cols * (int)sizeof(float);
  cudaStream_t cs = (cudaStream_t)stream;
#define NHA_NORM_BWD(P)                                                                                                \
  case P: {                                                                                                            \
    cudaError_t e = set_max_smem((const void*)nha_silu_rmsnorm_bwd_kernel<P>, smem);                                   \
    if (e != cudaSuccess) return record_cuda_error(e);                                                                 \
    nha_silu_rmsnorm_bwd_kernel<P><<<grid, kNormThreads, smem, cs>>>((const bf16*)o, weight, rstd, (const bf16*)dy,    \
                                                                     (bf16*)d_o, part_w, part_b, rows, cols);          \
  } break;
  switch (cols / 256) {
    NHA_NORM_BWD(1) NHA_NORM_BWD(2) NHA_NORM_BWD(3) NHA_NORM_BWD(4) NHA_NORM_BWD(5) NHA_NORM_BWD(6) NHA_NORM_BWD(7) NHA_NORM_BWD(8)
    default: return NHA_ERR_UNSUPPORTED;
  }
#undef NHA_NORM_BWD
  return check_launch();
}
