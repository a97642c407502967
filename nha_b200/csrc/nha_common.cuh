// Shared device helpers of the NHA kernels (sm_100a).
#pragma once

#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <mma.h>
#include <stdint.h>

#include "../../include/nha_b200.h"

namespace nha {

typedef __nv_bfloat16 bf16;

constexpr int kChunk = NHA_CHUNK;       // tokens per chunk
constexpr int kBlock = 16;              // row block inside a chunk (one decay reference per block and slot)
constexpr float kExpClamp = 75.0f;      // exponent clamp of the factorised decays
constexpr int kMaxSmem = 227 * 1024;

// ---- status plumbing -------------------------------------------------------------------------
int record_cuda_error(cudaError_t e);   // stores the text for nha_last_cuda_error(), returns NHA_ERR_LAUNCH
int check_launch();                     // cudaGetLastError() -> status
// raises a kernel's dynamic shared-memory limit; remembered per (device, kernel), so the runtime is asked only
// the first time or when more is needed
cudaError_t set_max_smem(const void* func, int bytes);

// ---- small device utilities ------------------------------------------------------------------
__device__ __forceinline__ float bf2f(bf16 x) { return __bfloat162float(x); }
__device__ __forceinline__ bf16 f2bf(float x) { return __float2bfloat16_rn(x); }

__device__ __forceinline__ float clamp_exp(float x) {
  return __expf(fminf(fmaxf(x, -kExpClamp), kExpClamp));
}

// 8 bf16 packed in a uint4 <-> 8 floats
__device__ __forceinline__ void unpack8(const uint4& u, float* f) {
  const __nv_bfloat162* h = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) {
    float2 t = __bfloat1622float2(h[i]);
    f[2 * i] = t.x;
    f[2 * i + 1] = t.y;
  }
}
__device__ __forceinline__ uint4 pack8(const float* f) {
  uint4 u;
  __nv_bfloat162* h = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
  for (int i = 0; i < 4; ++i) h[i] = __floats2bfloat162_rn(f[2 * i], f[2 * i + 1]);
  return u;
}

__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
  return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
  return v;
}

// ---- shared-memory tile GEMM on the warp-level tensor-core API --------------------------------
// C[Mt*16 x Nt*16] (fp32, row-major, ldc) (+)= A * B with bf16 operands in shared memory.
//   A(m,k) = A_ROW ? A[m*lda + k] : A[k*lda + m]
//   B(k,n) = B_ROW ? B[k*ldb + n] : B[n*ldb + k]
// Output tiles are dealt round-robin to the warps of the CTA.  KSEL restricts the k tiles of an
// output tile in row block mt: 0 = all, 1 = kt <= mt (A block lower triangular), 2 = kt >= mt
// (A block upper triangular).  NSEL: 0 = all output tiles, 1 = only nt <= mt.
template <bool A_ROW, bool B_ROW, bool ACC, int KSEL = 0, int NSEL = 0>
__device__ __forceinline__ void tile_gemm(float* C, int ldc, const bf16* A, int lda, const bf16* B, int ldb, int Mt,
                                          int Nt, int Kt, int warp, int nwarps) {
  using namespace nvcuda::wmma;
  typedef typename std::conditional<A_ROW, row_major, col_major>::type ALayout;
  typedef typename std::conditional<B_ROW, row_major, col_major>::type BLayout;
  for (int t = warp; t < Mt * Nt; t += nwarps) {
    const int mt = t / Nt, nt = t % Nt;
    if (NSEL == 1 && nt > mt) continue;
    fragment<accumulator, 16, 16, 16, float> acc;
    float* cptr = C + (size_t)mt * 16 * ldc + nt * 16;
    if (ACC) load_matrix_sync(acc, cptr, ldc, mem_row_major);
    else fill_fragment(acc, 0.0f);
    const int k0 = (KSEL == 2) ? mt : 0;
    const int k1 = (KSEL == 1) ? min(Kt, mt + 1) : Kt;
    for (int kt = k0; kt < k1; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, ALayout> fa;
      fragment<matrix_b, 16, 16, 16, bf16, BLayout> fb;
      const bf16* ap = A_ROW ? A + (size_t)mt * 16 * lda + kt * 16 : A + (size_t)kt * 16 * lda + mt * 16;
      const bf16* bp = B_ROW ? B + (size_t)kt * 16 * ldb + nt * 16 : B + (size_t)nt * 16 * ldb + kt * 16;
      load_matrix_sync(fa, ap, lda);
      load_matrix_sync(fb, bp, ldb);
      mma_sync(acc, fa, fb, acc);
    }
    store_matrix_sync(cptr, acc, ldc, mem_row_major);
  }
}

// Copy `rows` x `cols` bf16 (cols % 8 == 0) from global (row stride gstride elements) to shared
// (row stride sstride), rows with src_row(r) < 0 or >= limit are zero-filled.  `row0` is the global
// row of tile row 0.
__device__ __forceinline__ void load_tile_bf16(bf16* dst, int sstride, const bf16* src, int64_t gstride, int row0,
                                               int row_lo, int row_hi, int rows, int cols, int tid, int nthreads) {
  const int c8 = cols >> 3;
  for (int i = tid; i < rows * c8; i += nthreads) {
    const int r = i / c8, c = i - r * c8;
    const int gr = row0 + r;
    uint4 val = make_uint4(0u, 0u, 0u, 0u);
    if (gr >= row_lo && gr < row_hi) val = *reinterpret_cast<const uint4*>(src + (int64_t)gr * gstride + 8 * c);
    *reinterpret_cast<uint4*>(dst + r * sstride + 8 * c) = val;
  }
}

struct SeqInfo {
  int seq;      // sequence index
  int t0;       // first packed token of the sequence
  int len;      // tokens in the sequence
  int chunk;    // chunk index inside the sequence
  int wl;       // window_left (<0 = unbounded)
  int shift;    // gsa_kv_shift
};

// Per-chunk record of the plan: {sequence (-1 = unused chunk), chunk index inside the sequence, first packed token of
// the sequence, length of the sequence}, one 16-byte load instead of a chain of dependent ones.  The records follow
// the plan's other tables (offsets, chunk -> sequence, flags, error word) at the next multiple of four ints.
__host__ __device__ __forceinline__ int64_t plan_rec_offset(int64_t N, int64_t NCB, int64_t H) {
  return (N + 1 + NCB + NCB * H + 4 + 3) & ~(int64_t)3;
}
struct ChunkRec { int n, ci, t0, len; };
__device__ __forceinline__ ChunkRec chunk_rec(const nha_chunk_desc& d, int cg) {
  const int ncb = (int)((d.Ttot + kChunk - 1) / kChunk + d.N);
  const int4 r = __ldg(reinterpret_cast<const int4*>(d.plan + plan_rec_offset(d.N, ncb, d.H)) + cg);
  ChunkRec c;
  c.n = r.x; c.ci = r.y; c.t0 = r.z; c.len = r.w;
  return c;
}

// Scratch of the state pass: L [NCB*H][K*M + M*V] bf16 (the chunk-start states it is summed into are bf16 too; the
// running sum itself stays fp32), then Gend [NCB*H][M] fp32, then Gtot [N*H][M] fp32 (the log gates of each sequence
// summed over its chunks, left by the scan for nha_chunk_gate_totals).
struct StateWs {
  bf16* local;
  float* gend;
  float* gtot;
};

__device__ __forceinline__ int seq_window(const nha_chunk_desc& d, int n) {
  return d.window_left ? d.window_left[n] : d.window_left_all;
}
__device__ __forceinline__ int seq_shift(const nha_chunk_desc& d, int n) {
  int s = d.shift ? d.shift[n] : d.shift_all;
  return s < 0 ? 0 : s;
}

}  // namespace nha
