// Backward of the chunked NHA operator (sm_100a).
//
// With p = softmax([ok | sw]) recomputed from the saved log-sum-exps, dp = <do, values>,
// delta = <do, o> and dz = p .* (dp - delta) (+ d_lse_gsa * softmax(ok) on the slot part):
//   1. window rows    (chunk-parallel)  dq_swa = scale * dz_win k_swa            (+ delta, joint LSE)
//   2. window columns (chunk-parallel)  dk_swa = scale * dz_win^T q_swa, dv_win = p_win^T do
//   3. slot pass      (chunk-parallel)  dq_gsa and the parts of dk', dv', ds' that stay inside a chunk,
//                                       dgA = ok .* dz + p .* dp, and the decayed dz / p the march needs
//   4. state-gradient march (16-row / 16-column slices per sequence and kv head, last chunk first)
//      stores the gradients DK, DV of the slot memory at every chunk end; the inter-chunk pass
//      (chunk-parallel) adds the inter-chunk parts of dk', dv', ds', turns dgA - s' .* ds' into dg by a
//      reverse cumulative sum inside the chunk plus a carry rebuilt from <DK,hk> + <DV,hv>, undoes the
//      shift and writes the results.
// Primes are the inputs shifted right by gsa_kv_shift inside their sequence.
//
// Replaces ChunkNativeHybridAttentionFunction.backward (nha_fla/ops/nha/chunk.py:491-564): the
// flash-attn varlen backward called with the merged output and the joint LSE (:500-512), fla's
// chunk_gsa backward with the folded d_lse (nha_fla/ops/nha/chunk_gsa.py:52-122) and the shift
// adjoints (chunk.py:80-126).  A gradient on lse_swa is ignored, as there (:491-512).
#include <stdlib.h>

#include "nha_common.cuh"
#include "nha_bwd_common.cuh"

namespace nha {

constexpr int kBwThreads = 256;
constexpr int kBwWarps = kBwThreads / 32;

__host__ __device__ inline int bup128(int x) { return (x + 127) & ~127; }
__device__ __forceinline__ int sb_row0b(int I) { return 8 * I * (I + 1); }
__device__ __forceinline__ float block_refb(const float* G, int ldg, int I, int m) {
  const float gn = I > 0 ? G[(16 * I - 1) * ldg + m] : 0.f;
  return 0.5f * (gn + G[(16 * I + 15) * ldg + m]);
}

// ================================================================================================
// 1. window rows: delta, joint LSE, dq_swa
// ================================================================================================
struct WRowLayout { int qb, dob, wt, SA, DP, PB, DQ, rows, total; };
__host__ __device__ inline WRowLayout wrow_layout(int K, int V) {
  WRowLayout L; int off = 0;
  const int KV = K > V ? K : V;
  L.qb = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.dob = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.wt = off; off = bup128(off + kChunk * (KV + 8) * 2);
  L.SA = off; off = bup128(off + kChunk * (kChunk + 4) * 4);
  L.DP = off; off = bup128(off + kChunk * (kChunk + 4) * 4);
  L.PB = off; off = bup128(off + kChunk * (kChunk + 8) * 2);
  L.DQ = off; off = bup128(off + kChunk * (K + 4) * 4);
  L.rows = off; off = bup128(off + 2 * kChunk * 4);
  L.total = off;
  return L;
}

__device__ __forceinline__ void nha_bwd_window_rows_kernel_body(const nha_chunk_desc d, const BwdWs w, const int cgb) {
  ChunkCtx c;
  if (!chunk_ctx(d, cgb, c)) return;
  if (!chunk_gate(w, cgb, blockIdx.y, d.H)) return;
  const int K = d.K, V = d.V, H = d.H, HQ = d.HQ, NG = HQ / H, h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5;
  extern __shared__ __align__(128) unsigned char smem[];
  const WRowLayout L = wrow_layout(K, V);
  const int KV = K > V ? K : V;
  const int ldk = K + 8, ldv = V + 8, ldw = KV + 8, lds = kChunk + 4, ldp = kChunk + 8, ldq = K + 4;
  bf16* qb = (bf16*)(smem + L.qb);
  bf16* dob = (bf16*)(smem + L.dob);
  bf16* wt = (bf16*)(smem + L.wt);
  float* SA = (float*)(smem + L.SA);
  float* DP = (float*)(smem + L.DP);
  bf16* PB = (bf16*)(smem + L.PB);
  float* DQ = (float*)(smem + L.DQ);
  float* row_L = (float*)(smem + L.rows);
  float* row_d = row_L + kChunk;
  const int jt_hi = c.ci;
  const int jt_lo = c.wl < 0 ? 0 : max(0, c.c0 - c.wl) / kChunk;
  const int rq = tid >> 2, sub = tid & 3;

  for (int qh = 0; qh < NG; ++qh) {
    const int hq = h * NG + qh;
    __syncthreads();
    load_tile_bf16(qb, ldk, (const bf16*)d.q_swa + ((size_t)c.t0 * HQ + hq) * K, (int64_t)HQ * K, c.c0, 0, c.len, kChunk,
                   K, tid, kBwThreads);
    load_tile_bf16(dob, ldv, (const bf16*)d.d_o + ((size_t)c.t0 * HQ + hq) * V, (int64_t)HQ * V, c.c0, 0, c.len, kChunk, V,
                   tid, kBwThreads);
    // delta = <do, o>, joint LSE
    {
      const int pos = c.c0 + rq;
      float acc = 0.f;
      if (pos < c.len) {
        const bf16* orow = (const bf16*)d.o + ((size_t)(c.t0 + pos) * HQ + hq) * V;
        const bf16* grow = (const bf16*)d.d_o + ((size_t)(c.t0 + pos) * HQ + hq) * V;
        for (int v8 = sub; v8 < V / 8; v8 += 4) {
          float a[8], b[8];
          unpack8(*reinterpret_cast<const uint4*>(orow + 8 * v8), a);
          unpack8(*reinterpret_cast<const uint4*>(grow + 8 * v8), b);
#pragma unroll
          for (int e = 0; e < 8; ++e) acc += a[e] * b[e];
        }
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (sub == 0) {
        float Lj = 0.f;
        if (pos < c.len) {
          const float a = d.lse_swa[(size_t)(c.t0 + pos) * HQ + hq], b = d.lse_gsa[(size_t)(c.t0 + pos) * HQ + hq];
          const float mx = fmaxf(a, b);
          Lj = mx + __logf(__expf(a - mx) + __expf(b - mx));
          w.delta[(size_t)(c.t0 + pos) * HQ + hq] = acc;
          w.lj[(size_t)(c.t0 + pos) * HQ + hq] = Lj;
        }
        row_L[rq] = Lj;
        row_d[rq] = acc;
      }
    }
    for (int i = tid; i < kChunk * ldq; i += kBwThreads) DQ[i] = 0.f;
    for (int jt = jt_lo; jt <= jt_hi; ++jt) {
      __syncthreads();
      load_tile_bf16(wt, ldw, (const bf16*)d.v + ((size_t)c.t0 * H + h) * V, (int64_t)H * V, jt * kChunk, 0, c.len, kChunk,
                     V, tid, kBwThreads);
      __syncthreads();
      tile_gemm<true, false, false>(DP, lds, dob, ldv, wt, ldw, 4, 4, V / 16, warp, kBwWarps);   // do v^T
      __syncthreads();
      load_tile_bf16(wt, ldw, (const bf16*)d.k_swa + ((size_t)c.t0 * H + h) * K, (int64_t)H * K, jt * kChunk, 0, c.len,
                     kChunk, K, tid, kBwThreads);
      __syncthreads();
      tile_gemm<true, false, false>(SA, lds, qb, ldk, wt, ldw, 4, 4, K / 16, warp, kBwWarps);    // q k^T
      __syncthreads();
      for (int i = tid; i < kChunk * kChunk; i += kBwThreads) {
        const int r = i >> 6, cc = i & 63;
        const int key = jt * kChunk + cc, pq = c.c0 + r;
        const bool ok = key <= pq && (c.wl < 0 || key >= pq - c.wl) && pq < c.len;
        float dz = 0.f;
        if (ok) dz = __expf(SA[r * lds + cc] * d.scale - row_L[r]) * (DP[r * lds + cc] - row_d[r]) * d.scale;
        PB[r * ldp + cc] = f2bf(dz);
      }
      __syncthreads();
      tile_gemm<true, true, true>(DQ, ldq, PB, ldp, wt, ldw, 4, K / 16, 4, warp, kBwWarps);      // dq += dz k
    }
    __syncthreads();
    for (int i = tid; i < kChunk * (K / 8); i += kBwThreads) {
      const int r = i / (K / 8), c8 = i - r * (K / 8);
      const int pq = c.c0 + r;
      if (pq < c.len)
        *reinterpret_cast<uint4*>((bf16*)d.dq_swa + ((size_t)(c.t0 + pq) * HQ + hq) * K + 8 * c8) = pack8(DQ + r * ldq + 8 * c8);
    }
  }
}

// One CTA walks `cpc` consecutive chunks (1 when the kernel handles every chunk; more when it is launched gated
// on the chunk flags and most chunks return at once, so that an all-clear launch costs few CTAs).
__global__ void __launch_bounds__(kBwThreads) nha_bwd_window_rows_kernel(const nha_chunk_desc d, const BwdWs w, const int cpc) {
  const int ncb = (int)((d.Ttot + kChunk - 1) / kChunk + d.N);
  // which of my chunks have work: one flag load per chunk, all at once (cpc <= 32)
  __shared__ unsigned todo;
  if (threadIdx.x < 32) {
    const int cgl = blockIdx.x * cpc + threadIdx.x;
    const bool mine = (int)threadIdx.x < cpc && cgl < ncb && chunk_gate(w, cgl, blockIdx.y, d.H);
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (threadIdx.x == 0) todo = m;
  }
  __syncthreads();
  unsigned left = todo;
  while (left) {
    const int i = __ffs(left) - 1;
    left &= left - 1;
    nha_bwd_window_rows_kernel_body(d, w, blockIdx.x * cpc + i);
    __syncthreads();
  }
}

// ================================================================================================
// 2. window columns: dk_swa, window part of dv; one CTA per (key chunk, kv head)
// ================================================================================================
struct WColLayout { int kt, vt, qb, dob, SA, DP, PB, ZB, DK, DV, rows, total; };
__host__ __device__ inline WColLayout wcol_layout(int K, int V) {
  WColLayout L; int off = 0;
  L.kt = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.vt = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.qb = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.dob = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.SA = off; off = bup128(off + kChunk * (kChunk + 4) * 4);
  L.DP = off; off = bup128(off + kChunk * (kChunk + 4) * 4);
  L.PB = off; off = bup128(off + kChunk * (kChunk + 8) * 2);
  L.ZB = off; off = bup128(off + kChunk * (kChunk + 8) * 2);
  L.DK = off; off = bup128(off + kChunk * (K + 4) * 4);
  L.DV = off; off = bup128(off + kChunk * (V + 4) * 4);
  L.rows = off; off = bup128(off + 2 * kChunk * 4);
  L.total = off;
  return L;
}

__global__ void __launch_bounds__(kBwThreads) nha_bwd_window_cols_kernel(const nha_chunk_desc d, const BwdWs w) {
  ChunkCtx c;
  if (!chunk_ctx(d, blockIdx.x, c)) return;
  const int K = d.K, V = d.V, H = d.H, HQ = d.HQ, NG = HQ / H, h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5;
  extern __shared__ __align__(128) unsigned char smem[];
  const WColLayout L = wcol_layout(K, V);
  const int ldk = K + 8, ldv = V + 8, lds = kChunk + 4, ldp = kChunk + 8, lddk = K + 4, lddv = V + 4;
  bf16* kt = (bf16*)(smem + L.kt);
  bf16* vt = (bf16*)(smem + L.vt);
  bf16* qb = (bf16*)(smem + L.qb);
  bf16* dob = (bf16*)(smem + L.dob);
  float* SA = (float*)(smem + L.SA);
  float* DP = (float*)(smem + L.DP);
  bf16* PB = (bf16*)(smem + L.PB);
  bf16* ZB = (bf16*)(smem + L.ZB);
  float* DK = (float*)(smem + L.DK);
  float* DV = (float*)(smem + L.DV);
  float* row_L = (float*)(smem + L.rows);
  float* row_d = row_L + kChunk;
  const int nchunks = (c.len + kChunk - 1) / kChunk;
  // query chunks that can see a key of this chunk
  const int qi_lo = c.ci;
  const int qi_hi = c.wl < 0 ? nchunks - 1 : min(nchunks - 1, (c.c0 + kChunk - 1 + c.wl) / kChunk);

  load_tile_bf16(kt, ldk, (const bf16*)d.k_swa + ((size_t)c.t0 * H + h) * K, (int64_t)H * K, c.c0, 0, c.len, kChunk, K, tid,
                 kBwThreads);
  load_tile_bf16(vt, ldv, (const bf16*)d.v + ((size_t)c.t0 * H + h) * V, (int64_t)H * V, c.c0, 0, c.len, kChunk, V, tid,
                 kBwThreads);
  for (int i = tid; i < kChunk * lddk; i += kBwThreads) DK[i] = 0.f;
  for (int i = tid; i < kChunk * lddv; i += kBwThreads) DV[i] = 0.f;
  for (int qi = qi_lo; qi <= qi_hi; ++qi) {
    const int q0 = qi * kChunk;
    for (int qh = 0; qh < NG; ++qh) {
      const int hq = h * NG + qh;
      __syncthreads();
      load_tile_bf16(qb, ldk, (const bf16*)d.q_swa + ((size_t)c.t0 * HQ + hq) * K, (int64_t)HQ * K, q0, 0, c.len, kChunk, K,
                     tid, kBwThreads);
      load_tile_bf16(dob, ldv, (const bf16*)d.d_o + ((size_t)c.t0 * HQ + hq) * V, (int64_t)HQ * V, q0, 0, c.len, kChunk, V,
                     tid, kBwThreads);
      if (tid < kChunk) {
        const int pq = q0 + tid;
        row_L[tid] = pq < c.len ? w.lj[(size_t)(c.t0 + pq) * HQ + hq] : 0.f;
        row_d[tid] = pq < c.len ? w.delta[(size_t)(c.t0 + pq) * HQ + hq] : 0.f;
      }
      __syncthreads();
      tile_gemm<true, false, false>(SA, lds, qb, ldk, kt, ldk, 4, 4, K / 16, warp, kBwWarps);    // q k^T
      tile_gemm<true, false, false>(DP, lds, dob, ldv, vt, ldv, 4, 4, V / 16, warp, kBwWarps);   // do v^T
      __syncthreads();
      for (int i = tid; i < kChunk * kChunk; i += kBwThreads) {
        const int r = i >> 6, cc = i & 63;
        const int key = c.c0 + cc, pq = q0 + r;
        const bool ok = key <= pq && (c.wl < 0 || key >= pq - c.wl) && pq < c.len;
        float p = 0.f, dz = 0.f;
        if (ok) {
          p = __expf(SA[r * lds + cc] * d.scale - row_L[r]);
          dz = p * (DP[r * lds + cc] - row_d[r]) * d.scale;
        }
        PB[r * ldp + cc] = f2bf(p);
        ZB[r * ldp + cc] = f2bf(dz);
      }
      __syncthreads();
      tile_gemm<false, true, true>(DV, lddv, PB, ldp, dob, ldv, 4, V / 16, 4, warp, kBwWarps);   // dv += p^T do
      tile_gemm<false, true, true>(DK, lddk, ZB, ldp, qb, ldk, 4, K / 16, 4, warp, kBwWarps);    // dk += dz^T q
    }
  }
  __syncthreads();
  for (int i = tid; i < kChunk * (K / 8); i += kBwThreads) {
    const int r = i / (K / 8), c8 = i - r * (K / 8);
    const int pk = c.c0 + r;
    if (pk < c.len)
      *reinterpret_cast<uint4*>((bf16*)d.dk_swa + ((size_t)(c.t0 + pk) * H + h) * K + 8 * c8) = pack8(DK + r * lddk + 8 * c8);
  }
  for (int i = tid; i < kChunk * (V / 4); i += kBwThreads) {
    const int r = i / (V / 4), c4 = i - r * (V / 4);
    const int pk = c.c0 + r;
    if (pk < c.len)
      *reinterpret_cast<float4*>(w.dvacc + ((size_t)(c.t0 + pk) * H + h) * V + 4 * c4) =
          *reinterpret_cast<const float4*>(DV + r * lddv + 4 * c4);
  }
}

// ================================================================================================
// 3. slot pass: everything of the slot branch that stays inside a chunk
// ================================================================================================
// Two tiles share storage with tiles that are dead while they are live, where the sizes allow it (this is what lets
// K = V = 128 with M = 64 fit the 227 KB): Hv is only read by the first product of a head (do Hv^T), before tril(A)
// and tril(Av) are written, so it may sit in their two tiles and is then fetched again for every query head; DQ is
// written after the last read of OK and Y (step 3) and may lie over that pair.
struct SlotLayout { int kp, vp, G, Hk, Hv, SB, qb, dob, OK, Y, SA, AB, AvB, dzg, dza, paq, DQ, rows, total, hv_alias; };
__host__ __device__ inline SlotLayout slot_layout(int K, int V, int M) {
  SlotLayout L; int off = 0;
  const int KV = K > V ? K : V;
  const int sz_hv = bup128(M * (V + 8) * 2), sz_ab = bup128(kChunk * (kChunk + 8) * 2);
  const int sz_ok = bup128(kChunk * (M + 4) * 4), sz_dq = bup128(kChunk * (KV + 4) * 4);
  L.hv_alias = sz_hv <= 2 * sz_ab;
  L.kp = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.vp = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.G = off; off = bup128(off + kChunk * (M + 4) * 4);
  L.Hk = off; off = bup128(off + K * (M + 8) * 2);
  L.Hv = off; if (!L.hv_alias) off += sz_hv;
  L.SB = off; off = bup128(off + 160 * (M + 8) * 2);
  L.qb = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.dob = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.OK = off; off += sz_ok;
  L.Y = off; off += sz_ok;
  const int sa_cols = M > kChunk ? M : kChunk;
  L.SA = off; off = bup128(off + kChunk * (sa_cols + 4) * 4);
  L.AB = off; off += sz_ab;
  L.AvB = off; off += sz_ab;
  if (L.hv_alias) L.Hv = L.AB;
  L.dzg = off; off = bup128(off + kChunk * (M + 8) * 2);
  L.dza = off; off = bup128(off + kChunk * (M + 8) * 2);
  L.paq = off; off = bup128(off + kChunk * (M + 8) * 2);
  if (sz_dq <= 2 * sz_ok) L.DQ = L.OK;
  else { L.DQ = off; off += sz_dq; }
  L.rows = off; off = bup128(off + 4 * kChunk * 4);
  L.total = off;
  return L;
}

__device__ __forceinline__ void tril_bf16(bf16* AB, int ldab, const float* SA, int ldsa, int tid) {
  for (int i = tid; i < kChunk * kChunk; i += kBwThreads) {
    const int r = i >> 6, c = i & 63;
    AB[r * ldab + c] = f2bf(c <= r ? SA[r * ldsa + c] : 0.f);
  }
}

// X[16I.., :M] = AB[16I.., 0:16(I+1)] * SB_I
__device__ __forceinline__ void rows_times_sb(float* X, int ldx, const bf16* AB, int ldab, const bf16* SB, int ldsb,
                                              int M, int warp) {
  using namespace nvcuda::wmma;
  const int Nt = M / 16;
  for (int t = warp; t < 4 * Nt; t += kBwWarps) {
    const int I = t / Nt, nt = t % Nt;
    fragment<accumulator, 16, 16, 16, float> acc;
    fill_fragment(acc, 0.f);
    for (int kt = 0; kt <= I; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
      fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
      load_matrix_sync(fa, AB + 16 * I * ldab + 16 * kt, ldab);
      load_matrix_sync(fb, SB + (sb_row0b(I) + 16 * kt) * ldsb + 16 * nt, ldsb);
      mma_sync(acc, fa, fb, acc);
    }
    store_matrix_sync(X + 16 * I * ldx + 16 * nt, acc, ldx, mem_row_major);
  }
}

// Y[16I.., 0:16(I+1)] = PA[16I.., :M] * SB_I^T
__device__ __forceinline__ void rows_times_sbT(float* Y, int ldy, const bf16* PA, int ldpa, const bf16* SB, int ldsb,
                                               int M, int warp) {
  using namespace nvcuda::wmma;
  for (int t = warp; t < 16; t += kBwWarps) {
    const int I = t >> 2, nt = t & 3;
    if (nt > I) continue;
    fragment<accumulator, 16, 16, 16, float> acc;
    fill_fragment(acc, 0.f);
    for (int kt = 0; kt < M / 16; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
      fragment<matrix_b, 16, 16, 16, bf16, col_major> fb;
      load_matrix_sync(fa, PA + 16 * I * ldpa + 16 * kt, ldpa);
      load_matrix_sync(fb, SB + (sb_row0b(I) + 16 * nt) * ldsb + 16 * kt, ldsb);
      mma_sync(acc, fa, fb, acc);
    }
    store_matrix_sync(Y + 16 * I * ldy + 16 * nt, acc, ldy, mem_row_major);
  }
}

__device__ __forceinline__ void nha_bwd_slot_kernel_body(const nha_chunk_desc d, const BwdWs w, const int cgb) {
  using namespace nvcuda::wmma;
  ChunkCtx c;
  const int cg = cgb;
  if (!chunk_ctx(d, cg, c)) return;
  if (!chunk_gate(w, cg, blockIdx.y, d.H)) return;
  const int K = d.K, V = d.V, M = d.M, H = d.H, HQ = d.HQ, NG = HQ / H, h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5;
  extern __shared__ __align__(128) unsigned char smem[];
  const SlotLayout L = slot_layout(K, V, M);
  const int KV = K > V ? K : V;
  const int ldk = K + 8, ldv = V + 8, ldg = M + 4, ldhk = M + 8, ldhv = V + 8, ldsb = M + 8;
  const int ldsa = (M > kChunk ? M : kChunk) + 4, ldab = kChunk + 8, ldp = M + 8, lddq = KV + 4;
  bf16* kp = (bf16*)(smem + L.kp);
  bf16* vp = (bf16*)(smem + L.vp);
  float* G = (float*)(smem + L.G);
  bf16* Hk = (bf16*)(smem + L.Hk);
  bf16* Hv = (bf16*)(smem + L.Hv);
  bf16* SB = (bf16*)(smem + L.SB);
  bf16* qb = (bf16*)(smem + L.qb);
  bf16* dob = (bf16*)(smem + L.dob);
  float* OK = (float*)(smem + L.OK);
  float* Y = (float*)(smem + L.Y);
  float* SA = (float*)(smem + L.SA);
  bf16* AB = (bf16*)(smem + L.AB);
  bf16* AvB = (bf16*)(smem + L.AvB);
  bf16* dzg = (bf16*)(smem + L.dzg);
  bf16* dza = (bf16*)(smem + L.dza);
  bf16* paq = (bf16*)(smem + L.paq);
  float* DQ = (float*)(smem + L.DQ);
  float* row_L = (float*)(smem + L.rows);
  float* row_d = row_L + kChunk;
  float* row_lg = row_d + kChunk;      // lse_gsa
  float* row_dl = row_lg + kChunk;     // d_lse_gsa

  // ---- kv-head data (same staging as the forward output pass) -------------------------------------
  {
    const int lo = 0, hi = c.len - c.shift;
    load_tile_bf16(kp, ldk, (const bf16*)d.k_gsa + ((size_t)c.t0 * H + h) * K, (int64_t)H * K, c.c0 - c.shift, lo, hi,
                   kChunk, K, tid, kBwThreads);
    load_tile_bf16(vp, ldv, (const bf16*)d.v + ((size_t)c.t0 * H + h) * V, (int64_t)H * V, c.c0 - c.shift, lo, hi, kChunk,
                   V, tid, kBwThreads);
    load_tile_bf16(dzg, ldp, (const bf16*)d.s + ((size_t)c.t0 * H + h) * M, (int64_t)H * M, c.c0 - c.shift, lo, hi,
                   kChunk, M, tid, kBwThreads);                                   // s' staged in dzg
    const bf16* gg = (const bf16*)d.g + ((size_t)c.t0 * H + h) * M;
    for (int i = tid; i < kChunk * (M / 8); i += kBwThreads) {
      const int r = i / (M / 8), c8 = i - r * (M / 8);
      const int j = c.c0 + r - c.shift;
      float gv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (j >= lo && j < hi) unpack8(*reinterpret_cast<const uint4*>(gg + (size_t)j * H * M + 8 * c8), gv);
#pragma unroll
      for (int e = 0; e < 8; ++e) G[r * ldg + 8 * c8 + e] = gv[e];
    }
    load_tile_bf16(Hk, ldhk, (const bf16*)d.hk_chunks + ((size_t)cg * H + h) * K * M, M, 0, 0, K, K, M, tid, kBwThreads);
    if (!L.hv_alias)
      load_tile_bf16(Hv, ldhv, (const bf16*)d.hv_chunks + ((size_t)cg * H + h) * M * V, V, 0, 0, M, M, V, tid, kBwThreads);
  }
  __syncthreads();
  for (int m = tid; m < M; m += kBwThreads) {
    float run = 0.f;
#pragma unroll 16
    for (int r = 0; r < kChunk; ++r) {
      run += G[r * ldg + m];
      G[r * ldg + m] = run;
    }
  }
  __syncthreads();
  for (int i = tid; i < 160 * M; i += kBwThreads) {
    const int row = i / M, m = i - row * M;
    const int I = row < 16 ? 0 : (row < 48 ? 1 : (row < 96 ? 2 : 3));
    const int r = row - sb_row0b(I);
    SB[row * ldsb + m] = f2bf(bf2f(dzg[r * ldp + m]) * clamp_exp(block_refb(G, ldg, I, m) - G[r * ldg + m]));
  }
  // register accumulators of dk' [64 x K] and dv' [64 x V]: warp -> row tile (warp & 3), col tiles (warp >> 2) + 2 i
  constexpr int kMaxCT = 4;
  const int mt = warp & 3;
  const int CTK = K / 32, CTV = V / 32;
  fragment<accumulator, 16, 16, 16, float> dkacc[kMaxCT], dvacc[kMaxCT];
#pragma unroll
  for (int i = 0; i < kMaxCT; ++i) { fill_fragment(dkacc[i], 0.f); fill_fragment(dvacc[i], 0.f); }
  __syncthreads();

  for (int qh = 0; qh < NG; ++qh) {
    const int hq = h * NG + qh;
    // ---- 1. tiles of this head ------------------------------------------------------------------
    load_tile_bf16(qb, ldk, (const bf16*)d.q_gsa + ((size_t)c.t0 * HQ + hq) * K, (int64_t)HQ * K, c.c0, 0, c.len, kChunk, K,
                   tid, kBwThreads);
    load_tile_bf16(dob, ldv, (const bf16*)d.d_o + ((size_t)c.t0 * HQ + hq) * V, (int64_t)HQ * V, c.c0, 0, c.len, kChunk, V,
                   tid, kBwThreads);
    if (L.hv_alias)                                    // tril(A) / tril(Av) of the previous head have been consumed
      load_tile_bf16(Hv, ldhv, (const bf16*)d.hv_chunks + ((size_t)cg * H + h) * M * V, V, 0, 0, M, M, V, tid, kBwThreads);
    if (tid < kChunk) {
      const int pq = c.c0 + tid;
      const bool in = pq < c.len;
      const size_t idx = (size_t)(c.t0 + pq) * HQ + hq;
      row_L[tid] = in ? w.lj[idx] : 0.f;
      row_d[tid] = in ? w.delta[idx] : 0.f;
      row_lg[tid] = in ? d.lse_gsa[idx] : 0.f;
      row_dl[tid] = (in && d.d_lse_gsa) ? d.d_lse_gsa[idx] : 0.f;
    }
    __syncthreads();
    // ---- 2. slot logits OK (as in the forward) and Y0 = do Hv^T, A = q k'^T, Av = do v'^T ----------
    tile_gemm<true, true, false>(OK, ldg, qb, ldk, Hk, ldhk, 4, M / 16, K / 16, warp, kBwWarps);
    tile_gemm<true, false, false>(Y, ldg, dob, ldv, Hv, ldhv, 4, M / 16, V / 16, warp, kBwWarps);
    tile_gemm<true, false, false, 0, 1>(SA, ldsa, qb, ldk, kp, ldk, 4, 4, K / 16, warp, kBwWarps);
    __syncthreads();
    tril_bf16(AB, ldab, SA, ldsa, tid);
    __syncthreads();
    tile_gemm<true, false, false, 0, 1>(SA, ldsa, dob, ldv, vp, ldv, 4, 4, V / 16, warp, kBwWarps);
    __syncthreads();
    tril_bf16(AvB, ldab, SA, ldsa, tid);
    for (int i = tid; i < kChunk * M; i += kBwThreads) {
      const int r = i / M, m = i - r * M;
      const float eg = __expf(G[r * ldg + m]);
      OK[r * ldg + m] *= d.scale * eg;
      Y[r * ldg + m] *= eg;
    }
    __syncthreads();
    rows_times_sb(SA, ldsa, AB, ldab, SB, ldsb, M, warp);
    __syncthreads();
    for (int i = tid; i < kChunk * M; i += kBwThreads) {
      const int r = i / M, m = i - r * M;
      OK[r * ldg + m] += d.scale * clamp_exp(G[r * ldg + m] - block_refb(G, ldg, r >> 4, m)) * SA[r * ldsa + m];
    }
    __syncthreads();
    rows_times_sb(SA, ldsa, AvB, ldab, SB, ldsb, M, warp);
    __syncthreads();
    // ---- 3. dz on the slot part; decayed copies for the march; dgA ---------------------------------
    for (int i = tid; i < kChunk * M; i += kBwThreads) {
      const int r = i / M, m = i - r * M;
      const int pq = c.c0 + r;
      const float gl = G[r * ldg + m];
      const float aI = clamp_exp(gl - block_refb(G, ldg, r >> 4, m));
      const float ok = OK[r * ldg + m];
      const float dps = Y[r * ldg + m] + aI * SA[r * ldsa + m];
      float ps = 0.f, dz = 0.f;
      if (pq < c.len) {
        ps = __expf(ok - row_L[r]);
        dz = ps * (dps - row_d[r]) + row_dl[r] * __expf(ok - row_lg[r]);
      }
      const float eg = __expf(gl);
      const bf16 zg = f2bf(d.scale * dz * eg), pg = f2bf(ps * eg);
      dzg[r * ldp + m] = zg;
      dza[r * ldp + m] = f2bf(d.scale * dz * aI);
      paq[r * ldp + m] = f2bf(ps * aI);
      if (pq < c.len) {
        const size_t gi = ((size_t)(c.t0 + pq) * HQ + hq) * M + m;
        w.dzg[gi] = zg;
        w.pgq[gi] = pg;
        const size_t hi = ((size_t)(c.t0 + pq) * H + h) * M + m;
        const float val = ok * dz + ps * dps;
        w.dga[hi] = qh == 0 ? val : w.dga[hi] + val;
      }
    }
    __syncthreads();
    // ---- 4. intra-chunk ds': for every row block I, b_I .* (A_I^T dza_I + Av_I^T pa_I) ---------------
    for (int I = 0; I < 4; ++I) {
      const int Nt = M / 16;
      for (int t = warp; t < (I + 1) * Nt; t += kBwWarps) {
        const int it = t / Nt, nt = t % Nt;
        fragment<accumulator, 16, 16, 16, float> acc;
        fill_fragment(acc, 0.f);
        fragment<matrix_a, 16, 16, 16, bf16, col_major> fa;
        fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
        load_matrix_sync(fa, AB + 16 * I * ldab + 16 * it, ldab);
        load_matrix_sync(fb, dza + 16 * I * ldp + 16 * nt, ldp);
        mma_sync(acc, fa, fb, acc);
        load_matrix_sync(fa, AvB + 16 * I * ldab + 16 * it, ldab);
        load_matrix_sync(fb, paq + 16 * I * ldp + 16 * nt, ldp);
        mma_sync(acc, fa, fb, acc);
        store_matrix_sync(SA + 16 * it * ldsa + 16 * nt, acc, ldsa, mem_row_major);
      }
      __syncthreads();
      for (int i = tid; i < 16 * (I + 1) * M; i += kBwThreads) {
        const int r = i / M, m = i - r * M;
        const int p = c.c0 + r;
        if (p < c.len) {
          const float bI = clamp_exp(block_refb(G, ldg, I, m) - G[r * ldg + m]);
          const size_t hi = ((size_t)(c.t0 + p) * H + h) * M + m;
          const float val = bI * SA[r * ldsa + m];
          w.dsp[hi] = (qh == 0 && I == 0) ? val : ((qh == 0 && r >= 16 * I) ? val : w.dsp[hi] + val);
        }
      }
      __syncthreads();
    }
    // ---- 5. E = tril(dza SB^T), Bv = tril(pa SB^T) (reuse AB / AvB), dq_gsa -----------------------------
    rows_times_sbT(SA, ldsa, dza, ldp, SB, ldsb, M, warp);
    __syncthreads();
    tril_bf16(AB, ldab, SA, ldsa, tid);
    __syncthreads();
    rows_times_sbT(SA, ldsa, paq, ldp, SB, ldsb, M, warp);
    tile_gemm<true, false, false>(DQ, lddq, dzg, ldp, Hk, ldhk, 4, K / 16, M / 16, warp, kBwWarps);   // (dz exp G) Hk^T
    __syncthreads();
    tril_bf16(AvB, ldab, SA, ldsa, tid);
    tile_gemm<true, true, true, 1>(DQ, lddq, AB, ldab, kp, ldk, 4, K / 16, 4, warp, kBwWarps);          // + E k'
    __syncthreads();
    for (int i = tid; i < kChunk * (K / 8); i += kBwThreads) {
      const int r = i / (K / 8), c8 = i - r * (K / 8);
      const int pq = c.c0 + r;
      if (pq < c.len)
        *reinterpret_cast<uint4*>((bf16*)d.dq_gsa + ((size_t)(c.t0 + pq) * HQ + hq) * K + 8 * c8) = pack8(DQ + r * lddq + 8 * c8);
    }
    // ---- 6. dk' += E^T q, dv' += Bv^T do (register accumulators, k tiles kt >= mt) ---------------------
    for (int kt = mt; kt < 4; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, col_major> fa;
      load_matrix_sync(fa, AB + 16 * kt * ldab + 16 * mt, ldab);
#pragma unroll
      for (int i = 0; i < kMaxCT; ++i) {
        if (i < CTK) {
          fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
          load_matrix_sync(fb, qb + 16 * kt * ldk + 16 * ((warp >> 2) + 2 * i), ldk);
          mma_sync(dkacc[i], fa, fb, dkacc[i]);
        }
      }
      load_matrix_sync(fa, AvB + 16 * kt * ldab + 16 * mt, ldab);
#pragma unroll
      for (int i = 0; i < kMaxCT; ++i) {
        if (i < CTV) {
          fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
          load_matrix_sync(fb, dob + 16 * kt * ldv + 16 * ((warp >> 2) + 2 * i), ldv);
          mma_sync(dvacc[i], fa, fb, dvacc[i]);
        }
      }
    }
    __syncthreads();
  }
  // ---- intra-chunk dk', dv' to the workspace (row = shifted position) ---------------------------------
#pragma unroll
  for (int i = 0; i < kMaxCT; ++i)
    if (i < CTK) store_matrix_sync(DQ + 16 * mt * lddq + 16 * ((warp >> 2) + 2 * i), dkacc[i], lddq, mem_row_major);
  __syncthreads();
  for (int i = tid; i < kChunk * (K / 4); i += kBwThreads) {
    const int r = i / (K / 4), c4 = i - r * (K / 4);
    const int p = c.c0 + r;
    if (p < c.len)
      *reinterpret_cast<float4*>(w.dkp + ((size_t)(c.t0 + p) * H + h) * K + 4 * c4) =
          *reinterpret_cast<const float4*>(DQ + r * lddq + 4 * c4);
  }
  __syncthreads();
#pragma unroll
  for (int i = 0; i < kMaxCT; ++i)
    if (i < CTV) store_matrix_sync(DQ + 16 * mt * lddq + 16 * ((warp >> 2) + 2 * i), dvacc[i], lddq, mem_row_major);
  __syncthreads();
  for (int i = tid; i < kChunk * (V / 4); i += kBwThreads) {
    const int r = i / (V / 4), c4 = i - r * (V / 4);
    const int p = c.c0 + r;
    if (p < c.len)
      *reinterpret_cast<float4*>(w.dvp + ((size_t)(c.t0 + p) * H + h) * V + 4 * c4) =
          *reinterpret_cast<const float4*>(DQ + r * lddq + 4 * c4);
  }
}

// One CTA walks `cpc` consecutive chunks (1 when the kernel handles every chunk; more when it is launched gated
// on the chunk flags and most chunks return at once, so that an all-clear launch costs few CTAs).
__global__ void __launch_bounds__(kBwThreads) nha_bwd_slot_kernel(const nha_chunk_desc d, const BwdWs w, const int cpc) {
  const int ncb = (int)((d.Ttot + kChunk - 1) / kChunk + d.N);
  // which of my chunks have work: one flag load per chunk, all at once (cpc <= 32)
  __shared__ unsigned todo;
  if (threadIdx.x < 32) {
    const int cgl = blockIdx.x * cpc + threadIdx.x;
    const bool mine = (int)threadIdx.x < cpc && cgl < ncb && chunk_gate(w, cgl, blockIdx.y, d.H);
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (threadIdx.x == 0) todo = m;
  }
  __syncthreads();
  unsigned left = todo;
  while (left) {
    const int i = __ffs(left) - 1;
    left &= left - 1;
    nha_bwd_slot_kernel_body(d, w, blockIdx.x * cpc + i);
    __syncthreads();
  }
}

// ================================================================================================
// 4a. state gradients at every chunk end.  The gradient D of the slot memory obeys, last chunk first,
//         D_end[c-1] = D_end[c] .* exp(Gend_c) + L_c,
//     L_c = q^T (scale dz exp G) for hk and (p exp G)^T do for hv, summed over the query heads of the
//     group.  L_c depends on chunk c alone, so it is produced chunk-parallel (by the tensor-memory rows
//     pass, or by the kernel below for the chunks the general kernels own) and what remains is an
//     element-wise scan over the chunks, done in place over the buffers that held L.
// ================================================================================================
struct LocalLayout { int qb, dob, zt, pt, G, OK, OV, total; };
__host__ __device__ inline LocalLayout local_layout(int K, int V, int M) {
  LocalLayout L; int off = 0;
  L.qb = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.dob = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.zt = off; off = bup128(off + kChunk * (M + 8) * 2);
  L.pt = off; off = bup128(off + kChunk * (M + 8) * 2);
  L.G = off; off = bup128(off + M * 4);
  L.OK = off; off = bup128(off + K * (M + 4) * 4);
  L.OV = off; off = bup128(off + M * (V + 4) * 4);
  L.total = off;
  return L;
}

__device__ __forceinline__ void nha_bwd_local_terms_kernel_body(const nha_chunk_desc d, const BwdWs w, const int cgb) {
  ChunkCtx c;
  const int cg = cgb;
  if (!chunk_ctx(d, cg, c)) return;
  if (!chunk_gate(w, cg, blockIdx.y, d.H)) return;
  const int K = d.K, V = d.V, M = d.M, H = d.H, HQ = d.HQ, NG = HQ / H, h = blockIdx.y;
  const int tid = threadIdx.x, warp = tid >> 5;
  extern __shared__ __align__(128) unsigned char smem[];
  const LocalLayout L = local_layout(K, V, M);
  const int ldk = K + 8, ldv = V + 8, ldm = M + 8, ldok = M + 4, ldov = V + 4;
  bf16* qb = (bf16*)(smem + L.qb);
  bf16* dob = (bf16*)(smem + L.dob);
  bf16* zt = (bf16*)(smem + L.zt);
  bf16* pt = (bf16*)(smem + L.pt);
  float* OK = (float*)(smem + L.OK);
  float* OV = (float*)(smem + L.OV);
  {
    // total shifted log gate of the chunk per slot
    const bf16* gg = (const bf16*)d.g + ((size_t)c.t0 * H + h) * M;
    const int r_lo = max(0, c.shift - c.c0), r_hi = min(kChunk, c.len - c.c0);
    for (int m = tid; m < M; m += kBwThreads) {
      float acc = 0.f;
      for (int r = r_lo; r < r_hi; ++r) acc += bf2f(gg[(size_t)(c.c0 + r - c.shift) * H * M + m]);
      w.gend[((size_t)cg * H + h) * M + m] = acc;
    }
  }
  for (int qh = 0; qh < NG; ++qh) {
    const int hq = h * NG + qh;
    __syncthreads();
    load_tile_bf16(qb, ldk, (const bf16*)d.q_gsa + ((size_t)c.t0 * HQ + hq) * K, (int64_t)HQ * K, c.c0, 0, c.len, kChunk, K,
                   tid, kBwThreads);
    load_tile_bf16(dob, ldv, (const bf16*)d.d_o + ((size_t)c.t0 * HQ + hq) * V, (int64_t)HQ * V, c.c0, 0, c.len, kChunk, V,
                   tid, kBwThreads);
    load_tile_bf16(zt, ldm, w.dzg + ((size_t)c.t0 * HQ + hq) * M, (int64_t)HQ * M, c.c0, 0, c.len, kChunk, M, tid, kBwThreads);
    load_tile_bf16(pt, ldm, w.pgq + ((size_t)c.t0 * HQ + hq) * M, (int64_t)HQ * M, c.c0, 0, c.len, kChunk, M, tid, kBwThreads);
    __syncthreads();
    if (qh == 0) {
      tile_gemm<false, true, false>(OK, ldok, qb, ldk, zt, ldm, K / 16, M / 16, 4, warp, kBwWarps);
      tile_gemm<false, true, false>(OV, ldov, pt, ldm, dob, ldv, M / 16, V / 16, 4, warp, kBwWarps);
    } else {
      tile_gemm<false, true, true>(OK, ldok, qb, ldk, zt, ldm, K / 16, M / 16, 4, warp, kBwWarps);
      tile_gemm<false, true, true>(OV, ldov, pt, ldm, dob, ldv, M / 16, V / 16, 4, warp, kBwWarps);
    }
  }
  __syncthreads();
  float* dk = w.dkc + ((size_t)cg * H + h) * K * M;
  float* dv = w.dvc + ((size_t)cg * H + h) * M * V;
  for (int i = tid; i < K * M; i += kBwThreads) dk[i] = OK[(i / M) * ldok + (i % M)];
  for (int i = tid; i < M * V; i += kBwThreads) dv[i] = OV[(i / V) * ldov + (i % V)];
}

// One CTA walks `cpc` consecutive chunks (1 when the kernel handles every chunk; more when it is launched gated
// on the chunk flags and most chunks return at once, so that an all-clear launch costs few CTAs).
__global__ void __launch_bounds__(kBwThreads) nha_bwd_local_terms_kernel(const nha_chunk_desc d, const BwdWs w, const int cpc) {
  const int ncb = (int)((d.Ttot + kChunk - 1) / kChunk + d.N);
  // which of my chunks have work: one flag load per chunk, all at once (cpc <= 32)
  __shared__ unsigned todo;
  if (threadIdx.x < 32) {
    const int cgl = blockIdx.x * cpc + threadIdx.x;
    const bool mine = (int)threadIdx.x < cpc && cgl < ncb && chunk_gate(w, cgl, blockIdx.y, d.H);
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (threadIdx.x == 0) todo = m;
  }
  __syncthreads();
  unsigned left = todo;
  while (left) {
    const int i = __ffs(left) - 1;
    left &= left - 1;
    nha_bwd_local_terms_kernel_body(d, w, blockIdx.x * cpc + i);
    __syncthreads();
  }
}

// In-place reverse scan over the chunks of one (sequence, kv head): on entry dkc/dvc hold L_c, on exit
// the gradient at the END of chunk c; the value carried past chunk 0 is the initial state's gradient.
// One thread owns four consecutive state elements and fetches kScanBatch chunks ahead of the serial
// recurrence so that enough loads are in flight to cover the memory latency.
constexpr int kScanBatch = 8;
__global__ void __launch_bounds__(256) nha_bwd_state_scan_kernel(const nha_chunk_desc d, const BwdWs w) {
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int KM = K * M, MV = M * V;
  const size_t nh = blockIdx.x;                     // (sequence, kv head) in x: no 65535 limit on packed batches
  const int n = nh / H, h = nh % H;
  const int len = d.cu_seqlens[n + 1] - d.cu_seqlens[n];
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int chunk0 = d.plan[n];
  const int el = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (el >= KM + MV) return;
  const bool is_k = el < KM;
  const int e = is_k ? el : el - KM;
  const int m = is_k ? e % M : e / V;
  const size_t per = is_k ? KM : MV;
  float* buf = is_k ? w.dkc : w.dvc;
  float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
  const float* dht = is_k ? d.d_hkt : d.d_hvt;
  if (dht) run = *(const float4*)(dht + nh * per + e);
  for (int hi = nchunks - 1; hi >= 0; hi -= kScanBatch) {
    float4 local[kScanBatch], decay[kScanBatch];
#pragma unroll
    for (int u = 0; u < kScanBatch; ++u) {
      const int ci = hi - u;
      if (ci >= 0) {
        const size_t cgi = (size_t)(chunk0 + ci) * H + h;
        local[u] = __ldcs((const float4*)(buf + cgi * per + e));
        if (is_k) decay[u] = *(const float4*)(w.gend + cgi * M + m);
        else decay[u].x = w.gend[cgi * M + m];
      }
    }
#pragma unroll
    for (int u = 0; u < kScanBatch; ++u) {
      const int ci = hi - u;
      if (ci >= 0) {
        const size_t cgi = (size_t)(chunk0 + ci) * H + h;
        __stcs((float4*)(buf + cgi * per + e), run);
        float4 a;
        if (is_k) a = make_float4(__expf(decay[u].x), __expf(decay[u].y), __expf(decay[u].z), __expf(decay[u].w));
        else { const float x = __expf(decay[u].x); a = make_float4(x, x, x, x); }
        run.x = run.x * a.x + local[u].x;
        run.y = run.y * a.y + local[u].y;
        run.z = run.z * a.z + local[u].z;
        run.w = run.w * a.w + local[u].w;
      }
    }
  }
  float* d0 = is_k ? d.dhk0 : d.dhv0;
  if (d0) *(float4*)(d0 + nh * per + e) = run;
}

// ================================================================================================
// 4b. inter-chunk pass (chunk-parallel): with DK, DV at the chunk's end, adds the inter-chunk parts of
//     dk', dv', ds', turns dgA - s' .* ds' into dg (reverse cumulative sum inside the chunk plus the
//     carry of all later chunks), undoes the shift and writes dk_gsa, dv, ds, dg.
// ================================================================================================
struct MarchLayout { int kp, vp, sp, sbe, G, DK, DV, DKb, DVb, X, cg, red, total; };
__host__ __device__ inline MarchLayout march_layout(int K, int V, int M) {
  MarchLayout L; int off = 0;
  const int kv_ = K > V ? K : V;
  const int mx = kv_ > M ? kv_ : M;
  L.kp = off; off = bup128(off + kChunk * (K + 8) * 2);
  L.vp = off; off = bup128(off + kChunk * (V + 8) * 2);
  L.sp = off; off = bup128(off + kChunk * (M + 8) * 2);
  L.sbe = off; off = bup128(off + kChunk * (M + 8) * 2);
  L.G = off; off = bup128(off + kChunk * (M + 4) * 4);
  L.DK = off; off = bup128(off + K * (M + 4) * 4);
  L.DV = off; off = bup128(off + M * (V + 4) * 4);
  L.DKb = off; off = bup128(off + K * (M + 8) * 2);
  L.DVb = off; off = bup128(off + M * (V + 8) * 2);
  L.X = off; off = bup128(off + kChunk * (mx + 4) * 4);
  L.cg = off; off = bup128(off + M * 4);
  L.red = off; off = bup128(off + kBwThreads * 4);
  L.total = off;
  return L;
}

__device__ __forceinline__ void nha_bwd_inter_kernel_body(const nha_chunk_desc d, const BwdWs w, const int cgb) {
  ChunkCtx c;
  const int cgx = cgb;
  if (!chunk_ctx(d, cgx, c)) return;
  // a chunk that another kernel handles is skipped, except that the CTA of a sequence's first chunk
  // always finishes the tail rows at the end of this kernel
  const bool mine = chunk_gate(w, cgx, blockIdx.y, d.H);
  if (!mine && c.ci != 0) return;
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int n = c.n, h = blockIdx.y;
  const int t0 = c.t0;
  const int len = c.len;
  const int shift = c.shift;
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int tid = threadIdx.x, warp = tid >> 5;
  const size_t nh = (size_t)n * H + h;
  extern __shared__ __align__(128) unsigned char smem[];
  const MarchLayout L = march_layout(K, V, M);
  const int mx = max(max(K, V), M);
  const int ldk = K + 8, ldv = V + 8, ldm = M + 8, ldg = M + 4, lddk = M + 4, lddv = V + 4, ldx = mx + 4;
  bf16* kp = (bf16*)(smem + L.kp);
  bf16* vp = (bf16*)(smem + L.vp);
  bf16* sp = (bf16*)(smem + L.sp);
  bf16* sbe = (bf16*)(smem + L.sbe);
  float* G = (float*)(smem + L.G);
  float* DK = (float*)(smem + L.DK);        // [K][M+4]
  float* DV = (float*)(smem + L.DV);        // [M][V+4]
  bf16* DKb = (bf16*)(smem + L.DKb);        // [K][M+8]
  bf16* DVb = (bf16*)(smem + L.DVb);        // [M][V+8]
  float* X = (float*)(smem + L.X);
  float* cgv = (float*)(smem + L.cg);
  float* red = (float*)(smem + L.red);
  const int chunk0 = d.plan[n];

  const int ci = c.ci;
  if (mine) {
  // ---- state gradients at this chunk's end
  {
    const float* dkg = w.dkc + ((size_t)cgx * H + h) * K * M;
    const float* dvg = w.dvc + ((size_t)cgx * H + h) * M * V;
    for (int i = tid; i < K * M; i += kBwThreads) DK[(i / M) * lddk + (i % M)] = dkg[i];
    for (int i = tid; i < M * V; i += kBwThreads) DV[(i / V) * lddv + (i % V)] = dvg[i];
  }
  for (int m = tid; m < M; m += kBwThreads) {
    float acc = 0.f;
    if (ci == nchunks - 1 && d.d_hkt && d.hkt && d.hvt) {
      for (int kk = 0; kk < K; ++kk) acc += d.d_hkt[nh * K * M + (size_t)kk * M + m] * d.hkt[nh * K * M + (size_t)kk * M + m];
      for (int vv = 0; vv < V; ++vv) acc += d.d_hvt[nh * M * V + (size_t)m * V + vv] * d.hvt[nh * M * V + (size_t)m * V + vv];
    }
    cgv[m] = acc;
  }
  __syncthreads();

  {
    const int c0 = ci * kChunk;
    const int lo = 0, hi = len - shift;
    // ---- gate-gradient carry of all later chunks, rebuilt from the state and its gradient at this
    //      chunk's end: cg[m] = <DK[:,m], hk[:,m]> + <DV[m,:], hv[m,:]>.  A running sum of
    //      dgA - s' ds' over the later tokens equals it exactly but would pile up rounding noise
    //      along the whole sequence.
    if (ci < nchunks - 1) {
      const bf16* hkn = (const bf16*)d.hk_chunks + ((size_t)(chunk0 + ci + 1) * H + h) * K * M;
      const bf16* hvn = (const bf16*)d.hv_chunks + ((size_t)(chunk0 + ci + 1) * H + h) * M * V;
      const int parts = kBwThreads / M;
      const int m = tid % M, part = tid / M;
      float acc = 0.f;
      if (part < parts) {
        for (int kk = part; kk < K; kk += parts) acc += DK[kk * lddk + m] * bf2f(hkn[(size_t)kk * M + m]);
        for (int vv = part; vv < V; vv += parts) acc += DV[m * lddv + vv] * bf2f(hvn[(size_t)m * V + vv]);
      }
      red[tid] = acc;
      __syncthreads();
      if (tid < M) {
        float sum = 0.f;
        for (int q = 0; q < parts; ++q) sum += red[q * M + tid];
        cgv[tid] = sum;
      }
      __syncthreads();
    }
    // ---- shifted kv-head tiles, cumulative gates, s' exp(Gend - G) --------------------------------------
    load_tile_bf16(kp, ldk, (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * K, (int64_t)H * K, c0 - shift, lo, hi, kChunk, K,
                   tid, kBwThreads);
    load_tile_bf16(vp, ldv, (const bf16*)d.v + ((size_t)t0 * H + h) * V, (int64_t)H * V, c0 - shift, lo, hi, kChunk, V, tid,
                   kBwThreads);
    load_tile_bf16(sp, ldm, (const bf16*)d.s + ((size_t)t0 * H + h) * M, (int64_t)H * M, c0 - shift, lo, hi, kChunk, M, tid,
                   kBwThreads);
    {
      const bf16* gg = (const bf16*)d.g + ((size_t)t0 * H + h) * M;
      for (int i = tid; i < kChunk * (M / 8); i += kBwThreads) {
        const int r = i / (M / 8), c8 = i - r * (M / 8);
        const int j = c0 + r - shift;
        float gv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
        if (j >= lo && j < hi) unpack8(*reinterpret_cast<const uint4*>(gg + (size_t)j * H * M + 8 * c8), gv);
#pragma unroll
        for (int e = 0; e < 8; ++e) G[r * ldg + 8 * c8 + e] = gv[e];
      }
    }
    for (int i = tid; i < K * M; i += kBwThreads) DKb[(i / M) * ldm + (i % M)] = f2bf(DK[(i / M) * lddk + (i % M)]);
    for (int i = tid; i < M * V; i += kBwThreads) DVb[(i / V) * ldv + (i % V)] = f2bf(DV[(i / V) * lddv + (i % V)]);
    __syncthreads();
    for (int m = tid; m < M; m += kBwThreads) {
      float run = 0.f;
#pragma unroll 16
      for (int r = 0; r < kChunk; ++r) {
        run += G[r * ldg + m];
        G[r * ldg + m] = run;
      }
    }
    __syncthreads();
    for (int i = tid; i < kChunk * M; i += kBwThreads) {
      const int r = i / M, m = i - r * M;
      sbe[r * ldm + m] = f2bf(bf2f(sp[r * ldm + m]) * __expf(G[(kChunk - 1) * ldg + m] - G[r * ldg + m]));
    }
    __syncthreads();
    // ---- dk = intra + sbe DK^T --------------------------------------------------------------------------
    tile_gemm<true, false, false>(X, ldx, sbe, ldm, DKb, ldm, 4, K / 16, M / 16, warp, kBwWarps);
    __syncthreads();
    for (int i = tid; i < kChunk * (K / 8); i += kBwThreads) {
      const int r = i / (K / 8), c8 = i - r * (K / 8);
      const int p = c0 + r, j = p - shift;
      if (j >= 0 && p < len) {
        const float* in = w.dkp + ((size_t)(t0 + p) * H + h) * K + 8 * c8;
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = X[r * ldx + 8 * c8 + e] + in[e];
        *reinterpret_cast<uint4*>((bf16*)d.dk_gsa + ((size_t)(t0 + j) * H + h) * K + 8 * c8) = pack8(f);
      }
    }
    __syncthreads();
    // ---- dv = window part + intra + sbe DV ----------------------------------------------------------------
    tile_gemm<true, true, false>(X, ldx, sbe, ldm, DVb, ldv, 4, V / 16, M / 16, warp, kBwWarps);
    __syncthreads();
    for (int i = tid; i < kChunk * (V / 8); i += kBwThreads) {
      const int r = i / (V / 8), c8 = i - r * (V / 8);
      const int p = c0 + r, j = p - shift;
      if (j >= 0 && p < len) {
        const float* in = w.dvp + ((size_t)(t0 + p) * H + h) * V + 8 * c8;
        const float* wa = w.dvacc + ((size_t)(t0 + j) * H + h) * V + 8 * c8;
        float f[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) f[e] = X[r * ldx + 8 * c8 + e] + in[e] + wa[e];
        *reinterpret_cast<uint4*>((bf16*)d.dv + ((size_t)(t0 + j) * H + h) * V + 8 * c8) = pack8(f);
      }
    }
    __syncthreads();
    // ---- ds = intra + exp(Gend - G) .* (k' DK + v' DV^T); dg by reverse cumulative sum ------------------------
    tile_gemm<true, true, false>(X, ldx, kp, ldk, DKb, ldm, 4, M / 16, K / 16, warp, kBwWarps);
    __syncthreads();
    tile_gemm<true, false, true>(X, ldx, vp, ldv, DVb, ldv, 4, M / 16, V / 16, warp, kBwWarps);
    __syncthreads();
    for (int i = tid; i < kChunk * M; i += kBwThreads) {
      const int r = i / M, m = i - r * M;
      const int p = c0 + r, j = p - shift;
      float ds = 0.f, dgraw = 0.f;
      if (j >= 0 && p < len) {
        const size_t hi2 = ((size_t)(t0 + p) * H + h) * M + m;
        ds = w.dsp[hi2] + __expf(G[(kChunk - 1) * ldg + m] - G[r * ldg + m]) * X[r * ldx + m];
        dgraw = w.dga[hi2] - bf2f(sp[r * ldm + m]) * ds;
        ((bf16*)d.ds)[((size_t)(t0 + j) * H + h) * M + m] = f2bf(ds);
      }
      X[r * ldx + m] = dgraw;
    }
    __syncthreads();
    for (int m = tid; m < M; m += kBwThreads) {
      float run = cgv[m];
      for (int r = kChunk - 1; r >= 0; --r) {
        run += X[r * ldx + m];
        const int p = c0 + r, j = p - shift;
        if (j >= 0 && p < len) ((bf16*)d.dg)[((size_t)(t0 + j) * H + h) * M + m] = f2bf(run);
      }
    }
  }
  }  // mine
  // ---- tokens that never enter the slot memory (done by the CTA of the sequence's first chunk) ---------------
  if (ci != 0) return;
  const int tail0 = max(0, len - shift);
  for (int i = tid; i < (len - tail0) * (V / 8); i += kBwThreads) {
    const int j = tail0 + i / (V / 8), c8 = i % (V / 8);
    const float* wa = w.dvacc + ((size_t)(t0 + j) * H + h) * V + 8 * c8;
    *reinterpret_cast<uint4*>((bf16*)d.dv + ((size_t)(t0 + j) * H + h) * V + 8 * c8) = pack8(wa);
  }
  const uint4 z4 = make_uint4(0u, 0u, 0u, 0u);
  for (int i = tid; i < (len - tail0) * (K / 8); i += kBwThreads) {
    const int j = tail0 + i / (K / 8), c8 = i % (K / 8);
    *reinterpret_cast<uint4*>((bf16*)d.dk_gsa + ((size_t)(t0 + j) * H + h) * K + 8 * c8) = z4;
  }
  for (int i = tid; i < (len - tail0) * (M / 8); i += kBwThreads) {
    const int j = tail0 + i / (M / 8), c8 = i % (M / 8);
    *reinterpret_cast<uint4*>((bf16*)d.ds + ((size_t)(t0 + j) * H + h) * M + 8 * c8) = z4;
    *reinterpret_cast<uint4*>((bf16*)d.dg + ((size_t)(t0 + j) * H + h) * M + 8 * c8) = z4;
  }
}

// One CTA walks `cpc` consecutive chunks (1 when the kernel handles every chunk; more when it is launched gated
// on the chunk flags and most chunks return at once, so that an all-clear launch costs few CTAs).
__global__ void __launch_bounds__(kBwThreads) nha_bwd_inter_kernel(const nha_chunk_desc d, const BwdWs w, const int cpc) {
  const int ncb = (int)((d.Ttot + kChunk - 1) / kChunk + d.N);
  // which of my chunks have work: one flag load per chunk, all at once (cpc <= 32)
  __shared__ unsigned todo;
  if (threadIdx.x < 32) {
    const int cgl = blockIdx.x * cpc + threadIdx.x;
    // (the CTA of a sequence's first chunk always runs: it finishes the sequence's tail rows)
    bool mine = (int)threadIdx.x < cpc && cgl < ncb;
    if (mine && !chunk_gate(w, cgl, blockIdx.y, d.H)) {
      const int n = d.plan[d.N + 1 + cgl];
      mine = n >= 0 && d.plan[n] == cgl;
    }
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (threadIdx.x == 0) todo = m;
  }
  __syncthreads();
  unsigned left = todo;
  while (left) {
    const int i = __ffs(left) - 1;
    left &= left - 1;
    nha_bwd_inter_kernel_body(d, w, blockIdx.x * cpc + i);
    __syncthreads();
  }
}


int check_chunk_desc(const nha_chunk_desc* d);
bool bwd_umma_supported(const nha_chunk_desc* d);
int bwd_umma_launch(const nha_chunk_desc* d, const BwdWs& w, int which, int* err, cudaStream_t cs);
bool bwd_wcols_umma_supported(const nha_chunk_desc* d);
int bwd_wcols_umma_launch(const nha_chunk_desc* d, const BwdWs& w, int* err, cudaStream_t cs);

}  // namespace nha

using namespace nha;

extern "C" int64_t nha_chunk_bwd_workspace_bytes(const nha_chunk_desc* d) {
  if (!d) return 0;
  return bwd_ws_layout(d, nullptr, nullptr);
}

static int bwd_run(const nha_chunk_desc* d, int stage_mask, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->o || !d->lse_swa || !d->lse_gsa || !d->hk_chunks || !d->hv_chunks || !d->d_o || !d->dq_gsa || !d->dq_swa ||
      !d->dk_gsa || !d->dk_swa || !d->dv || !d->ds || !d->dg)
    return NHA_ERR_BAD_ARG;
  if ((d->d_hkt == nullptr) != (d->d_hvt == nullptr)) return NHA_ERR_BAD_ARG;
  if (d->d_hkt && (!d->hkt || !d->hvt)) return NHA_ERR_BAD_ARG;
  if (d->V % 32 || d->K % 32) return NHA_ERR_UNSUPPORTED;
  if (d->q_offset != 0) return NHA_ERR_UNSUPPORTED;        // late-starting queries exist in the forward only
  const int64_t need = bwd_ws_layout(d, nullptr, nullptr);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  BwdWs w;
  bwd_ws_layout(d, &w, d->workspace);
  const WRowLayout L1 = wrow_layout(d->K, d->V);
  const WColLayout L2 = wcol_layout(d->K, d->V);
  const SlotLayout L3 = slot_layout(d->K, d->V, d->M);
  const MarchLayout L4 = march_layout(d->K, d->V, d->M);
  if (L1.total > kMaxSmem || L2.total > kMaxSmem || L3.total > kMaxSmem || L4.total > kMaxSmem) return NHA_ERR_SMEM;
  cudaStream_t cs = (cudaStream_t)stream;
  cudaError_t e;
  e = set_max_smem((const void*)nha_bwd_window_rows_kernel, L1.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  e = set_max_smem((const void*)nha_bwd_window_cols_kernel, L2.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  e = set_max_smem((const void*)nha_bwd_slot_kernel, L3.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  e = set_max_smem((const void*)nha_bwd_inter_kernel, L4.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  const LocalLayout L5 = local_layout(d->K, d->V, d->M);
  if (L5.total > kMaxSmem) return NHA_ERR_SMEM;
  e = set_max_smem((const void*)nha_bwd_local_terms_kernel, L5.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  dim3 grid(NCB, d->H), block(kBwThreads);
  // gated launches (only the chunks the forward flagged do work): sixteen chunks per CTA
  const int cpc = 16;
  dim3 ggrid((NCB + cpc - 1) / cpc, d->H);
  // Shapes with tensor-memory kernels: those handle every chunk the forward did not flag, the general
  // kernels below are launched gated on the flags and pick up the rest.
  const char* off = getenv("NHA_B200_NO_UMMA");
  const bool umma = bwd_umma_supported(d) && !(off && off[0] == '1');
  int* flags = d->plan + d->N + 1 + NCB;
  int* err = flags + (size_t)NCB * d->H;
  BwdWs wu = w, wg = w;                 // tensor-memory kernels: unflagged chunks; general kernels: flagged ones
  if (umma) {
    wu.flags = flags; wu.gate = 2;
    wg.flags = flags; wg.gate = 1;
  }
  if (stage_mask & 1) {
    if (umma && d->HQ != d->H) {
      // several query heads add their gate terms atomically; with one head per kv head every element has one writer
      cudaError_t e2 = cudaMemsetAsync(w.dga, 0, (size_t)d->Ttot * d->H * d->M * sizeof(float), cs);
      if (e2 != cudaSuccess) return record_cuda_error(e2);
    }
    if (umma) {
      st = bwd_umma_launch(d, wu, 0, err, cs);
      if (st != NHA_OK) return st;
    }
    if (umma) nha_bwd_window_rows_kernel<<<ggrid, block, L1.total, cs>>>(*d, wg, cpc);
    else nha_bwd_window_rows_kernel<<<grid, block, L1.total, cs>>>(*d, wg, 1);
    st = check_launch();
    if (st != NHA_OK) return st;
  }
  if (stage_mask & 2) {
    // the window part does not depend on the gates: every chunk takes the tensor-memory kernel when the
    // shape has one
    if (bwd_wcols_umma_supported(d) && !(off && off[0] == '1')) {
      st = bwd_wcols_umma_launch(d, w, err, cs);
    } else {
      nha_bwd_window_cols_kernel<<<grid, block, L2.total, cs>>>(*d, w);
      st = check_launch();
    }
    if (st != NHA_OK) return st;
  }
  if (stage_mask & 4) {
    if (umma) nha_bwd_slot_kernel<<<ggrid, block, L3.total, cs>>>(*d, wg, cpc);
    else nha_bwd_slot_kernel<<<grid, block, L3.total, cs>>>(*d, wg, 1);
    st = check_launch();
    if (st != NHA_OK) return st;
  }
  if (stage_mask & 8) {
    if (umma) nha_bwd_local_terms_kernel<<<ggrid, block, L5.total, cs>>>(*d, wg, cpc);
    else nha_bwd_local_terms_kernel<<<grid, block, L5.total, cs>>>(*d, wg, 1);
    st = check_launch();
    if (st != NHA_OK) return st;
    const int SD = d->K * d->M + d->M * d->V;
    nha_bwd_state_scan_kernel<<<dim3(d->N * d->H, (SD / 4 + 255) / 256), 256, 0, cs>>>(*d, w);
    st = check_launch();
    if (st != NHA_OK) return st;
  }
  if (stage_mask & 16) {
    if (umma) {
      st = bwd_umma_launch(d, wu, 1, err, cs);
      if (st != NHA_OK) return st;
    }
    if (umma) nha_bwd_inter_kernel<<<ggrid, block, L4.total, cs>>>(*d, wg, cpc);
    else nha_bwd_inter_kernel<<<grid, block, L4.total, cs>>>(*d, wg, 1);
    st = check_launch();
  }
  return st;
}

extern "C" int nha_chunk_bwd(const nha_chunk_desc* d, void* stream) { return bwd_run(d, 31, stream); }

extern "C" int nha_chunk_bwd_stage(const nha_chunk_desc* d, int stage, void* stream) {
  if (stage < 0 || stage > 4) return NHA_ERR_BAD_ARG;
  return bwd_run(d, 1 << stage, stream);
}
