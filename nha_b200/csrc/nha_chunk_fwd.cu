// Output pass of the chunked NHA forward (sm_100a): one CTA per (chunk, kv head), all query heads
// of the group served from the same shared-memory copies of the chunk's k', v', gates and
// chunk-start states.  Per query head and 64-token chunk it forms
//     slot logits   ok = scale * ( exp(G) .* (q Hk)  +  a_I .* (tril(q k'^T) (s' .* b_I)) )
//     window logits sw = scale * q_swa k_swa^T       (keys t-wl .. t, tiles of 64 keys)
//     ONE softmax over [ok | sw]   (two sweeps: statistics, then probabilities)
//     o = (p_slot .* exp(G)) Hv + tril((p_slot .* a_I)(s' .* b_I)^T) v' + p_win v_win
// with G the chunk-local cumulative shifted log gate and (a_I, b_I) the decay factors of 16-row
// block I around that block's own per-slot reference, so no factor leaves exp(+-75).
//
// Replaces chunk_nha_fused_o_kernel (nha_fla/ops/nha/chunk_fused.py:117-283) and, for chunk_nha,
// the flash-attn varlen forward + fla chunk_gsa forward + log-sum-exp merge
// (nha_fla/ops/nha/chunk.py:423-470).
#include <stdlib.h>

#include "nha_common.cuh"

namespace nha {

constexpr int kFwdThreads = 256;
constexpr int kFwdWarps = kFwdThreads / 32;

struct FwdLayout {
  int kp, vp, G, Hk, Hv, SB, qb, OK, SA, AB, wt, pg, pa, patch, rows, total;
};

__host__ __device__ inline int up128(int x) { return (x + 127) & ~127; }

__host__ __device__ inline FwdLayout fwd_layout(int K, int V, int M) {
  FwdLayout L;
  int off = 0;
  const int KV = K > V ? K : V;
  L.kp = off; off = up128(off + kChunk * (K + 8) * 2);
  L.vp = off; off = up128(off + kChunk * (V + 8) * 2);
  L.G = off; off = up128(off + kChunk * (M + 4) * 4);
  L.Hk = off; off = up128(off + K * (M + 8) * 2);
  L.Hv = off; off = up128(off + M * (V + 8) * 2);
  L.SB = off; off = up128(off + 160 * (M + 8) * 2);
  L.qb = off; off = up128(off + kChunk * (K + 8) * 2);
  L.OK = off; off = up128(off + kChunk * (M + 4) * 4);
  const int sa_cols = M > kChunk ? M : kChunk;
  L.SA = off; off = up128(off + kChunk * (sa_cols + 4) * 4);
  L.AB = off; off = up128(off + kChunk * (kChunk + 8) * 2);
  L.wt = off; off = up128(off + kChunk * (KV + 8) * 2);
  L.pg = off; off = up128(off + kChunk * (M + 8) * 2);
  L.pa = off; off = up128(off + kChunk * (M + 8) * 2);
  L.patch = off; off = up128(off + kFwdWarps * 256 * 4);
  L.rows = off; off = up128(off + 6 * kChunk * 4);
  L.total = off;
  return L;
}

// first row of SB_I inside the stacked block operand (blocks of 16, 32, 48, 64 rows)
__device__ __forceinline__ int sb_row0(int I) { return 8 * I * (I + 1); }

// Per-block reference exponent of slot m for row block I: midpoint of the block's own range.
__device__ __forceinline__ float block_ref(const float* G, int ldg, int I, int m) {
  const float gn = I > 0 ? G[(16 * I - 1) * ldg + m] : 0.f;
  return 0.5f * (gn + G[(16 * I + 15) * ldg + m]);
}

// X[16I.., :M] = AB[16I.., 0:16(I+1)] * SB_I            (tiles (I, nt) dealt to the warps)
__device__ __forceinline__ void gemm_rows_times_sb(float* X, int ldx, const bf16* AB, int ldab, const bf16* SB,
                                                   int ldsb, int M, int warp) {
  using namespace nvcuda::wmma;
  const int Nt = M / 16;
  for (int t = warp; t < 4 * Nt; t += kFwdWarps) {
    const int I = t / Nt, nt = t % Nt;
    fragment<accumulator, 16, 16, 16, float> acc;
    fill_fragment(acc, 0.f);
    for (int kt = 0; kt <= I; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
      fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
      load_matrix_sync(fa, AB + 16 * I * ldab + 16 * kt, ldab);
      load_matrix_sync(fb, SB + (sb_row0(I) + 16 * kt) * ldsb + 16 * nt, ldsb);
      mma_sync(acc, fa, fb, acc);
    }
    store_matrix_sync(X + 16 * I * ldx + 16 * nt, acc, ldx, mem_row_major);
  }
}

// Y[16I.., 0:16(I+1)] = PA[16I.., :M] * SB_I^T           (tiles (I, nt <= I))
__device__ __forceinline__ void gemm_rows_times_sbT(float* Y, int ldy, const bf16* PA, int ldpa, const bf16* SB,
                                                    int ldsb, int M, int warp) {
  using namespace nvcuda::wmma;
  for (int t = warp; t < 16; t += kFwdWarps) {
    const int I = t >> 2, nt = t & 3;
    if (nt > I) continue;
    fragment<accumulator, 16, 16, 16, float> acc;
    fill_fragment(acc, 0.f);
    for (int kt = 0; kt < M / 16; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
      fragment<matrix_b, 16, 16, 16, bf16, col_major> fb;
      load_matrix_sync(fa, PA + 16 * I * ldpa + 16 * kt, ldpa);
      load_matrix_sync(fb, SB + (sb_row0(I) + 16 * nt) * ldsb + 16 * kt, ldsb);
      mma_sync(acc, fa, fb, acc);
    }
    store_matrix_sync(Y + 16 * I * ldy + 16 * nt, acc, ldy, mem_row_major);
  }
}

// AB = bf16(lower-triangular part of SA[64][64]) (diagonal blocks masked element-wise, upper blocks zero)
__device__ __forceinline__ void tril_to_bf16(bf16* AB, int ldab, const float* SA, int ldsa, int tid) {
  for (int i = tid; i < kChunk * kChunk; i += kFwdThreads) {
    const int r = i >> 6, c = i & 63;
    AB[r * ldab + c] = f2bf(c <= r ? SA[r * ldsa + c] : 0.f);
  }
}

// `only_flagged` (optional): [chunks, H] flags; when given, a CTA whose flag is zero has nothing to do
// (the tensor-memory kernel already produced that chunk).
__device__ __forceinline__ void nha_chunk_fwd_kernel_body(const nha_chunk_desc d, const int* __restrict__ only_flagged, const int cgb) {
  using namespace nvcuda::wmma;
  const int K = d.K, V = d.V, M = d.M, H = d.H, HQ = d.HQ, NG = HQ / H;
  const int N = d.N;
  const int cg = cgb;                       // global chunk index
  const int h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
  if (only_flagged && only_flagged[(size_t)cg * H + h] == 0) return;
  const int ci = rc.ci;
  const int t0 = rc.t0;
  const int len = rc.len;
  const int c0 = ci * kChunk;
  if (c0 < d.q_offset) return;                     // chunks below q_offset have no queries (q_offset is a multiple of 64)
  const int tq0 = t0 - d.q_offset;                 // row of q / o / lse that holds position 0 of the sequence
  const int wl = seq_window(d, n);
  const int shift = seq_shift(d, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ __align__(128) unsigned char smem[];
  const FwdLayout L = fwd_layout(K, V, M);
  const int KV = K > V ? K : V;
  const int ldk = K + 8, ldv = V + 8, ldg = M + 4, ldhk = M + 8, ldhv = V + 8, ldsb = M + 8;
  const int ldsa = (M > kChunk ? M : kChunk) + 4, ldab = kChunk + 8, ldw = KV + 8, ldp = M + 8;
  bf16* kp = (bf16*)(smem + L.kp);
  bf16* vp = (bf16*)(smem + L.vp);
  float* G = (float*)(smem + L.G);
  bf16* Hk = (bf16*)(smem + L.Hk);
  bf16* Hv = (bf16*)(smem + L.Hv);
  bf16* SB = (bf16*)(smem + L.SB);
  bf16* qb = (bf16*)(smem + L.qb);
  float* OK = (float*)(smem + L.OK);
  float* SA = (float*)(smem + L.SA);
  bf16* AB = (bf16*)(smem + L.AB);
  bf16* wt = (bf16*)(smem + L.wt);
  bf16* pg = (bf16*)(smem + L.pg);
  bf16* pa = (bf16*)(smem + L.pa);
  float* patch = (float*)(smem + L.patch) + warp * 256;
  float* row_m = (float*)(smem + L.rows);          // running max of the window logits
  float* row_l = row_m + kChunk;                   // running sum
  float* row_L = row_l + kChunk;                   // joint log-sum-exp

  // ---- kv-head data of the chunk: shifted k', v', s', g' and the chunk-start states ----------------
  {
    const bf16* kg = (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * K;
    const bf16* vg = (const bf16*)d.v + ((size_t)t0 * H + h) * V;
    const int lo = 0, hi = len - shift;            // valid source rows j = p - shift in [0, len - shift)
    load_tile_bf16(kp, ldk, kg, (int64_t)H * K, c0 - shift, lo, hi, kChunk, K, tid, kFwdThreads);
    load_tile_bf16(vp, ldv, vg, (int64_t)H * V, c0 - shift, lo, hi, kChunk, V, tid, kFwdThreads);
    const bf16* sg = (const bf16*)d.s + ((size_t)t0 * H + h) * M;
    load_tile_bf16(pg, ldp, sg, (int64_t)H * M, c0 - shift, lo, hi, kChunk, M, tid, kFwdThreads);   // s' staged in pg
    const bf16* gg = (const bf16*)d.g + ((size_t)t0 * H + h) * M;
    for (int i = tid; i < kChunk * (M / 8); i += kFwdThreads) {
      const int r = i / (M / 8), c8 = i - r * (M / 8);
      const int j = c0 + r - shift;
      float gv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (j >= lo && j < hi) unpack8(*reinterpret_cast<const uint4*>(gg + (size_t)j * H * M + 8 * c8), gv);
#pragma unroll
      for (int e = 0; e < 8; ++e) G[r * ldg + 8 * c8 + e] = gv[e];
    }
    const bf16* hkc = (const bf16*)d.hk_chunks + ((size_t)cg * H + h) * K * M;
    const bf16* hvc = (const bf16*)d.hv_chunks + ((size_t)cg * H + h) * M * V;
    load_tile_bf16(Hk, ldhk, hkc, M, 0, 0, K, K, M, tid, kFwdThreads);
    load_tile_bf16(Hv, ldhv, hvc, V, 0, 0, M, M, V, tid, kFwdThreads);
  }
  __syncthreads();
  for (int m = tid; m < M; m += kFwdThreads) {
    float run = 0.f;
#pragma unroll 16
    for (int r = 0; r < kChunk; ++r) {
      run += G[r * ldg + m];
      G[r * ldg + m] = run;
    }
  }
  __syncthreads();
  // stacked block operands SB_I[i][m] = s'[i][m] * exp(R_I[m] - G[i][m]), i < 16(I+1)
  for (int i = tid; i < 160 * M; i += kFwdThreads) {
    const int row = i / M, m = i - row * M;
    const int I = row < 16 ? 0 : (row < 48 ? 1 : (row < 96 ? 2 : 3));
    const int r = row - sb_row0(I);
    const float ref = block_ref(G, ldg, I, m);
    SB[row * ldsb + m] = f2bf(bf2f(pg[r * ldp + m]) * clamp_exp(ref - G[r * ldg + m]));
  }
  __syncthreads();

  const int jt_hi = ci;
  const int jt_lo = wl < 0 ? 0 : max(0, c0 - wl) / kChunk;
  const int rq = tid >> 2, sub = tid & 3;          // 4 threads per query row for the row statistics

  for (int qh = 0; qh < NG; ++qh) {
    const int hq = h * NG + qh;
    // ---- slot logits ---------------------------------------------------------------------------
    load_tile_bf16(qb, ldk, (const bf16*)d.q_gsa + ((int64_t)tq0 * HQ + hq) * K, (int64_t)HQ * K, c0, 0, len, kChunk, K,
                   tid, kFwdThreads);
    __syncthreads();
    tile_gemm<true, true, false>(OK, ldg, qb, ldk, Hk, ldhk, 4, M / 16, K / 16, warp, kFwdWarps);
    tile_gemm<true, false, false, 0, 1>(SA, ldsa, qb, ldk, kp, ldk, 4, 4, K / 16, warp, kFwdWarps);
    __syncthreads();
    tril_to_bf16(AB, ldab, SA, ldsa, tid);
    for (int i = tid; i < kChunk * M; i += kFwdThreads) {
      const int r = i / M, m = i - r * M;
      OK[r * ldg + m] *= d.scale * __expf(G[r * ldg + m]);
    }
    __syncthreads();
    gemm_rows_times_sb(SA, ldsa, AB, ldab, SB, ldsb, M, warp);
    __syncthreads();
    for (int i = tid; i < kChunk * M; i += kFwdThreads) {
      const int r = i / M, m = i - r * M;
      const float aI = clamp_exp(G[r * ldg + m] - block_ref(G, ldg, r >> 4, m));
      OK[r * ldg + m] += d.scale * aI * SA[r * ldsa + m];
    }
    __syncthreads();
    // row statistics of the slot logits
    float mg = -INFINITY, lg = 0.f;
    {
      for (int m = sub; m < M; m += 4) mg = fmaxf(mg, OK[rq * ldg + m]);
      mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, 1));
      mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, 2));
      for (int m = sub; m < M; m += 4) lg += __expf(OK[rq * ldg + m] - mg);
      lg += __shfl_xor_sync(0xffffffffu, lg, 1);
      lg += __shfl_xor_sync(0xffffffffu, lg, 2);
    }
    // ---- window logits, sweep 1: statistics ----------------------------------------------------
    load_tile_bf16(qb, ldk, (const bf16*)d.q_swa + ((int64_t)tq0 * HQ + hq) * K, (int64_t)HQ * K, c0, 0, len, kChunk, K,
                   tid, kFwdThreads);
    float ms = -INFINITY, ls = 0.f;
    const int pos = c0 + rq;
    for (int jt = jt_lo; jt <= jt_hi; ++jt) {
      __syncthreads();
      load_tile_bf16(wt, ldw, (const bf16*)d.k_swa + ((size_t)t0 * H + h) * K, (int64_t)H * K, jt * kChunk, 0, len,
                     kChunk, K, tid, kFwdThreads);
      __syncthreads();
      tile_gemm<true, false, false>(SA, ldsa, qb, ldk, wt, ldw, 4, 4, K / 16, warp, kFwdWarps);
      __syncthreads();
      float tmax = -INFINITY;
      for (int c = sub; c < kChunk; c += 4) {
        const int key = jt * kChunk + c;
        const bool ok = key <= pos && (wl < 0 || key >= pos - wl);
        if (ok) tmax = fmaxf(tmax, SA[rq * ldsa + c] * d.scale);
      }
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 1));
      tmax = fmaxf(tmax, __shfl_xor_sync(0xffffffffu, tmax, 2));
      // every lane takes part in the shuffles; rows without a visible key in this tile add nothing
      const float mnew = fmaxf(ms, tmax);
      float part = 0.f;
      for (int c = sub; c < kChunk; c += 4) {
        const int key = jt * kChunk + c;
        const bool ok = key <= pos && (wl < 0 || key >= pos - wl);
        if (ok) part += __expf(SA[rq * ldsa + c] * d.scale - mnew);
      }
      part += __shfl_xor_sync(0xffffffffu, part, 1);
      part += __shfl_xor_sync(0xffffffffu, part, 2);
      if (mnew > -INFINITY) {
        ls = ls * __expf(ms - mnew) + part;
        ms = mnew;
      }
    }
    {
      const float lse_g = mg + __logf(lg);
      const float lse_s = ms + __logf(ls);
      const float mx = fmaxf(lse_g, lse_s);
      const float Lj = mx + __logf(__expf(lse_g - mx) + __expf(lse_s - mx));
      if (sub == 0) {
        row_L[rq] = Lj;
        if (pos < len) {
          d.lse_gsa[(size_t)(tq0 + pos) * HQ + hq] = lse_g;
          d.lse_swa[(size_t)(tq0 + pos) * HQ + hq] = lse_s;
        }
      }
    }
    __syncthreads();
    // ---- sweep 2: probabilities and the output ---------------------------------------------------
    for (int i = tid; i < kChunk * M; i += kFwdThreads) {
      const int r = i / M, m = i - r * M;
      const float p = __expf(OK[r * ldg + m] - row_L[r]);
      const float gl = G[r * ldg + m];
      pg[r * ldp + m] = f2bf(p * __expf(gl));
      pa[r * ldp + m] = f2bf(p * clamp_exp(gl - block_ref(G, ldg, r >> 4, m)));
    }
    __syncthreads();
    // output tiles: warp -> row tile (warp & 3), column tiles (warp >> 2) + 2 * i
    const int mt = warp & 3;
    constexpr int kMaxCT = 4;                       // V <= 128
    const int CT = V / 32;                          // column tiles per warp
    fragment<accumulator, 16, 16, 16, float> oacc[kMaxCT];
#pragma unroll
    for (int i = 0; i < kMaxCT; ++i) fill_fragment(oacc[i], 0.f);
    // (p_slot .* exp(G)) Hv
    for (int kt = 0; kt < M / 16; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
      load_matrix_sync(fa, pg + 16 * mt * ldp + 16 * kt, ldp);
#pragma unroll
      for (int i = 0; i < kMaxCT; ++i) {
        if (i < CT) {
          fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
          load_matrix_sync(fb, Hv + 16 * kt * ldhv + 16 * ((warp >> 2) + 2 * i), ldhv);
          mma_sync(oacc[i], fa, fb, oacc[i]);
        }
      }
    }
    // tril((p_slot .* a_I) SB_I^T) v'
    gemm_rows_times_sbT(SA, ldsa, pa, ldp, SB, ldsb, M, warp);
    __syncthreads();
    tril_to_bf16(AB, ldab, SA, ldsa, tid);
    __syncthreads();
    for (int kt = 0; kt <= mt; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
      load_matrix_sync(fa, AB + 16 * mt * ldab + 16 * kt, ldab);
#pragma unroll
      for (int i = 0; i < kMaxCT; ++i) {
        if (i < CT) {
          fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
          load_matrix_sync(fb, vp + 16 * kt * ldv + 16 * ((warp >> 2) + 2 * i), ldv);
          mma_sync(oacc[i], fa, fb, oacc[i]);
        }
      }
    }
    // window tiles
    for (int jt = jt_lo; jt <= jt_hi; ++jt) {
      __syncthreads();
      load_tile_bf16(wt, ldw, (const bf16*)d.k_swa + ((size_t)t0 * H + h) * K, (int64_t)H * K, jt * kChunk, 0, len,
                     kChunk, K, tid, kFwdThreads);
      __syncthreads();
      tile_gemm<true, false, false>(SA, ldsa, qb, ldk, wt, ldw, 4, 4, K / 16, warp, kFwdWarps);
      __syncthreads();
      for (int i = tid; i < kChunk * kChunk; i += kFwdThreads) {
        const int r = i >> 6, c = i & 63;
        const int key = jt * kChunk + c, pq = c0 + r;
        const bool ok = key <= pq && (wl < 0 || key >= pq - wl) && pq < len;
        AB[r * ldab + c] = f2bf(ok ? __expf(SA[r * ldsa + c] * d.scale - row_L[r]) : 0.f);
      }
      load_tile_bf16(wt, ldw, (const bf16*)d.v + ((size_t)t0 * H + h) * V, (int64_t)H * V, jt * kChunk, 0, len, kChunk,
                     V, tid, kFwdThreads);
      __syncthreads();
      for (int kt = 0; kt < 4; ++kt) {
        fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
        load_matrix_sync(fa, AB + 16 * mt * ldab + 16 * kt, ldab);
#pragma unroll
        for (int i = 0; i < kMaxCT; ++i) {
          if (i < CT) {
            fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
            load_matrix_sync(fb, wt + 16 * kt * ldw + 16 * ((warp >> 2) + 2 * i), ldw);
            mma_sync(oacc[i], fa, fb, oacc[i]);
          }
        }
      }
    }
    // ---- store the output tiles through a per-warp patch ------------------------------------------
#pragma unroll
    for (int i = 0; i < kMaxCT; ++i) {
      if (i < CT) {
        store_matrix_sync(patch, oacc[i], 16, mem_row_major);
        __syncwarp();
        const int ct = (warp >> 2) + 2 * i;
        const int r = lane >> 1, half = lane & 1;
        const int pq = c0 + 16 * mt + r;
        if (pq < len) {
          float f[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) f[e] = patch[r * 16 + 8 * half + e];
          *reinterpret_cast<uint4*>((bf16*)d.o + ((size_t)(tq0 + pq) * HQ + hq) * V + 16 * ct + 8 * half) = pack8(f);
        }
        __syncwarp();
      }
    }
    __syncthreads();
  }
}

// One CTA walks `cpc` consecutive chunks (1 when the kernel handles every chunk; more when it is launched gated
// on the chunk flags and most chunks return at once, so that an all-clear launch costs few CTAs).
__global__ void __launch_bounds__(kFwdThreads) nha_chunk_fwd_kernel(const nha_chunk_desc d, const int* __restrict__ only_flagged, const int cpc) {
  const int ncb = (int)((d.Ttot + kChunk - 1) / kChunk + d.N);
  // which of my chunks have work: one flag load per chunk, all at once (cpc <= 32)
  __shared__ unsigned todo;
  if (threadIdx.x < 32) {
    const int cgl = blockIdx.x * cpc + threadIdx.x;
    const bool mine = (int)threadIdx.x < cpc && cgl < ncb &&
                      (only_flagged == nullptr || only_flagged[(size_t)cgl * d.H + blockIdx.y] != 0);
    const unsigned m = __ballot_sync(0xffffffffu, mine);
    if (threadIdx.x == 0) todo = m;
  }
  __syncthreads();
  unsigned left = todo;
  while (left) {
    const int i = __ffs(left) - 1;
    left &= left - 1;
    nha_chunk_fwd_kernel_body(d, only_flagged, blockIdx.x * cpc + i);
    __syncthreads();
  }
}

int64_t state_workspace_bytes(const nha_chunk_desc* d);
int check_chunk_desc(const nha_chunk_desc* d);
int chunk_output_pass_umma(const nha_chunk_desc* d, int* flags, int* err, cudaStream_t cs);
bool fwd_pipe_supported(const nha_chunk_desc* d);

}  // namespace nha

using namespace nha;

extern "C" int64_t nha_chunk_fwd_workspace_bytes(const nha_chunk_desc* d) {
  if (!d) return 0;
  return state_workspace_bytes(d);
}

extern "C" int nha_chunk_output_pass(const nha_chunk_desc* d, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->o || !d->lse_swa || !d->lse_gsa || !d->hk_chunks || !d->hv_chunks) return NHA_ERR_BAD_ARG;
  if (d->V % 32) return NHA_ERR_UNSUPPORTED;
  if (d->q_offset != 0 && (d->q_offset < 0 || d->q_offset % kChunk || d->N != 1 || !fwd_pipe_supported(d)))
    return NHA_ERR_UNSUPPORTED;                    // only the pipelined output pass knows queries that start late
  cudaStream_t cs = (cudaStream_t)stream;
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  // Shapes with a tensor-memory kernel run it first; it flags the (rare) chunks whose gates decay too
  // fast for its single decay reference, and the general kernel below then computes only those.
  int* flags = d->plan + d->N + 1 + NCB;
  int* err = flags + (size_t)NCB * d->H;
  const char* off = getenv("NHA_B200_NO_UMMA");
  bool umma_done = false;
  if (!(off && off[0] == '1')) {
    st = chunk_output_pass_umma(d, flags, err, cs);
    if (st == NHA_OK) umma_done = true;
    else if (st != NHA_ERR_UNSUPPORTED) return st;
  }
  if (!umma_done) {
    // every chunk is the general kernels' job, in the backward too
    cudaError_t e0 = cudaMemsetAsync(flags, 1, (size_t)NCB * d->H * sizeof(int), cs);
    if (e0 != cudaSuccess) return record_cuda_error(e0);
  }
  const FwdLayout L = fwd_layout(d->K, d->V, d->M);
  if (L.total > kMaxSmem) return umma_done ? NHA_OK : NHA_ERR_SMEM;
  cudaError_t e = set_max_smem((const void*)nha_chunk_fwd_kernel, L.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  dim3 grid(NCB, d->H), block(kFwdThreads);
  if (umma_done) {
    // only the flagged chunks do work: sixteen chunks per CTA keep an all-clear launch short
    const int cpc = 16;
    nha_chunk_fwd_kernel<<<dim3((grid.x + cpc - 1) / cpc, grid.y), block, L.total, cs>>>(*d, flags, cpc);
  } else {
    nha_chunk_fwd_kernel<<<grid, block, L.total, cs>>>(*d, nullptr, 1);
  }
  return check_launch();
}

// Device-side error word of the last tensor-memory output pass that used this descriptor's plan
// (non-zero: a bounded wait on an MMA completion barrier ran out).  Synchronises the stream.
extern "C" int nha_chunk_device_error(const nha_chunk_desc* d, void* stream) {
  if (!d || !d->plan) return -1;
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, d->plan + d->N + 1 + NCB + (size_t)NCB * d->H, sizeof(int), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return -1;
  return v;
}

extern "C" int nha_chunk_fwd(const nha_chunk_desc* d, void* stream) {
  int st = nha_chunk_plan(d, stream);
  if (st != NHA_OK) return st;
  st = nha_chunk_state_pass(d, stream);
  if (st != NHA_OK) return st;
  return nha_chunk_output_pass(d, stream);
}
