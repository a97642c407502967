// Backward of the chunked NHA operator on the sm_100a tensor-core path (tcgen05.mma, accumulators in
// tensor memory, one thread per row for the element-wise work).  Two chunk-parallel kernels bracket the
// state-gradient march of nha_chunk_bwd.cu:
//
//   rows pass  (per chunk, kv head; query-row side)
//       ok, p_slot recomputed as in the forward;  dp_slot = exp(G) .* (do Hv^T) + a .* (tril(do v'^T) SB)
//       dz_slot = p (dp - delta) + d_lse_gsa softmax(ok);  dz_win = p_win (do v_win^T - delta)
//       dq_gsa = scale (dz exp G) Hk^T + tril(scale (dz a) SB^T) k',   dq_swa = scale dz_win k_swa
//       stores delta, the joint LSE, dgA = ok dz + p dp, and the bf16 copies of dz and p (decayed by
//       exp(G) for the march, by a for the columns pass)
//   columns pass (per chunk, kv head; key-row side), after the march has left DK, DV at every chunk end
//       dk' = tril(dza SB^T)^T q + sbe DK^T,   dv' = tril(pa SB^T)^T do + sbe DV
//       ds' = b .* (tril(q k'^T)^T dza + tril(do v'^T)^T pa) + be .* (k' DK + v' DV^T)
//       dg  = reverse cumulative sum of dgA - s' ds' inside the chunk + carry <DK,hk> + <DV,hv>
//       un-shifted stores of dk_gsa, dv (+ window part), ds, dg
//   (SB = s' .* b, sbe = s' .* exp(Gend - G), a = exp(G - R), b = exp(R - G), R = Gend / 2 per slot.)
// Transposed products use MN-major operand descriptors, so no tile is ever transposed in memory.
// Chunks the forward flagged (gates too steep for the single reference R) are skipped here and
// handled by the general kernels.
//
// Replaces, with nha_chunk_bwd.cu, ChunkNativeHybridAttentionFunction.backward
// (nha_fla/ops/nha/chunk.py:491-564) and chunk_gsa_bwd_with_lse (nha_fla/ops/nha/chunk_gsa.py:52-122).
#include "nha_bwd_common.cuh"
#include "nha_common.cuh"
#include "nha_umma.cuh"

namespace nha {

using namespace umma;

constexpr int kRowsThreads = 256;        // rows pass: two threads per row
constexpr int kColsThreads = 256;        // columns pass: likewise

// ================================================================================================
// rows pass
// ================================================================================================
template <int D, int R>
struct RowsLayout {
  static constexpr int KT = D / 64;
  static constexpr int kATile = R * 128;
  static constexpr int tQ = 0;                          // q_gsa; reused for the window key/value tiles
  static constexpr int tQS = tQ + KT * kATile;          // q_swa
  static constexpr int tDO = tQS + KT * kATile;         // do
  static constexpr int tK = tDO + KT * kATile;          // k'
  static constexpr int tV = tK + KT * 8192;             // v'
  static constexpr int tHk = tV + KT * 8192;            // Hk [D][64]
  static constexpr int tHv = tHk + D * 128;             // Hv [64][D]
  static constexpr int tSB = tHv + KT * 8192;           // s' .* b
  static constexpr int tWVx = tSB + 8192;               // window values when they do not fit behind tQ
  static constexpr int bufA = tWVx + (R == 128 ? 0 : KT * 8192);   // tril(A) -> dza -> tril(E) -> dz_win
  static constexpr int bufB = bufA + kATile;            // tril(Av) -> dzg
  static constexpr int oA = bufB + kATile;              // fp32 [64][65]: cumulative gates, then a = exp(G - R)
  static constexpr int oR = oA + 64 * 65 * 4;           // fp32 [64] exp(R)
  static constexpr int oX = oR + 256;                   // fp32 [2 halves][128 rows]: partial <do, o> of the column halves
  static constexpr int oBar = oX + 1024;
  static constexpr int total = oBar + 64 + 1024;
  // One head per CTA (R == 64): tiles are reused as soon as the last product that reads them has completed.
  //   v' and Hv are read by MMA group 1 only      -> p .* a and p .* exp(G) (operands of the local terms, and the
  //                                              source of the coalesced copy-out of the four bf16 copies)
  //   k' and Hk are dead after dq_gsa          -> window keys / values of the even window tiles
  //   q_gsa is dead after the local terms     -> window keys of the odd window tiles (values: tWVx)
  // so the window loop is double-buffered and needs no global round trip.  With two heads per tile (R == 128)
  // k', v', Hk, Hv serve every head tile and nothing is reused: one window buffer behind q_gsa.
  static constexpr bool kAlias = R == 64;
  static constexpr int tPA = tV, tPG = tHv;             // only with kAlias
  static constexpr int tW0 = kAlias ? tK : tQ, tWV0 = kAlias ? tHk : (R == 128 ? tQ + KT * 8192 : tWVx);
  static constexpr int tW1 = tQ, tWV1 = R == 128 ? tQ + KT * 8192 : tWVx;
  // Tensor-memory columns.  D == 64 fits 256 columns (two CTAs per SM) by reusing columns as soon as
  // their accumulator has been read: A, Av, QH, Y -> X, X2 -> E -> dq_gsa (over QH), local terms (over
  // Av, Y), then the window loop's S, dP, dq_swa (over A, Av, Y).
  static constexpr int kTmemCols = D == 64 ? 256 : 512;
  static constexpr int cA = 0, cAv = 64, cQH = 128, cY = 192;
  static constexpr int cDQ = D == 64 ? 128 : 256, cDQS = D == 64 ? 192 : 384;
  static constexpr int cS = D == 64 ? 0 : 128, cDP = D == 64 ? 64 : 192;
  // chunk-local state-gradient terms, read out before the window loop reuses the columns
  static constexpr int cLK = D == 64 ? 64 : 0, cLV = D == 64 ? 192 : 128;
  static_assert(total <= 227 * 1024, "shared memory of the rows pass");
};

// Two threads per row: the warps w and w + 4 share a TMEM lane quarter and take alternate 32-column
// halves of every 64-column accumulator.
template <int D, int R>
__global__ void __launch_bounds__(kRowsThreads, (D == 64 && R == 64) ? 2 : 1)
    nha_bwd_rows_umma_kernel(const nha_chunk_desc d, const BwdWs w, int* __restrict__ err) {
  typedef RowsLayout<D, R> L;
  constexpr int KT = L::KT, TH = R / 64, M = 64, NT = kRowsThreads;
  constexpr float kLog2e = 1.4426950408889634f;
  const int H = d.H, HQ = d.HQ, NG = HQ / H, N = d.N;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
  if (!chunk_gate(w, cg, h, H)) return;
  const int ci = rc.ci;
  const int t0 = rc.t0;
  const int len = rc.len;
  const int c0 = ci * kChunk;
  const int wl = seq_window(d, n);
  const int shift = seq_shift(d, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* As = (float*)(sm + L::oA);
  float* ER = (float*)(sm + L::oR);
  float* xch = (float*)(sm + L::oX);
  uint64_t* mbar = (uint64_t*)(sm + L::oBar);
  uint32_t* tslot = (uint32_t*)(sm + L::oBar + 16);

  // row of this thread: the warps w and w + 4 share a TMEM lane quarter and the rows in it
  const int quarter = warp & 3, half = warp >> 2;
  const bool active = R == 128 ? true : lane < 16;
  const int row = R == 128 ? quarter * 32 + lane : quarter * 16 + (lane & 15);
  const int tk = row & 63, th = row >> 6;
  const int pos = c0 + tk;
  const bool in_seq = pos < len;
  const bool live = active && in_seq;

  // gates and write weights through registers; their loads and the first head tile's row scalars go out
  // first, the tile copies follow
  const int lo = 0, hi = len - shift;
  constexpr int kGS = 512 / NT;
  uint4 sreg[kGS], greg[kGS];
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    const int src = c0 + r - shift;
    sreg[j] = make_uint4(0u, 0u, 0u, 0u);
    greg[j] = make_uint4(0u, 0u, 0u, 0u);
    if (src >= lo && src < hi) {
      greg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.g + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
      sreg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.s + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
    }
  }
  // per-row scalars: delta = <do, o> (each thread its half of the columns), joint LSE, lse_gsa, d_lse_gsa
  float delta = 0.f, Lj = 0.f, lse_g = 0.f, dlse = 0.f;
#define NHA_ROW_SCALARS(hq_)                                                                     \
  do {                                                                                           \
    delta = 0.f; Lj = 0.f; lse_g = 0.f; dlse = 0.f;                                              \
    if (live) {                                                                                  \
      const size_t rq_ = (size_t)(t0 + pos) * HQ + (hq_);                                        \
      const bf16* orow = (const bf16*)d.o + rq_ * D + (D / 2) * half;                            \
      const bf16* grow = (const bf16*)d.d_o + rq_ * D + (D / 2) * half;                          \
      uint4 ou[D / 16], gu[D / 16];                                                              \
      _Pragma("unroll") for (int c8 = 0; c8 < D / 16; ++c8) {                                    \
        ou[c8] = *reinterpret_cast<const uint4*>(orow + 8 * c8);                                 \
        gu[c8] = *reinterpret_cast<const uint4*>(grow + 8 * c8);                                 \
      }                                                                                          \
      const float ls_ = d.lse_swa[rq_];                                                          \
      lse_g = d.lse_gsa[rq_];                                                                    \
      dlse = d.d_lse_gsa ? d.d_lse_gsa[rq_] : 0.f;                                               \
      _Pragma("unroll") for (int c8 = 0; c8 < D / 16; ++c8) {                                    \
        float a8[8], b8[8];                                                                      \
        unpack8(ou[c8], a8);                                                                     \
        unpack8(gu[c8], b8);                                                                     \
        _Pragma("unroll") for (int e = 0; e < 8; ++e) delta += a8[e] * b8[e];                    \
      }                                                                                          \
      const float mx_ = fmaxf(ls_, lse_g);                                                       \
      Lj = mx_ + __logf(__expf(ls_ - mx_) + __expf(lse_g - mx_));                                \
    }                                                                                            \
  } while (0)
  uint4 ou0[D / 16], gu0[D / 16];
  float ls0 = 0.f;
  if (live) {
    const size_t rq = (size_t)(t0 + pos) * HQ + h * NG + th;
    const bf16* orow = (const bf16*)d.o + rq * D + (D / 2) * half;
    const bf16* grow = (const bf16*)d.d_o + rq * D + (D / 2) * half;
#pragma unroll
    for (int c8 = 0; c8 < D / 16; ++c8) {
      ou0[c8] = *reinterpret_cast<const uint4*>(orow + 8 * c8);
      gu0[c8] = *reinterpret_cast<const uint4*>(grow + 8 * c8);
    }
    ls0 = d.lse_swa[rq];
    lse_g = d.lse_gsa[rq];
    dlse = d.d_lse_gsa ? d.d_lse_gsa[rq] : 0.f;
  }
  load_sw<D, NT>(sm + L::tK, 8192, (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0 - shift, lo, hi, 64, 0, tid);
  load_sw<D, NT>(sm + L::tV, 8192, (const bf16*)d.v + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0 - shift, lo, hi, 64, 0, tid);
  load_sw<64, NT>(sm + L::tHk, 0, (const bf16*)d.hk_chunks + ((size_t)cg * H + h) * D * M, M, 0, 0, D, D, 0, tid);
  load_sw<D, NT>(sm + L::tHv, 8192, (const bf16*)d.hv_chunks + ((size_t)cg * H + h) * M * D, D, 0, 0, M, M, 0, tid);
#define NHA_LOAD_HEAD_TILE(ht_)                                                                                        \
  do {                                                                                                                 \
    const int hq0_ = h * NG + (ht_) * TH;                                                                              \
    _Pragma("unroll") for (int t2 = 0; t2 < TH; ++t2) {                                                                \
      load_sw<D, NT>(sm + L::tQ, L::kATile, (const bf16*)d.q_gsa + ((size_t)t0 * HQ + hq0_ + t2) * D,                  \
                     (int64_t)HQ * D, c0, 0, len, 64, 64 * t2, tid);                                                   \
      load_sw<D, NT>(sm + L::tQS, L::kATile, (const bf16*)d.q_swa + ((size_t)t0 * HQ + hq0_ + t2) * D,                 \
                     (int64_t)HQ * D, c0, 0, len, 64, 64 * t2, tid);                                                   \
      load_sw<D, NT>(sm + L::tDO, L::kATile, (const bf16*)d.d_o + ((size_t)t0 * HQ + hq0_ + t2) * D,                   \
                     (int64_t)HQ * D, c0, 0, len, 64, 64 * t2, tid);                                                   \
    }                                                                                                                  \
    cp_commit();                                                                                                       \
  } while (0)
  NHA_LOAD_HEAD_TILE(0);
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    float gv[8];
    unpack8(greg[j], gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) As[r * 65 + 8 * c8 + e] = gv[e];
  }
  if (live) {
#pragma unroll
    for (int c8 = 0; c8 < D / 16; ++c8) {
      float a8[8], b8[8];
      unpack8(ou0[c8], a8);
      unpack8(gu0[c8], b8);
#pragma unroll
      for (int e = 0; e < 8; ++e) delta += a8[e] * b8[e];
    }
    const float mx = fmaxf(ls0, lse_g);
    Lj = mx + __logf(__expf(ls0 - mx) + __expf(lse_g - mx));
  }
  if (tid == 0) mbar_init(mbar, 1);
  __syncthreads();
  // inclusive scan along the rows: four threads per column (16 rows each), then the earlier quarters' totals
  {
    const int m = tid & 63, seg = tid >> 6;
    float run = 0.f;
#pragma unroll
    for (int r = 16 * seg; r < 16 * seg + 16; ++r) {
      run += As[r * 65 + m];
      As[r * 65 + m] = run;
    }
    __syncthreads();
    float add = 0.f;
    for (int s2 = 0; s2 < seg; ++s2) add += As[(16 * s2 + 15) * 65 + m];
    __syncthreads();
    if (seg > 0) {
#pragma unroll
      for (int r = 16 * seg; r < 16 * seg + 16; ++r) As[r * 65 + m] += add;
    }
    __syncthreads();
  }
  if (tid < 64) w.gend[((size_t)cg * H + h) * M + tid] = As[63 * 65 + tid];
  // a = exp(G - R) replaces G in place; s' .* b = s' exp(R - G) goes into its swizzled tile
  float rref[8];
  {
    const int c8 = tid & 7;
#pragma unroll
    for (int e = 0; e < 8; ++e) rref[e] = 0.5f * As[63 * 65 + 8 * c8 + e];
  }
  __syncthreads();
  if (tid < 8) {
#pragma unroll
    for (int e = 0; e < 8; ++e) ER[8 * tid + e] = __expf(rref[e]);
  }
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    float sv[8], out[8];
    unpack8(sreg[j], sv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float x = As[r * 65 + 8 * c8 + e] - rref[e];
      As[r * 65 + 8 * c8 + e] = __expf(x);
      out[e] = sv[e] * __expf(-x);
    }
    *reinterpret_cast<uint4*>(sm + L::tSB + sw_off(r, c8)) = pack8(out);
  }
  if (warp == 0) tmem_alloc(tslot, L::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tslot;
  const uint32_t tlane = tbase + ((uint32_t)(quarter * 32) << 16);
  uint32_t phase = 0;
  bool failed = false;

  const int jt_hi = ci;
  const int jt_lo = wl < 0 ? 0 : max(0, c0 - wl) / kChunk;
  // visible keys of this row: klo <= key <= pos, tested as (unsigned)(key - klo) <= kspan
  const int klo = in_seq ? (wl < 0 ? 0 : max(0, pos - wl)) : (1 << 30);
  const unsigned kspan = in_seq ? (unsigned)(pos - klo) : 0u;
  const float sc2 = d.scale * kLog2e;
  const uint32_t aQ = smem_u32(sm + L::tQ), aQS = smem_u32(sm + L::tQS), aDO = smem_u32(sm + L::tDO);
  const uint32_t aK = smem_u32(sm + L::tK), aV = smem_u32(sm + L::tV), aHk = smem_u32(sm + L::tHk);
  const uint32_t aHv = smem_u32(sm + L::tHv), aSB = smem_u32(sm + L::tSB);
  const uint32_t aA = smem_u32(sm + L::bufA), aB = smem_u32(sm + L::bufB);
  const uint32_t aPG = smem_u32(sm + L::tPG);
  const bf16* ksw = (const bf16*)d.k_swa + ((size_t)t0 * H + h) * D;
  const bf16* vsw = (const bf16*)d.v + ((size_t)t0 * H + h) * D;

#define NHA_MMA_WAIT()                                   \
  do {                                                   \
    if (tid == 0) commit(mbar);                          \
    if (!failed && !mbar_wait(mbar, phase)) failed = true;          \
    phase ^= 1;                                          \
    tc_fence_after();                                    \
  } while (0)
#define NHA_SMEM_TO_MMA()                                \
  do {                                                   \
    fence_async_smem();                                  \
    tc_fence_before();                                   \
    __syncthreads();                                     \
    tc_fence_after();                                    \
  } while (0)
// this thread's half of tril of a [R][64] accumulator (row token tk keeps columns i <= tk) -> bf16 A-operand tile
#define NHA_TRIL_TO_SMEM(col0, dst_off)                                                          \
  do {                                                                                           \
    float tv_[32];                                                                               \
    tmem_ld32(tlane + (col0) + 32 * half, tv_);                                                  \
    if (active) {                                                                                \
      _Pragma("unroll") for (int c8 = 0; c8 < 4; ++c8) {                                         \
        float o8[8];                                                                             \
        _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                          \
          const int i_ = 32 * half + 8 * c8 + e;                                                 \
          o8[e] = i_ <= tk ? tv_[8 * c8 + e] : 0.f;                                              \
        }                                                                                        \
        *reinterpret_cast<uint4*>(sm + (dst_off) + sw_off(row, 4 * half + c8)) = pack8(o8);      \
      }                                                                                          \
    }                                                                                            \
  } while (0)

  for (int ht = 0; ht < NG / TH; ++ht) {
    const int hq0 = h * NG + ht * TH;
    const int hq = hq0 + th;
    const size_t rowq = (size_t)(t0 + pos) * HQ + hq;          // (token, query head) index of this thread's row
    if (ht > 0) {
      NHA_LOAD_HEAD_TILE(ht);
      NHA_ROW_SCALARS(hq);
    }
    xch[half * 128 + row] = delta;
    cp_wait_all();
    NHA_SMEM_TO_MMA();                                           // its barrier also publishes the partial deltas
    delta += xch[(half ^ 1) * 128 + row];
    if (live && half == 0) {
      w.delta[rowq] = delta;
      w.lj[rowq] = Lj;
    }
    // ---- A = q k'^T, Av = do v'^T, QH = q Hk, Y0 = do Hv^T ---------------------------------------------------
    if (tid == 0) {
      const MmaOp ops[4] = {
          {tbase + L::cA, aQ, aK, L::kATile, 8192, 0, 0, 64, D / 16, false},
          {tbase + L::cAv, aDO, aV, L::kATile, 8192, 0, 0, 64, D / 16, false},
          {tbase + L::cQH, aQ, aHk, L::kATile, 0, 0, 1, 64, D / 16, false},
          {tbase + L::cY, aDO, aHv, L::kATile, 8192, 0, 0, 64, D / 16, false}};   // Hv tiles as K-major [m][v]
      mma_interleaved(ops, R);
    }
    NHA_MMA_WAIT();
    NHA_TRIL_TO_SMEM(L::cA, L::bufA);
    NHA_TRIL_TO_SMEM(L::cAv, L::bufB);
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
      const MmaOp ops[2] = {{tbase + L::cA, aA, aSB, L::kATile, 0, 0, 1, 64, 4, false},      // X  = tril(A)  SB
                            {tbase + L::cAv, aB, aSB, L::kATile, 0, 0, 1, 64, 4, false}};    // X2 = tril(Av) SB
      mma_interleaved(ops, R);
    }
    NHA_MMA_WAIT();
    // ---- slot part of dz (this thread's 32 slots, 16 at a time); decayed bf16 copies; gate terms -------------------
    // (the MMAs that read bufA / bufB, v' and Hv have completed, so the tiles can take the copies now)
    {
      const float nLj = -Lj * kLog2e, nLg = -lse_g * kLog2e;
#pragma unroll
      for (int hh = 0; hh < 2; ++hh) {
        const int m0 = 32 * half + 16 * hh;
        float qh[16], xv[16], y0[16], x2[16];
        tmem_ld16(tlane + L::cQH + m0, qh);
        tmem_ld16(tlane + L::cA + m0, xv);
        tmem_ld16(tlane + L::cY + m0, y0);
        tmem_ld16(tlane + L::cAv + m0, x2);
        if (active) {
#pragma unroll
          for (int c8 = 0; c8 < 2; ++c8) {
            float zg8[8], za8[8], pg8[8], pa8[8], ga8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              const int m = m0 + 8 * c8 + e;
              const float aI = As[tk * 65 + m], er = ER[m];
              const float ok = d.scale * aI * (er * qh[8 * c8 + e] + xv[8 * c8 + e]);
              const float dps = aI * (er * y0[8 * c8 + e] + x2[8 * c8 + e]);
              float ps = 0.f, dz = 0.f;
              if (in_seq) {
                ps = exp2f(fmaf(ok, kLog2e, nLj));
                dz = ps * (dps - delta) + dlse * exp2f(fmaf(ok, kLog2e, nLg));
              }
              ga8[e] = ok * dz + ps * dps;
              za8[e] = d.scale * dz * aI;
              zg8[e] = za8[e] * er;
              pa8[e] = ps * aI;
              pg8[e] = pa8[e] * er;
            }
            const int ch = (m0 >> 3) + c8;                       // 16-byte chunk of the row
            if (in_seq) {
              float4* gdst = reinterpret_cast<float4*>(w.dga + ((size_t)(t0 + pos) * H + h) * M + 8 * ch);
              if (NG == 1) {                                     // one writer per element: plain stores
                gdst[0] = make_float4(ga8[0], ga8[1], ga8[2], ga8[3]);
                gdst[1] = make_float4(ga8[4], ga8[5], ga8[6], ga8[7]);
              } else {
                atomicAdd(gdst, make_float4(ga8[0], ga8[1], ga8[2], ga8[3]));
                atomicAdd(gdst + 1, make_float4(ga8[4], ga8[5], ga8[6], ga8[7]));
              }
            }
            const uint4 zg = pack8(zg8), za = pack8(za8), pg = pack8(pg8), pa = pack8(pa8);
            *reinterpret_cast<uint4*>(sm + L::bufB + sw_off(row, ch)) = zg;
            *reinterpret_cast<uint4*>(sm + L::bufA + sw_off(row, ch)) = za;
            if constexpr (L::kAlias) {
              *reinterpret_cast<uint4*>(sm + L::tPG + sw_off(row, ch)) = pg;
              *reinterpret_cast<uint4*>(sm + L::tPA + sw_off(row, ch)) = pa;
            } else if (in_seq) {
              const size_t gi = rowq * M + 8 * ch;
              *reinterpret_cast<uint4*>(w.dza + gi) = za;
              *reinterpret_cast<uint4*>(w.pgq + gi) = pg;
              *reinterpret_cast<uint4*>(w.paq + gi) = pa;
            }
          }
        }
      }
    }
    NHA_SMEM_TO_MMA();
    if (tid == 0) mma_tile(tbase + L::cA, aA, L::kATile, aSB, 0, R, 64, 4, 0, false);  // E = (scale dz a) SB^T
    if constexpr (L::kAlias) {
      // while E runs: the two bf16 copies the columns pass reads (scale dz a, p a) leave through coalesced
      // 128-byte rows; the copies decayed by exp(G) are used inside this CTA only
      const bf16* tiles[2] = {(const bf16*)(sm + L::bufA), (const bf16*)(sm + L::tPA)};
      bf16* dsts[2] = {w.dza, w.paq};
#pragma unroll
      for (int t4 = 0; t4 < 2; ++t4) {
#pragma unroll
        for (int j = 0; j < 512 / NT; ++j) {
          const int i = tid + NT * j;
          const int r = i >> 3, c = i & 7;
          const uint4 v4 = *reinterpret_cast<const uint4*>((const unsigned char*)tiles[t4] + sw_off(r, c));
          if (c0 + r < len)
            *reinterpret_cast<uint4*>(dsts[t4] + ((size_t)(t0 + c0 + r) * HQ + hq0) * M + 8 * c) = v4;
        }
      }
      __syncthreads();                                          // bufA is read out before tril(E) replaces it
    }
    NHA_MMA_WAIT();
    NHA_TRIL_TO_SMEM(L::cA, L::bufA);
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
#pragma unroll
      for (int nb = 0; nb < KT; ++nb) {
        // dq_gsa columns [64 nb, 64 nb + 64): (scale dz exp G) Hk^T (Hk rows kk as K-major N rows) + tril(E) k'
        mma_tile(tbase + L::cDQ + 64 * nb, aB, L::kATile, aHk + nb * 8192, 0, R, 64, 4, 0, false);
        mma_tile(tbase + L::cDQ + 64 * nb, aA, L::kATile, aK + nb * 8192, 0, R, 64, 4, 1, true);
      }
    }
    NHA_MMA_WAIT();
    // ---- the chunk's own contribution to the state gradients: q^T (scale dz exp G) and (p exp G)^T do -------------
    const int ntile = jt_hi - jt_lo + 1;
    uint32_t aLP = aPG;
    if constexpr (L::kAlias) {
      // k' and Hk are dead: the first window tile goes in flight behind the local terms
      load_sw<D, NT>(sm + L::tW0, 8192, ksw, (int64_t)H * D, jt_lo * kChunk, 0, len, 64, 0, tid);
      load_sw<D, NT>(sm + L::tWV0, 8192, vsw, (int64_t)H * D, jt_lo * kChunk, 0, len, 64, 0, tid);
      cp_commit();
    } else {
      // (p exp G) comes back from the scratch this CTA just wrote; bufA (tril(E)) is free again
      tc_fence_before();
      __syncthreads();
#pragma unroll
      for (int t2 = 0; t2 < TH; ++t2)
        load_sw<64, NT>(sm + L::bufA, 0, w.pgq + ((size_t)t0 * HQ + hq0 + t2) * M, (int64_t)HQ * M, c0, 0, len, 64, 64 * t2,
                        tid);
      cp_commit();
      cp_wait_all();
      NHA_SMEM_TO_MMA();
      aLP = aA;
    }
    if (tid == 0) {
#pragma unroll
      for (int nb = 0; nb < KT; ++nb) {
        mma_tile_ex(tbase + L::cLK + 64 * nb, aQ + nb * L::kATile, 0, 1, aB, 0, 1, 64, 64, R / 16, false);
        mma_tile_ex(tbase + L::cLV + 64 * nb, aLP, 0, 1, aDO + nb * L::kATile, 0, 1, 64, 64, R / 16, false);
      }
    }
    NHA_MMA_WAIT();
    if constexpr (L::kAlias) {
      if (ntile > 1) {
        // q_gsa is dead: the second window tile goes in flight behind the read-out of the local terms
        load_sw<D, NT>(sm + L::tW1, 8192, ksw, (int64_t)H * D, (jt_lo + 1) * kChunk, 0, len, 64, 0, tid);
        load_sw<D, NT>(sm + L::tWV1, 8192, vsw, (int64_t)H * D, (jt_lo + 1) * kChunk, 0, len, 64, 0, tid);
        cp_commit();
      }
    }
    {
      // 64-row products: rows in the first 16 lanes of each quarter; this thread's half of the columns
      const bool kact = lane < 16;
      const int krow = quarter * 16 + (lane & 15);
      float lv[32];
#pragma unroll
      for (int nb = 0; nb < KT; ++nb) {
        tmem_ld32(tlane + L::cLK + 64 * nb + 32 * half, lv);
        if (kact) {
          float* dst = w.dkc + (((size_t)cg * H + h) * D + 64 * nb + krow) * M + 32 * half;
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            float4 v4 = make_float4(lv[e], lv[e + 1], lv[e + 2], lv[e + 3]);
            if (ht > 0) {
              const float4 o4 = *reinterpret_cast<const float4*>(dst + e);
              v4.x += o4.x; v4.y += o4.y; v4.z += o4.z; v4.w += o4.w;
            }
            *reinterpret_cast<float4*>(dst + e) = v4;
          }
        }
        tmem_ld32(tlane + L::cLV + 64 * nb + 32 * half, lv);
        if (kact) {
          float* dst = w.dvc + (((size_t)cg * H + h) * M + krow) * D + 64 * nb + 32 * half;
#pragma unroll
          for (int e = 0; e < 32; e += 4) {
            float4 v4 = make_float4(lv[e], lv[e + 1], lv[e + 2], lv[e + 3]);
            if (ht > 0) {
              const float4 o4 = *reinterpret_cast<const float4*>(dst + e);
              v4.x += o4.x; v4.y += o4.y; v4.z += o4.z; v4.w += o4.w;
            }
            *reinterpret_cast<float4*>(dst + e) = v4;
          }
        }
      }
    }
    // ---- window part: dz_win tile by tile, dq_swa --------------------------------------------------------------------
    const float nLjw = -Lj * kLog2e;
    for (int jt = jt_lo; jt <= jt_hi; ++jt) {
      const int wi = jt - jt_lo;
      const int set = L::kAlias ? (wi & 1) : 0;
      const uint32_t aW = smem_u32(sm + (set ? L::tW1 : L::tW0)), aWV = smem_u32(sm + (set ? L::tWV1 : L::tWV0));
      tc_fence_before();
      if constexpr (L::kAlias) {
        // tiles wi and (when it exists) wi + 1 are in flight; groups complete in order
        if (wi + 1 < ntile) cp_wait_but_one(); else cp_wait_all();
      } else {
        __syncthreads();
        load_sw<D, NT>(sm + L::tW0, 8192, ksw, (int64_t)H * D, jt * kChunk, 0, len, 64, 0, tid);
        load_sw<D, NT>(sm + L::tWV0, 8192, vsw, (int64_t)H * D, jt * kChunk, 0, len, 64, 0, tid);
        cp_commit();
        cp_wait_all();
      }
      NHA_SMEM_TO_MMA();
      if (tid == 0) {
        const MmaOp ops[2] = {{tbase + L::cS, aQS, aW, L::kATile, 8192, 0, 0, 64, D / 16, false},     // S  = q_swa k^T
                              {tbase + L::cDP, aDO, aWV, L::kATile, 8192, 0, 0, 64, D / 16, false}};  // dP = do v^T
        mma_interleaved(ops, R);
      }
      NHA_MMA_WAIT();
      {
        float sv[32], dp[32];
        tmem_ld32(tlane + L::cS + 32 * half, sv);
        tmem_ld32(tlane + L::cDP + 32 * half, dp);
        if (active) {
          const int off = jt * kChunk + 32 * half - klo;
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) {
            float o8[8];
#pragma unroll
            for (int e = 0; e < 8; ++e)
              o8[e] = (unsigned)(off + 8 * c8 + e) <= kspan
                          ? exp2f(fmaf(sv[8 * c8 + e], sc2, nLjw)) * (dp[8 * c8 + e] - delta) * d.scale : 0.f;
            *reinterpret_cast<uint4*>(sm + L::bufA + sw_off(row, 4 * half + c8)) = pack8(o8);
          }
        }
      }
      NHA_SMEM_TO_MMA();
      if (tid == 0) {
#pragma unroll
        for (int nb = 0; nb < KT; ++nb)                     // dq_swa += dz_win k_swa (keys as the k dimension)
          mma_tile(tbase + L::cDQS + 64 * nb, aA, L::kATile, aW + nb * 8192, 0, R, 64, 4, 1, jt > jt_lo);
      }
      NHA_MMA_WAIT();
      if constexpr (L::kAlias) {
        if (wi + 2 < ntile) {
          // this tile's buffers are free again (every product that read them has completed): tile wi + 2 goes in flight
          load_sw<D, NT>(sm + (set ? L::tW1 : L::tW0), 8192, ksw, (int64_t)H * D, (jt + 2) * kChunk, 0, len, 64, 0, tid);
          load_sw<D, NT>(sm + (set ? L::tWV1 : L::tWV0), 8192, vsw, (int64_t)H * D, (jt + 2) * kChunk, 0, len, 64, 0, tid);
          cp_commit();
        }
      }
    }
    // ---- dq rows out: this thread's half of the columns --------------------------------------------------------------------
    {
      float ov[32];
#pragma unroll
      for (int pp = 0; pp < D / 64; ++pp) {
        const int part = (D / 64) * half + pp;
        tmem_ld32(tlane + L::cDQ + 32 * part, ov);
        if (live) {
          bf16* orow = (bf16*)d.dq_gsa + rowq * D + 32 * part;
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) *reinterpret_cast<uint4*>(orow + 8 * c8) = pack8(ov + 8 * c8);
        }
        tmem_ld32(tlane + L::cDQS + 32 * part, ov);
        if (live) {
          bf16* orow = (bf16*)d.dq_swa + rowq * D + 32 * part;
#pragma unroll
          for (int c8 = 0; c8 < 4; ++c8) *reinterpret_cast<uint4*>(orow + 8 * c8) = pack8(ov + 8 * c8);
        }
      }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
#undef NHA_LOAD_HEAD_TILE
#undef NHA_ROW_SCALARS
  if (failed) atomicExch(err, 1);
  cp_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, L::kTmemCols);
}
#undef NHA_MMA_WAIT
#undef NHA_SMEM_TO_MMA
#undef NHA_TRIL_TO_SMEM

// ================================================================================================
// gate-gradient carry and bf16 copies of the state gradients (between the scan and the columns pass)
// ================================================================================================
// For chunk c the gate gradient of every later chunk enters as one number per slot,
//     carry[m] = <DK_end[:, m], hk_next[:, m]> + <DV_end[m, :], hv_next[m, :]>,
// with the states at the end of chunk c (the next chunk's start state; the fp32 final state for the
// last chunk of a sequence).  The same sweep over DK_end / DV_end stores the bf16 operand copies the
// columns pass multiplies with.  One CTA per (chunk, kv head); M == 64.
constexpr int kCarryThreads = 256;
__global__ void __launch_bounds__(kCarryThreads) nha_bwd_gate_carry_kernel(const nha_chunk_desc d, const BwdWs w) {
  constexpr int M = 64;
  const int H = d.H, N = d.N, K = d.K, V = d.V;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
  if (!chunk_gate(w, cg, h, H)) return;
  const int ci = rc.ci;
  const int len = rc.len;
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int tid = threadIdx.x, lane = tid & 31;
  const size_t nh = (size_t)n * H + h, ch = (size_t)cg * H + h;
  // per-warp partial sums, added in a fixed order afterwards (no floating-point atomics: the result must not
  // depend on the order in which warps arrive)
  constexpr int kCW = kCarryThreads / 32;
  __shared__ float part_k[kCW][M];
  __shared__ float part_v[kCarryThreads / 32][M];
  const int warp = tid >> 5;
  for (int i = tid; i < kCW * M; i += kCarryThreads) (&part_v[0][0])[i] = 0.f;
  __syncthreads();
  const bool last = ci >= nchunks - 1;
  const bool have_next = !last || (d.d_hkt && d.hkt && d.hvt);
  const float* dkg = w.dkc + ch * K * M;
  const float* dvg = w.dvc + ch * M * V;
  bf16* dkb = w.dkb + ch * K * M;
  bf16* dvb = w.dvb + ch * M * V;
  const bf16* hkn = (const bf16*)d.hk_chunks + ((size_t)(cg + 1) * H + h) * K * M;
  const bf16* hvn = (const bf16*)d.hv_chunks + ((size_t)(cg + 1) * H + h) * M * V;
  const float* hkf = d.hkt ? d.hkt + nh * K * M : nullptr;
  const float* hvf = d.hvt ? d.hvt + nh * M * V : nullptr;
  // DK [K][64]: a thread always owns the same four slots
  float ck[4] = {0.f, 0.f, 0.f, 0.f};
  for (int i = tid; i < K * (M / 4); i += kCarryThreads) {
    const float4 f = *reinterpret_cast<const float4*>(dkg + 4 * (size_t)i);
    float4 nx = make_float4(0.f, 0.f, 0.f, 0.f);
    if (have_next) {
      if (!last) {
        const uint2 u = *reinterpret_cast<const uint2*>(hkn + 4 * (size_t)i);
        const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        nx = make_float4(lo2.x, lo2.y, hi2.x, hi2.y);
      } else {
        nx = *reinterpret_cast<const float4*>(hkf + 4 * (size_t)i);
      }
    }
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(f.x, f.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(f.z, f.w);
    *reinterpret_cast<uint2*>(dkb + 4 * (size_t)i) = o;
    ck[0] += f.x * nx.x; ck[1] += f.y * nx.y; ck[2] += f.z * nx.z; ck[3] += f.w * nx.w;
  }
#pragma unroll
  for (int e = 0; e < 4; ++e) ck[e] += __shfl_xor_sync(0xffffffffu, ck[e], 16);
  if (lane < 16) {
#pragma unroll
    for (int e = 0; e < 4; ++e) part_k[warp][4 * lane + e] = ck[e];
  }
  // DV [64][V]: a slot's row is spread over V/4 neighbouring lanes
  const int C4 = V / 4;
  for (int i = tid; i < M * C4; i += kCarryThreads) {
    const int r = i / C4, c = i - r * C4;
    const float4 f = *reinterpret_cast<const float4*>(dvg + 4 * (size_t)i);
    float4 nx = make_float4(0.f, 0.f, 0.f, 0.f);
    if (have_next) {
      if (!last) {
        const uint2 u = *reinterpret_cast<const uint2*>(hvn + 4 * (size_t)i);
        const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.x));
        const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&u.y));
        nx = make_float4(lo2.x, lo2.y, hi2.x, hi2.y);
      } else {
        nx = *reinterpret_cast<const float4*>(hvf + 4 * (size_t)i);
      }
    }
    uint2 o;
    *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(f.x, f.y);
    *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(f.z, f.w);
    *reinterpret_cast<uint2*>(dvb + 4 * (size_t)i) = o;
    float acc = f.x * nx.x + f.y * nx.y + f.z * nx.z + f.w * nx.w;
    for (int o2 = 1; o2 < C4 && o2 < 32; o2 <<= 1) acc += __shfl_xor_sync(0xffffffffu, acc, o2);
    if (c == 0) part_v[warp][r] = acc;                 // one writer per (warp, slot): row r belongs to one warp only
  }
  __syncthreads();
  if (tid < M) {
    float sum = 0.f;
#pragma unroll
    for (int w8 = 0; w8 < kCW; ++w8) sum += part_k[w8][tid];
#pragma unroll
    for (int w8 = 0; w8 < kCW; ++w8) sum += part_v[w8][tid];
    w.gcarry[ch * M + tid] = sum;
  }
}

// ================================================================================================
// columns pass
// ================================================================================================
#define NHA_MMA_WAIT()                                   \
  do {                                                   \
    if (tid == 0) commit(mbar);                          \
    if (!failed && !mbar_wait(mbar, phase)) failed = true;          \
    phase ^= 1;                                          \
    tc_fence_after();                                    \
  } while (0)
#define NHA_SMEM_TO_MMA()                                \
  do {                                                   \
    fence_async_smem();                                  \
    tc_fence_before();                                   \
    __syncthreads();                                     \
    tc_fence_after();                                    \
  } while (0)
// this thread's half of tril of a [R][64] accumulator (row token tk keeps columns i <= tk) -> bf16 A-operand tile
#define NHA_TRIL_TO_SMEM(col0, dst_off)                                                          \
  do {                                                                                           \
    float tv_[32];                                                                               \
    tmem_ld32(tlane + (col0) + 32 * half, tv_);                                                  \
    if (active) {                                                                                \
      _Pragma("unroll") for (int c8 = 0; c8 < 4; ++c8) {                                         \
        float o8[8];                                                                             \
        _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                          \
          const int i_ = 32 * half + 8 * c8 + e;                                                 \
          o8[e] = i_ <= tk ? tv_[8 * c8 + e] : 0.f;                                              \
        }                                                                                        \
        *reinterpret_cast<uint4*>(sm + (dst_off) + sw_off(row, 4 * half + c8)) = pack8(o8);      \
      }                                                                                          \
    }                                                                                            \
  } while (0)

template <int D, int R>
struct ColsLayout {
  static constexpr int KT = D / 64;
  static constexpr int kATile = R * 128;
  // per-head tiles and the tril buffers first: together they are dead once the head loop is over and
  // then hold the staged epilogue inputs (gate terms, window dv, s') and the dg scan
  static constexpr int tQ = 0;                          // q_gsa [R][D]
  static constexpr int tDO = tQ + KT * kATile;          // do [R][D]
  static constexpr int tZA = tDO + KT * kATile;         // scale dz a [R][64]
  static constexpr int tPA = tZA + kATile;              // p a [R][64]
  static constexpr int bufA = tPA + kATile;             // tril(A) -> tril(E)
  static constexpr int bufB = bufA + kATile;            // tril(Av) -> tril(Bv)
  static constexpr int tK = bufB + kATile;              // k' [64][D]
  static constexpr int tV = tK + KT * 8192;             // v' [64][D]
  static constexpr int tSB = tV + KT * 8192;            // s' b, after the head loop s' exp(Gend - G)
  static constexpr int tDK = tSB + 8192;                // DK at the chunk end [D][64]
  static constexpr int tDV = tDK + D * 128;             // DV at the chunk end [64][D]
  static constexpr int oG = tDV + KT * 8192;
  static constexpr int oR = oG + 64 * 65 * 4;           // [64] reference, [64] carry
  static constexpr int oBar = oR + 512;
  static constexpr int total = oBar + 64 + 1024;
  // staged epilogue inputs, fp32 rows padded to 16-byte multiples that spread over the banks
  static constexpr int kLdG = 68, kLdV = D + 4, kLdS = 72;
  static constexpr int eG = 0;                          // [64][68] fp32 dgA, then dgraw and its scan
  static constexpr int eV = eG + 64 * kLdG * 4;         // [64][D+4] fp32 window part of dv
  static constexpr int eS = eV + 64 * kLdV * 4;         // [64][72] bf16 s'
  static_assert(eS + 64 * kLdS * 2 <= tK, "the staged epilogue inputs must fit in the per-head tiles");
  // D == 64 with one query head per kv head: 256 columns, so two CTAs share an SM; the intra-chunk ds'
  // accumulator then borrows the dk' columns for one MMA group and waits in registers
  static constexpr bool kDsInRegs = D == 64 && R == 64;
  static constexpr int kTmemCols = kDsInRegs ? 256 : 512;
  static constexpr int cA = 0, cAv = 64, cDK = 128, cDV = 128 + D, cDS = kDsInRegs ? cDK : 128 + 2 * D, cDS2 = cA;
};

// Two threads per row, as in the rows pass: the warps w and w + 4 share a TMEM lane quarter and take
// alternate 32-column halves of every 64-column accumulator.
template <int D, int R>
__global__ void __launch_bounds__(kColsThreads, (D == 64 && R == 64) ? 2 : 1)
    nha_bwd_cols_umma_kernel(const nha_chunk_desc d, const BwdWs w, int* __restrict__ err) {
  typedef ColsLayout<D, R> L;
  constexpr int KT = L::KT, TH = R / 64, M = 64, NT = kColsThreads;
  const int H = d.H, HQ = d.HQ, NG = HQ / H, N = d.N;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
  if (!chunk_gate(w, cg, h, H)) return;
  const int ci = rc.ci;
  const int t0 = rc.t0;
  const int len = rc.len;
  const int c0 = ci * kChunk;
  const int shift = seq_shift(d, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const size_t ch = (size_t)cg * H + h;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* Bs = (float*)(sm + L::oG);                   // cumulative gates, then b = exp(R - G)
  float* ER = (float*)(sm + L::oR);                   // exp(R)
  float* cgv = ER + 64;
  uint64_t* mbar = (uint64_t*)(sm + L::oBar);
  uint32_t* tslot = (uint32_t*)(sm + L::oBar + 16);

  // ---- gate / write-weight loads first, then everything the first head tile needs goes in flight at once -------
  const int lo = 0, hi = len - shift;
  constexpr int kGS = 512 / NT;
  uint4 sreg[kGS], greg[kGS];
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    const int src = c0 + r - shift;
    sreg[j] = make_uint4(0u, 0u, 0u, 0u);
    greg[j] = make_uint4(0u, 0u, 0u, 0u);
    if (src >= lo && src < hi) {
      greg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.g + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
      sreg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.s + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
    }
  }
  float carry_in = 0.f;
  if (tid < 64) carry_in = w.gcarry[ch * M + tid];
  load_sw<D, NT>(sm + L::tK, 8192, (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0 - shift, lo, hi, 64, 0, tid);
  load_sw<D, NT>(sm + L::tV, 8192, (const bf16*)d.v + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0 - shift, lo, hi, 64, 0, tid);
  load_sw<64, NT>(sm + L::tDK, 0, w.dkb + ch * D * M, M, 0, 0, D, D, 0, tid);
  load_sw<D, NT>(sm + L::tDV, 8192, w.dvb + ch * M * D, D, 0, 0, M, M, 0, tid);
#define NHA_LOAD_HEAD_TILE(ht_)                                                                                      \
  do {                                                                                                               \
    const int hq0_ = h * NG + (ht_) * TH;                                                                            \
    _Pragma("unroll") for (int t2 = 0; t2 < TH; ++t2) {                                                              \
      load_sw<D, NT>(sm + L::tQ, L::kATile, (const bf16*)d.q_gsa + ((size_t)t0 * HQ + hq0_ + t2) * D,                \
                     (int64_t)HQ * D, c0, 0, len, 64, 64 * t2, tid);                                                 \
      load_sw<D, NT>(sm + L::tDO, L::kATile, (const bf16*)d.d_o + ((size_t)t0 * HQ + hq0_ + t2) * D,                 \
                     (int64_t)HQ * D, c0, 0, len, 64, 64 * t2, tid);                                                 \
      load_sw<64, NT>(sm + L::tZA, 0, w.dza + ((size_t)t0 * HQ + hq0_ + t2) * M, (int64_t)HQ * M, c0, 0, len, 64,    \
                      64 * t2, tid);                                                                                 \
      load_sw<64, NT>(sm + L::tPA, 0, w.paq + ((size_t)t0 * HQ + hq0_ + t2) * M, (int64_t)HQ * M, c0, 0, len, 64,    \
                      64 * t2, tid);                                                                                 \
    }                                                                                                                \
    cp_commit();                                                                                                     \
  } while (0)
  NHA_LOAD_HEAD_TILE(0);
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    float gv[8];
    unpack8(greg[j], gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) Bs[r * 65 + 8 * c8 + e] = gv[e];
  }
  if (tid < 64) cgv[tid] = carry_in;
  if (tid == 0) mbar_init(mbar, 1);
  __syncthreads();
  // inclusive scan along the rows: four threads per column (16 rows each), then the earlier quarters' totals
  {
    const int m = tid & 63, seg = tid >> 6;
    float run = 0.f;
#pragma unroll
    for (int r = 16 * seg; r < 16 * seg + 16; ++r) {
      run += Bs[r * 65 + m];
      Bs[r * 65 + m] = run;
    }
    __syncthreads();
    float add = 0.f;
    for (int s2 = 0; s2 < seg; ++s2) add += Bs[(16 * s2 + 15) * 65 + m];
    __syncthreads();
    if (seg > 0) {
#pragma unroll
      for (int r = 16 * seg; r < 16 * seg + 16; ++r) Bs[r * 65 + m] += add;
    }
    __syncthreads();
  }
  // b = exp(R - G) replaces G in place; s' .* b goes into its swizzled tile (s' .* b .* exp(R) = s' exp(Gend - G)
  // follows after the head loop)
  float rref[8];
  {
    const int c8 = tid & 7;
#pragma unroll
    for (int e = 0; e < 8; ++e) rref[e] = 0.5f * Bs[63 * 65 + 8 * c8 + e];
  }
  __syncthreads();
  if (tid < 8) {
#pragma unroll
    for (int e = 0; e < 8; ++e) ER[8 * tid + e] = __expf(rref[e]);
  }
  uint4 sbe[kGS];                                      // s' exp(Gend - G), written after the head loop
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    float sv[8], o1[8], o2[8];
    unpack8(sreg[j], sv);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float b = __expf(rref[e] - Bs[r * 65 + 8 * c8 + e]);
      Bs[r * 65 + 8 * c8 + e] = b;
      o1[e] = sv[e] * b;
      o2[e] = o1[e] * __expf(rref[e]);
    }
    *reinterpret_cast<uint4*>(sm + L::tSB + sw_off(r, c8)) = pack8(o1);
    sbe[j] = pack8(o2);
  }
  if (warp == 0) tmem_alloc(tslot, L::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tslot;
  const int quarter = warp & 3, half = warp >> 2;
  const uint32_t tlane = tbase + ((uint32_t)(quarter * 32) << 16);
  uint32_t phase = 0;
  bool failed = false;

  // rows of the R-row products (query rows) and of the 64-row products (key rows)
  const bool active = R == 128 ? true : lane < 16;
  const int row = R == 128 ? quarter * 32 + lane : quarter * 16 + (lane & 15);
  const int tk = row & 63;
  const bool kactive = lane < 16;
  const int krow = quarter * 16 + (lane & 15);
  const uint32_t aQ = smem_u32(sm + L::tQ), aDO = smem_u32(sm + L::tDO), aZA = smem_u32(sm + L::tZA);
  const uint32_t aPA = smem_u32(sm + L::tPA), aK = smem_u32(sm + L::tK), aV = smem_u32(sm + L::tV);
  const uint32_t aSB = smem_u32(sm + L::tSB), aDK = smem_u32(sm + L::tDK);
  const uint32_t aDV = smem_u32(sm + L::tDV), aA = smem_u32(sm + L::bufA), aB = smem_u32(sm + L::bufB);
  float dsk[L::kDsInRegs ? 32 : 1];                   // this thread's half of the intra-chunk ds' accumulator

  for (int ht = 0; ht < NG / TH; ++ht) {
    if (ht > 0) NHA_LOAD_HEAD_TILE(ht);
    cp_wait_all();
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
      mma_tile(tbase + L::cA, aQ, L::kATile, aK, 8192, R, 64, D / 16, 0, false);         // A  = q k'^T
      mma_tile(tbase + L::cAv, aDO, L::kATile, aV, 8192, R, 64, D / 16, 0, false);       // Av = do v'^T
    }
    NHA_MMA_WAIT();
    NHA_TRIL_TO_SMEM(L::cA, L::bufA);
    NHA_TRIL_TO_SMEM(L::cAv, L::bufB);
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
      // ds' (intra) += tril(A)^T dza + tril(Av)^T pa      (both operands MN-major, k = query row)
      mma_tile_ex(tbase + L::cDS, aA, 0, 1, aZA, 0, 1, 64, 64, R / 16, ht > 0);
      mma_tile_ex(tbase + L::cDS, aB, 0, 1, aPA, 0, 1, 64, 64, R / 16, true);
      mma_tile(tbase + L::cA, aZA, L::kATile, aSB, 0, R, 64, 4, 0, false);                // E  = dza SB^T
      mma_tile(tbase + L::cAv, aPA, L::kATile, aSB, 0, R, 64, 4, 0, false);               // Bv = pa SB^T
    }
    NHA_MMA_WAIT();
    if constexpr (L::kDsInRegs) tmem_ld32(tlane + L::cDS + 32 * half, dsk);
    NHA_TRIL_TO_SMEM(L::cA, L::bufA);
    NHA_TRIL_TO_SMEM(L::cAv, L::bufB);
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
#pragma unroll
      for (int nb = 0; nb < KT; ++nb) {
        // dk' += tril(E)^T q,  dv' += tril(Bv)^T do      (64 output columns at a time)
        mma_tile_ex(tbase + L::cDK + 64 * nb, aA, 0, 1, aQ + nb * L::kATile, 0, 1, 64, 64, R / 16, ht > 0);
        mma_tile_ex(tbase + L::cDV + 64 * nb, aB, 0, 1, aDO + nb * L::kATile, 0, 1, 64, 64, R / 16, ht > 0);
      }
    }
    NHA_MMA_WAIT();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
#undef NHA_LOAD_HEAD_TILE
  // ---- inter-chunk parts from the state gradients at the chunk end ------------------------------------------
  // The per-head tiles are dead now: the rows the epilogue needs from global memory (gate terms of the
  // rows pass, window part of dv, s') are fetched into their place while the last products run.
  const int kp = c0 + krow, kj = kp - shift;                     // this thread's key row: shifted position, source token
  const bool keep = kactive && kj >= 0 && kp < len;
  float* eG = (float*)(sm + L::eG);
  float* eV = (float*)(sm + L::eV);
  bf16* eS = (bf16*)(sm + L::eS);
  {
    const float* gsrc = w.dga + ((size_t)t0 * H + h) * M;
    for (int i = tid; i < 64 * 16; i += NT) {
      const int r = i >> 4, c = i & 15;
      const int p = c0 + r;
      const bool ok = p - shift >= 0 && p < len;
      cp16(eG + r * L::kLdG + 4 * c, gsrc + (size_t)(ok ? p : 0) * H * M + 4 * c, ok);
    }
    const float* vsrc = w.dvacc + ((size_t)t0 * H + h) * D;
    for (int i = tid; i < 64 * (D / 4); i += NT) {
      const int r = i / (D / 4), c = i % (D / 4);
      const int p = c0 + r, j = p - shift;
      const bool ok = j >= 0 && p < len;
      cp16(eV + r * L::kLdV + 4 * c, vsrc + (size_t)(ok ? j : 0) * H * D + 4 * c, ok);
    }
    const bf16* ssrc = (const bf16*)d.s + ((size_t)t0 * H + h) * M;
    for (int i = tid; i < 64 * 8; i += NT) {
      const int r = i >> 3, c = i & 7;
      const int p = c0 + r, j = p - shift;
      const bool ok = j >= 0 && p < len;
      cp16(eS + r * L::kLdS + 8 * c, ssrc + (size_t)(ok ? j : 0) * H * M + 8 * c, ok);
    }
    cp_commit();
  }
  // s' exp(Gend - G) replaces s' b (every product that read it has completed)
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + NT * j;
    const int r = i >> 3, c8 = i & 7;
    *reinterpret_cast<uint4*>(sm + L::tSB + sw_off(r, c8)) = sbe[j];
  }
  NHA_SMEM_TO_MMA();
  if (!failed) {
    if (tid == 0) {
#pragma unroll
      for (int nb = 0; nb < KT; ++nb) {
        // dk' += sbe DK^T (DK rows kk as the N rows of a K-major operand), dv' += sbe DV (DV as MN-major, k = slot)
        mma_tile(tbase + L::cDK + 64 * nb, aSB, 0, aDK + nb * 8192, 0, 64, 64, 4, 0, true);
        mma_tile(tbase + L::cDV + 64 * nb, aSB, 0, aDV + nb * 8192, 0, 64, 64, 4, 1, true);
      }
      // DS2 = k' DK + v' DV^T
      mma_tile(tbase + L::cDS2, aK, 8192, aDK, 0, 64, 64, D / 16, 1, false);
      mma_tile(tbase + L::cDS2, aV, 8192, aDV, 8192, 64, 64, D / 16, 0, true);
    }
    NHA_MMA_WAIT();
  }
  cp_wait_all();
  __syncthreads();
  // ---- epilogue: two threads per key row, each its half of the columns ----------------------------------------------
  {
    float dsi[32], ds2[32];
    if constexpr (L::kDsInRegs) {
#pragma unroll
      for (int e = 0; e < 32; ++e) dsi[e] = dsk[e];
    } else {
      tmem_ld32(tlane + L::cDS + 32 * half, dsi);
    }
    tmem_ld32(tlane + L::cDS2 + 32 * half, ds2);
    if (kactive) {
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        const int m0 = 32 * half + 8 * c8;
        float ds8[8], sv[8];
        unpack8(*reinterpret_cast<const uint4*>(eS + krow * L::kLdS + m0), sv);
        float* grow = eG + krow * L::kLdG + m0;
        const float4 g0 = *reinterpret_cast<const float4*>(grow), g1 = *reinterpret_cast<const float4*>(grow + 4);
        const float ga[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
        float gr[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int m = m0 + e;
          // ds' = b .* (intra-chunk part) + exp(Gend - G) .* (inter-chunk part), exp(Gend - G) = b exp(R)
          const float ds = Bs[krow * 65 + m] * (dsi[8 * c8 + e] + ER[m] * ds2[8 * c8 + e]);
          ds8[e] = ds;
          gr[e] = keep ? ga[e] - sv[e] * ds : 0.f;
        }
        *reinterpret_cast<float4*>(grow) = make_float4(gr[0], gr[1], gr[2], gr[3]);
        *reinterpret_cast<float4*>(grow + 4) = make_float4(gr[4], gr[5], gr[6], gr[7]);
        if (keep) *reinterpret_cast<uint4*>((bf16*)d.ds + ((size_t)(t0 + kj) * H + h) * M + m0) = pack8(ds8);
      }
    }
    float ov[32];
#pragma unroll
    for (int pp = 0; pp < D / 64; ++pp) {
      const int part = (D / 64) * half + pp;
      tmem_ld32(tlane + L::cDK + 32 * part, ov);
      if (keep) {
        bf16* orow = (bf16*)d.dk_gsa + ((size_t)(t0 + kj) * H + h) * D + 32 * part;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) *reinterpret_cast<uint4*>(orow + 8 * c8) = pack8(ov + 8 * c8);
      }
      tmem_ld32(tlane + L::cDV + 32 * part, ov);
      if (keep) {
        const float* wa = eV + krow * L::kLdV + 32 * part;
#pragma unroll
        for (int e = 0; e < 32; e += 4) {
          const float4 a4 = *reinterpret_cast<const float4*>(wa + e);
          ov[e] += a4.x; ov[e + 1] += a4.y; ov[e + 2] += a4.z; ov[e + 3] += a4.w;
        }
        bf16* orow = (bf16*)d.dv + ((size_t)(t0 + kj) * H + h) * D + 32 * part;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) *reinterpret_cast<uint4*>(orow + 8 * c8) = pack8(ov + 8 * c8);
      }
    }
  }
  // the accumulators are drained: release the tensor memory before the tail of the epilogue
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, L::kTmemCols);
  // reverse cumulative sum of dgraw along the rows (four threads per column), plus the carry
  {
    const int m = tid & 63, seg = tid >> 6;
    float run = 0.f;
#pragma unroll
    for (int r = 16 * seg + 15; r >= 16 * seg; --r) {
      run += eG[r * L::kLdG + m];
      eG[r * L::kLdG + m] = run;
    }
    __syncthreads();
    float add = cgv[m];
    for (int s2 = seg + 1; s2 < 4; ++s2) add += eG[(16 * s2) * L::kLdG + m];
    __syncthreads();                                  // every read of the later quarters' totals precedes their update
#pragma unroll
    for (int r = 16 * seg; r < 16 * seg + 16; ++r) eG[r * L::kLdG + m] += add;
    __syncthreads();
  }
  if (keep) {
#pragma unroll
    for (int c8 = 0; c8 < 4; ++c8) {
      const int m0 = 32 * half + 8 * c8;
      const float* grow = eG + krow * L::kLdG + m0;
      const float4 g0 = *reinterpret_cast<const float4*>(grow), g1 = *reinterpret_cast<const float4*>(grow + 4);
      const float g8[8] = {g0.x, g0.y, g0.z, g0.w, g1.x, g1.y, g1.z, g1.w};
      *reinterpret_cast<uint4*>((bf16*)d.dg + ((size_t)(t0 + kj) * H + h) * M + m0) = pack8(g8);
    }
  }
  if (failed) atomicExch(err, 1);
}
#undef NHA_MMA_WAIT
#undef NHA_SMEM_TO_MMA
#undef NHA_TRIL_TO_SMEM

template <int D, int R>
static int launch_rows(const nha_chunk_desc* d, const BwdWs& w, int* err, cudaStream_t cs) {
  typedef RowsLayout<D, R> L;
  cudaError_t e = set_max_smem((const void*)nha_bwd_rows_umma_kernel<D, R>, L::total);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  nha_bwd_rows_umma_kernel<D, R><<<dim3(NCB, d->H), kRowsThreads, L::total, cs>>>(*d, w, err);
  return check_launch();
}

template <int D, int R>
static int launch_cols(const nha_chunk_desc* d, const BwdWs& w, int* err, cudaStream_t cs) {
  typedef ColsLayout<D, R> L;
  cudaError_t e = set_max_smem((const void*)nha_bwd_cols_umma_kernel<D, R>, L::total);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  nha_bwd_gate_carry_kernel<<<dim3(NCB, d->H), kCarryThreads, 0, cs>>>(*d, w);
  int st = check_launch();
  if (st != NHA_OK) return st;
  nha_bwd_cols_umma_kernel<D, R><<<dim3(NCB, d->H), kColsThreads, L::total, cs>>>(*d, w, err);
  return check_launch();
}

bool bwd_umma_supported(const nha_chunk_desc* d) {
  const int NG = d->HQ / d->H;
  return d->K == d->V && d->M == 64 && (d->K == 64 || d->K == 128) && (NG == 1 || NG % 2 == 0);
}

// which: 0 = rows pass, 1 = columns pass.  The caller has checked bwd_umma_supported().
int bwd_umma_launch(const nha_chunk_desc* d, const BwdWs& w, int which, int* err, cudaStream_t cs) {
  const int NG = d->HQ / d->H;
  const bool one = NG == 1;
  if (d->K == 64) {
    if (which == 0) return one ? launch_rows<64, 64>(d, w, err, cs) : launch_rows<64, 128>(d, w, err, cs);
    return one ? launch_cols<64, 64>(d, w, err, cs) : launch_cols<64, 128>(d, w, err, cs);
  }
  if (which == 0) return one ? launch_rows<128, 64>(d, w, err, cs) : launch_rows<128, 128>(d, w, err, cs);
  return one ? launch_cols<128, 64>(d, w, err, cs) : launch_cols<128, 128>(d, w, err, cs);
}

}  // namespace nha
