// Output pass of the chunked NHA forward on the sm_100a tensor-core path: tcgen05.mma with operands in
// 128-byte-swizzled shared memory, accumulators in tensor memory (TMEM), two (D = 64) or four (D = 128)
// threads per query row for the softmax: tcgen05.ld hands a thread 32 or 16 columns of its row, the warps
// that share a TMEM lane quarter (w, w + 4, ...) take alternate parts of the columns and combine row maxima
// and sums through shared memory.  Eight or sixteen warps per CTA keep the element-wise phases, which are bound by
// instruction issue, from stalling on their own dependencies.  One CTA per (chunk, kv head); an MMA tile is 64 tokens x 1 head (R = 64, for
// HQ == H) or 64 tokens x 2 heads of the group (R = 128), and the CTA walks the heads of the group
// reusing the chunk's k', v', gates and chunk-start states.
//
// Per tile:   A  = q k'^T,  QH = q Hk,  S = q_swa k_swa^T (newest window step)           MMA group 1
//             X  = tril(A) (s' .* b)                                                      MMA group 2
//             ok = scale a .* (e^R .* QH + X);   window maxima step by step (older steps: load, S, max)
//             O  = (p~ a e^R) Hv,  Bv = (p~ a)(s' .* b)^T                                  MMA group 3
//             O += tril(Bv) v' + P~ v_win (newest step, its S still in TMEM)              MMA group 4
//             older window steps: load, S, P~, O += P~ v_win
// a = exp(G - R), b = exp(R - G) with ONE reference R[m] = Gend[m] / 2 per chunk and slot, kept as a
// shared fp32 table so the row threads spend no exponentials on the decay.  That keeps every factor
// inside exp(+-70) as long as a chunk decays by less than 140 nats per slot; a chunk beyond that is left
// untouched and flagged, and the general kernel (16-row block references, nha_chunk_fwd.cu) computes it
// instead, so the result never depends on the bound.  Probabilities are formed unnormalised against the
// joint row maximum (p~ = exp(x - max)), accumulated in one TMEM accumulator and divided by the row sum
// at the end, so every logit is exponentiated once.  A window step is two 64-key tiles for D = 64 and
// one for D = 128; a window of up to one step (W <= 64 at D = 64) needs no loop at all.
//
// Replaces chunk_nha_fused_o_kernel (nha_fla/ops/nha/chunk_fused.py:117-283) and, for chunk_nha, the
// flash-attn varlen forward + fla chunk_gsa forward + log-sum-exp merge (nha_fla/ops/nha/chunk.py:423-470).
#include <cuda.h>
#include <string.h>

#include "nha_common.cuh"
#include "nha_umma.cuh"
#include "nha_tma.cuh"

namespace nha {

using namespace umma;

constexpr float kUmmaDecayLimit = 140.0f;

// Tensor maps of the window keys (k_swa) and values (v) seen as [Ttot][H][D] bf16: a box is the 64-column half of
// 64 consecutive tokens of one kv head and lands as one 128-byte-swizzled [64][64] operand tile.
struct WindowMaps {
  CUtensorMap k, v;
  int use;                                            // 0: no tensor maps (copies go through cp.async)
};

template <int D, int R>
struct UmmaLayout {
  static constexpr int KT = D / 64;
  static constexpr int TP = D == 64 ? 2 : 1;          // 64-key tiles per window step
  static constexpr int NS = D == 64 ? 2 : 4;          // threads per row (D = 128 runs one CTA per SM: more warps)
  static constexpr int kThreads = 128 * NS;
  static constexpr int kATile = R * 128;              // one 64-wide k tile of an R-row A operand
  static constexpr int kWTile = TP * 8192;            // one 64-wide k tile of a window-step operand (64 TP rows)
  static constexpr bool kAlias = R == 64;             // one head per CTA: k' and Hk are dead after MMA group 1
  static constexpr bool kPOverW = R <= D;             // P~ fits over the window keys it was computed from
  static constexpr int tQ = 0;                        // q_gsa; later p~ .* a
  static constexpr int tQS = tQ + KT * kATile;        // q_swa
  static constexpr int tK = tQS + KT * kATile;        // k'
  static constexpr int tV = tK + KT * 8192;           // v'
  static constexpr int tHk = tV + KT * 8192;          // Hk [D][64]
  static constexpr int tHv = tHk + D * 128;           // Hv [64][D]
  static constexpr int tSB = tHv + KT * 8192;         // s' .* b [64][64]
  static constexpr int tW = tSB + 8192;               // window keys of one step [64 TP][D]
  static constexpr int tWV = tW + KT * kWTile;        // window values of one step [64 TP][D]
  static constexpr int end0 = tWV + KT * kWTile;
  static constexpr int tP = kPOverW ? tW : end0;      // P~ [R][64 TP]
  static constexpr int end1 = kPOverW ? end0 : end0 + TP * kATile;
  static constexpr int tAB = kAlias ? tHk : end1;     // tril(A) / tril(Bv)  [R][64]
  static constexpr int tPG = kAlias ? tK : end1 + kATile;   // p~ .* a .* e^R   [R][64]
  static constexpr int end2 = kAlias ? end1 : end1 + 2 * kATile;
  // D = 128 runs one CTA per SM, so the window loops are pipelined inside the CTA: a second set of window
  // buffers (behind k' and Hk, which are dead after MMA group 1 and fetched again for the next head tile; with one
  // head per CTA those tiles hold p~ and tril(A), so the set gets room of its own) and a second S accumulator.
  static constexpr bool kPipe = D == 128;
  static constexpr int end3 = (kPipe && kAlias) ? end2 + 2 * KT * kWTile : end2;
  static constexpr int tW2 = !kPipe ? tW : (kAlias ? end2 : tK);
  static constexpr int tWV2 = !kPipe ? tWV : (kAlias ? end2 + KT * kWTile : tHk);
  static constexpr int oA = end3;                     // fp32 [64][65]: cumulative gates, then a = exp(G - R)
  static constexpr int oR = oA + 64 * 65 * 4;         // fp32 [64] exp(R)
  static constexpr int oX = oR + 256;                 // fp32 [4][NS][128] row statistics swapped between the column parts
  static constexpr int oBar = oX + 4 * NS * 128 * 4;  // mbarriers (MMA groups; loads, S and PV of the pipelined loops) + TMEM slot              // mbarrier + TMEM slot
  static constexpr int total = oBar + 128 + 1024;     // + slack for the 1024-byte alignment of the base
  static constexpr int kTmemCols = D == 64 ? 256 : 512;
  // O reuses QH's columns at D = 64 (QH has been read by then)
  static constexpr int cA = 0, cQH = 64, cS = 128, cO = D == 64 ? 64 : 256;
  static constexpr int cS2 = kPipe ? 192 : cS;        // second S accumulator of the pipelined loops
  static_assert(total <= 227 * 1024, "shared memory of the output pass");
};

template <int D, int R>
__global__ void __launch_bounds__(UmmaLayout<D, R>::kThreads, (D == 64 && R == 64) ? 2 : 1) nha_fwd_umma_kernel(const nha_chunk_desc d, int* __restrict__ flags,
                                                                  int* __restrict__ err,
                                                                  const __grid_constant__ WindowMaps maps) {
  typedef UmmaLayout<D, R> L;
  constexpr int KT = L::KT, TH = R / 64, M = 64, TP = L::TP, WK = 64 * TP;
  constexpr int NS = L::NS, kUThreads = L::kThreads;
  constexpr int CW = 64 / NS;                       // columns of a 64-column accumulator per thread
  constexpr int KW = WK / NS;                       // keys of a window step per thread
  constexpr int LW = KW < 32 ? KW : 32;             // columns per tensor-memory load of the window logits
  const int H = d.H, HQ = d.HQ, NG = HQ / H, N = d.N;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
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
  uint64_t* mbar = (uint64_t*)(sm + L::oBar);
  uint32_t* tslot = (uint32_t*)(sm + L::oBar + 16);
  uint64_t* bl = (uint64_t*)(sm + L::oBar + 32);     // [2] window loads of the two buffer sets
  uint64_t* bs = bl + 2;                              // [2] S products of the two accumulators
  uint64_t* bpv = bl + 4;                             // P~ V product of the pipelined loop

  // window steps, newest first: step p covers the keys [kbase(p), kbase(p) + WK)
  const int jt_hi = ci;
  const int jt_lo = wl < 0 ? 0 : max(0, c0 - wl) / kChunk;
  const int nsteps = (jt_hi - jt_lo + TP) / TP;
#define NHA_KBASE(p_) ((jt_hi + 1 - TP * ((p_) + 1)) * kChunk)
  const bf16* ksw = (const bf16*)d.k_swa + ((size_t)t0 * H + h) * D;
  const bf16* vsw = (const bf16*)d.v + ((size_t)t0 * H + h) * D;

  // gates and write weights through registers (G needs an fp32 scan, s' is folded into s' .* b): their loads
  // go out first, the tile copies follow, and the registers are consumed after those have been issued
  const int lo = 0, hi = len - shift;              // valid source rows of the shifted inputs
  constexpr int kGS = 512 / kUThreads;              // 16-byte pieces of the [64][64] gate / write-weight tiles per thread
  uint4 sreg[kGS], greg[kGS];
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + kUThreads * j;
    const int r = i >> 3, c8 = i & 7;
    const int src = c0 + r - shift;
    sreg[j] = make_uint4(0u, 0u, 0u, 0u);
    greg[j] = make_uint4(0u, 0u, 0u, 0u);
    if (src >= lo && src < hi) {
      greg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.g + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
      sreg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.s + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
    }
  }
  // ---- everything the first head tile needs goes in flight at once -------------------------------------
  load_sw<D, kUThreads>(sm + L::tK, 8192, (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0 - shift, lo, hi, 64, 0, tid);
  load_sw<D, kUThreads>(sm + L::tV, 8192, (const bf16*)d.v + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0 - shift, lo, hi, 64, 0, tid);
  load_sw<64, kUThreads>(sm + L::tHk, 0, (const bf16*)d.hk_chunks + ((size_t)cg * H + h) * D * M, M, 0, 0, D, D, 0, tid);
  load_sw<D, kUThreads>(sm + L::tHv, 8192, (const bf16*)d.hv_chunks + ((size_t)cg * H + h) * M * D, D, 0, 0, M, M, 0, tid);
#define NHA_LOAD_HEAD_TILE(ht_)                                                                                       \
  do {                                                                                                                \
    const int hq0_ = h * NG + (ht_) * TH;                                                                             \
    _Pragma("unroll") for (int t2 = 0; t2 < TH; ++t2) {                                                               \
      load_sw<D, kUThreads>(sm + L::tQ, L::kATile, (const bf16*)d.q_gsa + ((size_t)t0 * HQ + hq0_ + t2) * D, (int64_t)HQ * D,    \
                 c0, 0, len, 64, 64 * t2, tid);                                                                       \
      load_sw<D, kUThreads>(sm + L::tQS, L::kATile, (const bf16*)d.q_swa + ((size_t)t0 * HQ + hq0_ + t2) * D, (int64_t)HQ * D,   \
                 c0, 0, len, 64, 64 * t2, tid);                                                                       \
    }                                                                                                                 \
    if (L::kPipe && !L::kAlias && (ht_) > 0) {     /* the second window buffer set has overwritten k' and Hk */       \
      load_sw<D, kUThreads>(sm + L::tK, 8192, (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * D, (int64_t)H * D,          \
                            c0 - shift, lo, hi, 64, 0, tid);                                                            \
      load_sw<64, kUThreads>(sm + L::tHk, 0, (const bf16*)d.hk_chunks + ((size_t)cg * H + h) * D * M, M, 0, 0, D, D,    \
                             0, tid);                                                                                   \
    }                                                                                                                 \
    /* keys of the OLDEST step (the first one the maxima sweep needs); with a single step also its values */         \
    load_sw<D, kUThreads>(sm + L::tW, L::kWTile, ksw, (int64_t)H * D, NHA_KBASE(nsteps - 1), 0, len, WK, 0, tid);                \
    if (nsteps == 1) load_sw<D, kUThreads>(sm + L::tWV, L::kWTile, vsw, (int64_t)H * D, NHA_KBASE(0), 0, len, WK, 0, tid);       \
    cp_commit();                                                                                                      \
  } while (0)
  NHA_LOAD_HEAD_TILE(0);
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + kUThreads * j;
    const int r = i >> 3, c8 = i & 7;
    float gv[8];
    unpack8(greg[j], gv);
#pragma unroll
    for (int e = 0; e < 8; ++e) As[r * 65 + 8 * c8 + e] = gv[e];
  }
  if (tid == 0) {
    mbar_init(mbar, 1);
    for (int i = 0; i < 5; ++i) mbar_init(&bl[i], 1);
  }
  __syncthreads();
  // inclusive scan along the rows: kUThreads / 64 threads per column (a segment of rows each), then the totals
  // of the earlier segments are added
  {
    constexpr int NSEG = kUThreads / 64, RS = 64 / NSEG;
    const int m = tid & 63, seg = tid >> 6;
    float run = 0.f;
#pragma unroll
    for (int r = RS * seg; r < RS * seg + RS; ++r) {
      run += As[r * 65 + m];
      As[r * 65 + m] = run;
    }
    __syncthreads();
    float add = 0.f;
    for (int s2 = 0; s2 < seg; ++s2) add += As[(RS * s2 + RS - 1) * 65 + m];
    __syncthreads();                                  // every total is read before any of them changes
    if (seg > 0) {
#pragma unroll
      for (int r = RS * seg; r < RS * seg + RS; ++r) As[r * 65 + m] += add;
    }
    __syncthreads();
  }
  const bool mine_unsafe = tid < 64 && fabsf(As[63 * 65 + tid]) > kUmmaDecayLimit;
  const int unsafe = __syncthreads_or(mine_unsafe ? 1 : 0);
  if (tid == 0) flags[(size_t)cg * H + h] = unsafe;
  if (unsafe) {
    cp_wait_all();
    return;
  }
  // a = exp(G - R) replaces G in place, s' .* b = s' exp(R - G) goes into its swizzled tile ([64 i][64 m]:
  // K-major for (p~ a) SB^T, MN-major for tril(A) SB); each thread converts the elements it also reads
  float rref[8];
  {
    const int c8 = tid & 7;
#pragma unroll
    for (int e = 0; e < 8; ++e) rref[e] = 0.5f * As[63 * 65 + 8 * c8 + e];
  }
  __syncthreads();                                    // every thread holds its references before the table changes
  if (tid < 8) {
#pragma unroll
    for (int e = 0; e < 8; ++e) ER[8 * tid + e] = __expf(rref[e]);
  }
#pragma unroll
  for (int j = 0; j < kGS; ++j) {
    const int i = tid + kUThreads * j;
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
  const int quarter = warp & 3, cpart = warp >> 2;  // TMEM lane quarter of this warp; column part it works on
  const uint32_t tlane = tbase + ((uint32_t)(quarter * 32) << 16);
  uint32_t phase = 0;
  bool failed = false;

  // row of this thread inside the tile (NS threads, one per column part, share a row)
  const bool active = R == 128 ? true : lane < 16;
  const int row = R == 128 ? quarter * 32 + lane : quarter * 16 + (lane & 15);
  const int tk = row & 63;                          // token inside the chunk
  const int th = row >> 6;                          // head inside the tile
  const int pos = c0 + tk;
  const bool in_seq = pos < len;
  float* xch = (float*)(sm + L::oX);                // [4 exchange points][NS parts][128 rows]
  // visible keys of this row: klo <= key <= pos, tested as (unsigned)(key - klo) <= kspan; a row past the
  // sequence end sees nothing
  constexpr float kLog2e = 1.4426950408889634f;
  const int klo = in_seq ? (wl < 0 ? 0 : max(0, pos - wl)) : (1 << 30);
  const unsigned kspan = in_seq ? (unsigned)(pos - klo) : 0u;
  const float sc2 = d.scale * kLog2e;
  const uint32_t aQ = smem_u32(sm + L::tQ), aQS = smem_u32(sm + L::tQS), aK = smem_u32(sm + L::tK);
  const uint32_t aV = smem_u32(sm + L::tV), aHk = smem_u32(sm + L::tHk), aHv = smem_u32(sm + L::tHv);
  const uint32_t aSB = smem_u32(sm + L::tSB), aW = smem_u32(sm + L::tW), aWV = smem_u32(sm + L::tWV);
  const uint32_t aAB = smem_u32(sm + L::tAB), aPG = smem_u32(sm + L::tPG), aPA = aQ, aP = smem_u32(sm + L::tP);

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
// this thread's part of tril of a [R][64] accumulator (row token tk keeps columns i <= tk) -> bf16 A-operand tile
#define NHA_TRIL_TO_SMEM(col0, dst_off)                                                          \
  do {                                                                                           \
    float tv_[CW];                                                                               \
    tmem_ldw<CW>(tlane + (col0) + CW * cpart, tv_);                                              \
    if (active) {                                                                                \
      _Pragma("unroll") for (int c8 = 0; c8 < CW / 8; ++c8) {                                    \
        float o8[8];                                                                             \
        _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                          \
          const int i_ = CW * cpart + 8 * c8 + e;                                                \
          o8[e] = i_ <= tk ? tv_[8 * c8 + e] : 0.f;                                              \
        }                                                                                        \
        *reinterpret_cast<uint4*>(sm + (dst_off) + sw_off(row, (CW / 8) * cpart + c8)) = pack8(o8); \
      }                                                                                          \
    }                                                                                            \
  } while (0)
// S = q_swa (window keys of one step)^T
#define NHA_ISSUE_S_AT(cs_, aw_) mma_tile(tbase + (cs_), aQS, L::kATile, (aw_), L::kWTile, R, WK, D / 16, 0, false)
#define NHA_ISSUE_S() NHA_ISSUE_S_AT(L::cS, aW)
// this thread's KW keys of a window step: keys kb_ + KW cpart + [0, KW)
#define NHA_STEP_MAX(kb_) NHA_STEP_MAX_AT(kb_, L::cS)
#define NHA_STEP_MAX_AT(kb_, cs_)                                                                \
  do {                                                                                           \
    float sv_[LW];                                                                               \
    _Pragma("unroll") for (int pp = 0; pp < KW / LW; ++pp) {                                     \
      const int key0 = KW * cpart + LW * pp;                                                     \
      tmem_ldw<LW>(tlane + (cs_) + key0, sv_);                                                   \
      const int off_ = (kb_) + key0 - klo;                                                       \
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};                                \
      _Pragma("unroll") for (int e = 0; e < LW; ++e)                                             \
        m4[e & 3] = fmaxf(m4[e & 3], (unsigned)(off_ + e) <= kspan ? sv_[e] : -INFINITY);        \
      ms = fmaxf(ms, d.scale * fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3])));                 \
    }                                                                                            \
  } while (0)
// P~ = exp(scale S - ms) cw of this thread's keys of a step, into the swizzled tile; row sum into ls
#define NHA_STEP_PROB(kb_) NHA_STEP_PROB_AT(kb_, L::cS, L::tP)
#define NHA_STEP_PROB_AT(kb_, cs_, tp_)                                                          \
  do {                                                                                           \
    float sv_[LW];                                                                               \
    const float nms_ = -ms * kLog2e;                                                             \
    _Pragma("unroll") for (int pp = 0; pp < KW / LW; ++pp) {                                     \
      const int key0 = KW * cpart + LW * pp;                                                     \
      tmem_ldw<LW>(tlane + (cs_) + key0, sv_);                                                   \
      const int off_ = (kb_) + key0 - klo;                                                       \
      if (active) {                                                                              \
        float l4[4] = {0.f, 0.f, 0.f, 0.f};                                                      \
        _Pragma("unroll") for (int c8 = 0; c8 < LW / 8; ++c8) {                                  \
          float o8[8];                                                                           \
          _Pragma("unroll") for (int e = 0; e < 8; ++e) {                                        \
            const float pe = (unsigned)(off_ + 8 * c8 + e) <= kspan                              \
                                 ? exp2f(fmaf(sv_[8 * c8 + e], sc2, nms_)) : 0.f;                \
            l4[e & 3] += pe;                                                                     \
            o8[e] = pe * cw;                                                                     \
          }                                                                                      \
          const int kk_ = key0 + 8 * c8;                                                         \
          *reinterpret_cast<uint4*>(sm + (tp_) + (kk_ >> 6) * L::kATile +                        \
                                    sw_off(row, (kk_ & 63) >> 3)) = pack8(o8);                   \
        }                                                                                        \
        ls += (l4[0] + l4[1]) + (l4[2] + l4[3]);                                                 \
      }                                                                                          \
    }                                                                                            \
  } while (0)
// O += P~ (window values of one step)
#define NHA_ISSUE_PV() NHA_ISSUE_PV_AT(aP, aWV)
#define NHA_ISSUE_PV_AT(ap_, awv_)                                                               \
  do {                                                                                           \
    _Pragma("unroll") for (int ct = 0; ct < KT; ++ct)                                            \
      mma_tile(tbase + L::cO + 64 * ct, (ap_), L::kATile, (awv_) + ct * L::kWTile, 0, R, 64, 4 * TP, 1, true); \
  } while (0)
// combine a row statistic over the NS threads of the row (slot_: exchange point 0..3; OP_: fmaxf or addf);
// the barrier inside is reached by every thread of the CTA
#define NHA_XCHG(slot_, v_, OP_)                                                                 \
  do {                                                                                           \
    xch[((slot_) * NS + cpart) * 128 + row] = (v_);                                              \
    __syncthreads();                                                                             \
    float r_ = xch[((slot_) * NS) * 128 + row];                                                  \
    _Pragma("unroll") for (int p_ = 1; p_ < NS; ++p_) r_ = OP_(r_, xch[((slot_) * NS + p_) * 128 + row]); \
    (v_) = r_;                                                                                   \
  } while (0)
  auto addf = [](float x, float y) { return x + y; };

// pipelined loops (D = 128): window step p_ into buffer set set_ (its keys, with wv_ also its values).  A step whose
// 64 keys lie inside the sequence comes by TMA (one thread, two or four boxes, bytes counted on the set's mbarrier);
// a step that sticks out of the sequence is copied with zero fill by every thread and then arrives on the same
// barrier.  Every thread of the CTA runs the macro.  Issue work is spread over three threads of three warps so that
// it does not queue behind one thread: thread 0 the MMA groups and P~ V, thread 32 the TMA loads, thread 64 the S
// products of the loops.
#define NHA_LOAD_STEP(set_, p_, wv_)                                                                                \
  do {                                                                                                              \
    const int kb__ = NHA_KBASE(p_);                                                                                 \
    unsigned char* w__ = sm + ((set_) ? L::tW2 : L::tW);                                                            \
    unsigned char* v__ = sm + ((set_) ? L::tWV2 : L::tWV);                                                          \
    if (maps.use && kb__ >= 0 && kb__ + WK <= len) {                                                                \
      if (tid == 32) {                                                                                              \
        mbar_expect_tx(&bl[set_], (uint32_t)((wv_) ? 2 : 1) * WK * D * 2);                                          \
        _Pragma("unroll") for (int kt = 0; kt < KT; ++kt) {                                                         \
          tma_load_3d(w__ + kt * L::kWTile, &maps.k, 64 * kt, h, t0 + kb__, &bl[set_]);                             \
          if (wv_) tma_load_3d(v__ + kt * L::kWTile, &maps.v, 64 * kt, h, t0 + kb__, &bl[set_]);                    \
        }                                                                                                           \
      }                                                                                                             \
    } else {                                                                                                        \
      load_sw<D, kUThreads>(w__, L::kWTile, ksw, (int64_t)H * D, kb__, 0, len, WK, 0, tid);                         \
      if (wv_) load_sw<D, kUThreads>(v__, L::kWTile, vsw, (int64_t)H * D, kb__, 0, len, WK, 0, tid);                \
      cp_commit();                                                                                                  \
      cp_wait_all();                                                                                                \
      fence_async_smem();                                                                                           \
      __syncthreads();                                                                                              \
      if (tid == 32) mbar_arrive(&bl[set_]);                                                                        \
    }                                                                                                               \
  } while (0)
// bounded wait on one of the pipeline's mbarriers; bit_ of `phases` holds its parity
#define NHA_WAIT_BAR(bar_, bit_)                                                                                    \
  do {                                                                                                              \
    if (!failed && !mbar_wait((bar_), (phases >> (bit_)) & 1u)) failed = true;                                                 \
    phases ^= 1u << (bit_);                                                                                         \
    tc_fence_after();                                                                                               \
  } while (0)
  uint32_t phases = 0u;                               // parities: bits 0-1 loads, 2-3 S products, 4 P~ V product

  for (int ht = 0; ht < NG / TH; ++ht) {
    const int hq0 = h * NG + ht * TH;
    const int hq = hq0 + th;
    if (ht > 0) NHA_LOAD_HEAD_TILE(ht);
    cp_wait_all();
    NHA_SMEM_TO_MMA();
    // ---- MMA group 1: A = q k'^T, QH = q Hk, S of the oldest window step --------------------------------------
    if (tid == 0) {
      mma_tile(tbase + L::cA, aQ, L::kATile, aK, 8192, R, 64, D / 16, 0, false);
      mma_tile(tbase + L::cQH, aQ, L::kATile, aHk, 0, R, 64, D / 16, 1, false);
      NHA_ISSUE_S();
    }
    NHA_MMA_WAIT();
    NHA_TRIL_TO_SMEM(L::cA, L::tAB);
    NHA_SMEM_TO_MMA();
    // ---- MMA group 2: X = tril(A) SB; the window maxima are taken while it runs ---------------------------------
    if (tid == 0) mma_tile(tbase + L::cA, aAB, L::kATile, aSB, 0, R, 64, 4, 1, false);
    float ms = -INFINITY;
    NHA_STEP_MAX(NHA_KBASE(nsteps - 1));
    NHA_MMA_WAIT();
    // ---- this thread's 32 slot logits ok = scale a .* (e^R .* QH + X), kept in registers --------------------------
    float ok[CW];
    float mg = -INFINITY;
    {
      float qh[CW];
      tmem_ldw<CW>(tlane + L::cQH + CW * cpart, qh);
      tmem_ldw<CW>(tlane + L::cA + CW * cpart, ok);
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int e = 0; e < CW; ++e) {
        const int m = CW * cpart + e;
        const float v = d.scale * As[tk * 65 + m] * (ER[m] * qh[e] + ok[e]);
        ok[e] = v;
        m4[e & 3] = fmaxf(m4[e & 3], v);
      }
      mg = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
    }
    NHA_XCHG(0, mg, fmaxf);
    float lg = 0.f;
    {
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      const float nmg = -mg * kLog2e;
#pragma unroll
      for (int e = 0; e < CW; ++e) {
        ok[e] = exp2f(fmaf(ok[e], kLog2e, nmg));      // from here on ok holds exp(ok - mg)
        l4[e & 3] += ok[e];
      }
      lg = (l4[0] + l4[1]) + (l4[2] + l4[3]);
    }
    // ---- maxima of the newer window steps (the newest one last: its S stays in TMEM) -----------------------------
    int rset = 0;                                      // buffer set / accumulator that hold the newest step afterwards
    if constexpr (L::kPipe) {
      // step index i counts from the oldest step (i = 0: loaded with the head tile, S formed in MMA group 1); step i uses
      // buffer set and accumulator i & 1.  The load of step i + 1 and the maximum of step i - 1 overlap S of step i.
      if (nsteps > 1) NHA_LOAD_STEP(1, nsteps - 2, nsteps - 2 == 0);
      for (int i = 1; i < nsteps; ++i) {
        const int b = i & 1, p = nsteps - 1 - i;
        NHA_WAIT_BAR(&bl[b], b);
        tc_fence_before();
        __syncthreads();                               // every thread has read the maxima of step i - 2 from this accumulator
        tc_fence_after();
        if (tid == 64) {
          NHA_ISSUE_S_AT(b ? L::cS2 : L::cS, smem_u32(sm + (b ? L::tW2 : L::tW)));
          commit(&bs[b]);
        }
        // the other set's keys were read by S of step i - 1, which has completed
        if (i + 1 < nsteps) {
          if (b) NHA_LOAD_STEP(0, p - 1, p - 1 == 0); else NHA_LOAD_STEP(1, p - 1, p - 1 == 0);
        }
        if (i >= 2) {
          if (b) NHA_STEP_MAX_AT(NHA_KBASE(p + 1), L::cS); else NHA_STEP_MAX_AT(NHA_KBASE(p + 1), L::cS2);
        }
        NHA_WAIT_BAR(&bs[b], 2 + b);
      }
      if (nsteps > 1) {
        rset = (nsteps - 1) & 1;
        if (rset) NHA_STEP_MAX_AT(NHA_KBASE(0), L::cS2); else NHA_STEP_MAX_AT(NHA_KBASE(0), L::cS);
        // the other set is free: the first older step of the probability sweep goes in flight now
        tc_fence_before();
        __syncthreads();
        if (rset) NHA_LOAD_STEP(0, 1, true); else NHA_LOAD_STEP(1, 1, true);
      }
    } else {
      for (int p = nsteps - 2; p >= 0; --p) {
        tc_fence_before();
        __syncthreads();
        load_sw<D, kUThreads>(sm + L::tW, L::kWTile, ksw, (int64_t)H * D, NHA_KBASE(p), 0, len, WK, 0, tid);
        if (p == 0) load_sw<D, kUThreads>(sm + L::tWV, L::kWTile, vsw, (int64_t)H * D, NHA_KBASE(0), 0, len, WK, 0, tid);
        cp_commit();
        cp_wait_all();
        NHA_SMEM_TO_MMA();
        if (tid == 0) NHA_ISSUE_S();
        NHA_MMA_WAIT();
        NHA_STEP_MAX(NHA_KBASE(p));
      }
    }
    // ---- joint maximum; unnormalised slot probabilities as bf16 A operands -----------------------------------------
    tc_fence_before();
    NHA_XCHG(1, ms, fmaxf);                           // its barrier also puts every thread past its reads of QH / X
                                                      // and of the products that read tQ
    const float mx = fmaxf(mg, ms);
    const float cgs = __expf(mg - mx);               // slot entries:   p~ = exp(ok - mg) cgs
    const float cw = __expf(ms - mx);                // window entries: p~ = exp(s  - ms) cw
    if (active) {
#pragma unroll
      for (int c8 = 0; c8 < CW / 8; ++c8) {
        float pg8[8], pa8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int m = CW * cpart + 8 * c8 + e;
          const float pa = in_seq ? ok[8 * c8 + e] * cgs * As[tk * 65 + m] : 0.f;
          pa8[e] = pa;
          pg8[e] = pa * ER[m];
        }
        *reinterpret_cast<uint4*>(sm + L::tPG + sw_off(row, (CW / 8) * cpart + c8)) = pack8(pg8);
        *reinterpret_cast<uint4*>(sm + L::tQ + sw_off(row, (CW / 8) * cpart + c8)) = pack8(pa8);
      }
    }
    NHA_SMEM_TO_MMA();
    // ---- MMA group 3: O = (p~ a e^R) Hv, Bv = (p~ a) SB^T; the newest step's P~ is formed while it runs ---------------
    if (tid == 0) {
#pragma unroll
      for (int ct = 0; ct < KT; ++ct)
        mma_tile(tbase + L::cO + 64 * ct, aPG, L::kATile, aHv + ct * 8192, 0, R, 64, 4, 1, false);
      mma_tile(tbase + L::cA, aPA, L::kATile, aSB, 0, R, 64, 4, 0, false);
    }
    float ls = 0.f;
    if (rset) NHA_STEP_PROB_AT(NHA_KBASE(0), L::cS2, L::tW2); else NHA_STEP_PROB(NHA_KBASE(0));
    NHA_MMA_WAIT();
    NHA_TRIL_TO_SMEM(L::cA, L::tAB);
    NHA_SMEM_TO_MMA();
    // ---- MMA group 4: O += tril(Bv) v' + P~ v_win (newest step) -------------------------------------------------------------
    if (tid == 0) {
#pragma unroll
      for (int ct = 0; ct < KT; ++ct)
        mma_tile(tbase + L::cO + 64 * ct, aAB, L::kATile, aV + ct * 8192, 0, R, 64, 4, 1, true);
      if (rset) NHA_ISSUE_PV_AT(smem_u32(sm + L::tW2), smem_u32(sm + L::tWV2)); else NHA_ISSUE_PV();
    }
    NHA_MMA_WAIT();
    // ---- older window steps ------------------------------------------------------------------------------------------------
    if constexpr (L::kPipe) {
      // step j (j = 1: the first older one) uses buffer set and accumulator (rset + j) & 1; its load was issued one
      // step ahead, P~ V of step j runs while step j + 1 is prepared
      for (int j = 1; j < nsteps; ++j) {
        const int b = (rset + j) & 1;
        NHA_WAIT_BAR(&bl[b], b);
        tc_fence_before();
        __syncthreads();                               // every thread has read S of step j - 2 from this accumulator
        tc_fence_after();
        if (tid == 64) {
          NHA_ISSUE_S_AT(b ? L::cS2 : L::cS, smem_u32(sm + (b ? L::tW2 : L::tW)));
          commit(&bs[b]);
        }
        if (j >= 2) NHA_WAIT_BAR(bpv, 4);              // P~ V of step j - 1 has completed: the other set is free
        if (j + 1 < nsteps) {
          if (b) NHA_LOAD_STEP(0, j + 1, true); else NHA_LOAD_STEP(1, j + 1, true);
        }
        NHA_WAIT_BAR(&bs[b], 2 + b);
        if (b) NHA_STEP_PROB_AT(NHA_KBASE(j), L::cS2, L::tW2); else NHA_STEP_PROB_AT(NHA_KBASE(j), L::cS, L::tW);
        NHA_SMEM_TO_MMA();
        if (tid == 0) {
          if (b) NHA_ISSUE_PV_AT(smem_u32(sm + L::tW2), smem_u32(sm + L::tWV2));
          else NHA_ISSUE_PV_AT(smem_u32(sm + L::tW), smem_u32(sm + L::tWV));
          commit(bpv);
        }
      }
      if (nsteps > 1) NHA_WAIT_BAR(bpv, 4);
    } else {
      for (int p = 1; p < nsteps; ++p) {
        tc_fence_before();
        __syncthreads();
        load_sw<D, kUThreads>(sm + L::tW, L::kWTile, ksw, (int64_t)H * D, NHA_KBASE(p), 0, len, WK, 0, tid);
        load_sw<D, kUThreads>(sm + L::tWV, L::kWTile, vsw, (int64_t)H * D, NHA_KBASE(p), 0, len, WK, 0, tid);
        cp_commit();
        cp_wait_all();
        NHA_SMEM_TO_MMA();
        if (tid == 0) NHA_ISSUE_S();
        NHA_MMA_WAIT();
        NHA_STEP_PROB(NHA_KBASE(p));
        NHA_SMEM_TO_MMA();
        if (tid == 0) NHA_ISSUE_PV();
        NHA_MMA_WAIT();
      }
    }
    // ---- row sums of all column parts, normalise and store ----------------------------------------------------------------
    {
      xch[(2 * NS + cpart) * 128 + row] = lg;
      xch[(3 * NS + cpart) * 128 + row] = ls;
      __syncthreads();
      lg = 0.f;
      ls = 0.f;
#pragma unroll
      for (int p2 = 0; p2 < NS; ++p2) {
        lg += xch[(2 * NS + p2) * 128 + row];
        ls += xch[(3 * NS + p2) * 128 + row];
      }
    }
    const float lsum = lg * cgs + ls * cw;
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    if (active && in_seq && cpart == 0) {
      d.lse_gsa[(size_t)(t0 + pos) * HQ + hq] = mg + __logf(lg);
      d.lse_swa[(size_t)(t0 + pos) * HQ + hq] = ms + __logf(ls);
    }
    {
      // D / NS = 32 output columns per thread
      static_assert(D / NS == 32, "output columns per thread");
      float ov[32];
      tmem_ld32(tlane + L::cO + 32 * cpart, ov);
      if (active && in_seq) {
#pragma unroll
        for (int e = 0; e < 32; ++e) ov[e] *= inv;
        bf16* orow = (bf16*)d.o + ((size_t)(t0 + pos) * HQ + hq) * D + 32 * cpart;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) *reinterpret_cast<uint4*>(orow + 8 * c8) = pack8(ov + 8 * c8);
      }
    }
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
#undef NHA_MMA_WAIT
#undef NHA_SMEM_TO_MMA
#undef NHA_TRIL_TO_SMEM
#undef NHA_ISSUE_S
#undef NHA_ISSUE_S_AT
#undef NHA_STEP_MAX_AT
#undef NHA_STEP_PROB_AT
#undef NHA_ISSUE_PV_AT
#undef NHA_LOAD_STEP
#undef NHA_WAIT_BAR
#undef NHA_STEP_MAX
#undef NHA_STEP_PROB
#undef NHA_ISSUE_PV
#undef NHA_XCHG
#undef NHA_LOAD_HEAD_TILE
#undef NHA_KBASE
  if (failed) atomicExch(err, 1);
  cp_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, L::kTmemCols);
}

template <int D, int R>
static int launch_umma(const nha_chunk_desc* d, int* flags, int* err, cudaStream_t cs) {
  typedef UmmaLayout<D, R> L;
  cudaError_t e = set_max_smem((const void*)nha_fwd_umma_kernel<D, R>, L::total);
  if (e != cudaSuccess) return record_cuda_error(e);
  WindowMaps maps;
  memset(&maps, 0, sizeof(maps));
  if (L::kPipe) {
    const char* off = getenv("NHA_B200_NO_TMA");
    maps.use = !(off && off[0] == '1') && make_map_rows_heads(&maps.k, d->k_swa, d->Ttot, d->H, D) &&
               make_map_rows_heads(&maps.v, d->v, d->Ttot, d->H, D);
  }
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  nha_fwd_umma_kernel<D, R><<<dim3(NCB, d->H), L::kThreads, L::total, cs>>>(*d, flags, err, maps);
  return check_launch();
}

// Runs the tensor-memory output pass when the shape has one (K == V in {64, 128}, M == 64, one or an
// even number of query heads per kv head, positive scale).  Returns NHA_ERR_UNSUPPORTED otherwise.
bool fwd_pipe_supported(const nha_chunk_desc* d);
int fwd_pipe_launch(const nha_chunk_desc* d, int* flags, int* err, cudaStream_t cs);

int chunk_output_pass_umma(const nha_chunk_desc* d, int* flags, int* err, cudaStream_t cs) {
  const int NG = d->HQ / d->H;
  if (d->K != d->V || d->M != 64) return NHA_ERR_UNSUPPORTED;
  if (!(d->scale > 0.f)) return NHA_ERR_UNSUPPORTED;     // row maxima are taken before scaling
  // head dim 128 with groups of four query heads: the warp-specialised pipeline (nha_chunk_fwd_pipe.cu)
  if (fwd_pipe_supported(d)) {
    const int st = fwd_pipe_launch(d, flags, err, cs);
    if (st != NHA_ERR_UNSUPPORTED) return st;
  }
  if (d->K == 64 && NG == 1) return launch_umma<64, 64>(d, flags, err, cs);
  if (d->K == 64 && NG % 2 == 0) return launch_umma<64, 128>(d, flags, err, cs);
  if (d->K == 128 && NG == 1) return launch_umma<128, 64>(d, flags, err, cs);
  if (d->K == 128 && NG % 2 == 0) return launch_umma<128, 128>(d, flags, err, cs);
  return NHA_ERR_UNSUPPORTED;
}

}  // namespace nha
