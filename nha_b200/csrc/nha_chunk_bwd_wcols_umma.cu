// Key side of the sliding-window backward on the sm_100a tensor-core path: dk_swa and the window part of
// dv.  One CTA per (key chunk, kv head).  The query rows that can see the chunk - every (query chunk,
// query head of the group) pair - are taken two 64-row blocks at a time as the 128 rows of
//     S = q_swa k_swa^T,   dP = do v^T                           (tcgen05.mma, accumulators in TMEM)
// with two threads per query row (alternate 32-key halves) for p = exp(scale S - L) and dz = scale p (dP - delta):
// the row's joint log-sum-exp L and delta = <do, o> sit in registers.  The transposed products
//     dv_win += p^T do,   dk_swa += dz^T q_swa
// read p, dz, do and q_swa through MN-major descriptors (k = query row), so nothing is transposed in
// memory.  The window part does not depend on the gates, so every chunk takes this path.
//
// Replaces, with the rows pass, the flash-attn varlen backward reached from
// ChunkNativeHybridAttentionFunction.backward (nha_fla/ops/nha/chunk.py:491-564).
#include "nha_bwd_common.cuh"
#include "nha_common.cuh"
#include "nha_umma.cuh"

namespace nha {

using namespace umma;

constexpr int kWCThreads = 256;          // two threads per query row (alternate 32-key halves)

template <int D>
struct WColsLayout {
  static constexpr int KT = D / 64;
  static constexpr int kATile = 128 * 128;              // one 64-wide k tile of a 128-row operand
  static constexpr int tK = 0;                           // k_swa of the chunk [64][D]
  static constexpr int tV = tK + KT * 8192;              // v of the chunk [64][D]
  static constexpr int tQS = tV + KT * 8192;             // q_swa of the two row blocks [128][D]
  static constexpr int tDO = tQS + KT * kATile;          // do of the two row blocks [128][D]
  static constexpr int tP = tDO + KT * kATile;           // p  [128][64]
  static constexpr int tZ = tP + kATile;                 // dz [128][64]
  static constexpr int oBar = tZ + kATile;
  static constexpr int total = oBar + 64 + 1024;
  static constexpr int kTmemCols = D == 64 ? 256 : 512;
  static constexpr int cS = 0, cDP = 64, cDV = 128, cDK = 128 + D;
};

template <int D>
__global__ void __launch_bounds__(kWCThreads, D == 64 ? 2 : 1) nha_bwd_wcols_umma_kernel(const nha_chunk_desc d, const BwdWs w,
                                                                        int* __restrict__ err) {
  typedef WColsLayout<D> L;
  constexpr int KT = L::KT;
  const int H = d.H, HQ = d.HQ, NG = HQ / H, N = d.N;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
  const int ci = rc.ci;
  const int t0 = rc.t0;
  const int len = rc.len;
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int c0 = ci * kChunk;
  const int wl = seq_window(d, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  uint64_t* mbar = (uint64_t*)(sm + L::oBar);
  uint32_t* tslot = (uint32_t*)(sm + L::oBar + 16);

  // query chunks that can see a key of this chunk, and the 64-row blocks (query chunk, query head) they make
  const int qi_lo = ci;
  const int qi_hi = wl < 0 ? nchunks - 1 : min(nchunks - 1, (c0 + kChunk - 1 + wl) / kChunk);
  const int nblk = (qi_hi - qi_lo + 1) * NG;
  const int npairs = (nblk + 1) >> 1;

  load_sw<D, kWCThreads>(sm + L::tK, 8192, (const bf16*)d.k_swa + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0, 0, len, 64, 0, tid);
  load_sw<D, kWCThreads>(sm + L::tV, 8192, (const bf16*)d.v + ((size_t)t0 * H + h) * D, (int64_t)H * D, c0, 0, len, 64, 0, tid);
  if (tid == 0) mbar_init(mbar, 1);
  if (warp == 0) tmem_alloc(tslot, L::kTmemCols);
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tslot;
  const int quarter = warp & 3, chalf = warp >> 2;    // TMEM lane quarter of this warp; key half it works on
  const uint32_t tlane = tbase + ((uint32_t)(quarter * 32) << 16);
  constexpr float kLog2e = 1.4426950408889634f;
  const float sc2 = d.scale * kLog2e;
  uint32_t phase = 0;
  bool failed = false;
  const uint32_t aK = smem_u32(sm + L::tK), aV = smem_u32(sm + L::tV), aQS = smem_u32(sm + L::tQS);
  const uint32_t aDO = smem_u32(sm + L::tDO), aP = smem_u32(sm + L::tP), aZ = smem_u32(sm + L::tZ);
  const int row = quarter * 32 + lane;                // this thread's row of the 128-row products
  const int half = row >> 6, tk = row & 63;           // block of the pair, query inside the chunk

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

  for (int pr = 0; pr < npairs; ++pr) {
    // ---- the two row blocks of this pair ---------------------------------------------------------------------
#pragma unroll
    for (int t2 = 0; t2 < 2; ++t2) {
      const int b = 2 * pr + t2;
      const bool valid = b < nblk;
      const int qi = qi_lo + (valid ? b / NG : 0), hq = h * NG + (valid ? b % NG : 0);
      load_sw<D, kWCThreads>(sm + L::tQS, L::kATile, (const bf16*)d.q_swa + ((size_t)t0 * HQ + hq) * D, (int64_t)HQ * D, qi * kChunk, 0,
                 valid ? len : 0, 64, 64 * t2, tid);
      load_sw<D, kWCThreads>(sm + L::tDO, L::kATile, (const bf16*)d.d_o + ((size_t)t0 * HQ + hq) * D, (int64_t)HQ * D, qi * kChunk, 0,
                 valid ? len : 0, 64, 64 * t2, tid);
    }
    cp_commit();
    const int b = 2 * pr + half;
    const int pq = (qi_lo + b / NG) * kChunk + tk;
    const bool live = b < nblk && pq < len;
    float Lj = 0.f, delta = 0.f;
    if (live) {
      const size_t rowq = (size_t)(t0 + pq) * HQ + h * NG + b % NG;
      Lj = w.lj[rowq];
      delta = w.delta[rowq];
    }
    cp_wait_all();
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
      mma_tile(tbase + L::cS, aQS, L::kATile, aK, 8192, 128, 64, D / 16, 0, false);      // S  = q_swa k^T
      mma_tile(tbase + L::cDP, aDO, L::kATile, aV, 8192, 128, 64, D / 16, 0, false);     // dP = do v^T
    }
    NHA_MMA_WAIT();
    {
      // visible keys of this query row: klo <= key <= pq, tested as (unsigned)(key - klo) <= kspan
      const int klo = live ? (wl < 0 ? 0 : max(0, pq - wl)) : (1 << 30);
      const unsigned kspan = live ? (unsigned)(pq - klo) : 0u;
      const float nLj = -Lj * kLog2e;
      const int off = c0 + 32 * chalf - klo;
      float sv[32], dp[32];
      tmem_ld32(tlane + L::cS + 32 * chalf, sv);
      tmem_ld32(tlane + L::cDP + 32 * chalf, dp);
#pragma unroll
      for (int c8 = 0; c8 < 4; ++c8) {
        float p8[8], z8[8];
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float p = (unsigned)(off + 8 * c8 + e) <= kspan ? exp2f(fmaf(sv[8 * c8 + e], sc2, nLj)) : 0.f;
          p8[e] = p;
          z8[e] = p * (dp[8 * c8 + e] - delta) * d.scale;
        }
        *reinterpret_cast<uint4*>(sm + L::tP + sw_off(row, 4 * chalf + c8)) = pack8(p8);
        *reinterpret_cast<uint4*>(sm + L::tZ + sw_off(row, 4 * chalf + c8)) = pack8(z8);
      }
    }
    NHA_SMEM_TO_MMA();
    if (tid == 0) {
#pragma unroll
      for (int nb = 0; nb < KT; ++nb) {
        // dv_win += p^T do,  dk_swa += dz^T q_swa   (k = query row: both operands MN-major)
        mma_tile_ex(tbase + L::cDV + 64 * nb, aP, 0, 1, aDO + nb * L::kATile, 0, 1, 64, 64, 8, pr > 0);
        mma_tile_ex(tbase + L::cDK + 64 * nb, aZ, 0, 1, aQS + nb * L::kATile, 0, 1, 64, 64, 8, pr > 0);
      }
    }
    NHA_MMA_WAIT();
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
  }
#undef NHA_MMA_WAIT
#undef NHA_SMEM_TO_MMA
  // ---- two threads per key row (rows of a 64-row product sit in the first 16 lanes of each quarter), each its half
  //      of the columns
  {
    const bool kactive = lane < 16;
    const int krow = quarter * 16 + (lane & 15);
    const int pk = c0 + krow;
    const bool keep = kactive && pk < len && !failed;
    float ov[32];
#pragma unroll
    for (int pp = 0; pp < D / 64; ++pp) {
      const int part = (D / 64) * chalf + pp;
      tmem_ld32(tlane + L::cDK + 32 * part, ov);
      if (keep) {
        bf16* orow = (bf16*)d.dk_swa + ((size_t)(t0 + pk) * H + h) * D + 32 * part;
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) *reinterpret_cast<uint4*>(orow + 8 * c8) = pack8(ov + 8 * c8);
      }
      tmem_ld32(tlane + L::cDV + 32 * part, ov);
      if (keep) {
        float* orow = w.dvacc + ((size_t)(t0 + pk) * H + h) * D + 32 * part;
#pragma unroll
        for (int e = 0; e < 32; e += 4) *reinterpret_cast<float4*>(orow + e) = make_float4(ov[e], ov[e + 1], ov[e + 2], ov[e + 3]);
      }
    }
  }
  if (failed) atomicExch(err, 1);
  cp_wait_all();
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, L::kTmemCols);
}

template <int D>
static int launch_wcols(const nha_chunk_desc* d, const BwdWs& w, int* err, cudaStream_t cs) {
  typedef WColsLayout<D> L;
  cudaError_t e = set_max_smem((const void*)nha_bwd_wcols_umma_kernel<D>, L::total);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  nha_bwd_wcols_umma_kernel<D><<<dim3(NCB, d->H), kWCThreads, L::total, cs>>>(*d, w, err);
  return check_launch();
}

bool bwd_wcols_umma_supported(const nha_chunk_desc* d) { return d->K == d->V && (d->K == 64 || d->K == 128); }

// The caller has checked bwd_wcols_umma_supported().
int bwd_wcols_umma_launch(const nha_chunk_desc* d, const BwdWs& w, int* err, cudaStream_t cs) {
  return d->K == 64 ? launch_wcols<64>(d, w, err, cs) : launch_wcols<128>(d, w, err, cs);
}

}  // namespace nha
