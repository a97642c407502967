// Output pass of the chunked NHA forward for head dim 128 with four (or a multiple of four) query heads per kv head,
// as a warp-specialised pipeline on the sm_100a tensor-core path.
//
// One CTA = one (64-token chunk, kv head, group of four query heads) = two 128-row tiles (two heads x 64 tokens each)
// that share the chunk's slot operands (k', v', Hk, Hv, s' .* b) and every window key / value tile.  352 threads:
//   warps 0-3 / 4-7  softmax group of tile 0 / tile 1: ONE thread per row (tcgen05.ld gives it its row of the
//                    accumulator), element-wise work only;
//   warp 8           loads: all operand tiles by TMA (cp.async.bulk.tensor on maps of this GPU's own tensors, no
//                    multicast) into 128-byte-swizzled tiles, bytes counted on mbarriers; the slot operands and the
//                    window tiles stream through one ring of six 16 KB slots (window keys and values are polled
//                    independently, a slot is refilled as soon as both tiles have read it); a tile that sticks out
//                    of its sequence is written by the warp itself with zero fill, so that no row of a neighbouring
//                    sequence ever enters a product;
//   warp 9 / 10      one thread each issues the tcgen05.mma of tile 0 / tile 1 and commits completions to mbarriers,
//                    so each tile's chain (group hands over -> products -> group continues) runs at its own pace.
// While one tile's group does its element-wise step the tensor pipe works on the other tile:
//     G1  A = q k'^T, QH = q Hk                group: tril(A) -> bf16 operand
//     G2  X = tril(A) (s' .* b)                group: slot logits ok = scale a .* (e^R .* QH + X), p~ = exp(ok - max),
//                                                     operands p~ a e^R and p~ a
//     G3  O = (p~ a e^R) Hv, Bv = (p~ a)(s' .* b)^T      group: tril(Bv) -> bf16 operand
//     G4  O += tril(Bv) v'
//     window steps, newest key tile first (64 keys each):   S_j = q_swa K_j^T (two accumulators, S_{j+2} is issued as
//         soon as the group has read S_j);   group: P~_j = exp(scale S_j - m) written as bf16 pairs over the first 32
//         columns of S_j in tensor memory;   O += P~_j V_j with P~_j as the tensor-memory A operand
// Shared-memory bandwidth is what bounds the tensor pipe here (a 128 x 64 x 16 product reads 6 KB of operands in its
// 32 cycles): the value products therefore take all 128 columns of V at once (an MN-major operand spanning two
// swizzle atoms) and read P~ from tensor memory, which halves their shared-memory traffic.
// ONE softmax over the slot logits and all window logits, in a single sweep: the running reference m of a row starts
// as its slot maximum and is only raised when a window logit exceeds it by more than 8 ln 2 (probabilities then stay
// below 256, exact in the fp32 accumulator); raising it rescales the row of O in tensor memory (tcgen05.ld / st by the
// row's thread, after the products in flight on O have completed).  Decay factorisation, flags for chunks that decay
// too fast for one reference per chunk, and the general kernel that takes those: as in nha_chunk_fwd_umma.cu.
//
// Replaces chunk_nha_fused_o_kernel (nha_fla/ops/nha/chunk_fused.py:117-283) at the long-context shape.
#include <cuda.h>
#include <string.h>

#include "nha_common.cuh"
#include "nha_tma.cuh"
#include "nha_umma.cuh"

namespace nha {

using namespace umma;

namespace pipe {
constexpr int D = 128, M = 64;
constexpr int kThreads = 352;
constexpr int kQTile = 128 * 128;                 // one 64-wide k tile of a 128-row A operand
constexpr int kSlot = 16384, kNSlot = 4;
constexpr int oQG = 0;                            // q_gsa [2 tiles][2 k tiles][128][64]; later tril / p~ operands, P~
constexpr int oQS = oQG + 4 * kQTile;             // q_swa, same shape
constexpr int oRing = oQS + 4 * kQTile;
constexpr int oSB = oRing + kNSlot * kSlot;       // s' .* b [64][64]
constexpr int kLdA = 68;                          // row pitch of the decay table: 16-byte aligned rows, conflict-free float4 reads
constexpr int oA = oSB + 8192;                    // fp32 [64][kLdA]: cumulative gates, then a = exp(G - R)
constexpr int oER = oA + 64 * kLdA * 4;           // fp32 [64] exp(R)
constexpr int oBar = oER + 256;
constexpr int total = oBar + 512 + 1024;          // + slack for the 1024-byte alignment of the base
static_assert(total <= 227 * 1024, "shared memory of the pipelined output pass");
// mbarriers
constexpr int bQ = 0, bFull = 2, bEmpty = 8, bG = 14, bW = 16, bS = 18, bP = 22, bPV = 26, nBar = 28;
constexpr int kPoll = 1 << 20;
constexpr float kDecayLimit = 140.0f;
constexpr float kRaise = 5.545177f;               // 8 ln 2
}  // namespace pipe

// Phase clocks for tuning (a build with -DNHA_PIPE_PROF only): cycles per phase summed over all CTAs, read back with
// nha_debug_pipe_prof().
#ifdef NHA_PIPE_PROF
__device__ unsigned long long g_pipe_prof[64];
__device__ unsigned int g_pipe_trace[4 * 512];       // one CTA's events: (phase id << 24) | cycles since the CTA began
#define PROF_INIT()                                                            \
  long long tp_ = clock64();                                                   \
  const long long tp0_ = tp_;                                                  \
  int tn_ = 0;                                                                 \
  const int trole_ = threadIdx.x == 0 ? 0 : (threadIdx.x == 128 ? 1 : (threadIdx.x == 256 ? 2 : 3));                \
  const bool ttrace_ = blockIdx.x == 40 && blockIdx.y == 0
#define PROF(i_)                                                               \
  do {                                                                         \
    const long long n_ = clock64();                                            \
    if (trole_ != 1) atomicAdd(&g_pipe_prof[i_], (unsigned long long)(n_ - tp_)); \
    if (ttrace_ && tn_ < 511) g_pipe_trace[trole_ * 512 + 1 + tn_++] = ((unsigned)(i_) << 24) | (unsigned)((n_ - tp0_) & 0xffffff); \
    if (ttrace_) g_pipe_trace[trole_ * 512] = tn_;                             \
    tp_ = n_;                                                                  \
  } while (0)
#else
#define PROF_INIT()
#define PROF(i_)
#endif

struct PipeMaps {
  CUtensorMap qg, qs, kg, ks, v, hk, hv;
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const float* in) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};" ::"r"(taddr),
      "r"(__float_as_uint(in[0])), "r"(__float_as_uint(in[1])), "r"(__float_as_uint(in[2])), "r"(__float_as_uint(in[3])),
      "r"(__float_as_uint(in[4])), "r"(__float_as_uint(in[5])), "r"(__float_as_uint(in[6])), "r"(__float_as_uint(in[7])),
      "r"(__float_as_uint(in[8])), "r"(__float_as_uint(in[9])), "r"(__float_as_uint(in[10])), "r"(__float_as_uint(in[11])),
      "r"(__float_as_uint(in[12])), "r"(__float_as_uint(in[13])), "r"(__float_as_uint(in[14])), "r"(__float_as_uint(in[15])),
      "r"(__float_as_uint(in[16])), "r"(__float_as_uint(in[17])), "r"(__float_as_uint(in[18])), "r"(__float_as_uint(in[19])),
      "r"(__float_as_uint(in[20])), "r"(__float_as_uint(in[21])), "r"(__float_as_uint(in[22])), "r"(__float_as_uint(in[23])),
      "r"(__float_as_uint(in[24])), "r"(__float_as_uint(in[25])), "r"(__float_as_uint(in[26])), "r"(__float_as_uint(in[27])),
      "r"(__float_as_uint(in[28])), "r"(__float_as_uint(in[29])), "r"(__float_as_uint(in[30])), "r"(__float_as_uint(in[31]))
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }

__global__ void __launch_bounds__(pipe::kThreads, 1)
    nha_fwd_pipe_kernel(const nha_chunk_desc d, int* __restrict__ flags, int* __restrict__ err,
                        const __grid_constant__ PipeMaps maps) {
  using namespace pipe;
  const int H = d.H, HQ = d.HQ, NG = HQ / H;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  if (rc.n < 0) return;
  const int n = rc.n, ci = rc.ci, t0 = rc.t0, len = rc.len, c0 = ci * kChunk;
  const int wl = seq_window(d, n), shift = seq_shift(d, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hq0 = h * NG + 4 * blockIdx.z;
  PROF_INIT();

  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  float* As = (float*)(sm + oA);
  float* ER = (float*)(sm + oER);
  uint64_t* bar = (uint64_t*)(sm + oBar);
  uint32_t* tslot = (uint32_t*)(bar + nBar);
  __shared__ int s_abort;

  // window key tiles, newest first: step j covers the keys [64 (ci - j), 64 (ci - j) + 64)
  const int jt_lo = wl < 0 ? 0 : max(0, c0 - wl) / kChunk;
  const int nst = ci - jt_lo + 1;
  const int nloads = 4 + 2 * nst;

  if (warp == 9) {
    if (lane < nBar) {
      const bool many = (lane >= bW && lane < bW + 2) || (lane >= bP && lane < bP + 4);
      const bool two = lane >= bEmpty && lane < bEmpty + 6;         // released by both MMA warps
      mbar_init(&bar[lane], many ? 128 : (two ? 2 : 1));
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 31) s_abort = *(volatile int*)err;    // an earlier CTA of this launch gave up on a wait: do not start
  }
  if (warp == 0) tmem_alloc(tslot, 512);
  // gates and write weights of the chunk's shifted rows through registers (threads 0..255: two 16-byte pieces each)
  const int lo = 0, hi = len - shift;
  uint4 sreg[2], greg[2];
  if (tid < 256) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + 256 * j;
      const int r = i >> 3, c8 = i & 7;
      const int src = c0 + r - shift;
      sreg[j] = make_uint4(0u, 0u, 0u, 0u);
      greg[j] = make_uint4(0u, 0u, 0u, 0u);
      if (src >= lo && src < hi) {
        greg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.g + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
        sreg[j] = *reinterpret_cast<const uint4*>((const bf16*)d.s + ((size_t)(t0 + src) * H + h) * M + 8 * c8);
      }
    }
  }
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tslot;
  if (s_abort) {
    if (warp == 0) tmem_dealloc(tbase, 512);
    return;
  }
  if (tid == 0 || tid == 128) PROF(0);
  bool failed = false;
#define NHA_WAIT(idx_, par_)                                                       \
  do {                                                                             \
    if (!failed && !mbar_wait_limit(&bar[idx_], (uint32_t)(par_), kPoll)) failed = true; \
  } while (0)

  // ---- loads (warp 8) ---------------------------------------------------------------------------------------------
  // load 0: k' (shifted un-rotated keys), 1: Hk, 2: Hv, 3: v' (shifted values), 4 + 2 j: window keys of step j,
  // 5 + 2 j: window values of step j; load i goes to ring slot i % 4.
  auto ragged_fill = [&](unsigned char* dst, const bf16* base, int r0, int rlo, int rhi) {
    // [64 rows][128 columns] as two swizzled 64-column tiles; rows outside [rlo, rhi) become zeros
#pragma unroll 1
    for (int it = 0; it < 32; it += 8) {
      uint4 v[8];
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = lane + 32 * (it + u);
        const int r = i >> 4, c = i & 15;
        const int gr = r0 + r;
        v[u] = make_uint4(0u, 0u, 0u, 0u);
        if (gr >= rlo && gr < rhi) v[u] = __ldg(reinterpret_cast<const uint4*>(base + (size_t)gr * H * D + 8 * c));
      }
#pragma unroll
      for (int u = 0; u < 8; ++u) {
        const int i = lane + 32 * (it + u);
        const int r = i >> 4, c = i & 15;
        *reinterpret_cast<uint4*>(dst + (c >> 3) * 8192 + sw_off(r, c & 7)) = v[u];
      }
    }
    fence_async_smem();
    __syncwarp();
  };
  // Ring of six 16 KB slots: slots 0-3 lie in their own region, slots 4 and 5 are the second operand tile (p~ a e^R)
  // of tile 0 and tile 1, free once the product that reads it (G3 of that tile) has completed.  The slot operands
  // (loads 0-3) use slots 0-3; window keys of step j use slot 2 (j % 3), window values slot 2 (j % 3) + 1.
  auto slot_ptr = [&](int slot) { return sm + (slot < 4 ? oRing + slot * kSlot : oQG + (2 * (slot - 4) + 1) * kQTile); };
  auto slot_of = [&](int idx) { return idx < 4 ? idx : 2 * (((idx - 4) >> 1) % 3) + (idx & 1); };
  auto issue_load = [&](int idx) {
    const int slot = slot_of(idx);
    unsigned char* dst = slot_ptr(slot);
    uint64_t* fb = &bar[bFull + slot];
    if (idx == 1) {
      if (lane == 0) {
        mbar_expect_tx(fb, 16384);
        tma_load_2d(dst, &maps.hk, 0, (cg * H + h) * D, fb);
      }
      return;
    }
    if (idx == 2) {
      if (lane == 0) {
        mbar_expect_tx(fb, 16384);
        tma_load_2d(dst, &maps.hv, 0, (cg * H + h) * M, fb);
        tma_load_2d(dst + 8192, &maps.hv, 64, (cg * H + h) * M, fb);
      }
      return;
    }
    const CUtensorMap* mp;
    const bf16* base;
    int r0, rlo = 0, rhi;
    if (idx == 0) { mp = &maps.kg; base = (const bf16*)d.k_gsa; r0 = c0 - shift; rhi = hi; }
    else if (idx == 3) { mp = &maps.v; base = (const bf16*)d.v; r0 = c0 - shift; rhi = hi; }
    else {
      const int j = (idx - 4) >> 1;
      r0 = (ci - j) * kChunk;
      rhi = len;
      if ((idx & 1) == 0) { mp = &maps.ks; base = (const bf16*)d.k_swa; }
      else { mp = &maps.v; base = (const bf16*)d.v; }
    }
    if (r0 >= rlo && r0 + kChunk <= rhi) {
      if (lane == 0) {
        mbar_expect_tx(fb, 16384);
        tma_load_3d(dst, mp, 0, h, t0 + r0, fb);
        tma_load_3d(dst + 8192, mp, 64, h, t0 + r0, fb);
      }
    } else {
      ragged_fill(dst, base + ((size_t)t0 * H + h) * D, r0, rlo, rhi);
      if (lane == 0) mbar_arrive(fb);
    }
  };
  if (warp == 8) {
    if (lane == 0) {
#pragma unroll
      for (int t = 0; t < 2; ++t) {
        mbar_expect_tx(&bar[bQ + t], 65536);
#pragma unroll
        for (int hh = 0; hh < 2; ++hh)
#pragma unroll
          for (int kt = 0; kt < 2; ++kt) {
            tma_load_3d(sm + oQG + (2 * t + kt) * kQTile + hh * 8192, &maps.qg, 64 * kt, hq0 + 2 * t + hh, t0 + c0, &bar[bQ + t]);
            tma_load_3d(sm + oQS + (2 * t + kt) * kQTile + hh * 8192, &maps.qs, 64 * kt, hq0 + 2 * t + hh, t0 + c0, &bar[bQ + t]);
          }
      }
    }
    for (int idx = 0; idx < 4; ++idx) issue_load(idx);
  }

  // ---- decay tables (threads 0..255), as in nha_chunk_fwd_umma.cu -------------------------------------------------
  if (tid < 256) {
#pragma unroll
    for (int j = 0; j < 2; ++j) {
      const int i = tid + 256 * j;
      const int r = i >> 3, c8 = i & 7;
      float gv[8];
      unpack8(greg[j], gv);
#pragma unroll
      for (int e = 0; e < 8; ++e) As[r * kLdA + 8 * c8 + e] = gv[e];
    }
  }
  __syncthreads();
  {
    // inclusive scan along the rows: four threads per column (16 rows each), then the totals of the earlier segments
    const int m = tid & 63, seg = tid >> 6;
    if (tid < 256) {
      float run = 0.f;
#pragma unroll
      for (int r = 16 * seg; r < 16 * seg + 16; ++r) {
        run += As[r * kLdA + m];
        As[r * kLdA + m] = run;
      }
    }
    __syncthreads();
    float add = 0.f;
    if (tid < 256)
      for (int s2 = 0; s2 < seg; ++s2) add += As[(16 * s2 + 15) * kLdA + m];
    __syncthreads();
    if (tid < 256 && seg > 0) {
#pragma unroll
      for (int r = 16 * seg; r < 16 * seg + 16; ++r) As[r * kLdA + m] += add;
    }
    __syncthreads();
  }
  const bool mine_unsafe = tid < 64 && fabsf(As[63 * kLdA + tid]) > kDecayLimit;
  const int unsafe = __syncthreads_or(mine_unsafe ? 1 : 0);
  if (tid == 0 && blockIdx.z == 0) flags[(size_t)cg * H + h] = unsafe;
  if (unsafe) {
    // the general kernel computes this chunk; the loads already in flight must land before the CTA may leave
    if (warp == 8 && lane == 0) {
      NHA_WAIT(bQ, 0);
      NHA_WAIT(bQ + 1, 0);
      for (int i = 0; i < 4; ++i) NHA_WAIT(bFull + i, 0);
      if (failed) atomicExch(err, 1);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, 512);
    return;
  }
  {
    float rref[8];
    const int c8 = tid & 7;
    if (tid < 256) {
#pragma unroll
      for (int e = 0; e < 8; ++e) rref[e] = 0.5f * As[63 * kLdA + 8 * c8 + e];
    }
    __syncthreads();                                  // every thread holds its references before the table changes
    if (tid < 8) {
#pragma unroll
      for (int e = 0; e < 8; ++e) ER[8 * tid + e] = __expf(rref[e]);
    }
    if (tid < 256) {
#pragma unroll
      for (int j = 0; j < 2; ++j) {
        const int i = tid + 256 * j;
        const int r = i >> 3;
        float sv[8], out[8];
        unpack8(sreg[j], sv);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const float x = As[r * kLdA + 8 * c8 + e] - rref[e];
          As[r * kLdA + 8 * c8 + e] = __expf(x);
          out[e] = sv[e] * __expf(-x);
        }
        *reinterpret_cast<uint4*>(sm + oSB + sw_off(r, c8)) = pack8(out);
      }
    }
    fence_async_smem();
    __syncthreads();
  }

  if (tid == 0 || tid == 128) PROF(1);
  if (tid == 256) PROF(24);
  if (tid == 288) PROF(16);
  const uint32_t aSB = smem_u32(sm + oSB);
  if (warp == 8) {
    // ================= load warp: the rest of the ring ============================================================
    // Window keys go through slots 0, 2, 4, values through slots 1, 3, 5; every slot has had one earlier occupant (a
    // slot operand, or a tile's p~ a e^R), so step j waits for release number j / 3 + 1 of its slot.  A key tile is
    // released as soon as both tiles' S products have read it, long before the value tile of the same step, so the
    // two sequences are polled side by side: whichever next load finds its slot free is issued.
    int kn = 0, vn = 0, spins = 0;
    while (kn < nst || vn < nst) {
      bool did = false;
      if (kn < nst) {
        const int idx = 4 + 2 * kn;
        const int free_ = lane == 0 ? (int)mbar_test(&bar[bEmpty + slot_of(idx)], (kn / 3) & 1) : 0;
        if (__shfl_sync(0xffffffffu, free_, 0)) {
          issue_load(idx);
          ++kn;
          did = true;
        }
      }
      if (vn < nst) {
        const int idx = 5 + 2 * vn;
        const int free_ = lane == 0 ? (int)mbar_test(&bar[bEmpty + slot_of(idx)], (vn / 3) & 1) : 0;
        if (__shfl_sync(0xffffffffu, free_, 0)) {
          issue_load(idx);
          ++vn;
          did = true;
        }
      }
      if (did) spins = 0;
      else __nanosleep(64);
      if (!did && ++spins > kPoll) {                        // nothing was released for a very long time: give up
        failed = true;
        break;
      }
    }
    if (lane == 0) PROF(25);
  } else if (warp >= 9) {
    // ================= MMA warps: warp 9 issues for tile 0, warp 10 for tile 1 (one thread each) ====================
    // Each tile's chain (group hands over -> products issued -> group continues) then runs at its own pace; a ring slot
    // is released when BOTH issuers have committed behind their last product that reads it (barrier count 2).
    if (lane == 0) {
      const int t = warp - 9;
      auto ring = [&](int idx) { return smem_u32(slot_ptr(slot_of(idx))); };
      constexpr uint32_t kT16 = kQTile >> 4;             // k-tile pitch of a 128-row A operand, in descriptor units
      const uint32_t iK = make_idesc(128, 64, 0), iMN = make_idesc(128, 64, 1), iMN128 = make_idesc(128, 128, 1);
      const uint64_t dSB = make_desc(aSB);
      const uint64_t dQG = make_desc(smem_u32(sm + oQG + 2 * t * kQTile));
      const uint64_t dQS = make_desc(smem_u32(sm + oQS + 2 * t * kQTile));
      const uint32_t tt = tbase + 256 * t;               // S0 at +0, S1 at +64, O at +128
      auto wait_full = [&](int idx) {
        // fill number of the slot: slots 0-3 were filled once by the slot operands before the window tiles
        const int slot = slot_of(idx);
        const int fills = idx < 4 ? 0 : ((idx - 4) >> 1) / 3 + (slot < 4 ? 1 : 0);
        NHA_WAIT(bFull + slot, fills & 1);
        tc_fence_after();
      };
      auto s_mma = [&](int j) {          // S_j into accumulator j & 1 (window keys = load 4 + 2 j), then release the keys
        wait_full(4 + 2 * j);
        mma_run<8, 0>(tt + 64 * (j & 1), dQS, kT16, make_desc(ring(4 + 2 * j)), 8192 >> 4, iK, false);
        commit(&bar[bS + 2 * t + (j & 1)]);
        commit(&bar[bEmpty + slot_of(4 + 2 * j)]);
      };
      uint32_t wph = 0u;
      // G1: A = q k'^T, QH = q Hk
      NHA_WAIT(bQ + t, 0);
      wait_full(0);
      wait_full(1);
      PROF(17);
      mma_run<8, 0>(tt, dQG, kT16, make_desc(ring(0)), 8192 >> 4, iK, false);
      mma_run<8, 1>(tt + 64, dQG, kT16, make_desc(ring(1)), 0, iMN, false);
      commit(&bar[bG + t]);
      commit(&bar[bEmpty + 0]);
      commit(&bar[bEmpty + 1]);
      PROF(18);
      // G2: X = tril(A) (s' .* b)
      NHA_WAIT(bW + t, wph); wph ^= 1u;
      tc_fence_after();
      PROF(19);
      mma_run<4, 1>(tt, dQG, kT16, dSB, 0, iMN, false);
      commit(&bar[bG + t]);
      PROF(18);
      // G3: O = (p~ a e^R) Hv over all 128 columns (the two 64-column tiles of Hv are 8192 bytes apart), Bv = (p~ a) SB^T
      NHA_WAIT(bW + t, wph); wph ^= 1u;
      PROF(19);
      wait_full(2);
      PROF(17);
      mma_run<4, 1>(tt + 128, dQG + kT16, 0, make_desc_lbo(ring(2), 8192), 0, iMN128, false);
      mma_run<4, 0>(tt + 64, dQG, 0, dSB, 0, iK, false);
      commit(&bar[bG + t]);
      commit(&bar[bEmpty + 2]);
      commit(&bar[bEmpty + 4 + t]);                      // this tile's p~ a e^R operand becomes ring slot 4 + t:
      commit(&bar[bEmpty + 4 + t]);                      // nobody else reads it, so this issuer gives both arrivals
      PROF(18);
      s_mma(0);                                          // S0 is free: QH and X have been read
      PROF(18);
      // G4: O += tril(Bv) v'
      NHA_WAIT(bW + t, wph); wph ^= 1u;
      PROF(19);
      wait_full(3);
      PROF(17);
      mma_run<4, 1>(tt + 128, dQG, 0, make_desc_lbo(ring(3), 8192), 0, iMN128, true);
      commit(&bar[bG + t]);
      commit(&bar[bEmpty + 3]);
      PROF(18);
      if (nst > 1) s_mma(1);                             // S1 is free: Bv has been read
      PROF(18);
      // window steps: O += P~_j V_j with P~_j read from tensor memory (the group wrote it over the first 32 columns of
      // S_j), then S_{j+2} into the accumulator the group has just finished with
      for (int j = 0; j < nst; ++j) {
        const int b = j & 1;
        NHA_WAIT(bP + 2 * t + b, (j >> 1) & 1);
        PROF(20);
        wait_full(5 + 2 * j);
        PROF(21);
        {
          const uint64_t dV = make_desc_lbo(ring(5 + 2 * j), 8192);
          const uint32_t aP = tt + 64 * b;
#pragma unroll
          for (int ks = 0; ks < 4; ++ks) mma_f16_ta(tt + 128, aP + 8 * ks, dV + (uint64_t)(ks * 128), iMN128, true);
        }
        commit(&bar[bPV + t]);
        commit(&bar[bEmpty + slot_of(5 + 2 * j)]);
        PROF(22);
        if (j + 2 < nst) s_mma(j + 2);
        PROF(22);
      }
    }
  } else {
    // ================= softmax groups: tile t = warp / 4, one thread per row =======================================
    const int t = warp >> 2, quarter = warp & 3;
    const int row = quarter * 32 + lane;
    const int tk = row & 63, th = row >> 6;
    const int pos = c0 + tk;
    const bool in_seq = pos < len;
    const int hq = hq0 + 2 * t + th;
    const uint32_t tl = tbase + ((uint32_t)(quarter * 32) << 16) + 256 * t;   // S0 at +0, S1 at +64, O at +128
    unsigned char* opA = sm + oQG + 2 * t * kQTile;      // tril(A) / p~ a / tril(Bv); then P~ of every window step
    unsigned char* opB = opA + kQTile;                   // p~ a e^R (afterwards a slot of the operand ring)
    constexpr float kLog2e = 1.4426950408889634f;
    const int klo = in_seq ? (wl < 0 ? 0 : max(0, pos - wl)) : (1 << 30);
    const unsigned kspan = in_seq ? (unsigned)(pos - klo) : 0u;
    const float sc2 = d.scale * kLog2e;
    uint32_t gph = 0u;
    const float* arow = As + tk * kLdA;
    // one lane of a warp polls a barrier, the others wait at the warp barrier: far fewer shared-memory polls
#define NHA_WAIT_WARP(idx_, par_)                        \
  do {                                                   \
    if (lane == 0) NHA_WAIT(idx_, par_);                 \
    __syncwarp();                                        \
  } while (0)
    // this thread's row of tril of a [128][64] accumulator (token tk keeps columns i <= tk) -> bf16 A-operand tile
    auto tril_to = [&](uint32_t col0, unsigned char* dst) {
      float v[32];
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        tmem_ld32(tl + col0 + 32 * half, v);
#pragma unroll
        for (int c8 = 0; c8 < 4; ++c8) {
          float o8[8];
#pragma unroll
          for (int e = 0; e < 8; ++e) o8[e] = (32 * half + 8 * c8 + e) <= tk ? v[8 * c8 + e] : 0.f;
          *reinterpret_cast<uint4*>(dst + sw_off(row, 4 * half + c8)) = pack8(o8);
        }
      }
    };
    auto hand_over = [&](int b_) {
      fence_async_smem();
      tc_fence_before();
      mbar_arrive(&bar[b_]);
    };
    // G1 -> tril(A)
    NHA_WAIT_WARP(bG + t, gph); gph ^= 1u;
    tc_fence_after();
    if (tid == 0 || tid == 128) PROF(2);
    tril_to(0, opA);
    hand_over(bW + t);
    if (tid == 0 || tid == 128) PROF(3);
    // G2 -> slot logits, p~, operands
    NHA_WAIT_WARP(bG + t, gph); gph ^= 1u;
    tc_fence_after();
    if (tid == 0 || tid == 128) PROF(4);
    float mg, lg0;
    {
      float ok[64];
      tmem_ld64(tl + 64, ok);
      float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
#pragma unroll
      for (int half = 0; half < 2; ++half) {
        float x[32];
        tmem_ld32(tl + 32 * half, x);
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int m = 32 * half + 4 * q;
          const float4 a4 = *reinterpret_cast<const float4*>(arow + m);
          const float4 e4 = *reinterpret_cast<const float4*>(ER + m);
          ok[m] = d.scale * a4.x * (e4.x * ok[m] + x[4 * q]);
          ok[m + 1] = d.scale * a4.y * (e4.y * ok[m + 1] + x[4 * q + 1]);
          ok[m + 2] = d.scale * a4.z * (e4.z * ok[m + 2] + x[4 * q + 2]);
          ok[m + 3] = d.scale * a4.w * (e4.w * ok[m + 3] + x[4 * q + 3]);
          m4[0] = fmaxf(m4[0], ok[m]); m4[1] = fmaxf(m4[1], ok[m + 1]);
          m4[2] = fmaxf(m4[2], ok[m + 2]); m4[3] = fmaxf(m4[3], ok[m + 3]);
        }
      }
      mg = fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
      const float nmg = -mg * kLog2e;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8) {
        float pg8[8], pa8[8], a8[8], e8[8];
        *reinterpret_cast<float4*>(a8) = *reinterpret_cast<const float4*>(arow + 8 * c8);
        *reinterpret_cast<float4*>(a8 + 4) = *reinterpret_cast<const float4*>(arow + 8 * c8 + 4);
        *reinterpret_cast<float4*>(e8) = *reinterpret_cast<const float4*>(ER + 8 * c8);
        *reinterpret_cast<float4*>(e8 + 4) = *reinterpret_cast<const float4*>(ER + 8 * c8 + 4);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          const int m = 8 * c8 + e;
          const float p = exp2f(fmaf(ok[m], kLog2e, nmg));
          l4[e & 3] += p;
          const float pa = in_seq ? p * a8[e] : 0.f;
          pa8[e] = pa;
          pg8[e] = pa * e8[e];
        }
        *reinterpret_cast<uint4*>(opA + sw_off(row, c8)) = pack8(pa8);
        *reinterpret_cast<uint4*>(opB + sw_off(row, c8)) = pack8(pg8);
      }
      lg0 = (l4[0] + l4[1]) + (l4[2] + l4[3]);
    }
    hand_over(bW + t);
    if (tid == 0 || tid == 128) PROF(5);
    // G3 -> tril(Bv)
    NHA_WAIT_WARP(bG + t, gph); gph ^= 1u;
    tc_fence_after();
    if (tid == 0 || tid == 128) PROF(6);
    tril_to(64, opA);
    hand_over(bW + t);
    if (tid == 0 || tid == 128) PROF(7);
    // G4: the operand tiles are free for the P~ tiles from here on
    NHA_WAIT_WARP(bG + t, gph); gph ^= 1u;
    tc_fence_after();
    if (tid == 0 || tid == 128) PROF(8);

    float mref = mg;            // reference of the unnormalised probabilities of this row
    float lgs = lg0;            // slot sum, in units of exp(-mref)
    float ls = 0.f;             // window sum, same units
    int pvseen = 0;
    // observe the completions of P~ V of steps 0 .. upto-1 (one barrier per tile, read phase by phase: P~ V of step j
    // is only issued after this group has handed over P~_j, so the barrier is never more than one phase ahead)
    auto wait_pv = [&](int upto) {
      while (pvseen < upto) {
        NHA_WAIT_WARP(bPV + t, pvseen & 1);
        ++pvseen;
      }
    };
    for (int j = 0; j < nst; ++j) {
      const int b = j & 1;
      NHA_WAIT_WARP(bS + 2 * t + b, (j >> 1) & 1);
      tc_fence_after();
      if (tid == 0 || tid == 128) PROF(9);
      float s[64];
      tmem_ld64(tl + 64 * b, s);
      const int kb = (ci - j) * kChunk;
      const int off = kb - klo;
      // the diagonal tile (causal edge) and tiles that reach below the oldest visible key of the chunk's last row need
      // the per-element test; every row of the chunk sees all keys of the tiles in between
      const bool masked = j == 0 || (wl >= 0 && kb < c0 + kChunk - 1 - wl) || c0 + kChunk > len;
      {
        float m4[4] = {-INFINITY, -INFINITY, -INFINITY, -INFINITY};
        if (masked) {
#pragma unroll
          for (int e = 0; e < 64; ++e) m4[e & 3] = fmaxf(m4[e & 3], (unsigned)(off + e) <= kspan ? s[e] : -INFINITY);
        } else {
#pragma unroll
          for (int e = 0; e < 64; ++e) m4[e & 3] = fmaxf(m4[e & 3], s[e]);
        }
        const float mc = d.scale * fmaxf(fmaxf(m4[0], m4[1]), fmaxf(m4[2], m4[3]));
        const bool raise = mc > mref + kRaise;
        float f = 1.f;
        if (raise) {
          f = __expf(mref - mc);
          mref = mc;
        }
        if (__any_sync(0xffffffffu, raise)) {
          // rescale this warp's rows of O: everything issued on O so far must have completed
          wait_pv(j);
          tc_fence_after();
#pragma unroll 1
          for (int q4 = 0; q4 < 4; ++q4) {
            float ov[32];
            tmem_ld32(tl + 128 + 32 * q4, ov);
#pragma unroll
            for (int e = 0; e < 32; ++e) ov[e] *= f;
            tmem_st32(tl + 128 + 32 * q4, ov);
          }
          tmem_st_wait();
          lgs *= f;
          ls *= f;
        }
      }
      if (tid == 0 || tid == 128) PROF(10);
      if (tid == 0 || tid == 128) PROF(11);
      const float nm = -mref * kLog2e;
      float l4[4] = {0.f, 0.f, 0.f, 0.f};
      if (masked) {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          s[e] = (unsigned)(off + e) <= kspan ? exp2f(fmaf(s[e], sc2, nm)) : 0.f;
          l4[e & 3] += s[e];
        }
      } else {
#pragma unroll
        for (int e = 0; e < 64; ++e) {
          s[e] = exp2f(fmaf(s[e], sc2, nm));
          l4[e & 3] += s[e];
        }
      }
      if (tid == 0 || tid == 128) PROF(27);
      {
        // P~_j as bf16 pairs over the first 32 columns of S_j: the A operand of the value product
        float pk[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) {
          const __nv_bfloat162 h2 = __floats2bfloat162_rn(s[2 * e], s[2 * e + 1]);
          pk[e] = __uint_as_float(*reinterpret_cast<const uint32_t*>(&h2));
        }
        tmem_st32(tl + 64 * b, pk);
        tmem_st_wait();
      }
      if (tid == 0 || tid == 128) PROF(28);
      ls += (l4[0] + l4[1]) + (l4[2] + l4[3]);
      // Every completion phase of the value products is observed before the next one can happen: P~ V of step j is only
      // issued after this hand-over, so seeing step j - 1 complete here (it was issued a whole step ago) keeps the
      // barrier at most one phase ahead of what this thread has seen.
      wait_pv(j);
      tc_fence_before();
      mbar_arrive(&bar[bP + 2 * t + b]);
      if (tid == 0 || tid == 128) PROF(12);
    }
    wait_pv(nst);
    tc_fence_after();
    if (tid == 0 || tid == 128) PROF(13);
    const float lsum = lgs + ls;
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    if (in_seq) {
      d.lse_gsa[(size_t)(t0 + pos) * HQ + hq] = mg + __logf(lg0);
      d.lse_swa[(size_t)(t0 + pos) * HQ + hq] = mref + __logf(ls);
    }
    // Output rows leave through shared memory: a thread holds one whole row (256 bytes), and stores of 32 lanes to 32
    // rows 8 KB apart would cost one memory transaction per lane.  The rows are staged in this tile's q_swa tiles (dead:
    // every S product has completed) with the 16-byte pieces of a row rotated by the row index (no bank conflicts), and
    // each warp then writes its own 32 rows, two whole rows per instruction.
    unsigned char* stage = sm + oQS + 2 * t * kQTile + (size_t)(quarter * 32) * 256;     // this warp's 32 rows
#pragma unroll 1
    for (int q2 = 0; q2 < 2; ++q2) {
      float ov[64];
      tmem_ld64(tl + 128 + 64 * q2, ov);
#pragma unroll
      for (int e = 0; e < 64; ++e) ov[e] *= inv;
#pragma unroll
      for (int c8 = 0; c8 < 8; ++c8)
        *reinterpret_cast<uint4*>(stage + lane * 256 + (((8 * q2 + c8) ^ (lane & 15)) << 4)) = pack8(ov + 8 * c8);
    }
    __syncwarp();
    {
      const int half = lane >> 4, c = lane & 15;          // two rows per instruction, 16 pieces of 16 bytes per row
#pragma unroll 4
      for (int i = 0; i < 16; ++i) {
        const int r = 2 * i + half;                       // row of this warp
        const int rr = quarter * 32 + r;                  // row of the tile
        const int p2 = c0 + (rr & 63);
        if (p2 < len) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((c ^ (r & 15)) << 4));
          bf16* dst = (bf16*)d.o + ((size_t)(t0 + p2) * HQ + hq0 + 2 * t + (rr >> 6)) * D + 8 * c;
          *reinterpret_cast<uint4*>(dst) = v;
        }
      }
    }
  }
  if (tid == 0 || tid == 128) PROF(14);
#undef NHA_WAIT_WARP
#undef NHA_WAIT
  if (failed) atomicExch(err, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, 512);
}

#ifdef NHA_PIPE_PROF
}  // namespace nha
extern "C" int nha_debug_pipe_prof(unsigned long long* out, int reset) {
  cudaError_t e = cudaMemcpyFromSymbol(out, nha::g_pipe_prof, sizeof(unsigned long long) * 64);
  if (e == cudaSuccess && reset) {
    unsigned long long z[64] = {0};
    e = cudaMemcpyToSymbol(nha::g_pipe_prof, z, sizeof(z));
  }
  return e == cudaSuccess ? 0 : 4;
}
extern "C" int nha_debug_pipe_trace(unsigned int* out) {
  return cudaMemcpyFromSymbol(out, nha::g_pipe_trace, sizeof(unsigned int) * 4 * 512) == cudaSuccess ? 0 : 4;
}
namespace nha {
#endif

bool fwd_pipe_supported(const nha_chunk_desc* d) {
  const int NG = d->HQ / d->H;
  if (d->K != 128 || d->V != 128 || d->M != 64 || NG % 4 != 0 || !(d->scale > 0.f)) return false;
  const char* off = getenv("NHA_B200_NO_PIPE");
  return !(off && off[0] == '1');
}

// Launches the pipelined output pass; NHA_ERR_UNSUPPORTED when the tensor maps cannot be made (the caller then takes
// the non-pipelined tensor-memory kernel).
int fwd_pipe_launch(const nha_chunk_desc* d, int* flags, int* err, cudaStream_t cs) {
  using namespace pipe;
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  PipeMaps maps;
  memset(&maps, 0, sizeof(maps));
  const bool ok = make_map_rows_heads(&maps.qg, d->q_gsa, d->Ttot, d->HQ, D) &&
                  make_map_rows_heads(&maps.qs, d->q_swa, d->Ttot, d->HQ, D) &&
                  make_map_rows_heads(&maps.kg, d->k_gsa, d->Ttot, d->H, D) &&
                  make_map_rows_heads(&maps.ks, d->k_swa, d->Ttot, d->H, D) &&
                  make_map_rows_heads(&maps.v, d->v, d->Ttot, d->H, D) &&
                  make_map_matrix(&maps.hk, d->hk_chunks, (int64_t)NCB * d->H * D, M, 128) &&
                  make_map_matrix(&maps.hv, d->hv_chunks, (int64_t)NCB * d->H * M, D, 64);
  if (!ok) return NHA_ERR_UNSUPPORTED;
  cudaError_t e = set_max_smem((const void*)nha_fwd_pipe_kernel, total);
  if (e != cudaSuccess) return record_cuda_error(e);
  nha_fwd_pipe_kernel<<<dim3(NCB, d->H, d->HQ / d->H / 4), kThreads, total, cs>>>(*d, flags, err, maps);
  return check_launch();
}

}  // namespace nha
