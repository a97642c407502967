// Output pass of the chunked NHA forward for head dim 128 with an even number of query heads per kv head, as a
// warp-specialised pipeline on the sm_100a tensor-core path.
//
// One CTA = one 128-row tile: a 64-token chunk of TWO query heads of one kv head.  192 threads and about 107 KB of
// shared memory, so that TWO CTAs share an SM: while one of them runs its prologue, its slot phase (a chain of four
// short product groups with element-wise work in between) or its epilogue, the other keeps the tensor pipe and the
// exponential unit busy with window steps.  Roles:
//   warps 0-3   softmax group: ONE thread per row (tcgen05.ld gives it its row of an accumulator); element-wise work
//               only.  Everything it hands to the tensor pipe is written back into TENSOR MEMORY as bf16 pairs
//               (tcgen05.st) and read from there as the A operand of the next product, so it never stores an operand
//               to shared memory;
//   warp 4      loads: every operand tile by TMA (cp.async.bulk.tensor on maps of this GPU's own tensors, no
//               multicast) into 128-byte-swizzled tiles, bytes counted on mbarriers; q_gsa, the slot operands and the
//               window tiles stream through a ring of 16 KB slots (three, and the decay table's storage as a fourth
//               once the table is dead); window keys and values are polled independently, a slot is refilled as soon as
//               the product that read it has completed; a tile that sticks out of its sequence is written by the
//               warp itself with zero fill, so that no row of a neighbouring sequence ever enters a product;
//   warp 5      one thread issues every tcgen05.mma and commits completions to mbarriers.
// Products of a tile (S0, S1: two 64-column accumulators; O: the 128-column output accumulator):
//     G1  A = q k'^T -> S0, QH = q Hk -> S1          group: tril(A) -> bf16 in O's first columns
//     G2  X = tril(A) (s' .* b) -> S0                group: slot logits ok = scale a .* (e^R .* QH + X), p~ = exp(ok - max),
//                                                            p~ a e^R and p~ a -> bf16 in S0
//     G3  O = (p~ a e^R) Hv, Bv = (p~ a)(s' .* b)^T -> S1      group: tril(Bv) -> bf16 in S1
//     G4  O += tril(Bv) v'
//     window steps, newest key tile first (64 keys each):   S_j = q_swa K_j^T into S(j & 1) (S_{j+2} is issued as soon
//         as the group has read S_j);   group: P~_j = exp(scale S_j - m) -> bf16 over the first 32 columns of S_j;
//         O += P~_j V_j
// Shared-memory bandwidth is what bounds the tensor pipe here (a 128 x 64 x 16 product reads 6 KB of operands in its
// 32 cycles): the value products therefore take all 128 columns of V at once (an MN-major operand spanning two
// swizzle atoms) and every A operand but q comes from tensor memory.
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
constexpr int kThreads = 192;
constexpr int kQTile = 128 * 128;                 // one 64-wide k tile of a 128-row A operand
constexpr int kSlot = 16384;
constexpr int kLdA = 68;                          // row pitch of the decay table: 16-byte aligned rows, conflict-free float4 reads
constexpr int oQS = 0;                            // q_swa [2 k tiles][128][64]; at the end the staging of the output rows
constexpr int oRing = oQS + 2 * kQTile;           // ring slots 0-2
constexpr int oA = oRing + 3 * kSlot;             // fp32 [64][kLdA]: cumulative gates, then a = exp(G - R); later ring slot 3
constexpr int oSB = oA + 64 * kLdA * 4;           // s' .* b [64][64]
constexpr int oER = oSB + 8192;                   // fp32 [64] exp(R)
constexpr int oBar = oER + 256;
constexpr int total = oBar + 256 + 1024;          // + slack for the 1024-byte alignment of the base
static_assert(64 * kLdA * 4 >= kSlot, "the decay table's storage doubles as a ring slot");
static_assert(total <= 113 * 1024, "two CTAs of the pipelined output pass per SM");
// mbarriers
constexpr int bQ = 0, bFull = 1, bEmpty = 5, bTab = 9, bG = 10, bW = 11, bS = 12, bP = 14, bPV = 16, bKq = 17, nBar = 18;
constexpr int kPoll = 1 << 15;                    // polls of a bounded wait (each sleeps up to 20 us in hardware)
constexpr float kDecayLimit = 140.0f;
constexpr float kRaise = 5.545177f;               // 8 ln 2
constexpr int kTmemCols = 256;
}  // namespace pipe

struct PipeMaps {
  CUtensorMap qg, qs, kg, ks, v, hk, hv;
};

__device__ __forceinline__ void tmem_st32(uint32_t taddr, const uint32_t* in) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x32.b32 [%0], "
      "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,"
      "%31,%32};" ::"r"(taddr),
      "r"(in[0]), "r"(in[1]), "r"(in[2]), "r"(in[3]), "r"(in[4]), "r"(in[5]), "r"(in[6]), "r"(in[7]), "r"(in[8]), "r"(in[9]),
      "r"(in[10]), "r"(in[11]), "r"(in[12]), "r"(in[13]), "r"(in[14]), "r"(in[15]), "r"(in[16]), "r"(in[17]), "r"(in[18]),
      "r"(in[19]), "r"(in[20]), "r"(in[21]), "r"(in[22]), "r"(in[23]), "r"(in[24]), "r"(in[25]), "r"(in[26]), "r"(in[27]),
      "r"(in[28]), "r"(in[29]), "r"(in[30]), "r"(in[31])
      : "memory");
}
__device__ __forceinline__ void tmem_st16(uint32_t taddr, const uint32_t* in) {
  asm volatile(
      "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], {%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
      "r"(in[0]), "r"(in[1]), "r"(in[2]), "r"(in[3]), "r"(in[4]), "r"(in[5]), "r"(in[6]), "r"(in[7]), "r"(in[8]), "r"(in[9]),
      "r"(in[10]), "r"(in[11]), "r"(in[12]), "r"(in[13]), "r"(in[14]), "r"(in[15])
      : "memory");
}
__device__ __forceinline__ void tmem_st_wait() { asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory"); }
__device__ __forceinline__ uint32_t bf16_pair(float lo, float hi) {
  const __nv_bfloat162 h2 = __floats2bfloat162_rn(lo, hi);
  return *reinterpret_cast<const uint32_t*>(&h2);
}

__global__ void __launch_bounds__(pipe::kThreads, 2)
    nha_fwd_pipe_kernel(const nha_chunk_desc d, int* __restrict__ flags, int* __restrict__ err,
                        const __grid_constant__ PipeMaps maps) {
  using namespace pipe;
  const int H = d.H, HQ = d.HQ, NG = HQ / H;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  if (rc.n < 0) return;
  const int n = rc.n, ci = rc.ci, t0 = rc.t0, len = rc.len, c0 = ci * kChunk;
  if (c0 < d.q_offset) return;                     // chunks below q_offset have no queries (q_offset is a multiple of 64)
  const int tq0 = t0 - d.q_offset;                 // row of q / o / lse that holds position 0 of the sequence
  const int wl = seq_window(d, n), shift = seq_shift(d, n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int hq0 = h * NG + 2 * blockIdx.z;

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

  if (warp == 5) {
    if (lane < nBar) {
      const bool many = lane == bTab || lane == bW || lane == bP || lane == bP + 1;
      mbar_init(&bar[lane], many ? 128 : 1);
    }
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    if (lane == 31) s_abort = *(volatile int*)err;    // an earlier CTA of this launch gave up on a wait: do not start
  }
  if (warp == 0) tmem_alloc(tslot, kTmemCols);
  // gates and write weights of the chunk's shifted rows through registers (threads 0..127: four 16-byte pieces each)
  const int lo = 0, hi = len - shift;
  uint4 sreg[4], greg[4];
  if (tid < 128) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + 128 * j;
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
    if (warp == 0) tmem_dealloc(tbase, kTmemCols);
    return;
  }
  bool failed = false;
#define NHA_WAIT(idx_, par_)                                                       \
  do {                                                                             \
    if (!failed && !mbar_wait_limit(&bar[idx_], (uint32_t)(par_), kPoll)) failed = true; \
  } while (0)

  // ---- loads (warp 4) ---------------------------------------------------------------------------------------------
  // Ring slots and what passes through them, in fill order:
  //   slot 0: q_gsa k tile 0, Hv, window values of the even steps      slot 1: q_gsa k tile 1, v', window keys of the odd steps
  //   slot 2: Hk, window keys of the even steps (k' passes through the q_swa tiles)                    slot 3 (the decay table's storage): values of the odd steps
  // Fill number f of a slot waits for release number f - 1 of that slot (a commit of the MMA thread behind the last
  // product that read it); the first fill of slot 3 waits for the softmax group to have finished with the table.
  auto slot_ptr = [&](int slot) { return sm + (slot < 3 ? oRing + slot * kSlot : oA); };
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
  // rows [r0, r0 + 64) of one kv head of a [tokens][H][128] tensor into a slot: by TMA when they lie inside [rlo, rhi)
  auto load_rows_to = [&](unsigned char* dst, uint64_t* fb, const CUtensorMap* mp, const bf16* base, int r0, int rlo, int rhi) {
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
  auto load_rows = [&](int slot, const CUtensorMap* mp, const bf16* base, int r0, int rlo, int rhi) {
    load_rows_to(slot_ptr(slot), &bar[bFull + slot], mp, base, r0, rlo, rhi);
  };
  if (warp == 4) {
    // Everything the first product group needs goes in flight at once: q_gsa (k tile kt into slot kt; rows 0-63 head hq0,
    // rows 64-127 head hq0 + 1), Hk into slot 2, and k' into the first half of the q_swa tiles, which the window steps
    // need only much later (q_swa is fetched once A = q k'^T has read k').
    if (lane == 0) {
      mbar_expect_tx(&bar[bFull + 0], 16384);
      mbar_expect_tx(&bar[bFull + 1], 16384);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
          tma_load_3d(slot_ptr(kt) + hh * 8192, &maps.qg, 64 * kt, hq0 + hh, tq0 + c0, &bar[bFull + kt]);
      mbar_expect_tx(&bar[bFull + 2], 16384);
      tma_load_2d(slot_ptr(2), &maps.hk, 0, (cg * H + h) * D, &bar[bFull + 2]);              // Hk [128][64]
    }
    load_rows_to(sm + oQS, &bar[bQ], &maps.kg, (const bf16*)d.k_gsa, c0 - shift, 0, hi);     // k'
  }

  // ---- decay tables (threads 0..127), as in nha_chunk_fwd_umma.cu -------------------------------------------------
  if (tid < 128) {
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const int i = tid + 128 * j;
      const int r = i >> 3, c8 = i & 7;
      float gv[8];
      unpack8(greg[j], gv);
      *reinterpret_cast<float4*>(As + r * kLdA + 8 * c8) = make_float4(gv[0], gv[1], gv[2], gv[3]);
      *reinterpret_cast<float4*>(As + r * kLdA + 8 * c8 + 4) = make_float4(gv[4], gv[5], gv[6], gv[7]);
    }
  }
  __syncthreads();
  {
    // inclusive scan along the rows: two threads per column (32 rows each), then the first half's total is added
    const int m = tid & 63, seg = tid >> 6;
    if (tid < 128) {
      float run = 0.f;
#pragma unroll 8
      for (int r = 32 * seg; r < 32 * seg + 32; ++r) {
        run += As[r * kLdA + m];
        As[r * kLdA + m] = run;
      }
    }
    __syncthreads();
    if (tid >= 64 && tid < 128) {
      const float add = As[31 * kLdA + m];
#pragma unroll 8
      for (int r = 32; r < 64; ++r) As[r * kLdA + m] += add;
    }
    __syncthreads();
  }
  const bool mine_unsafe = tid < 64 && fabsf(As[63 * kLdA + tid]) > kDecayLimit;
  const int unsafe = __syncthreads_or(mine_unsafe ? 1 : 0);
  if (tid == 0 && blockIdx.z == 0) flags[(size_t)cg * H + h] = unsafe;
  if (unsafe) {
    // the general kernel computes this chunk; the loads already in flight must land before the CTA may leave
    if (warp == 4 && lane == 0) {
      NHA_WAIT(bQ, 0);
      for (int i = 0; i < 3; ++i) NHA_WAIT(bFull + i, 0);
      if (failed) atomicExch(err, 1);
    }
    __syncthreads();
    if (warp == 0) tmem_dealloc(tbase, kTmemCols);
    return;
  }
  {
    float rref[8];
    const int c8 = tid & 7;
    if (tid < 128) {
#pragma unroll
      for (int e = 0; e < 8; ++e) rref[e] = 0.5f * As[63 * kLdA + 8 * c8 + e];
    }
    __syncthreads();                                  // every thread holds its references before the table changes
    if (tid < 8) {
#pragma unroll
      for (int e = 0; e < 8; ++e) ER[8 * tid + e] = __expf(rref[e]);
    }
    if (tid < 128) {
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        const int i = tid + 128 * j;
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

  if (warp == 4) {
    // ================= load warp: the rest of the slot operands, then the window tiles ===============================
    NHA_WAIT(bKq, 0);                                                          // k' has been read (A = q k'^T)
    if (lane == 0) {
      mbar_expect_tx(&bar[bQ], 32768);
#pragma unroll
      for (int hh = 0; hh < 2; ++hh)
#pragma unroll
        for (int kt = 0; kt < 2; ++kt)
          tma_load_3d(sm + oQS + kt * kQTile + hh * 8192, &maps.qs, 64 * kt, hq0 + hh, tq0 + c0, &bar[bQ]);
    }
    NHA_WAIT(bEmpty + 0, 0);                                                   // q_gsa has been read (QH = q Hk)
    if (lane == 0) {
      mbar_expect_tx(&bar[bFull + 0], 16384);
      tma_load_2d(slot_ptr(0), &maps.hv, 0, (cg * H + h) * M, &bar[bFull + 0]);            // Hv [64][128] as two tiles
      tma_load_2d(slot_ptr(0) + 8192, &maps.hv, 64, (cg * H + h) * M, &bar[bFull + 0]);
    }
    NHA_WAIT(bEmpty + 1, 0);
    load_rows(1, &maps.v, (const bf16*)d.v, c0 - shift, 0, hi);               // v'
    // Window keys: step j into slot 2 (j even) or 1 (j odd) as that slot's fill 2 + j / 2; values: slot 0 (j even, fill
    // 2 + j / 2) or 3 (j odd, fill j / 2).  The two sequences are polled side by side: whichever next load finds its
    // slot free is issued.
    int kn = 0, vn = 0, spins = 0;
    while (kn < nst || vn < nst) {
      bool did = false;
      if (kn < nst) {
        const int slot = (kn & 1) ? 1 : 2;
        // fill f of a slot waits for its release f - 1; keys are fills 1, 2, .. of slot 2 (after Hk) and 2, 3, .. of slot 1
        const int free_ = lane == 0 ? (int)mbar_test(&bar[bEmpty + slot], ((kn & 1) + (kn >> 1)) & 1) : 0;
        if (__shfl_sync(0xffffffffu, free_, 0)) {
          load_rows(slot, &maps.ks, (const bf16*)d.k_swa, (ci - kn) * kChunk, 0, len);
          ++kn;
          did = true;
        }
      }
      if (vn < nst) {
        const int slot = (vn & 1) ? 3 : 0;
        const int f = vn >> 1;                           // fill number on slot 3; on slot 0 it is 2 + f
        int free_ = 0;
        if (lane == 0) {
          if (slot == 0) free_ = mbar_test(&bar[bEmpty + 0], (1 + f) & 1);
          else free_ = f == 0 ? mbar_test(&bar[bTab], 0) : mbar_test(&bar[bEmpty + 3], (f - 1) & 1);
        }
        if (__shfl_sync(0xffffffffu, free_, 0)) {
          load_rows(slot, &maps.v, (const bf16*)d.v, (ci - vn) * kChunk, 0, len);
          ++vn;
          did = true;
        }
      }
      if (did) spins = 0;
      else __nanosleep(256);
      if (!did && ++spins > 64 * kPoll) {                     // nothing was released for a very long time: give up
        failed = true;
        break;
      }
    }
  } else if (warp == 5) {
    // ================= MMA warp: one thread issues everything ========================================================
    if (lane == 0) {
      constexpr uint32_t kT16 = kQTile >> 4;             // k-tile pitch of a 128-row A operand, in descriptor units
      const uint32_t iK = make_idesc(128, 64, 0), iMN = make_idesc(128, 64, 1), iMN128 = make_idesc(128, 128, 1);
      const uint64_t dSB = make_desc(smem_u32(sm + oSB));
      const uint64_t dQS = make_desc(smem_u32(sm + oQS));
      const uint32_t aS[4] = {smem_u32(slot_ptr(0)), smem_u32(slot_ptr(1)), smem_u32(slot_ptr(2)), smem_u32(slot_ptr(3))};
      const uint32_t cS0 = tbase, cS1 = tbase + 64, cO = tbase + 128;
      auto wait_full = [&](int slot, int fill) {
        NHA_WAIT(bFull + slot, fill & 1);
        tc_fence_after();
      };
      // D (+)= A B with A from tensor memory: 4 k steps of 16 (8 columns of bf16 pairs each), B MN-major or K-major
      auto mma_ta = [&](uint32_t dcol, uint32_t acol, uint64_t db, bool b_mn, uint32_t idesc, bool acc) {
#pragma unroll
        for (int ks = 0; ks < 4; ++ks)
          mma_f16_ta(dcol, acol + 8 * ks, db + (uint64_t)(b_mn ? ks * 128 : ks * 2), idesc, acc || ks > 0);
      };
      auto s_mma = [&](int j) {          // S_j into accumulator j & 1, then release the keys
        const int slot = (j & 1) ? 1 : 2;
        wait_full(slot, (j & 1) + 1 + (j >> 1));
        mma_run<8, 0>((j & 1) ? cS1 : cS0, dQS, kT16, make_desc(aS[slot]), 8192 >> 4, iK, false);
        commit(&bar[bS + (j & 1)]);
        commit(&bar[bEmpty + slot]);
      };
      uint32_t wph = 0u;
      // G1: A = q k'^T (q_gsa k tiles in slots 0 and 1, 16384 bytes apart; k' in the q_swa tiles), QH = q Hk (Hk in slot 2)
      wait_full(0, 0);
      wait_full(1, 0);
      NHA_WAIT(bQ, 0);                                   // k' in the first half of the q_swa tiles
      tc_fence_after();
      const uint64_t dQG = make_desc(aS[0]);
      mma_run<8, 0>(cS0, dQG, kSlot >> 4, make_desc(smem_u32(sm + oQS)), 8192 >> 4, iK, false);
      commit(&bar[bKq]);
      wait_full(2, 0);
      mma_run<8, 1>(cS1, dQG, kSlot >> 4, make_desc(aS[2]), 0, iMN, false);
      commit(&bar[bG]);
      commit(&bar[bEmpty + 0]);
      commit(&bar[bEmpty + 1]);
      commit(&bar[bEmpty + 2]);
      // G2: X = tril(A) (s' .* b), tril(A) in the first 32 columns of O
      NHA_WAIT(bW, wph); wph ^= 1u;
      tc_fence_after();
      mma_ta(cS0, cO, dSB, true, iMN, false);
      commit(&bar[bG]);
      // G3: O = (p~ a e^R) Hv over all 128 columns (the two 64-column tiles of Hv are 8192 bytes apart), Bv = (p~ a) SB^T;
      //     p~ a e^R in columns 0-31 of S0, p~ a in columns 32-63
      NHA_WAIT(bW, wph); wph ^= 1u;
      wait_full(0, 1);
      mma_ta(cO, cS0, make_desc_lbo(aS[0], 8192), true, iMN128, false);
      mma_ta(cS1, cS0 + 32, dSB, false, iK, false);
      commit(&bar[bG]);
      commit(&bar[bEmpty + 0]);
      NHA_WAIT(bQ, 1);                                   // q_swa
      s_mma(0);                                          // S0 is free once G3 has read the operands in it (in order)
      // G4: O += tril(Bv) v', tril(Bv) in the first 32 columns of S1
      NHA_WAIT(bW, wph); wph ^= 1u;
      wait_full(1, 1);
      mma_ta(cO, cS1, make_desc_lbo(aS[1], 8192), true, iMN128, true);
      commit(&bar[bG]);
      commit(&bar[bEmpty + 1]);
      if (nst > 1) s_mma(1);
      // window steps: O += P~_j V_j with P~_j read from the first 32 columns of S_j, then S_{j+2} into that accumulator
      for (int j = 0; j < nst; ++j) {
        const int b = j & 1;
        NHA_WAIT(bP + b, (j >> 1) & 1);
        const int vslot = b ? 3 : 0;
        wait_full(vslot, b ? (j >> 1) : 2 + (j >> 1));
        mma_ta(cO, b ? cS1 : cS0, make_desc_lbo(aS[vslot], 8192), true, iMN128, true);
        commit(&bar[bPV]);
        commit(&bar[bEmpty + vslot]);
        if (j + 2 < nst) s_mma(j + 2);
      }
    }
  } else {
    // ================= softmax group: one thread per row ============================================================
    const int row = warp * 32 + lane;
    const int tk = row & 63, th = row >> 6;
    const int pos = c0 + tk;
    const bool in_seq = pos < len;
    const int hq = hq0 + th;
    const uint32_t tl = tbase + ((uint32_t)(warp * 32) << 16);     // S0 at +0, S1 at +64, O at +128
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
    // this thread's row of tril of a [128][64] accumulator (token tk keeps columns i <= tk) as 32 columns of bf16 pairs
    auto tril_to = [&](uint32_t src_col, uint32_t dst_col) {
      float v[64];
      tmem_ld64(tl + src_col, v);
      uint32_t pk[32];
#pragma unroll
      for (int e = 0; e < 32; ++e) pk[e] = bf16_pair(2 * e <= tk ? v[2 * e] : 0.f, 2 * e + 1 <= tk ? v[2 * e + 1] : 0.f);
      tmem_st32(tl + dst_col, pk);
      tmem_st_wait();
    };
    auto hand_over = [&](int b_) {
      tc_fence_before();
      mbar_arrive(&bar[b_]);
    };
    // G1 -> tril(A) into the first columns of O (not used before G3)
    NHA_WAIT_WARP(bG, gph); gph ^= 1u;
    tc_fence_after();
    tril_to(0, 128);
    hand_over(bW);
    // G2 -> slot logits, p~, operands
    NHA_WAIT_WARP(bG, gph); gph ^= 1u;
    tc_fence_after();
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
      // p~ a e^R -> columns 0-31 of S0, p~ a -> columns 32-63 (X and QH are in registers by now)
#pragma unroll
      for (int hf = 0; hf < 2; ++hf) {
        uint32_t pg[16], pa[16];
#pragma unroll
        for (int q = 0; q < 8; ++q) {
          const int m = 32 * hf + 4 * q;
          const float4 a4 = *reinterpret_cast<const float4*>(arow + m);
          const float4 e4 = *reinterpret_cast<const float4*>(ER + m);
          const float p0 = exp2f(fmaf(ok[m], kLog2e, nmg)), p1 = exp2f(fmaf(ok[m + 1], kLog2e, nmg));
          const float p2 = exp2f(fmaf(ok[m + 2], kLog2e, nmg)), p3 = exp2f(fmaf(ok[m + 3], kLog2e, nmg));
          l4[0] += p0; l4[1] += p1; l4[2] += p2; l4[3] += p3;
          const float a0 = in_seq ? p0 * a4.x : 0.f, a1 = in_seq ? p1 * a4.y : 0.f;
          const float a2 = in_seq ? p2 * a4.z : 0.f, a3 = in_seq ? p3 * a4.w : 0.f;
          pa[2 * q] = bf16_pair(a0, a1);
          pa[2 * q + 1] = bf16_pair(a2, a3);
          pg[2 * q] = bf16_pair(a0 * e4.x, a1 * e4.y);
          pg[2 * q + 1] = bf16_pair(a2 * e4.z, a3 * e4.w);
        }
        tmem_st16(tl + 16 * hf, pg);
        tmem_st16(tl + 32 + 16 * hf, pa);
      }
      tmem_st_wait();
      lg0 = (l4[0] + l4[1]) + (l4[2] + l4[3]);
    }
    tc_fence_before();
    mbar_arrive(&bar[bTab]);                             // the decay table is dead: its storage becomes ring slot 3
    mbar_arrive(&bar[bW]);
    // G3 -> tril(Bv) over the first columns of S1
    NHA_WAIT_WARP(bG, gph); gph ^= 1u;
    tc_fence_after();
    tril_to(64, 64);
    hand_over(bW);
    // G4
    NHA_WAIT_WARP(bG, gph); gph ^= 1u;
    tc_fence_after();

    float mref = mg;            // reference of the unnormalised probabilities of this row
    float lgs = lg0;            // slot sum, in units of exp(-mref)
    float ls = 0.f;             // window sum, same units
    int pvseen = 0;
    // observe the completions of P~ V of steps 0 .. upto-1 (one barrier, read phase by phase)
    auto wait_pv = [&](int upto) {
      while (pvseen < upto) {
        NHA_WAIT_WARP(bPV, pvseen & 1);
        ++pvseen;
      }
    };
    for (int j = 0; j < nst; ++j) {
      const int b = j & 1;
      NHA_WAIT_WARP(bS + b, (j >> 1) & 1);
      tc_fence_after();
      float s[64];
      tmem_ld64(tl + 64 * b, s);
      const int kb = (ci - j) * kChunk;
      const int off = kb - klo;
      // the diagonal tile (causal edge) and tiles that reach below the oldest visible key of the chunk's last row need
      // the per-element test; every row of the chunk sees all keys of the tiles in between
      const bool masked = j == 0 || (wl >= 0 && kb < c0 + kChunk - 1 - wl) || c0 + kChunk > len;
      {
        float m0 = -INFINITY, m1 = -INFINITY;
        if (masked) {
#pragma unroll
          for (int e = 0; e < 64; e += 4) {
            m0 = max3(m0, (unsigned)(off + e) <= kspan ? s[e] : -INFINITY, (unsigned)(off + e + 1) <= kspan ? s[e + 1] : -INFINITY);
            m1 = max3(m1, (unsigned)(off + e + 2) <= kspan ? s[e + 2] : -INFINITY,
                      (unsigned)(off + e + 3) <= kspan ? s[e + 3] : -INFINITY);
          }
        } else {
#pragma unroll
          for (int e = 0; e < 64; e += 4) {
            m0 = max3(m0, s[e], s[e + 1]);
            m1 = max3(m1, s[e + 2], s[e + 3]);
          }
        }
        const float mc = d.scale * fmaxf(m0, m1);
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
            tmem_st32(tl + 128 + 32 * q4, reinterpret_cast<const uint32_t*>(ov));
          }
          tmem_st_wait();
          lgs *= f;
          ls *= f;
        }
      }
      const float nm = -mref * kLog2e;
      const uint64_t sc2p = pack2(sc2, sc2), nmp = pack2(nm, nm);
      uint64_t l0 = pack2(0.f, 0.f), l1 = l0;
      if (masked) {
#pragma unroll
        for (int e = 0; e < 64; e += 4) {
          float a0, a1, a2, a3;
          unpack2(ffma2(pack2(s[e], s[e + 1]), sc2p, nmp), a0, a1);
          unpack2(ffma2(pack2(s[e + 2], s[e + 3]), sc2p, nmp), a2, a3);
          s[e] = (unsigned)(off + e) <= kspan ? exp2f(a0) : 0.f;
          s[e + 1] = (unsigned)(off + e + 1) <= kspan ? exp2f(a1) : 0.f;
          s[e + 2] = (unsigned)(off + e + 2) <= kspan ? exp2f(a2) : 0.f;
          s[e + 3] = (unsigned)(off + e + 3) <= kspan ? exp2f(a3) : 0.f;
          l0 = fadd2(l0, pack2(s[e], s[e + 1]));
          l1 = fadd2(l1, pack2(s[e + 2], s[e + 3]));
        }
      } else {
#pragma unroll
        for (int e = 0; e < 64; e += 4) {
          float a0, a1, a2, a3;
          unpack2(ffma2(pack2(s[e], s[e + 1]), sc2p, nmp), a0, a1);
          unpack2(ffma2(pack2(s[e + 2], s[e + 3]), sc2p, nmp), a2, a3);
          s[e] = exp2f(a0);
          s[e + 1] = exp2f(a1);
          s[e + 2] = exp2f(a2);
          s[e + 3] = exp2f(a3);
          l0 = fadd2(l0, pack2(s[e], s[e + 1]));
          l1 = fadd2(l1, pack2(s[e + 2], s[e + 3]));
        }
      }
      {
        // P~_j as bf16 pairs over the first 32 columns of S_j: the A operand of the value product
        uint32_t pk[32];
#pragma unroll
        for (int e = 0; e < 32; ++e) pk[e] = bf16_pair(s[2 * e], s[2 * e + 1]);
        tmem_st32(tl + 64 * b, pk);
        tmem_st_wait();
      }
      {
        float a0, a1;
        unpack2(fadd2(l0, l1), a0, a1);
        ls += a0 + a1;
      }
      // Every completion phase of the value products is observed before the next one can happen: P~ V of step j is only
      // issued after this hand-over, so seeing step j - 1 complete here (it was issued a whole step ago) keeps the
      // barrier at most one phase ahead of what this thread has seen.
      wait_pv(j);
      tc_fence_before();
      mbar_arrive(&bar[bP + b]);
    }
    wait_pv(nst);
    tc_fence_after();
    const float lsum = lgs + ls;
    const float inv = lsum > 0.f ? 1.f / lsum : 0.f;
    if (in_seq) {
      d.lse_gsa[(size_t)(tq0 + pos) * HQ + hq] = mg + __logf(lg0);
      d.lse_swa[(size_t)(tq0 + pos) * HQ + hq] = mref + __logf(ls);
    }
    // Output rows leave through shared memory: a thread holds one whole row (256 bytes), and stores of 32 lanes to 32
    // rows 8 KB apart would cost one memory transaction per lane.  The rows are staged in the q_swa tiles (dead: every
    // S product has completed) with the 16-byte pieces of a row rotated by the row index (no bank conflicts), and each
    // warp then writes its own 32 rows, two whole rows per instruction.
    unsigned char* stage = sm + oQS + (size_t)(warp * 32) * 256;     // this warp's 32 rows
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
        const int rr = warp * 32 + r;                     // row of the tile
        const int p2 = c0 + (rr & 63);
        if (p2 < len) {
          const uint4 v = *reinterpret_cast<const uint4*>(stage + r * 256 + ((c ^ (r & 15)) << 4));
          bf16* dst = (bf16*)d.o + ((size_t)(tq0 + p2) * HQ + hq0 + (rr >> 6)) * D + 8 * c;
          *reinterpret_cast<uint4*>(dst) = v;
        }
      }
    }
#undef NHA_WAIT_WARP
  }
#undef NHA_WAIT
  if (failed) atomicExch(err, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, kTmemCols);
}

bool fwd_pipe_supported(const nha_chunk_desc* d) {
  const int NG = d->HQ / d->H;
  if (d->K != 128 || d->V != 128 || d->M != 64 || NG % 2 != 0 || !(d->scale > 0.f)) return false;
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
  const bool ok = make_map_rows_heads(&maps.qg, d->q_gsa, d->Ttot - d->q_offset, d->HQ, D) &&
                  make_map_rows_heads(&maps.qs, d->q_swa, d->Ttot - d->q_offset, d->HQ, D) &&
                  make_map_rows_heads(&maps.kg, d->k_gsa, d->Ttot, d->H, D) &&
                  make_map_rows_heads(&maps.ks, d->k_swa, d->Ttot, d->H, D) &&
                  make_map_rows_heads(&maps.v, d->v, d->Ttot, d->H, D) &&
                  make_map_matrix(&maps.hk, d->hk_chunks, (int64_t)NCB * d->H * D, M, 128) &&
                  make_map_matrix(&maps.hv, d->hv_chunks, (int64_t)NCB * d->H * M, D, 64);
  if (!ok) return NHA_ERR_UNSUPPORTED;
  cudaError_t e = set_max_smem((const void*)nha_fwd_pipe_kernel, total);
  if (e != cudaSuccess) return record_cuda_error(e);
  nha_fwd_pipe_kernel<<<dim3(NCB, d->H, d->HQ / d->H / 2), kThreads, total, cs>>>(*d, flags, err, maps);
  return check_launch();
}

}  // namespace nha
