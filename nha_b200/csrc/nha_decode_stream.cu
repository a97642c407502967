// Streaming variant of the fused NHA decode step (sm_100a) for the common shapes: K == V in {64, 128},
// window keys in the cache (not caller-supplied logits).  Same arithmetic and the same split / merge
// protocol as nha_decode.cu, organised so that the whole grid is resident at once and every byte a CTA
// needs is requested as early as shared memory allows:
//
//   * a (sequence, kv head) is cut into SPLITS CTAs chosen so that B*H*SPLITS CTAs fit the GPU in ONE
//     wave (two CTAs per SM); split s owns a contiguous range of window keys and of slots;
//   * the small inputs (queries, gates, the token that enters the slot memory, the rotary row of the query) and the
//     CTA's hk columns are requested first, into registers, so that they are not queued behind the window;
//   * window keys and values stream through a ring of four 64-key slots filled by 16-byte asynchronous
//     copies with one commit group per stage (the rows of one kv head are 2 D bytes long and H times that
//     apart, too short for bulk copies to pay: one cp.async.bulk per row measured slower): first every key
//     stage, then - into slots as their keys have been used - the value stages.  A warp owns eight rows of every
//     stage: it copies them, rotates them in place (rotate-half on packed bf16 pairs), multiplies them
//     (ldmatrix + mma.sync m16n8k16 for the logits, m16n8k8 over its eight keys for the value readout) and refills
//     them, so the stage loops synchronise with cp.async.wait_group and __syncwarp only - no block-wide barrier.
//     All logits of the CTA are kept ([16][keys] fp32), so the softmax is exact in one pass and the value readout
//     accumulates in registers without rescaling; the eight warps' partial outputs are summed at the end;
//   * the hk columns of the split never touch shared memory: a thread updates its elements in registers,
//     stores them back and contributes to the slot logits of all query heads, which are then summed over
//     the warps; the hv rows, contiguous in memory, arrive by ONE bulk copy (cp.async.bulk on an mbarrier)
//     and are updated and read out before the value stages, while those stream in;
//   * splits are merged by the last CTA of a (sequence, kv head) to arrive (a ticket in global memory); with up
//     to four splits every thread fetches the partial results of its output element in one trip to L2.
//
// Replaces the two Triton launches of fused_recurrent_nha_decode
// (nha_fla/ops/nha/fused_recurrent.py:229-353 k-kernel, :356-428 v-kernel).
#include <stdlib.h>
#include <string.h>

#include <atomic>

#include "nha_common.cuh"
#include "nha_umma.cuh"

namespace nha {

constexpr int kStrThreads = 256;
constexpr int kStrWarps = kStrThreads / 32;
constexpr int kStrStage = 64;            // keys per ring slot
constexpr int kStrSlots = 4;

struct DecodeStreamArgs {
  const bf16* q; const bf16* sq; const bf16* k; const bf16* v; const bf16* g; const bf16* s;
  const bf16* sw_k; const bf16* sw_v; const bf16* cosp; const bf16* sinp;
  float* hk; float* hv; bf16* o;
  float* part_o;      // [B*H, SPLITS, NG, V] unnormalised partial outputs
  float* part_ml;     // [B*H, SPLITS, NG, 2] maximum and sum of each split
  int* tickets;       // [B*H] arrival counters, zero between calls
  int* err;           // device error word (a bounded wait ran out)
  // ring mode (head != NULL): sw_k / sw_v are rings of W physical rows per sequence whose oldest entry sits at
  // row head[b]; that entry is the token that leaves the window and enters the slot memory in this step (its
  // gate row comes from ring_g, the popped k / v from the rings), the token of this step (k, v: not yet in the
  // ring) is the newest window entry
  const int* head; const bf16* ring_g;
  // WR: rows of a ring (W outside ring mode).  nopop != 0: the rings are still filling - they hold the W - 1 oldest
  // window entries in rows 0 .. W - 2, nothing leaves the window and the slot memory keeps its value
  int WR, nopop;
  // ring_kraw != NULL (ring mode only): sw_k is a ring of keys that were rotated when they entered it (rotary by
  // absolute position does not change while the window slides), so only the token of this step is rotated here;
  // the raw key that enters the slot memory comes from ring_kraw
  const bf16* ring_kraw;
  // fused append (ring mode, raw keys): g_new != NULL makes the CTA that merges the splits of a (sequence, kv head)
  // also store the step's token (k, v, g_new) over the entry that left the window (or into the next free row of a
  // filling ring) and advance that kv head's index.  `head` then holds one index per (sequence, kv head), [B*H]: every
  // (sequence, kv head) is finished by exactly one CTA, after all its splits have read the rings, so no other CTA
  // reads the index or the row that is overwritten.
  const bf16* g_new;
  // state_bf16 != 0: hk and hv point to bf16 tensors (half the state bytes; arithmetic stays fp32 in registers)
  int state_bf16;
  int64_t cs_batch, cs_row;
  int B, HQ, H, M, W, NG, SPLITS, KSPL, MQ, zero_state;
  int cluster;        // 1: the SPLITS CTAs of a (sequence, kv head) form a thread-block cluster and merge through shared memory
  // programmatic dependent launch: 0 = plain launch; 1 = the grid may be scheduled before the kernel in front of it on
  // the stream has finished and waits for it before its first global read; 2 = as 1, but the slot memory and the
  // window of this call are requested BEFORE that wait (the caller asserts that the kernel in front writes neither)
  int pdl;
  float scale;
  int off_ring, off_hv, off_S, off_red, off_q, off_sqA, off_oks, off_eg, off_sv, off_kpop, off_vpop, off_ml, off_bar;
};

__device__ __forceinline__ void bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   umma::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(umma::smem_u32(mbar))
               : "memory");
}
// one element of the slot memory, fp32 or bf16 storage
__device__ __forceinline__ float ld_state(const float* base, size_t idx, int is_bf16) {
  return is_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(base)[idx]) : base[idx];
}
__device__ __forceinline__ void st_state(float* base, size_t idx, float& v, int is_bf16) {
  if (is_bf16) {
    const bf16 r = __float2bfloat16_rn(v);
    reinterpret_cast<bf16*>(base)[idx] = r;
    v = __bfloat162float(r);                 // the rounded value is the state from here on
  } else {
    base[idx] = v;
  }
}
__device__ __forceinline__ void mbar_expect(uint64_t* mbar, uint32_t bytes) {
  asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(umma::smem_u32(mbar)), "r"(bytes) : "memory");
}

// warp-level matrix fragments straight from shared memory, and the two mma.sync shapes the kernel uses
__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(umma::smem_u32(p)) : "memory");
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
               : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(umma::smem_u32(p)) : "memory");
}
__device__ __forceinline__ void ldsm_x2(uint32_t (&r)[2], const void* p) {
  asm volatile("ldmatrix.sync.aligned.m8n8.x2.shared.b16 {%0,%1}, [%2];"
               : "=r"(r[0]), "=r"(r[1]) : "r"(umma::smem_u32(p)) : "memory");
}
// thread-block cluster: barrier over all threads of all CTAs, and loads from another CTA's shared memory
__device__ __forceinline__ void cluster_sync_all() {
  asm volatile("barrier.cluster.arrive.release.aligned;\nbarrier.cluster.wait.acquire.aligned;" ::: "memory");
}
__device__ __forceinline__ uint32_t cluster_map(const void* p, uint32_t rank) {
  uint32_t r;
  asm volatile("mapa.shared::cluster.u32 %0, %1, %2;" : "=r"(r) : "r"(umma::smem_u32(p)), "r"(rank));
  return r;
}
__device__ __forceinline__ float4 ld_cluster_f4(uint32_t addr) {
  float4 v;
  asm volatile("ld.shared::cluster.v4.f32 {%0,%1,%2,%3}, [%4];" : "=f"(v.x), "=f"(v.y), "=f"(v.z), "=f"(v.w) : "r"(addr) : "memory");
  return v;
}
__device__ __forceinline__ float2 ld_cluster_f2(uint32_t addr) {
  float2 v;
  asm volatile("ld.shared::cluster.v2.f32 {%0,%1}, [%2];" : "=f"(v.x), "=f"(v.y) : "r"(addr) : "memory");
  return v;
}

// programmatic dependent launch: wait until the grids this one depends on have completed and their writes are
// visible; let the grid behind this one on the stream be scheduled
__device__ __forceinline__ void grid_dep_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void grid_dep_launch() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

// c[16x8] += a[16x16] b[16x8]
__device__ __forceinline__ void mma_16816(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
  asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
               : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// c[16x8] += a[16x8] b[8x8]
__device__ __forceinline__ void mma_1688(float (&c)[4], uint32_t a0, uint32_t a1, uint32_t b0) {
  asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5}, {%6}, {%0,%1,%2,%3};"
               : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a0), "r"(a1), "r"(b0));
}

template <int D, bool SB16>
__global__ void __launch_bounds__(kStrThreads, 2) nha_decode_stream_kernel(const DecodeStreamArgs a) {
  using namespace nvcuda::wmma;
  extern __shared__ __align__(128) unsigned char smem[];
  constexpr int K = D, V = D, ldk = D + 8, ldq = D + 8, ldo = D + 8;
  constexpr int kSlotBytes = kStrStage * ldk * 2;
  unsigned char* ring = smem + a.off_ring;                         // [4 slots][64][D+8] bf16
  float* hvS = reinterpret_cast<float*>(smem + a.off_hv);          // [MQ][V] my rows of hv
  float* S = reinterpret_cast<float*>(smem + a.off_S);             // [16][nkp+8] logits, then bf16 weights in place
  float* red = reinterpret_cast<float*>(smem + a.off_red);         // [warps][NG][32] partial slot logits
  float* qs = reinterpret_cast<float*>(smem + a.off_q);            // [NG][K] raw query, fp32
  bf16* sqA = reinterpret_cast<bf16*>(smem + a.off_sqA);           // [16][K+8] rotated query (rows >= NG zero)
  float* oks = reinterpret_cast<float*>(smem + a.off_oks);         // [NG][MQ] slot logits -> unnormalised weights
  float* eg = reinterpret_cast<float*>(smem + a.off_eg);
  float* sv = reinterpret_cast<float*>(smem + a.off_sv);
  float* kpop = reinterpret_cast<float*>(smem + a.off_kpop);
  float* vpop = reinterpret_cast<float*>(smem + a.off_vpop);
  float* ml = reinterpret_cast<float*>(smem + a.off_ml);
  uint64_t* bars = reinterpret_cast<uint64_t*>(smem + a.off_bar);  // [4] ring slots, [4] = hv rows

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int SPL = a.SPLITS, NG = a.NG, M = a.M, W = a.W, MQ = a.MQ;
  const int bh = blockIdx.x / SPL, sp = blockIdx.x % SPL;
  const int b = bh / a.H, h = bh % a.H;
  const bool rotary = a.cosp != nullptr;
  const int w0 = sp * a.KSPL;
  const int nkeys = max(0, min(a.KSPL, W - w0));
  const int nst = (nkeys + kStrStage - 1) / kStrStage;
  const int nkp = nst * kStrStage;
  const int lds = nkp + 8;
  const int m0 = sp * MQ;
  const int nslots = max(0, min(MQ, M - m0));
  const int nloads = 2 * nst;                                      // key stages, then value stages
  const bool isring = a.head != nullptr;
  const int WR = a.WR;
  if (a.pdl == 1) {                                                // before the first global read
    grid_dep_wait();
    grid_dep_launch();
  }
  const int hd = isring ? (a.nopop ? -1 : a.head[a.g_new ? bh : b]) : 0;   // physical row of the oldest ring entry
  // the token that enters the slot memory: separate small tensors, or the oldest ring entry
  const bool prerot = a.ring_kraw != nullptr;
  const bf16* kpop_g = isring ? (prerot ? a.ring_kraw : a.sw_k) + (((size_t)b * WR + max(hd, 0)) * a.H + h) * D
                              : a.k + (size_t)bh * D;
  const bf16* vpop_g = isring ? a.sw_v + (((size_t)b * WR + max(hd, 0)) * a.H + h) * D : a.v + (size_t)bh * D;
  const bf16* gpop_g = isring ? a.ring_g + (((size_t)b * WR + max(hd, 0)) * a.H + h) * M : a.g + (size_t)bh * M;
  bool failed = false;
  // the step's token into the rings (called by the one CTA that finishes this (sequence, kv head))
  auto append_token = [&]() {
    if (!a.g_new) return;
    const int row = a.nopop ? W - 1 : hd;                          // a filling ring holds W - 1 entries: next free row
    const size_t at = ((size_t)b * WR + row) * a.H + h;
    uint4* rk = reinterpret_cast<uint4*>(const_cast<bf16*>(a.sw_k) + at * D);
    uint4* rv = reinterpret_cast<uint4*>(const_cast<bf16*>(a.sw_v) + at * D);
    uint4* rg = reinterpret_cast<uint4*>(const_cast<bf16*>(a.ring_g) + at * M);
    const uint4* kn = reinterpret_cast<const uint4*>(a.k + (size_t)bh * D);
    const uint4* vn = reinterpret_cast<const uint4*>(a.v + (size_t)bh * D);
    const uint4* gn = reinterpret_cast<const uint4*>(a.g_new + (size_t)bh * M);
    const int nd = D / 8, ng = M / 8;
    for (int i = tid; i < 2 * nd + ng; i += kStrThreads) {
      if (i < nd) rk[i] = kn[i];
      else if (i < 2 * nd) rv[i - nd] = vn[i - nd];
      else rg[i - 2 * nd] = gn[i - 2 * nd];
    }
    if (tid == 0 && !a.nopop) const_cast<int*>(a.head)[bh] = hd + 1 == WR ? 0 : hd + 1;
  };

  if (tid == 0) {
    for (int i = 0; i < kStrSlots + 1; ++i) umma::mbar_init(&bars[i], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();

  // ring load j (j < nst: keys of stage j; else values of stage j - nst) into slot j % 4 by 16-byte asynchronous
  // copies.  A warp copies, rotates and multiplies only ITS OWN eight rows of every stage (rows 8 warp .. 8 warp + 7),
  // so a stage is handed from the copies to the arithmetic by cp.async.wait_group + __syncwarp alone and the loops
  // below hold no block-wide barrier.  A lane always copies the same 16-byte column, so the address arithmetic
  // is one add per copy; rows past the end of the split are zero-filled.  One commit group per load and thread:
  // groups complete in order, which is the order the stages are consumed in.
  constexpr int kC8 = D / 8;                                       // 16-byte columns of a row
  constexpr int kRStep = 32 / kC8;                                 // rows between two copies of a lane
  const int lc = lane % kC8, lr = 8 * warp + lane / kC8;
#define NHA_ISSUE_LOAD(j_)                                                                          \
  do {                                                                                              \
    const int j__ = (j_);                                                                           \
    const int st__ = j__ < nst ? j__ : j__ - nst;                                                   \
    const bf16* base__ = (j__ < nst ? a.sw_k : a.sw_v) + ((size_t)b * WR * a.H + h) * D + 8 * lc;   \
    const bf16* new__ = (j__ < nst ? a.k : a.v) + (size_t)bh * D + 8 * lc;                          \
    unsigned char* dst__ = ring + (j__ % kStrSlots) * kSlotBytes + 16 * lc;                         \
    const int rows__ = min(kStrStage, nkeys - st__ * kStrStage);                                    \
    _Pragma("unroll") for (int i__ = 0; i__ < kC8 / 4; ++i__) {                                     \
      const int r__ = lr + i__ * kRStep;                                                            \
      const bool ok__ = r__ < rows__;                                                               \
      const int lw__ = w0 + st__ * kStrStage + (ok__ ? r__ : 0);      /* logical window index */    \
      const bf16* src__;                                                                            \
      if (!isring) src__ = base__ + (size_t)lw__ * a.H * D;                                         \
      else if (lw__ == W - 1) src__ = new__;                          /* the token of this step */  \
      else { int pr__ = hd + 1 + lw__; if (pr__ >= WR) pr__ -= WR; src__ = base__ + (size_t)pr__ * a.H * D; } \
      umma::cp16(dst__ + r__ * ldk * 2, src__, ok__);                                               \
    }                                                                                               \
    umma::cp_commit();                                                                              \
  } while (0)
// wait until ring load j_ has landed: the loads issued after it may stay in flight
#define NHA_WAIT_LOAD(j_, issued_)                                                                  \
  do {                                                                                              \
    const int pend__ = (issued_) - (j_) - 1;                                                        \
    if (pend__ >= 3) asm volatile("cp.async.wait_group 3;\n" ::);                                   \
    else if (pend__ == 2) asm volatile("cp.async.wait_group 2;\n" ::);                              \
    else if (pend__ == 1) asm volatile("cp.async.wait_group 1;\n" ::);                              \
    else asm volatile("cp.async.wait_group 0;\n" ::);                                               \
  } while (0)

  // ---- the small inputs first, into registers, so that they are not queued behind the window in the memory system;
  //      then everything that fits goes in flight: my columns of hk, the first ring loads, my rows of hv.
  //      Disjoint groups of threads fetch the four small inputs, so that their loads overlap. ----------------------
  // my columns of hk: thread -> column m = lane (+32 per block of columns), rows k = kRowsPer warp + j.  The first
  // block of columns (all of them unless the split owns more than 32 slots) is fetched in the prologue.
  constexpr int kRowsPer = K / kStrWarps;
  float hreg[kRowsPer];
  const int ncb = (nslots + 31) / 32;
#define NHA_LOAD_HK_FIRST()                                                                         \
  do {                                                                                              \
    if (!a.zero_state && nslots > 0) {                                                              \
      _Pragma("unroll") for (int j = 0; j < kRowsPer; ++j)                                          \
        hreg[j] = lane < nslots ? ld_state(a.hk, ((size_t)bh * K + kRowsPer * warp + j) * M + m0 + lane, SB16) : 0.f; \
    }                                                                                               \
  } while (0)
#define NHA_LOAD_HV_ROWS()                                                                          \
  do {                                                                                              \
    if (nslots > 0 && !a.zero_state && tid == 0) {                                                  \
      if (SB16) {     /* bf16 rows land in the second half of their fp32 home */                \
        mbar_expect(&bars[kStrSlots], (uint32_t)nslots * V * 2);                                    \
        bulk_g2s(reinterpret_cast<bf16*>(hvS) + (size_t)nslots * V,                                 \
                 reinterpret_cast<const bf16*>(a.hv) + ((size_t)bh * M + m0) * V, (uint32_t)nslots * V * 2, &bars[kStrSlots]); \
      } else {                                                                                      \
        mbar_expect(&bars[kStrSlots], (uint32_t)nslots * V * 4);                                    \
        bulk_g2s(hvS, a.hv + ((size_t)bh * M + m0) * V, (uint32_t)nslots * V * 4, &bars[kStrSlots]); \
      }                                                                                             \
    }                                                                                               \
  } while (0)
  // Dependent launch with early requests (pdl == 2): the state and the window of this call do not depend on the
  // kernel in front, so they go in flight before the wait.  In ring mode the newest window entry is the token of
  // this step (a.k / a.v, written by the caller's projections): the ring loads from the first one that holds it on
  // are issued after the wait, in the same order as always (groups complete in issue order).
  const int ninit = min(nloads, kStrSlots);
  int npre = 0;
  if (a.pdl == 2) {
    npre = ninit;
    if (isring && w0 + nkeys == W && nst > 0) npre = min(npre, nst - 1);
    NHA_LOAD_HK_FIRST();
    for (int j = 0; j < npre; ++j) NHA_ISSUE_LOAD(j);
    NHA_LOAD_HV_ROWS();
    grid_dep_wait();
    grid_dep_launch();
  }
  constexpr int c8h = K >> 4;
  const int qi = tid - 128, q_r = qi / c8h, q_c = qi - q_r * c8h;
  const bool qthread = tid >= 128 && qi < 16 * c8h, qlive = qthread && q_r < NG;
  uint4 rq_x = make_uint4(0u, 0u, 0u, 0u), rq_y = rq_x, rq_c1 = rq_x, rq_s1 = rq_x, rq_c2 = rq_x, rq_s2 = rq_x;
  if (qlive) {
    const bf16* qrow = a.q + ((size_t)b * a.HQ + h * NG + q_r) * K;
    rq_x = __ldg(reinterpret_cast<const uint4*>(qrow + 8 * q_c));
    rq_y = __ldg(reinterpret_cast<const uint4*>(qrow + 8 * (q_c + c8h)));
    if (rotary) {
      // the query position is the last row of the window tables
      const bf16* cq = a.cosp + b * a.cs_batch + (int64_t)(W - 1) * a.cs_row;
      const bf16* sn = a.sinp + b * a.cs_batch + (int64_t)(W - 1) * a.cs_row;
      rq_c1 = __ldg(reinterpret_cast<const uint4*>(cq + 8 * q_c));
      rq_s1 = __ldg(reinterpret_cast<const uint4*>(sn + 8 * q_c));
      rq_c2 = __ldg(reinterpret_cast<const uint4*>(cq + 8 * (q_c + c8h)));
      rq_s2 = __ldg(reinterpret_cast<const uint4*>(sn + 8 * (q_c + c8h)));
    } else {
      const bf16* srow = a.sq + ((size_t)b * a.HQ + h * NG + q_r) * K;
      rq_c1 = __ldg(reinterpret_cast<const uint4*>(srow + 8 * q_c));
      rq_c2 = __ldg(reinterpret_cast<const uint4*>(srow + 8 * (q_c + c8h)));
    }
  }
  if (a.pdl != 2) NHA_LOAD_HK_FIRST();
  // the gates (threads 0..63) and the popped token (one warp each for k and v)
  bf16 gb[2], sb[2];
  gb[0] = gb[1] = sb[0] = sb[1] = f2bf(0.f);
  uint4 rpop = make_uint4(0u, 0u, 0u, 0u);
  if (tid < 64) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int m = tid + 64 * u;
      if (m < nslots && !a.nopop) {
        gb[u] = gpop_g[m0 + m];
        if (a.s) sb[u] = a.s[(size_t)bh * M + m0 + m];
      }
    }
  } else if (tid < 96) {
    if (tid - 64 < (K >> 3) && !a.nopop) rpop = __ldg(reinterpret_cast<const uint4*>(kpop_g + 8 * (tid - 64)));
  } else if (tid < 128) {
    if (tid - 96 < (V >> 3) && !a.nopop) rpop = __ldg(reinterpret_cast<const uint4*>(vpop_g + 8 * (tid - 96)));
  }
  for (int j = npre; j < ninit; ++j) NHA_ISSUE_LOAD(j);
  if (a.pdl != 2) NHA_LOAD_HV_ROWS();
#undef NHA_LOAD_HK_FIRST
#undef NHA_LOAD_HV_ROWS
  // registers -> shared memory
  if (tid < 64) {
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int m = tid + 64 * u;
      if (m < MQ) {
        float e = 1.f, sm = 0.f;
        if (m < nslots) {
          e = __expf(bf2f(gb[u]));
          sm = a.s ? bf2f(sb[u]) : 1.0f - e;
        }
        eg[m] = e;
        sv[m] = sm;
      }
    }
  } else if (tid < 128) {
    const int i = (tid - 64) & 31;
    if (i < (K >> 3)) {
      float f[8];
      unpack8(rpop, f);
      float* dstp = tid < 96 ? kpop : vpop;
#pragma unroll
      for (int e = 0; e < 8; ++e) dstp[8 * i + e] = f[e];
    }
  } else if (qthread) {
    uint4 o1 = make_uint4(0u, 0u, 0u, 0u), o2 = o1;
    if (qlive) {
      if (rotary) {
        float x[8], y[8], c1[8], s1[8], c2[8], s2[8], p1[8], p2[8];
        unpack8(rq_x, x); unpack8(rq_y, y);
        unpack8(rq_c1, c1); unpack8(rq_s1, s1); unpack8(rq_c2, c2); unpack8(rq_s2, s2);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          p1[e] = x[e] * c1[e] - y[e] * s1[e];
          p2[e] = y[e] * c2[e] + x[e] * s2[e];
        }
        o1 = pack8(p1); o2 = pack8(p2);
      } else {
        o1 = rq_c1; o2 = rq_c2;
      }
      float fx[8], fy[8];
      unpack8(rq_x, fx); unpack8(rq_y, fy);
      float4* qd = reinterpret_cast<float4*>(qs + q_r * K + 8 * q_c);
      qd[0] = make_float4(fx[0], fx[1], fx[2], fx[3]);
      qd[1] = make_float4(fx[4], fx[5], fx[6], fx[7]);
      qd = reinterpret_cast<float4*>(qs + q_r * K + 8 * (q_c + c8h));
      qd[0] = make_float4(fy[0], fy[1], fy[2], fy[3]);
      qd[1] = make_float4(fy[4], fy[5], fy[6], fy[7]);
    }
    *reinterpret_cast<uint4*>(sqA + q_r * ldq + 8 * q_c) = o1;
    *reinterpret_cast<uint4*>(sqA + q_r * ldq + 8 * (q_c + c8h)) = o2;
  }
  __syncthreads();
  // ---- my columns of hk <- hk exp(g) + k s^T (registers -> global), partial slot logits of every query head ----
  for (int cb = 0; cb < ncb; ++cb) {
    const int m = 32 * cb + lane;
    if (cb > 0 && !a.zero_state) {
#pragma unroll
      for (int j = 0; j < kRowsPer; ++j)
        hreg[j] = m < nslots ? ld_state(a.hk, ((size_t)bh * K + kRowsPer * warp + j) * M + m0 + m, SB16) : 0.f;
    }
    const float e = m < MQ ? eg[m] : 1.f, sm = m < MQ ? sv[m] : 0.f;
    float hval[kRowsPer];
#pragma unroll
    for (int j = 0; j < kRowsPer; ++j) {
      const int kk = kRowsPer * warp + j;
      hval[j] = (a.zero_state ? 0.f : hreg[j]) * e + kpop[kk] * sm;
      if (m < nslots) st_state(a.hk, ((size_t)bh * K + kk) * M + m0 + m, hval[j], SB16);
    }
    // this warp's rows of every query head: 16-byte loads of the query (the same address for all lanes)
#pragma unroll
    for (int qh = 0; qh < 16; ++qh) {
      if (qh < NG) {
        float acc = 0.f;
#pragma unroll
        for (int c4 = 0; c4 < kRowsPer / 4; ++c4) {
          const float4 q4 = *reinterpret_cast<const float4*>(qs + qh * K + kRowsPer * warp + 4 * c4);
          acc += q4.x * hval[4 * c4] + q4.y * hval[4 * c4 + 1] + q4.z * hval[4 * c4 + 2] + q4.w * hval[4 * c4 + 3];
        }
        red[(warp * NG + qh) * 32 + lane] = acc;
      }
    }
    __syncthreads();
    for (int i = tid; i < NG * 32; i += kStrThreads) {
      const int qh = i >> 5, l = i & 31;
      float sum = 0.f;
#pragma unroll
      for (int w8 = 0; w8 < kStrWarps; ++w8) sum += red[(w8 * NG + qh) * 32 + l];
      if (32 * cb + l < MQ) oks[qh * MQ + 32 * cb + l] = sum * a.scale;
    }
    __syncthreads();
  }

  // ---- key stages, warp-private: wait for my rows, rotate-half in place, S[:, my 8 keys] = sq K^T by m16n8k16 MMAs
  //      with the query fragments held in registers; the freed rows take the next ring load -------------------------
  constexpr int kTasks = 8 * c8h / 32;                             // rotary tasks per lane (8 values x 2 halves each)
  const int gq = lane >> 2, tq = lane & 3;                         // fragment coordinates of the lane
  uint32_t afr[K / 16][4];
#pragma unroll
  for (int ks = 0; ks < K / 16; ++ks) ldsm_x4(afr[ks], sqA + (lane & 15) * ldq + 16 * ks + 8 * (lane >> 4));
  uint4 cs[kTasks][4];                                             // rotate-half table entries of the stage being rotated
#define NHA_LOAD_TABLE(st_)                                                                         \
  _Pragma("unroll") for (int u = 0; u < kTasks; ++u) {                                              \
    const int i = lane + 32 * u;                                                                    \
    const int r = i / c8h, c = i - r * c8h;                                                         \
    const int wraw = w0 + (st_) * kStrStage + 8 * warp + r;                                         \
    const int wpos = min(wraw, W - 1);                                                              \
    if (!prerot || wraw == W - 1) {                     /* rotated ring: only the token of this step */ \
      const bf16* crow = a.cosp + b * a.cs_batch + (int64_t)wpos * a.cs_row;                        \
      const bf16* srow = a.sinp + b * a.cs_batch + (int64_t)wpos * a.cs_row;                        \
      cs[u][0] = __ldg(reinterpret_cast<const uint4*>(crow + 8 * c));                               \
      cs[u][1] = __ldg(reinterpret_cast<const uint4*>(srow + 8 * c));                               \
      cs[u][2] = __ldg(reinterpret_cast<const uint4*>(crow + 8 * (c + c8h)));                       \
      cs[u][3] = __ldg(reinterpret_cast<const uint4*>(srow + 8 * (c + c8h)));                       \
    }                                                                                               \
  }
  if (rotary && nst > 0) { NHA_LOAD_TABLE(0) }
  for (int st = 0; st < nst; ++st) {
    const int slot = st % kStrSlots;
    bf16* kst = reinterpret_cast<bf16*>(ring + slot * kSlotBytes) + (size_t)8 * warp * ldk;   // my rows of the stage
    NHA_WAIT_LOAD(st, min(nloads, kStrSlots + st));
    __syncwarp();                                                  // every lane's copies of my rows have landed
    if (rotary) {
#pragma unroll
      for (int u = 0; u < kTasks; ++u) {
        const int i = lane + 32 * u;
        const int r = i / c8h, c = i - r * c8h;
        if (prerot && w0 + st * kStrStage + 8 * warp + r != W - 1) continue;
        // packed bf16 arithmetic: x c1 - y s1 and y c2 + x s2 on pairs, the first product rounded to bf16
        uint4 xu = *reinterpret_cast<const uint4*>(kst + r * ldk + 8 * c);
        uint4 yu = *reinterpret_cast<const uint4*>(kst + r * ldk + 8 * (c + c8h));
        uint4 o1u, o2u;
        const __nv_bfloat162* xv = reinterpret_cast<const __nv_bfloat162*>(&xu);
        const __nv_bfloat162* yv = reinterpret_cast<const __nv_bfloat162*>(&yu);
        const __nv_bfloat162* c1v = reinterpret_cast<const __nv_bfloat162*>(&cs[u][0]);
        const __nv_bfloat162* s1v = reinterpret_cast<const __nv_bfloat162*>(&cs[u][1]);
        const __nv_bfloat162* c2v = reinterpret_cast<const __nv_bfloat162*>(&cs[u][2]);
        const __nv_bfloat162* s2v = reinterpret_cast<const __nv_bfloat162*>(&cs[u][3]);
        __nv_bfloat162* o1v = reinterpret_cast<__nv_bfloat162*>(&o1u);
        __nv_bfloat162* o2v = reinterpret_cast<__nv_bfloat162*>(&o2u);
#pragma unroll
        for (int e = 0; e < 4; ++e) {
          o1v[e] = __hfma2(xv[e], c1v[e], __hneg2(__hmul2(yv[e], s1v[e])));
          o2v[e] = __hfma2(yv[e], c2v[e], __hmul2(xv[e], s2v[e]));
        }
        *reinterpret_cast<uint4*>(kst + r * ldk + 8 * c) = o1u;
        *reinterpret_cast<uint4*>(kst + r * ldk + 8 * (c + c8h)) = o2u;
      }
      // the next stage's table entries travel while this stage's logits are formed
      if (st + 1 < nst) { NHA_LOAD_TABLE(st + 1) }
      __syncwarp();
    }
    float c0[4] = {0.f, 0.f, 0.f, 0.f}, c1[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
    for (int k2 = 0; k2 < K / 32; ++k2) {
      uint32_t bfr[4];                                             // my 8 keys x 32 features: two k-steps
      ldsm_x4(bfr, kst + (lane & 7) * ldk + 32 * k2 + 8 * (lane >> 3));
      mma_16816(c0, afr[2 * k2], bfr[0], bfr[1]);
      mma_16816(c1, afr[2 * k2 + 1], bfr[2], bfr[3]);
    }
    float* sdst = S + st * kStrStage + 8 * warp + 2 * tq;
    *reinterpret_cast<float2*>(sdst + (size_t)gq * lds) = make_float2(c0[0] + c1[0], c0[1] + c1[1]);
    *reinterpret_cast<float2*>(sdst + (size_t)(gq + 8) * lds) = make_float2(c0[2] + c1[2], c0[3] + c1[3]);
    __syncwarp();                                                  // every lane is done with my rows of the slot
    if (st + kStrSlots < nloads) NHA_ISSUE_LOAD(st + kStrSlots);
  }
#undef NHA_LOAD_TABLE
  __syncthreads();                                                 // all logits of the CTA are in S

  // ---- my rows of hv <- diag(exp(g)) hv + s v^T (in place; they arrived behind the keys) ----------------------------
  constexpr int V4 = V >> 2;
  if (nslots > 0) {
    if (!a.zero_state && !umma::mbar_wait(&bars[kStrSlots], 0)) failed = true;
    float4* hg = reinterpret_cast<float4*>(a.hv + ((size_t)bh * M + m0) * V);
    uint2* hg16 = reinterpret_cast<uint2*>(reinterpret_cast<bf16*>(a.hv) + ((size_t)bh * M + m0) * V);
    const uint2* stage16 = reinterpret_cast<const uint2*>(reinterpret_cast<const bf16*>(hvS) + (size_t)nslots * V);
    // four elements per thread and round: all loads of a round before its stores.  bf16 states: the rows were staged
    // in the second half of the fp32 rows they are expanded into, so a block barrier separates a round's loads from its
    // stores (round r writes the bytes [16 KB r, 16 KB (r + 1)), the staging of the later rounds lies behind them)
    for (int i0 = tid; i0 - tid < nslots * V4; i0 += 4 * kStrThreads) {
      float4 hh[4], vp4[4];
      float e[4], sm[4];
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kStrThreads;
        if (i < nslots * V4) {
          const int m = i / V4, c = i - m * V4;
          if (a.zero_state) {
            hh[u] = make_float4(0.f, 0.f, 0.f, 0.f);
          } else if (SB16) {
            const uint2 raw = stage16[i];
            const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.x));
            const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&raw.y));
            hh[u] = make_float4(lo2.x, lo2.y, hi2.x, hi2.y);
          } else {
            hh[u] = *reinterpret_cast<const float4*>(hvS + m * V + 4 * c);
          }
          vp4[u] = *reinterpret_cast<const float4*>(vpop + 4 * c);
          e[u] = eg[m]; sm[u] = sv[m];
        }
      }
      if (SB16) __syncthreads();
#pragma unroll
      for (int u = 0; u < 4; ++u) {
        const int i = i0 + u * kStrThreads;
        if (i < nslots * V4) {
          hh[u].x = hh[u].x * e[u] + sm[u] * vp4[u].x;
          hh[u].y = hh[u].y * e[u] + sm[u] * vp4[u].y;
          hh[u].z = hh[u].z * e[u] + sm[u] * vp4[u].z;
          hh[u].w = hh[u].w * e[u] + sm[u] * vp4[u].w;
          if (SB16) {
            // the rounded value is the state from here on: the readout uses what the next step will read
            uint2 pk;
            *reinterpret_cast<__nv_bfloat162*>(&pk.x) = __floats2bfloat162_rn(hh[u].x, hh[u].y);
            *reinterpret_cast<__nv_bfloat162*>(&pk.y) = __floats2bfloat162_rn(hh[u].z, hh[u].w);
            hg16[i] = pk;
            const float2 lo2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.x));
            const float2 hi2 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&pk.y));
            reinterpret_cast<float4*>(hvS)[i] = make_float4(lo2.x, lo2.y, hi2.x, hi2.y);
          } else {
            reinterpret_cast<float4*>(hvS)[i] = hh[u];
            hg[i] = hh[u];
          }
        }
      }
    }
  }

  // ---- partial softmax over [my slots | my keys], one warp per query head; weights replace the logits in place ---
  for (int qh = warp; qh < NG; qh += kStrWarps) {
    float* srow = S + (size_t)qh * lds;
    bf16* prow = reinterpret_cast<bf16*>(srow);
    float mx = -INFINITY;
    for (int m = lane; m < nslots; m += 32) mx = fmaxf(mx, oks[qh * MQ + m]);
    // a lane takes 8 consecutive keys of every block of 256
    for (int w8 = 8 * lane; w8 < nkp; w8 += 256) {
      const float4 x0 = *reinterpret_cast<const float4*>(srow + w8), x1 = *reinterpret_cast<const float4*>(srow + w8 + 4);
      const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
      for (int e8 = 0; e8 < 8; ++e8)
        if (w8 + e8 < nkeys) mx = fmaxf(mx, xs[e8] * a.scale);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int m = lane; m < nslots; m += 32) {
      const float e = __expf(oks[qh * MQ + m] - mx);
      oks[qh * MQ + m] = e;
      sum += e;
    }
    // the bf16 weight of key w lands inside the fp32 logit of key w / 2: convert a block of 256 keys at a time,
    // blocks in ascending order, reading all of a block before any of it is written
    for (int blk = 0; blk < nkp; blk += 256) {
      const int w8 = blk + 8 * lane;
      float es[8];
      if (w8 < nkp) {
        const float4 x0 = *reinterpret_cast<const float4*>(srow + w8), x1 = *reinterpret_cast<const float4*>(srow + w8 + 4);
        const float xs[8] = {x0.x, x0.y, x0.z, x0.w, x1.x, x1.y, x1.z, x1.w};
#pragma unroll
        for (int e8 = 0; e8 < 8; ++e8) {
          es[e8] = w8 + e8 < nkeys ? __expf(xs[e8] * a.scale - mx) : 0.f;
          sum += es[e8];
        }
      }
      __syncwarp();
      if (w8 < nkp) *reinterpret_cast<uint4*>(prow + w8) = pack8(es);
      __syncwarp();
    }
    sum = warp_sum(sum);
    if (lane == 0) {
      ml[2 * qh] = (nslots + nkeys) > 0 ? mx : -INFINITY;
      ml[2 * qh + 1] = sum;
    }
  }
  __syncthreads();

  // ---- slot readout of my output elements, kept in registers while the values stream in ---------------------------
  float4 sacc[2];
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    sacc[u] = make_float4(0.f, 0.f, 0.f, 0.f);
    const int i = tid + u * kStrThreads;
    if (i < NG * V4) {
      const int qh = i / V4, c = i - qh * V4;
      // nslots is a multiple of four: four slots at a time, all loads of a block before its arithmetic
#pragma unroll 2
      for (int m = 0; m < nslots; m += 4) {
        const float4 pm = *reinterpret_cast<const float4*>(oks + qh * MQ + m);
        const float4 h0 = *reinterpret_cast<const float4*>(hvS + m * V + 4 * c);
        const float4 h1 = *reinterpret_cast<const float4*>(hvS + (m + 1) * V + 4 * c);
        const float4 h2 = *reinterpret_cast<const float4*>(hvS + (m + 2) * V + 4 * c);
        const float4 h3 = *reinterpret_cast<const float4*>(hvS + (m + 3) * V + 4 * c);
        sacc[u].x += pm.x * h0.x; sacc[u].y += pm.x * h0.y; sacc[u].z += pm.x * h0.z; sacc[u].w += pm.x * h0.w;
        sacc[u].x += pm.y * h1.x; sacc[u].y += pm.y * h1.y; sacc[u].z += pm.y * h1.z; sacc[u].w += pm.y * h1.w;
        sacc[u].x += pm.z * h2.x; sacc[u].y += pm.z * h2.y; sacc[u].z += pm.z * h2.z; sacc[u].w += pm.z * h2.w;
        sacc[u].x += pm.w * h3.x; sacc[u].y += pm.w * h3.y; sacc[u].z += pm.w * h3.z; sacc[u].w += pm.w * h3.w;
      }
    }
  }

  // ---- value stages, warp-private: O_w += P[:, my 8 keys] V[my 8 keys, :] by m16n8k8 MMAs, all V columns per warp,
  //      accumulated in registers; the partial outputs of the eight warps are summed at the end ---------------------
  float oacc[V / 8][4];
#pragma unroll
  for (int nt = 0; nt < V / 8; ++nt) oacc[nt][0] = oacc[nt][1] = oacc[nt][2] = oacc[nt][3] = 0.f;
  const bf16* P = reinterpret_cast<const bf16*>(S);
  const int ldp = 2 * lds;
  for (int st = 0; st < nst; ++st) {
    const int j = nst + st, slot = j % kStrSlots;
    const bf16* vst = reinterpret_cast<const bf16*>(ring + slot * kSlotBytes) + (size_t)8 * warp * ldk;
    NHA_WAIT_LOAD(j, min(nloads, kStrSlots + j));
    __syncwarp();
    uint32_t pa[2];
    ldsm_x2(pa, P + (size_t)(lane & 15) * ldp + st * kStrStage + 8 * warp);
#pragma unroll
    for (int n4 = 0; n4 < V / 32; ++n4) {
      uint32_t vb[4];                                              // my 8 keys x 32 value columns, transposed
      ldsm_x4_trans(vb, vst + (lane & 7) * ldk + 32 * n4 + 8 * (lane >> 3));
#pragma unroll
      for (int t = 0; t < 4; ++t) mma_1688(oacc[4 * n4 + t], pa[0], pa[1], vb[t]);
    }
    __syncwarp();
    if (j + kStrSlots < nloads) NHA_ISSUE_LOAD(j + kStrSlots);
  }
#undef NHA_ISSUE_LOAD
#undef NHA_WAIT_LOAD
  __syncthreads();                                                 // the logits / weights and the ring are dead
  float* osm = reinterpret_cast<float*>(ring);                     // [8 warps][16][V+8] window parts of the output
  {
    float* ow = osm + (size_t)warp * 16 * ldo + 2 * tq;
#pragma unroll
    for (int nt = 0; nt < V / 8; ++nt) {
      *reinterpret_cast<float2*>(ow + gq * ldo + 8 * nt) = make_float2(oacc[nt][0], oacc[nt][1]);
      *reinterpret_cast<float2*>(ow + (gq + 8) * ldo + 8 * nt) = make_float2(oacc[nt][2], oacc[nt][3]);
    }
  }

  __syncthreads();
  // partial output of this split: slot part + window part, unnormalised
  float* po = a.part_o + ((size_t)bh * SPL + sp) * NG * V;
#pragma unroll
  for (int u = 0; u < 2; ++u) {
    const int i = tid + u * kStrThreads;
    if (i < NG * V4) {
      const int qh = i / V4, c = i - qh * V4;
      float4 acc = sacc[u];
      if (nkeys > 0) {
#pragma unroll
        for (int w8 = 0; w8 < kStrWarps; ++w8) {
          const float4 wv = *reinterpret_cast<const float4*>(osm + ((size_t)w8 * 16 + qh) * ldo + 4 * c);
          acc.x += wv.x; acc.y += wv.y; acc.z += wv.z; acc.w += wv.w;
        }
      }
      if (SPL == 1) {
        const float inv = 1.0f / ml[2 * qh + 1];
        bf16* orow = a.o + ((size_t)b * a.HQ + h * NG + qh) * V + 4 * c;
        orow[0] = f2bf(acc.x * inv); orow[1] = f2bf(acc.y * inv); orow[2] = f2bf(acc.z * inv); orow[3] = f2bf(acc.w * inv);
      } else if (a.cluster) {
        *reinterpret_cast<float4*>(hvS + qh * V + 4 * c) = acc;      // my rows of hv are dead: the partial output goes there
      } else {
        *reinterpret_cast<float4*>(po + qh * V + 4 * c) = acc;
      }
    }
  }
  if (failed && tid == 0 && a.err) atomicExch(a.err, 1);
  if (SPL == 1) {
    append_token();
    return;
  }

  if (a.cluster) {
    // ---- merge inside the cluster: CTA 0 reads the partial outputs, maxima and sums of its peers from their shared
    //      memory; the second barrier keeps the peers' memory alive until it has ----------------------------------
    cluster_sync_all();
    if (sp == 0) {
      append_token();
#pragma unroll
      for (int u = 0; u < 2; ++u) {
        const int i = tid + u * kStrThreads;
        if (i < NG * V4) {
          const int qh = i / V4, c = i - qh * V4;
          float mx = -INFINITY;
          for (int s2 = 0; s2 < SPL; ++s2) mx = fmaxf(mx, ld_cluster_f2(cluster_map(ml + 2 * qh, s2)).x);
          float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
          float den = 0.f;
          for (int s2 = 0; s2 < SPL; ++s2) {
            const float2 t2 = ld_cluster_f2(cluster_map(ml + 2 * qh, s2));
            const float4 pv = ld_cluster_f4(cluster_map(hvS + qh * V + 4 * c, s2));
            const float w2 = t2.x > -INFINITY ? __expf(t2.x - mx) : 0.f;
            den += t2.y * w2;
            acc.x += w2 * pv.x; acc.y += w2 * pv.y; acc.z += w2 * pv.z; acc.w += w2 * pv.w;
          }
          const float inv = 1.0f / den;
          bf16* orow = a.o + ((size_t)b * a.HQ + h * NG + qh) * V + 4 * c;
          orow[0] = f2bf(acc.x * inv); orow[1] = f2bf(acc.y * inv); orow[2] = f2bf(acc.z * inv); orow[3] = f2bf(acc.w * inv);
        }
      }
    }
    cluster_sync_all();
    return;
  }

  // ---- merge: the last split of this (sequence, kv head) to arrive combines all partials ------------
  float* pml = a.part_ml + ((size_t)bh * SPL + sp) * NG * 2;
  for (int i = tid; i < NG * 2; i += kStrThreads) pml[i] = ml[i];
  __syncthreads();
  __shared__ int s_last;
  if (tid == 0) {
    __threadfence();                    // the partials of this CTA are visible before its ticket
    const int t = atomicAdd(a.tickets + bh, 1);
    s_last = (t == SPL - 1);
    if (s_last) a.tickets[bh] = 0;      // leave the counter at zero for the next call
  }
  __syncthreads();
  if (!s_last) return;
  __threadfence();
  append_token();
  const float* all_ml = a.part_ml + (size_t)bh * SPL * NG * 2;
  const float* all_o = a.part_o + (size_t)bh * SPL * NG * V;
  if (SPL <= 4) {
    // few splits: a thread fetches the maxima, sums and partial outputs of its element in one go (one trip to L2)
    // and forms the merge weights itself
#pragma unroll
    for (int u = 0; u < 2; ++u) {
      const int i = tid + u * kStrThreads;
      if (i < NG * V4) {
        const int qh = i / V4, c = i - qh * V4;
        float4 pv[4];
        float m2[4], l2[4];
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          if (s2 < SPL) {
            pv[s2] = __ldcg(reinterpret_cast<const float4*>(all_o + ((size_t)s2 * NG + qh) * V + 4 * c));
            const float2 t2 = __ldcg(reinterpret_cast<const float2*>(all_ml + ((size_t)s2 * NG + qh) * 2));
            m2[s2] = t2.x; l2[s2] = t2.y;
          } else {
            pv[s2] = make_float4(0.f, 0.f, 0.f, 0.f);
            m2[s2] = -INFINITY; l2[s2] = 0.f;
          }
        }
        const float mx = fmaxf(fmaxf(m2[0], m2[1]), fmaxf(m2[2], m2[3]));
        float wq[4], den = 0.f;
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          wq[s2] = m2[s2] > -INFINITY ? __expf(m2[s2] - mx) : 0.f;
          den += l2[s2] * wq[s2];
        }
        float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
        for (int s2 = 0; s2 < 4; ++s2) {
          const float w2 = wq[s2] / den;
          acc.x += w2 * pv[s2].x; acc.y += w2 * pv[s2].y; acc.z += w2 * pv[s2].z; acc.w += w2 * pv[s2].w;
        }
        bf16* orow = a.o + ((size_t)b * a.HQ + h * NG + qh) * V + 4 * c;
        orow[0] = f2bf(acc.x); orow[1] = f2bf(acc.y); orow[2] = f2bf(acc.z); orow[3] = f2bf(acc.w);
      }
    }
    return;
  }
  float* wgt = red;                     // [SPL][NG] merge weights exp(m_s - m) / denominator
  for (int qh = tid; qh < NG; qh += kStrThreads) {
    float mx = -INFINITY;
    for (int s2 = 0; s2 < SPL; ++s2) mx = fmaxf(mx, __ldcg(all_ml + ((size_t)s2 * NG + qh) * 2));
    float den = 0.f;
    for (int s2 = 0; s2 < SPL; ++s2) {
      const float m2 = __ldcg(all_ml + ((size_t)s2 * NG + qh) * 2);
      const float l2 = __ldcg(all_ml + ((size_t)s2 * NG + qh) * 2 + 1);
      den += m2 > -INFINITY ? l2 * __expf(m2 - mx) : 0.f;
    }
    for (int s2 = 0; s2 < SPL; ++s2) {
      const float m2 = __ldcg(all_ml + ((size_t)s2 * NG + qh) * 2);
      wgt[s2 * NG + qh] = m2 > -INFINITY ? __expf(m2 - mx) / den : 0.f;
    }
  }
  __syncthreads();
  for (int i = tid; i < NG * V4; i += kStrThreads) {
    const int qh = i / V4, c = i - qh * V4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int s2 = 0; s2 < SPL; ++s2) {
      const float wq = wgt[s2 * NG + qh];
      const float4 pv = __ldcg(reinterpret_cast<const float4*>(all_o + ((size_t)s2 * NG + qh) * V + 4 * c));
      acc.x += wq * pv.x; acc.y += wq * pv.y; acc.z += wq * pv.z; acc.w += wq * pv.w;
    }
    bf16* orow = a.o + ((size_t)b * a.HQ + h * NG + qh) * V + 4 * c;
    orow[0] = f2bf(acc.x); orow[1] = f2bf(acc.y); orow[2] = f2bf(acc.z); orow[3] = f2bf(acc.w);
  }
}

static int stream_layout(DecodeStreamArgs& a, int D, int nkp) {
  const int NG = a.NG, MQ = a.MQ;
  int off = 0;
  auto take = [&](int bytes) { int o = off; off = (off + bytes + 127) / 128 * 128; return o; };
  a.off_ring = take(kStrSlots * kStrStage * (D + 8) * 2);
  a.off_hv = take(MQ * D * 4);
  const int s_bytes = 16 * (nkp + 8) * 4, red_bytes = kStrWarps * NG * 32 * 4;
  a.off_S = take(s_bytes > red_bytes ? s_bytes : red_bytes);
  a.off_red = a.off_S;                               // the partial slot logits are summed before the first S tile lands
  a.off_q = take(NG * D * 4);
  a.off_sqA = take(16 * (D + 8) * 2);
  a.off_oks = take(NG * MQ * 4);
  a.off_eg = take(MQ * 4);
  a.off_sv = take(MQ * 4);
  a.off_kpop = take(D * 4);
  a.off_vpop = take(D * 4);
  a.off_ml = take(NG * 2 * 4);
  a.off_bar = take((kStrSlots + 1) * 8);
  return off;
}

// Splits of a (sequence, kv head) for the streaming kernel: as many as keep the whole grid in one wave of two
// CTAs per SM, each split keeping at least 64 keys and 4 slots.
int decode_stream_splits(int B, int H, int W, int M) {
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  int spl = 1;
  while (spl < 16 && (int64_t)B * H * spl * 2 <= 2 * (int64_t)sms && W / (spl * 2) >= kStrStage && M / (spl * 2) >= 4 &&
         M % (spl * 2 * 4) == 0)
    spl *= 2;
  // a CTA keeps all logits of its key range in shared memory: very wide windows are split further (more than one wave
  // then) so that a split holds at most 512 keys
  while (spl < 16 && (W + spl - 1) / spl > 512 && M / (spl * 2) >= 4 && M % (spl * 2 * 4) == 0) spl *= 2;
  return spl;
}

// Mode of the programmatic dependent launch of the streaming kernel (see DecodeStreamArgs::pdl): set by
// nha_decode_set_pdl(), else taken once from the environment variable NHA_PDL (the reference's switch of the same
// name, nha_fla/ops/nha/fused_recurrent.py:32-34: "0" turns it off), default 1.
static std::atomic<int> g_pdl_mode{-1};
int decode_pdl_mode() {
  int m = g_pdl_mode.load(std::memory_order_relaxed);
  if (m < 0) {
    const char* e = getenv("NHA_PDL");
    m = 1;
    if (e && e[0] >= '0' && e[0] <= '2' && e[1] == 0) m = e[0] - '0';
    g_pdl_mode.store(m, std::memory_order_relaxed);
  }
  return m;
}
void decode_set_pdl_mode(int m) { g_pdl_mode.store(m, std::memory_order_relaxed); }

bool decode_stream_supported(int K, int V, int M, int W, int NG, bool logits_mode) {
  return !logits_mode && K == V && (K == 64 || K == 128) && M % 4 == 0 && M <= 128 && NG <= 16 && W >= 1;
}

// The caller has checked decode_stream_supported() and sized the workspace for `splits`.
int decode_stream_launch(const DecodeStreamArgs& in, int D, cudaStream_t st) {
  DecodeStreamArgs a = in;
  a.KSPL = ((a.W + a.SPLITS - 1) / a.SPLITS + kStrStage - 1) / kStrStage * kStrStage;
  a.MQ = ((a.M + a.SPLITS - 1) / a.SPLITS + 3) / 4 * 4;
  const int nkp = a.KSPL;
  const int smem = stream_layout(a, D, nkp);
  if (smem > kMaxSmem) return NHA_ERR_SMEM;
  dim3 grid(a.B * a.H * a.SPLITS), block(kStrThreads);
  // 2, 4 or 8 splits whose partial outputs fit the (dead) hv rows merge through the cluster's shared memory
  a.cluster = (a.SPLITS == 2 || a.SPLITS == 4 || a.SPLITS == 8) && a.NG <= a.MQ;
  if (const char* nc = getenv("NHA_B200_DECODE_NO_CLUSTER")) {
    if (nc[0] == '1') a.cluster = 0;                 // merge through the workspace instead
  }
  const void* fn = a.state_bf16 ? (D == 128 ? (const void*)nha_decode_stream_kernel<128, true> : (const void*)nha_decode_stream_kernel<64, true>)
                                : (D == 128 ? (const void*)nha_decode_stream_kernel<128, false>
                                            : (const void*)nha_decode_stream_kernel<64, false>);
  cudaError_t e = set_max_smem(fn, smem);
  if (e != cudaSuccess) return record_cuda_error(e);
  cudaLaunchConfig_t cfg;
  memset(&cfg, 0, sizeof(cfg));
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attr[2];
  attr[0].id = cudaLaunchAttributeClusterDimension;
  attr[0].val.clusterDim.x = a.cluster ? a.SPLITS : 1;
  attr[0].val.clusterDim.y = 1;
  attr[0].val.clusterDim.z = 1;
  a.pdl = decode_pdl_mode();
  attr[1].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attr[1].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attr;
  cfg.numAttrs = a.pdl ? 2 : 1;
  void* args[1] = {(void*)&a};
  e = cudaLaunchKernelExC(&cfg, fn, args);
  if (e != cudaSuccess && a.cluster) {
    // the device could not place the cluster (partitioned GPU, ...): the same kernel merges through the workspace
    (void)cudaGetLastError();
    a.cluster = 0;
    attr[0].val.clusterDim.x = 1;
    e = cudaLaunchKernelExC(&cfg, fn, args);
  }
  if (e != cudaSuccess) return record_cuda_error(e);
  return check_launch();
}

// Runs the streaming kernel when the shape has one; *used tells the caller whether it did.
int decode_stream_try(const void* q, const void* sq, const void* k, const void* v, const void* g, const void* s,
                      const void* sw_k, const void* sw_v, const void* cosp, const void* sinp, int64_t cs_batch,
                      int64_t cs_row, float* hk, float* hv, int zero_state, void* o, int* tickets, int* err,
                      float* part_ml, float* part_o, int splits, int B, int HQ, int H, int D, int M, int W, float scale,
                      cudaStream_t st, const int* head, const void* ring_g, int ring_rows, int nopop,
                      const void* ring_kraw, const void* g_new, int state_bf16) {
  DecodeStreamArgs a;
  a.q = (const bf16*)q; a.sq = (const bf16*)sq; a.k = (const bf16*)k; a.v = (const bf16*)v; a.g = (const bf16*)g;
  a.s = (const bf16*)s; a.sw_k = (const bf16*)sw_k; a.sw_v = (const bf16*)sw_v; a.cosp = (const bf16*)cosp;
  a.sinp = (const bf16*)sinp;
  a.hk = hk; a.hv = hv; a.o = (bf16*)o;
  a.part_o = part_o; a.part_ml = part_ml; a.tickets = tickets; a.err = err;
  a.head = head; a.ring_g = (const bf16*)ring_g;
  a.WR = head ? ring_rows : W; a.nopop = head ? nopop : 0;
  a.ring_kraw = head ? (const bf16*)ring_kraw : nullptr;
  a.g_new = (head && !ring_kraw) ? (const bf16*)g_new : nullptr;
  a.state_bf16 = state_bf16;
  a.cs_batch = cs_batch; a.cs_row = cs_row;
  a.B = B; a.HQ = HQ; a.H = H; a.M = M; a.W = W; a.NG = HQ / H; a.SPLITS = splits;
  a.zero_state = zero_state; a.scale = scale;
  return decode_stream_launch(a, D, st);
}

}  // namespace nha
