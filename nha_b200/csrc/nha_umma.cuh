// Thin wrappers over the sm_100a tensor-core path: tcgen05.mma with operands in 128-byte-swizzled
// shared memory and accumulators in tensor memory (TMEM), tcgen05.ld for the epilogues, mbarrier
// completion.  Layout facts used by the kernels (checked on B200 against a host reference):
//   * K-major operand tile [rows][64 bf16]: row r at (r/8)*1024 + (r%8)*128 bytes, its 16-byte chunk c
//     stored at chunk slot c ^ (r%8); descriptor SBO = 1024; a 16-element k step advances the start
//     address by 32 bytes.
//   * MN-major operand tile [k rows][64 bf16 along N]: same physical layout; descriptor SBO = 1024;
//     a 16-row k step advances the start address by 2048 bytes.
//   * D of an M = 128 product: row r in TMEM lane r.  D of an M = 64 product: row r in lane
//     (r/16)*32 + r%16 (each warp's 32-lane quarter holds 16 rows).
#pragma once

#include <cuda_bf16.h>
#include <stdint.h>

namespace nha {
namespace umma {

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ uint64_t make_desc(uint32_t saddr) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(1024 >> 4) << 16;   // LBO (not used by the single-atom-wide tiles here)
  d |= (uint64_t)(1024 >> 4) << 32;   // SBO: 8-row group pitch
  d |= (uint64_t)1 << 46;             // descriptor version of sm_100
  d |= (uint64_t)2 << 61;             // SWIZZLE_128B
  return d;
}

// same, with the byte distance between consecutive 64-element blocks along the MN dimension of an MN-major operand
// wider than one swizzle atom (N > 64) in the LBO field
__device__ __forceinline__ uint64_t make_desc_lbo(uint32_t saddr, uint32_t lbo_bytes) {
  uint64_t d = 0;
  d |= (uint64_t)((saddr & 0x3FFFF) >> 4);
  d |= (uint64_t)(lbo_bytes >> 4) << 16;
  d |= (uint64_t)(1024 >> 4) << 32;
  d |= (uint64_t)1 << 46;
  d |= (uint64_t)2 << 61;
  return d;
}

// kind::f16 instruction descriptor: bf16 x bf16 -> f32, A K-major, B K-major or MN-major
__device__ __forceinline__ uint32_t make_idesc(int M, int N, int b_mn_major) {
  uint32_t d = 0;
  d |= 1u << 4;                       // D = f32
  d |= 1u << 7;                       // A = bf16
  d |= 1u << 10;                      // B = bf16
  d |= (uint32_t)b_mn_major << 16;
  d |= (uint32_t)(N >> 3) << 17;
  d |= (uint32_t)(M >> 4) << 24;
  return d;
}

// byte offset of 16-byte chunk c of row r inside a swizzled [rows][64 bf16] tile
__device__ __forceinline__ int sw_off(int r, int c) { return (r >> 3) * 1024 + (r & 7) * 128 + ((c ^ (r & 7)) << 4); }

__device__ __forceinline__ void mma_f16(uint32_t d_tmem, uint64_t adesc, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
      "l"(adesc), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// the same with the A operand in tensor memory: a_tmem addresses M lanes x 8 columns, each column holding two
// consecutive bf16 elements of the row along k (the lower half first)
__device__ __forceinline__ void mma_f16_ta(uint32_t d_tmem, uint32_t a_tmem, uint64_t bdesc, uint32_t idesc, bool accumulate) {
  const uint32_t acc = accumulate ? 1u : 0u;
  asm volatile(
      "{\n.reg .pred p;\nsetp.ne.b32 p, %4, 0;\n"
      "tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], %2, %3, p;\n}\n" ::"r"(d_tmem),
      "r"(a_tmem), "l"(bdesc), "r"(idesc), "r"(acc)
      : "memory");
}

// D[M x N] (+)= A[M x 16*ksteps] * B: A K-major tile(s), B K-major (b_mn = 0) or MN-major (b_mn = 1).
// a_tile_bytes / b_tile_bytes: distance between consecutive 64-wide k tiles of the operand.
__device__ __forceinline__ void mma_tile(uint32_t d_tmem, uint32_t a_addr, int a_tile_bytes, uint32_t b_addr,
                                         int b_tile_bytes, int M, int N, int ksteps, int b_mn, bool accumulate) {
  const uint32_t idesc = make_idesc(M, N, b_mn);
  for (int ks = 0; ks < ksteps; ++ks) {
    const int kt = ks >> 2, kin = ks & 3;
    const uint64_t da = make_desc(a_addr + kt * a_tile_bytes + kin * 32);
    const uint64_t db = b_mn ? make_desc(b_addr + ks * 2048) : make_desc(b_addr + kt * b_tile_bytes + kin * 32);
    mma_f16(d_tmem, da, db, idesc, accumulate || ks > 0);
  }
}

// KS k steps of one product with the operand descriptors formed once: a k step advances the start-address field
// (bits 0-13, units of 16 bytes) by 2 inside a 64-wide k tile of a K-major operand, by tile16 (tile bytes / 16) from
// one k tile to the next, and by 128 (16 k rows) for an MN-major B.  A is K-major.
template <int KS, int BMN>
__device__ __forceinline__ void mma_run(uint32_t d_tmem, uint64_t da, uint32_t a_tile16, uint64_t db, uint32_t b_tile16,
                                        uint32_t idesc, bool accumulate) {
#pragma unroll
  for (int ks = 0; ks < KS; ++ks) {
    const uint32_t kt = ks >> 2, kin = ks & 3;
    const uint64_t a = da + (uint64_t)(kt * a_tile16 + kin * 2);
    const uint64_t b = BMN ? db + (uint64_t)(ks * 128) : db + (uint64_t)(kt * b_tile16 + kin * 2);
    mma_f16(d_tmem, a, b, idesc, accumulate || ks > 0);
  }
}

// General form: either operand K-major (mn = 0: 64-wide k tiles `tile_bytes` apart, 32 bytes per k step)
// or MN-major (mn = 1: 16 k rows = 2048 bytes per k step).
__device__ __forceinline__ void mma_tile_ex(uint32_t d_tmem, uint32_t a_addr, int a_tile_bytes, int a_mn, uint32_t b_addr,
                                            int b_tile_bytes, int b_mn, int M, int N, int ksteps, bool accumulate) {
  const uint32_t idesc = make_idesc(M, N, b_mn) | ((uint32_t)a_mn << 15);
  for (int ks = 0; ks < ksteps; ++ks) {
    const int kt = ks >> 2, kin = ks & 3;
    const uint64_t da = a_mn ? make_desc(a_addr + ks * 2048) : make_desc(a_addr + kt * a_tile_bytes + kin * 32);
    const uint64_t db = b_mn ? make_desc(b_addr + ks * 2048) : make_desc(b_addr + kt * b_tile_bytes + kin * 32);
    mma_f16(d_tmem, da, db, idesc, accumulate || ks > 0);
  }
}

// Several products issued with their k steps interleaved.  The k steps of ONE product accumulate into the same
// tensor-memory columns, so each waits for the one before it; a product of a few small k steps is therefore bound
// by the latency of the instruction, not by the tensor pipe, and independent products issued one after the other
// add their latencies up.  Issuing step ks of every product before step ks + 1 of any lets the chains overlap.
// (Products that accumulate into the same columns must be given as ONE chain: list them in order with the same d
// and accumulate = true on the later ones; they are issued in list order within each step, which keeps them
// ordered because the hardware executes one thread's MMAs in issue order.)
struct MmaOp {
  uint32_t d;        // tensor-memory column address of the accumulator
  uint32_t a, b;     // shared-memory addresses of the operands
  int a_tile, b_tile;   // bytes between consecutive 64-wide k tiles of a K-major operand
  int a_mn, b_mn;    // 1: operand is MN-major (16 k rows = 2048 bytes per k step)
  int N, ksteps;
  bool acc;          // accumulate onto what the columns already hold
};

template <int NOPS>
__device__ __forceinline__ void mma_interleaved(const MmaOp (&ops)[NOPS], int M) {
  int kmax = 0;
#pragma unroll
  for (int i = 0; i < NOPS; ++i) kmax = ops[i].ksteps > kmax ? ops[i].ksteps : kmax;
  for (int ks = 0; ks < kmax; ++ks) {
    const int kt = ks >> 2, kin = ks & 3;
#pragma unroll
    for (int i = 0; i < NOPS; ++i) {
      if (ks < ops[i].ksteps) {
        const uint32_t idesc = make_idesc(M, ops[i].N, ops[i].b_mn) | ((uint32_t)ops[i].a_mn << 15);
        const uint64_t da = ops[i].a_mn ? make_desc(ops[i].a + ks * 2048) : make_desc(ops[i].a + kt * ops[i].a_tile + kin * 32);
        const uint64_t db = ops[i].b_mn ? make_desc(ops[i].b + ks * 2048) : make_desc(ops[i].b + kt * ops[i].b_tile + kin * 32);
        mma_f16(ops[i].d, da, db, idesc, ops[i].acc || ks > 0);
      }
    }
  }
}

__device__ __forceinline__ void commit(uint64_t* mbar) {
  asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(mbar))
               : "memory");
}

__device__ __forceinline__ void mbar_init(uint64_t* mbar, int count) {
  asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(mbar)), "r"(count));
}

// Bounded wait on an mbarrier phase; returns false when the limit is hit (the caller records an
// error and leaves instead of spinning forever).  Every try_wait carries a suspend-time hint: the thread sleeps in
// hardware until the phase completes or the hint runs out, instead of re-issuing the poll - waiting threads then leave
// the issue slots to the warps (and the other CTA of the SM) that have work.  `limit` polls of at most kWaitHintNs each.
constexpr uint32_t kWaitHintNs = 20000;
__device__ __forceinline__ bool mbar_wait_limit(uint64_t* mbar, uint32_t parity, int limit) {
  uint32_t done = 0;
  for (int it = 0; it < limit && !done; ++it) {
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(smem_u32(mbar)), "r"(parity), "r"(kWaitHintNs)
        : "memory");
  }
  return done != 0;
}
__device__ __forceinline__ bool mbar_wait(uint64_t* mbar, uint32_t parity) { return mbar_wait_limit(mbar, parity, 1 << 15); }
// Packed fp32 pairs (one instruction for two lanes of arithmetic) and the three-input maximum: the element-wise loops of
// the softmax threads are bound by instruction count, and these halve it for the multiply-adds, sums and maxima.
__device__ __forceinline__ float max3(float a, float b, float c) {
  float d;
  asm("max.f32 %0, %1, %2, %3;" : "=f"(d) : "f"(a), "f"(b), "f"(c));
  return d;
}
__device__ __forceinline__ uint64_t pack2(float a, float b) {
  uint64_t d;
  asm("mov.b64 %0, {%1, %2};" : "=l"(d) : "f"(a), "f"(b));
  return d;
}
__device__ __forceinline__ void unpack2(uint64_t v, float& a, float& b) {
  asm("mov.b64 {%0, %1}, %2;" : "=f"(a), "=f"(b) : "l"(v));
}
__device__ __forceinline__ uint64_t ffma2(uint64_t a, uint64_t b, uint64_t c) {
  uint64_t d;
  asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
  return d;
}
__device__ __forceinline__ uint64_t fadd2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}
__device__ __forceinline__ uint64_t fmul2(uint64_t a, uint64_t b) {
  uint64_t d;
  asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
  return d;
}

// one non-blocking test of an mbarrier phase
__device__ __forceinline__ bool mbar_test(uint64_t* mbar, uint32_t parity) {
  uint32_t done;
  asm volatile(
      "{\n.reg .pred p;\nmbarrier.test_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
      : "=r"(done)
      : "r"(smem_u32(mbar)), "r"(parity)
      : "memory");
  return done != 0;
}

__device__ __forceinline__ void fence_async_smem() { asm volatile("fence.proxy.async.shared::cta;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

__device__ __forceinline__ void tmem_alloc(uint32_t* slot, int cols) {
  asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(slot)), "r"(cols)
               : "memory");
  asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t base, int cols) {
  asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(base), "r"(cols) : "memory");
}

// 32 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, float* out) {
  uint32_t r[32];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 32; ++i) out[i] = __uint_as_float(r[i]);
}

// the same load without the wait: several loads can be in flight before one tmem_ld_wait()
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t* r) {
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,"
      "%30,%31}, [%32];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15]), "=r"(r[16]),
        "=r"(r[17]), "=r"(r[18]), "=r"(r[19]), "=r"(r[20]), "=r"(r[21]), "=r"(r[22]), "=r"(r[23]), "=r"(r[24]),
        "=r"(r[25]), "=r"(r[26]), "=r"(r[27]), "=r"(r[28]), "=r"(r[29]), "=r"(r[30]), "=r"(r[31])
      : "r"(taddr)
      : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }
// 64 consecutive fp32 columns of this thread's TMEM lane, one wait for both halves
__device__ __forceinline__ void tmem_ld64(uint32_t taddr, float* out) {
  uint32_t* r = reinterpret_cast<uint32_t*>(out);
  tmem_ld32_nowait(taddr, r);
  tmem_ld32_nowait(taddr + 32, r + 32);
  tmem_ld_wait();
}

// 16 consecutive fp32 columns of this thread's TMEM lane
__device__ __forceinline__ void tmem_ld16(uint32_t taddr, float* out) {
  uint32_t r[16];
  asm volatile(
      "tcgen05.ld.sync.aligned.32x32b.x16.b32 "
      "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15}, [%16];"
      : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]), "=r"(r[4]), "=r"(r[5]), "=r"(r[6]), "=r"(r[7]), "=r"(r[8]),
        "=r"(r[9]), "=r"(r[10]), "=r"(r[11]), "=r"(r[12]), "=r"(r[13]), "=r"(r[14]), "=r"(r[15])
      : "r"(taddr)
      : "memory");
  asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
  for (int i = 0; i < 16; ++i) out[i] = __uint_as_float(r[i]);
}

// W consecutive fp32 columns (W = 16 or 32)
template <int W>
__device__ __forceinline__ void tmem_ldw(uint32_t taddr, float* out) {
  if constexpr (W == 32) tmem_ld32(taddr, out);
  else tmem_ld16(taddr, out);
}

// ---- asynchronous 16-byte copies into swizzled tiles (NT-thread CTAs) ------------------------------
__device__ __forceinline__ void cp16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_commit() { asm volatile("cp.async.commit_group;\n" ::); }
__device__ __forceinline__ void cp_wait_all() { asm volatile("cp.async.wait_group 0;\n" ::); }
// wait until at most the newest committed group is still in flight
__device__ __forceinline__ void cp_wait_but_one() { asm volatile("cp.async.wait_group 1;\n" ::); }

// Asynchronously copy `rows` x COLS bf16 (global rows row0.., stride gstride elements; rows outside
// [lo, hi) become zeros) into COLS/64 swizzled tiles of `tile_bytes` each, starting at tile row dst_row0.
template <int COLS, int NT = 128>
__device__ __forceinline__ void load_sw(unsigned char* tile, int tile_bytes, const bf16* base, int64_t gstride, int row0,
                                        int lo, int hi, int rows, int dst_row0, int tid) {
  constexpr int C8 = COLS / 8;
  for (int i = tid; i < rows * C8; i += NT) {
    const int r = i / C8, c = i % C8;
    const int gr = row0 + r;
    const bool ok = gr >= lo && gr < hi;
    const bf16* src = base + (int64_t)(ok ? gr : lo) * gstride + 8 * c;
    cp16(tile + (c >> 3) * tile_bytes + sw_off(dst_row0 + r, c & 7), src, ok);
  }
}


}  // namespace umma
}  // namespace nha
