// State pass, per-chunk terms on the tensor cores (sm_100a): TMA loads, tcgen05 products, accumulators in tensor memory.
//
// One CTA per (chunk, kv head) forms, for K == V in {64, 128} and M == 64,
//     E[r,m]  = sum_{i > r} g'[i,m]                    (log decay from row r to the end of the chunk)
//     sb[r,m] = s'[r,m] exp(E[r,m])
//     L_k = k'^T sb  [K x M],   L_v = sb^T v'  [M x V],   Gend[m] = E[0,m] + g'[0,m]
// (primes: rows shifted right by gsa_kv_shift inside their sequence).  The running sum over rows is itself a matrix
// product, E = U g' with U the strictly upper triangular matrix of ones, so no thread scans anything: the gate tile
// goes from global memory to the tensor core without passing through registers, and bf16 gates times 1.0 summed in
// fp32 are exact up to the order of the additions.  All four inputs arrive by TMA into 128-byte-swizzled tiles that
// the products read in place (k', v', g', sb as MN-major operands: the token index is the contraction dimension of
// every product).  The wmma version of this kernel (nha_state_local_kernel) was bound by shared-memory bandwidth
// (fragment loads); this one touches shared memory from threads only for the 8 KB weight tile.
//
// Chunks whose rows are not all inside their sequence (the first chunks of a shifted sequence, a ragged last chunk,
// a sequence start inside a packed buffer) are filled by the threads with zero fill instead of TMA, so that no row of
// a neighbouring sequence enters a product.
//
// Same outputs as nha_state_local_kernel: L [NCB*H][K*M + M*V] bf16 and Gend [NCB*H][M] fp32 in the state scratch,
// consumed by nha_state_scan_kernel.  Replaces the per-chunk part of chunk_nha_fused_state_kernel
// (nha_fla/ops/nha/chunk_fused.py:31-114).
#include <cstdlib>
#include <cstring>

#include "nha_common.cuh"
#include "nha_tma.cuh"
#include "nha_umma.cuh"

namespace nha {

using namespace umma;

namespace stu {
constexpr int kThreads = 128;
constexpr int kTile = 8192;        // one [64][64] bf16 operand tile
constexpr int kTmemCols = 128;     // E then L_k in columns 0-63, a 64-column half of L_v in columns 64-127
constexpr int kPoll = 1 << 12;     // polls of at most kWaitHintNs each before a wait gives up
}  // namespace stu

struct StateMaps {
  CUtensorMap k, v, g, s;
};

template <int D>
__global__ void __launch_bounds__(stu::kThreads) nha_state_local_umma_kernel(const nha_chunk_desc d, const StateWs w,
                                                                             int* __restrict__ err, const int chunk_lo,
                                                                             const __grid_constant__ StateMaps maps) {
  using namespace stu;
  constexpr int DT = D / 64;                      // 64-column tiles of k' and v'
  constexpr int M = 64;
  const int cg = chunk_lo + blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  if (rc.n < 0) return;
  const int H = d.H;
  const int t0 = rc.t0, len = rc.len, p0 = rc.ci * kChunk;
  const int shift = seq_shift(d, rc.n);
  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;

  extern __shared__ unsigned char smem_raw[];
  unsigned char* sm = (unsigned char*)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
  unsigned char* sU = sm;                         // strictly upper triangular ones [64][64], K-major
  unsigned char* sG = sm + kTile;                 // g' [64 rows][64 slots]
  unsigned char* sS = sm + 2 * kTile;             // s', overwritten by sb
  unsigned char* sK = sm + 3 * kTile;             // k' [64 rows][D] as DT tiles
  unsigned char* sV = sK + DT * kTile;
  uint64_t* bar = (uint64_t*)(sV + DT * kTile);   // [0] loads, [1] products
  uint32_t* tslot = (uint32_t*)(bar + 2);
  __shared__ int s_abort;

  if (warp == 0) tmem_alloc(tslot, kTmemCols);
  if (tid == 32) {
    mbar_init(&bar[0], 1);
    mbar_init(&bar[1], 1);
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    s_abort = *(volatile int*)err;                // an earlier CTA of this launch gave up on a wait: do not start
  }
  if (tid < 64) {
    // row r of U: ones right of the diagonal
#pragma unroll
    for (int c = 0; c < 8; ++c) {
      uint32_t pr[4];
#pragma unroll
      for (int e = 0; e < 4; ++e) {
        const int i = 8 * c + 2 * e;
        pr[e] = (i > tid ? 0x3F80u : 0u) | (i + 1 > tid ? 0x3F800000u : 0u);
      }
      *reinterpret_cast<uint4*>(sU + sw_off(tid, c)) = make_uint4(pr[0], pr[1], pr[2], pr[3]);
    }
  }
  // rows of the chunk hold shifted positions p = p0 + r, token p - shift; valid while shift <= p < len
  const bool full = p0 >= shift && p0 + kChunk <= len;
  const int64_t row0 = (int64_t)t0 + p0 - shift;  // packed row of the chunk's first row
  if (!full) {
    // zero-filling copies by the threads: 16-byte pieces into the swizzled tiles
    auto fill = [&](unsigned char* dst, const bf16* base, int width, int col0) {
      for (int i = tid; i < kChunk * 8; i += kThreads) {
        const int r = i >> 3, c = i & 7;
        const int p = p0 + r;
        uint4 val = make_uint4(0u, 0u, 0u, 0u);
        if (p >= shift && p < len) val = *reinterpret_cast<const uint4*>(base + ((row0 + r) * H + h) * width + col0 + 8 * c);
        *reinterpret_cast<uint4*>(dst + sw_off(r, c)) = val;
      }
    };
    fill(sG, (const bf16*)d.g, M, 0);
    fill(sS, (const bf16*)d.s, M, 0);
#pragma unroll
    for (int kt = 0; kt < DT; ++kt) {
      fill(sK + kt * kTile, (const bf16*)d.k_gsa, D, 64 * kt);
      fill(sV + kt * kTile, (const bf16*)d.v, D, 64 * kt);
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  tc_fence_after();
  const uint32_t tbase = *tslot;
  if (s_abort) {
    if (warp == 0) tmem_dealloc(tbase, kTmemCols);
    return;
  }
  bool failed = false;
  if (full && tid == 0) {
    mbar_expect_tx(&bar[0], (2 + 2 * DT) * kTile);
    tma_load_3d(sG, &maps.g, 0, h, (int)row0, &bar[0]);
    tma_load_3d(sS, &maps.s, 0, h, (int)row0, &bar[0]);
#pragma unroll
    for (int kt = 0; kt < DT; ++kt) {
      tma_load_3d(sK + kt * kTile, &maps.k, 64 * kt, h, (int)row0, &bar[0]);
      tma_load_3d(sV + kt * kTile, &maps.v, 64 * kt, h, (int)row0, &bar[0]);
    }
  }
  // every thread observes the arrival of the tiles itself (it reads the weight tile with ordinary loads later)
  if (full && !mbar_wait_limit(&bar[0], 0, kPoll)) failed = true;
  if (tid == 0 && !failed) {
    tc_fence_after();
    mma_tile_ex(tbase, smem_u32(sU), 0, 0, smem_u32(sG), 0, 1, 64, 64, 4, false);
    commit(&bar[1]);
  }
  if (!failed && !mbar_wait_limit(&bar[1], 0, kPoll)) failed = true;
  tc_fence_after();
  // E is an M = 64 accumulator: row 16 w + l sits in lane l < 16 of warp w's lane quarter
  const uint32_t tl = tbase + ((uint32_t)(warp * 32) << 16);
  const int r = 16 * warp + lane;
  {
    float e[64];
    tmem_ld64(tl, e);
    if (lane < 16 && !failed) {
      if (r == 0) {
        float* ge = w.gend + ((size_t)cg * H + h) * M;
#pragma unroll
        for (int c = 0; c < 8; ++c) {
          float g0[8];
          unpack8(*reinterpret_cast<const uint4*>(sG + sw_off(0, c)), g0);
          *reinterpret_cast<float4*>(ge + 8 * c) = make_float4(e[8 * c] + g0[0], e[8 * c + 1] + g0[1], e[8 * c + 2] + g0[2],
                                                                e[8 * c + 3] + g0[3]);
          *reinterpret_cast<float4*>(ge + 8 * c + 4) = make_float4(e[8 * c + 4] + g0[4], e[8 * c + 5] + g0[5],
                                                                    e[8 * c + 6] + g0[6], e[8 * c + 7] + g0[7]);
        }
      }
#pragma unroll
      for (int c = 0; c < 8; ++c) {
        uint4* cell = reinterpret_cast<uint4*>(sS + sw_off(r, c));
        float sv[8];
        unpack8(*cell, sv);
#pragma unroll
        for (int i = 0; i < 8; ++i) sv[i] *= __expf(e[8 * c + i]);
        *cell = pack8(sv);
      }
    }
  }
  fence_async_smem();
  tc_fence_before();
  __syncthreads();
  if (tid == 0 && !failed) {
    tc_fence_after();
    // L_k [D x 64] = k'^T sb: both operands MN-major, 16 tokens per k step; with D = 128 the A operand spans two
    // 64-column tiles, kTile bytes apart (LBO)
    const uint32_t idk = make_idesc(D, 64, 1) | (1u << 15);
    const uint32_t idv = make_idesc(64, 64, 1) | (1u << 15);
#pragma unroll
    for (int ks = 0; ks < 4; ++ks) {
      mma_f16(tbase, make_desc_lbo(smem_u32(sK) + ks * 2048, kTile), make_desc(smem_u32(sS) + ks * 2048), idk, ks > 0);
      // L_v [64 x 64] (columns 0-63 of V) = sb^T v'
      mma_f16(tbase + 64, make_desc(smem_u32(sS) + ks * 2048), make_desc(smem_u32(sV) + ks * 2048), idv, ks > 0);
    }
    commit(&bar[1]);
  }
  if (!failed && !mbar_wait_limit(&bar[1], 1, kPoll)) failed = true;
  tc_fence_after();
  bf16* Lk = w.local + ((size_t)cg * H + h) * ((size_t)D * M + (size_t)M * D);
  bf16* Lv = Lk + (size_t)D * M;
  auto store_row = [&](uint32_t taddr, bf16* dst, bool active) {
    float x[64];
    tmem_ld64(taddr, x);
    if (active && !failed) {
#pragma unroll
      for (int c = 0; c < 8; ++c) *reinterpret_cast<uint4*>(dst + 8 * c) = pack8(x + 8 * c);
    }
  };
  if (D == 128) store_row(tl, Lk + (size_t)tid * M, true);                 // M = 128 accumulator: row = lane
  else store_row(tl, Lk + (size_t)r * M, lane < 16);
  store_row(tl + 64, Lv + (size_t)r * D, lane < 16);
  if (DT == 2) {
    tc_fence_before();
    __syncthreads();
    if (tid == 0 && !failed) {
      tc_fence_after();
      const uint32_t idv = make_idesc(64, 64, 1) | (1u << 15);
#pragma unroll
      for (int ks = 0; ks < 4; ++ks)
        mma_f16(tbase, make_desc(smem_u32(sS) + ks * 2048), make_desc(smem_u32(sV) + kTile + ks * 2048), idv, ks > 0);
      commit(&bar[1]);
    }
    if (!failed && !mbar_wait_limit(&bar[1], 0, kPoll)) failed = true;
    tc_fence_after();
    store_row(tl, Lv + (size_t)r * D + 64, lane < 16);
  }
  if (failed) atomicExch(err, 1);
  tc_fence_before();
  __syncthreads();
  if (warp == 0) tmem_dealloc(tbase, kTmemCols);
}

bool state_local_umma_supported(const nha_chunk_desc* d) {
  if (d->K != d->V || (d->K != 64 && d->K != 128) || d->M != 64) return false;
  const char* off = getenv("NHA_B200_NO_UMMA");
  if (off && off[0] == '1') return false;
  off = getenv("NHA_B200_NO_STATE_UMMA");
  return !(off && off[0] == '1');
}

// Launches the tensor-core version of the per-chunk terms; NHA_ERR_UNSUPPORTED when the tensor maps cannot be made (the
// caller then runs nha_state_local_kernel).
int state_local_umma_launch(const nha_chunk_desc* d, const StateWs& w, int* err, int chunk_lo, int chunk_n, cudaStream_t cs) {
  using namespace stu;
  StateMaps maps;
  memset(&maps, 0, sizeof(maps));
  const bool ok = make_map_rows_heads(&maps.k, d->k_gsa, d->Ttot, d->H, d->K) &&
                  make_map_rows_heads(&maps.v, d->v, d->Ttot, d->H, d->V) &&
                  make_map_rows_heads(&maps.g, d->g, d->Ttot, d->H, d->M) &&
                  make_map_rows_heads(&maps.s, d->s, d->Ttot, d->H, d->M);
  if (!ok) return NHA_ERR_UNSUPPORTED;
  const int DT = d->K / 64;
  const int total = 1024 + (3 + 2 * DT) * kTile + 64;
  const void* fn = DT == 2 ? (const void*)nha_state_local_umma_kernel<128> : (const void*)nha_state_local_umma_kernel<64>;
  cudaError_t e = set_max_smem(fn, total);
  if (e != cudaSuccess) return record_cuda_error(e);
  if (DT == 2) nha_state_local_umma_kernel<128><<<dim3(chunk_n, d->H), kThreads, total, cs>>>(*d, w, err, chunk_lo, maps);
  else nha_state_local_umma_kernel<64><<<dim3(chunk_n, d->H), kThreads, total, cs>>>(*d, w, err, chunk_lo, maps);
  return check_launch();
}

}  // namespace nha
