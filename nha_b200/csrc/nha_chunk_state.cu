// Chunk plan and state pass of the chunked NHA kernels (sm_100a).
//
// The slot memory obeys a per-element linear recurrence
//     hk[k,m] <- hk[k,m] * exp(g'[m]) + k'[k] * s'[m],   hv[m,v] <- hv[m,v] * exp(g'[m]) + s'[m] * v'[v]
// (primes = inputs shifted right by gsa_kv_shift inside their sequence).  Over one chunk this is
//     h_end = h_start .* exp(Gend) + L,   L_k = k'^T (s' exp(Gend - G)),  L_v = (s' exp(Gend - G))^T v',
// with G the running sum of g' inside the chunk and Gend its total.  L and Gend depend on their own
// chunk only, so a chunk-parallel kernel produces them with two 64-deep matrix products per
// (chunk, kv head), and what remains of the march is an element-wise scan over the chunks that stores
// the state at every chunk start (bf16, the operand type of the later matrix products) and the fp32
// final state.  Every exponent is <= 0, so no reference point is needed.  The chunk-parallel kernel of this file
// (nha_state_local_kernel, wmma) serves every shape; K == V in {64, 128} with M == 64 takes the tensor-core version in
// nha_chunk_state_umma.cu.  The scan streams the per-chunk terms through a ring of bulk copies (nha_tma.cuh).
//
// Replaces chunk_nha_fused_state_kernel (nha_fla/ops/nha/chunk_fused.py:31-114) and the state part of
// fla's chunk_gsa_fwd reached from nha_fla/ops/nha/chunk_gsa.py:38-45; the in-sequence shift replaces
// _packed_shift_right / _batch_shift_right (nha_fla/ops/nha/chunk.py:53-111).
#include <algorithm>
#include <mutex>

#include "nha_common.cuh"
#include "nha_tma.cuh"
#include "nha_umma.cuh"

namespace nha {

bool state_local_umma_supported(const nha_chunk_desc* d);
int state_local_umma_launch(const nha_chunk_desc* d, const StateWs& w, int* err, int chunk_lo, int chunk_n, cudaStream_t cs);

constexpr int kStThreads = 256;
constexpr int kStWarps = kStThreads / 32;

// ---------------------------------------------------------------------------------------------
__global__ void nha_plan_kernel(const int32_t* __restrict__ cu, int32_t* __restrict__ plan, int N, int NCB, int H) {
  if (threadIdx.x == 0) plan[N + 1 + NCB + (size_t)NCB * H] = 0;   // device-side error word
  // plan[0..N]: first chunk of each sequence; plan[N+1+c]: sequence of chunk c (-1 = unused)
  __shared__ int total;
  if (threadIdx.x == 0) {
    int acc = 0;
    for (int n = 0; n < N; ++n) {
      plan[n] = acc;
      const int len = cu[n + 1] - cu[n];
      acc += (len + kChunk - 1) / kChunk;
    }
    plan[N] = acc;
    total = acc;
  }
  __syncthreads();
  for (int c = total + threadIdx.x; c < NCB; c += blockDim.x) plan[N + 1 + c] = -1;
  int4* rec = reinterpret_cast<int4*>(plan + plan_rec_offset(N, NCB, H));
  for (int c = total + threadIdx.x; c < NCB; c += blockDim.x) rec[c] = make_int4(-1, 0, 0, 0);
  // one thread per chunk: its sequence is the last one whose first chunk is <= c (binary search over plan[0..N])
  for (int c = threadIdx.x; c < total; c += blockDim.x) {
    int lo = 0, hi = N - 1;
    while (lo < hi) {
      const int mid = (lo + hi + 1) >> 1;
      if (plan[mid] <= c) lo = mid; else hi = mid - 1;
    }
    while (lo + 1 < N && plan[lo + 1] <= c) ++lo;      // empty sequences share their first chunk with the next one
    plan[N + 1 + c] = lo;
    rec[c] = make_int4(lo, c - plan[lo], cu[lo], cu[lo + 1] - cu[lo]);
  }
}

// ---------------------------------------------------------------------------------------------
// C[Mt*16 x Nt*16] = A^T B as tile_gemm<false, true, false>, with the fp32 accumulator tiles rounded to bf16 on their way
// to global memory: a warp parks its 16 x 16 tile in its own 1 KB patch of shared memory and writes it out as 16 rows
// of 32 bytes (whole sectors).
__device__ __forceinline__ void tile_gemm_tn_bf16(bf16* C, int ldc, const bf16* A, int lda, const bf16* B, int ldb, int Mt,
                                                  int Nt, int Kt, int warp, int nwarps, float* patch) {
  using namespace nvcuda::wmma;
  const int lane = threadIdx.x & 31;
  float* mine = patch + warp * 256;
  for (int t = warp; t < Mt * Nt; t += nwarps) {
    const int mt = t / Nt, nt = t % Nt;
    fragment<accumulator, 16, 16, 16, float> acc;
    fill_fragment(acc, 0.0f);
    for (int kt = 0; kt < Kt; ++kt) {
      fragment<matrix_a, 16, 16, 16, bf16, col_major> fa;
      fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
      load_matrix_sync(fa, A + (size_t)kt * 16 * lda + mt * 16, lda);
      load_matrix_sync(fb, B + (size_t)kt * 16 * ldb + nt * 16, ldb);
      mma_sync(acc, fa, fb, acc);
    }
    store_matrix_sync(mine, acc, 16, mem_row_major);
    __syncwarp();
    const int r = lane >> 1, hf = lane & 1;
    *reinterpret_cast<uint4*>(C + (size_t)(mt * 16 + r) * ldc + nt * 16 + 8 * hf) = pack8(mine + r * 16 + 8 * hf);
    __syncwarp();
  }
}

struct StLocalLayout { int kt, vt, sbe, G, patch, total; };
__host__ __device__ inline int st_up128(int x) { return (x + 127) & ~127; }
__host__ __device__ inline StLocalLayout st_local_layout(int K, int V, int M) {
  StLocalLayout L; int off = 0;
  L.kt = off; off = st_up128(off + kChunk * (K + 8) * 2);
  L.vt = off; off = st_up128(off + kChunk * (V + 8) * 2);
  L.sbe = off; off = st_up128(off + kChunk * (M + 8) * 2);
  L.G = off; off = st_up128(off + kChunk * (M + 4) * 4);
  L.patch = off; off = st_up128(off + kStWarps * 256 * 4);
  L.total = off;
  return L;
}

// One CTA per (chunk, kv head): L_k, L_v and Gend of that chunk.
__global__ void __launch_bounds__(kStThreads) nha_state_local_kernel(const nha_chunk_desc d, const StateWs w, const int chunk_lo) {
  const int cg = chunk_lo + blockIdx.x, h = blockIdx.y;
  const int NCB = gridDim.x;
  const ChunkRec rc = chunk_rec(d, cg);
  const int n = rc.n;
  if (n < 0) return;
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int t0 = rc.t0;
  const int len = rc.len;
  const int p0 = rc.ci * kChunk;                  // shifted position of row 0
  const int shift = seq_shift(d, n);
  const int tid = threadIdx.x, warp = tid >> 5;
  (void)NCB;

  extern __shared__ __align__(128) unsigned char smem[];
  const StLocalLayout L = st_local_layout(K, V, M);
  const int ldk = K + 8, ldv = V + 8, ldsb = M + 8, ldg = M + 4;
  bf16* kt = (bf16*)(smem + L.kt);
  bf16* vt = (bf16*)(smem + L.vt);
  bf16* sbe = (bf16*)(smem + L.sbe);
  float* G = (float*)(smem + L.G);

  // rows of the chunk hold shifted tokens j = p - shift; rows before the sequence start or past its
  // end contribute nothing.  Every global load of the CTA is issued up front: the gate and write-weight rows into
  // registers (the gates are scanned first, the weights are needed right after), the key and value tiles by
  // asynchronous copies that land while the scan runs.
  const int lo = shift, hi = len;                  // valid shifted positions p: lo <= p < hi
  constexpr int kMaxPieces = 4;                    // 16-byte pieces of a [64][M <= 128] bf16 tile per thread (256 threads)
  const int M8 = M / 8, npieces = kChunk * M8;
  uint4 greg[kMaxPieces], sreg[kMaxPieces];
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int i = tid + u * kStThreads;
    greg[u] = make_uint4(0u, 0u, 0u, 0u);
    sreg[u] = make_uint4(0u, 0u, 0u, 0u);
    if (i < npieces) {
      const int r = i / M8, c8 = i - r * M8;
      const int p = p0 + r, j = p - shift;
      if (j >= 0 && p < len) {
        greg[u] = *reinterpret_cast<const uint4*>((const bf16*)d.g + ((size_t)(t0 + j) * H + h) * M + 8 * c8);
        sreg[u] = *reinterpret_cast<const uint4*>((const bf16*)d.s + ((size_t)(t0 + j) * H + h) * M + 8 * c8);
      }
    }
  }
  {
    const bf16* kbase = (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * K - (size_t)shift * H * K;
    const bf16* vbase = (const bf16*)d.v + ((size_t)t0 * H + h) * V - (size_t)shift * H * V;
    const int K8 = K / 8, V8 = V / 8;
    for (int i = tid; i < kChunk * K8; i += kStThreads) {
      const int r = i / K8, c = i - r * K8;
      const int p = p0 + r;
      const bool ok = p >= lo && p < hi;
      umma::cp16(kt + r * ldk + 8 * c, kbase + (size_t)(ok ? p : lo) * H * K + 8 * c, ok);
    }
    for (int i = tid; i < kChunk * V8; i += kStThreads) {
      const int r = i / V8, c = i - r * V8;
      const int p = p0 + r;
      const bool ok = p >= lo && p < hi;
      umma::cp16(vt + r * ldv + 8 * c, vbase + (size_t)(ok ? p : lo) * H * V + 8 * c, ok);
    }
    umma::cp_commit();
  }
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int i = tid + u * kStThreads;
    if (i < npieces) {
      const int r = i / M8, c8 = i - r * M8;
      float gv[8];
      unpack8(greg[u], gv);
#pragma unroll
      for (int e = 0; e < 8; ++e) G[r * ldg + 8 * c8 + e] = gv[e];
    }
  }
  __syncthreads();
  // inclusive running sum down the rows: two threads per column, the second adds the first half's total
  {
    const int m = tid >> 1, half = tid & 1;
    if (m < M) {
      float run = 0.f;
#pragma unroll 8
      for (int r = half * 32; r < half * 32 + 32; ++r) {
        run += G[r * ldg + m];
        G[r * ldg + m] = run;
      }
    }
    __syncthreads();
    if (m < M && half == 1) {
      const float add = G[31 * ldg + m];
#pragma unroll 8
      for (int r = 32; r < 64; ++r) G[r * ldg + m] += add;
    }
    __syncthreads();
  }
  if (tid < M) w.gend[((size_t)cg * H + h) * M + tid] = G[(kChunk - 1) * ldg + tid];
#pragma unroll
  for (int u = 0; u < kMaxPieces; ++u) {
    const int i = tid + u * kStThreads;
    if (i < npieces) {
      const int r = i / M8, c8 = i - r * M8;
      float sv[8], out[8];
      unpack8(sreg[u], sv);
#pragma unroll
      for (int e = 0; e < 8; ++e) {
        const int m = 8 * c8 + e;
        out[e] = sv[e] * __expf(G[(kChunk - 1) * ldg + m] - G[r * ldg + m]);
      }
      *reinterpret_cast<uint4*>(sbe + r * ldsb + 8 * c8) = pack8(out);
    }
  }
  umma::cp_wait_all();
  __syncthreads();
  bf16* Lk = w.local + ((size_t)cg * H + h) * ((size_t)K * M + (size_t)M * V);
  bf16* Lv = Lk + (size_t)K * M;
  // L_k [K x M] = k'^T [K x 64] * sbe [64 x M];  L_v [M x V] = sbe^T [M x 64] * v' [64 x V]
  float* patch = (float*)(smem + L.patch);
  tile_gemm_tn_bf16(Lk, M, kt, ldk, sbe, ldsb, K / 16, M / 16, kChunk / 16, warp, kStWarps, patch);
  tile_gemm_tn_bf16(Lv, V, sbe, ldsb, vt, ldv, M / 16, V / 16, kChunk / 16, warp, kStWarps, patch);
}

// Forward scan over the chunks of one (sequence, kv head): stores the state at every chunk start and the final state.
// A CTA owns 1024 consecutive state elements (a thread four of them: one 8-byte bf16 store per chunk) and walks the
// chunks in order.  The recurrence is serial, its inputs are not: a producer thread streams the CTA's 2 KB slice of L
// and the chunk's gate totals through a ring of kScanStages stages of kScanGroup chunks each (one bulk copy per slice,
// completion counted on the stage's mbarrier), so that tens of chunks are in flight per CTA whatever the sequence
// length - with one long sequence and few heads there are only N*H*SD/1024 CTAs to keep the memory system busy.
constexpr int kScanGroup = 8;                     // chunks per ring stage (two copies each: at most 16 issuing lanes)
constexpr int kScanMaxStages = 10;
constexpr int kScanPoll = 1 << 12;
// ELEMS state elements per CTA (a thread owns four); bytes per chunk in a stage: the L slice, then up to 128 gate totals
__host__ __device__ constexpr int scan_slot_bytes(int elems) { return elems * 2 + 512; }
__host__ __device__ constexpr int scan_smem_bytes(int elems, int stages) {
  return stages * kScanGroup * scan_slot_bytes(elems) + 2 * kScanMaxStages * 8 + 16;
}

// bounded wait without a suspend-time hint: the consumers of the scan wait often and briefly
__device__ __forceinline__ bool scan_wait(uint64_t* mbar, uint32_t parity) {
  uint32_t done = 0;
  for (int it = 0; it < (1 << 22) && !done; ++it) {
    asm volatile(
        "{\n.reg .pred p;\nmbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\nselp.u32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(umma::smem_u32(mbar)), "r"(parity)
        : "memory");
  }
  return done != 0;
}

__device__ __forceinline__ void scan_bulk_g2s(void* dst, const void* src, uint32_t bytes, uint64_t* mbar) {
  asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(
                   umma::smem_u32(dst)),
               "l"(src), "r"(bytes), "r"(umma::smem_u32(mbar))
               : "memory");
}

template <int kScanElems>
__global__ void __launch_bounds__(kScanElems / 4 + 32) nha_state_scan_kernel(const nha_chunk_desc d, const StateWs w,
                                                                             int* __restrict__ err, const int kScanStages) {
  constexpr int kScanThreads = kScanElems / 4;      // consumer threads; one more warp hosts the producer
  constexpr int kScanSlot = scan_slot_bytes(kScanElems);
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int KM = K * M, MV = M * V;
  const size_t SD = (size_t)KM + MV;
  const size_t nh = blockIdx.x;                     // (sequence, kv head) in x: no 65535 limit on packed batches
  const int n = nh / H, h = nh % H;
  const int len = d.cu_seqlens[n + 1] - d.cu_seqlens[n];
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int chunk0 = d.plan[n];
  const int el0 = blockIdx.y * kScanElems;
  const int nel = min(kScanElems, (int)SD - el0);   // a multiple of 8: K, V and M are multiples of 16
  const int tid = threadIdx.x;
  extern __shared__ __align__(128) unsigned char scan_smem[];
  uint64_t* full = (uint64_t*)(scan_smem + kScanStages * kScanGroup * kScanSlot);
  uint64_t* empty = full + kScanMaxStages;
  volatile int* abort_flag = (volatile int*)(empty + kScanMaxStages);
  if (tid == 0) {
    for (int s = 0; s < kScanStages; ++s) {
      umma::mbar_init(&full[s], 1);
      umma::mbar_init(&empty[s], kScanThreads / 32);
    }
    *abort_flag = 0;
    asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
  }
  __syncthreads();
  const int nrounds = (nchunks + kScanGroup - 1) / kScanGroup;
  if (tid >= kScanThreads) {
    // ---- producer: one warp; lane 0 keeps the books, every lane issues one copy of the stage (a single thread issuing
    // all copies of a stage was the bottleneck of the whole kernel) ----
    const int lane = tid - kScanThreads;
    const uint32_t lbytes = (uint32_t)nel * 2, gbytes = (uint32_t)M * 4;
    for (int it = 0; it < nrounds; ++it) {
      const int s = it % kScanStages, round = it / kScanStages;
      const int cnt = min(kScanGroup, nchunks - it * kScanGroup);
      int stop = 0;
      if (lane == 0) {
        stop = *abort_flag;
        if (!stop && round > 0 && !scan_wait(&empty[s], (round - 1) & 1)) {
          *abort_flag = 1;
          atomicExch(err, 1);
          stop = 1;
        }
        if (!stop) mbar_expect_tx(&full[s], cnt * (lbytes + gbytes));
      }
      stop = __shfl_sync(0xffffffffu, stop, 0);
      if (stop) break;
      const int u = lane >> 1;
      if (u < cnt) {
        const size_t cgi = (size_t)(chunk0 + it * kScanGroup + u) * H + h;
        unsigned char* slot = scan_smem + (size_t)(s * kScanGroup + u) * kScanSlot;
        if (lane & 1) scan_bulk_g2s(slot + kScanElems * 2, w.gend + cgi * M, gbytes, &full[s]);
        else scan_bulk_g2s(slot, w.local + cgi * SD + el0, lbytes, &full[s]);
      }
    }
    return;
  }
  // ---- consumers ----
  const int el = el0 + 4 * tid;
  const bool active = 4 * tid < nel;
  const bool is_k = el < KM;
  const int e = is_k ? el : el - KM;
  const int m = is_k ? e % M : e / V;
  const size_t per = is_k ? KM : MV;
  bf16* out = is_k ? (bf16*)d.hk_chunks : (bf16*)d.hv_chunks;
  float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
  float4 gsum = make_float4(0.f, 0.f, 0.f, 0.f);
  const bool sums = active && is_k && e < M;        // the threads of hk's first row also total the log gates
  if (active) {
    const float* h0 = is_k ? d.hk0 : d.hv0;
    if (h0) run = *reinterpret_cast<const float4*>(h0 + nh * per + e);
  }
  bool failed = false;
  for (int it = 0; it < nrounds; ++it) {
    const int s = it % kScanStages, round = it / kScanStages;
    if (*abort_flag) { failed = true; break; }
    if (!scan_wait(&full[s], round & 1)) {
      *abort_flag = 1;
      atomicExch(err, 1);
      failed = true;
      break;
    }
    const int cnt = min(kScanGroup, nchunks - it * kScanGroup);
    if (active) {
      // everything the stage holds for this thread comes into registers first (the stores below go through generic
      // pointers, so the compiler will not move a shared-memory load across them): the serial part is then four
      // multiply-adds per chunk
      uint2 la[kScanGroup];
      float4 da[kScanGroup];
#pragma unroll
      for (int u = 0; u < kScanGroup; ++u) {
        const unsigned char* slot = scan_smem + (size_t)(s * kScanGroup + u) * kScanSlot;
        la[u] = *reinterpret_cast<const uint2*>(slot + 8 * tid);
        const float* gp = reinterpret_cast<const float*>(slot + kScanElems * 2) + m;
        if (is_k) da[u] = *reinterpret_cast<const float4*>(gp);
        else da[u] = make_float4(*gp, 0.f, 0.f, 0.f);
      }
      float4 av[kScanGroup];
#pragma unroll
      for (int u = 0; u < kScanGroup; ++u) {
        if (is_k) av[u] = make_float4(__expf(da[u].x), __expf(da[u].y), __expf(da[u].z), __expf(da[u].w));
        else { const float x = __expf(da[u].x); av[u] = make_float4(x, x, x, x); }
      }
#pragma unroll
      for (int u = 0; u < kScanGroup; ++u) {
        if (u < cnt) {
          const size_t cgi = (size_t)(chunk0 + it * kScanGroup + u) * H + h;
          uint2 o;
          *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(run.x, run.y);
          *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(run.z, run.w);
          *reinterpret_cast<uint2*>(out + cgi * per + e) = o;
          if (sums) { gsum.x += da[u].x; gsum.y += da[u].y; gsum.z += da[u].z; gsum.w += da[u].w; }
          const float2 l01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&la[u].x));
          const float2 l23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&la[u].y));
          run.x = run.x * av[u].x + l01.x; run.y = run.y * av[u].y + l01.y;
          run.z = run.z * av[u].z + l23.x; run.w = run.w * av[u].w + l23.y;
        }
      }
    }
    __syncwarp();
    if ((tid & 31) == 0) mbar_arrive(&empty[s]);
  }
  if (failed || !active) return;
  float* ht = is_k ? d.hkt : d.hvt;
  if (ht) *reinterpret_cast<float4*>(ht + nh * per + e) = run;
  if (sums) *reinterpret_cast<float4*>(w.gtot + nh * M + m) = gsum;
}

int64_t state_workspace_bytes(const nha_chunk_desc* d) {
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  const int64_t rows = nha_chunk_count_bound(d->Ttot, d->N) * d->H;
  return rows * (SD * 2 + d->M * 4) + (int64_t)d->N * d->H * d->M * 4 + 256;
}

static void state_ws_layout(const nha_chunk_desc* d, void* scratch, StateWs* w) {
  const int64_t NCB = nha_chunk_count_bound(d->Ttot, d->N);
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  w->local = (bf16*)scratch;
  w->gend = (float*)(w->local + NCB * d->H * SD);
  w->gtot = w->gend + NCB * d->H * d->M;
}

// Per-chunk terms of the chunks [chunk_lo, chunk_lo + chunk_n) on `scratch`: the tensor-core kernel where it has the
// shape, else the wmma kernel.
static int state_terms_on(const nha_chunk_desc* d, void* scratch, int chunk_lo, int chunk_n, cudaStream_t cs) {
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  if (chunk_lo < 0 || chunk_n < 0 || chunk_lo + chunk_n > NCB) return NHA_ERR_BAD_ARG;
  if (chunk_n == 0) return NHA_OK;
  StateWs w;
  state_ws_layout(d, scratch, &w);
  int st = NHA_ERR_UNSUPPORTED;
  if (state_local_umma_supported(d)) {
    int* err = d->plan + d->N + 1 + NCB + (size_t)NCB * d->H;
    st = state_local_umma_launch(d, w, err, chunk_lo, chunk_n, cs);
    if (st != NHA_OK && st != NHA_ERR_UNSUPPORTED) return st;
  }
  if (st == NHA_ERR_UNSUPPORTED) {
    const StLocalLayout L = st_local_layout(d->K, d->V, d->M);
    cudaError_t e = set_max_smem((const void*)nha_state_local_kernel, L.total);
    if (e != cudaSuccess) return record_cuda_error(e);
    nha_state_local_kernel<<<dim3(chunk_n, d->H), kStThreads, L.total, cs>>>(*d, w, chunk_lo);
    st = check_launch();
  }
  return st;
}

// The scan over the chunks on `scratch` (>= state_workspace_bytes(d) bytes, 16-byte aligned).  Every scratch element
// that it reads has been written by state_terms_on with the same descriptor.
static int state_scan_on(const nha_chunk_desc* d, void* scratch, cudaStream_t cs) {
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  StateWs w;
  state_ws_layout(d, scratch, &w);
  {
    // Ring depth and CTA width: the scan of one CTA is a serial walk over the sequence's chunks whose inputs take a
    // memory round trip to arrive, so its speed is (chunks in flight) / (round trip).  Few CTAs (one long sequence, few
    // heads): 1024 elements per CTA and as deep a ring as the longest sequence can use; many CTAs (a batch): 512
    // elements and a ring short enough for several CTAs per SM.
    int maxlen = d->max_seqlen > 0 ? d->max_seqlen : (int)d->Ttot;
    const int rounds = ((maxlen + kChunk - 1) / kChunk + kScanGroup - 1) / kScanGroup;
    const int64_t wide_ctas = (int64_t)d->N * d->H * ((SD + 1023) / 1024);
    int* err = d->plan + d->N + 1 + NCB + (size_t)NCB * d->H;
    if (wide_ctas <= 160) {
      const int stages = std::max(2, std::min(kScanMaxStages, rounds));
      const int smem = scan_smem_bytes(1024, stages);
      cudaError_t e = set_max_smem((const void*)nha_state_scan_kernel<1024>, smem);
      if (e != cudaSuccess) return record_cuda_error(e);
      nha_state_scan_kernel<1024><<<dim3((unsigned)(d->N * d->H), (unsigned)((SD + 1023) / 1024)), 1024 / 4 + 32, smem, cs>>>(
          *d, w, err, stages);
    } else {
      const int stages = std::max(2, std::min(5, rounds));
      const int smem = scan_smem_bytes(512, stages);
      cudaError_t e = set_max_smem((const void*)nha_state_scan_kernel<512>, smem);
      if (e != cudaSuccess) return record_cuda_error(e);
      nha_state_scan_kernel<512><<<dim3((unsigned)(d->N * d->H), (unsigned)((SD + 511) / 512)), 512 / 4 + 32, smem, cs>>>(
          *d, w, err, stages);
    }
  }
  return check_launch();
}

// Both parts of the state pass.
static int state_pass_on(const nha_chunk_desc* d, void* scratch, cudaStream_t cs) {
  const int st = state_terms_on(d, scratch, 0, (int)nha_chunk_count_bound(d->Ttot, d->N), cs);
  return st != NHA_OK ? st : state_scan_on(d, scratch, cs);
}

// Start state folded into the zero-start chunk states, in two chunk-parallel steps.
// 1. exclusive prefix sums of the per-chunk log gates over the chunks of each sequence: one warp per (sequence, kv head,
//    slot); a lane sums a contiguous run of chunks, the lanes' totals are scanned with shuffles.  cum [NCB*H][M] fp32
//    lives where the per-chunk terms L were (dead once the scan has consumed them).
__global__ void __launch_bounds__(256) nha_state_gate_prefix_kernel(const nha_chunk_desc d, const StateWs w, float* __restrict__ cum) {
  const int M = d.M, H = d.H;
  const int gw = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
  if (gw >= d.N * H * M) return;
  const int m = gw % M, h = (gw / M) % H, n = gw / (M * H);
  const int len = d.cu_seqlens[n + 1] - d.cu_seqlens[n];
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int chunk0 = d.plan[n];
  const int per = (nchunks + 31) / 32;
  const int c_lo = min(nchunks, lane * per), c_hi = min(nchunks, c_lo + per);
  float tot = 0.f;
  for (int c = c_lo; c < c_hi; ++c) tot += w.gend[((size_t)(chunk0 + c) * H + h) * M + m];
  float incl = tot;
#pragma unroll
  for (int o = 1; o < 32; o <<= 1) {
    const float t = __shfl_up_sync(0xffffffffu, incl, o);
    if (lane >= o) incl += t;
  }
  float run = incl - tot;
  for (int c = c_lo; c < c_hi; ++c) {
    const size_t i = ((size_t)(chunk0 + c) * H + h) * M + m;
    cum[i] = run;
    run += w.gend[i];
  }
}
// 2. chunk start states += S .* exp(cum): one CTA per (chunk, kv head), 16-byte accesses; the CTAs of a sequence's
//    first chunk also add S .* exp(total) to the final state.
__global__ void __launch_bounds__(256) nha_state_prefix_add_kernel(const nha_chunk_desc d, const StateWs w, const float* __restrict__ cum,
                                                                   const float* __restrict__ sk, const float* __restrict__ sv) {
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int KM = K * M, MV = M * V;
  const int cg = blockIdx.x, h = blockIdx.y;
  const ChunkRec rc = chunk_rec(d, cg);
  if (rc.n < 0) return;
  const size_t nh = (size_t)rc.n * H + h, cgi = (size_t)cg * H + h;
  __shared__ float dec[128], dtot[128];
  for (int m = threadIdx.x; m < M; m += blockDim.x) {
    dec[m] = __expf(cum[cgi * M + m]);
    dtot[m] = __expf(w.gtot[nh * M + m]);
  }
  __syncthreads();
  const bool last = rc.ci == 0;                     // one CTA per (sequence, kv head) updates the final state
  for (int el = 8 * threadIdx.x; el < KM + MV; el += 8 * blockDim.x) {
    const bool is_k = el < KM;
    const int e = is_k ? el : el - KM;
    const size_t per = is_k ? KM : MV;
    const float* S = (is_k ? sk : sv) + nh * per + e;
    const float4 s0 = *reinterpret_cast<const float4*>(S), s1 = *reinterpret_cast<const float4*>(S + 4);
    const float sv8[8] = {s0.x, s0.y, s0.z, s0.w, s1.x, s1.y, s1.z, s1.w};
    bf16* out = (is_k ? (bf16*)d.hk_chunks : (bf16*)d.hv_chunks) + cgi * per + e;
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(out), f);
    const int m0 = is_k ? e % M : e / V;            // hk: eight consecutive slots; hv: one slot for all eight
#pragma unroll
    for (int i = 0; i < 8; ++i) f[i] += sv8[i] * dec[is_k ? m0 + i : m0];
    *reinterpret_cast<uint4*>(out) = pack8(f);
    float* ht = is_k ? d.hkt : d.hvt;
    if (last && ht) {
      float4* q = reinterpret_cast<float4*>(ht + nh * per + e);
      float4 t0 = q[0], t1 = q[1];
      t0.x += sv8[0] * dtot[is_k ? m0 : m0]; t0.y += sv8[1] * dtot[is_k ? m0 + 1 : m0];
      t0.z += sv8[2] * dtot[is_k ? m0 + 2 : m0]; t0.w += sv8[3] * dtot[is_k ? m0 + 3 : m0];
      t1.x += sv8[4] * dtot[is_k ? m0 + 4 : m0]; t1.y += sv8[5] * dtot[is_k ? m0 + 5 : m0];
      t1.z += sv8[6] * dtot[is_k ? m0 + 6 : m0]; t1.w += sv8[7] * dtot[is_k ? m0 + 7 : m0];
      q[0] = t0; q[1] = t1;
    }
  }
}

// Start state of rank `rank` of a sequence-parallel prefill from the summaries of all ranks (allp [world][P] fp32 with
// P = H*K*M + H*M*V + H*M: zero-start end states L_k, L_v and the log gate totals G of each rank's segment):
//   S = S0 .* exp(sum_{r<rank} G_r) + sum_{r<rank} L_r .* exp(sum_{r<r'<rank} G_r'),   marched over r in order.
__global__ void __launch_bounds__(256) nha_sp_fold_kernel(const float* __restrict__ allp, int rank, int H, int K, int M, int V,
                                                          const float* __restrict__ hk0, const float* __restrict__ hv0,
                                                          float* __restrict__ sk, float* __restrict__ sv) {
  const int nk = H * K * M, nv = H * M * V, P = nk + nv + H * M;
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i >= nk + nv) return;
  const bool is_k = i < nk;
  const int e = is_k ? i : i - nk;
  const int h = is_k ? e / (K * M) : e / (M * V);
  const int m = is_k ? e % M : (e / V) % M;
  float run = is_k ? (hk0 ? hk0[e] : 0.f) : (hv0 ? hv0[e] : 0.f);
  for (int r = 0; r < rank; ++r) {
    const float* p = allp + (size_t)r * P;
    run = run * __expf(p[nk + nv + h * M + m]) + p[i];
  }
  (is_k ? sk : sv)[e] = run;
}

int check_chunk_desc(const nha_chunk_desc* d) {
  if (!d) return NHA_ERR_BAD_ARG;
  if (!d->q_gsa || !d->q_swa || !d->k_gsa || !d->k_swa || !d->v || !d->s || !d->g || !d->cu_seqlens || !d->plan)
    return NHA_ERR_BAD_ARG;
  if (d->Ttot < 0 || d->N <= 0 || d->H <= 0 || d->HQ <= 0 || d->HQ % d->H != 0 || d->max_seqlen < 0)
    return NHA_ERR_BAD_ARG;
  if ((d->hk0 == nullptr) != (d->hv0 == nullptr)) return NHA_ERR_BAD_ARG;
  if (d->K % 16 || d->V % 16 || d->M % 16 || d->K < 16 || d->V < 16 || d->M < 16 || d->K > 128 || d->V > 128 ||
      d->M > 128)
    return NHA_ERR_UNSUPPORTED;
  return NHA_OK;
}

}  // namespace nha

using namespace nha;

extern "C" int64_t nha_chunk_count_bound(int64_t Ttot, int64_t N) { return (Ttot + kChunk - 1) / kChunk + N; }
extern "C" int64_t nha_chunk_plan_ints(int64_t Ttot, int64_t N, int64_t H) {
  const int64_t ncb = nha_chunk_count_bound(Ttot, N);
  // offsets, chunk -> sequence, per-(chunk, head) flags, error word; then one 4-int record per chunk
  return plan_rec_offset(N, ncb, H) + 4 * ncb;
}

extern "C" int nha_chunk_plan(const nha_chunk_desc* d, void* stream) {
  if (!d || !d->cu_seqlens || !d->plan || d->N <= 0) return NHA_ERR_BAD_ARG;
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  nha_plan_kernel<<<1, 256, 0, (cudaStream_t)stream>>>(d->cu_seqlens, d->plan, d->N, NCB, d->H);
  return check_launch();
}

extern "C" int nha_chunk_state_pass(const nha_chunk_desc* d, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->hk_chunks || !d->hv_chunks) return NHA_ERR_BAD_ARG;
  const int64_t need = state_workspace_bytes(d);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  return state_pass_on(d, d->workspace, (cudaStream_t)stream);
}

extern "C" int nha_chunk_state_terms(const nha_chunk_desc* d, int chunk_lo, int chunk_n, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  const int64_t need = state_workspace_bytes(d);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  return state_terms_on(d, d->workspace, chunk_lo, chunk_n, (cudaStream_t)stream);
}

extern "C" int nha_chunk_state_scan(const nha_chunk_desc* d, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->hk_chunks || !d->hv_chunks) return NHA_ERR_BAD_ARG;
  const int64_t need = state_workspace_bytes(d);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  return state_scan_on(d, d->workspace, (cudaStream_t)stream);
}

extern "C" int nha_chunk_apply_state_prefix(const nha_chunk_desc* d, const float* sk, const float* sv, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->hk_chunks || !d->hv_chunks || !sk || !sv) return NHA_ERR_BAD_ARG;
  if (d->hk0 || d->hv0) return NHA_ERR_BAD_ARG;            // the state pass must have run from a zero start
  if (d->K % 8 || d->V % 8 || d->M % 8) return NHA_ERR_UNSUPPORTED;
  const int64_t need = state_workspace_bytes(d);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  StateWs w;
  state_ws_layout(d, d->workspace, &w);
  float* cum = (float*)w.local;                             // the per-chunk terms are dead: [NCB*H][M] floats fit easily
  cudaStream_t cs = (cudaStream_t)stream;
  const int warps = d->N * d->H * d->M;
  nha_state_gate_prefix_kernel<<<(warps * 32 + 255) / 256, 256, 0, cs>>>(*d, w, cum);
  st = check_launch();
  if (st != NHA_OK) return st;
  nha_state_prefix_add_kernel<<<dim3(NCB, d->H), 256, 0, cs>>>(*d, w, cum, sk, sv);
  return check_launch();
}

extern "C" int nha_chunk_gate_totals(const nha_chunk_desc* d, const float** out) {
  if (!d || !out || !d->workspace) return NHA_ERR_BAD_ARG;
  if ((int64_t)d->workspace_bytes < state_workspace_bytes(d)) return NHA_ERR_WORKSPACE;
  StateWs w;
  state_ws_layout(d, d->workspace, &w);
  *out = w.gtot;
  return NHA_OK;
}

extern "C" int nha_sp_fold_start_state(const float* allp, int world, int rank, int H, int K, int M, int V, const float* hk0,
                                       const float* hv0, float* sk, float* sv, void* stream) {
  if (!allp || !sk || !sv || world <= 0 || rank < 0 || rank >= world || H <= 0 || K <= 0 || M <= 0 || V <= 0)
    return NHA_ERR_BAD_ARG;
  if ((hk0 == nullptr) != (hv0 == nullptr)) return NHA_ERR_BAD_ARG;
  const int n = H * K * M + H * M * V;
  nha_sp_fold_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(allp, rank, H, K, M, V, hk0, hv0, sk, sv);
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// State pass for callers that cannot allocate device memory.
//
// Some hosts of this library own no device allocator: a plugin that is handed only its input and
// output buffers, or a serving loop that forbids allocation after start-up because cudaMalloc
// synchronises the device and can fail under memory pressure.  nha_chunk_state_pass needs a
// caller-provided workspace for the per-chunk terms; the variant below takes that workspace from
// a fixed array that lives in the library's own device image instead.
// Every GPU that loads the library holds the array (kStaticScratchBytes) until the process exits.
constexpr size_t kStaticScratchBytes = 16u << 20;
static __device__ __align__(256) unsigned char g_state_scratch[kStaticScratchBytes];

// In host code `g_state_scratch` is only a handle for the runtime, not a device address, so the
// address is looked up once per device with cudaGetSymbolAddress and cached.
constexpr int kMaxDevices = 64;
static void* g_state_scratch_ptr[kMaxDevices] = {nullptr};
static std::mutex g_state_scratch_mutex;

static int static_scratch_for_current_device(void** out) {
  int dev = -1;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return nha::record_cuda_error(e);
  if (dev < 0 || dev >= kMaxDevices) return NHA_ERR_BAD_ARG;
  std::lock_guard<std::mutex> lock(g_state_scratch_mutex);
  if (!g_state_scratch_ptr[dev]) {
    void* p = nullptr;
    e = cudaGetSymbolAddress(&p, g_state_scratch);
    if (e != cudaSuccess) return nha::record_cuda_error(e);
    g_state_scratch_ptr[dev] = p;
  }
  *out = g_state_scratch_ptr[dev];
  return NHA_OK;
}

extern "C" int64_t nha_chunk_state_pass_static_max_bytes(void) { return (int64_t)kStaticScratchBytes; }

extern "C" int nha_chunk_state_pass_static(const nha_chunk_desc* d, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->hk_chunks || !d->hv_chunks) return NHA_ERR_BAD_ARG;
  const int64_t need = state_workspace_bytes(d);
  if (need > (int64_t)kStaticScratchBytes) return NHA_ERR_STATIC_SCRATCH;
  void* scratch = nullptr;
  st = static_scratch_for_current_device(&scratch);
  if (st != NHA_OK) return st;
  // every element of the scratch that is read is written earlier in this same call, so the contents
  // left by the previous call never matter and nothing has to be cleared
  return state_pass_on(d, scratch, (cudaStream_t)stream);
}
