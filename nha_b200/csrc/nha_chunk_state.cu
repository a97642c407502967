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
// final state.  Every exponent is <= 0, so no reference point is needed.
//
// Replaces chunk_nha_fused_state_kernel (nha_fla/ops/nha/chunk_fused.py:31-114) and the state part of
// fla's chunk_gsa_fwd reached from nha_fla/ops/nha/chunk_gsa.py:38-45; the in-sequence shift replaces
// _packed_shift_right / _batch_shift_right (nha_fla/ops/nha/chunk.py:53-111).
#include <mutex>

#include "nha_common.cuh"

namespace nha {

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
// Scratch of the state pass: L [NCB*H][K*M + M*V] bf16 (the chunk-start states it is summed into are bf16 too; the
// running sum itself stays fp32), then Gend [NCB*H][M] fp32.
struct StateWs {
  bf16* local;
  float* gend;
};

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
__global__ void __launch_bounds__(kStThreads) nha_state_local_kernel(const nha_chunk_desc d, const StateWs w) {
  const int cg = blockIdx.x, h = blockIdx.y;
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
  // end contribute nothing
  const int lo = shift, hi = len;                  // valid shifted positions p: lo <= p < hi
  load_tile_bf16(kt, ldk, (const bf16*)d.k_gsa + ((size_t)t0 * H + h) * K - (size_t)shift * H * K, (int64_t)H * K, p0, lo,
                 hi, kChunk, K, tid, kStThreads);
  load_tile_bf16(vt, ldv, (const bf16*)d.v + ((size_t)t0 * H + h) * V - (size_t)shift * H * V, (int64_t)H * V, p0, lo, hi,
                 kChunk, V, tid, kStThreads);
  for (int i = tid; i < kChunk * (M / 8); i += kStThreads) {
    const int r = i / (M / 8), c8 = i - r * (M / 8);
    const int p = p0 + r, j = p - shift;
    float gv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (j >= 0 && p < len) {
      const uint4 u = *reinterpret_cast<const uint4*>((const bf16*)d.g + ((size_t)(t0 + j) * H + h) * M + 8 * c8);
      unpack8(u, gv);
    }
#pragma unroll
    for (int e = 0; e < 8; ++e) G[r * ldg + 8 * c8 + e] = gv[e];
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
  for (int i = tid; i < kChunk * (M / 8); i += kStThreads) {
    const int r = i / (M / 8), c8 = i - r * (M / 8);
    const int p = p0 + r, j = p - shift;
    float sv[8] = {0, 0, 0, 0, 0, 0, 0, 0};
    if (j >= 0 && p < len) {
      const uint4 u = *reinterpret_cast<const uint4*>((const bf16*)d.s + ((size_t)(t0 + j) * H + h) * M + 8 * c8);
      unpack8(u, sv);
    }
    float out[8];
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const int m = 8 * c8 + e;
      out[e] = sv[e] * __expf(G[(kChunk - 1) * ldg + m] - G[r * ldg + m]);
    }
    *reinterpret_cast<uint4*>(sbe + r * ldsb + 8 * c8) = pack8(out);
  }
  __syncthreads();
  bf16* Lk = w.local + ((size_t)cg * H + h) * ((size_t)K * M + (size_t)M * V);
  bf16* Lv = Lk + (size_t)K * M;
  // L_k [K x M] = k'^T [K x 64] * sbe [64 x M];  L_v [M x V] = sbe^T [M x 64] * v' [64 x V]
  float* patch = (float*)(smem + L.patch);
  tile_gemm_tn_bf16(Lk, M, kt, ldk, sbe, ldsb, K / 16, M / 16, kChunk / 16, warp, kStWarps, patch);
  tile_gemm_tn_bf16(Lv, V, sbe, ldsb, vt, ldv, M / 16, V / 16, kChunk / 16, warp, kStWarps, patch);
}

// Forward scan over the chunks of one (sequence, kv head): stores the state at every chunk start and
// the final state.  One thread owns four consecutive state elements (one 8-byte bf16 store per chunk) and
// fetches kStScanBatch chunks of L ahead of the serial recurrence, so that a long sequence with few heads
// still keeps enough loads in flight.
constexpr int kStScanBatch = 16;
__global__ void __launch_bounds__(256) nha_state_scan_kernel(const nha_chunk_desc d, const StateWs w) {
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int KM = K * M, MV = M * V;
  const size_t SD = (size_t)KM + MV;
  const size_t nh = blockIdx.x;                     // (sequence, kv head) in x: no 65535 limit on packed batches
  const int n = nh / H, h = nh % H;
  const int len = d.cu_seqlens[n + 1] - d.cu_seqlens[n];
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int chunk0 = d.plan[n];
  const int el = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (el >= KM + MV) return;
  const bool is_k = el < KM;
  const int e = is_k ? el : el - KM;
  const int m = is_k ? e % M : e / V;
  const size_t per = is_k ? KM : MV;
  bf16* out = is_k ? (bf16*)d.hk_chunks : (bf16*)d.hv_chunks;
  float4 run = make_float4(0.f, 0.f, 0.f, 0.f);
  {
    const float* h0 = is_k ? d.hk0 : d.hv0;
    if (h0) run = *reinterpret_cast<const float4*>(h0 + nh * per + e);
  }
  for (int lo = 0; lo < nchunks; lo += kStScanBatch) {
    uint2 la[kStScanBatch];
    float4 da[kStScanBatch];
#pragma unroll
    for (int u = 0; u < kStScanBatch; ++u) {
      const int ci = lo + u;
      if (ci < nchunks) {
        const size_t cgi = (size_t)(chunk0 + ci) * H + h;
        la[u] = __ldcs((const uint2*)(w.local + cgi * SD + el));
        if (is_k) da[u] = *(const float4*)(w.gend + cgi * M + m);
        else da[u].x = w.gend[cgi * M + m];
      }
    }
#pragma unroll
    for (int u = 0; u < kStScanBatch; ++u) {
      const int ci = lo + u;
      if (ci < nchunks) {
        const size_t cgi = (size_t)(chunk0 + ci) * H + h;
        uint2 o;
        *reinterpret_cast<__nv_bfloat162*>(&o.x) = __floats2bfloat162_rn(run.x, run.y);
        *reinterpret_cast<__nv_bfloat162*>(&o.y) = __floats2bfloat162_rn(run.z, run.w);
        *reinterpret_cast<uint2*>(out + cgi * per + e) = o;
        float4 a;
        if (is_k) a = make_float4(__expf(da[u].x), __expf(da[u].y), __expf(da[u].z), __expf(da[u].w));
        else { const float x = __expf(da[u].x); a = make_float4(x, x, x, x); }
        const float2 l01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&la[u].x));
        const float2 l23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&la[u].y));
        run.x = run.x * a.x + l01.x; run.y = run.y * a.y + l01.y;
        run.z = run.z * a.z + l23.x; run.w = run.w * a.w + l23.y;
      }
    }
  }
  float* ht = is_k ? d.hkt : d.hvt;
  if (ht) *reinterpret_cast<float4*>(ht + nh * per + e) = run;
}

int64_t state_workspace_bytes(const nha_chunk_desc* d) {
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  const int64_t rows = nha_chunk_count_bound(d->Ttot, d->N) * d->H;
  return rows * (SD * 2 + d->M * 4) + 256;
}

// Both launches of the state pass on `scratch` (>= state_workspace_bytes(d) bytes, 16-byte aligned).
// Every scratch element that the scan reads is written by the first kernel of the same call.
static int state_pass_on(const nha_chunk_desc* d, void* scratch, cudaStream_t cs) {
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  StateWs w;
  w.local = (bf16*)scratch;
  w.gend = (float*)(w.local + (int64_t)NCB * d->H * SD);
  const StLocalLayout L = st_local_layout(d->K, d->V, d->M);
  cudaError_t e = set_max_smem((const void*)nha_state_local_kernel, L.total);
  if (e != cudaSuccess) return record_cuda_error(e);
  nha_state_local_kernel<<<dim3(NCB, d->H), kStThreads, L.total, cs>>>(*d, w);
  int st = check_launch();
  if (st != NHA_OK) return st;
  nha_state_scan_kernel<<<dim3((unsigned)(d->N * d->H), (unsigned)((SD / 4 + 255) / 256)), 256, 0, cs>>>(*d, w);
  return check_launch();
}

// Adds S .* exp(log gates of the chunks before c) to the zero-start state at the start of every chunk c of a sequence
// (and S .* exp(all log gates) to the final state).  Same thread layout as the scan: one thread owns four consecutive
// state elements and walks the chunks of its (sequence, kv head) with the running decay in registers.
__global__ void __launch_bounds__(256) nha_state_prefix_kernel(const nha_chunk_desc d, const StateWs w, const float* __restrict__ sk,
                                                               const float* __restrict__ sv) {
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int KM = K * M, MV = M * V;
  const size_t nh = blockIdx.x;
  const int n = nh / H, h = nh % H;
  const int len = d.cu_seqlens[n + 1] - d.cu_seqlens[n];
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int chunk0 = d.plan[n];
  const int el = 4 * (blockIdx.y * blockDim.x + threadIdx.x);
  if (el >= KM + MV) return;
  const bool is_k = el < KM;
  const int e = is_k ? el : el - KM;
  const int m = is_k ? e % M : e / V;
  const size_t per = is_k ? KM : MV;
  bf16* out = is_k ? (bf16*)d.hk_chunks : (bf16*)d.hv_chunks;
  float4 run = *reinterpret_cast<const float4*>((is_k ? sk : sv) + nh * per + e);
  for (int ci = 0; ci < nchunks; ++ci) {
    const size_t cgi = (size_t)(chunk0 + ci) * H + h;
    uint2* p = reinterpret_cast<uint2*>(out + cgi * per + e);
    const uint2 o = *p;
    const float2 a01 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.x));
    const float2 a23 = __bfloat1622float2(*reinterpret_cast<const __nv_bfloat162*>(&o.y));
    uint2 r;
    *reinterpret_cast<__nv_bfloat162*>(&r.x) = __floats2bfloat162_rn(a01.x + run.x, a01.y + run.y);
    *reinterpret_cast<__nv_bfloat162*>(&r.y) = __floats2bfloat162_rn(a23.x + run.z, a23.y + run.w);
    *p = r;
    if (is_k) {
      const float4 g4 = *(const float4*)(w.gend + cgi * M + m);
      run.x *= __expf(g4.x); run.y *= __expf(g4.y); run.z *= __expf(g4.z); run.w *= __expf(g4.w);
    } else {
      const float x = __expf(w.gend[cgi * M + m]);
      run.x *= x; run.y *= x; run.z *= x; run.w *= x;
    }
  }
  float* ht = is_k ? d.hkt : d.hvt;
  if (ht) {
    float4* q = reinterpret_cast<float4*>(ht + nh * per + e);
    float4 t = *q;
    t.x += run.x; t.y += run.y; t.z += run.z; t.w += run.w;
    *q = t;
  }
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

extern "C" int nha_chunk_apply_state_prefix(const nha_chunk_desc* d, const float* sk, const float* sv, void* stream) {
  int st = check_chunk_desc(d);
  if (st != NHA_OK) return st;
  if (!d->hk_chunks || !d->hv_chunks || !sk || !sv) return NHA_ERR_BAD_ARG;
  if (d->hk0 || d->hv0) return NHA_ERR_BAD_ARG;            // the state pass must have run from a zero start
  const int64_t need = state_workspace_bytes(d);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  const int NCB = (int)nha_chunk_count_bound(d->Ttot, d->N);
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  StateWs w;
  w.local = (bf16*)d->workspace;
  w.gend = (float*)(w.local + (int64_t)NCB * d->H * SD);
  nha_state_prefix_kernel<<<dim3((unsigned)(d->N * d->H), (unsigned)((SD / 4 + 255) / 256)), 256, 0, (cudaStream_t)stream>>>(
      *d, w, sk, sv);
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
