// Chunk plan and state pass of the chunked NHA kernels (sm_100a).
//
// The slot memory obeys a per-element linear recurrence
//     hk[k,m] <- hk[k,m] * exp(g'[m]) + k'[k] * s'[m],   hv[m,v] <- hv[m,v] * exp(g'[m]) + s'[m] * v'[v]
// (primes = inputs shifted right by gsa_kv_shift inside their sequence).  The state pass marches over
// the chunks of a sequence and stores the state at every chunk start (bf16, the operand type of the
// later matrix products) plus the fp32 final state.  Parallelism: the K rows of hk and the V columns
// of hv are independent, so one CTA owns a 16-row / 16-column slice; long sequences are cut into
// segments whose local end states are computed from a zero start, combined by a short sequential
// scan (the recurrence is linear), and marched a second time from the true segment start.
//
// Replaces chunk_nha_fused_state_kernel (nha_fla/ops/nha/chunk_fused.py:31-114) and the state part of
// fla's chunk_gsa_fwd reached from nha_fla/ops/nha/chunk_gsa.py:38-45; the in-sequence shift replaces
// _packed_shift_right / _batch_shift_right (nha_fla/ops/nha/chunk.py:53-111).
#include <mutex>

#include "nha_common.cuh"

namespace nha {

constexpr int kStThreads = 128;
constexpr int kStWarps = kStThreads / 32;
constexpr int kDefaultSegChunks = 32;

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
  for (int n = threadIdx.x; n < N; n += blockDim.x) {
    const int c0 = plan[n], c1 = plan[n + 1];
    for (int c = c0; c < c1; ++c) plan[N + 1 + c] = n;
  }
}

// ---------------------------------------------------------------------------------------------
// mode 0: single march from the initial state (sequence fits one segment per grid.z slot)
// mode 1: local march from zero, emits segment end state + segment log-decay
// mode 2: march from the combined segment start, emits chunk-start states and the final state
struct StateArgs {
  nha_chunk_desc d;
  int mode;
  int seg_chunks;
  int nseg_max;
  float* seg_local;   // [N*H, nseg_max, K*M + M*V] end state of each segment marched from zero
  float* seg_start;   // [N*H, nseg_max, K*M + M*V] true state at each segment start
  float* seg_decay;   // [N*H, nseg_max, M] sum of the shifted log gates of the segment
};

__global__ void __launch_bounds__(kStThreads) nha_state_kernel(const StateArgs a) {
  const nha_chunk_desc& d = a.d;
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int nks = K / 16, nvs = V / 16;
  const int slice = blockIdx.x;                 // < nks: rows of hk, else columns of hv
  const bool is_k = slice < nks;
  const int s0 = (is_k ? slice : slice - nks) * 16;
  const int n = blockIdx.y / H, h = blockIdx.y % H;
  const int seg = blockIdx.z;
  const int t0 = d.cu_seqlens[n];
  const int len = d.cu_seqlens[n + 1] - t0;
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int c_begin = seg * a.seg_chunks;
  if (c_begin >= nchunks && !(seg == 0)) return;
  const int c_end = min(nchunks, c_begin + a.seg_chunks);
  const int shift = seq_shift(d, n);
  const int chunk0 = d.plan[n];
  const int tid = threadIdx.x, warp = tid >> 5;
  const int SD = K * M + M * V;

  extern __shared__ __align__(128) unsigned char smem[];
  const int ldg = M + 4, ldsb = M + 8, ldx = 16 + 8;
  float* G = reinterpret_cast<float*>(smem);                       // [64][M+4] cumulative shifted gates
  bf16* sbe = reinterpret_cast<bf16*>(G + kChunk * ldg);           // [64][M+8] s' * exp(Gend - G)
  bf16* xt = sbe + kChunk * ldsb;                                  // [64][24]  slice of k' or v'
  float* hs = reinterpret_cast<float*>(xt + kChunk * ldx);         // hk slice [16][M+4] or hv slice [M][16+4]
  const int ldh = is_k ? M + 4 : 16 + 4;
  const int hrows = is_k ? 16 : M, hcols = is_k ? M : 16;

  // ---- initial state of this march
  const size_t nh = (size_t)n * H + h;
  for (int i = tid; i < hrows * hcols; i += kStThreads) {
    const int r = i / hcols, c = i - r * hcols;
    float val = 0.f;
    const size_t el = is_k ? (size_t)(s0 + r) * M + c : (size_t)K * M + (size_t)r * V + s0 + c;
    if (a.mode == 2) {
      val = a.seg_start[(nh * a.nseg_max + seg) * SD + el];
    } else if (a.mode == 0) {
      if (is_k) { if (d.hk0) val = d.hk0[nh * K * M + el]; }
      else { if (d.hv0) val = d.hv0[nh * M * V + (el - (size_t)K * M)]; }
    }
    hs[r * ldh + c] = val;
  }
  float decay_sum = 0.f;   // per thread m = tid (< M): running sum of Gend over the segment
  __syncthreads();

  const bf16* xsrc = is_k ? (const bf16*)d.k_gsa : (const bf16*)d.v;
  const int D = is_k ? K : V;
  for (int c = c_begin; c < c_end; ++c) {
    const int p0 = c * kChunk;            // shifted position of row 0
    // ---- emit the chunk-start slice
    if (a.mode != 1) {
      const size_t cg = (size_t)(chunk0 + c) * H + h;
      if (is_k) {
        bf16* dst = (bf16*)d.hk_chunks + cg * K * M + (size_t)s0 * M;
        for (int i = tid; i < 16 * M; i += kStThreads) dst[i] = f2bf(hs[(i / M) * ldh + (i % M)]);
      } else {
        bf16* dst = (bf16*)d.hv_chunks + cg * M * V + s0;
        for (int i = tid; i < M * 16; i += kStThreads) dst[(size_t)(i / 16) * V + (i % 16)] = f2bf(hs[(i / 16) * ldh + (i % 16)]);
      }
    }
    // ---- load shifted g' (fp32) and the k'/v' slice
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
    for (int i = tid; i < kChunk * 2; i += kStThreads) {
      const int r = i >> 1, c8 = i & 1;
      const int p = p0 + r, j = p - shift;
      uint4 u = make_uint4(0u, 0u, 0u, 0u);
      if (j >= 0 && p < len) u = *reinterpret_cast<const uint4*>(xsrc + ((size_t)(t0 + j) * H + h) * D + s0 + 8 * c8);
      *reinterpret_cast<uint4*>(xt + r * ldx + 8 * c8) = u;
    }
    __syncthreads();
    // ---- inclusive cumsum along the rows, one column per thread
    for (int m = tid; m < M; m += kStThreads) {
      float run = 0.f;
#pragma unroll 16
      for (int r = 0; r < kChunk; ++r) {
        run += G[r * ldg + m];
        G[r * ldg + m] = run;
      }
      if (m == tid) decay_sum += run;
    }
    __syncthreads();
    // ---- sbe = s' * exp(Gend - G); scale the state slice by exp(Gend)
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
    for (int i = tid; i < hrows * hcols; i += kStThreads) {
      const int r = i / hcols, cc = i - r * hcols;
      const int m = is_k ? cc : r;
      hs[r * ldh + cc] *= __expf(G[(kChunk - 1) * ldg + m]);
    }
    __syncthreads();
    // ---- rank-64 update on the tensor cores
    if (is_k) {
      // hk_slice[16 x M] += k'_slice^T [16 x 64] * sbe [64 x M]
      tile_gemm<false, true, true>(hs, ldh, xt, ldx, sbe, ldsb, 1, M / 16, kChunk / 16, warp, kStWarps);
    } else {
      // hv_slice[M x 16] += sbe^T [M x 64] * v'_slice [64 x 16]
      tile_gemm<false, true, true>(hs, ldh, sbe, ldsb, xt, ldx, M / 16, 1, kChunk / 16, warp, kStWarps);
    }
    __syncthreads();
  }

  // ---- epilogue
  if (a.mode == 1) {
    float* dst = a.seg_local + (nh * a.nseg_max + seg) * SD;
    for (int i = tid; i < hrows * hcols; i += kStThreads) {
      const int r = i / hcols, c = i - r * hcols;
      const size_t el = is_k ? (size_t)(s0 + r) * M + c : (size_t)K * M + (size_t)r * V + s0 + c;
      dst[el] = hs[r * ldh + c];
    }
    if (slice == 0 && tid < M) a.seg_decay[(nh * a.nseg_max + seg) * M + tid] = decay_sum;
    if (slice == 0 && M > kStThreads)
      for (int m = tid + kStThreads; m < M; m += kStThreads) a.seg_decay[(nh * a.nseg_max + seg) * M + m] = 0.f;
  } else if (c_end >= nchunks) {
    // last segment (or an empty sequence on segment 0): final state
    if (is_k && d.hkt) {
      for (int i = tid; i < 16 * M; i += kStThreads) d.hkt[nh * K * M + (size_t)s0 * M + i] = hs[(i / M) * ldh + (i % M)];
    } else if (!is_k && d.hvt) {
      for (int i = tid; i < M * 16; i += kStThreads)
        d.hvt[nh * M * V + (size_t)(i / 16) * V + s0 + (i % 16)] = hs[(i / 16) * ldh + (i % 16)];
    }
  }
}

// Sequential combine over the segments of one (sequence, kv head): start[0] = h0,
// start[z+1] = start[z] * exp(decay[z]) + local[z].
__global__ void nha_state_combine_kernel(const StateArgs a) {
  const nha_chunk_desc& d = a.d;
  const int K = d.K, V = d.V, M = d.M, H = d.H;
  const int SD = K * M + M * V;
  const size_t nh = blockIdx.y;
  const int n = nh / H;
  const int len = d.cu_seqlens[n + 1] - d.cu_seqlens[n];
  const int nchunks = (len + kChunk - 1) / kChunk;
  const int nseg = max(1, (nchunks + a.seg_chunks - 1) / a.seg_chunks);
  const int el = blockIdx.x * blockDim.x + threadIdx.x;
  if (el >= SD) return;
  const int m = el < K * M ? el % M : (el - K * M) / V;
  float val = 0.f;
  if (el < K * M) { if (d.hk0) val = d.hk0[nh * K * M + el]; }
  else { if (d.hv0) val = d.hv0[nh * M * V + (el - K * M)]; }
  for (int z = 0; z < nseg; ++z) {
    const size_t base = nh * a.nseg_max + z;
    a.seg_start[base * SD + el] = val;
    val = val * __expf(a.seg_decay[base * M + m]) + a.seg_local[base * SD + el];
  }
}

static int state_smem(int M) {
  const int hs = max(16 * (M + 4), M * (16 + 4)) * 4;
  return kChunk * (M + 4) * 4 + kChunk * (M + 8) * 2 + kChunk * 24 * 2 + hs;
}

static int seg_chunks_of(const nha_chunk_desc* d) { return d->seg_chunks > 0 ? d->seg_chunks : kDefaultSegChunks; }

static int nseg_max_of(const nha_chunk_desc* d) {
  const int maxchunks = (d->max_seqlen + kChunk - 1) / kChunk;
  const int sc = seg_chunks_of(d);
  return max(1, (maxchunks + sc - 1) / sc);
}

int64_t state_workspace_bytes(const nha_chunk_desc* d) {
  const int nseg = nseg_max_of(d);
  if (nseg <= 1) return 0;
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  const int64_t per = (int64_t)d->N * d->H * nseg;
  return (per * SD * 2 + per * d->M) * 4 + 256;
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
  return N + 1 + ncb + ncb * H + 4;     // offsets, chunk -> sequence, per-(chunk, head) flags, error word
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
  cudaStream_t cs = (cudaStream_t)stream;
  StateArgs a;
  a.d = *d;
  a.seg_chunks = seg_chunks_of(d);
  a.nseg_max = nseg_max_of(d);
  a.seg_local = a.seg_start = a.seg_decay = nullptr;
  const int smem = state_smem(d->M);
  cudaError_t e = cudaFuncSetAttribute(nha_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int slices = d->K / 16 + d->V / 16;
  dim3 block(kStThreads);
  if (a.nseg_max <= 1) {
    a.mode = 0;
    dim3 grid(slices, d->N * d->H, 1);
    nha_state_kernel<<<grid, block, smem, cs>>>(a);
    return check_launch();
  }
  const int64_t need = state_workspace_bytes(d);
  if (!d->workspace || (int64_t)d->workspace_bytes < need) return NHA_ERR_WORKSPACE;
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  const int64_t per = (int64_t)d->N * d->H * a.nseg_max;
  a.seg_local = (float*)d->workspace;
  a.seg_start = a.seg_local + per * SD;
  a.seg_decay = a.seg_start + per * SD;
  dim3 grid(slices, d->N * d->H, a.nseg_max);
  a.mode = 1;
  nha_state_kernel<<<grid, block, smem, cs>>>(a);
  st = check_launch();
  if (st != NHA_OK) return st;
  dim3 cgrid((unsigned)((SD + 255) / 256), d->N * d->H);
  nha_state_combine_kernel<<<cgrid, 256, 0, cs>>>(a);
  st = check_launch();
  if (st != NHA_OK) return st;
  a.mode = 2;
  nha_state_kernel<<<grid, block, smem, cs>>>(a);
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// State pass for callers that cannot allocate device memory.
//
// Some hosts of this library own no device allocator: a plugin that is handed only its input and
// output buffers, or a serving loop that forbids allocation after start-up because cudaMalloc
// synchronises the device and can fail under memory pressure.  nha_chunk_state_pass needs a
// caller-provided workspace as soon as a sequence spans more than one segment; the variant below
// takes that workspace from a fixed array that lives in the library's own device image instead.
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
  cudaStream_t cs = (cudaStream_t)stream;
  StateArgs a;
  a.d = *d;
  a.seg_chunks = seg_chunks_of(d);
  a.nseg_max = nseg_max_of(d);
  a.seg_local = a.seg_start = a.seg_decay = nullptr;
  const int smem = state_smem(d->M);
  cudaError_t e = cudaFuncSetAttribute(nha_state_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, smem);
  if (e != cudaSuccess) return record_cuda_error(e);
  const int slices = d->K / 16 + d->V / 16;
  dim3 block(kStThreads);
  if (a.nseg_max <= 1) {
    a.mode = 0;
    nha_state_kernel<<<dim3(slices, d->N * d->H, 1), block, smem, cs>>>(a);
    return check_launch();
  }
  // every element of the scratch that is read below is written earlier in this same call, so the
  // contents left by the previous call never matter and nothing has to be cleared
  const int64_t SD = (int64_t)d->K * d->M + (int64_t)d->M * d->V;
  const int64_t per = (int64_t)d->N * d->H * a.nseg_max;
  a.seg_local = (float*)scratch;
  a.seg_start = a.seg_local + per * SD;
  a.seg_decay = a.seg_start + per * SD;
  dim3 grid(slices, d->N * d->H, a.nseg_max);
  a.mode = 1;
  nha_state_kernel<<<grid, block, smem, cs>>>(a);
  st = check_launch();
  if (st != NHA_OK) return st;
  nha_state_combine_kernel<<<dim3((unsigned)((SD + 255) / 256), d->N * d->H), 256, 0, cs>>>(a);
  st = check_launch();
  if (st != NHA_OK) return st;
  a.mode = 2;
  nha_state_kernel<<<grid, block, smem, cs>>>(a);
  return check_launch();
}
