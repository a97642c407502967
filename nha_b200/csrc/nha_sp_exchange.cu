// Sequence-parallel prefill: the exchange of the segment summaries over peer memory, fused with the fold that consumes
// them (sm_100a, NVLink / NVSwitch peer stores; no multicast, no tensor-map access to peer memory).
//
// Every rank of a sequence-parallel prefill ends its state pass with a summary of its segment (P = H*K*M + H*M*V + H*M
// floats: zero-start end state and total log decay) and needs, before its output pass, the summaries of the ranks
// BEFORE it (the recurrence is linear: S_start(r) = fold of the summaries of ranks < r).  With a library all-gather
// this is a collective of its own between two small kernels; here
//   * nha_sp_publish stores the rank's summary straight into the mailboxes of the ranks after it (plain 16-byte stores
//     to peer pointers) and then raises one flag per receiver (release, system scope), and
//   * nha_sp_fold_wait, the fold kernel, first waits (acquire, system scope, bounded) for the flags of the ranks before
//     it in its OWN memory and then folds their summaries from its own mailbox - a rank waits for exactly the data it
//     consumes, rank 0 for nothing.
// Mailboxes are symmetric: on every rank box[depth][world][P] floats and flag[depth][world] words, allocated by the
// caller so that every rank can address every other rank's copy (peer pointers in box_ptrs / flag_ptrs, device arrays
// of `world` pointers).  Calls are numbered by a per-rank device counter (ctr[0], advanced by nha_sp_publish; every
// rank makes the same sequence of calls), call e uses slot e % depth and the flag value e, so nothing is ever reset and
// the pair of kernels can sit in a CUDA graph.  A rank can run ahead of a later rank by less than `world` calls (each
// call's halo message to the next rank completes only once that rank has started the same call), so depth = world + 1
// slots never collide.
//
// The wait is bounded: a flag that does not arrive within about a second sets the error word and the kernel returns
// (outputs invalid, context intact).
#include "nha_common.cuh"

namespace nha {

constexpr int kPubThreads = 256;

__device__ __forceinline__ void st_release_sys(uint32_t* p, uint32_t v) {
  asm volatile("st.release.sys.global.u32 [%0], %1;" ::"l"(p), "r"(v) : "memory");
}
__device__ __forceinline__ uint32_t ld_acquire_sys(const uint32_t* p) {
  uint32_t v;
  asm volatile("ld.acquire.sys.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
  return v;
}

// ctr[0]: calls published so far; ctr[1]: arrival ticket of the CTAs of the running call (zero between calls)
__global__ void __launch_bounds__(kPubThreads) nha_sp_publish_kernel(const float* __restrict__ pack, int P, float* const* box_ptrs,
                                                                     uint32_t* const* flag_ptrs, uint32_t* ctr, int world,
                                                                     int rank, int depth) {
  const uint32_t epoch = *(volatile uint32_t*)ctr + 1u;
  if (rank + 1 >= world) {                               // the last rank has nobody to tell: it only counts the call
    if (blockIdx.x == 0 && threadIdx.x == 0) *(volatile uint32_t*)ctr = epoch;
    return;
  }
  const int slot = (int)(epoch % (uint32_t)depth);
  const int nvec = P >> 2;                               // P is a multiple of 4 (K, V, M are multiples of 16)
  const float4* src = reinterpret_cast<const float4*>(pack);
  for (int p = rank + 1; p < world; ++p) {
    float4* dst = reinterpret_cast<float4*>(box_ptrs[p] + ((size_t)slot * world + rank) * P);
    for (int i = blockIdx.x * kPubThreads + threadIdx.x; i < nvec; i += gridDim.x * kPubThreads) dst[i] = src[i];
  }
  __threadfence_system();                                // this thread's stores are visible to the receivers ...
  __syncthreads();
  if (threadIdx.x == 0) {
    __threadfence_system();                              // (cumulative: what the CTA's threads fenced, this thread orders too)
    const unsigned t = atomicAdd(ctr + 1, 1u);           // ... before its CTA is counted
    if (t == gridDim.x - 1) {
      __threadfence_system();                            // every CTA has been counted: all their stores precede the flags
      ctr[1] = 0u;
      for (int p = rank + 1; p < world; ++p) st_release_sys(flag_ptrs[p] + slot * world + rank, epoch);
      *(volatile uint32_t*)ctr = epoch;
    }
  }
}

// Start state of rank `rank` (see nha_sp_fold_kernel) from the mailbox of this rank, after the summaries of the ranks
// before it have arrived.
__global__ void __launch_bounds__(256) nha_sp_fold_wait_kernel(const float* __restrict__ box, const uint32_t* __restrict__ flag,
                                                               const uint32_t* __restrict__ ctr, int rank, int world, int depth,
                                                               int H, int K, int M, int V, const float* __restrict__ hk0,
                                                               const float* __restrict__ hv0, float* __restrict__ sk,
                                                               float* __restrict__ sv, int* __restrict__ err) {
  const uint32_t epoch = *(volatile const uint32_t*)ctr;   // this call's number: the publish kernel in front advanced it
  const int slot = (int)(epoch % (uint32_t)depth);
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = 0;
  __syncthreads();
  if ((int)threadIdx.x < rank) {
    const uint32_t* f = flag + slot * world + threadIdx.x;
    bool ok = false;
    for (int it = 0; it < (1 << 22) && !ok; ++it) {      // about a second with the sleeps
      ok = (int32_t)(ld_acquire_sys(f) - epoch) >= 0;
      if (!ok) __nanosleep(200);
    }
    if (!ok) s_bad = 1;
  }
  __syncthreads();
  if (s_bad) {
    if (threadIdx.x == 0 && err) atomicExch(err, 1);
    return;
  }
  // (the waiting threads' acquire loads, passed on by the barrier above, order the reads of every thread of the CTA;
  // the reads below bypass L1, which may still hold lines of an earlier call's slot)
  const float* allp = box + (size_t)slot * world * ((size_t)H * K * M + (size_t)H * M * V + (size_t)H * M);
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
    run = run * __expf(__ldcg(p + nk + nv + h * M + m)) + __ldcg(p + i);
  }
  (is_k ? sk : sv)[e] = run;
}

// ---------------------------------------------------------------------------------------------
// The halo of a sequence-parallel prefill over peer memory: a rank stores the last W rows of its kv-head tensors
// straight into the first W rows of the next rank's (halo-extended) tensors.  One-sided, so both directions are
// flagged: the receiver raises `ack` once it has finished reading the halo of call e (after its output pass), and the
// sender's call e + 1 waits for that before it overwrites the rows; the sender raises `flag` once the rows of call e
// are there, and the receiver's first kernel that reads them is preceded by a wait for it.  Calls are counted on both
// sides by device counters (every rank makes the same sequence of calls), so nothing is reset and all three kernels
// can sit in a CUDA graph.  Every wait is bounded (about a second, then the error word is set and the kernel returns).
struct HaloCopies {
  const uint4* src[5];
  uint4* dst[5];
  int64_t nvec[5];
};

__device__ __forceinline__ bool wait_word_at_least(const uint32_t* p, uint32_t want) {
  for (int it = 0; it < (1 << 22); ++it) {
    if ((int32_t)(ld_acquire_sys(p) - want) >= 0) return true;
    __nanosleep(200);
  }
  return false;
}

// ctr[0]: halos pushed so far; ctr[1]: arrival ticket of the CTAs of the running call
__global__ void __launch_bounds__(kPubThreads) nha_sp_halo_push_kernel(const HaloCopies c, uint32_t* flag_peer,
                                                                       const uint32_t* ack_local, uint32_t* ctr, int* err) {
  const uint32_t epoch = *(volatile uint32_t*)ctr + 1u;
  __shared__ int s_bad;
  if (threadIdx.x == 0) s_bad = wait_word_at_least(ack_local, epoch - 1u) ? 0 : 1;   // the halo before this one was consumed
  __syncthreads();
  if (!s_bad) {
    __threadfence_system();
#pragma unroll 1
    for (int t = 0; t < 5; ++t)
      for (int64_t i = (int64_t)blockIdx.x * kPubThreads + threadIdx.x; i < c.nvec[t]; i += (int64_t)gridDim.x * kPubThreads)
        c.dst[t][i] = c.src[t][i];
    __threadfence_system();
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    if (s_bad && err) atomicExch(err, 1);
    __threadfence_system();
    const unsigned t = atomicAdd(ctr + 1, 1u);
    if (t == gridDim.x - 1) {
      __threadfence_system();
      ctr[1] = 0u;
      st_release_sys(flag_peer, epoch);                  // raised even after a failed wait: the receiver must not hang too
      *(volatile uint32_t*)ctr = epoch;
    }
  }
}

// receiver: ctr[0] counts the halos received
__global__ void nha_sp_halo_wait_kernel(const uint32_t* flag_local, uint32_t* ctr, int* err) {
  const uint32_t epoch = *(volatile uint32_t*)ctr + 1u;
  if (!wait_word_at_least(flag_local, epoch) && err) atomicExch(err, 1);
  __threadfence_system();
  *(volatile uint32_t*)ctr = epoch;
}

// receiver, after the last kernel that reads the halo rows: tells the sender that they may be overwritten
__global__ void nha_sp_halo_ack_kernel(uint32_t* ack_peer, const uint32_t* ctr) {
  st_release_sys(ack_peer, *(volatile const uint32_t*)ctr);
}

}  // namespace nha

using namespace nha;

extern "C" int nha_sp_halo_push(const void* const* src, void* const* dst_peer, const int64_t* bytes, int count,
                                uint32_t* flag_peer, const uint32_t* ack_local, uint32_t* ctr, int* err_word, void* stream) {
  if (!src || !dst_peer || !bytes || count < 1 || count > 5 || !flag_peer || !ack_local || !ctr) return NHA_ERR_BAD_ARG;
  HaloCopies c;
  int64_t most = 0;
  for (int t = 0; t < 5; ++t) {
    c.src[t] = nullptr; c.dst[t] = nullptr; c.nvec[t] = 0;
    if (t >= count) continue;
    if (!src[t] || !dst_peer[t] || bytes[t] < 0 || bytes[t] % 16 || ((uintptr_t)src[t] & 15) || ((uintptr_t)dst_peer[t] & 15))
      return NHA_ERR_BAD_ARG;
    c.src[t] = (const uint4*)src[t]; c.dst[t] = (uint4*)dst_peer[t]; c.nvec[t] = bytes[t] / 16;
    most = most > c.nvec[t] ? most : c.nvec[t];
  }
  int grid = (int)((most + kPubThreads - 1) / kPubThreads);
  grid = grid < 1 ? 1 : (grid > 128 ? 128 : grid);
  nha_sp_halo_push_kernel<<<grid, kPubThreads, 0, (cudaStream_t)stream>>>(c, flag_peer, ack_local, ctr, err_word);
  return check_launch();
}

extern "C" int nha_sp_halo_wait(const uint32_t* flag_local, uint32_t* ctr, int* err_word, void* stream) {
  if (!flag_local || !ctr) return NHA_ERR_BAD_ARG;
  nha_sp_halo_wait_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(flag_local, ctr, err_word);
  return check_launch();
}

extern "C" int nha_sp_halo_ack(uint32_t* ack_peer, const uint32_t* ctr, void* stream) {
  if (!ack_peer || !ctr) return NHA_ERR_BAD_ARG;
  nha_sp_halo_ack_kernel<<<1, 1, 0, (cudaStream_t)stream>>>(ack_peer, ctr);
  return check_launch();
}

extern "C" int nha_sp_publish(const float* pack, int64_t P, float* const* box_ptrs, uint32_t* const* flag_ptrs, uint32_t* ctr,
                              int world, int rank, int depth, void* stream) {
  if (!pack || !box_ptrs || !flag_ptrs || !ctr || P <= 0 || P % 4 || world < 1 || rank < 0 || rank >= world || depth < 2)
    return NHA_ERR_BAD_ARG;
  if (((uintptr_t)pack & 15)) return NHA_ERR_BAD_ARG;
  // enough CTAs to keep the peer links busy (one 16-byte store per thread and receiver); one for the last rank
  int grid = (int)((P / 4 + kPubThreads - 1) / kPubThreads);
  grid = rank + 1 >= world ? 1 : (grid > 296 ? 296 : grid);
  nha_sp_publish_kernel<<<grid, kPubThreads, 0, (cudaStream_t)stream>>>(pack, (int)P, box_ptrs, flag_ptrs, ctr, world, rank,
                                                                        depth);
  return check_launch();
}

extern "C" int nha_sp_fold_wait(const float* box, const uint32_t* flag, const uint32_t* ctr, int world, int rank, int depth,
                                int H, int K, int M, int V, const float* hk0, const float* hv0, float* sk, float* sv,
                                int* err_word, void* stream) {
  if (!box || !flag || !ctr || !sk || !sv || world < 1 || rank < 0 || rank >= world || depth < 2 || world > 256)
    return NHA_ERR_BAD_ARG;
  if ((hk0 == nullptr) != (hv0 == nullptr)) return NHA_ERR_BAD_ARG;
  if (H <= 0 || K <= 0 || M <= 0 || V <= 0) return NHA_ERR_BAD_ARG;
  const int n = H * K * M + H * M * V;
  nha_sp_fold_wait_kernel<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(box, flag, ctr, rank, world, depth, H, K, M, V, hk0,
                                                                             hv0, sk, sv, err_word);
  return check_launch();
}
