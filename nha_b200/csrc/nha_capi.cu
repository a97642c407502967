// Status plumbing and size helpers of the C ABI.
#include <string.h>

#include <map>
#include <mutex>
#include <utility>

#include "nha_common.cuh"
#include "nha_umma.cuh"

namespace nha {

static thread_local char g_last_error[256] = "";

int record_cuda_error(cudaError_t e) {
  strncpy(g_last_error, cudaGetErrorString(e), sizeof(g_last_error) - 1);
  g_last_error[sizeof(g_last_error) - 1] = 0;
  return NHA_ERR_LAUNCH;
}

int check_launch() {
  cudaError_t e = cudaGetLastError();
  if (e != cudaSuccess) return record_cuda_error(e);
  return NHA_OK;
}

cudaError_t set_max_smem(const void* func, int bytes) {
  static std::mutex mu;
  static std::map<std::pair<int, const void*>, int> granted;
  int dev = 0;
  cudaError_t e = cudaGetDevice(&dev);
  if (e != cudaSuccess) return e;
  std::lock_guard<std::mutex> lock(mu);
  auto it = granted.find({dev, func});
  if (it != granted.end() && it->second >= bytes) return cudaSuccess;
  e = cudaFuncSetAttribute(func, cudaFuncAttributeMaxDynamicSharedMemorySize, bytes);
  if (e == cudaSuccess) granted[{dev, func}] = bytes;
  return e;
}

// One CTA waits, with a poll limit, on an mbarrier phase that nobody completes: the wait must come back as "ran out"
// and the kernel reports it in the error word, exactly as the tensor-core kernels report a completion that never came.
__global__ void nha_selftest_wait_kernel(int* err, int limit) {
  __shared__ uint64_t bar;
  if (threadIdx.x == 0) umma::mbar_init(&bar, 1);
  __syncthreads();
  if (!umma::mbar_wait_limit(&bar, 0, limit)) atomicExch(err, 1);
}

}  // namespace nha

extern "C" int nha_selftest_bounded_wait(int* err_word, int polls, void* stream) {
  if (!err_word || polls <= 0 || polls > (1 << 16)) return NHA_ERR_BAD_ARG;
  nha::nha_selftest_wait_kernel<<<1, 64, 0, (cudaStream_t)stream>>>(err_word, polls);
  return nha::check_launch();
}

extern "C" const char* nha_status_string(int status) {
  switch (status) {
    case NHA_OK: return "ok";
    case NHA_ERR_BAD_ARG: return "bad argument (null pointer, non-positive size or HQ not a multiple of H)";
    case NHA_ERR_UNSUPPORTED: return "unsupported head dim / slot count / group size";
    case NHA_ERR_SMEM: return "tile set does not fit in shared memory";
    case NHA_ERR_LAUNCH: return "CUDA launch failed (see nha_last_cuda_error)";
    case NHA_ERR_WORKSPACE: return "workspace missing or too small";
    case NHA_ERR_STATIC_SCRATCH: return "problem needs more scratch than the built-in static array holds";
    default: return "unknown status";
  }
}

extern "C" const char* nha_last_cuda_error(void) { return nha::g_last_error; }

extern "C" int nha_abi_version(void) { return 1; }

extern "C" int64_t nha_chunk_desc_size(void) { return (int64_t)sizeof(nha_chunk_desc); }
