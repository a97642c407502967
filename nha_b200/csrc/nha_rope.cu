// Rotary position embedding of the callers' queries and keys, both tensors in one launch.
//
// The layer rotates q and k before it calls the operator (nha_fla/layers/nha.py:145,235: RotaryEmbedding of
// head_k_dim, non-interleaved halves, positions restarting at every packed sequence when cu_seqlens is given;
// the hybrid models rotate with duplicated-halves tables, nha_fla/models/qwen3_nha/qwennha.py:240-244, which is
// the same arithmetic on the first K/2 table columns):
//     o[.., i]       = x[.., i] cos[p, i] - x[.., i + K/2] sin[p, i]
//     o[.., i + K/2] = x[.., i] sin[p, i] + x[.., i + K/2] cos[p, i]          i < K/2,  p = offset + position in sequence
// One CTA-strided pass: every thread owns 8 consecutive i of one (token, head) row, loads the two 16-byte halves
// and the 16-byte table pieces, writes two 16-byte results.  fp32 arithmetic, one rounding.  The backward is the
// same kernel with the sign of sin flipped (rotation by -theta).
#include "nha_common.cuh"

namespace nha {

constexpr int kRopeThreads = 256;

struct RopeArgs {
  const bf16* x[2];        // q [Ttot, H0, K], k [Ttot, H1, K]
  bf16* o[2];
  int heads[2];
  const bf16* cosp; const bf16* sinp;
  int64_t cs_row;          // elements between table rows
  const int* cu; int N;    // packed sequences, or cu == nullptr: sequences of `T` tokens each
  int T;
  int64_t Ttot;
  int K;
  int offset;              // position of the first token of every sequence
  int table_rows;
  float sin_sign;          // +1 forward, -1 backward
};

__global__ void __launch_bounds__(kRopeThreads) nha_rope_kernel(const RopeArgs a) {
  const int R8 = a.K >> 4;                                   // 16-byte pieces per half row
  const int htot = a.heads[0] + a.heads[1];
  const int64_t units = a.Ttot * htot * R8;
  for (int64_t u = (int64_t)blockIdx.x * kRopeThreads + threadIdx.x; u < units; u += (int64_t)gridDim.x * kRopeThreads) {
    const int c = (int)(u % R8);
    const int64_t r = u / R8;
    int hh = (int)(r % htot);
    const int64_t t = r / htot;
    const int which = hh >= a.heads[0];
    if (which) hh -= a.heads[0];
    // position inside the sequence
    int pos;
    if (a.cu) {
      int lo = 0, hi = a.N;                                   // last n with cu[n] <= t
      while (hi - lo > 1) {
        const int mid = (lo + hi) >> 1;
        if (__ldg(a.cu + mid) <= t) lo = mid; else hi = mid;
      }
      pos = (int)(t - __ldg(a.cu + lo));
    } else {
      pos = (int)(t % a.T);
    }
    pos = min(pos + a.offset, a.table_rows - 1);              // the host checked the table covers every position
    const bf16* xp = a.x[which] + (t * a.heads[which] + hh) * a.K + 8 * c;
    bf16* op = a.o[which] + (t * a.heads[which] + hh) * a.K + 8 * c;
    const uint4 x0 = __ldcs(reinterpret_cast<const uint4*>(xp));
    const uint4 x1 = __ldcs(reinterpret_cast<const uint4*>(xp + (a.K >> 1)));
    const uint4 cv = __ldg(reinterpret_cast<const uint4*>(a.cosp + pos * a.cs_row + 8 * c));
    const uint4 sv = __ldg(reinterpret_cast<const uint4*>(a.sinp + pos * a.cs_row + 8 * c));
    float f0[8], f1[8], fc[8], fs[8], o0[8], o1[8];
    unpack8(x0, f0); unpack8(x1, f1); unpack8(cv, fc); unpack8(sv, fs);
#pragma unroll
    for (int e = 0; e < 8; ++e) {
      const float sn = fs[e] * a.sin_sign;
      o0[e] = f0[e] * fc[e] - f1[e] * sn;
      o1[e] = f0[e] * sn + f1[e] * fc[e];
    }
    *reinterpret_cast<uint4*>(op) = pack8(o0);
    *reinterpret_cast<uint4*>(op + (a.K >> 1)) = pack8(o1);
  }
}

}  // namespace nha

using namespace nha;

extern "C" int nha_rope_pair(const void* q, const void* k, void* q_out, void* k_out, const void* cos, const void* sin,
                             int64_t cs_row, int table_rows, const int32_t* cu_seqlens, int N, int T, int64_t Ttot, int HQ,
                             int H, int K, int offset, int inverse, void* stream) {
  if (!q || !q_out || !cos || !sin || (k && !k_out)) return NHA_ERR_BAD_ARG;
  if (Ttot < 0 || HQ <= 0 || (k && H <= 0) || offset < 0 || table_rows <= 0) return NHA_ERR_BAD_ARG;
  if (cu_seqlens ? N <= 0 : T <= 0) return NHA_ERR_BAD_ARG;
  if (K <= 0 || K % 16 || cs_row % 8 || cs_row < K / 2) return NHA_ERR_UNSUPPORTED;   // 16-byte pieces of a half row
  const uintptr_t al = (uintptr_t)q | (uintptr_t)k | (uintptr_t)q_out | (uintptr_t)k_out | (uintptr_t)cos | (uintptr_t)sin;
  if (al & 15u) return NHA_ERR_BAD_ARG;
  if (Ttot == 0) return NHA_OK;
  RopeArgs a;
  a.x[0] = (const bf16*)q; a.x[1] = (const bf16*)k; a.o[0] = (bf16*)q_out; a.o[1] = (bf16*)k_out;
  a.heads[0] = HQ; a.heads[1] = k ? H : 0;
  a.cosp = (const bf16*)cos; a.sinp = (const bf16*)sin; a.cs_row = cs_row;
  a.cu = cu_seqlens; a.N = N; a.T = T; a.Ttot = Ttot; a.K = K; a.offset = offset; a.table_rows = table_rows;
  a.sin_sign = inverse ? -1.0f : 1.0f;
  int dev = 0, sms = 148;
  if (cudaGetDevice(&dev) == cudaSuccess) cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev);
  const int64_t units = Ttot * (a.heads[0] + a.heads[1]) * (K >> 4);
  const int64_t want = (units + kRopeThreads - 1) / kRopeThreads;
  const int64_t cap = (int64_t)sms * 8 * 4;                   // four trips of eight CTAs per SM at most
  nha_rope_kernel<<<(int)(want < cap ? want : cap), kRopeThreads, 0, (cudaStream_t)stream>>>(a);
  return check_launch();
}
