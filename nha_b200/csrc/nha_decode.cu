// Fused NHA decode step for sm_100a: slot-state update + slot logits + window logits + joint
// softmax + slot/window readout in ONE launch, one CTA per (sequence, kv head) serving all query
// heads of the group, so the fp32 state and the window K/V are read from HBM exactly once.
//
// The kernel is memory bound (about 6 flop per byte), so it is organised around keeping bytes in
// flight: at entry every thread issues asynchronous 16-byte copies (cp.async) for the whole state and
// the first window stages into shared memory, and each time a 128-key stage has been consumed the
// freed buffer is refilled with the next stage (keys first, then values).  The arithmetic (fp32 FMA
// for the state, warp-level tensor-core tiles for the window) runs underneath those copies.
//
// Replaces the two Triton launches of fused_recurrent_nha_decode
// (nha_fla/ops/nha/fused_recurrent.py:229-353 k-kernel, :356-428 v-kernel) and, with caller-supplied
// window logits, the kernels of fused_recurrent_nha (:48-147).
#include "nha_common.cuh"

namespace nha {

constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kStageRows = 16 * kDecWarps;   // keys per pipeline stage: one 16-key tile per warp
constexpr int kRing = 3;                     // stage buffers

struct DecodeArgs {
  const bf16* q; const bf16* sq; const bf16* k; const bf16* v; const bf16* g; const bf16* s;
  const bf16* sw_k; const bf16* sw_v; const bf16* cosp; const bf16* sinp; const bf16* win_logits;
  float* hk; float* hv; bf16* o; float* win_prob;
  int64_t cs_batch, cs_row;
  int B, HQ, H, K, V, M, W, NG, Wp, NS, zero_state;
  float scale;
  // shared-memory byte offsets
  int off_qraw, off_sqA, off_oks, off_eg, off_sv, off_kpop, off_vpop, off_P, off_ring, off_hv, off_S, off_oacc;
  int stage_bytes;
};

__host__ __device__ inline int align_up(int x, int a) { return (x + a - 1) / a * a; }

__device__ __forceinline__ void cp_async16(void* dst, const void* src, bool valid) {
  const unsigned d = (unsigned)__cvta_generic_to_shared(dst);
  const int n = valid ? 16 : 0;   // src-size 0 zero-fills the 16 destination bytes
  asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;\n" ::"r"(d), "l"(src), "r"(n));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;\n" ::); }
template <int N>
__device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;\n" ::"n"(N)); }

template <int NGMAX>
__global__ void __launch_bounds__(kDecThreads) nha_decode_kernel(const DecodeArgs a) {
  using namespace nvcuda::wmma;
  extern __shared__ __align__(128) unsigned char smem[];
  float* qraw = reinterpret_cast<float*>(smem + a.off_qraw);      // [NG][K]   scaled raw query
  bf16* sqA = reinterpret_cast<bf16*>(smem + a.off_sqA);          // [16][K+8] rotated query (rows >= NG zero)
  float* oks = reinterpret_cast<float*>(smem + a.off_oks);        // [NG][M]   slot logits -> slot probabilities
  float* eg = reinterpret_cast<float*>(smem + a.off_eg);          // [M]
  float* sv = reinterpret_cast<float*>(smem + a.off_sv);          // [M]
  float* kpop = reinterpret_cast<float*>(smem + a.off_kpop);      // [K]
  float* vpop = reinterpret_cast<float*>(smem + a.off_vpop);      // [V]
  bf16* P = reinterpret_cast<bf16*>(smem + a.off_P);              // [16][NS*128+8] window probabilities
  unsigned char* ring = smem + a.off_ring;                        // kRing stage buffers; the last one first holds hk
  float* hvS = reinterpret_cast<float*>(smem + a.off_hv);         // [M][V]
  float* S = reinterpret_cast<float*>(smem + a.off_S);            // [16][NS*128+8] window logits; also reduction scratch
  float* oacc = reinterpret_cast<float*>(smem + a.off_oacc);      // [16][V+8] window readout

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int b = blockIdx.x / a.H, h = blockIdx.x % a.H;
  const int bh = b * a.H + h;
  const int K = a.K, V = a.V, M = a.M, W = a.W, NG = a.NG, NS = a.NS;
  const int ldq = K + 8, ldw = NS * kStageRows + 8;
  const int KVmax = (K > V ? K : V);
  const int ldst = KVmax + 8;
  const bool rotary = a.cosp != nullptr;
  const bool logits_mode = a.win_logits != nullptr;
  const int n_items = logits_mode ? 0 : 2 * NS;                   // NS key stages, then NS value stages
  float* hkS = reinterpret_cast<float*>(ring + (size_t)(kRing - 1) * a.stage_bytes);   // [K][M]

  // issue the copies of pipeline item `it` into its ring slot (nothing for it >= n_items)
  auto issue_item = [&](int it) {
    if (it < n_items) {
      const bool is_k = it < NS;
      const int st = is_k ? it : it - NS;
      const int D = is_k ? K : V;
      const bf16* src = is_k ? a.sw_k : a.sw_v;
      bf16* dst = reinterpret_cast<bf16*>(ring + (size_t)(it % kRing) * a.stage_bytes);
      const int c8n = D >> 3;
      for (int i = tid; i < kStageRows * c8n; i += kDecThreads) {
        const int r = i / c8n, c = i - r * c8n;
        const int w = st * kStageRows + r;
        const bool ok = w < W;
        const bf16* p = src + (((size_t)b * W + (ok ? w : 0)) * a.H + h) * D + 8 * c;
        cp_async16(dst + r * ldst + 8 * c, p, ok);
      }
    }
    cp_async_commit();
  };

  // ---- group 0: the state; groups 1, 2: the first two window stages --------------------------------
  if (!a.zero_state) {
    const float* hk_g = a.hk + (size_t)bh * K * M;
    const float* hv_g = a.hv + (size_t)bh * M * V;
    for (int i = tid; i < (K * M) / 4; i += kDecThreads) cp_async16(hkS + 4 * i, hk_g + 4 * i, true);
    for (int i = tid; i < (M * V) / 4; i += kDecThreads) cp_async16(hvS + 4 * i, hv_g + 4 * i, true);
  }
  cp_async_commit();
  issue_item(0);
  issue_item(1);

  // ---- phase 0: the popped token, the gates and the queries -------------------------------------
  for (int m = tid; m < M; m += kDecThreads) {
    const float gm = bf2f(a.g[(size_t)bh * M + m]);
    const float e = __expf(gm);
    eg[m] = e;
    sv[m] = a.s ? bf2f(a.s[(size_t)bh * M + m]) : 1.0f - e;
  }
  for (int i = tid; i < K; i += kDecThreads) kpop[i] = bf2f(a.k[(size_t)bh * K + i]);
  for (int i = tid; i < V; i += kDecThreads) vpop[i] = bf2f(a.v[(size_t)bh * V + i]);
  for (int i = tid; i < NG * K; i += kDecThreads) {
    const int qh = i / K, kk = i - qh * K;
    qraw[i] = bf2f(a.q[((size_t)b * a.HQ + h * NG + qh) * K + kk]) * a.scale;
  }
  if (!logits_mode) {
    const bf16* cq = rotary ? a.cosp + b * a.cs_batch + (int64_t)(W - 1) * a.cs_row : nullptr;
    const bf16* sn = rotary ? a.sinp + b * a.cs_batch + (int64_t)(W - 1) * a.cs_row : nullptr;
    for (int i = tid; i < 16 * K; i += kDecThreads) {
      const int r = i / K, kk = i - r * K;
      float val = 0.f;
      if (r < NG) {
        const bf16* qrow = a.q + ((size_t)b * a.HQ + h * NG + r) * K;
        if (rotary) {
          const float x = bf2f(qrow[kk]);
          const float xp = kk < K / 2 ? -bf2f(qrow[kk + K / 2]) : bf2f(qrow[kk - K / 2]);
          val = x * bf2f(cq[kk]) + xp * bf2f(sn[kk]);
        } else {
          val = bf2f(a.sq[((size_t)b * a.HQ + h * NG + r) * K + kk]);
        }
      }
      sqA[r * ldq + kk] = f2bf(val);
    }
  }
  for (int i = tid; i < 16 * ldw; i += kDecThreads) P[i] = f2bf(0.f);
  cp_async_wait<2>();        // group 0 (the state) has landed
  __syncthreads();

  // ---- phase 1: hk <- hk * exp(g) + k s^T (written back in place), slot logits ok[qh][m] -----------
  {
    const int M4 = M >> 2;
    const int RL = kDecThreads / M4;
    const int m4 = tid % M4, rl = tid / M4;
    float acc[NGMAX][4];
#pragma unroll
    for (int qh = 0; qh < NGMAX; ++qh) acc[qh][0] = acc[qh][1] = acc[qh][2] = acc[qh][3] = 0.f;
    if (rl < RL) {
      const float4 e4 = *reinterpret_cast<const float4*>(eg + 4 * m4);
      const float4 s4 = *reinterpret_cast<const float4*>(sv + 4 * m4);
      float4* hg = reinterpret_cast<float4*>(a.hk + (size_t)bh * K * M) + m4;
      const float4* hsm = reinterpret_cast<const float4*>(hkS) + m4;
      for (int kk = rl; kk < K; kk += RL) {
        float4 hh = a.zero_state ? make_float4(0.f, 0.f, 0.f, 0.f) : hsm[(size_t)kk * M4];
        const float kv = kpop[kk];
        hh.x = hh.x * e4.x + kv * s4.x;
        hh.y = hh.y * e4.y + kv * s4.y;
        hh.z = hh.z * e4.z + kv * s4.z;
        hh.w = hh.w * e4.w + kv * s4.w;
        hg[(size_t)kk * M4] = hh;
#pragma unroll
        for (int qh = 0; qh < NGMAX; ++qh) {
          if (qh < NG) {
            const float qv = qraw[qh * K + kk];
            acc[qh][0] += qv * hh.x; acc[qh][1] += qv * hh.y; acc[qh][2] += qv * hh.z; acc[qh][3] += qv * hh.w;
          }
        }
      }
#pragma unroll
      for (int qh = 0; qh < NGMAX; ++qh)
        if (qh < NG)
          *reinterpret_cast<float4*>(S + ((size_t)rl * NG + qh) * M + 4 * m4) =
              make_float4(acc[qh][0], acc[qh][1], acc[qh][2], acc[qh][3]);
    }
    __syncthreads();
    for (int i = tid; i < NG * M; i += kDecThreads) {
      float sum = 0.f;
      for (int r = 0; r < RL; ++r) sum += S[(size_t)r * NG * M + i];
      oks[i] = sum;
    }
    __syncthreads();
  }
  issue_item(2);             // the buffer that held hk is free now

  // ---- phase 2: window logits S[qh][w] (unscaled), one 128-key stage at a time -----------------------
  if (logits_mode) {
    for (int i = tid; i < NG * W; i += kDecThreads) {
      const int qh = i / W, w = i - qh * W;
      S[qh * ldw + w] = bf2f(a.win_logits[((size_t)b * a.HQ + h * NG + qh) * W + w]);
    }
  }
  for (int it = 0; it < NS && !logits_mode; ++it) {
    cp_async_wait<2>();
    __syncthreads();
    bf16* st = reinterpret_cast<bf16*>(ring + (size_t)(it % kRing) * a.stage_bytes);
    if (rotary) {
      // rotate-half in place; one thread owns both halves of its 8-element column group
      const int c8h = K >> 4;
      for (int i = tid; i < kStageRows * c8h; i += kDecThreads) {
        const int r = i / c8h, c = i - r * c8h;
        const int w = it * kStageRows + r;
        if (w < W) {
          const bf16* crow = a.cosp + b * a.cs_batch + (int64_t)w * a.cs_row;
          const bf16* srow = a.sinp + b * a.cs_batch + (int64_t)w * a.cs_row;
          float x[8], y[8], c1[8], s1[8], c2[8], s2[8], o1[8], o2[8];
          unpack8(*reinterpret_cast<const uint4*>(st + r * ldst + 8 * c), x);
          unpack8(*reinterpret_cast<const uint4*>(st + r * ldst + 8 * (c + c8h)), y);
          unpack8(*reinterpret_cast<const uint4*>(crow + 8 * c), c1);
          unpack8(*reinterpret_cast<const uint4*>(srow + 8 * c), s1);
          unpack8(*reinterpret_cast<const uint4*>(crow + 8 * (c + c8h)), c2);
          unpack8(*reinterpret_cast<const uint4*>(srow + 8 * (c + c8h)), s2);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            o1[e] = x[e] * c1[e] - y[e] * s1[e];
            o2[e] = y[e] * c2[e] + x[e] * s2[e];
          }
          *reinterpret_cast<uint4*>(st + r * ldst + 8 * c) = pack8(o1);
          *reinterpret_cast<uint4*>(st + r * ldst + 8 * (c + c8h)) = pack8(o2);
        }
      }
      __syncthreads();
    }
    {
      fragment<accumulator, 16, 16, 16, float> acc;
      fill_fragment(acc, 0.f);
      for (int ks = 0; ks < K / 16; ++ks) {
        fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
        fragment<matrix_b, 16, 16, 16, bf16, col_major> fb;
        load_matrix_sync(fa, sqA + 16 * ks, ldq);
        load_matrix_sync(fb, st + (size_t)16 * warp * ldst + 16 * ks, ldst);
        mma_sync(acc, fa, fb, acc);
      }
      store_matrix_sync(S + it * kStageRows + 16 * warp, acc, ldw, mem_row_major);
    }
    __syncthreads();
    issue_item(it + kRing);
  }
  __syncthreads();

  // ---- phase 3: joint softmax over [M slots | W window keys], one warp per query head ------------
  const float wscale = logits_mode ? 1.0f : a.scale;
  for (int qh = warp; qh < NG; qh += kDecWarps) {
    float mx = -INFINITY;
    for (int m = lane; m < M; m += 32) mx = fmaxf(mx, oks[qh * M + m]);
    for (int w = lane; w < W; w += 32) mx = fmaxf(mx, S[qh * ldw + w] * wscale);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int m = lane; m < M; m += 32) sum += __expf(oks[qh * M + m] - mx);
    for (int w = lane; w < W; w += 32) sum += __expf(S[qh * ldw + w] * wscale - mx);
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int m = lane; m < M; m += 32) oks[qh * M + m] = __expf(oks[qh * M + m] - mx) * inv;
    for (int w = lane; w < W; w += 32) {
      const float pw = __expf(S[qh * ldw + w] * wscale - mx) * inv;
      P[qh * ldw + w] = f2bf(pw);
      if (a.win_prob) a.win_prob[((size_t)b * a.HQ + h * NG + qh) * W + w] = pw;
    }
  }
  __syncthreads();

  // ---- phase 4: window readout; each warp owns 16-column tiles of the output ----------------------
  if (!logits_mode) {
    constexpr int kMaxCT = 2;                         // V <= 256 with 8 warps
    fragment<accumulator, 16, 16, 16, float> acc[kMaxCT];
#pragma unroll
    for (int i = 0; i < kMaxCT; ++i) fill_fragment(acc[i], 0.f);
    for (int it = NS; it < 2 * NS; ++it) {
      cp_async_wait<2>();
      __syncthreads();
      const bf16* st = reinterpret_cast<const bf16*>(ring + (size_t)(it % kRing) * a.stage_bytes);
      const int col0 = (it - NS) * kStageRows;
      for (int kt = 0; kt < kStageRows / 16; ++kt) {
        fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
        load_matrix_sync(fa, P + col0 + 16 * kt, ldw);
#pragma unroll
        for (int i = 0; i < kMaxCT; ++i) {
          const int ct = warp + kDecWarps * i;
          if (ct < V / 16) {
            fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
            load_matrix_sync(fb, st + (size_t)16 * kt * ldst + 16 * ct, ldst);
            mma_sync(acc[i], fa, fb, acc[i]);
          }
        }
      }
      __syncthreads();
      issue_item(it + kRing);
    }
#pragma unroll
    for (int i = 0; i < kMaxCT; ++i) {
      const int ct = warp + kDecWarps * i;
      if (ct < V / 16) store_matrix_sync(oacc + 16 * ct, acc[i], V + 8, mem_row_major);
    }
  }
  cp_async_wait<0>();

  // ---- phase 5: hv <- diag(exp(g)) hv + s v^T (written back in place), slot readout, output --------
  {
    const int V4 = V >> 2;
    const int ML = kDecThreads / V4;
    const int v4 = tid % V4, ml = tid / V4;
    float* red2 = S;                                  // the window logits are dead by now
    float acc[NGMAX][4];
#pragma unroll
    for (int qh = 0; qh < NGMAX; ++qh) acc[qh][0] = acc[qh][1] = acc[qh][2] = acc[qh][3] = 0.f;
    if (ml < ML) {
      const float4 vp4 = *reinterpret_cast<const float4*>(vpop + 4 * v4);
      float4* hg = reinterpret_cast<float4*>(a.hv + (size_t)bh * M * V) + v4;
      const float4* hsm = reinterpret_cast<const float4*>(hvS) + v4;
      for (int m = ml; m < M; m += ML) {
        float4 hh = a.zero_state ? make_float4(0.f, 0.f, 0.f, 0.f) : hsm[(size_t)m * V4];
        const float e = eg[m], sm = sv[m];
        hh.x = hh.x * e + sm * vp4.x;
        hh.y = hh.y * e + sm * vp4.y;
        hh.z = hh.z * e + sm * vp4.z;
        hh.w = hh.w * e + sm * vp4.w;
        hg[(size_t)m * V4] = hh;
#pragma unroll
        for (int qh = 0; qh < NGMAX; ++qh) {
          if (qh < NG) {
            const float pm = oks[qh * M + m];
            acc[qh][0] += pm * hh.x; acc[qh][1] += pm * hh.y; acc[qh][2] += pm * hh.z; acc[qh][3] += pm * hh.w;
          }
        }
      }
#pragma unroll
      for (int qh = 0; qh < NGMAX; ++qh)
        if (qh < NG)
          *reinterpret_cast<float4*>(red2 + ((size_t)ml * NG + qh) * V + 4 * v4) =
              make_float4(acc[qh][0], acc[qh][1], acc[qh][2], acc[qh][3]);
    }
    __syncthreads();
    for (int i = tid; i < NG * V; i += kDecThreads) {
      const int qh = i / V, vv = i - qh * V;
      float sum = 0.f;
      for (int r = 0; r < ML; ++r) sum += red2[(size_t)r * NG * V + i];
      if (!logits_mode) sum += oacc[qh * (V + 8) + vv];
      a.o[((size_t)b * a.HQ + h * NG + qh) * V + vv] = f2bf(sum);
    }
  }
}

static int decode_layout(DecodeArgs& a) {
  const int K = a.K, V = a.V, M = a.M, NG = a.NG;
  const int KVmax = K > V ? K : V;
  const int ldw = a.NS * kStageRows + 8;
  int off = 0;
  auto take = [&](int bytes) { int o = off; off = align_up(off + bytes, 128); return o; };
  a.off_qraw = take(NG * K * 4);
  a.off_sqA = take(16 * (K + 8) * 2);
  a.off_oks = take(NG * M * 4);
  a.off_eg = take(M * 4);
  a.off_sv = take(M * 4);
  a.off_kpop = take(K * 4);
  a.off_vpop = take(V * 4);
  a.off_P = take(16 * ldw * 2);
  a.stage_bytes = align_up(max(kStageRows * (KVmax + 8) * 2, K * M * 4), 128);
  a.off_ring = take(kRing * a.stage_bytes);
  a.off_hv = take(M * V * 4);
  const int RL = kDecThreads / (M / 4);
  const int ML = kDecThreads / (V / 4);
  int sbytes = 16 * ldw * 4;                                  // window logits
  sbytes = max(sbytes, RL * NG * M * 4);                      // phase-1 reduction
  sbytes = max(sbytes, ML * NG * V * 4);                      // phase-5 reduction
  a.off_S = take(sbytes);
  a.off_oacc = take(16 * (V + 8) * 4);
  return off;
}

}  // namespace nha

using namespace nha;

extern "C" int nha_decode_step(const void* q, const void* sq, const void* k, const void* v, const void* g,
                               const void* s, const void* sw_k, const void* sw_v, const void* cosp, const void* sinp,
                               int64_t cs_batch, int64_t cs_row, const void* win_logits, float* hk, float* hv,
                               int zero_state, void* o, float* win_prob, int B, int HQ, int H, int K, int V, int M,
                               int W, float scale, void* stream) {
  if (!q || !k || !v || !g || !hk || !hv || !o) return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || HQ <= 0 || HQ % H != 0 || W < 1) return NHA_ERR_BAD_ARG;
  const bool logits_mode = win_logits != nullptr;
  if (!logits_mode) {
    if (!sw_k || !sw_v) return NHA_ERR_BAD_ARG;
    if ((cosp == nullptr) != (sinp == nullptr)) return NHA_ERR_BAD_ARG;
    if (!cosp && !sq) return NHA_ERR_BAD_ARG;
  }
  const int NG = HQ / H;
  if (K % 16 || V % 16 || K < 16 || V < 16 || K > 256 || V > 256 || M % 4 || M < 4 || M > 256 || NG > 16)
    return NHA_ERR_UNSUPPORTED;
  if (kDecThreads / (M / 4) < 1 || kDecThreads / (V / 4) < 1) return NHA_ERR_UNSUPPORTED;
  DecodeArgs a;
  a.q = (const bf16*)q; a.sq = (const bf16*)sq; a.k = (const bf16*)k; a.v = (const bf16*)v; a.g = (const bf16*)g;
  a.s = (const bf16*)s; a.sw_k = (const bf16*)sw_k; a.sw_v = (const bf16*)sw_v; a.cosp = (const bf16*)cosp;
  a.sinp = (const bf16*)sinp; a.win_logits = (const bf16*)win_logits;
  a.hk = hk; a.hv = hv; a.o = (bf16*)o; a.win_prob = win_prob;
  a.cs_batch = cs_batch; a.cs_row = cs_row;
  a.B = B; a.HQ = HQ; a.H = H; a.K = K; a.V = V; a.M = M; a.W = W; a.NG = NG; a.Wp = align_up(W, 16);
  a.NS = (W + kStageRows - 1) / kStageRows;
  a.zero_state = zero_state; a.scale = scale;
  const int smem = decode_layout(a);
  if (smem > kMaxSmem) return NHA_ERR_SMEM;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(B * H), block(kDecThreads);
#define NHA_LAUNCH_DECODE(NGM)                                                                              \
  do {                                                                                                      \
    cudaError_t e = cudaFuncSetAttribute(nha_decode_kernel<NGM>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                         smem);                                                             \
    if (e != cudaSuccess) return record_cuda_error(e);                                                      \
    nha_decode_kernel<NGM><<<grid, block, smem, st>>>(a);                                                   \
  } while (0)
  if (NG <= 1) NHA_LAUNCH_DECODE(1);
  else if (NG <= 2) NHA_LAUNCH_DECODE(2);
  else if (NG <= 4) NHA_LAUNCH_DECODE(4);
  else if (NG <= 8) NHA_LAUNCH_DECODE(8);
  else NHA_LAUNCH_DECODE(16);
#undef NHA_LAUNCH_DECODE
  return check_launch();
}
