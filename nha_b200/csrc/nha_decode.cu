// Fused NHA decode step for sm_100a: slot-state update + slot logits + window logits + joint
// softmax + slot/window readout in ONE launch.  The fp32 state and the window K/V of a
// (sequence, kv head) are read from HBM exactly once and serve all query heads of the group.
//
// The step is memory bound (about 6 flop per byte), so the kernel is organised around bytes in
// flight.  A (sequence, kv head) is cut into SPLITS independent CTAs; split s owns the window keys
// [s*KS, (s+1)*KS) (KS = 64) and the slots [s*MQ, (s+1)*MQ).  At entry every thread issues 16-byte
// asynchronous copies (cp.async) for the CTA's whole share - its columns of hk, its rows of hv, its
// key stage and its value stage - so everything the CTA will touch is in flight before any
// arithmetic starts, and three CTAs fit on an SM.  Each split computes an unnormalised partial
// softmax over its own logits (running max m_s, sum l_s, partial output o_s); the last CTA of a
// (sequence, kv head) to finish (an atomic ticket) merges the partials:
//     o = sum_s exp(m_s - m) o_s / sum_s exp(m_s - m) l_s,   m = max_s m_s.
//
// Replaces the two Triton launches of fused_recurrent_nha_decode
// (nha_fla/ops/nha/fused_recurrent.py:229-353 k-kernel, :356-428 v-kernel) and, with caller-supplied
// window logits, the kernels of fused_recurrent_nha (:48-147).
#include "nha_common.cuh"

namespace nha {

constexpr int kDecThreads = 256;
constexpr int kDecWarps = kDecThreads / 32;
constexpr int kMaxStageRows = 16 * kDecWarps;   // keys per CTA: one 16-key tile per warp
constexpr int kMaxSplits = 16;

struct DecodeArgs {
  const bf16* q; const bf16* sq; const bf16* k; const bf16* v; const bf16* g; const bf16* s;
  const bf16* sw_k; const bf16* sw_v; const bf16* cosp; const bf16* sinp; const bf16* win_logits;
  float* hk; float* hv; bf16* o; float* win_prob;
  float* part_o;      // [B*H, SPLITS, NG, V] unnormalised partial outputs
  float* part_ml;     // [B*H, SPLITS, NG, 2] running max and sum of each split
  int* tickets;       // [B*H] arrival counters, zero between calls
  int64_t cs_batch, cs_row;
  int B, HQ, H, K, V, M, W, NG, SPLITS, KS, KSp, MQ, zero_state;
  float scale;
  // shared-memory byte offsets
  int off_qraw, off_sqA, off_oks, off_eg, off_sv, off_kpop, off_vpop, off_ml, off_P, off_hk, off_hv, off_kst, off_vst,
      off_S;
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

// KT/VT: head dims known at compile time (0 = read them from the arguments), so that the index
// arithmetic of the copy loops folds into shifts.
template <int KT, int VT>
__global__ void __launch_bounds__(kDecThreads, 2) nha_decode_kernel(const DecodeArgs a) {
  using namespace nvcuda::wmma;
  extern __shared__ __align__(128) unsigned char smem[];
  float* qraw = reinterpret_cast<float*>(smem + a.off_qraw);      // [NG][K]   scaled raw query
  bf16* sqA = reinterpret_cast<bf16*>(smem + a.off_sqA);          // [16][K+8] rotated query (rows >= NG zero)
  float* oks = reinterpret_cast<float*>(smem + a.off_oks);        // [NG][MQ]  slot logits -> unnormalised slot weights
  float* eg = reinterpret_cast<float*>(smem + a.off_eg);          // [MQ]
  float* sv = reinterpret_cast<float*>(smem + a.off_sv);          // [MQ]
  float* kpop = reinterpret_cast<float*>(smem + a.off_kpop);      // [K]
  float* vpop = reinterpret_cast<float*>(smem + a.off_vpop);      // [V]
  float* ml = reinterpret_cast<float*>(smem + a.off_ml);          // [NG][2] running max, sum
  bf16* P = reinterpret_cast<bf16*>(smem + a.off_P);              // [16][KSp+8] unnormalised window weights
  float* hkS = reinterpret_cast<float*>(smem + a.off_hk);         // [K][MQ]   my columns of hk
  float* hvS = reinterpret_cast<float*>(smem + a.off_hv);         // [MQ][V]   my rows of hv
  bf16* kst = reinterpret_cast<bf16*>(smem + a.off_kst);          // [KSp][K+8]
  bf16* vst = reinterpret_cast<bf16*>(smem + a.off_vst);          // [KSp][V+8]
  float* S = reinterpret_cast<float*>(smem + a.off_S);            // [16][KSp+8] window logits; later [16][V+8] readout

  const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
  const int SPL = a.SPLITS;
  const int bh = blockIdx.x / SPL, sp = blockIdx.x % SPL;
  const int b = bh / a.H, h = bh % a.H;
  const int K = KT ? KT : a.K, V = VT ? VT : a.V;
  const int M = a.M, W = a.W, NG = a.NG, KSp = a.KSp, MQ = a.MQ;
  const int ldq = K + 8, ldk = K + 8, ldv = V + 8, lds = KSp + 8;
  const bool rotary = a.cosp != nullptr;
  const bool logits_mode = a.win_logits != nullptr;
  const int w0 = sp * a.KS;                                       // first key of this split
  const int nkeys = logits_mode ? 0 : max(0, min(a.KS, W - w0));  // keys of this split
  const int m0 = sp * MQ;                                         // first slot of this split
  const int nslots = max(0, min(MQ, M - m0));
  const int M4q = MQ >> 2;

  // ---- phase 0: the popped token, the gates and the queries (16-byte loads).  These few loads are
  //      issued before the bulk copies below so that they do not queue behind ~60 KB of traffic.
  for (int m = tid; m < MQ; m += kDecThreads) {
    float e = 1.f, sm = 0.f;
    if (m < nslots) {
      e = __expf(bf2f(a.g[(size_t)bh * M + m0 + m]));
      sm = a.s ? bf2f(a.s[(size_t)bh * M + m0 + m]) : 1.0f - e;
    }
    eg[m] = e;
    sv[m] = sm;
  }
  for (int i = tid; i < (K >> 3); i += kDecThreads) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(a.k + (size_t)bh * K + 8 * i), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) kpop[8 * i + e] = f[e];
  }
  for (int i = tid; i < (V >> 3); i += kDecThreads) {
    float f[8];
    unpack8(*reinterpret_cast<const uint4*>(a.v + (size_t)bh * V + 8 * i), f);
#pragma unroll
    for (int e = 0; e < 8; ++e) vpop[8 * i + e] = f[e];
  }
  {
    // queries: thread -> (row r of the 16-row A tile, 8-column group c); rows >= NG are zero
    const int c8h = K >> 4;
    const bf16* cq = rotary ? a.cosp + b * a.cs_batch + (int64_t)(W - 1) * a.cs_row : nullptr;
    const bf16* sn = rotary ? a.sinp + b * a.cs_batch + (int64_t)(W - 1) * a.cs_row : nullptr;
    for (int i = tid; i < 16 * c8h; i += kDecThreads) {
      const int r = i / c8h, c = i - r * c8h;
      float o1[8] = {0, 0, 0, 0, 0, 0, 0, 0}, o2[8] = {0, 0, 0, 0, 0, 0, 0, 0};
      if (r < NG) {
        const bf16* qrow = a.q + ((size_t)b * a.HQ + h * NG + r) * K;
        float x[8], y[8];
        unpack8(*reinterpret_cast<const uint4*>(qrow + 8 * c), x);
        unpack8(*reinterpret_cast<const uint4*>(qrow + 8 * (c + c8h)), y);
#pragma unroll
        for (int e = 0; e < 8; ++e) {
          qraw[r * K + 8 * c + e] = x[e] * a.scale;
          qraw[r * K + 8 * (c + c8h) + e] = y[e] * a.scale;
        }
        if (logits_mode) {
          // no window keys in this mode: the rotated query is not used
        } else if (rotary) {
          float c1[8], s1[8], c2[8], s2[8];
          unpack8(*reinterpret_cast<const uint4*>(cq + 8 * c), c1);
          unpack8(*reinterpret_cast<const uint4*>(sn + 8 * c), s1);
          unpack8(*reinterpret_cast<const uint4*>(cq + 8 * (c + c8h)), c2);
          unpack8(*reinterpret_cast<const uint4*>(sn + 8 * (c + c8h)), s2);
#pragma unroll
          for (int e = 0; e < 8; ++e) {
            o1[e] = x[e] * c1[e] - y[e] * s1[e];
            o2[e] = y[e] * c2[e] + x[e] * s2[e];
          }
        } else {
          const bf16* srow = a.sq + ((size_t)b * a.HQ + h * NG + r) * K;
          unpack8(*reinterpret_cast<const uint4*>(srow + 8 * c), o1);
          unpack8(*reinterpret_cast<const uint4*>(srow + 8 * (c + c8h)), o2);
        }
      }
      *reinterpret_cast<uint4*>(sqA + r * ldq + 8 * c) = pack8(o1);
      *reinterpret_cast<uint4*>(sqA + r * ldq + 8 * (c + c8h)) = pack8(o2);
    }
  }
  // ---- everything this CTA reads from the state and the window goes in flight now ------------------
  if (!a.zero_state && nslots > 0) {
    const float* hk_g = a.hk + (size_t)bh * K * M + m0;
    for (int i = tid; i < K * M4q; i += kDecThreads) {
      const int kk = i / M4q, c = i - kk * M4q;
      const bool ok = 4 * c < nslots;
      cp_async16(hkS + kk * MQ + 4 * c, hk_g + (size_t)kk * M + (ok ? 4 * c : 0), ok);
    }
    const float* hv_g = a.hv + ((size_t)bh * M + m0) * V;
    for (int i = tid; i < nslots * (V >> 2); i += kDecThreads) cp_async16(hvS + 4 * i, hv_g + 4 * i, true);
  }
  if (nkeys > 0) {
    const int c8k = K >> 3;
    for (int i = tid; i < KSp * c8k; i += kDecThreads) {
      const int r = i / c8k, c = i - r * c8k;
      const bool ok = r < nkeys;
      cp_async16(kst + r * ldk + 8 * c, a.sw_k + (((size_t)b * W + (ok ? w0 + r : 0)) * a.H + h) * K + 8 * c, ok);
    }
  }
  cp_async_commit();
  if (nkeys > 0) {
    const int c8v = V >> 3;
    for (int i = tid; i < KSp * c8v; i += kDecThreads) {
      const int r = i / c8v, c = i - r * c8v;
      const bool ok = r < nkeys;
      cp_async16(vst + r * ldv + 8 * c, a.sw_v + (((size_t)b * W + (ok ? w0 + r : 0)) * a.H + h) * V + 8 * c, ok);
    }
  }
  cp_async_commit();

  for (int i = tid; i < 16 * lds; i += kDecThreads) P[i] = f2bf(0.f);
  cp_async_wait<1>();        // state columns/rows and the key stage have landed
  __syncthreads();

  // ---- phase 1: my columns of hk <- hk * exp(g) + k s^T (in place), slot logits of my slots ---------
  if (nslots > 0) {
    float* hg = a.hk + (size_t)bh * K * M + m0;
    for (int i = tid; i < K * M4q; i += kDecThreads) {
      const int kk = i / M4q, c = i - kk * M4q;
      if (4 * c < nslots) {
        float4 hh = a.zero_state ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(hkS + kk * MQ + 4 * c);
        const float4 e4 = *reinterpret_cast<const float4*>(eg + 4 * c);
        const float4 s4 = *reinterpret_cast<const float4*>(sv + 4 * c);
        const float kv = kpop[kk];
        hh.x = hh.x * e4.x + kv * s4.x;
        hh.y = hh.y * e4.y + kv * s4.y;
        hh.z = hh.z * e4.z + kv * s4.z;
        hh.w = hh.w * e4.w + kv * s4.w;
        *reinterpret_cast<float4*>(hkS + kk * MQ + 4 * c) = hh;
        *reinterpret_cast<float4*>(hg + (size_t)kk * M + 4 * c) = hh;
      }
    }
    __syncthreads();
    // ok[qh][m] = sum_k q[qh][k] hk[k][m]: four threads per (qh, m), each over a quarter of k,
    // combined with two shuffles (every lane takes part; idle tasks add zero)
    for (int i0 = 0; i0 < NG * nslots * 4; i0 += kDecThreads) {
      const int i = i0 + tid;
      const int part = i & 3, om = i >> 2;
      float acc = 0.f;
      if (om < NG * nslots) {
        const int qh = om / nslots, m = om - qh * nslots;
        const int kq = K >> 2;
#pragma unroll 8
        for (int kk = part * kq; kk < (part + 1) * kq; ++kk) acc += qraw[qh * K + kk] * hkS[kk * MQ + m];
      }
      acc += __shfl_xor_sync(0xffffffffu, acc, 1);
      acc += __shfl_xor_sync(0xffffffffu, acc, 2);
      if (om < NG * nslots && part == 0) {
        const int qh = om / nslots, m = om - qh * nslots;
        oks[qh * MQ + m] = acc;
      }
    }
  }

  // ---- phase 2: window logits of my keys: in-place rotate-half, then S = sq K^T ----------------------
  if (logits_mode) {
    if (sp == 0)
      for (int i = tid; i < NG * W; i += kDecThreads) {
        const int qh = i / W, w = i - qh * W;
        S[qh * lds + w] = bf2f(a.win_logits[((size_t)b * a.HQ + h * NG + qh) * W + w]);
      }
  } else if (nkeys > 0) {
    if (rotary) {
      const int c8h = K >> 4;
      const int tasks = KSp * c8h;
      for (int i0 = tid; i0 < tasks; i0 += 4 * kDecThreads) {
        uint4 cs[4][4];
        // all table loads of up to four tasks are issued before any is used (one L2 round trip)
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * kDecThreads;
          const int r = i / c8h, c = i - r * c8h;
          if (i < tasks && r < nkeys) {
            const bf16* crow = a.cosp + b * a.cs_batch + (int64_t)(w0 + r) * a.cs_row;
            const bf16* srow = a.sinp + b * a.cs_batch + (int64_t)(w0 + r) * a.cs_row;
            cs[u][0] = __ldg(reinterpret_cast<const uint4*>(crow + 8 * c));
            cs[u][1] = __ldg(reinterpret_cast<const uint4*>(srow + 8 * c));
            cs[u][2] = __ldg(reinterpret_cast<const uint4*>(crow + 8 * (c + c8h)));
            cs[u][3] = __ldg(reinterpret_cast<const uint4*>(srow + 8 * (c + c8h)));
          }
        }
#pragma unroll
        for (int u = 0; u < 4; ++u) {
          const int i = i0 + u * kDecThreads;
          const int r = i / c8h, c = i - r * c8h;
          if (i < tasks && r < nkeys) {
            float x[8], y[8], c1[8], s1[8], c2[8], s2[8], o1[8], o2[8];
            unpack8(*reinterpret_cast<const uint4*>(kst + r * ldk + 8 * c), x);
            unpack8(*reinterpret_cast<const uint4*>(kst + r * ldk + 8 * (c + c8h)), y);
            unpack8(cs[u][0], c1); unpack8(cs[u][1], s1); unpack8(cs[u][2], c2); unpack8(cs[u][3], s2);
#pragma unroll
            for (int e = 0; e < 8; ++e) {
              o1[e] = x[e] * c1[e] - y[e] * s1[e];
              o2[e] = y[e] * c2[e] + x[e] * s2[e];
            }
            *reinterpret_cast<uint4*>(kst + r * ldk + 8 * c) = pack8(o1);
            *reinterpret_cast<uint4*>(kst + r * ldk + 8 * (c + c8h)) = pack8(o2);
          }
        }
      }
      __syncthreads();
    }
    for (int t = warp; t < KSp / 16; t += kDecWarps) {
      fragment<accumulator, 16, 16, 16, float> acc;
      fill_fragment(acc, 0.f);
      for (int ks = 0; ks < K / 16; ++ks) {
        fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
        fragment<matrix_b, 16, 16, 16, bf16, col_major> fb;
        load_matrix_sync(fa, sqA + 16 * ks, ldq);
        load_matrix_sync(fb, kst + (size_t)16 * t * ldk + 16 * ks, ldk);
        mma_sync(acc, fa, fb, acc);
      }
      store_matrix_sync(S + 16 * t, acc, lds, mem_row_major);
    }
  }
  __syncthreads();

  // ---- phase 3: partial softmax over [my slots | my keys], one warp per query head ----------------
  const float wscale = logits_mode ? 1.0f : a.scale;
  const int nwin = logits_mode ? (sp == 0 ? W : 0) : nkeys;
  for (int qh = warp; qh < NG; qh += kDecWarps) {
    float mx = -INFINITY;
    for (int m = lane; m < nslots; m += 32) mx = fmaxf(mx, oks[qh * MQ + m]);
    for (int w = lane; w < nwin; w += 32) mx = fmaxf(mx, S[qh * lds + w] * wscale);
    mx = warp_max(mx);
    float sum = 0.f;
    for (int m = lane; m < nslots; m += 32) {
      const float e = __expf(oks[qh * MQ + m] - mx);
      oks[qh * MQ + m] = e;
      sum += e;
    }
    for (int w = lane; w < nwin; w += 32) {
      const float e = __expf(S[qh * lds + w] * wscale - mx);
      if (logits_mode) S[qh * lds + w] = e;
      else P[qh * lds + w] = f2bf(e);
      sum += e;
    }
    sum = warp_sum(sum);
    if (lane == 0) {
      ml[2 * qh] = (nslots + nwin) > 0 ? mx : -INFINITY;
      ml[2 * qh + 1] = sum;
    }
  }
  cp_async_wait<0>();        // the value stage has landed
  __syncthreads();

  // fused_recurrent_nha mode: the window part of the softmax goes back to the caller (one split only)
  if (logits_mode && a.win_prob)
    for (int i = tid; i < NG * W; i += kDecThreads) {
      const int qh = i / W, w = i - qh * W;
      a.win_prob[((size_t)b * a.HQ + h * NG + qh) * W + w] = S[qh * lds + w] / ml[2 * qh + 1];
    }
  __syncthreads();

  // ---- phase 4: window readout of my keys (S is dead: its space takes the [16][V+8] result) ---------
  float* oacc = S;
  const int ldo = V + 8;
  if (!logits_mode && nkeys > 0) {
    for (int ct = warp; ct < V / 16; ct += kDecWarps) {
      fragment<accumulator, 16, 16, 16, float> acc;
      fill_fragment(acc, 0.f);
      for (int kt = 0; kt < KSp / 16; ++kt) {
        fragment<matrix_a, 16, 16, 16, bf16, row_major> fa;
        fragment<matrix_b, 16, 16, 16, bf16, row_major> fb;
        load_matrix_sync(fa, P + 16 * kt, lds);
        load_matrix_sync(fb, vst + (size_t)16 * kt * ldv + 16 * ct, ldv);
        mma_sync(acc, fa, fb, acc);
      }
      store_matrix_sync(oacc + 16 * ct, acc, ldo, mem_row_major);
    }
  }

  // ---- phase 5: my rows of hv <- diag(exp(g)) hv + s v^T (in place), slot readout -------------------
  const int V4 = V >> 2;
  if (nslots > 0) {
    float4* hg = reinterpret_cast<float4*>(a.hv + ((size_t)bh * M + m0) * V);
    for (int i = tid; i < nslots * V4; i += kDecThreads) {
      const int m = i / V4, c = i - m * V4;
      float4 hh = a.zero_state ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(hvS + m * V + 4 * c);
      const float4 vp4 = *reinterpret_cast<const float4*>(vpop + 4 * c);
      const float e = eg[m], sm = sv[m];
      hh.x = hh.x * e + sm * vp4.x;
      hh.y = hh.y * e + sm * vp4.y;
      hh.z = hh.z * e + sm * vp4.z;
      hh.w = hh.w * e + sm * vp4.w;
      *reinterpret_cast<float4*>(hvS + m * V + 4 * c) = hh;
      hg[i] = hh;
    }
  }
  __syncthreads();
  // partial output of this split: slot part + window part, unnormalised
  float* po = a.part_o + ((size_t)bh * SPL + sp) * NG * V;
  for (int i = tid; i < NG * V4; i += kDecThreads) {
    const int qh = i / V4, c = i - qh * V4;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    for (int m = 0; m < nslots; ++m) {
      const float pm = oks[qh * MQ + m];
      const float4 hh = *reinterpret_cast<const float4*>(hvS + m * V + 4 * c);
      acc.x += pm * hh.x; acc.y += pm * hh.y; acc.z += pm * hh.z; acc.w += pm * hh.w;
    }
    if (!logits_mode && nkeys > 0) {
      const float4 wv = *reinterpret_cast<const float4*>(oacc + qh * ldo + 4 * c);
      acc.x += wv.x; acc.y += wv.y; acc.z += wv.z; acc.w += wv.w;
    }
    if (SPL == 1) {
      const float inv = 1.0f / ml[2 * qh + 1];
      bf16* orow = a.o + ((size_t)b * a.HQ + h * NG + qh) * V + 4 * c;
      orow[0] = f2bf(acc.x * inv); orow[1] = f2bf(acc.y * inv); orow[2] = f2bf(acc.z * inv); orow[3] = f2bf(acc.w * inv);
    } else {
      *reinterpret_cast<float4*>(po + qh * V + 4 * c) = acc;
    }
  }
  if (SPL == 1) return;

  // ---- merge: the last split of this (sequence, kv head) to arrive combines all partials ------------
  float* pml = a.part_ml + ((size_t)bh * SPL + sp) * NG * 2;
  for (int i = tid; i < NG * 2; i += kDecThreads) pml[i] = ml[i];
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
  const float* all_ml = a.part_ml + (size_t)bh * SPL * NG * 2;
  float* wgt = qraw;                    // [SPL][NG] merge weights exp(m_s - m) / denominator
  for (int qh = tid; qh < NG; qh += kDecThreads) {
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
  const float* all_o = a.part_o + (size_t)bh * SPL * NG * V;
  for (int i = tid; i < NG * V4; i += kDecThreads) {
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

static int decode_layout(DecodeArgs& a) {
  const int K = a.K, V = a.V, NG = a.NG, KSp = a.KSp, MQ = a.MQ;
  int off = 0;
  auto take = [&](int bytes) { int o = off; off = align_up(off + bytes, 128); return o; };
  a.off_qraw = take(max(NG * K, kMaxSplits * NG) * 4);
  a.off_sqA = take(16 * (K + 8) * 2);
  a.off_oks = take(NG * MQ * 4);
  a.off_eg = take(MQ * 4);
  a.off_sv = take(MQ * 4);
  a.off_kpop = take(K * 4);
  a.off_vpop = take(V * 4);
  a.off_ml = take(NG * 2 * 4);
  a.off_P = take(16 * (KSp + 8) * 2);
  a.off_hk = take(K * MQ * 4);
  a.off_hv = take(MQ * V * 4);
  const int srows = a.win_logits ? 0 : KSp;          // no key/value stages when the caller supplies the logits
  a.off_kst = take(srows * (K + 8) * 2);
  a.off_vst = take(srows * (V + 8) * 2);
  a.off_S = take(16 * max(KSp + 8, V + 8) * 4);
  return off;
}

// splits of a (sequence, kv head): 64 keys per split for short windows, 128 from W = 256 on
static int decode_splits(int W, bool logits_mode) {
  if (logits_mode) return 1;
  const int per = W < 256 ? 64 : kMaxStageRows;
  return (W + per - 1) / per;
}

int decode_stream_splits(int B, int H, int W, int M);
int decode_pdl_mode();
void decode_set_pdl_mode(int m);
bool decode_stream_supported(int K, int V, int M, int W, int NG, bool logits_mode);
int decode_stream_try(const void* q, const void* sq, const void* k, const void* v, const void* g, const void* s,
                      const void* sw_k, const void* sw_v, const void* cosp, const void* sinp, int64_t cs_batch,
                      int64_t cs_row, float* hk, float* hv, int zero_state, void* o, int* tickets, int* err,
                      float* part_ml, float* part_o, int splits, int B, int HQ, int H, int D, int M, int W, float scale,
                      cudaStream_t st, const int* head, const void* ring_g, int ring_rows, int nopop,
                      const void* ring_kraw, const void* g_new, int state_bf16);

// Workspace: [B*H tickets | error word] (ints, zero between calls), then the (max, sum) and the partial outputs of
// every split.  Sized for whichever kernel cuts a (sequence, kv head) into more splits.
static int decode_max_splits(int B, int H, int W) {
  const int a = decode_splits(W, false), b = decode_stream_splits(B, H, W, 1 << 20);
  return a > b ? a : b;
}

}  // namespace nha

using namespace nha;

extern "C" int64_t nha_decode_workspace_bytes(int B, int HQ, int H, int V, int W) {
  if (B <= 0 || H <= 0 || HQ <= 0 || HQ % H) return 0;
  const int64_t spl = decode_max_splits(B, H, W);
  const int64_t NG = HQ / H;
  return (int64_t)B * H * spl * NG * (V + 2) * 4 + ((int64_t)B * H + 1) * 4 + 1024;
}

extern "C" int nha_decode_set_pdl(int mode) {
  if (mode < 0 || mode > 2) return NHA_ERR_BAD_ARG;
  decode_set_pdl_mode(mode);
  return NHA_OK;
}
extern "C" int nha_decode_get_pdl(void) { return decode_pdl_mode(); }

extern "C" int nha_decode_device_error(const void* workspace, int B, int H, void* stream) {
  if (!workspace || B <= 0 || H <= 0) return 0;
  int v = 0;
  cudaError_t e = cudaMemcpyAsync(&v, (const int*)workspace + (size_t)B * H, sizeof(int), cudaMemcpyDeviceToHost,
                                  (cudaStream_t)stream);
  if (e == cudaSuccess) e = cudaStreamSynchronize((cudaStream_t)stream);
  if (e != cudaSuccess) return record_cuda_error(e);
  return v;
}

static int decode_step_impl(const void* q, const void* sq, const void* k, const void* v, const void* g, const void* s,
                            const void* sw_k, const void* sw_v, const void* cosp, const void* sinp, int64_t cs_batch,
                            int64_t cs_row, const void* win_logits, float* hk, float* hv, int state_bf16, int zero_state,
                            void* o, float* win_prob, void* workspace, int64_t workspace_bytes, int B, int HQ, int H, int K,
                            int V, int M, int W, float scale, void* stream) {
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
  DecodeArgs a;
  a.q = (const bf16*)q; a.sq = (const bf16*)sq; a.k = (const bf16*)k; a.v = (const bf16*)v; a.g = (const bf16*)g;
  a.s = (const bf16*)s; a.sw_k = (const bf16*)sw_k; a.sw_v = (const bf16*)sw_v; a.cosp = (const bf16*)cosp;
  a.sinp = (const bf16*)sinp; a.win_logits = (const bf16*)win_logits;
  a.hk = hk; a.hv = hv; a.o = (bf16*)o; a.win_prob = win_prob;
  a.cs_batch = cs_batch; a.cs_row = cs_row;
  a.B = B; a.HQ = HQ; a.H = H; a.K = K; a.V = V; a.M = M; a.W = W; a.NG = NG;
  // common shapes take the streaming kernel (ring of bulk copies, whole grid resident in one wave)
  const char* force_general = getenv("NHA_B200_DECODE_GENERAL");
  const bool stream_ok = decode_stream_supported(K, V, M, W, NG, logits_mode) && !(force_general && force_general[0] == '1');
  if (state_bf16 && !stream_ok) return NHA_ERR_UNSUPPORTED;      // bf16 slot memory: streaming kernel only
  a.SPLITS = stream_ok ? decode_stream_splits(B, H, W, M) : decode_splits(W, logits_mode);
  if (a.SPLITS > kMaxSplits) return NHA_ERR_UNSUPPORTED;
  if (logits_mode) {
    a.KS = 0;
    a.KSp = align_up(W, 16);                  // S holds the caller's logits
  } else {
    a.KS = align_up((W + a.SPLITS - 1) / a.SPLITS, 16);
    a.KSp = a.KS;
  }
  a.MQ = align_up((M + a.SPLITS - 1) / a.SPLITS, 4);
  a.zero_state = zero_state; a.scale = scale;
  a.part_o = nullptr; a.part_ml = nullptr; a.tickets = nullptr;
  int* errw = nullptr;
  if (a.SPLITS > 1 || stream_ok) {
    if (a.SPLITS > 1 && (!workspace || workspace_bytes < nha_decode_workspace_bytes(B, HQ, H, V, W))) return NHA_ERR_WORKSPACE;
    if (workspace && workspace_bytes >= nha_decode_workspace_bytes(B, HQ, H, V, W)) {
      // tickets and the error word first (they must stay zero between calls), then the partials
      a.tickets = (int*)workspace;
      errw = a.tickets + (size_t)B * H;
      char* base = (char*)workspace + align_up((B * H + 1) * 4, 256);
      a.part_ml = (float*)base;
      a.part_o = (float*)(base + align_up(B * H * a.SPLITS * NG * 2 * 4, 256));
    }
  }
  if (stream_ok)
    return decode_stream_try(q, sq, k, v, g, s, sw_k, sw_v, cosp, sinp, cs_batch, cs_row, hk, hv, zero_state, o, a.tickets,
                             errw, a.part_ml, a.part_o, a.SPLITS, B, HQ, H, K, M, W, scale, (cudaStream_t)stream, nullptr,
                             nullptr, W, 0, nullptr, nullptr, state_bf16);
  const int smem = decode_layout(a);
  if (smem > kMaxSmem) return NHA_ERR_SMEM;
  cudaStream_t st = (cudaStream_t)stream;
  dim3 grid(B * H * a.SPLITS), block(kDecThreads);
#define NHA_LAUNCH_DECODE(KT_, VT_)                                                                               \
  do {                                                                                                            \
    cudaError_t e = set_max_smem((const void*)nha_decode_kernel<KT_, VT_>, \
                                         smem);                                                                   \
    if (e != cudaSuccess) return record_cuda_error(e);                                                            \
    nha_decode_kernel<KT_, VT_><<<grid, block, smem, st>>>(a);                                                    \
  } while (0)
  if (K == 128 && V == 128) NHA_LAUNCH_DECODE(128, 128);
  else if (K == 64 && V == 64) NHA_LAUNCH_DECODE(64, 64);
  else NHA_LAUNCH_DECODE(0, 0);
#undef NHA_LAUNCH_DECODE
  return check_launch();
}

extern "C" int nha_decode_step(const void* q, const void* sq, const void* k, const void* v, const void* g,
                               const void* s, const void* sw_k, const void* sw_v, const void* cosp, const void* sinp,
                               int64_t cs_batch, int64_t cs_row, const void* win_logits, float* hk, float* hv,
                               int zero_state, void* o, float* win_prob, void* workspace, int64_t workspace_bytes,
                               int B, int HQ, int H, int K, int V, int M, int W, float scale, void* stream) {
  return decode_step_impl(q, sq, k, v, g, s, sw_k, sw_v, cosp, sinp, cs_batch, cs_row, win_logits, hk, hv, 0, zero_state, o,
                          win_prob, workspace, workspace_bytes, B, HQ, H, K, V, M, W, scale, stream);
}

extern "C" int nha_decode_step_bf16_state(const void* q, const void* sq, const void* k, const void* v, const void* g,
                                          const void* s, const void* sw_k, const void* sw_v, const void* cosp,
                                          const void* sinp, int64_t cs_batch, int64_t cs_row, void* hk, void* hv,
                                          int zero_state, void* o, void* workspace, int64_t workspace_bytes, int B, int HQ,
                                          int H, int K, int V, int M, int W, float scale, void* stream) {
  if (((uintptr_t)hk & 15) || ((uintptr_t)hv & 15)) return NHA_ERR_BAD_ARG;
  return decode_step_impl(q, sq, k, v, g, s, sw_k, sw_v, cosp, sinp, cs_batch, cs_row, nullptr, (float*)hk, (float*)hv, 1,
                          zero_state, o, nullptr, workspace, workspace_bytes, B, HQ, H, K, V, M, W, scale, stream);
}

// ---------------------------------------------------------------------------------------------
// Decode on a device-resident ring buffer: the window keys / values / gate rows of a sequence live in rings of
// W rows whose oldest entry sits at row head[b].  One step = nha_decode_step_ring (the oldest entry enters the
// slot memory, the new token is the newest window entry) followed by nha_ring_append (the new token's rows
// overwrite the oldest entry, head advances) - no window is ever shifted in memory.
namespace nha {

__global__ void nha_ring_append_kernel(bf16* ring_k, bf16* ring_v, bf16* ring_g, const bf16* k, const bf16* v, const bf16* g,
                                       int* head, int H, int K, int V, int M, int W, int fill) {
  const int b = blockIdx.x;
  const int hd = fill < W ? fill : head[b];        // a ring that is still filling takes the token in its next free row
  const size_t row = (size_t)b * W + hd;
  for (int i = threadIdx.x; i < H * K / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(ring_k + row * H * K)[i] = reinterpret_cast<const uint4*>(k + (size_t)b * H * K)[i];
  for (int i = threadIdx.x; i < H * V / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(ring_v + row * H * V)[i] = reinterpret_cast<const uint4*>(v + (size_t)b * H * V)[i];
  for (int i = threadIdx.x; i < H * M / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(ring_g + row * H * M)[i] = reinterpret_cast<const uint4*>(g + (size_t)b * H * M)[i];
  __syncthreads();
  if (threadIdx.x == 0 && fill >= W) head[b] = hd + 1 == W ? 0 : hd + 1;
}

}  // namespace nha

extern "C" int nha_decode_step_ring(const void* q, const void* k_new, const void* v_new, const void* ring_k,
                                    const void* ring_v, const void* ring_g, const int32_t* head, const void* cosp,
                                    const void* sinp, int64_t cs_batch, int64_t cs_row, float* hk, float* hv, void* o,
                                    void* workspace, int64_t workspace_bytes, int B, int HQ, int H, int K, int V, int M,
                                    int W, int fill, float scale, void* stream) {
  if (!q || !k_new || !v_new || !ring_k || !ring_v || !ring_g || !head || !cosp || !sinp || !hk || !hv || !o)
    return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || HQ <= 0 || HQ % H != 0 || W < 1 || fill < 0 || fill > W) return NHA_ERR_BAD_ARG;
  const int NG = HQ / H;
  // a full ring: W window entries (the oldest leaves); a filling ring: its `fill` rows and the new token
  const int nopop = fill < W, Weff = nopop ? fill + 1 : W;
  if (!decode_stream_supported(K, V, M, Weff, NG, false) || M % 8) return NHA_ERR_UNSUPPORTED;
  const int splits = decode_stream_splits(B, H, Weff, M);
  if (!workspace || workspace_bytes < nha_decode_workspace_bytes(B, HQ, H, V, W)) return NHA_ERR_WORKSPACE;
  int* tickets = (int*)workspace;
  int* errw = tickets + (size_t)B * H;
  char* base = (char*)workspace + align_up((B * H + 1) * 4, 256);
  float* part_ml = (float*)base;
  float* part_o = (float*)(base + align_up(B * H * splits * NG * 2 * 4, 256));
  return decode_stream_try(q, nullptr, k_new, v_new, nullptr, nullptr, ring_k, ring_v, cosp, sinp, cs_batch, cs_row, hk, hv, 0,
                           o, tickets, errw, part_ml, part_o, splits, B, HQ, H, K, M, Weff, scale, (cudaStream_t)stream, head,
                           ring_g, W, nopop, nullptr, nullptr, 0);
}

extern "C" int nha_decode_step_ring_fused(const void* q, const void* k_new, const void* v_new, const void* g_new, void* ring_k,
                                          void* ring_v, void* ring_g, int32_t* head, const void* cosp, const void* sinp,
                                          int64_t cs_batch, int64_t cs_row, float* hk, float* hv, void* o, void* workspace,
                                          int64_t workspace_bytes, int B, int HQ, int H, int K, int V, int M, int W, int fill,
                                          float scale, void* stream) {
  if (!q || !k_new || !v_new || !g_new || !ring_k || !ring_v || !ring_g || !head || !cosp || !sinp || !hk || !hv || !o)
    return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || HQ <= 0 || HQ % H != 0 || W < 1 || fill < 0 || fill > W) return NHA_ERR_BAD_ARG;
  const int NG = HQ / H;
  const int nopop = fill < W, Weff = nopop ? fill + 1 : W;
  if (!decode_stream_supported(K, V, M, Weff, NG, false) || M % 8) return NHA_ERR_UNSUPPORTED;
  const int splits = decode_stream_splits(B, H, Weff, M);
  if (!workspace || workspace_bytes < nha_decode_workspace_bytes(B, HQ, H, V, W)) return NHA_ERR_WORKSPACE;
  int* tickets = (int*)workspace;
  int* errw = tickets + (size_t)B * H;
  char* base = (char*)workspace + align_up((B * H + 1) * 4, 256);
  float* part_ml = (float*)base;
  float* part_o = (float*)(base + align_up(B * H * splits * NG * 2 * 4, 256));
  return decode_stream_try(q, nullptr, k_new, v_new, nullptr, nullptr, ring_k, ring_v, cosp, sinp, cs_batch, cs_row, hk, hv, 0,
                           o, tickets, errw, part_ml, part_o, splits, B, HQ, H, K, M, Weff, scale, (cudaStream_t)stream, head,
                           ring_g, W, nopop, nullptr, g_new, 0);
}

extern "C" int nha_ring_append(void* ring_k, void* ring_v, void* ring_g, const void* k_new, const void* v_new,
                               const void* g_new, int32_t* head, int B, int H, int K, int V, int M, int W, int fill,
                               void* stream) {
  if (!ring_k || !ring_v || !ring_g || !k_new || !v_new || !g_new || !head) return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || W < 1 || fill < 0 || fill > W || (H * K) % 8 || (H * V) % 8 || (H * M) % 8) return NHA_ERR_BAD_ARG;
  nha_ring_append_kernel<<<B, 128, 0, (cudaStream_t)stream>>>((bf16*)ring_k, (bf16*)ring_v, (bf16*)ring_g, (const bf16*)k_new,
                                                              (const bf16*)v_new, (const bf16*)g_new, head, H, K, V, M, W, fill);
  return check_launch();
}

// ---------------------------------------------------------------------------------------------
// Rings with keys rotated on entry.  Rotary by absolute position does not change while the window slides, so a
// key can be rotated once, when it enters the ring, instead of at every step it stays in the window (the
// reference rotates the whole window every step, nha_fla/models/qwen3_moe_nha/qwennha.py:207-226, with a memo for
// the tables only).  The raw key is still needed once more, when the token leaves the window and enters the
// slot memory, so the cache keeps both rings.  The rotation below is the packed bf16 arithmetic of the streaming
// decode kernel, operation for operation, so that both layouts give the same bits.
namespace nha {

__device__ __forceinline__ void rotate_half_row(bf16* dst, const bf16* src, const bf16* crow, const bf16* srow, int H, int K,
                                                int tid, int nthreads) {
  const int c8h = K >> 4;
  for (int i = tid; i < H * c8h; i += nthreads) {
    const int hh = i / c8h, c = i - hh * c8h;
    const uint4 xu = *reinterpret_cast<const uint4*>(src + hh * K + 8 * c);
    const uint4 yu = *reinterpret_cast<const uint4*>(src + hh * K + 8 * (c + c8h));
    const uint4 c1u = __ldg(reinterpret_cast<const uint4*>(crow + 8 * c));
    const uint4 s1u = __ldg(reinterpret_cast<const uint4*>(srow + 8 * c));
    const uint4 c2u = __ldg(reinterpret_cast<const uint4*>(crow + 8 * (c + c8h)));
    const uint4 s2u = __ldg(reinterpret_cast<const uint4*>(srow + 8 * (c + c8h)));
    uint4 o1u, o2u;
    const __nv_bfloat162* xv = reinterpret_cast<const __nv_bfloat162*>(&xu);
    const __nv_bfloat162* yv = reinterpret_cast<const __nv_bfloat162*>(&yu);
    const __nv_bfloat162* c1v = reinterpret_cast<const __nv_bfloat162*>(&c1u);
    const __nv_bfloat162* s1v = reinterpret_cast<const __nv_bfloat162*>(&s1u);
    const __nv_bfloat162* c2v = reinterpret_cast<const __nv_bfloat162*>(&c2u);
    const __nv_bfloat162* s2v = reinterpret_cast<const __nv_bfloat162*>(&s2u);
    __nv_bfloat162* o1v = reinterpret_cast<__nv_bfloat162*>(&o1u);
    __nv_bfloat162* o2v = reinterpret_cast<__nv_bfloat162*>(&o2u);
#pragma unroll
    for (int e = 0; e < 4; ++e) {
      o1v[e] = __hfma2(xv[e], c1v[e], __hneg2(__hmul2(yv[e], s1v[e])));
      o2v[e] = __hfma2(yv[e], c2v[e], __hmul2(xv[e], s2v[e]));
    }
    *reinterpret_cast<uint4*>(dst + hh * K + 8 * c) = o1u;
    *reinterpret_cast<uint4*>(dst + hh * K + 8 * (c + c8h)) = o2u;
  }
}

// one CTA per (sequence, ring row): ring_kr[b, r] = rotate(ring_k[b, r]) with table row r
__global__ void nha_ring_rotate_rows_kernel(const bf16* ring_k, bf16* ring_kr, const bf16* cosp, const bf16* sinp,
                                            int64_t cs_batch, int64_t cs_row, int H, int K, int W) {
  const int b = blockIdx.y, r = blockIdx.x;
  const size_t row = ((size_t)b * W + r) * H * K;
  rotate_half_row(ring_kr + row, ring_k + row, cosp + b * cs_batch + r * cs_row, sinp + b * cs_batch + r * cs_row, H, K,
                  threadIdx.x, blockDim.x);
}

__global__ void nha_ring_append_rot_kernel(bf16* ring_k, bf16* ring_kr, bf16* ring_v, bf16* ring_g, const bf16* k,
                                           const bf16* v, const bf16* g, const bf16* cosq, const bf16* sinq, int64_t cs_batch,
                                           int* head, int H, int K, int V, int M, int W, int fill) {
  const int b = blockIdx.x;
  const int hd = fill < W ? fill : head[b];
  const size_t row = (size_t)b * W + hd;
  for (int i = threadIdx.x; i < H * K / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(ring_k + row * H * K)[i] = reinterpret_cast<const uint4*>(k + (size_t)b * H * K)[i];
  rotate_half_row(ring_kr + row * H * K, k + (size_t)b * H * K, cosq + b * cs_batch, sinq + b * cs_batch, H, K, threadIdx.x,
                  blockDim.x);
  for (int i = threadIdx.x; i < H * V / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(ring_v + row * H * V)[i] = reinterpret_cast<const uint4*>(v + (size_t)b * H * V)[i];
  for (int i = threadIdx.x; i < H * M / 8; i += blockDim.x)
    reinterpret_cast<uint4*>(ring_g + row * H * M)[i] = reinterpret_cast<const uint4*>(g + (size_t)b * H * M)[i];
  __syncthreads();
  if (threadIdx.x == 0 && fill >= W) head[b] = hd + 1 == W ? 0 : hd + 1;
}

}  // namespace nha

extern "C" int nha_ring_rotate_rows(const void* ring_k, void* ring_kr, const void* cosp, const void* sinp, int64_t cs_batch,
                                    int64_t cs_row, int B, int H, int K, int W, int rows, void* stream) {
  if (!ring_k || !ring_kr || !cosp || !sinp) return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || W < 1 || rows < 0 || rows > W) return NHA_ERR_BAD_ARG;
  if (K <= 0 || K % 16 || cs_row % 8 || cs_batch % 8) return NHA_ERR_UNSUPPORTED;
  if (rows == 0) return NHA_OK;
  nha_ring_rotate_rows_kernel<<<dim3(rows, B), 128, 0, (cudaStream_t)stream>>>((const bf16*)ring_k, (bf16*)ring_kr,
                                                                             (const bf16*)cosp, (const bf16*)sinp, cs_batch,
                                                                             cs_row, H, K, W);
  return check_launch();
}

extern "C" int nha_decode_step_ring_rot(const void* q, const void* k_new, const void* v_new, const void* ring_k,
                                        const void* ring_kr, const void* ring_v, const void* ring_g, const int32_t* head,
                                        const void* cos_q, const void* sin_q, int64_t cs_batch, float* hk, float* hv, void* o,
                                        void* workspace, int64_t workspace_bytes, int B, int HQ, int H, int K, int V, int M,
                                        int W, int fill, float scale, void* stream) {
  if (!q || !k_new || !v_new || !ring_k || !ring_kr || !ring_v || !ring_g || !head || !cos_q || !sin_q || !hk || !hv || !o)
    return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || HQ <= 0 || HQ % H != 0 || W < 1 || fill < 0 || fill > W) return NHA_ERR_BAD_ARG;
  const int NG = HQ / H;
  const int nopop = fill < W, Weff = nopop ? fill + 1 : W;
  if (!decode_stream_supported(K, V, M, Weff, NG, false) || M % 8) return NHA_ERR_UNSUPPORTED;
  const int splits = decode_stream_splits(B, H, Weff, M);
  if (!workspace || workspace_bytes < nha_decode_workspace_bytes(B, HQ, H, V, W)) return NHA_ERR_WORKSPACE;
  int* tickets = (int*)workspace;
  int* errw = tickets + (size_t)B * H;
  char* base = (char*)workspace + align_up((B * H + 1) * (int)sizeof(int), 256);
  float* part_ml = (float*)base;
  float* part_o = (float*)(base + align_up(B * H * splits * NG * 2 * 4, 256));
  // a table row stride of 0: every window position reads the query's row; the kernel rotates only the query and the
  // token of this step
  return decode_stream_try(q, nullptr, k_new, v_new, nullptr, nullptr, ring_kr, ring_v, cos_q, sin_q, cs_batch, 0, hk, hv, 0,
                           o, tickets, errw, part_ml, part_o, splits, B, HQ, H, K, M, Weff, scale, (cudaStream_t)stream, head,
                           ring_g, W, nopop, ring_k, nullptr, 0);
}

extern "C" int nha_ring_append_rot(void* ring_k, void* ring_kr, void* ring_v, void* ring_g, const void* k_new,
                                   const void* v_new, const void* g_new, const void* cos_q, const void* sin_q,
                                   int64_t cs_batch, int32_t* head, int B, int H, int K, int V, int M, int W, int fill,
                                   void* stream) {
  if (!ring_k || !ring_kr || !ring_v || !ring_g || !k_new || !v_new || !g_new || !cos_q || !sin_q || !head)
    return NHA_ERR_BAD_ARG;
  if (B <= 0 || H <= 0 || W < 1 || fill < 0 || fill > W || K % 16 || (H * V) % 8 || (H * M) % 8 || cs_batch % 8)
    return NHA_ERR_BAD_ARG;
  nha_ring_append_rot_kernel<<<B, 128, 0, (cudaStream_t)stream>>>((bf16*)ring_k, (bf16*)ring_kr, (bf16*)ring_v, (bf16*)ring_g,
                                                                  (const bf16*)k_new, (const bf16*)v_new, (const bf16*)g_new,
                                                                  (const bf16*)cos_q, (const bf16*)sin_q, cs_batch, head, H, K,
                                                                  V, M, W, fill);
  return check_launch();
}
