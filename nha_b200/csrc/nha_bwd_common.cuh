// Declarations shared by the backward kernels of the chunked NHA operator: the scratch layout and the
// per-chunk context.
#pragma once

#include "nha_common.cuh"

namespace nha {

struct BwdWs {
  float* delta;   // [Ttot, HQ]      <do, o>
  float* lj;      // [Ttot, HQ]      joint log-sum-exp
  float* dvacc;   // [Ttot, H, V]    window part of dv
  float* dkp;     // [Ttot, H, K]    intra-chunk part of dk' (row = shifted position)
  float* dvp;     // [Ttot, H, V]    intra-chunk part of dv'
  float* dsp;     // [Ttot, H, M]    intra-chunk part of ds'
  float* dga;     // [Ttot, H, M]    ok .* dz + p .* dp summed over the group
  bf16* dzg;      // [Ttot, HQ, M]   scale * dz_slot .* exp(G)   (general kernels; the tensor-memory rows pass keeps it on chip)
  bf16* pgq;      // [Ttot, HQ, M]   p_slot .* exp(G)            (general kernels, and the two-heads-per-tile rows pass)
  float* dkc;     // [NC, H, K, M]   first the chunk's own term q^T (scale dz exp G), then (after the scan)
                  //                 the gradient of hk at the END of the chunk
  float* dvc;     // [NC, H, M, V]   likewise (p exp G)^T do, then the gradient of hv at the chunk end
  float* gend;    // [NC, H, M]      total shifted log gate of each chunk
  bf16* dza;      // [Ttot, HQ, M]   scale * dz_slot .* a   (tensor-memory path only)
  bf16* paq;      // [Ttot, HQ, M]   p_slot .* a            (tensor-memory path only)
  bf16* dkb;      // [NC, H, K, M]   bf16 copy of the scanned dkc (tensor-memory path only)
  bf16* dvb;      // [NC, H, M, V]   bf16 copy of the scanned dvc
  float* gcarry;  // [NC, H, M]      gate-gradient carry of all later chunks
  const int* flags;   // [NC, H] chunks the tensor-memory forward left to the general kernels, or NULL
  int gate;           // 0: a kernel handles every chunk; 1: only flagged chunks; 2: only unflagged chunks
};

__host__ inline int64_t bwd_ws_layout(const nha_chunk_desc* d, BwdWs* w, void* base) {
  int64_t off = 0;
  auto take = [&](int64_t bytes) { int64_t o = off; off = (off + bytes + 255) & ~(int64_t)255; return o; };
  const int64_t T = d->Ttot;
  const int64_t o_delta = take(T * d->HQ * 4), o_lj = take(T * d->HQ * 4), o_dvacc = take(T * d->H * d->V * 4);
  const int64_t o_dkp = take(T * d->H * d->K * 4), o_dvp = take(T * d->H * d->V * 4);
  const int64_t o_dsp = take(T * d->H * d->M * 4), o_dga = take(T * d->H * d->M * 4);
  const int64_t o_dzg = take(T * d->HQ * d->M * 2), o_pgq = take(T * d->HQ * d->M * 2);
  const int64_t NC = nha_chunk_count_bound(d->Ttot, d->N);
  const int64_t o_dkc = take(NC * d->H * d->K * d->M * 4), o_dvc = take(NC * d->H * d->M * d->V * 4);
  const int64_t o_dza = take(T * d->HQ * d->M * 2), o_paq = take(T * d->HQ * d->M * 2);
  const int64_t o_gend = take(NC * d->H * d->M * 4);
  const int64_t o_dkb = take(NC * d->H * d->K * d->M * 2), o_dvb = take(NC * d->H * d->M * d->V * 2);
  const int64_t o_gcarry = take(NC * d->H * d->M * 4);
  if (w && base) {
    char* b = (char*)base;
    w->delta = (float*)(b + o_delta); w->lj = (float*)(b + o_lj); w->dvacc = (float*)(b + o_dvacc);
    w->dkp = (float*)(b + o_dkp); w->dvp = (float*)(b + o_dvp); w->dsp = (float*)(b + o_dsp);
    w->dga = (float*)(b + o_dga); w->dzg = (bf16*)(b + o_dzg); w->pgq = (bf16*)(b + o_pgq);
    w->dkc = (float*)(b + o_dkc); w->dvc = (float*)(b + o_dvc);
    w->dza = (bf16*)(b + o_dza); w->paq = (bf16*)(b + o_paq);
    w->gend = (float*)(b + o_gend);
    w->dkb = (bf16*)(b + o_dkb); w->dvb = (bf16*)(b + o_dvb); w->gcarry = (float*)(b + o_gcarry);
    w->flags = nullptr; w->gate = 0;
  }
  return off;
}

struct ChunkCtx {
  int n, ci, t0, len, c0, wl, shift;
};

// does a kernel launched with gating `w.gate` handle chunk (cg, h)?
__device__ __forceinline__ bool chunk_gate(const BwdWs& w, int cg, int h, int H) {
  if (w.gate == 0 || w.flags == nullptr) return true;
  const int f = w.flags[(size_t)cg * H + h];
  return w.gate == 1 ? f != 0 : f == 0;
}

__device__ __forceinline__ bool chunk_ctx(const nha_chunk_desc& d, int cg, ChunkCtx& c) {
  const ChunkRec rc = chunk_rec(d, cg);
  c.n = rc.n;
  if (c.n < 0) return false;
  c.ci = rc.ci;
  c.t0 = rc.t0;
  c.len = rc.len;
  c.c0 = c.ci * kChunk;
  c.wl = seq_window(d, c.n);
  c.shift = seq_shift(d, c.n);
  return true;
}


}  // namespace nha
