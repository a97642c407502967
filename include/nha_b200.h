/*
 * nha_b200 — C ABI of the B200 (sm_100a) implementation of the NHA attention operator.
 *
 * One shared library, plain pointers and sizes, no torch types.  Every entry
 * point returns an int status (NHA_OK == 0), never throws and never aborts;
 * nha_status_string() names a status.  All pointers are DEVICE pointers unless
 * stated otherwise; bf16 tensors are passed as `const void*`.  Entry points
 * allocate nothing: workspaces are sized by the *_workspace_bytes helpers and
 * passed in by the caller.  Launches go to the stream given (a cudaStream_t
 * passed as void*; NULL = the legacy default stream).
 *
 * Path names below are relative to the reference project (JusenD/NHA).
 *
 * Token layout: sequences are packed along the token axis, [Ttot, heads, dim]
 * row-major, delimited by cu_seqlens[N+1] (int32, device).  A batch of B
 * equal-length sequences [B, T, ...] is the same memory with N = B.
 * HQ query heads share H kv heads group-major (kv head = q head / (HQ/H)).
 */
#ifndef NHA_B200_H
#define NHA_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

enum {
  NHA_OK = 0,
  NHA_ERR_BAD_ARG = 1,       /* null pointer, negative size, HQ % H != 0 ... */
  NHA_ERR_UNSUPPORTED = 2,   /* head dim / slot count / window outside what the kernels cover */
  NHA_ERR_SMEM = 3,          /* tile set does not fit the 227 KB of shared memory */
  NHA_ERR_LAUNCH = 4,        /* cudaGetLastError() after a launch was not cudaSuccess */
  NHA_ERR_WORKSPACE = 5,     /* workspace pointer null or too small */
  NHA_ERR_STATIC_SCRATCH = 6 /* the call needs more scratch than the library's built-in array holds */
};

#define NHA_CHUNK 64         /* tokens per chunk of the chunked kernels */

const char* nha_status_string(int status);
/* Self test of the bounded waits.  Every wait of the tensor-core kernels on a completion barrier polls a limited
   number of times, then sets a device error word and carries on to the kernel's end instead of spinning.  This
   launches one small CTA that waits `polls` times (1 .. 65536) on a barrier that nothing ever completes and writes
   1 into *err_word (device int32, zeroed by the caller) when the wait runs out.  No counterpart in the reference. */
int nha_selftest_bounded_wait(int32_t* err_word, int polls, void* stream);
/* last CUDA error text seen by this library on the calling thread ("" if none) */
const char* nha_last_cuda_error(void);
int nha_abi_version(void);

/* ------------------------------------------------------------------------------------------
 * Fused decode step.  Replaces fused_recurrent_nha_decode
 * (nha_fla/ops/nha/fused_recurrent.py:431-584: the k-kernel :229-353 and v-kernel :356-428)
 * and, with `win_logits` given, fused_recurrent_nha (nha_fla/ops/nha/fused_recurrent.py:588-682).
 *
 *   q        [B, HQ, K] bf16   raw query (slot logits; rotated in-kernel when cos/sin given)
 *   sq       [B, HQ, K] bf16   pre-rotated query, or NULL
 *   k, v, g  [B, H, K|V|M] bf16  the token leaving the window (enters the slot memory)
 *   s        [B, H, M] bf16 or NULL (then s = 1 - exp(g) in fp32)
 *   sw_k     [B, W, H, K] bf16 window keys, time ascending (raw when cos/sin given), or NULL
 *   sw_v     [B, W, H, V] bf16 window values, or NULL
 *   cos, sin [1|B, W, K] bf16 rotate-half tables for the W window positions (row W-1 = query),
 *            row stride `cs_row`, batch stride `cs_batch` (0 = shared), or NULL
 *   win_logits [B, HQ, W] bf16 caller-computed window logits (fused_recurrent_nha mode), or NULL
 *   hk [B,H,K,M], hv [B,H,M,V] fp32: state, read as the initial state (or taken as zero when
 *            `zero_state` != 0) and OVERWRITTEN IN PLACE with the updated state
 *   o        [B, HQ, V] bf16   output (slot readout + window readout; slot readout only in
 *            win_logits mode)
 *   win_prob [B, HQ, W] fp32   window probabilities of the joint softmax, or NULL
 *   workspace  scratch of nha_decode_workspace_bytes(B, HQ, H, V, W) bytes, needed when W > 64
 *            (a (sequence, kv head) is then split over several CTAs whose partial softmaxes are
 *            merged by the last one to finish).  Its first B*H int32 are arrival counters, the next
 *            int32 is a device error word (nha_decode_device_error): they must be zero before the
 *            first call and every call leaves the counters zero, so one zero-initialised buffer can
 *            be reused by all calls with the same B*H that do not overlap on the GPU.  May be NULL
 *            for W <= 64.
 * K == V in {64, 128} with window keys takes a streaming kernel (ring of asynchronous copies, whole
 * grid resident in one wave; 2, 4 or 8 splits run as a thread-block cluster and merge through shared
 * memory without touching the workspace, which must be passed all the same); other shapes and the
 * win_logits mode take the general kernel.
 */
int64_t nha_decode_workspace_bytes(int B, int HQ, int H, int V, int W);
int nha_decode_step(const void* q, const void* sq, const void* k, const void* v, const void* g, const void* s,
                    const void* sw_k, const void* sw_v, const void* cos, const void* sin, int64_t cs_batch,
                    int64_t cs_row, const void* win_logits, float* hk, float* hv, int zero_state, void* o,
                    float* win_prob, void* workspace, int64_t workspace_bytes, int B, int HQ, int H, int K, int V,
                    int M, int W, float scale, void* stream);

/* nha_decode_step with the slot memory kept in bf16 (hk [B,H,K,M], hv [B,H,M,V] bf16, 16-byte aligned, updated in
 * place): half the state bytes per step.  Arithmetic stays fp32 in registers; the state is rounded once per step when
 * it is stored, and the step's own readout uses the rounded values, so a step sees exactly what the next one reads.
 * An extension: the reference keeps fp32 states (nha_fla/ops/nha/fused_recurrent.py:536-545), so results follow it
 * only to bf16 accuracy of the state.  Window-key mode with K == V in {64, 128} (streaming kernel) only;
 * NHA_ERR_UNSUPPORTED otherwise.  Arguments as nha_decode_step without win_logits / win_prob. */
int nha_decode_step_bf16_state(const void* q, const void* sq, const void* k, const void* v, const void* g, const void* s,
                               const void* sw_k, const void* sw_v, const void* cos, const void* sin, int64_t cs_batch,
                               int64_t cs_row, void* hk, void* hv, int zero_state, void* o, void* workspace,
                               int64_t workspace_bytes, int B, int HQ, int H, int K, int V, int M, int W, float scale,
                               void* stream);
/* Programmatic dependent launch of the streaming decode kernel (the reference chains its two decode kernels the same
 * way and switches it with the environment variable NHA_PDL, nha_fla/ops/nha/fused_recurrent.py:13-44, 560-582).
 *   0  plain launches.
 *   1  (default; NHA_PDL unset or "1") the kernel may be scheduled while the kernel in front of it on the stream is
 *      still draining and waits for that kernel before its first global read: always safe, hides the launch gap.
 *   2  as 1, and the slot memory (hk, hv) and the window (sw_k / sw_v, or the rings and head) of the call are
 *      requested BEFORE the wait; q, the popped or new token and the gates are read after it.  Only for callers who
 *      know that the kernel immediately in front on the stream writes neither this call's slot memory nor its window
 *      (a stack of layers with one cache per layer: the kernel in front works on another layer, or is a projection).
 * The mode is process-wide; NHA_PDL ("0", "1", "2") gives the initial value. */
int nha_decode_set_pdl(int mode);
int nha_decode_get_pdl(void);
/* reads the workspace's device error word (synchronises the stream): non-zero when a bounded wait
   inside the streaming decode kernel ran out.  No counterpart in the reference. */
int nha_decode_device_error(const void* workspace, int B, int H, void* stream);

/* Decode on a device-resident ring buffer (the rolling window of the reference's NHACache,
 * nha_fla/models/nha_cache.py:105-126, without its per-step torch.cat shift; pop and rope plumbing of the
 * callers: nha_fla/models/qwennha.py:149-176,207-218).  Per sequence the window keys, values and gate rows
 * live in rings `ring_k [B,W,H,K]`, `ring_v [B,W,H,V]`, `ring_g [B,W,H,M]` (bf16) of W physical rows; `head [B]`
 * (int32, device) is the row of the OLDEST entry.  `fill` is the number of entries the rings hold: W once they
 * are full (e.g. the last W tokens of the prefill); while a short prompt is still filling them, the entries sit
 * in rows 0 .. fill-1 in time order and head[b] stays 0.
 *   nha_decode_step_ring: one decode step.  The oldest entry (k, v, g = log decay, s = 1 - exp(g)) enters the
 *     slot memory; the window is the other W-1 entries followed by the token of this step (`k_new [B,H,K]`,
 *     `v_new [B,H,V]`, raw keys, not yet in the ring); cos/sin as for nha_decode_step (row w = logical window
 *     position, row W-1 = query).  hk, hv updated in place; `o [B,HQ,V]`.  K == V in {64, 128}; other shapes
 *     return NHA_ERR_UNSUPPORTED.  Rings and head are only read.  With fill < W nothing leaves the window and the
 *     slot memory keeps its value (the reference's callers pass an all-zero entry then, qwennha.py:152-160); the
 *     window is the `fill` entries and the new token, and cos/sin hold fill+1 rows (row fill = query).
 *   nha_ring_append: after the step, in stream order: the new token's rows (`g_new [B,H,M]` = its log decay)
 *     overwrite the oldest entry and head[b] advances by one (mod W); with fill < W they go to row `fill` and
 *     head is left alone (the caller passes fill+1 next time).
 * Both are plain launches on `stream`; once the rings are full they carry no host-side state, so a step can be
 * captured once and replayed. */
int nha_decode_step_ring(const void* q, const void* k_new, const void* v_new, const void* ring_k, const void* ring_v,
                         const void* ring_g, const int32_t* head, const void* cos, const void* sin, int64_t cs_batch,
                         int64_t cs_row, float* hk, float* hv, void* o, void* workspace, int64_t workspace_bytes, int B,
                         int HQ, int H, int K, int V, int M, int W, int fill, float scale, void* stream);
int nha_ring_append(void* ring_k, void* ring_v, void* ring_g, const void* k_new, const void* v_new, const void* g_new,
                    int32_t* head, int B, int H, int K, int V, int M, int W, int fill, void* stream);

/* nha_decode_step_ring and nha_ring_append in ONE launch.  `head [B*H]` holds one index per (sequence, kv head)
 * (all H entries of a sequence are equal between calls): the CTA that merges the splits of a (sequence, kv head) -
 * the last to touch it, after every split has read the rings - stores the step's token (k_new, v_new, g_new) over
 * the entry that left the window (fill == W) or into row `fill` of a ring that is still filling, and advances that
 * kv head's index.  Same results as the two separate calls; K == V in {64, 128} with the streaming kernel only
 * (NHA_ERR_UNSUPPORTED otherwise).  The reference shifts its window with three torch.cat per layer and token
 * (nha_fla/models/nha_cache.py:119-126). */
int nha_decode_step_ring_fused(const void* q, const void* k_new, const void* v_new, const void* g_new, void* ring_k,
                               void* ring_v, void* ring_g, int32_t* head, const void* cos, const void* sin,
                               int64_t cs_batch, int64_t cs_row, float* hk, float* hv, void* o, void* workspace,
                               int64_t workspace_bytes, int B, int HQ, int H, int K, int V, int M, int W, int fill,
                               float scale, void* stream);

/* Rings with keys rotated on entry (optional layout of the ring cache above).  Rotary by absolute position does
 * not change while the window slides, so a key is rotated once, when it enters the ring, and the decode step no
 * longer rotates (or reads tables for) the W-1 old window keys; the reference rotates the whole window at every
 * step (nha_fla/models/qwen3_moe_nha/qwennha.py:207-226).  `ring_k` keeps the raw keys (a token's raw key enters the
 * slot memory when it leaves the window), `ring_kr [B,W,H,K]` the rotated ones.  `cos_q, sin_q [1|B, K]` (bf16,
 * duplicated halves; `cs_batch` elements between sequences, 0 when shared) are the table row of the position of
 * this step's token.  Same results, bit for bit, as nha_decode_step_ring on raw keys with absolute-position tables.
 *   nha_ring_rotate_rows: fills rows 0 .. rows-1 of ring_kr from ring_k with table rows 0 .. rows-1 (after the
 *     prefill, rings in time order, head == 0).
 *   nha_decode_step_ring_rot / nha_ring_append_rot: as nha_decode_step_ring / nha_ring_append. */
int nha_ring_rotate_rows(const void* ring_k, void* ring_kr, const void* cos, const void* sin, int64_t cs_batch,
                         int64_t cs_row, int B, int H, int K, int W, int rows, void* stream);
int nha_decode_step_ring_rot(const void* q, const void* k_new, const void* v_new, const void* ring_k, const void* ring_kr,
                             const void* ring_v, const void* ring_g, const int32_t* head, const void* cos_q,
                             const void* sin_q, int64_t cs_batch, float* hk, float* hv, void* o, void* workspace,
                             int64_t workspace_bytes, int B, int HQ, int H, int K, int V, int M, int W, int fill,
                             float scale, void* stream);
int nha_ring_append_rot(void* ring_k, void* ring_kr, void* ring_v, void* ring_g, const void* k_new, const void* v_new,
                        const void* g_new, const void* cos_q, const void* sin_q, int64_t cs_batch, int32_t* head, int B,
                        int H, int K, int V, int M, int W, int fill, void* stream);

/* ------------------------------------------------------------------------------------------
 * Chunked prefill / training.  One descriptor serves the state pass, the output pass and the
 * backward.  Replaces chunk_nha (nha_fla/ops/nha/chunk.py:568-690; autograd node :352-564,
 * GSA half nha_fla/ops/nha/chunk_gsa.py:16-122, third-party flash-attn varlen fwd/bwd call
 * sites chunk.py:241-270,333-344) and fused_chunk_nha_prefill
 * (nha_fla/ops/nha/chunk_fused.py:291-380: state kernel :31-114, output kernel :117-283).
 */
typedef struct nha_chunk_desc {
  /* inputs, bf16 */
  const void* q_gsa;            /* [Ttot, HQ, K] un-rotated query (slot logits) */
  const void* q_swa;            /* [Ttot, HQ, K] rotated query (window logits) */
  const void* k_gsa;            /* [Ttot, H, K]  un-rotated key (slot memory) */
  const void* k_swa;            /* [Ttot, H, K]  rotated key (window) */
  const void* v;                /* [Ttot, H, V] */
  const void* s;                /* [Ttot, H, M]  slot write weights */
  const void* g;                /* [Ttot, H, M]  log forget gates (<= 0) */
  const int32_t* cu_seqlens;    /* [N+1] */
  const int32_t* window_left;   /* [N] per-sequence window (keys t-wl..t; <0 = unbounded) or NULL */
  const int32_t* shift;         /* [N] per-sequence gsa_kv_shift or NULL */
  const float* hk0;             /* [N, H, K, M] or NULL (zero) */
  const float* hv0;             /* [N, H, M, V] or NULL (zero) */
  /* forward outputs */
  void* o;                      /* [Ttot, HQ, V] bf16 */
  float* lse_swa;               /* [Ttot, HQ] */
  float* lse_gsa;               /* [Ttot, HQ] */
  float* hkt;                   /* [N, H, K, M] or NULL */
  float* hvt;                   /* [N, H, M, V] or NULL */
  /* chunk-start states written by the state pass, read by the output pass and the backward */
  void* hk_chunks;              /* [NC, H, K, M] bf16 */
  void* hv_chunks;              /* [NC, H, M, V] bf16 */
  /* plan (int32 workspace of nha_chunk_plan_ints(Ttot, N, H) entries, written by nha_chunk_plan):
     [0..N] first chunk of each sequence, [N+1 .. N+1+NC) the sequence of each chunk, then NC*H
     per-(chunk, head) flags and a device error word used by the output pass, then (at the next
     multiple of four ints) one record {sequence, chunk in sequence, first token, length} per chunk;
     NC = nha_chunk_count_bound(Ttot, N).  The buffer must be 16-byte aligned. */
  int32_t* plan;
  void* workspace;              /* scratch, see nha_chunk_*_workspace_bytes */
  size_t workspace_bytes;
  /* backward inputs */
  const void* d_o;              /* [Ttot, HQ, V] bf16 */
  const float* d_lse_gsa;       /* [Ttot, HQ] or NULL */
  const float* d_hkt;           /* [N, H, K, M] or NULL */
  const float* d_hvt;           /* [N, H, M, V] or NULL (both or neither) */
  /* backward outputs, bf16 like the inputs */
  void* dq_gsa; void* dq_swa; void* dk_gsa; void* dk_swa; void* dv; void* ds; void* dg;
  float* dhk0;                  /* [N, H, K, M] or NULL */
  float* dhv0;                  /* [N, H, M, V] or NULL */
  /* sizes */
  int32_t Ttot, N, HQ, H, K, V, M;
  int32_t max_seqlen;           /* longest sequence (grid sizing of the state pass) */
  int32_t window_left_all;      /* used when window_left == NULL */
  int32_t shift_all;            /* used when shift == NULL */
  int32_t q_offset;             /* 0, or (forward only, N == 1, a multiple of 64): q_gsa, q_swa, o, lse_swa and lse_gsa hold
                                   only the positions >= q_offset of the sequence (row i = position q_offset + i), while the
                                   kv-head tensors hold all Ttot positions.  The state pass covers every position; the output
                                   pass skips the chunks below q_offset.  Used by the sequence-parallel prefill, whose ranks
                                   prepend the last window of the rank before them to their kv-head tensors only.  Honoured by
                                   the pipelined output pass (K == V == 128, M == 64, even HQ / H); other shapes return
                                   NHA_ERR_UNSUPPORTED */
  float scale;
} nha_chunk_desc;

/* sizeof(nha_chunk_desc) as compiled into the library, for bindings that mirror the struct */
int64_t nha_chunk_desc_size(void);
/* upper bound of the number of chunks of N packed sequences holding Ttot tokens */
int64_t nha_chunk_count_bound(int64_t Ttot, int64_t N);
/* number of int32 of desc->plan */
int64_t nha_chunk_plan_ints(int64_t Ttot, int64_t N, int64_t H);
/* bytes of desc->workspace for the forward (state pass + output pass) / the backward */
int64_t nha_chunk_fwd_workspace_bytes(const nha_chunk_desc* d);
int64_t nha_chunk_bwd_workspace_bytes(const nha_chunk_desc* d);

/* fills desc->plan from cu_seqlens on the device (no host synchronisation) */
int nha_chunk_plan(const nha_chunk_desc* d, void* stream);
/* state pass: chunk-start states hk_chunks/hv_chunks (+ final states hkt/hvt when non-NULL) */
int nha_chunk_state_pass(const nha_chunk_desc* d, void* stream);
/* The two halves of nha_chunk_state_pass, for callers that have part of their inputs early (the sequence-parallel
   prefill starts on the chunks that read only its own rows while the rows of the rank before it are still on the wire):
   nha_chunk_state_terms computes the per-chunk terms of the chunks [chunk_lo, chunk_lo + chunk_n) into desc->workspace
   (chunk c reads the rows [64 c - shift, 64 c + 64 - shift) of its sequence's k_gsa, v, s, g); nha_chunk_state_scan,
   once every chunk's terms are there, writes hk_chunks / hv_chunks and hkt / hvt.  Same workspace and plan as
   nha_chunk_state_pass, which is terms over all chunks followed by the scan. */
int nha_chunk_state_terms(const nha_chunk_desc* d, int chunk_lo, int chunk_n, void* stream);
int nha_chunk_state_scan(const nha_chunk_desc* d, void* stream);
/* Adds a start state to the result of a state pass that ran from a ZERO start (hk0 == hv0 == NULL) with this
   descriptor: the recurrence is linear, so the state at the start of chunk c is the zero-start state plus
   S .* exp(sum of the log gates of the chunks before c).  sk [N,H,K,M], sv [N,H,M,V] fp32.  Updates hk_chunks,
   hv_chunks (bf16, rounded again) and, when non-NULL, hkt / hvt.  Reads the per-chunk gate totals the state pass left
   in desc->workspace, so it must follow that state pass directly (same descriptor, same stream order).  This is what
   lets a rank of the sequence-parallel prefill run ONE state pass: it summarises its segment from a zero start, the
   ranks exchange the summaries, and the true start state is folded in afterwards.  The reference's resumption
   contract is initial_state (nha_fla/ops/nha/chunk_fused.py:337-342); it has no counterpart of this call. */
int nha_chunk_apply_state_prefix(const nha_chunk_desc* d, const float* sk, const float* sv, void* stream);
/* *out = device pointer (inside desc->workspace) of the log gates of every sequence summed over its chunks,
   [N, H, M] fp32, as left by the last state pass run with this descriptor: the total decay of the tokens that entered
   the slot memory, the second half of a segment's summary in the sequence-parallel prefill. */
int nha_chunk_gate_totals(const nha_chunk_desc* d, const float** out);
/* Start state of rank `rank` of a sequence-parallel prefill of ONE sequence from the all-gathered summaries
   allp [world][H*K*M + H*M*V + H*M] fp32 (zero-start end states L_k [H,K,M], L_v [H,M,V] and log gate totals G [H,M] of
   every rank's segment):  S = S0 .* exp(sum_{r<rank} G_r) + sum_{r<rank} L_r .* exp(sum_{r<r'<rank} G_r').
   hk0 / hv0: start state of the whole sequence or NULL (both).  One launch.  No counterpart in the reference, which has
   no distributed code. */
int nha_sp_fold_start_state(const float* allp, int world, int rank, int H, int K, int M, int V, const float* hk0,
                            const float* hv0, float* sk, float* sv, void* stream);

/* The same exchange without a collective library: summaries travel over peer memory (NVLink) and the fold waits for
 * exactly the ranks it consumes.  Symmetric mailboxes, allocated by the caller so that every rank can address every
 * other rank's copy: box float [depth][world][P] and flag uint32 [depth][world] (zero before the first call) on every
 * rank, P = H*K*M + H*M*V + H*M; box_ptrs / flag_ptrs: DEVICE arrays of `world` pointers to the ranks' copies;
 * ctr: two zero-initialised uint32 in this rank's own memory; depth >= world + 1.
 *   nha_sp_publish: stores this rank's summary `pack [P]` into the mailboxes of the ranks after it and raises their
 *     flags; advances ctr[0].  Every rank calls it once per prefill, the last rank too.
 *   nha_sp_fold_wait: after nha_sp_publish on the same stream; waits (bounded: about a second, then *err_word = 1 and
 *     the outputs are invalid) for the summaries of the ranks before this one in this rank's own mailbox
 *     (box, flag: this rank's copies) and writes the start state sk [1,H,K,M], sv [1,H,M,V] like
 *     nha_sp_fold_start_state.  Both launches may be captured in a CUDA graph. */
int nha_sp_publish(const float* pack, int64_t P, float* const* box_ptrs, uint32_t* const* flag_ptrs, uint32_t* ctr, int world,
                   int rank, int depth, void* stream);
int nha_sp_fold_wait(const float* box, const uint32_t* flag, const uint32_t* ctr, int world, int rank, int depth, int H, int K,
                     int M, int V, const float* hk0, const float* hv0, float* sk, float* sv, int* err_word, void* stream);

/* The halo of the sequence-parallel prefill over peer memory (instead of a send / receive pair of a collective library):
 * a rank stores the last rows of its kv-head tensors straight into the first rows of the next rank's halo-extended
 * tensors, which therefore live in buffers that the sender can address (symmetric allocations).
 *   nha_sp_halo_push (sender): waits (bounded) until the receiver has acknowledged the halo before this one
 *     (ack_local, a word in this rank's memory written by the receiver), copies `count` (<= 5) byte ranges src[i] ->
 *     dst_peer[i] (host arrays of device pointers; 16-byte aligned, sizes multiples of 16) and raises the receiver's
 *     flag (flag_peer).  ctr: two zero-initialised uint32 of this rank (halos pushed, ticket).
 *   nha_sp_halo_wait (receiver): before the first kernel that reads the halo rows; waits (bounded) for its flag
 *     (flag_local).  ctr: one zero-initialised uint32 of this rank (halos received).
 *   nha_sp_halo_ack (receiver): after the last kernel that reads the halo rows; writes the count of halos received into
 *     the sender's ack word (ack_peer).
 * A wait that runs out (about a second) sets *err_word and the kernel returns.  All three may be captured in a graph. */
int nha_sp_halo_push(const void* const* src, void* const* dst_peer, const int64_t* bytes, int count, uint32_t* flag_peer,
                     const uint32_t* ack_local, uint32_t* ctr, int* err_word, void* stream);
int nha_sp_halo_wait(const uint32_t* flag_local, uint32_t* ctr, int* err_word, void* stream);
int nha_sp_halo_ack(uint32_t* ack_peer, const uint32_t* ctr, void* stream);
/* output pass: o, lse_swa, lse_gsa from the inputs and the chunk-start states */
int nha_chunk_output_pass(const nha_chunk_desc* d, void* stream);
/* device-side error word of the last output pass run with this descriptor's plan (0 = none; non-zero:
   a bounded wait on a tensor-core completion barrier ran out and the affected chunks are invalid);
   synchronises the stream.  No counterpart in the reference. */
int nha_chunk_device_error(const nha_chunk_desc* d, void* stream);
/* plan + state pass + output pass */
int nha_chunk_fwd(const nha_chunk_desc* d, void* stream);
/* backward: needs the forward's o, lse_swa, lse_gsa, hk_chunks, hv_chunks, plan (and hkt/hvt
   when d_hkt/d_hvt are given); writes dq_*, dk_*, dv, ds, dg (+ dhk0/dhv0 when non-NULL) */
int nha_chunk_bwd(const nha_chunk_desc* d, void* stream);

/* State pass for callers that cannot allocate device memory (a plugin host that passes only
   input and output buffers, a serving loop that forbids allocation after start-up).  Same
   inputs, outputs and results as nha_chunk_state_pass, but desc->workspace is ignored: the
   per-chunk scratch comes from a fixed array inside the library's device image
   (nha_chunk_state_pass_static_max_bytes() bytes, 16 MiB, held on every GPU that loads the
   library until the process exits).  The call itself allocates nothing.  A problem whose
   scratch (nha_chunk_count_bound(Ttot, N)*H*((K*M+M*V)*2 + M*4) + 256 bytes, = nha_chunk_fwd_workspace_bytes)
   exceeds the array is refused with NHA_ERR_STATIC_SCRATCH and nothing is launched.  The first
   call on each device looks up the array's device address (cudaGetSymbolAddress, with that
   device current); make that first call before any stream capture begins.  All calls on a
   device share the one array: calls that overlap on the GPU (different streams) race; calls
   in stream order do not, and no call depends on what an earlier call left in the array.
   No counterpart in the reference (its ops allocate through torch). */
int64_t nha_chunk_state_pass_static_max_bytes(void);
int nha_chunk_state_pass_static(const nha_chunk_desc* d, void* stream);

/* one stage of nha_chunk_bwd on its own, so a harness can time each part with events on the
   launching stream: 0 = query-row side (delta, joint LSE, dq_gsa, dq_swa, gate terms, bf16 copies of
   dz and p, the chunks' own state-gradient terms), 1 = key side of the window (dk_swa, window part
   of dv), 2 = general slot kernel (chunks flagged by the forward only), 3 = scan of the state
   gradients over the chunks (dhk0/dhv0), 4 = gate carry and key-row side of the slot branch
   (dk_gsa, dv, ds, dg).  The stages of one backward must run in this order; running all five
   equals nha_chunk_bwd.  No counterpart in the reference (it has no timing hooks). */
int nha_chunk_bwd_stage(const nha_chunk_desc* d, int stage, void* stream);

/* ------------------------------------------------------------------------------------------
 * Slot gates of the callers, fused.  The layers turn the gate projection f [.., H, M] into the
 * operator's two gate inputs with a chain of element-wise torch kernels
 * (nha_fla/layers/nha.py:229-231; hybrid models nha_fla/models/qwen3_nha/qwennha.py:116):
 *     g = logsigmoid(f) / normalizer,   s = 1 - exp(g).
 *   nha_slot_gates_fwd: f, g, s bf16 with n elements each (any shape, contiguous, 16-byte aligned);
 *     s may be NULL.  s is computed from the bf16-rounded g, as the reference does.
 *   nha_slot_gates_bwd: df = (dg - ds * exp(g)) * sigmoid(-f) / normalizer; dg or ds may be NULL.
 * One launch each on `stream`, no workspace. */
int nha_slot_gates_fwd(const void* f, void* g, void* s, int64_t n, float normalizer, void* stream);
int nha_slot_gates_bwd(const void* f, const void* dg, const void* ds, void* df, int64_t n, float normalizer,
                       void* stream);

/* ------------------------------------------------------------------------------------------
 * Rotary embedding of the callers' queries and keys, both tensors in one launch (the layer's
 * RotaryEmbedding call, nha_fla/layers/nha.py:145,235: non-interleaved halves, positions restart
 * at every packed sequence; the hybrid models' rotate-half on duplicated-halves tables,
 * nha_fla/models/qwen3_nha/qwennha.py:240-244, is the same arithmetic on the first K/2 columns).
 *   q [Ttot,HQ,K], k [Ttot,H,K] (k and k_out may be NULL), outputs of the same shape (may alias
 *   the inputs), bf16.  cos, sin: bf16 tables of `table_rows` rows, `cs_row` elements apart, of
 *   which the first K/2 columns are read; row = offset + position of the token in its sequence.
 *   Sequences: cu_seqlens [N+1] (device) or, when NULL, Ttot / T sequences of T tokens each.
 *   The caller guarantees offset + longest sequence <= table_rows.  inverse != 0 rotates by the
 *   opposite angle (the backward).  K % 16 == 0, cs_row % 8 == 0, 16-byte aligned pointers. */
int nha_rope_pair(const void* q, const void* k, void* q_out, void* k_out, const void* cos, const void* sin,
                  int64_t cs_row, int table_rows, const int32_t* cu_seqlens, int N, int T, int64_t Ttot, int HQ,
                  int H, int K, int offset, int inverse, void* stream);

/* ------------------------------------------------------------------------------------------
 * Feature map and value activation of the calling layer, up to three tensors in one launch
 * (nha_fla/layers/nha.py:219-223: q_gsa = feature_map(q), k_gsa = feature_map(k), v = silu(v); the 'swish'
 * feature map of flash-linear-attention is x * sigmoid(x), the same function as silu; 'relu' is max(x, 0)).
 *   x, y (dx), dy: host arrays of `count` (1..3) device pointers, bf16, n[i] elements each, contiguous,
 *   16-byte aligned; relu[i] != 0 selects max(x, 0) for tensor i (NULL: all swish).  y may alias x.
 *   nha_act3_bwd: dx = dy * act'(x). */
int nha_act3_fwd(const void* const* x, void* const* y, const int64_t* n, const int* relu, int count, void* stream);
int nha_act3_bwd(const void* const* x, const void* const* dy, void* const* dx, const int64_t* n, const int* relu,
                 int count, void* stream);

/* ------------------------------------------------------------------------------------------
 * Output side of the calling layer: the normalisation in front of the output projection
 * (nha_fla/layers/nha.py:277-278, o = rms_norm_linear(silu(o), g_norm.weight, g_norm.bias, o_proj.weight,
 * o_proj.bias); flash-linear-attention's rms_norm_linear is RMS norm + affine, then F.linear).
 *   nha_silu_rmsnorm_fwd: y = silu(o) * rstd * weight + bias with rstd = rsqrt(mean(silu(o)^2) + eps) per row;
 *     o, y bf16 [rows, cols]; weight, bias (may be NULL) fp32 [cols]; rstd fp32 [rows] (may be NULL; needed by
 *     the backward).  cols a multiple of 256, at most 2048 (NHA_ERR_UNSUPPORTED otherwise).
 *   nha_silu_rmsnorm_bwd: d_o from dy (gradient of y); part_w, part_b (may be NULL) fp32
 *     [nha_silu_rmsnorm_bwd_ctas(rows), cols]: per-CTA partial sums of the weight and bias gradients, to be
 *     summed over their first axis by the caller.
 * The projection itself is a plain GEMM and stays with the GEMM library. */
int nha_silu_rmsnorm_fwd(const void* o, const float* weight, const float* bias, void* y, float* rstd, int64_t rows,
                         int cols, float eps, void* stream);
int nha_silu_rmsnorm_bwd_ctas(int64_t rows);
int nha_silu_rmsnorm_bwd(const void* o, const float* weight, const float* rstd, const void* dy, void* d_o,
                         float* part_w, float* part_b, int64_t rows, int cols, void* stream);

/* ------------------------------------------------------------------------------------------
 * Layer-side consumers of lse_swa / lse_gsa, fused (the training layer's aux loss and compression
 * statistic, nha_fla/layers/nha.py:255-264, 288-323): with delta = lse_gsa - lse_swa over n = T*HQ
 * elements (fp32),
 *     out[0] = mean(binary_cross_entropy_with_logits(delta, target)),   out[1] = mean(sigmoid(delta))
 * (the latter is the reference's gsa_ratio = mean(w_gsa / (w_swa + w_gsa))).  Results stay on the device.
 *   nha_lse_stats: one launch; `scratch` of nha_lse_stats_scratch_bytes() bytes, zeroed ONCE by the caller
 *     before its first use (the kernel leaves it ready for the next call; calls sharing a scratch must be
 *     in stream order).  The sum order is fixed: equal inputs give equal bits.
 *   nha_lse_aux_grad: d_lse_gsa[i] = dloss[0] * (sigmoid(delta_i) - target) / n, the gradient the layer's
 *     autograd sends into the operator (lse_swa is detached there, :303). */
int64_t nha_lse_stats_scratch_bytes(void);
int nha_lse_stats(const float* lse_swa, const float* lse_gsa, int64_t n, float target, float* out, void* scratch,
                  void* stream);
int nha_lse_aux_grad(const float* lse_swa, const float* lse_gsa, const float* dloss, int64_t n, float target,
                     float* d_lse_gsa, void* stream);

#ifdef __cplusplus
}
#endif
#endif /* NHA_B200_H */
