"""Multi-GPU use of the NHA ops: one process per GPU, ``torch.distributed`` for the plumbing.

Two modes, following how the operator shards:

* Batch / head sharding needs no code here: sequences and kv heads are independent, so every rank
  simply calls the ops on its own rows (no collective).
* Sequence-parallel prefill (one long sequence cut into contiguous segments, rank r owning tokens
  ``[r*T/P, (r+1)*T/P)``) has exactly one exchange step, implemented by
  :func:`sequence_parallel_prefill`:

    1. every rank summarises its own tokens from a zero start, in two parts (all but the last ``W``
       tokens, and the last ``W``): the slot memory ``L`` they would leave and their total log decay
       ``G`` - the recurrence is linear, so ``S_after = S_before * exp(G) + L``;
    2. halo: rank r receives from rank r-1 the last ``W`` tokens of ``k, rotary_k, v, s, g`` (the
       keys/values its first ``W`` queries still see, and the tokens that enter the slot memory during
       them because of the shift by ``W``) - one point-to-point message - and one all-gather of the
       summaries;
    3. every rank folds the parts before it: the state before its first token, and the state ``W``
       tokens earlier;
    4. the rank's forward runs on its own tensors (no copy of the segment) from the state before its
       first token, fully parallel with the other ranks; its first ``W`` rows, which need the halo, are
       recomputed by a second, small forward over the ``2W`` tokens around the boundary.

  The reference has no distributed code at all (its long-context story is the O(1) state plus
  ``initial_state`` resumption, nha_fla/ops/nha/chunk_fused.py:337-342); the single-device op is the
  oracle for this function.

The arithmetic is injected (``local_state`` / ``forward``) so the host logic can be exercised on CPU
ranks with the ``gloo`` backend; the defaults are the CUDA ops of this package.
"""
from __future__ import annotations

from typing import Callable, Optional, Tuple

import torch
import torch.distributed as dist


def _cuda_local_state(k, v, s, g, W):
    from .chunk import chunk_final_state
    B, T = k.shape[0], k.shape[1]
    flat = lambda x: x.reshape(B * T, *x.shape[2:]).to(torch.bfloat16).contiguous()
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=k.device)
    return chunk_final_state(flat(k), flat(v), flat(s), flat(g), cu, T, W)


def _cuda_forward(q, k, v, rq, rk, s, g, W, scale, state):
    from .chunk_fused import fused_chunk_nha_prefill
    o, (hk, hv) = fused_chunk_nha_prefill(q=q, k=k, v=v, rotary_q=rq, rotary_k=rk, s=s, g=g, window_size=W,
                                          initial_state=state, output_final_state=True, scale=scale)
    return o, hk, hv


def sequence_parallel_prefill(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rotary_q: torch.Tensor, rotary_k: torch.Tensor,
    s: torch.Tensor, g: torch.Tensor, window_size: int,
    initial_state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    scale: Optional[float] = None,
    group: Optional[dist.ProcessGroup] = None,
    local_state: Callable = _cuda_local_state,
    forward: Callable = _cuda_forward,
):
    """``fused_chunk_nha_prefill`` over a sequence sharded along tokens.

    Every rank passes ITS segment: ``q, rotary_q [B,Tr,HQ,K]``, ``k, rotary_k [B,Tr,H,K]``,
    ``v [B,Tr,H,V]``, ``s, g [B,Tr,H,M]`` (segments in rank order, each at least ``window_size``
    tokens long), plus on every rank the same ``initial_state`` of the whole sequence (or None).
    Returns ``(o [B,Tr,HQ,V], (hk, hv))`` where the state is the slot memory at the END of this
    rank's segment (the last rank holds the final state of the sequence).
    """
    W = int(window_size)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, Tr = k.shape[0], k.shape[1]
    assert Tr >= W, f'every segment must hold at least window_size={W} tokens, got {Tr}'
    if scale is None:
        scale = q.shape[-1] ** -0.5
    dev = k.device

    H, K, M, V = k.shape[2], k.shape[3], s.shape[3], v.shape[3]
    nk, nv = H * K * M, H * M * V

    # ---- 1. summaries of this rank's own tokens from a zero start, in two parts: A = all but the last W tokens,
    #         B = the last W.  They need nothing from another rank.  `local_state` absorbs all but the last W
    #         tokens of what it is given, so B is followed by W tokens of padding. -----------------------------------
    LkA, LvA = local_state(k, v, s, g, W)
    tail = lambda x: torch.cat([x[:, Tr - W:], torch.zeros_like(x[:, :W])], 1)
    LkB, LvB = local_state(tail(k), tail(v), tail(s), tail(g), W)
    GA = g[:, :Tr - W].sum(1, dtype=torch.float32)                         # [B,H,M] total log decay of each part
    GB = g[:, Tr - W:].sum(1, dtype=torch.float32)
    part = lambda lk, lv, G: torch.cat([lk.reshape(B, -1).float(), lv.reshape(B, -1).float(), G.reshape(B, -1)], 1)
    pack = torch.stack([part(LkA, LvA, GA), part(LkB, LvB, GB)]).contiguous()   # [2, B, nk + nv + H*M]

    # ---- 2. the exchange: halo of W tokens from the left neighbour (kv-head tensors only) and the all-gather of
    #         the summaries ---------------------------------------------------------------------------------------
    send = [x[:, Tr - W:].contiguous() for x in (k, rotary_k, v, s, g)]
    recv = [torch.empty_like(x) for x in send]
    ops = []
    if rank + 1 < world:
        ops += [dist.P2POp(dist.isend, x, dist.get_global_rank(group, rank + 1) if group else rank + 1, group) for x in send]
    if rank > 0:
        ops += [dist.P2POp(dist.irecv, x, dist.get_global_rank(group, rank - 1) if group else rank - 1, group) for x in recv]
    works = dist.batch_isend_irecv(ops) if ops else []
    allp = [torch.empty_like(pack) for _ in range(world)]
    dist.all_gather(allp, pack, group=group)
    for w in works:
        w.wait()

    # ---- 3. fold the parts before this rank: the recurrence is linear, S_after = S_before * exp(G) + L.  Parts in
    #         time order are A_0, B_0, A_1, B_1, ...; the state before this rank's first token has absorbed the first
    #         2*rank of them, the state W tokens earlier one part less. ------------------------------------------------
    if initial_state is not None and initial_state != (None, None):
        S0k, S0v = initial_state[0].float(), initial_state[1].float()
    else:
        S0k = torch.zeros(B, H, K, M, dtype=torch.float32, device=dev)
        S0v = torch.zeros(B, H, M, V, dtype=torch.float32, device=dev)

    def fold(n):
        if n == 0:
            return S0k.clone(), S0v.clone()
        P = torch.cat(allp[:(n + 1) // 2])[:n]                             # [n, B, nk + nv + H*M], time order
        Gs = P[:, :, nk + nv:].reshape(n, B, H, M)
        after = Gs.flip(0).cumsum(0).flip(0) - Gs                          # total log decay of the parts after each
        wgt, tot = after.exp(), Gs.sum(0).exp()
        Sk = S0k * tot[:, :, None, :] + (P[:, :, :nk].reshape(n, B, H, K, M) * wgt[:, :, :, None, :]).sum(0)
        Sv = S0v * tot[:, :, :, None] + (P[:, :, nk:nk + nv].reshape(n, B, H, M, V) * wgt[:, :, :, :, None]).sum(0)
        return Sk, Sv

    # ---- 4. the rank's own tokens from the state before its first token: no copies of the segment.  Rows >= W are
    #         final; the first W rows lack the neighbour's keys and are recomputed below. ------------------------------
    o, hk, hv = forward(q, k, v, rotary_q, rotary_k, s, g, W, scale, fold(2 * rank))
    if rank > 0:
        # ---- 5. the first W rows: the 2W tokens around the boundary (halo + own first W), queries of the halo
        #         rows zero, from the state W tokens before the boundary ------------------------------------------------
        hk_, hrk, hv_, hs, hg = recv
        zq = q.new_zeros(B, W, *q.shape[2:])
        head = lambda h, x: torch.cat([h, x[:, :W]], 1)
        oh, _, _ = forward(head(zq, q), head(hk_, k), head(hv_, v), head(zq, rotary_q), head(hrk, rotary_k), head(hs, s),
                           head(hg, g), W, scale, fold(2 * rank - 1))
        o[:, :W] = oh[:, W:]
    return o, (hk, hv)
