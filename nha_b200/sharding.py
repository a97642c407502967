"""Multi-GPU use of the NHA ops: one process per GPU, ``torch.distributed`` for the plumbing.

Two modes, following how the operator shards:

* Batch / head sharding needs no code here: sequences and kv heads are independent, so every rank
  simply calls the ops on its own rows (no collective).
* Sequence-parallel prefill (one long sequence cut into contiguous segments, rank r owning tokens
  ``[r*T/P, (r+1)*T/P)``) has exactly one exchange step, implemented by
  :func:`sequence_parallel_prefill`:

    1. halo: rank r receives from rank r-1 the last ``W`` tokens of ``k, rotary_k, v, s, g`` (the
       keys/values its first queries still see, and the tokens that enter its slot memory late
       because of the shift by ``W``) - one point-to-point message;
    2. every rank summarises its segment: the slot memory it would end with from a zero start,
       ``L_r``, and the total log decay ``G_r`` of the tokens that enter - the recurrence is linear,
       so ``S_start(r+1) = S_start(r) * exp(G_r) + L_r``;
    3. one all-gather of ``(L_r, G_r)``; every rank folds the ranks before it;
    4. the rank's forward runs from its true start state, fully parallel with the other ranks.

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

    # ---- 1. halo of W tokens from the left neighbour (kv-head tensors only) ---------------------------
    send = [x[:, Tr - W:].contiguous() for x in (k, rotary_k, v, s, g)]
    recv = [torch.empty_like(x) for x in send]
    ops = []
    if rank + 1 < world:
        ops += [dist.P2POp(dist.isend, x, dist.get_global_rank(group, rank + 1) if group else rank + 1, group) for x in send]
    if rank > 0:
        ops += [dist.P2POp(dist.irecv, x, dist.get_global_rank(group, rank - 1) if group else rank - 1, group) for x in recv]
    if ops:
        for w in dist.batch_isend_irecv(ops):
            w.wait()
    if rank > 0:
        hk_, hrk, hv_, hs, hg = recv
        zq = q.new_zeros(B, W, *q.shape[2:])
        q_e, rq_e = torch.cat([zq, q], 1), torch.cat([zq, rotary_q], 1)
        k_e, rk_e = torch.cat([hk_, k], 1), torch.cat([hrk, rotary_k], 1)
        v_e, s_e, g_e = torch.cat([hv_, v], 1), torch.cat([hs, s], 1), torch.cat([hg, g], 1)
    else:
        q_e, rq_e, k_e, rk_e, v_e, s_e, g_e = q, rotary_q, k, rotary_k, v, s, g

    # ---- 2. segment summary from a zero start --------------------------------------------------------------
    # tokens entering the slot memory during this rank's steps: all of the extended segment but its last W
    n_enter = k_e.shape[1] - W
    Lk, Lv = local_state(k_e, v_e, s_e, g_e, W)
    G = g_e[:, :n_enter].float().sum(1)                                   # [B,H,M] total log decay

    # ---- 3. all-gather of the summaries, fold the ranks before this one ------------------------------------------
    pack = torch.cat([Lk.reshape(B, -1).float(), Lv.reshape(B, -1).float(), G.reshape(B, -1)], 1).contiguous()
    allp = [torch.empty_like(pack) for _ in range(world)]
    dist.all_gather(allp, pack, group=group)
    H, K, M = Lk.shape[1], Lk.shape[2], Lk.shape[3]
    V = Lv.shape[3]
    nk, nv = H * K * M, H * M * V
    if initial_state is not None and initial_state != (None, None):
        Sk, Sv = initial_state[0].float().clone(), initial_state[1].float().clone()
    else:
        Sk = torch.zeros(B, H, K, M, dtype=torch.float32, device=dev)
        Sv = torch.zeros(B, H, M, V, dtype=torch.float32, device=dev)
    for r in range(rank):
        pr = allp[r]
        lk = pr[:, :nk].reshape(B, H, K, M)
        lv = pr[:, nk:nk + nv].reshape(B, H, M, V)
        dec = pr[:, nk + nv:].reshape(B, H, M).exp()
        Sk = Sk * dec[:, :, None, :] + lk
        Sv = Sv * dec[:, :, :, None] + lv

    # ---- 4. forward from the true start state -----------------------------------------------------------------------
    o, hk, hv = forward(q_e, k_e, v_e, rq_e, rk_e, s_e, g_e, W, scale, (Sk, Sv))
    if rank > 0:
        o = o[:, W:]
    return o, (hk, hv)
