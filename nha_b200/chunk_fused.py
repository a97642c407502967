"""``fused_chunk_nha_prefill``: inference prefill on the chunked sm_100a forward.

Same signature and return convention as ``nha_fla/ops/nha/chunk_fused.py:291-380``
(window ``[t-W+1, t]``, slot memory holds tokens ``<= t-W``, inputs in the kv-head
layout).  The reference restricts ``W <= 64`` and power-of-two ``K, V, M <= 128``;
this op takes any ``W >= 1`` (the window loop walks 64-key tiles) and
``K, V in {32,64,96,128}``, ``M`` a multiple of 16 that fits shared memory.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from .chunk import chunk_forward

_BF16 = torch.bfloat16


@torch.no_grad()
def fused_chunk_nha_prefill(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    rotary_q: torch.Tensor,
    rotary_k: torch.Tensor,
    s: torch.Tensor,
    g: torch.Tensor,
    window_size: int,
    initial_state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    output_final_state: bool = False,
    scale: Optional[float] = None,
) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    r"""Fused NHA prefill (inference only, no autograd).

    Args: ``q, rotary_q [B,T,HQ,K]``; ``k, rotary_k [B,T,H,K]``; ``v [B,T,H,V]``;
    ``s, g [B,T,H,M]`` (kv heads); ``window_size`` W >= 1; ``initial_state``
    ``(hk0 [B,H,K,M], hv0 [B,H,M,V])`` fp32 at the kv-head count.
    Returns ``(o [B,T,HQ,V], (hkt, hvt))`` with fp32 final states or ``(None, None)``.
    """
    B, T, HQ, K = q.shape
    H = k.shape[2]
    V = v.shape[-1]
    M = s.shape[-1]
    W = int(window_size)
    assert k.shape[1] == T and v.shape[1] == T and s.shape[1] == T and g.shape[1] == T
    assert rotary_q.shape == q.shape and rotary_k.shape == k.shape
    assert HQ % H == 0
    assert W >= 1
    hk0 = hv0 = None
    if initial_state is not None and initial_state != (None, None):
        hk0, hv0 = initial_state[0].float().contiguous(), initial_state[1].float().contiguous()
        assert hk0.shape == (B, H, K, M) and hv0.shape == (B, H, M, V), \
            f"initial_state must be at the kv-head count [B, {H}, ...], got {hk0.shape} / {hv0.shape}"
    if scale is None:
        scale = K ** -0.5
    dev = q.device
    out_dtype = q.dtype

    def flat(x):
        x = x.reshape(B * T, *x.shape[2:])
        return (x if x.dtype == _BF16 else x.to(_BF16)).contiguous()

    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=dev)
    o, _, _, hkt, hvt, _ = chunk_forward(
        flat(q), flat(rotary_q), flat(k), flat(rotary_k), flat(v), flat(s), flat(g), cu, T, scale,
        W - 1, W, hk0, hv0, output_final_state)
    o = o.view(B, T, HQ, V)
    if out_dtype != _BF16:
        o = o.to(out_dtype)
    return o, ((hkt, hvt) if output_final_state else (None, None))
