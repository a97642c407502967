"""``rotary_pair``: the callers' rotary embedding of q and k in one launch.

The reference's layer rotates its queries and keys with ``self.rotary(q, k, seqlen_offset=...)``
(``nha_fla/layers/nha.py:145,235``; non-interleaved halves, tables of ``K/2`` columns, positions that
restart at every packed sequence) before it calls ``chunk_nha``; the hybrid models use rotate-half with
duplicated-halves tables of ``K`` columns (``nha_fla/models/qwen3_nha/qwennha.py:240-244``).  Both are
the same arithmetic on the first ``K/2`` table columns, so one kernel serves both: ``q_swa, k_swa =
rotary_pair(q, k, cos, sin, seqlen_offset, cu_seqlens)``.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_BF16 = torch.bfloat16


def _launch(q, k, cos, sin, offset, cu, T, inverse):
    lib = _lib.load()
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    K = q.shape[-1]
    Ttot = q.numel() // (q.shape[-2] * K)
    if Ttot:
        st = torch.cuda.current_stream(q.device).cuda_stream
        with torch.cuda.device(q.device):
            _lib.check(lib.nha_rope_pair(q.data_ptr(), k.data_ptr(), qo.data_ptr(), ko.data_ptr(), cos.data_ptr(),
                                         sin.data_ptr(), cos.stride(0), cos.shape[0], _lib.ptr(cu),
                                         0 if cu is None else cu.numel() - 1, T, Ttot, q.shape[-2], k.shape[-2], K,
                                         offset, inverse, st), 'nha_rope_pair')
    return qo, ko


class _RotaryPair(torch.autograd.Function):

    @staticmethod
    def forward(ctx, q, k, cos, sin, offset, cu, T):
        ctx.save_for_backward(cos, sin, cu)
        ctx.meta = (offset, T, q.dtype, k.dtype)
        return _launch(q.to(_BF16).contiguous(), k.to(_BF16).contiguous(), cos, sin, offset, cu, T, 0)

    @staticmethod
    def backward(ctx, dq, dk):
        cos, sin, cu = ctx.saved_tensors
        offset, T, qd, kd = ctx.meta
        gq, gk = _launch(dq.to(_BF16).contiguous(), dk.to(_BF16).contiguous(), cos, sin, offset, cu, T, 1)
        return gq.to(qd), gk.to(kd), None, None, None, None, None


def rotary_pair(q: torch.Tensor, k: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, seqlen_offset: int = 0,
                cu_seqlens: Optional[torch.Tensor] = None) -> Tuple[torch.Tensor, torch.Tensor]:
    """Rotate ``q [B,T,HQ,K]`` and ``k [B,T,H,K]`` (``B == 1`` with ``cu_seqlens``); returns bf16 ``(q_rot, k_rot)``.

    ``cos, sin``: tables ``[P, K/2]`` (or ``[P, K]`` with duplicated halves), row ``p`` for position ``p``;
    token ``t`` of a sequence uses row ``seqlen_offset + t``.  Differentiable with respect to ``q`` and ``k``.
    """
    assert q.is_cuda and k.is_cuda, 'rotary_pair runs on the CUDA library only (there is no CPU path)'
    assert q.dim() == 4 and k.dim() == 4 and q.shape[:2] == k.shape[:2] and q.shape[-1] == k.shape[-1]
    B, T, _, K = q.shape
    assert K % 16 == 0, 'head dim must be a multiple of 16'
    assert cos.shape == sin.shape and cos.dim() == 2 and cos.shape[1] in (K // 2, K)
    assert seqlen_offset >= 0
    if cu_seqlens is not None:
        assert B == 1, 'packed input has batch size 1'
        cu_seqlens = cu_seqlens.to(torch.int32).contiguous()
    else:
        assert seqlen_offset + T <= cos.shape[0], 'cos/sin tables do not cover the positions'
    cosc, sinc = cos.to(_BF16).contiguous(), sin.to(_BF16).contiguous()
    if cosc.shape[1] % 8:                                   # rows of 16-byte pieces
        pad = 8 - cosc.shape[1] % 8
        cosc, sinc = torch.nn.functional.pad(cosc, (0, pad)), torch.nn.functional.pad(sinc, (0, pad))
    return _RotaryPair.apply(q, k, cosc, sinc, int(seqlen_offset), cu_seqlens, T)
