"""``gsa_aux_loss``: the training layer's consumers of the operator's two log-sum-exps, in one launch.

The reference's layer computes, from ``lse_swa`` and ``lse_gsa`` (``nha_fla/layers/nha.py:255-264, 288-323``)::

    gsa_ratio = (w_gsa / (w_swa + w_gsa)).mean()                       # monitoring, with an .item()
    delta     = lse_gsa.float() - lse_swa.detach().float()
    aux_loss  = F.binary_cross_entropy_with_logits(delta, full_like(delta, target), reduction='mean')

``gsa_aux_loss(lse_swa, lse_gsa, target)`` returns ``(aux_loss, gsa_ratio)`` as 0-dim device tensors (no host
synchronisation); ``aux_loss`` is differentiable with respect to ``lse_gsa`` only, as in the reference.
"""
from __future__ import annotations

from typing import Dict, Tuple

import torch

from . import _lib

_scratch: Dict[Tuple[int, int], torch.Tensor] = {}


def _scratch_for(dev: torch.device) -> torch.Tensor:
    key = (dev.index, torch.cuda.current_stream(dev).cuda_stream)
    t = _scratch.get(key)
    if t is None:
        t = torch.zeros(int(_lib.load().nha_lse_stats_scratch_bytes()), dtype=torch.uint8, device=dev)
        _scratch[key] = t
    return t


class _GsaAuxLoss(torch.autograd.Function):

    @staticmethod
    def forward(ctx, lse_swa: torch.Tensor, lse_gsa: torch.Tensor, target: float):
        lib = _lib.load()
        ls, lg = lse_swa.detach().float().contiguous(), lse_gsa.detach().float().contiguous()
        assert ls.shape == lg.shape and ls.numel() > 0
        out = torch.empty(2, dtype=torch.float32, device=ls.device)
        with torch.cuda.device(ls.device):
            _lib.check(lib.nha_lse_stats(ls.data_ptr(), lg.data_ptr(), ls.numel(), target, out.data_ptr(),
                                         _scratch_for(ls.device).data_ptr(),
                                         torch.cuda.current_stream(ls.device).cuda_stream), 'nha_lse_stats')
        ctx.save_for_backward(ls, lg)
        ctx.target = target
        ctx.in_dtype = lse_gsa.dtype
        ratio = out[1]
        ctx.mark_non_differentiable(ratio)
        return out[0], ratio

    @staticmethod
    def backward(ctx, dloss, _dratio):
        lib = _lib.load()
        ls, lg = ctx.saved_tensors
        d = torch.empty_like(lg)
        dl = dloss.detach().float().reshape(1).contiguous()
        with torch.cuda.device(ls.device):
            _lib.check(lib.nha_lse_aux_grad(ls.data_ptr(), lg.data_ptr(), dl.data_ptr(), ls.numel(), ctx.target,
                                            d.data_ptr(), torch.cuda.current_stream(ls.device).cuda_stream),
                       'nha_lse_aux_grad')
        return None, d.to(ctx.in_dtype), None


def gsa_aux_loss(lse_swa: torch.Tensor, lse_gsa: torch.Tensor, target_ratio: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """``(aux_loss, gsa_ratio)``: mean BCE-with-logits of ``lse_gsa - lse_swa`` against ``target_ratio`` and the mean
    share of the slot branch ``sigmoid(lse_gsa - lse_swa)``; both 0-dim fp32 tensors on the device."""
    assert lse_swa.is_cuda and lse_gsa.is_cuda, 'gsa_aux_loss runs on the CUDA library only (there is no CPU path)'
    return _GsaAuxLoss.apply(lse_swa, lse_gsa, float(target_ratio))
