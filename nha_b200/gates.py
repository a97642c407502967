"""``slot_gates``: the callers' gate chain in one launch.

The reference's layers compute the operator's two gate inputs from the gate projection with a chain of
element-wise torch kernels (``nha_fla/layers/nha.py:229-231``)::

    f = F.logsigmoid(f) / self.gate_logit_normalizer
    s = (1 - f.exp()).to(f.dtype)
    g = f

and the hybrid models do the same around their own ``g`` (``nha_fla/models/qwen3_nha/qwennha.py:116``).
``slot_gates(f, gate_logit_normalizer)`` returns ``(g, s)`` from one pass over ``f`` (and one pass for the
backward), so a layer replaces those three lines with ``g, s = slot_gates(f, self.gate_logit_normalizer)``.
"""
from __future__ import annotations

from typing import Tuple

import torch

from . import _lib

_BF16 = torch.bfloat16


class _SlotGates(torch.autograd.Function):

    @staticmethod
    def forward(ctx, f: torch.Tensor, normalizer: float):
        lib = _lib.load()
        fc = f.to(_BF16).contiguous()
        g = torch.empty_like(fc)
        s = torch.empty_like(fc)
        st = torch.cuda.current_stream(fc.device).cuda_stream
        with torch.cuda.device(fc.device):
            if fc.numel():
                _lib.check(lib.nha_slot_gates_fwd(fc.data_ptr(), g.data_ptr(), s.data_ptr(), fc.numel(), normalizer, st),
                           'nha_slot_gates_fwd')
        ctx.save_for_backward(fc)
        ctx.normalizer = normalizer
        ctx.in_dtype = f.dtype
        return g, s

    @staticmethod
    def backward(ctx, dg, ds):
        lib = _lib.load()
        (fc,) = ctx.saved_tensors
        dgc = None if dg is None else dg.to(_BF16).contiguous()
        dsc = None if ds is None else ds.to(_BF16).contiguous()
        if dgc is None and dsc is None:
            return None, None
        df = torch.empty_like(fc)
        st = torch.cuda.current_stream(fc.device).cuda_stream
        with torch.cuda.device(fc.device):
            if fc.numel():
                _lib.check(lib.nha_slot_gates_bwd(fc.data_ptr(), _lib.ptr(dgc), _lib.ptr(dsc), df.data_ptr(), fc.numel(),
                                                  ctx.normalizer, st), 'nha_slot_gates_bwd')
        return df.to(ctx.in_dtype), None


def slot_gates(f: torch.Tensor, gate_logit_normalizer: float = 8.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """``g = logsigmoid(f) / gate_logit_normalizer`` and ``s = 1 - exp(g)``, both bf16, same shape as ``f``.

    ``f`` is the gate projection on a CUDA device (any shape; cast to bf16 like the other inputs of the
    operator).  Differentiable with respect to ``f``.
    """
    assert f.is_cuda, 'slot_gates runs on the CUDA library only (there is no CPU path)'
    assert gate_logit_normalizer > 0
    return _SlotGates.apply(f, float(gate_logit_normalizer))
