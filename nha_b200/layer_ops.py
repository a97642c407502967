"""Element-wise work of the calling layer around the operator, one launch each.

``feature_maps(q, k, v, feature_map='swish')`` replaces the layer's three element-wise kernels in front of the
operator (``nha_fla/layers/nha.py:219-223``)::

    q_gsa, k_gsa = map(lambda x: self.feature_map(x), (q, k))
    v = F.silu(v)

and ``silu_rms_norm_linear(o, norm_weight, norm_bias, linear_weight, linear_bias)`` the output side
(``nha_fla/layers/nha.py:277-278``)::

    o = rms_norm_linear(F.silu(o), self.g_norm.weight, self.g_norm.bias, self.o_proj.weight, self.o_proj.bias)

with silu, the RMS normalisation and its affine part in one pass over ``o`` (and one for the backward); the
projection stays a library GEMM (``F.linear``).
"""
from __future__ import annotations

import ctypes
from typing import Optional, Tuple

import torch
import torch.nn.functional as F

from . import _lib

_BF16 = torch.bfloat16


def _ptr_array(tensors):
    return (ctypes.c_void_p * len(tensors))(*[t.data_ptr() for t in tensors])


def _act3(xs, dys, relu: bool):
    lib = _lib.load()
    dev = xs[0].device
    outs = [torch.empty_like(x) for x in xs]
    n = (ctypes.c_int64 * len(xs))(*[x.numel() for x in xs])
    flags = (ctypes.c_int * len(xs))(*[1 if relu else 0] * len(xs))
    st = torch.cuda.current_stream(dev).cuda_stream
    with torch.cuda.device(dev):
        if dys is None:
            _lib.check(lib.nha_act3_fwd(_ptr_array(xs), _ptr_array(outs), n, flags, len(xs), st), 'nha_act3_fwd')
        else:
            _lib.check(lib.nha_act3_bwd(_ptr_array(xs), _ptr_array(dys), _ptr_array(outs), n, flags, len(xs), st),
                       'nha_act3_bwd')
    return outs


class _FeatureMaps(torch.autograd.Function):

    @staticmethod
    def forward(ctx, relu: bool, *xs):
        xc = [x.to(_BF16).contiguous() for x in xs]
        ctx.save_for_backward(*xc)
        ctx.relu = relu
        ctx.dtypes = [x.dtype for x in xs]
        return tuple(_act3(xc, None, relu))

    @staticmethod
    def backward(ctx, *dys):
        xc = list(ctx.saved_tensors)
        dyc = [torch.zeros_like(x) if dy is None else dy.to(_BF16).contiguous() for x, dy in zip(xc, dys)]
        dxs = _act3(xc, dyc, ctx.relu)
        return (None,) + tuple(dx.to(dt) for dx, dt in zip(dxs, ctx.dtypes))


def feature_maps(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, feature_map: Optional[str] = 'swish'
                 ) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """``(feature_map(q), feature_map(k), silu(v))`` in bf16, one launch forward and one backward.

    ``feature_map``: ``'swish'`` (``x * sigmoid(x)``), ``'relu'`` or ``None`` (q and k pass through and only ``silu(v)``
    is computed).  CUDA tensors of any shape."""
    assert q.is_cuda and k.is_cuda and v.is_cuda, 'feature_maps runs on the CUDA library only (there is no CPU path)'
    if feature_map is None:
        return q, k, _FeatureMaps.apply(False, v)[0]
    if feature_map not in ('swish', 'relu'):
        raise NotImplementedError(f'Feature map `{feature_map}` is not supported now.')
    if feature_map == 'swish':
        return _FeatureMaps.apply(False, q, k, v)
    qg, kg = _FeatureMaps.apply(True, q, k)
    return qg, kg, _FeatureMaps.apply(False, v)[0]


class _SiluRmsNorm(torch.autograd.Function):

    @staticmethod
    def forward(ctx, o, weight, bias, eps):
        lib = _lib.load()
        cols = o.shape[-1]
        oc = o.to(_BF16).contiguous().view(-1, cols)
        rows = oc.shape[0]
        w = weight.float().contiguous()
        b = None if bias is None else bias.float().contiguous()
        y = torch.empty_like(oc)
        rstd = torch.empty(rows, dtype=torch.float32, device=oc.device)
        st = torch.cuda.current_stream(oc.device).cuda_stream
        with torch.cuda.device(oc.device):
            _lib.check(lib.nha_silu_rmsnorm_fwd(oc.data_ptr(), w.data_ptr(), _lib.ptr(b), y.data_ptr(), rstd.data_ptr(), rows,
                                                cols, float(eps), st), 'nha_silu_rmsnorm_fwd')
        ctx.save_for_backward(oc, w, rstd)
        ctx.has_bias = bias is not None
        ctx.meta = (o.shape, o.dtype, weight.dtype, None if bias is None else bias.dtype)
        return y.view(o.shape)

    @staticmethod
    def backward(ctx, dy):
        lib = _lib.load()
        oc, w, rstd = ctx.saved_tensors
        shape, odt, wdt, bdt = ctx.meta
        rows, cols = oc.shape
        dyc = dy.to(_BF16).contiguous().view(rows, cols)
        d_o = torch.empty_like(oc)
        nparts = max(1, int(lib.nha_silu_rmsnorm_bwd_ctas(rows)))
        pw = torch.zeros(nparts, cols, dtype=torch.float32, device=oc.device)
        pb = torch.zeros(nparts, cols, dtype=torch.float32, device=oc.device) if ctx.has_bias else None
        st = torch.cuda.current_stream(oc.device).cuda_stream
        with torch.cuda.device(oc.device):
            _lib.check(lib.nha_silu_rmsnorm_bwd(oc.data_ptr(), w.data_ptr(), rstd.data_ptr(), dyc.data_ptr(), d_o.data_ptr(),
                                                pw.data_ptr(), _lib.ptr(pb), rows, cols, st), 'nha_silu_rmsnorm_bwd')
        dw = pw.sum(0).to(wdt)
        db = pb.sum(0).to(bdt) if ctx.has_bias else None
        return d_o.view(shape).to(odt), dw, db, None


def silu_rms_norm(o: torch.Tensor, weight: torch.Tensor, bias: Optional[torch.Tensor] = None, eps: float = 1e-5
                  ) -> torch.Tensor:
    """``rms_norm(silu(o)) * weight + bias`` over the last dimension (a multiple of 256, at most 2048), bf16."""
    assert o.is_cuda, 'silu_rms_norm runs on the CUDA library only (there is no CPU path)'
    return _SiluRmsNorm.apply(o, weight, bias, eps)


def silu_rms_norm_linear(o: torch.Tensor, norm_weight: torch.Tensor, norm_bias: Optional[torch.Tensor],
                         linear_weight: torch.Tensor, linear_bias: Optional[torch.Tensor] = None, eps: float = 1e-5
                         ) -> torch.Tensor:
    """The layer's ``rms_norm_linear(F.silu(o), norm_weight, norm_bias, linear_weight, linear_bias)``
    (nha_fla/layers/nha.py:277-278; eps is that function's default, which the layer does not override)."""
    y = silu_rms_norm(o, norm_weight, norm_bias, eps)
    return F.linear(y.to(linear_weight.dtype), linear_weight, linear_bias)
