"""Single-token NHA ops on the fused sm_100a decode kernel.

Same names, arguments, return values and error behaviour as
``nha_fla/ops/nha/fused_recurrent.py`` (``fused_recurrent_nha_decode`` :431-584,
``fused_recurrent_nha`` :588-682); the arithmetic runs in one CUDA launch through
``nha_decode_step`` of the C ABI.
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch

from . import _lib

_BF16 = torch.bfloat16


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


_WORKSPACES = {}


def _decode_workspace(device, B, HQ, H, V, W):
    """Zero-initialised scratch for the split decode kernels, one per (device, stream, B * H); the
    kernels leave their counters at zero, so the buffer is reused by later calls on the same stream."""
    lib = _lib.load()
    need = int(lib.nha_decode_workspace_bytes(B, HQ, H, V, W))
    key = (device.index, torch.cuda.current_stream(device).cuda_stream, B * H)   # the layout depends on B * H
    ws = _WORKSPACES.get(key)
    if ws is None or ws.numel() < need:
        ws = torch.zeros(need, dtype=torch.uint8, device=device)
        _WORKSPACES[key] = ws
    return ws


class _Bf16StateSwitch:
    """Set while ``fused_recurrent_nha_decode_bf16_state`` runs: the decode op then keeps the slot memory in bf16."""
    active = False


_BF16_STATE = _Bf16StateSwitch()


def _bf16c(x: Optional[torch.Tensor]) -> Optional[torch.Tensor]:
    if x is None:
        return None
    if x.dtype != _BF16:
        x = x.to(_BF16)
    return x.contiguous()


def _state(initial_state, B, H, K, V, M, device, output_final_state, dtype=torch.float32):
    """Returns (hk, hv, zero_state).  The kernel updates the state buffers in place."""
    if initial_state is not None and initial_state != (None, None):
        hk0, hv0 = initial_state
        assert hk0.shape == (B, H, K, M) and hv0.shape == (B, H, M, V), \
            f"initial_state must be ([B,H,K,M], [B,H,M,V]) at the kv-head count {H}, got {tuple(hk0.shape)} / {tuple(hv0.shape)}"
        inplace_ok = (output_final_state and hk0.dtype == dtype and hv0.dtype == dtype
                      and hk0.is_contiguous() and hv0.is_contiguous())
        if inplace_ok:
            return hk0, hv0, 0
        return hk0.to(dtype).contiguous().clone(), hv0.to(dtype).contiguous().clone(), 0
    hk = torch.empty(B, H, K, M, dtype=dtype, device=device)
    hv = torch.empty(B, H, M, V, dtype=dtype, device=device)
    return hk, hv, 1


def fused_recurrent_nha_decode(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    g: torch.Tensor,
    sw_k: torch.Tensor,
    sw_v: torch.Tensor,
    sq: Optional[torch.Tensor] = None,
    s: Optional[torch.Tensor] = None,
    cos: Optional[torch.Tensor] = None,
    sin: Optional[torch.Tensor] = None,
    initial_state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    output_final_state: bool = False,
    scale: Optional[float] = None,
) -> Tuple[torch.Tensor, Tuple[torch.Tensor, torch.Tensor]]:
    r"""Single-token fused NHA decode step with GQA support (one kernel launch).

    Args (as nha_fla/ops/nha/fused_recurrent.py:446-486):
        q: raw queries ``[B, 1, HQ, K]``.
        k, v, g: the entry leaving the window, ``[B, 1, H, K|V|M]`` (kv heads).
        sw_k, sw_v: window keys/values ``[B, W, H, K|V]``, time ascending; keys
            un-rotated when ``cos``/``sin`` are given, pre-rotated otherwise.
        sq: pre-rotated queries ``[B, 1, HQ, K]`` (required without cos/sin).
        s: optional slot write weight ``[B, 1, H, M]``; ``1 - exp(g)`` in fp32 if omitted.
        cos, sin: rotate-half tables ``[B | 1, W2 >= W, K]``; the last W rows are the
            window positions and row ``W-1`` is the query position.
        initial_state: ``(hk0 [B,H,K,M], hv0 [B,H,M,V])`` fp32, or None / (None, None) for zeros.
        output_final_state: return the updated state.
        scale: defaults to ``K ** -0.5``.

    Returns ``(o [B,1,HQ,V], (hkt, hvt))``; the tuple is ``(None, None)`` when
    ``output_final_state=False``.

    State aliasing: with ``output_final_state=True`` and a contiguous fp32
    ``initial_state`` the returned states ARE the input buffers, updated in place
    (the reference does this for ``HQ == H`` and allocates new tensors otherwise;
    its callers always store the returned tuple back into the cache).
    """
    B, T, HQ, K = q.shape
    H = sw_k.shape[2]
    V = v.shape[-1]
    M = g.shape[-1]
    W = sw_k.shape[1]
    assert T == 1 and k.shape[1] == 1 and g.shape[1] == 1
    assert k.shape[2] == H and v.shape[2] == H and g.shape[2] == H, \
        f"popped-entry head count must match the kv-head count ({H}) of the window tensors"
    assert sw_v.shape[1] == W and sw_v.shape[2] == H
    assert HQ % H == 0
    assert K >= 16 and V >= 16
    if scale is None:
        scale = K ** -0.5
    rotary = cos is not None
    cs_batch = cs_row = 0
    if rotary:
        assert sq is None, "pass either sq (pre-rotated) or cos/sin (in-kernel rotary), not both"
        assert sin is not None and cos.shape == sin.shape
        assert cos.shape[0] in (1, B) and cos.shape[1] >= W and cos.shape[2] == K, \
            f"rotary cos/sin must be [1|{B}, W2>={W}, K={K}], got {tuple(cos.shape)}"
        assert K % 2 == 0, "in-kernel rotate-half requires an even head dim"
        if cos.shape[1] != W:
            cos = cos[:, -W:]
            sin = sin[:, -W:]

        def vec_ok(t):
            return (t.dtype == _BF16 and t.stride(-1) == 1 and t.stride(1) % 8 == 0 and t.stride(0) % 8 == 0
                    and t.data_ptr() % 16 == 0)
        if not (vec_ok(cos) and vec_ok(sin) and cos.stride() == sin.stride()):
            cos, sin = cos.to(_BF16).contiguous(), sin.to(_BF16).contiguous()
        cs_batch = cos.stride(0) if cos.shape[0] == B and B > 1 else 0
        cs_row = cos.stride(1)
    else:
        assert sq is not None and sq.shape == q.shape
    if s is not None:
        assert s.shape == g.shape

    dev = q.device
    out_dtype = q.dtype
    qf = _bf16c(q.reshape(B, HQ, K))
    sqf = None if sq is None else _bf16c(sq.reshape(B, HQ, K))
    kf, vf, gf = _bf16c(k.reshape(B, H, K)), _bf16c(v.reshape(B, H, V)), _bf16c(g.reshape(B, H, M))
    sf = None if s is None else _bf16c(s.reshape(B, H, M))
    swk, swv = _bf16c(sw_k), _bf16c(sw_v)
    bf16_state = _BF16_STATE.active
    hk, hv, zero = _state(initial_state, B, H, K, V, M, dev, output_final_state, _BF16 if bf16_state else torch.float32)
    o = torch.empty(B, HQ, V, dtype=_BF16, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        ws = _decode_workspace(dev, B, HQ, H, V, W) if (W > 64 or bf16_state) else None
        if bf16_state:
            st = lib.nha_decode_step_bf16_state(
                _lib.ptr(qf), _lib.ptr(sqf), _lib.ptr(kf), _lib.ptr(vf), _lib.ptr(gf), _lib.ptr(sf),
                _lib.ptr(swk), _lib.ptr(swv), _lib.ptr(cos if rotary else None), _lib.ptr(sin if rotary else None),
                cs_batch, cs_row, _lib.ptr(hk), _lib.ptr(hv), zero, _lib.ptr(o),
                _lib.ptr(ws), 0 if ws is None else ws.numel(),
                B, HQ, H, K, V, M, W, float(scale), _stream(dev))
        else:
            st = lib.nha_decode_step(
                _lib.ptr(qf), _lib.ptr(sqf), _lib.ptr(kf), _lib.ptr(vf), _lib.ptr(gf), _lib.ptr(sf),
                _lib.ptr(swk), _lib.ptr(swv), _lib.ptr(cos if rotary else None), _lib.ptr(sin if rotary else None),
                cs_batch, cs_row, None, _lib.ptr(hk), _lib.ptr(hv), zero, _lib.ptr(o), None,
                _lib.ptr(ws), 0 if ws is None else ws.numel(),
                B, HQ, H, K, V, M, W, float(scale), _stream(dev))
        _lib.check(st, 'nha_decode_step')
        _lib.check_decode_device(lib, ws, B, H, _stream(dev), 'nha_decode_step')
    o = o.view(B, 1, HQ, V)
    if out_dtype != _BF16:
        o = o.to(out_dtype)
    return o, ((hk, hv) if output_final_state else (None, None))


@torch.compiler.disable
def fused_recurrent_nha_decode_bf16_state(*args, **kwargs):
    """``fused_recurrent_nha_decode`` with the slot memory kept in bf16: same arguments; ``initial_state`` tensors in
    bf16 are updated in place (others are converted once), and the returned states are bf16.  Half the state bytes per
    step.  An extension: the reference keeps fp32 states (nha_fla/ops/nha/fused_recurrent.py:536-545), so results follow
    it to bf16 accuracy of the state only.  ``K == V`` in {64, 128} with window keys (the streaming kernel)."""
    _BF16_STATE.active = True
    try:
        return fused_recurrent_nha_decode(*args, **kwargs)
    finally:
        _BF16_STATE.active = False


@torch.compiler.disable
def fused_recurrent_nha(
    q: torch.Tensor,
    k: torch.Tensor,
    v: torch.Tensor,
    sliding_window: torch.Tensor,
    s: torch.Tensor,
    g: torch.Tensor,
    scale: Optional[float] = None,
    initial_state: Optional[Tuple[torch.Tensor]] = None,
    output_final_state: Optional[bool] = False,
) -> Tuple[torch.Tensor, torch.Tensor, list]:
    r"""Single-token NHA inference step with caller-supplied window logits.

    Args (as nha_fla/ops/nha/fused_recurrent.py:599-623): ``q [B,1,HQ,K]``,
    ``k [B,1,H,K]``, ``v [B,1,H,V]``, ``sliding_window [B,1,HQ,W]`` logits of the
    current token, ``s, g [B,1,H,M]``.  Returns ``(o, swa_score, [hkt, hvt])``:
    the slot-only readout ``[B,1,HQ,V]``, the window part of the joint softmax
    ``[B,1,HQ,W]`` (fp32) and the updated states (``[None, None]`` unless
    ``output_final_state``).  Raises ``ValueError`` for ``T != 1`` and asserts that no
    gradient is requested, like the reference (:656-660).
    """
    T = q.shape[1]
    if T != 1:
        raise ValueError(
            f"fused_recurrent_nha is the single-token inference path and expects T == 1, got T = {T}."
        )
    assert not q.requires_grad, "fused_recurrent_nha is inference-only (no autograd)"
    B, _, HQ, K = q.shape
    H, V, M = k.shape[2], v.shape[-1], s.shape[-1]
    W = sliding_window.shape[-1]
    assert HQ % H == 0
    if scale is None:
        scale = k.shape[-1] ** -0.5
    dev = q.device
    out_dtype = v.dtype
    qf, kf, vf = _bf16c(q.reshape(B, HQ, K)), _bf16c(k.reshape(B, H, K)), _bf16c(v.reshape(B, H, V))
    sf, gf = _bf16c(s.reshape(B, H, M)), _bf16c(g.reshape(B, H, M))
    wlog = _bf16c(sliding_window.reshape(B, HQ, W))
    hk, hv, zero = _state(initial_state, B, H, K, V, M, dev, output_final_state)
    o = torch.empty(B, HQ, V, dtype=_BF16, device=dev)
    prob = torch.empty(B, HQ, W, dtype=torch.float32, device=dev)
    lib = _lib.load()
    with torch.cuda.device(dev):
        st = lib.nha_decode_step(
            _lib.ptr(qf), None, _lib.ptr(kf), _lib.ptr(vf), _lib.ptr(gf), _lib.ptr(sf),
            None, None, None, None, 0, 0, _lib.ptr(wlog), _lib.ptr(hk), _lib.ptr(hv), zero, _lib.ptr(o),
            _lib.ptr(prob), None, 0, B, HQ, H, K, V, M, W, float(scale), _stream(dev))
    _lib.check(st, 'nha_decode_step')
    o = o.view(B, 1, HQ, V)
    if out_dtype != _BF16:
        o = o.to(out_dtype)
    return o, prob.view(B, 1, HQ, W), ([hk, hv] if output_final_state else [None, None])
