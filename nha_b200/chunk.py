"""``chunk_nha``: training / prefill NHA with autograd on the chunked sm_100a kernels.

Same signature, return convention and error behaviour as
``nha_fla/ops/nha/chunk.py:568-690``.  Where the reference chains flash-attn
(window branch), fla's chunk_gsa (slot branch) and a log-sum-exp merge, this op
runs one state pass and one output pass (forward) and the chunked backward of the
C ABI (``nha_chunk_fwd`` / ``nha_chunk_bwd``); the joint softmax is never split.

Extension: ``window_size_left`` and ``gsa_kv_shift`` may be int32 tensors ``[N]``
(one value per packed sequence) in varlen mode, and k/v/s/g may be given at the
kv-head count ``H`` (``HQ % H == 0``), in which case states are per kv head.
"""
from __future__ import annotations

from typing import Optional, Tuple, Union

import torch

from . import _lib

_BF16 = torch.bfloat16
IntOrTensor = Union[int, torch.Tensor]


def _stream(device) -> int:
    return torch.cuda.current_stream(device).cuda_stream


def _per_seq(x: IntOrTensor, N: int, device) -> Tuple[Optional[torch.Tensor], int]:
    """(device int32 [N] tensor or None, scalar) for a window/shift argument."""
    if torch.is_tensor(x):
        if x.numel() == 1:
            return None, int(x.item())
        assert x.numel() == N, f"per-sequence tensor must have {N} entries, got {x.numel()}"
        return x.to(device=device, dtype=torch.int32).contiguous(), 0
    return None, int(x)


class _Geometry:
    """Sizes + device-side plan shared by the forward and the backward of one call."""

    def __init__(self, q_gsa, k_gsa, v, s, cu_seqlens, max_seqlen, q_offset=0):
        self.Ttot = k_gsa.shape[0]                       # q may hold fewer rows (q_offset > 0)
        _, self.HQ, self.K = q_gsa.shape
        self.H = k_gsa.shape[1]
        self.V = v.shape[-1]
        self.M = s.shape[-1]
        self.N = cu_seqlens.numel() - 1
        self.max_seqlen = int(max_seqlen)
        self.q_offset = int(q_offset)
        self.device = q_gsa.device
        lib = _lib.load()
        self.ncb = int(lib.nha_chunk_count_bound(self.Ttot, self.N))
        self.plan = torch.empty(int(lib.nha_chunk_plan_ints(self.Ttot, self.N, self.H)), dtype=torch.int32, device=self.device)


def _fill_desc(geo: _Geometry, t: dict, scale, wl_t, wl_all, sh_t, sh_all) -> _lib.ChunkDesc:
    d = _lib.ChunkDesc()
    for name in ('q_gsa', 'q_swa', 'k_gsa', 'k_swa', 'v', 's', 'g', 'cu_seqlens', 'hk0', 'hv0', 'o', 'lse_swa',
                 'lse_gsa', 'hkt', 'hvt', 'hk_chunks', 'hv_chunks', 'workspace', 'd_o', 'd_lse_gsa', 'd_hkt', 'd_hvt',
                 'dq_gsa', 'dq_swa', 'dk_gsa', 'dk_swa', 'dv', 'ds', 'dg', 'dhk0', 'dhv0'):
        setattr(d, name, _lib.ptr(t.get(name)))
    d.window_left = _lib.ptr(wl_t)
    d.shift = _lib.ptr(sh_t)
    d.plan = geo.plan.data_ptr()
    ws = t.get('workspace')
    d.workspace_bytes = 0 if ws is None else ws.numel()
    d.Ttot, d.N, d.HQ, d.H, d.K, d.V, d.M = geo.Ttot, geo.N, geo.HQ, geo.H, geo.K, geo.V, geo.M
    d.max_seqlen = geo.max_seqlen
    d.window_left_all, d.shift_all = wl_all, sh_all
    d.q_offset = geo.q_offset
    d.scale = float(scale)
    return d


def chunk_forward(q_gsa, q_swa, k_gsa, k_swa, v, s, g, cu_seqlens, max_seqlen, scale, window_left, shift,
                  hk0=None, hv0=None, output_final_state=False, q_offset=0):
    """Flat packed forward on ``[Ttot, heads, dim]`` bf16 tensors.  Returns
    ``(o, lse_swa, lse_gsa, hkt, hvt, saved)`` where ``saved`` carries what the backward needs."""
    lib = _lib.load()
    geo = _Geometry(q_gsa, k_gsa, v, s, cu_seqlens, max_seqlen, q_offset)
    dev = geo.device
    wl_t, wl_all = _per_seq(window_left, geo.N, dev)
    sh_t, sh_all = _per_seq(shift, geo.N, dev)
    t = dict(q_gsa=q_gsa, q_swa=q_swa, k_gsa=k_gsa, k_swa=k_swa, v=v, s=s, g=g, cu_seqlens=cu_seqlens,
             hk0=hk0, hv0=hv0)
    nq = geo.Ttot - geo.q_offset
    assert q_gsa.shape[0] == nq and q_swa.shape[0] == nq, 'q tensors must hold the positions from q_offset on'
    t['o'] = torch.empty(nq, geo.HQ, geo.V, dtype=_BF16, device=dev)
    t['lse_swa'] = torch.empty(nq, geo.HQ, dtype=torch.float32, device=dev)
    t['lse_gsa'] = torch.empty(nq, geo.HQ, dtype=torch.float32, device=dev)
    if output_final_state:
        t['hkt'] = torch.empty(geo.N, geo.H, geo.K, geo.M, dtype=torch.float32, device=dev)
        t['hvt'] = torch.empty(geo.N, geo.H, geo.M, geo.V, dtype=torch.float32, device=dev)
    t['hk_chunks'] = torch.empty(geo.ncb, geo.H, geo.K, geo.M, dtype=_BF16, device=dev)
    t['hv_chunks'] = torch.empty(geo.ncb, geo.H, geo.M, geo.V, dtype=_BF16, device=dev)
    d = _fill_desc(geo, t, scale, wl_t, wl_all, sh_t, sh_all)
    nbytes = int(lib.nha_chunk_fwd_workspace_bytes(d))
    if nbytes > 0:
        t['workspace'] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        d = _fill_desc(geo, t, scale, wl_t, wl_all, sh_t, sh_all)
    with torch.cuda.device(dev):
        _lib.check(lib.nha_chunk_fwd(d, _stream(dev)), 'nha_chunk_fwd')
        _lib.check_chunk_device(lib, d, _stream(dev), 'nha_chunk_fwd')
    saved = dict(geo=geo, wl=(wl_t, wl_all), sh=(sh_t, sh_all), hk_chunks=t['hk_chunks'], hv_chunks=t['hv_chunks'])
    return t['o'], t['lse_swa'], t['lse_gsa'], t.get('hkt'), t.get('hvt'), saved


def chunk_backward(q_gsa, q_swa, k_gsa, k_swa, v, s, g, cu_seqlens, scale, saved, o, lse_swa, lse_gsa, d_o,
                   d_lse_gsa=None, d_hkt=None, d_hvt=None, hkt=None, hvt=None, hk0=None, hv0=None,
                   need_state_grad=False):
    """Flat packed backward.  Returns ``(dq_swa, dk_swa, dq_gsa, dk_gsa, dv, ds, dg, dhk0, dhv0)``."""
    lib = _lib.load()
    geo: _Geometry = saved['geo']
    dev = geo.device
    wl_t, wl_all = saved['wl']
    sh_t, sh_all = saved['sh']
    t = dict(q_gsa=q_gsa, q_swa=q_swa, k_gsa=k_gsa, k_swa=k_swa, v=v, s=s, g=g, cu_seqlens=cu_seqlens,
             hk0=hk0, hv0=hv0, o=o, lse_swa=lse_swa, lse_gsa=lse_gsa, hkt=hkt, hvt=hvt,
             hk_chunks=saved['hk_chunks'], hv_chunks=saved['hv_chunks'], d_o=d_o, d_lse_gsa=d_lse_gsa,
             d_hkt=d_hkt, d_hvt=d_hvt)
    for name, ref in (('dq_gsa', q_gsa), ('dq_swa', q_swa), ('dk_gsa', k_gsa), ('dk_swa', k_swa), ('dv', v),
                      ('ds', s), ('dg', g)):
        t[name] = torch.empty_like(ref)
    if need_state_grad:
        t['dhk0'] = torch.empty(geo.N, geo.H, geo.K, geo.M, dtype=torch.float32, device=dev)
        t['dhv0'] = torch.empty(geo.N, geo.H, geo.M, geo.V, dtype=torch.float32, device=dev)
    d = _fill_desc(geo, t, scale, wl_t, wl_all, sh_t, sh_all)
    nbytes = int(lib.nha_chunk_bwd_workspace_bytes(d))
    t['workspace'] = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=dev)
    d = _fill_desc(geo, t, scale, wl_t, wl_all, sh_t, sh_all)
    with torch.cuda.device(dev):
        _lib.check(lib.nha_chunk_bwd(d, _stream(dev)), 'nha_chunk_bwd')
        _lib.check_chunk_device(lib, d, _stream(dev), 'nha_chunk_bwd')
    return (t['dq_swa'], t['dk_swa'], t['dq_gsa'], t['dk_gsa'], t['dv'], t['ds'], t['dg'],
            t.get('dhk0'), t.get('dhv0'))


class ChunkNativeHybridAttentionFunction(torch.autograd.Function):
    """Autograd node of ``chunk_nha`` on flat packed tensors.

    Mirrors nha_fla/ops/nha/chunk.py:352-564: gradients flow to q_swa, k_swa, q_gsa,
    k_gsa, v, s, g and the initial states; a gradient arriving on ``lse_gsa`` is
    honoured, one arriving on ``lse_swa`` is dropped exactly as the reference drops it
    (chunk.py:491-512)."""

    @staticmethod
    def forward(ctx, q_swa, k_swa, q_gsa, k_gsa, v, s, g, cu_seqlens, max_seqlen, scale, window_left, shift,
                hk0, hv0, output_final_state, q_offset):
        o, lse_swa, lse_gsa, hkt, hvt, saved = chunk_forward(
            q_gsa, q_swa, k_gsa, k_swa, v, s, g, cu_seqlens, max_seqlen, scale, window_left, shift,
            hk0, hv0, output_final_state, q_offset)
        ctx.save_for_backward(q_swa, k_swa, q_gsa, k_gsa, v, s, g, cu_seqlens, o, lse_swa, lse_gsa,
                              saved['hk_chunks'], saved['hv_chunks'], hk0, hv0, hkt, hvt)
        ctx.saved_meta = saved
        ctx.scale = scale
        ctx.state_grad = hk0 is not None and (hk0.requires_grad or hv0.requires_grad)
        ctx.mark_non_differentiable(lse_swa)
        if hkt is None:
            return o, lse_swa, lse_gsa, None, None
        return o, lse_swa, lse_gsa, hkt, hvt

    @staticmethod
    def backward(ctx, d_o, d_lse_swa, d_lse_gsa, d_hkt, d_hvt):
        (q_swa, k_swa, q_gsa, k_gsa, v, s, g, cu_seqlens, o, lse_swa, lse_gsa, hk_chunks, hv_chunks, hk0, hv0,
         hkt, hvt) = ctx.saved_tensors
        saved = dict(ctx.saved_meta, hk_chunks=hk_chunks, hv_chunks=hv_chunks)
        d_o = d_o.contiguous().to(_BF16)
        if d_lse_gsa is not None:
            d_lse_gsa = d_lse_gsa.float().contiguous()
        if d_hkt is not None or d_hvt is not None:
            d_hkt = torch.zeros_like(hkt) if d_hkt is None else d_hkt.float().contiguous()
            d_hvt = torch.zeros_like(hvt) if d_hvt is None else d_hvt.float().contiguous()
        grads = chunk_backward(q_gsa, q_swa, k_gsa, k_swa, v, s, g, cu_seqlens, ctx.scale, saved, o, lse_swa, lse_gsa,
                               d_o, d_lse_gsa, d_hkt, d_hvt, hkt, hvt, hk0, hv0, need_state_grad=ctx.state_grad)
        dq_swa, dk_swa, dq_gsa, dk_gsa, dv, ds, dg, dhk0, dhv0 = grads
        return (dq_swa, dk_swa, dq_gsa, dk_gsa, dv, ds, dg, None, None, None, None, None, dhk0, dhv0, None, None)


@torch.compiler.disable
def chunk_nha(
    q_swa: torch.Tensor,
    k_swa: torch.Tensor,
    q_gsa: torch.Tensor,
    k_gsa: torch.Tensor,
    v: torch.Tensor,
    s: torch.Tensor,
    g: torch.Tensor,
    cu_seqlens: Optional[torch.Tensor] = None,
    max_seqlen: Optional[int] = None,
    scale: Optional[float] = None,
    window_size_left: IntOrTensor = -1,
    window_size_right: int = -1,
    head_first: Optional[bool] = False,
    gsa_kv_shift: IntOrTensor = 0,
    initial_state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    output_final_state: bool = False,
):
    r"""Chunk-level Native Hybrid Attention (sliding window + gated slot memory, one softmax).

    Args (as nha_fla/ops/nha/chunk.py:586-632):
        q_swa, k_swa: rotated query/key of the window branch, ``[B, T, H, D]``.
        q_gsa, k_gsa: un-rotated query/key of the slot branch, ``[B, T, H, D]``.
        v: shared values ``[B, T, H, V]``;  s, g: slot write weights and log forget gates ``[B, T, H, M]``.
        cu_seqlens: ``[N+1]`` packed-sequence boundaries (then ``B == 1``); max_seqlen: longest sequence.
        scale: defaults to ``D ** -0.5``.
        window_size_left: the window covers keys ``t - window_size_left .. t`` (``-1`` = unbounded).
        window_size_right: must be ``0`` or ``-1`` (the window is causal either way).
        head_first: deprecated; ``True`` raises ``DeprecationWarning`` like the reference.
        gsa_kv_shift: token ``t - gsa_kv_shift`` enters the slot memory at step ``t``.
        initial_state: ``(hk0 [N,H,K,M], hv0 [N,H,M,V])``;  output_final_state: also return the fp32 final states.

    Returns ``(o [B,T,H,V], lse_swa [B,T,H], lse_gsa [B,T,H])`` and, only when
    ``output_final_state=True``, a 4th element ``(hkt, hvt)``.
    """
    if head_first:
        raise DeprecationWarning(
            "head_first is deprecated and will be removed in a future version. "
            "Please use head_first=False for now instead.",
        )
    if scale is None:
        scale = q_swa.shape[-1] ** -0.5
    assert q_swa.dim() == 4, "Expected [B, T, H, D] for input"
    assert window_size_right in (0, -1), "the window branch is causal: window_size_right must be 0 or -1"
    B, T, HQ, D = q_swa.shape
    dev = q_swa.device
    is_varlen = cu_seqlens is not None
    if is_varlen:
        assert B == 1, "varlen inputs must be packed into a single batch row"
        cu = cu_seqlens.to(device=dev, dtype=torch.int32).contiguous()
        if max_seqlen is None:
            max_seqlen = int((cu[1:] - cu[:-1]).max().item())
    else:
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=dev)
        max_seqlen = T
    out_dtype = q_swa.dtype

    def flat(x):
        x = x.reshape(B * T, *x.shape[2:])
        if x.dtype != _BF16:
            x = x.to(_BF16)
        return x.contiguous()

    hk0, hv0 = (None, None) if initial_state is None else initial_state
    if hk0 is not None:
        hk0, hv0 = hk0.float().contiguous(), hv0.float().contiguous()
    o, lse_swa, lse_gsa, hkt, hvt = ChunkNativeHybridAttentionFunction.apply(
        flat(q_swa), flat(k_swa), flat(q_gsa), flat(k_gsa), flat(v), flat(s), flat(g), cu, max_seqlen, scale,
        window_size_left, gsa_kv_shift, hk0, hv0, output_final_state, 0)
    o = o.view(B, T, HQ, -1)
    if out_dtype != _BF16:
        o = o.to(out_dtype)
    lse_swa = lse_swa.view(B, T, HQ)
    lse_gsa = lse_gsa.view(B, T, HQ)
    if output_final_state:
        return o, lse_swa, lse_gsa, (hkt, hvt)
    return o, lse_swa, lse_gsa


def chunk_final_state(k_gsa, v, s, g, cu_seqlens, max_seqlen, shift, hk0=None, hv0=None):
    """State pass alone on flat packed ``[Ttot, H, dim]`` bf16 tensors: the fp32 slot memory
    ``(hkt [N,H,K,M], hvt [N,H,M,V])`` after the last token that enters it.  Used by the
    sequence-parallel prefill to summarise a rank's segment before the cross-rank scan."""
    lib = _lib.load()
    geo = _Geometry(k_gsa, k_gsa, v, s, cu_seqlens, max_seqlen)
    dev = geo.device
    sh_t, sh_all = _per_seq(shift, geo.N, dev)
    t = dict(q_gsa=k_gsa, q_swa=k_gsa, k_gsa=k_gsa, k_swa=k_gsa, v=v, s=s, g=g, cu_seqlens=cu_seqlens, hk0=hk0, hv0=hv0)
    t['hkt'] = torch.empty(geo.N, geo.H, geo.K, geo.M, dtype=torch.float32, device=dev)
    t['hvt'] = torch.empty(geo.N, geo.H, geo.M, geo.V, dtype=torch.float32, device=dev)
    t['hk_chunks'] = torch.empty(geo.ncb, geo.H, geo.K, geo.M, dtype=_BF16, device=dev)
    t['hv_chunks'] = torch.empty(geo.ncb, geo.H, geo.M, geo.V, dtype=_BF16, device=dev)
    d = _fill_desc(geo, t, 1.0, None, 0, sh_t, sh_all)
    nbytes = int(lib.nha_chunk_fwd_workspace_bytes(d))
    if nbytes > 0:
        t['workspace'] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        d = _fill_desc(geo, t, 1.0, None, 0, sh_t, sh_all)
    with torch.cuda.device(dev):
        _lib.check(lib.nha_chunk_plan(d, _stream(dev)), 'nha_chunk_plan')
        _lib.check(lib.nha_chunk_state_pass(d, _stream(dev)), 'nha_chunk_state_pass')
    return t['hkt'], t['hvt']


class SegmentForward:
    """The forward of ONE packed sequence in three separately callable steps, for the sequence-parallel prefill: a rank
    summarises its segment with a state pass from a zero start, the ranks exchange the summaries, the rank folds its
    true start state into the chunk-start states, and only then runs the output pass.

    kv-head tensors ``k_gsa, k_swa, v, s, g`` are flat ``[Tkv, H, dim]`` bf16 and may begin with ``q_offset`` tokens
    of the rank before (its last window); ``q_gsa, q_swa`` hold the ``Tkv - q_offset`` positions after them."""

    def __init__(self, q_gsa, q_swa, k_gsa, k_swa, v, s, g, scale, window_left, shift, q_offset=0):
        lib = _lib.load()
        dev = k_gsa.device
        Tkv = k_gsa.shape[0]
        self.cu = torch.zeros(2, dtype=torch.int32, device=dev)      # built by kernels only: legal inside a graph capture
        self.cu[1:].fill_(Tkv)
        self.geo = geo = _Geometry(q_gsa, k_gsa, v, s, self.cu, Tkv, q_offset)
        self.scale, self.wl, self.shift = float(scale), int(window_left), int(shift)
        nq = Tkv - geo.q_offset
        assert q_gsa.shape[0] == nq and q_swa.shape[0] == nq
        H, K, M, V = geo.H, geo.K, geo.M, geo.V
        self.nk, self.nv = H * K * M, H * M * V
        # the segment's message to the other ranks, [L_k | L_v | G]: the state pass writes its end state straight into it
        self.pack = torch.empty(1, self.nk + self.nv + H * M, dtype=torch.float32, device=dev)
        t = dict(q_gsa=q_gsa, q_swa=q_swa, k_gsa=k_gsa, k_swa=k_swa, v=v, s=s, g=g, cu_seqlens=self.cu)
        t['o'] = torch.empty(nq, geo.HQ, V, dtype=_BF16, device=dev)
        t['lse_swa'] = torch.empty(nq, geo.HQ, dtype=torch.float32, device=dev)
        t['lse_gsa'] = torch.empty(nq, geo.HQ, dtype=torch.float32, device=dev)
        t['hkt'] = self.pack[0, :self.nk].view(1, H, K, M)
        t['hvt'] = self.pack[0, self.nk:self.nk + self.nv].view(1, H, M, V)
        t['hk_chunks'] = torch.empty(geo.ncb, H, K, M, dtype=_BF16, device=dev)
        t['hv_chunks'] = torch.empty(geo.ncb, H, M, V, dtype=_BF16, device=dev)
        d = _fill_desc(geo, t, self.scale, None, self.wl, None, self.shift)
        t['workspace'] = torch.empty(max(16, int(lib.nha_chunk_fwd_workspace_bytes(d))), dtype=torch.uint8, device=dev)
        d.workspace = t['workspace'].data_ptr()
        d.workspace_bytes = t['workspace'].numel()
        self.t, self.desc = t, d

    def _halo_chunks(self):
        """Chunks whose shifted rows ``[64 c - shift, 64 c + 64 - shift)`` touch the first ``q_offset`` kv rows."""
        ncb, q_off, shift = self.geo.ncb, self.geo.q_offset, max(0, self.shift)
        if q_off == 0:
            return 0, 0
        lo = max(0, (shift - 64) // 64 + 1)
        hi = min(ncb, -(-(q_off + shift) // 64))
        return min(lo, hi), hi

    def start(self):
        """Plan and the per-chunk terms of every chunk that does not read the first ``q_offset`` kv rows (the rows of
        the rank before): callable while those rows are still arriving."""
        lib, dev = _lib.load(), self.geo.device
        lo, hi = self._halo_chunks()
        with torch.cuda.device(dev):
            _lib.check(lib.nha_chunk_plan(self.desc, _stream(dev)), 'nha_chunk_plan')
            if lo > 0:
                _lib.check(lib.nha_chunk_state_terms(self.desc, 0, lo, _stream(dev)), 'nha_chunk_state_terms')
            _lib.check(lib.nha_chunk_state_terms(self.desc, hi, self.geo.ncb - hi, _stream(dev)), 'nha_chunk_state_terms')
        self._started = True

    def summary(self):
        """The rest of the state pass from a zero start (the terms of the chunks that read the first ``q_offset`` kv
        rows, then the scan; all of it when :meth:`start` was not called).  Returns the segment's message
        ``[1, H*K*M + H*M*V + H*M]`` fp32: its zero-start end state and the total log decay of the tokens that entered
        the slot memory."""
        import ctypes
        lib, dev = _lib.load(), self.geo.device
        with torch.cuda.device(dev):
            if getattr(self, '_started', False):
                lo, hi = self._halo_chunks()
                if hi > lo:
                    _lib.check(lib.nha_chunk_state_terms(self.desc, lo, hi - lo, _stream(dev)), 'nha_chunk_state_terms')
                _lib.check(lib.nha_chunk_state_scan(self.desc, _stream(dev)), 'nha_chunk_state_scan')
                self._started = False
            else:
                _lib.check(lib.nha_chunk_plan(self.desc, _stream(dev)), 'nha_chunk_plan')
                _lib.check(lib.nha_chunk_state_pass(self.desc, _stream(dev)), 'nha_chunk_state_pass')
        ptr = ctypes.c_void_p()
        _lib.check(lib.nha_chunk_gate_totals(self.desc, ctypes.byref(ptr)), 'nha_chunk_gate_totals')
        off = ptr.value - self.t['workspace'].data_ptr()
        hm = self.geo.H * self.geo.M
        self.pack[0, self.nk + self.nv:].copy_(self.t['workspace'][off:off + 4 * hm].view(torch.float32))
        return self.pack

    def fold(self, allp: torch.Tensor, rank: int, initial_state=None):
        """Start state of rank ``rank`` from the all-gathered messages ``allp [world, P]`` (one launch)."""
        lib, dev, g = _lib.load(), self.geo.device, self.geo
        sk = torch.empty(1, g.H, g.K, g.M, dtype=torch.float32, device=dev)
        sv = torch.empty(1, g.H, g.M, g.V, dtype=torch.float32, device=dev)
        hk0 = hv0 = None
        if initial_state is not None and initial_state != (None, None):
            hk0, hv0 = initial_state[0].float().contiguous(), initial_state[1].float().contiguous()
        allp = allp.contiguous()
        with torch.cuda.device(dev):
            _lib.check(lib.nha_sp_fold_start_state(allp.data_ptr(), allp.shape[0], rank, g.H, g.K, g.M, g.V, _lib.ptr(hk0),
                                                   _lib.ptr(hv0), sk.data_ptr(), sv.data_ptr(), _stream(dev)),
                       'nha_sp_fold_start_state')
        return sk, sv

    def fold_from_mailbox(self, box, rank: int, initial_state=None):
        """Start state of rank ``rank`` from the peer-memory mailbox ``box`` (a ``sharding.PeerMailbox`` whose
        ``publish`` ran on this stream for this call): one launch that waits for the ranks before this one."""
        lib, dev, g = _lib.load(), self.geo.device, self.geo
        sk = torch.empty(1, g.H, g.K, g.M, dtype=torch.float32, device=dev)
        sv = torch.empty(1, g.H, g.M, g.V, dtype=torch.float32, device=dev)
        hk0 = hv0 = None
        if initial_state is not None and initial_state != (None, None):
            hk0, hv0 = initial_state[0].float().contiguous(), initial_state[1].float().contiguous()
        err = g.plan.data_ptr() + 4 * (g.N + 1 + g.ncb + g.ncb * g.H)          # the plan's device error word
        with torch.cuda.device(dev):
            _lib.check(lib.nha_sp_fold_wait(box.box.data_ptr(), box.flag.data_ptr(), box.ctr.data_ptr(), box.world, rank,
                                            box.depth, g.H, g.K, g.M, g.V, _lib.ptr(hk0), _lib.ptr(hv0), sk.data_ptr(),
                                            sv.data_ptr(), err, _stream(dev)), 'nha_sp_fold_wait')
        return sk, sv

    def apply_prefix(self, sk: torch.Tensor, sv: torch.Tensor):
        """Fold the true start state ``sk [1,H,K,M], sv [1,H,M,V]`` (fp32) into every chunk-start state and the end state."""
        lib, dev = _lib.load(), self.geo.device
        sk, sv = sk.float().contiguous(), sv.float().contiguous()
        with torch.cuda.device(dev):
            _lib.check(lib.nha_chunk_apply_state_prefix(self.desc, sk.data_ptr(), sv.data_ptr(), _stream(dev)),
                       'nha_chunk_apply_state_prefix')

    def output_pass(self):
        """Output pass; returns ``(o [Tq,HQ,V], lse_swa, lse_gsa, hk, hv)``."""
        lib, dev = _lib.load(), self.geo.device
        with torch.cuda.device(dev):
            _lib.check(lib.nha_chunk_output_pass(self.desc, _stream(dev)), 'nha_chunk_output_pass')
            _lib.check_chunk_device(lib, self.desc, _stream(dev), 'nha_chunk_output_pass')
        t = self.t
        return t['o'], t['lse_swa'], t['lse_gsa'], t['hkt'], t['hvt']
