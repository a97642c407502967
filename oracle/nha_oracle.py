"""CPU oracle for the NHA attention operator (TEST INFRASTRUCTURE, not product code).

This module restates, in plain fp64 PyTorch, the arithmetic of the reference's
naive implementation of Native Hybrid Attention.  It exists only to check the
CUDA kernels: nothing under ``nha_b200/`` imports it, and the product path
never falls back to it.  Only ``tests/``, ``__graft_entry__.smoke()`` and the
``cpu_baseline`` / ``--impl reference`` legs of ``bench.py`` may call it.

Parity pinning: every function here is checked against the reference's own
fp64 functions ``ref_gsa_step`` / ``ref_decode`` / ``ref_fused_recurrent`` /
``ref_prefill`` (``scripts/verify_opt_parity.py:76-191``) on the reference's
case grids by ``tests/golden/make_golden.py``; the outputs of those reference
functions are committed as fixtures under ``tests/golden/`` and re-checked by
``tests/test_oracle.py``.  The training op ``chunk_nha`` has no CPU
implementation in the reference (its arithmetic lives in the third-party
``flash-attn`` and ``flash-linear-attention 0.5.1`` GPU kernels), so for the
overlapping window convention and for gradients the pin is a CPU replay of
``nha_fla/ops/nha/chunk.py:401-470`` built from the reference's shift helpers,
``fla.ops.gsa.naive.naive_recurrent_gsa`` and a masked softmax (same script).

Semantics (per sequence, per kv head ``h``; ``NG = HQ // H`` query heads share
kv head ``q // NG``), following ``scripts/verify_opt_parity.py:81-83,176-190``
and the merge in ``nha_fla/ops/nha/chunk.py:458-470``::

    j = t - shift
    if j >= 0:   hk[:, m] = hk[:, m] * exp(g[j, m]) + k_gsa[j] * s[j, m]
                 hv[m, :] = hv[m, :] * exp(g[j, m]) + s[j, m] * v[j]
    ok[m] = scale * <q_gsa[t], hk[:, m]>
    sw[w] = scale * <q_swa[t], k_swa[w]>      for w in [max(0, t - window_left), t]
    p     = softmax(concat(ok, sw))
    o[t]  = sum_m p[m] hv[m, :] + sum_w p[M + w] v[w]
    lse_gsa[t] = logsumexp(ok),  lse_swa[t] = logsumexp(sw)
"""
from __future__ import annotations

from typing import Optional, Sequence, Tuple

import torch

__all__ = [
    "rope_rotate_half",
    "gsa_step",
    "nha_sequence",
    "nha_varlen",
    "nha_batched",
    "prefill",
    "decode_step",
    "recurrent_step",
    "slot_gates",
    "feature_maps",
    "silu_rms_norm",
    "rotary_positions",
    "gsa_aux",
    "rel_l2",
]


def rel_l2(a: torch.Tensor, b: torch.Tensor) -> float:
    """Relative L2 error of ``a`` against the truth ``b`` (scripts/verify_opt_parity.py:57-60)."""
    a = a.detach().double().flatten()
    b = b.detach().double().flatten()
    return (a - b).norm().item() / max(b.norm().item(), 1e-30)


def rope_rotate_half(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """HF rotate-half rotary on ``[..., T, H, K]`` with duplicated-halves tables ``[..., T, K]``
    (scripts/verify_opt_parity.py:48-54, 111-114)."""
    x1, x2 = x.chunk(2, dim=-1)
    rot = torch.cat([-x2, x1], dim=-1)
    return x * cos.unsqueeze(-2) + rot * sin.unsqueeze(-2)


def gsa_step(hk, hv, k, v, s, g):
    """One slot-memory update (scripts/verify_opt_parity.py:81-83).

    hk [H,K,M], hv [H,M,V]; k [H,K], v [H,V], s/g [H,M]."""
    eg = g.exp()
    hk = hk * eg[:, None, :] + k[:, :, None] * s[:, None, :]
    hv = hv * eg[:, :, None] + s[:, :, None] * v[:, None, :]
    return hk, hv


def nha_sequence(
    q_gsa: torch.Tensor,
    q_swa: torch.Tensor,
    k_gsa: torch.Tensor,
    k_swa: torch.Tensor,
    v: torch.Tensor,
    s: torch.Tensor,
    g: torch.Tensor,
    scale: float,
    window_left: int,
    shift: int,
    hk0: Optional[torch.Tensor] = None,
    hv0: Optional[torch.Tensor] = None,
):
    """NHA over ONE sequence, token by token, in fp64 and differentiable.

    q_* [T,HQ,K]; k_* [T,H,K]; v [T,H,V]; s,g [T,H,M]; hk0 [H,K,M]; hv0 [H,M,V].
    ``window_left < 0`` means an unbounded causal window.
    Returns ``o [T,HQ,V], lse_swa [T,HQ], lse_gsa [T,HQ], hkt, hvt``.
    Follows scripts/verify_opt_parity.py:147-191 with the window/shift made
    independent as in nha_fla/ops/nha/chunk.py:579-581.
    """
    dd = torch.float64
    q_gsa, q_swa, k_gsa, k_swa, v, s, g = (x.to(dd) for x in (q_gsa, q_swa, k_gsa, k_swa, v, s, g))
    T, HQ, K = q_gsa.shape
    H = k_gsa.shape[1]
    M = s.shape[-1]
    V = v.shape[-1]
    NG = HQ // H
    hk = torch.zeros(H, K, M, dtype=dd) if hk0 is None else hk0.to(dd)
    hv = torch.zeros(H, M, V, dtype=dd) if hv0 is None else hv0.to(dd)
    outs, lses, lseg = [], [], []
    for t in range(T):
        j = t - shift
        if j >= 0:
            hk, hv = gsa_step(hk, hv, k_gsa[j], v[j], s[j], g[j])
        hkq = hk.repeat_interleave(NG, dim=0)                       # [HQ,K,M]
        hvq = hv.repeat_interleave(NG, dim=0)                       # [HQ,M,V]
        ok = torch.einsum('qk,qkm->qm', q_gsa[t] * scale, hkq)      # [HQ,M]
        lo = 0 if window_left < 0 else max(0, t - window_left)
        kw = k_swa[lo:t + 1].repeat_interleave(NG, dim=1)            # [w,HQ,K]
        vw = v[lo:t + 1].repeat_interleave(NG, dim=1)                # [w,HQ,V]
        sw = torch.einsum('qk,wqk->qw', q_swa[t] * scale, kw)        # [HQ,w]
        z = torch.cat([ok, sw], dim=-1)
        p = torch.softmax(z, dim=-1)
        o = torch.einsum('qm,qmv->qv', p[:, :M], hvq) + torch.einsum('qw,wqv->qv', p[:, M:], vw)
        outs.append(o)
        lseg.append(torch.logsumexp(ok, dim=-1))
        lses.append(torch.logsumexp(sw, dim=-1))
    return torch.stack(outs), torch.stack(lses), torch.stack(lseg), hk, hv


def nha_varlen(
    q_gsa, q_swa, k_gsa, k_swa, v, s, g,
    cu_seqlens: Sequence[int],
    scale: float,
    window_left,
    shift,
    hk0: Optional[torch.Tensor] = None,
    hv0: Optional[torch.Tensor] = None,
):
    """Packed sequences ``[Ttot, H*, *]`` with boundaries ``cu_seqlens``.

    ``window_left`` / ``shift`` are ints or per-sequence lists.  Each sequence is
    independent (its own zero or given initial state), which is what the
    reference's packed shift + varlen kernels compute
    (nha_fla/ops/nha/chunk.py:53-77, 423-445).  Returns flat outputs and stacked
    final states ``[N,H,K,M] / [N,H,M,V]``.
    """
    cu = [int(x) for x in cu_seqlens]
    N = len(cu) - 1
    wl = list(window_left) if hasattr(window_left, '__len__') else [int(window_left)] * N
    sh = list(shift) if hasattr(shift, '__len__') else [int(shift)] * N
    os_, ls_, lg_, hks, hvs = [], [], [], [], []
    for n in range(N):
        a, b = cu[n], cu[n + 1]
        o, ls, lg, hk, hv = nha_sequence(
            q_gsa[a:b], q_swa[a:b], k_gsa[a:b], k_swa[a:b], v[a:b], s[a:b], g[a:b],
            scale, int(wl[n]), int(sh[n]),
            None if hk0 is None else hk0[n], None if hv0 is None else hv0[n])
        os_.append(o); ls_.append(ls); lg_.append(lg); hks.append(hk); hvs.append(hv)
    return torch.cat(os_), torch.cat(ls_), torch.cat(lg_), torch.stack(hks), torch.stack(hvs)


def nha_batched(q_gsa, q_swa, k_gsa, k_swa, v, s, g, scale, window_left, shift, hk0=None, hv0=None):
    """Equal-length batch ``[B,T,H*,*]`` -> ``o [B,T,HQ,V], lse_swa, lse_gsa [B,T,HQ], hkt, hvt``."""
    B = q_gsa.shape[0]
    res = [nha_sequence(q_gsa[b], q_swa[b], k_gsa[b], k_swa[b], v[b], s[b], g[b], scale, window_left, shift,
                        None if hk0 is None else hk0[b], None if hv0 is None else hv0[b]) for b in range(B)]
    return tuple(torch.stack([r[i] for r in res]) for i in range(5))


def prefill(q, k, v, rotary_q, rotary_k, s, g, window_size: int, scale: float, hk0=None, hv0=None):
    """``fused_chunk_nha_prefill`` semantics (nha_fla/ops/nha/chunk_fused.py:291-380 and
    scripts/verify_opt_parity.py:147-191): window ``[t-W+1, t]``, slot memory holds tokens ``<= t-W``.

    q/rotary_q [B,T,HQ,K]; k/rotary_k [B,T,H,K]; v [B,T,H,V]; s,g [B,T,H,M].
    Returns ``o [B,T,HQ,V], hkt [B,H,K,M], hvt [B,H,M,V]`` (fp64)."""
    o, _, _, hkt, hvt = nha_batched(q, rotary_q, k, rotary_k, v, s, g, scale, window_size - 1, window_size, hk0, hv0)
    return o, hkt, hvt


def decode_step(q, k, v, g, sw_k, sw_v, scale: float, sq=None, s=None, cos=None, sin=None, hk0=None, hv0=None):
    """``fused_recurrent_nha_decode`` semantics (nha_fla/ops/nha/fused_recurrent.py:431-584,
    scripts/verify_opt_parity.py:88-125).

    q [B,1,HQ,K] raw; popped k [B,1,H,K], v [B,1,H,V], g [B,1,H,M]; window sw_k [B,W,H,K]
    (raw if cos/sin given, else pre-rotated), sw_v [B,W,H,V]; ``sq`` pre-rotated query or
    ``cos/sin [1|B, W2>=W, K]`` whose last W rows are the window positions (row W-1 = query).
    ``s`` defaults to ``1 - exp(g)``.  Returns ``o [B,1,HQ,V], hkt, hvt, p_slot [B,HQ,M], p_win [B,HQ,W]``.
    """
    dd = torch.float64
    q, k, v, g, sw_k, sw_v = (x.to(dd) for x in (q, k, v, g, sw_k, sw_v))
    B, _, HQ, K = q.shape
    W, H = sw_k.shape[1], sw_k.shape[2]
    M, V = g.shape[-1], v.shape[-1]
    NG = HQ // H
    s = (1.0 - g.exp()) if s is None else s.to(dd)
    if cos is not None:
        cos, sin = cos.to(dd)[:, -W:], sin.to(dd)[:, -W:]
        sqd = rope_rotate_half(q, cos[:, -1:], sin[:, -1:])
        skd = rope_rotate_half(sw_k, cos, sin)
    else:
        sqd, skd = sq.to(dd), sw_k
    hk = torch.zeros(B, H, K, M, dtype=dd) if hk0 is None else hk0.to(dd)
    hv = torch.zeros(B, H, M, V, dtype=dd) if hv0 is None else hv0.to(dd)
    eg = g[:, 0].exp()
    hk1 = hk * eg[:, :, None, :] + k[:, 0][:, :, :, None] * s[:, 0][:, :, None, :]
    hv1 = hv * eg[:, :, :, None] + s[:, 0][:, :, :, None] * v[:, 0][:, :, None, :]
    ok = torch.einsum('bqk,bqkm->bqm', q[:, 0] * scale, hk1.repeat_interleave(NG, dim=1))
    sw = torch.einsum('bqk,bwqk->bqw', sqd[:, 0] * scale, skd.repeat_interleave(NG, dim=2))
    p = torch.softmax(torch.cat([ok, sw], dim=-1), dim=-1)
    ps, pw = p[..., :M], p[..., M:]
    o = torch.einsum('bqm,bqmv->bqv', ps, hv1.repeat_interleave(NG, dim=1)) \
        + torch.einsum('bqw,bwqv->bqv', pw, sw_v.repeat_interleave(NG, dim=2))
    return o[:, None], hk1, hv1, ps, pw


def recurrent_step(q, k, v, sliding_window, s, g, scale: float, hk0=None, hv0=None):
    """``fused_recurrent_nha`` semantics (nha_fla/ops/nha/fused_recurrent.py:588-682,
    scripts/verify_opt_parity.py:128-144): the caller supplies the window logits
    ``[B,1,HQ,W]``; the op returns the slot-only readout, the window probabilities
    and the updated states."""
    dd = torch.float64
    q, k, v, sw, s, g = (x.to(dd) for x in (q, k, v, sliding_window, s, g))
    B, _, HQ, K = q.shape
    H = k.shape[2]
    M, V = s.shape[-1], v.shape[-1]
    NG = HQ // H
    hk = torch.zeros(B, H, K, M, dtype=dd) if hk0 is None else hk0.to(dd)
    hv = torch.zeros(B, H, M, V, dtype=dd) if hv0 is None else hv0.to(dd)
    eg = g[:, 0].exp()
    hk1 = hk * eg[:, :, None, :] + k[:, 0][:, :, :, None] * s[:, 0][:, :, None, :]
    hv1 = hv * eg[:, :, :, None] + s[:, 0][:, :, :, None] * v[:, 0][:, :, None, :]
    ok = torch.einsum('bqk,bqkm->bqm', q[:, 0] * scale, hk1.repeat_interleave(NG, dim=1))
    p = torch.softmax(torch.cat([ok, sw[:, 0]], dim=-1), dim=-1)
    ps, pw = p[..., :M], p[..., M:]
    o = torch.einsum('bqm,bqmv->bqv', ps, hv1.repeat_interleave(NG, dim=1))
    return o[:, None], pw[:, None], hk1, hv1


def slot_gates(f: torch.Tensor, normalizer: float = 8.0) -> Tuple[torch.Tensor, torch.Tensor]:
    """The callers' gate chain in fp64: ``g = logsigmoid(f) / normalizer``, ``s = 1 - exp(g)``
    (nha_fla/layers/nha.py:229-231; differentiable through autograd)."""
    g = torch.nn.functional.logsigmoid(f.double()) / normalizer
    return g, -torch.expm1(g)


def rotary_positions(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, positions: torch.Tensor) -> torch.Tensor:
    """Non-interleaved rotary of ``x [T, H, K]`` in fp64 with tables ``cos, sin [P, K/2]`` and one table row per
    token (``positions [T]``): the layer's ``self.rotary(q, k, seqlen_offset)`` (nha_fla/layers/nha.py:145,235), whose
    arithmetic is the third-party ``fla.modules.rotary.rotary_embedding_ref`` (flash-linear-attention 0.5.1):
    ``o[:K/2] = x[:K/2] cos - x[K/2:] sin``, ``o[K/2:] = x[:K/2] sin + x[K/2:] cos``."""
    x = x.double()
    R = x.shape[-1] // 2
    c = cos.double()[positions, None, :R]
    s = sin.double()[positions, None, :R]
    x0, x1 = x[..., :R], x[..., R:]
    return torch.cat([x0 * c - x1 * s, x0 * s + x1 * c], -1)


def feature_maps(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, feature_map: str = 'swish'):
    """The layer's feature map on q and k and ``silu`` on v in fp64 (nha_fla/layers/nha.py:219-223; the 'swish'
    feature map of flash-linear-attention 0.5.1 is ``x * sigmoid(x)``, 'relu' is ``max(x, 0)``)."""
    act = (lambda x: x * torch.sigmoid(x)) if feature_map == 'swish' else torch.relu
    q, k, v = q.double(), k.double(), v.double()
    return act(q), act(k), v * torch.sigmoid(v)


def silu_rms_norm(o: torch.Tensor, weight: torch.Tensor, bias=None, eps: float = 1e-5) -> torch.Tensor:
    """``rms_norm(silu(o)) * weight + bias`` over the last dimension in fp64: what the layer's
    ``rms_norm_linear(F.silu(o), ...)`` computes in front of its projection (nha_fla/layers/nha.py:277-278;
    flash-linear-attention 0.5.1 ``layer_norm_linear(..., is_rms_norm=True)``, eps 1e-5)."""
    x = o.double()
    x = x * torch.sigmoid(x)
    y = x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + eps) * weight.double()
    return y if bias is None else y + bias.double()


def gsa_aux(lse_swa: torch.Tensor, lse_gsa: torch.Tensor, target: float) -> Tuple[torch.Tensor, torch.Tensor]:
    """The training layer's two scalars in fp64 (nha_fla/layers/nha.py:255-264, 288-313): the aux loss
    ``mean(BCE_with_logits(lse_gsa - lse_swa.detach(), target))`` (differentiable in ``lse_gsa``) and the monitoring
    ratio ``mean(w_gsa / (w_swa + w_gsa))`` with ``w_x = exp(lse_x - max(lse_swa, lse_gsa))``."""
    ls, lg = lse_swa.double().detach(), lse_gsa.double()
    d = lg - ls
    loss = (d.clamp(min=0) - d * target + torch.log1p(torch.exp(-d.abs()))).mean()
    mx = torch.maximum(ls, lg.detach())
    ws, wg = (ls - mx).exp(), (lg.detach() - mx).exp()
    return loss, (wg / (ws + wg)).mean()
