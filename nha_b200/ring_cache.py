"""Device-resident ring-buffer window cache for decode.

The reference keeps the sliding window of a layer as three tensors that it shifts with ``torch.cat``
on every generated token (``NHACache.update``, nha_fla/models/nha_cache.py:105-126) and hands the
oldest entry to the layer with ``get_pop_kvf`` (:143-154).  Here the window lives in rings of ``W``
rows per sequence and a per-sequence head index, all on the device; a decode step is two launches
(``nha_decode_step_ring`` + ``nha_ring_append``).  Once the rings are full the launches carry no
host-side state, so a step can be captured in a CUDA graph; while a short prompt is still filling them
the host passes the fill level (one integer per layer) and nothing leaves the window, as in the
reference, whose callers feed the op an all-zero entry then (qwennha.py:152-160).  The rings hold the raw (un-rotated) keys, the values and the log-decay rows ``g`` of the
window tokens; the layer computes ``g = logsigmoid(f) / 8`` exactly as it does for the reference op.

:class:`NHARingCache` keeps one ring set per layer and mirrors the parts of the ``NHACache`` surface
that the decode path uses (``get_seq_length``, ``get_pop_kvf``, ``__len__``).
"""
from __future__ import annotations

from typing import List, Optional, Tuple

import torch

from . import _lib
from .fused_recurrent import _decode_workspace, _stream

_BF16 = torch.bfloat16


class RingLayer:
    """Rings, head indices and slot memory of one layer."""

    def __init__(self, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, hk: torch.Tensor, hv: torch.Tensor,
                 window_size: Optional[int] = None, rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None):
        # k [B,T,H,K], v [B,T,H,V], g [B,T,H,M]: the last T <= W tokens, oldest first; hk [B,H,K,M], hv [B,H,M,V] fp32.
        # With T < W the rings are still filling: entries in rows 0 .. T-1, `fill` counts them (host side).
        assert k.dim() == 4 and v.dim() == 4 and g.dim() == 4 and k.shape[:3] == v.shape[:3] == g.shape[:3]
        W = k.shape[1] if window_size is None else int(window_size)
        assert k.shape[1] <= W
        self.fill = k.shape[1]

        def ring(x):
            r = torch.zeros(x.shape[0], W, *x.shape[2:], dtype=_BF16, device=x.device)
            r[:, :x.shape[1]] = x.to(_BF16)
            return r
        self.ring_k, self.ring_v, self.ring_g = ring(k), ring(v), ring(g)
        self.head = torch.zeros(k.shape[0], dtype=torch.int32, device=k.device)
        self.hk = hk.float().contiguous().clone()
        self.hv = hv.float().contiguous().clone()
        # rope = (cos, sin) [1|B, T, K] of the T kept tokens' absolute positions: a second key ring holds the keys
        # rotated on entry, and a decode step then rotates only its own token (rotary by absolute position does
        # not change while the window slides)
        self.ring_kr = None
        if rope is not None:
            cos, sin = (t.to(_BF16).contiguous() for t in rope)
            assert cos.dim() == 3 and cos.shape == sin.shape and cos.shape[1] == self.fill and cos.shape[2] == k.shape[3]
            self.ring_kr = torch.zeros_like(self.ring_k)
            if self.fill:
                cs_batch = cos.stride(0) if cos.shape[0] > 1 else 0
                with torch.cuda.device(k.device):
                    _lib.check(_lib.load().nha_ring_rotate_rows(
                        self.ring_k.data_ptr(), self.ring_kr.data_ptr(), cos.data_ptr(), sin.data_ptr(), cs_batch,
                        cos.stride(1), k.shape[0], k.shape[2], k.shape[3], W, self.fill,
                        torch.cuda.current_stream(k.device).cuda_stream), 'nha_ring_rotate_rows')

    @property
    def window(self) -> int:
        return self.ring_k.shape[1]

    def ordered(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """The window in time order (oldest first), as the reference cache would hold it (copies)."""
        W = self.window
        if self.fill < W:
            return self.ring_k[:, :self.fill].clone(), self.ring_v[:, :self.fill].clone(), self.ring_g[:, :self.fill].clone()
        idx = (self.head.long()[:, None] + torch.arange(W, device=self.head.device)[None]) % W
        gather = lambda r: torch.gather(r, 1, idx[:, :, None, None].expand(-1, -1, *r.shape[2:]))
        return gather(self.ring_k), gather(self.ring_v), gather(self.ring_g)


def fused_recurrent_nha_decode_ring(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, layer: RingLayer,
                                    cos: torch.Tensor, sin: torch.Tensor, scale: Optional[float] = None) -> torch.Tensor:
    """One decode step on a ring cache: returns ``o [B,1,HQ,V]``; the layer's state and rings are updated.

    ``q [B,1,HQ,K]``, ``k [B,1,H,K]`` (raw), ``v [B,1,H,V]``, ``g [B,1,H,M]`` (log decay of the new token),
    ``cos/sin [1|B, W, K]`` for the W window positions (row W-1 = the query's position); while the rings are
    still filling (``layer.fill < W``) the window is ``layer.fill + 1`` long and so are the tables.
    """
    lib = _lib.load()
    B, one, HQ, K = q.shape
    if one != 1:
        raise ValueError('decode takes one token per sequence')
    H, V, M, W = k.shape[2], v.shape[3], g.shape[3], layer.window
    fill = layer.fill
    wlen = W if fill >= W else fill + 1
    if layer.ring_kr is not None:
        return _decode_ring_rot(q, k, v, g, layer, cos, sin, scale)
    assert cos.shape[-2] == wlen and cos.shape[-1] == K, 'cos/sin must cover the window positions'
    dev = q.device
    qc, kc, vc, gc = (x.to(_BF16).contiguous() for x in (q, k, v, g))
    cosc, sinc = cos.to(_BF16).contiguous(), sin.to(_BF16).contiguous()
    cs_batch = cosc.stride(0) if (cosc.dim() == 3 and cosc.shape[0] > 1) else 0
    o = torch.empty(B, 1, HQ, V, dtype=_BF16, device=dev)
    sc = float(K ** -0.5 if scale is None else scale)
    with torch.cuda.device(dev):                       # split count and launches follow the tensors' device
        ws = _decode_workspace(dev, B, HQ, H, V, W)
        st = _stream(dev)
        _lib.check(lib.nha_decode_step_ring(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), layer.ring_k.data_ptr(),
                                            layer.ring_v.data_ptr(), layer.ring_g.data_ptr(), layer.head.data_ptr(),
                                            cosc.data_ptr(), sinc.data_ptr(), cs_batch, cosc.stride(-2),
                                            layer.hk.data_ptr(), layer.hv.data_ptr(), o.data_ptr(), ws.data_ptr(),
                                            ws.numel(), B, HQ, H, K, V, M, W, fill, sc, st), 'nha_decode_step_ring')
        _lib.check(lib.nha_ring_append(layer.ring_k.data_ptr(), layer.ring_v.data_ptr(), layer.ring_g.data_ptr(),
                                       kc.data_ptr(), vc.data_ptr(), gc.data_ptr(), layer.head.data_ptr(), B, H, K, V, M,
                                       W, fill, st), 'nha_ring_append')
        _lib.check_decode_device(lib, ws, B, H, st, 'nha_decode_step_ring')
    layer.fill = min(fill + 1, W)
    return o


def _decode_ring_rot(q, k, v, g, layer: RingLayer, cos, sin, scale) -> torch.Tensor:
    """Decode step on rings whose keys were rotated on entry: only the last row of ``cos/sin [1|B, >=1, K]`` (the
    position of this step's token) is read."""
    lib = _lib.load()
    B, _, HQ, K = q.shape
    H, V, M, W = k.shape[2], v.shape[3], g.shape[3], layer.window
    assert cos.shape[-1] == K and cos.shape == sin.shape
    dev = q.device
    qc, kc, vc, gc = (x.to(_BF16).contiguous() for x in (q, k, v, g))
    cosq, sinq = cos[:, -1].to(_BF16).contiguous(), sin[:, -1].to(_BF16).contiguous()        # [1|B, K]
    cs_batch = cosq.stride(0) if cosq.shape[0] > 1 else 0
    sc = float(scale) if scale is not None else K ** -0.5
    o = torch.empty(B, 1, HQ, V, device=dev, dtype=_BF16)
    fill = layer.fill
    with torch.cuda.device(dev):
        ws = _decode_workspace(dev, B, HQ, H, V, W)
        st = _stream(dev)
        _lib.check(lib.nha_decode_step_ring_rot(qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), layer.ring_k.data_ptr(),
                                                layer.ring_kr.data_ptr(), layer.ring_v.data_ptr(), layer.ring_g.data_ptr(),
                                                layer.head.data_ptr(), cosq.data_ptr(), sinq.data_ptr(), cs_batch,
                                                layer.hk.data_ptr(), layer.hv.data_ptr(), o.data_ptr(), ws.data_ptr(),
                                                ws.numel(), B, HQ, H, K, V, M, W, fill, sc, st),
                   'nha_decode_step_ring_rot')
        _lib.check(lib.nha_ring_append_rot(layer.ring_k.data_ptr(), layer.ring_kr.data_ptr(), layer.ring_v.data_ptr(),
                                           layer.ring_g.data_ptr(), kc.data_ptr(), vc.data_ptr(), gc.data_ptr(),
                                           cosq.data_ptr(), sinq.data_ptr(), cs_batch, layer.head.data_ptr(), B, H, K, V,
                                           M, W, fill, st), 'nha_ring_append_rot')
        _lib.check_decode_device(lib, ws, B, H, st, 'nha_decode_step_ring_rot')
    layer.fill = min(fill + 1, W)
    return o


class NHARingCache:
    """Per-layer ring caches with the read-side surface of the reference's ``NHACache``."""

    def __init__(self, seen_tokens: int = 0):
        self.layers: List[Optional[RingLayer]] = []
        self._seen_tokens = seen_tokens

    def __len__(self) -> int:
        return len(self.layers)

    def __getitem__(self, layer_idx: int) -> RingLayer:
        if layer_idx < len(self.layers) and self.layers[layer_idx] is not None:
            return self.layers[layer_idx]
        raise KeyError(f'Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}')

    def init_layer(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, window_size: int,
                   recurrent_state: Tuple[torch.Tensor, torch.Tensor],
                   rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> RingLayer:
        """Fill a layer from its prefill: ``k, v, g [B,T,H,*]`` (the last ``window_size`` tokens are kept, as
        ``NHACache.update`` does; a shorter prompt leaves the rings partly filled) and the slot memory after the
        prefill.  With ``rope = (cos, sin) [1|B, T, K]`` (tables of the T tokens' absolute positions) the layer also
        keeps the keys rotated on entry, and ``decode`` then needs only the table row of the new token's position
        (the last row of what it is given); rotary positions must be absolute for this layout."""
        if rope is not None:
            rope = tuple(t[:, -window_size:] for t in rope)
        while len(self.layers) <= layer_idx:
            self.layers.append(None)
        layer = RingLayer(k[:, -window_size:], v[:, -window_size:], g[:, -window_size:], *recurrent_state,
                          window_size=window_size, rope=rope)
        self.layers[layer_idx] = layer
        return layer

    def decode(self, layer_idx: int, q, k, v, g, cos, sin, scale=None) -> torch.Tensor:
        if layer_idx == 0:
            self._seen_tokens += 1
        return fused_recurrent_nha_decode_ring(q, k, v, g, self[layer_idx], cos, sin, scale)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen_tokens if layer_idx < len(self.layers) else 0

    def get_pop_kvf(self, layer_idx: int, window_size: int):
        """The oldest window entry ``(k, v, g)`` as ``[B,1,H*D]`` views' equivalents (copies), or Nones."""
        if layer_idx >= len(self.layers) or self.layers[layer_idx] is None:
            return (None, None, None)
        L = self.layers[layer_idx]
        if L.fill < L.window:
            return (None, None, None)                 # as NHACache: nothing leaves a window that is not full
        b = torch.arange(L.head.shape[0], device=L.head.device)
        pick = lambda r: r[b, L.head.long()].reshape(r.shape[0], 1, -1)
        return pick(L.ring_k), pick(L.ring_v), pick(L.ring_g)
