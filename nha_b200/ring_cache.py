"""Device-resident ring-buffer window cache for decode.

The reference keeps the sliding window of a layer as three tensors that it shifts with ``torch.cat``
on every generated token (``NHACache.update``, nha_fla/models/nha_cache.py:105-126) and hands the
oldest entry to the layer with ``get_pop_kvf`` (:143-154).  Here the window lives in rings of ``W``
rows per sequence and an index of the oldest entry, all on the device; a decode step is ONE launch
(``nha_decode_step_ring_fused``: the CTA that finishes a (sequence, kv head) also stores the step's token over the
entry that left the window; with ``fused=False`` two launches, ``nha_decode_step_ring`` + ``nha_ring_append``).  Once the rings are full the launches carry no
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
                 window_size: Optional[int] = None, rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
                 fused: bool = True):
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
        # fused: the decode kernel also appends the step's token (one launch per step); the index of the oldest entry
        # is then kept per (sequence, kv head), [B, H] with equal entries along H, because each (sequence, kv head) is
        # finished - and advanced - by its own CTA.  Otherwise one index per sequence and a separate append launch.
        self.fused = bool(fused) and rope is None
        self.head = torch.zeros((k.shape[0], k.shape[2]) if self.fused else (k.shape[0],), dtype=torch.int32,
                                device=k.device)
        self.hk = None if hk is None else hk.float().contiguous().clone()
        self.hv = None if hv is None else hv.float().contiguous().clone()
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

    conv_state = None
    ffn_state = None

    def __getitem__(self, key: str):
        """The reference cache hands its callers a dict per layer (nha_fla/models/nha_cache.py:31-35); the same keys read
        from the rings: ``recurrent_state`` -> ``(hk, hv)``, ``attn_state`` -> the window in time order, flattened to
        ``[B, fill, H*D]`` as the reference stores it (copies)."""
        if key == 'recurrent_state':
            return None if self.hk is None else (self.hk, self.hv)
        if key == 'attn_state':
            return tuple(x.flatten(2) for x in self.ordered())
        if key in ('conv_state', 'ffn_state'):
            return getattr(self, key)
        raise KeyError(key)

    def as_dict(self) -> dict:
        return {k: self[k] for k in ('recurrent_state', 'attn_state', 'conv_state', 'ffn_state')}

    def set_state(self, recurrent_state) -> None:
        hk, hv = recurrent_state
        if self.hk is not None and hk.data_ptr() == self.hk.data_ptr() and hv.data_ptr() == self.hv.data_ptr():
            return                                     # the kernels already updated the layer's own tensors in place
        self.hk, self.hv = hk.float().contiguous().clone(), hv.float().contiguous().clone()

    def append(self, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor) -> None:
        """Append ``n < W`` tokens ``[B,n,H,*]`` (oldest first) without a decode step: index arithmetic in torch, for
        callers that drive the cache through ``update`` as they drive the reference cache.  Rings with keys rotated on
        entry are appended to by their decode step only."""
        assert self.ring_kr is None, 'a ring with rotated keys is advanced by its decode step'
        W, n = self.window, k.shape[1]
        assert n < W
        if self.fill + n > W:                          # the prompt's tail and the new tokens together: keep the last W
            ok, ov, og = self.ordered()
            cat = lambda a, b: torch.cat([a, b.to(_BF16).reshape(b.shape[0], n, *a.shape[2:])], 1)[:, -W:]
            self.ring_k, self.ring_v, self.ring_g = (cat(a, b).contiguous() for a, b in ((ok, k), (ov, v), (og, g)))
            self.head.zero_()
            self.fill = W
            return
        if self.fill < W:
            rows = torch.arange(self.fill, self.fill + n, device=self.head.device)[None].expand(self.head.shape[0], -1)
        else:
            rows = (self.oldest()[:, None] + torch.arange(n, device=self.head.device)[None]) % W
        b = torch.arange(self.head.shape[0], device=self.head.device)[:, None]
        for ring, x in ((self.ring_k, k), (self.ring_v, v), (self.ring_g, g)):
            ring[b, rows] = x.to(_BF16).reshape(x.shape[0], n, *ring.shape[2:])
        if self.fill < W:
            self.fill += n
        else:
            self.head.copy_((self.head + n) % W)

    def oldest(self) -> torch.Tensor:
        """Row of the oldest entry per sequence, ``[B]`` int64."""
        return (self.head if self.head.dim() == 1 else self.head[:, 0]).long()

    def ordered(self) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
        """The window in time order (oldest first), as the reference cache would hold it (copies)."""
        W = self.window
        if self.fill < W:
            return self.ring_k[:, :self.fill].clone(), self.ring_v[:, :self.fill].clone(), self.ring_g[:, :self.fill].clone()
        idx = (self.oldest()[:, None] + torch.arange(W, device=self.head.device)[None]) % W
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
        if layer.fused:
            if layer.head.shape[1] != H:               # rings made through update(): the kv-head count is known only now
                layer.head = layer.head[:, :1].repeat(1, H)
            _lib.check(lib.nha_decode_step_ring_fused(
                qc.data_ptr(), kc.data_ptr(), vc.data_ptr(), gc.data_ptr(), layer.ring_k.data_ptr(), layer.ring_v.data_ptr(),
                layer.ring_g.data_ptr(), layer.head.data_ptr(), cosc.data_ptr(), sinc.data_ptr(), cs_batch, cosc.stride(-2),
                layer.hk.data_ptr(), layer.hv.data_ptr(), o.data_ptr(), ws.data_ptr(), ws.numel(), B, HQ, H, K, V, M, W, fill,
                sc, st), 'nha_decode_step_ring_fused')
        else:
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
    """Per-layer ring caches with the surface of the reference's ``NHACache`` (nha_fla/models/nha_cache.py:11-182).

    Two ways to drive it.  A caller written against the rings uses :meth:`init_layer` after the prefill and
    :meth:`decode` per token (two launches, nothing shifted).  A caller written against the reference cache keeps its
    calls - ``get_pop_kvf``, ``update(attn_state=...)``, ``update(recurrent_state=...)``, ``get_seq_length``,
    ``cache[layer]['recurrent_state']`` - and gets the reference's answers (the window comes back in time order,
    gathered from the ring, which costs what the reference's ``torch.cat`` costs).  One deviation: a window that is
    not yet full and receives more tokens than it has room for keeps the newest ``window_size`` tokens, where the
    reference's cat lets that layer's cache grow past ``window_size`` for good (nha_cache.py:127-131)."""

    def __init__(self, seen_tokens: int = 0):
        self.layers: List[Optional[RingLayer]] = []
        self.former_tokens = seen_tokens
        self._seen_tokens = seen_tokens

    def __len__(self) -> int:
        return len(self.layers)

    def __iter__(self):
        for layer in self.layers:
            yield layer

    def update(self, recurrent_state=None, attn_state=None, conv_state=None, ffn_state=None, layer_idx: int = 0,
               offset: Optional[int] = 1, cache_kwargs: Optional[dict] = None) -> dict:
        """``NHACache.update`` (nha_cache.py:44-141) on rings: same arguments, same returned dict.  ``attn_state`` is
        ``(k, v, g)`` of the new tokens, ``[B, n, H*D]`` (or ``[B, n, H, D]``), ``cache_kwargs['window_size']`` the
        window.  The first call for a layer keeps the last ``window_size`` tokens; later calls slide the window; a chunk
        longer than the window replaces it and is handed back whole, as the reference does."""
        if layer_idx == 0:
            self.former_tokens = self._seen_tokens
            self._seen_tokens += offset
        W = None
        if attn_state is not None:
            if not isinstance(attn_state, tuple) or len(attn_state) != 3:
                raise ValueError('`attn_state` must be a tuple of three tensors (key, value, gate states)')
            W = (cache_kwargs or {}).get('window_size', None)
            if W is None:
                raise ValueError("a ring needs its size: pass cache_kwargs={'window_size': W}")
            n = attn_state[0].shape[1]
        four_d = lambda x: x if x.dim() == 4 else x.unsqueeze(2)        # head split unknown here: one "head" of H*D
        hand_back = None
        if len(self.layers) <= layer_idx or self.layers[layer_idx] is None:
            while len(self.layers) <= layer_idx:
                self.layers.append(None)
            if attn_state is None:
                raise ValueError('the first update of a layer must bring its window (attn_state)')
            k, v, g = (four_d(x)[:, -W:] for x in attn_state)
            rs = recurrent_state if recurrent_state is not None else (None, None)
            layer = self.layers[layer_idx] = RingLayer(k, v, g, rs[0], rs[1], window_size=W)
        else:
            layer = self.layers[layer_idx]
            if recurrent_state is not None:
                layer.set_state(recurrent_state)
            if attn_state is not None:
                assert W == layer.window, 'the window size of a layer is fixed by its first update'
                k, v, g = (four_d(x) for x in attn_state)
                if n >= W:
                    fresh = RingLayer(k[:, -W:], v[:, -W:], g[:, -W:], layer.hk, layer.hv, window_size=W)
                    layer.ring_k, layer.ring_v, layer.ring_g = fresh.ring_k, fresh.ring_v, fresh.ring_g
                    layer.head.zero_()
                    was_full, layer.fill = layer.fill == W, W
                    if was_full and n > W:
                        hand_back = attn_state                           # nha_cache.py:106-118
                else:
                    layer.append(k, v, g)
        if conv_state is not None:
            layer.conv_state = conv_state
        if ffn_state is not None:
            layer.ffn_state = ffn_state
        state = layer.as_dict()
        if attn_state is not None and attn_state[0].dim() == 4:
            state['attn_state'] = tuple(x.view(x.shape[0], x.shape[1], *y.shape[2:])
                                        for x, y in zip(state['attn_state'], attn_state))
        if hand_back is not None:
            state['attn_state'] = hand_back
        return state

    def get_max_length(self) -> Optional[int]:
        return None

    def to_legacy_cache(self) -> tuple:
        return tuple(None if layer is None else layer.as_dict() for layer in self.layers)

    @classmethod
    def from_legacy_cache(cls, past_key_values=None, seen_tokens: int = 0, window_size: Optional[int] = None):
        """From the reference cache's list of per-layer dicts (nha_cache.py:170-182).  ``window_size`` sizes the rings;
        without it each layer's ring is as long as its stored window."""
        cache = cls(seen_tokens)
        if isinstance(past_key_values, (list, tuple)):
            for i, st in enumerate(past_key_values):
                if st is None or st.get('attn_state') is None:
                    cache.layers.append(None)
                    continue
                W = window_size or st['attn_state'][0].shape[1]
                cache.update(attn_state=tuple(st['attn_state']), recurrent_state=st.get('recurrent_state'), layer_idx=i,
                             offset=0, cache_kwargs={'window_size': W})
                cache.layers[i].conv_state, cache.layers[i].ffn_state = st.get('conv_state'), st.get('ffn_state')
        return cache

    def __getitem__(self, layer_idx: int) -> RingLayer:
        if layer_idx < len(self.layers) and self.layers[layer_idx] is not None:
            return self.layers[layer_idx]
        raise KeyError(f'Cache only has {len(self)} layers, attempted to access layer with index {layer_idx}')

    def init_layer(self, layer_idx: int, k: torch.Tensor, v: torch.Tensor, g: torch.Tensor, window_size: int,
                   recurrent_state: Tuple[torch.Tensor, torch.Tensor],
                   rope: Optional[Tuple[torch.Tensor, torch.Tensor]] = None, fused: bool = True) -> RingLayer:
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
                          window_size=window_size, rope=rope, fused=fused)
        self.layers[layer_idx] = layer
        return layer

    def decode(self, layer_idx: int, q, k, v, g, cos, sin, scale=None) -> torch.Tensor:
        if layer_idx == 0:
            self._seen_tokens += 1
            self.former_tokens = self._seen_tokens
        return fused_recurrent_nha_decode_ring(q, k, v, g, self[layer_idx], cos, sin, scale)

    def get_seq_length(self, layer_idx: int = 0) -> int:
        """Tokens seen before the update in progress, as the reference counts them (nha_cache.py:156-160); after
        :meth:`decode` steps, all tokens decoded so far."""
        return self.former_tokens if layer_idx < len(self.layers) else 0

    def get_pop_kvf(self, layer_idx: int, window_size: int):
        """The oldest window entry ``(k, v, g)`` as ``[B,1,H*D]`` views' equivalents (copies), or Nones."""
        if layer_idx >= len(self.layers) or self.layers[layer_idx] is None:
            return (None, None, None)
        L = self.layers[layer_idx]
        if L.fill < L.window:
            return (None, None, None)                 # as NHACache: nothing leaves a window that is not full
        b = torch.arange(L.head.shape[0], device=L.head.device)
        pick = lambda r: r[b, L.oldest()].reshape(r.shape[0], 1, -1)
        return pick(L.ring_k), pick(L.ring_v), pick(L.ring_g)
