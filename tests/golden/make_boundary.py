"""Fixtures that pin the drop-in boundary on the reference's own code (run where a checkout is readable):

    python tests/golden/make_boundary.py --reference <path of a JusenD/NHA checkout>

1. ``boundary.json``: names, kinds and defaults of the parameters of the reference's four operators
   (nha_fla/ops/nha/chunk.py:568-585, chunk_fused.py:291-303, fused_recurrent.py:431-445 and :588-598), read with
   ``inspect.signature``; ``tests/test_abi.py`` holds this package's operators against them.
2. ``cache_walk.npz``: the reference's REAL ``NHACache`` (nha_fla/models/nha_cache.py:11-182, constructed with the
   base-class patch of scripts/verify_opt_parity.py:618-630) driven the way the hybrid model's attention drives it
   (nha_fla/models/qwen3_moe_nha/qwennha.py:149-176 and :388-393): a prompt is cached with
   ``update(attn_state=(k, v, g) flattened to [B, T, H*D], window_size=W)``, then every generated token does
   ``get_pop_kvf`` -> ``update(attn_state=...)`` -> decode op -> ``update(recurrent_state=...)``.  The decode op is
   the reference's fp64 ``ref_decode`` (scripts/verify_opt_parity.py:88-125); the prompt's state comes from
   ``ref_prefill`` (:147-191).  Stored per step: the tensors exactly as the cache handed them to the op (views of
   its ``[B, W, H*D]`` buffers reshaped to heads) and the op's outputs, so a GPU test can feed the CUDA op the same
   hand-over and compare, and can step the device ring cache beside it.
3. ``cache_update_walk.npz``: the same real ``NHACache`` driven through ``update`` / ``get_pop_kvf`` /
   ``get_seq_length`` alone (no operator) on tiny tensors: a long prompt, single tokens, a short chunk, a chunk longer
   than the window; and a prompt shorter than the window that fills up token by token.  Every call's inputs and
   answers are stored in call order; ``tests/test_ring_cache_update.py`` replays the calls on ``NHARingCache``.
"""
import argparse
import inspect
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from tests import inputs as gen               # noqa: E402


def signatures():
    from nha_fla.ops.nha import chunk_nha, fused_recurrent_nha, fused_recurrent_nha_decode
    from nha_fla.ops.nha.chunk_fused import fused_chunk_nha_prefill
    out = {}
    for f in (chunk_nha, fused_chunk_nha_prefill, fused_recurrent_nha, fused_recurrent_nha_decode):
        out[f.__name__] = [[p.name, str(p.kind), None if p.default is inspect.Parameter.empty else repr(p.default)]
                           for p in inspect.signature(f).parameters.values()]
    return out


def cache_walk(vp):
    import transformers.cache_utils as tcu

    def lenient_init(self, layers=None, layer_class_to_replicate=None, offloading=False, offload_only_non_sliding=True):
        self.layers = layers if layers is not None else []
        self.layer_class_to_replicate = layer_class_to_replicate
        self.offloading = offloading
        self.offload_only_non_sliding = offload_only_non_sliding
    tcu.Cache.__init__ = lenient_init
    from nha_fla.models.nha_cache import NHACache

    B, H, NG, K, M, W, T, STEPS = 2, 2, 2, 64, 32, 16, 40, 4
    HQ = H * NG
    d = gen.prefill_inputs(777, B, H, NG, K, K, M, W, T + STEPS, with_state=False)
    scale = K ** -0.5
    cos_all, sin_all = gen.rope_tables(T + STEPS, K, first_pos=0)          # [1, T+STEPS, K], absolute positions
    out = {}
    # ---- prompt: ref_prefill takes pre-rotated q/k; the cache keeps the RAW keys, values and gate rows
    rq = gen.eager_rope(d['q'][:, :T], cos_all[:, :T], sin_all[:, :T]).to(torch.bfloat16)
    rk = gen.eager_rope(d['k'][:, :T], cos_all[:, :T], sin_all[:, :T]).to(torch.bfloat16)
    r = vp.ref_prefill(dict(q=d['q'][:, :T], k=d['k'][:, :T], v=d['v'][:, :T], rotary_q=rq, rotary_k=rk, s=d['s'][:, :T],
                            g=d['g'][:, :T], W=W, scale=scale))
    o, hk, hv = r['o'], r['hkt'], r['hvt']
    out['prompt/o'], out['prompt/hk'], out['prompt/hv'] = o, hk, hv
    out['prompt/rq'], out['prompt/rk'] = rq.float(), rk.float()
    cache = NHACache()
    cache.update(attn_state=(d['k'][:, :T].flatten(-2, -1), d['v'][:, :T].flatten(-2, -1), d['g'][:, :T].flatten(-2, -1)),
                 layer_idx=0, offset=0, cache_kwargs=dict(window_size=W))
    cache.update(recurrent_state=(hk.float(), hv.float()), layer_idx=0, offset=T)
    # ---- generated tokens, as qwennha.py drives the cache
    for i in range(STEPS):
        t = T + i
        q, k, v, g = (d[n][:, t:t + 1] for n in ('q', 'k', 'v', 'g'))
        last_k, last_v, last_g = cache.get_pop_kvf(0, W)
        assert last_k is not None
        last_k, last_v, last_g = (x.reshape(B, 1, H, -1) for x in (last_k, last_v, last_g))
        st = cache.update(attn_state=(k.flatten(-2, -1), v.flatten(-2, -1), g.flatten(-2, -1)), layer_idx=0, offset=0,
                          cache_kwargs=dict(window_size=W))['attn_state']
        assert cache.get_seq_length(0) > 0
        sw_k, sw_v = st[0].reshape(B, W, H, K), st[1].reshape(B, W, H, K)
        cos, sin = cos_all[:, t - W + 1:t + 1], sin_all[:, t - W + 1:t + 1]
        rec = cache[0]['recurrent_state']
        # the model passes no s on this path (rotary and the slot residual are folded into the kernel, qwennha.py:346-348),
        # and the reference kernel then forms s = 1 - exp(g) in fp32 (fused_recurrent.py:266-267): no bf16 rounding of s
        last_s = 1 - last_g.double().exp()
        r = vp.ref_decode(dict(q=q, k=last_k, v=last_v, s=last_s, g=last_g, sw_k_raw=sw_k, vw=sw_v, cos=cos, sin=sin,
                               hk0=rec[0], hv0=rec[1], scale=scale))
        o, hk, hv = r['o'], r['hkt'], r['hvt']
        for name, x in (('q', q), ('last_k', last_k), ('last_v', last_v), ('last_g', last_g), ('sw_k', sw_k), ('sw_v', sw_v),
                        ('cos', cos), ('sin', sin), ('hk_in', rec[0]), ('hv_in', rec[1]), ('o', o), ('hk', hk), ('hv', hv),
                        ('k_new', k), ('v_new', v), ('g_new', g)):
            out[f'step{i}/{name}'] = x
        cache.update(recurrent_state=(hk.float(), hv.float()), layer_idx=0, offset=1)
    meta = dict(B=B, H=H, NG=NG, K=K, M=M, W=W, T=T, steps=STEPS, seed=777, digest=gen.digest(d))
    return {k: v.detach().float().numpy() for k, v in out.items()}, meta


def _patched_cache_class():
    import transformers.cache_utils as tcu

    def lenient_init(self, layers=None, layer_class_to_replicate=None, offloading=False, offload_only_non_sliding=True):
        self.layers = layers if layers is not None else []
        self.layer_class_to_replicate = layer_class_to_replicate
        self.offloading = offloading
        self.offload_only_non_sliding = offload_only_non_sliding
    tcu.Cache.__init__ = lenient_init
    from nha_fla.models.nha_cache import NHACache
    return NHACache


def cache_update_walk():
    """Scripts of ``update`` calls; per call i of script S: ``S/i/in_k|in_v|in_g`` (the new tokens), ``S/i/pop_*`` (what
    get_pop_kvf gave before the call, absent when it gave None), ``S/i/ret_*`` (the returned window) and
    ``S/i/seq`` (get_seq_length after the call)."""
    NHACache = _patched_cache_class()
    B, DK, DV, DG, W = 2, 12, 12, 6, 16
    gen_ = torch.Generator().manual_seed(2024)
    out, scripts = {}, {'long_prompt': [40, 1, 1, 1, 5, 1, 20, 1, 1], 'short_prompt': [6] + [1] * 14}
    for name, lens in scripts.items():
        cache = NHACache()
        for i, n in enumerate(lens):
            k, v, g = (torch.randn(B, n, D, generator=gen_).to(torch.bfloat16) for D in (DK, DV, DG))
            pop = cache.get_pop_kvf(0, W)
            st = cache.update(attn_state=(k, v, g), layer_idx=0, offset=0, cache_kwargs=dict(window_size=W))['attn_state']
            cache.update(recurrent_state=(torch.zeros(1), torch.zeros(1)), layer_idx=0, offset=n)
            for tag, x in zip(('k', 'v', 'g'), (k, v, g)):
                out[f'{name}/{i}/in_{tag}'] = x
            if pop[0] is not None:
                for tag, x in zip(('k', 'v', 'g'), pop):
                    out[f'{name}/{i}/pop_{tag}'] = x
            for tag, x in zip(('k', 'v', 'g'), st):
                out[f'{name}/{i}/ret_{tag}'] = x
            out[f'{name}/{i}/seq'] = torch.tensor([cache.get_seq_length(0)])
    meta = dict(B=B, DK=DK, DV=DV, DG=DG, W=W, scripts=scripts)
    return {k: v.detach().float().numpy() for k, v in out.items()}, meta


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='path of a checkout of the reference project')
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, 'scripts'))
    sys.path.insert(0, args.reference)
    import verify_opt_parity as vp
    vp.DEVICE = 'cpu'
    walk, meta = cache_walk(vp)
    np.savez_compressed(os.path.join(HERE, 'cache_walk.npz'), **walk)
    upd, upd_meta = cache_update_walk()
    np.savez_compressed(os.path.join(HERE, 'cache_update_walk.npz'), **upd)
    with open(os.path.join(HERE, 'boundary.json'), 'w') as f:
        json.dump({'signatures': signatures(), 'cache_walk': meta, 'cache_update_walk': upd_meta}, f, indent=1)
    print('wrote boundary.json, cache_walk.npz and cache_update_walk.npz', meta)


if __name__ == '__main__':
    main()
