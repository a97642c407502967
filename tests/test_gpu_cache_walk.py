"""GPU: the ops fed exactly what the reference's NHACache hands out.

tests/golden/cache_walk.npz was recorded by driving the reference's real ``NHACache`` the way its hybrid model does
(prompt cached, then per token get_pop_kvf -> update(attn_state) -> decode op -> update(recurrent_state)) with the
reference's fp64 functions as the op; see tests/golden/make_boundary.py.  Here the CUDA ops take the recorded
hand-over (the popped entry, the [B,W,H,D] views of the cache's window, the cached state) and must reproduce the
recorded outputs; the device ring cache is stepped beside it from the same prompt.
"""
import json
import os

import numpy as np
import pytest
import torch

from tests import inputs as gen
from tests.gpu_util import TOL_OUT, assert_close

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), 'golden')
META = json.load(open(os.path.join(GOLD, 'boundary.json')))['cache_walk']


def _walk():
    z = np.load(os.path.join(GOLD, 'cache_walk.npz'))
    return {k: torch.from_numpy(z[k]) for k in z.files}


def test_prompt_then_decode_steps_through_the_cache_contract():
    from nha_b200 import fused_chunk_nha_prefill, fused_recurrent_nha_decode
    m, z = META, _walk()
    B, H, NG, K, M, W, T = m['B'], m['H'], m['NG'], m['K'], m['M'], m['W'], m['T']
    d = gen.prefill_inputs(m['seed'], B, H, NG, K, K, M, W, T + m['steps'], with_state=False)
    assert gen.digest(d) == m['digest']
    bf = lambda x: x.to(torch.bfloat16).cuda()
    o, (hk, hv) = fused_chunk_nha_prefill(q=bf(d['q'][:, :T]), k=bf(d['k'][:, :T]), v=bf(d['v'][:, :T]),
                                          rotary_q=bf(z['prompt/rq']), rotary_k=bf(z['prompt/rk']), s=bf(d['s'][:, :T]),
                                          g=bf(d['g'][:, :T]), window_size=W, output_final_state=True)
    assert_close(o, z['prompt/o'], TOL_OUT, 'prompt o')
    assert_close(hk, z['prompt/hk'], TOL_OUT, 'prompt hk')
    assert_close(hv, z['prompt/hv'], TOL_OUT, 'prompt hv')
    state = (hk, hv)
    for i in range(m['steps']):
        s = lambda n: z[f'step{i}/{n}']
        # the recorded state is the reference's; ours differs from it by bf16 rounding of the prompt pass, so each
        # step is checked from the recorded state AND the chain of our own states is carried along
        for tag, st_in in (('ref-state', (s('hk_in').cuda(), s('hv_in').cuda())), ('own-state', state)):
            o, st_out = fused_recurrent_nha_decode(q=bf(s('q')), k=bf(s('last_k')), v=bf(s('last_v')), g=bf(s('last_g')),
                                                   sw_k=bf(s('sw_k')), sw_v=bf(s('sw_v')), cos=bf(s('cos')), sin=bf(s('sin')),
                                                   initial_state=(st_in[0].clone(), st_in[1].clone()),
                                                   output_final_state=True)
            assert_close(o, s('o'), TOL_OUT, f'step {i} o ({tag})')
            assert_close(st_out[0], s('hk'), 1e-5 if tag == 'ref-state' else TOL_OUT, f'step {i} hk ({tag})')
            assert_close(st_out[1], s('hv'), 1e-5 if tag == 'ref-state' else TOL_OUT, f'step {i} hv ({tag})')
        state = st_out


def test_ring_cache_beside_the_reference_cache():
    """NHARingCache initialised from the same prompt and stepped with the same new tokens gives the outputs the
    reference's cache flow gave, and pops the same entry the reference's get_pop_kvf popped."""
    from nha_b200 import NHARingCache
    m, z = META, _walk()
    B, H, NG, K, M, W, T = m['B'], m['H'], m['NG'], m['K'], m['M'], m['W'], m['T']
    d = gen.prefill_inputs(m['seed'], B, H, NG, K, K, M, W, T + m['steps'], with_state=False)
    bf = lambda x: x.to(torch.bfloat16).cuda()
    cache = NHARingCache(seen_tokens=T)
    cache.init_layer(0, bf(d['k'][:, :T]), bf(d['v'][:, :T]), bf(d['g'][:, :T]), W,
                     (z['step0/hk_in'].cuda(), z['step0/hv_in'].cuda()))
    for i in range(m['steps']):
        s = lambda n: z[f'step{i}/{n}']
        pk, pv, pg = cache.get_pop_kvf(0, W)
        assert torch.equal(pk.reshape(B, 1, H, K).float().cpu(), s('last_k'))
        assert torch.equal(pg.reshape(B, 1, H, M).float().cpu(), s('last_g'))
        o = cache.decode(0, bf(s('q')), bf(s('k_new')), bf(s('v_new')), bf(s('g_new')), bf(s('cos')), bf(s('sin')))
        assert_close(o, s('o'), TOL_OUT, f'ring step {i} o')
        assert_close(cache[0].hk, s('hk'), 1e-4, f'ring step {i} hk')
        assert_close(cache[0].hv, s('hv'), 1e-4, f'ring step {i} hv')
    assert cache.get_seq_length(0) == T + m['steps']


def test_ring_cache_filled_through_update_then_decoded():
    """The layer filled the reference's way - ``update(attn_state=(k, v, g) flattened to [B, T, H*D])`` then
    ``update(recurrent_state=...)`` - and stepped with the ring decode: same outputs and states as the reference's flow."""
    from nha_b200 import NHARingCache
    m, z = META, _walk()
    B, H, NG, K, M, W, T = m['B'], m['H'], m['NG'], m['K'], m['M'], m['W'], m['T']
    d = gen.prefill_inputs(m['seed'], B, H, NG, K, K, M, W, T + m['steps'], with_state=False)
    bf = lambda x: x.to(torch.bfloat16).cuda()
    cache = NHARingCache()
    st = cache.update(attn_state=tuple(bf(d[n][:, :T]).flatten(-2, -1) for n in ('k', 'v', 'g')), layer_idx=0, offset=0,
                      cache_kwargs=dict(window_size=W))
    assert st['attn_state'][0].shape == (B, W, H * K)
    cache.update(recurrent_state=(z['step0/hk_in'].cuda(), z['step0/hv_in'].cuda()), layer_idx=0, offset=T)
    for i in range(m['steps']):
        s = lambda n: z[f'step{i}/{n}']
        o = cache.decode(0, bf(s('q')), bf(s('k_new')), bf(s('v_new')), bf(s('g_new')), bf(s('cos')), bf(s('sin')))
        assert_close(o, s('o'), TOL_OUT, f'step {i} o')
        assert_close(cache[0]['recurrent_state'][0], s('hk'), 1e-4, f'step {i} hk')
        assert_close(cache[0]['recurrent_state'][1], s('hv'), 1e-4, f'step {i} hv')
    assert cache.get_seq_length(0) == T + m['steps']
