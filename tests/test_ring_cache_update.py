"""CPU: ``NHARingCache`` driven through the reference cache's own calls (``get_pop_kvf`` / ``update`` /
``get_seq_length``) must answer as the reference's real ``NHACache`` answered the same calls
(nha_fla/models/nha_cache.py:44-160).  The answers were recorded by ``tests/golden/make_boundary.py`` from the
reference's class: a long prompt followed by single tokens, a short chunk and a chunk longer than the window,
and a prompt shorter than the window that fills up token by token."""
import json
import os

import numpy as np
import pytest
import torch

from nha_b200 import NHARingCache

GOLD = os.path.join(os.path.dirname(__file__), 'golden')
META = json.load(open(os.path.join(GOLD, 'boundary.json')))['cache_update_walk']


@pytest.fixture(scope='module')
def walk():
    z = np.load(os.path.join(GOLD, 'cache_update_walk.npz'))
    return {k: torch.from_numpy(z[k]) for k in z.files}


@pytest.mark.parametrize('script', sorted(META['scripts']))
def test_update_calls_answer_like_the_reference_cache(walk, script):
    W = META['W']
    cache = NHARingCache()
    for i, n in enumerate(META['scripts'][script]):
        new = tuple(walk[f'{script}/{i}/in_{t}'].to(torch.bfloat16) for t in 'kvg')
        assert new[0].shape[1] == n
        pop = cache.get_pop_kvf(0, W)
        if f'{script}/{i}/pop_k' in walk:
            for t, x in zip('kvg', pop):
                assert torch.equal(x.float(), walk[f'{script}/{i}/pop_{t}']), f'call {i}: popped {t}'
        else:
            assert pop == (None, None, None), f'call {i}: the reference popped nothing'
        st = cache.update(attn_state=new, layer_idx=0, offset=0, cache_kwargs=dict(window_size=W))
        cache.update(recurrent_state=(torch.zeros(1, 1, 2, 2), torch.zeros(1, 1, 2, 2)), layer_idx=0, offset=n)
        for t, x in zip('kvg', st['attn_state']):
            want = walk[f'{script}/{i}/ret_{t}']
            assert x.shape == want.shape, f'call {i}: window {t} shape {tuple(x.shape)} vs {tuple(want.shape)}'
            assert torch.equal(x.float(), want), f'call {i}: window {t}'
        assert cache.get_seq_length(0) == int(walk[f'{script}/{i}/seq'][0]), f'call {i}: seq length'
    assert len(cache) == 1 and cache[0]['recurrent_state'] is not None


def test_update_argument_errors_and_legacy_round_trip():
    cache = NHARingCache()
    k = torch.randn(1, 5, 8).bfloat16()
    with pytest.raises(ValueError):
        cache.update(attn_state=(k, k), layer_idx=0, cache_kwargs=dict(window_size=4))        # not three tensors
    with pytest.raises(ValueError):
        cache.update(attn_state=(k, k, k), layer_idx=0)                                       # no ring size
    cache.update(attn_state=(k, k, k), recurrent_state=(torch.ones(1, 2, 4, 3), torch.ones(1, 2, 3, 4)), layer_idx=0,
                 offset=5, cache_kwargs=dict(window_size=4))
    # the token count moves before the arguments are looked at, as in the reference (nha_cache.py:76-79)
    assert cache.get_seq_length(0) == 2 and cache._seen_tokens == 7
    with pytest.raises(KeyError):
        cache[1]
    legacy = cache.to_legacy_cache()
    assert torch.equal(legacy[0]['attn_state'][0], k[:, -4:])
    again = NHARingCache.from_legacy_cache(list(legacy), seen_tokens=5)
    for a, b in zip(again[0]['attn_state'], legacy[0]['attn_state']):
        assert torch.equal(a, b)
    assert torch.equal(again[0]['recurrent_state'][0], legacy[0]['recurrent_state'][0])
    assert again.get_max_length() is None and [x for x in again] == again.layers
