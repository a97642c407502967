"""GPU: decode on the device ring-buffer cache against decode on a window that is shifted every step.

The reference's NHACache shifts its window with torch.cat on every token (nha_fla/models/nha_cache.py:105-126)
and pops the oldest entry for the slot memory (:143-154).  The ring cache must give the same outputs and states
step by step, through more than W steps so that the head wraps, and its first step must match the oracle.
"""
import pytest
import torch
import torch.nn.functional as F

from oracle import nha_oracle as orc
from tests import inputs as gen
from tests.gpu_util import TOL_OUT, assert_close

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('B,H,NG,D,M,W,steps', [(2, 2, 4, 64, 32, 64, 70), (3, 4, 8, 128, 64, 256, 20), (1, 1, 1, 64, 64, 16, 40)])
def test_ring_decode_matches_shifted_window(B, H, NG, D, M, W, steps):
    from nha_b200 import NHARingCache, fused_recurrent_nha_decode
    dev = 'cuda'
    g0 = torch.Generator().manual_seed(100 + W)
    r = lambda *s: torch.randn(*s, generator=g0)
    HQ = H * NG
    # history: W tokens already in the window, plus the state
    win_k = (r(B, W, H, D) * D ** -0.5).bfloat16().to(dev)
    win_v = (r(B, W, H, D) * D ** -0.5).bfloat16().to(dev)
    win_g = (F.logsigmoid(r(B, W, H, M)) / 8).bfloat16().to(dev)
    hk = (r(B, H, D, M) * 0.5).to(dev)
    hv = (r(B, H, M, D) * 0.5).to(dev)
    cos, sin = gen.rope_tables(W, D, first_pos=1000)
    cos, sin = cos.to(dev), sin.to(dev)
    cache = NHARingCache()
    cache.init_layer(0, win_k, win_v, win_g, W, (hk, hv))
    ref_k, ref_v, ref_g = win_k.clone(), win_v.clone(), win_g.clone()
    ref_hk, ref_hv = hk.clone(), hv.clone()
    for t in range(steps):
        q = (r(B, 1, HQ, D) * D ** -0.5).bfloat16().to(dev)
        k = (r(B, 1, H, D) * D ** -0.5).bfloat16().to(dev)
        v = (r(B, 1, H, D) * D ** -0.5).bfloat16().to(dev)
        g = (F.logsigmoid(r(B, 1, H, M)) / 8).bfloat16().to(dev)
        # reference flow: pop the oldest entry, shift the window, append the new token, decode
        pop_k, pop_v, pop_g = ref_k[:, :1], ref_v[:, :1], ref_g[:, :1]
        if t == 0:
            pk, pv, pg = cache.get_pop_kvf(0, W)
            assert torch.equal(pk.view_as(pop_k), pop_k) and torch.equal(pg.view_as(pop_g), pop_g)
        ref_k = torch.cat([ref_k[:, 1:], k], 1)
        ref_v = torch.cat([ref_v[:, 1:], v], 1)
        ref_g = torch.cat([ref_g[:, 1:], g], 1)
        o_ref, (ref_hk, ref_hv) = fused_recurrent_nha_decode(q=q, k=pop_k.contiguous(), v=pop_v.contiguous(),
                                                             g=pop_g.contiguous(), sw_k=ref_k, sw_v=ref_v, cos=cos, sin=sin,
                                                             initial_state=(ref_hk, ref_hv), output_final_state=True)
        o = cache.decode(0, q, k, v, g, cos, sin)
        if t == 0:
            want = orc.decode_step(q.cpu(), pop_k.cpu(), pop_v.cpu(), pop_g.cpu(), ref_k.cpu(), ref_v.cpu(), D ** -0.5,
                                   cos=cos.cpu(), sin=sin.cpu(), hk0=hk.cpu(), hv0=hv.cpu())
            assert_close(o, want[0], TOL_OUT, 'o (first step vs oracle)')
        assert torch.equal(o, o_ref), f'step {t}: output differs from the shifted-window decode'
        assert torch.equal(cache[0].hk, ref_hk) and torch.equal(cache[0].hv, ref_hv), f'step {t}: state differs'
    ok, ov, og = cache[0].ordered()
    assert torch.equal(ok, ref_k) and torch.equal(ov, ref_v) and torch.equal(og, ref_g)
    assert cache.get_seq_length() == steps
