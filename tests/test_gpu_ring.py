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


@pytest.mark.parametrize('fused', [True, False], ids=['one_launch', 'two_launches'])
@pytest.mark.parametrize('B,H,NG,D,M,W,steps', [(2, 2, 4, 64, 32, 64, 70), (3, 4, 8, 128, 64, 256, 20), (1, 1, 1, 64, 64, 16, 40),
                                                (48, 4, 8, 128, 64, 512, 6)])
def test_ring_decode_matches_shifted_window(B, H, NG, D, M, W, steps, fused):
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
    cache.init_layer(0, win_k, win_v, win_g, W, (hk, hv), fused=fused)
    assert cache[0].head.shape == ((B, H) if fused else (B,))
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


@pytest.mark.parametrize('fused', [True, False], ids=['one_launch', 'two_launches'])
@pytest.mark.parametrize('B,H,NG,D,M,W,T0,steps', [(2, 2, 4, 64, 32, 16, 0, 40), (2, 4, 8, 128, 64, 64, 5, 80)])
def test_ring_decode_warm_up_matches_growing_window(B, H, NG, D, M, W, T0, steps, fused):
    """A prompt shorter than the window: the rings fill up step by step.  Until they are full nothing leaves the
    window; the reference's callers hand the op an all-zero entry then (qwennha.py:152-160) and a window that grows
    by one token per step (NHACache.update).  Same flow here with the shifted-window decode as the reference arm."""
    from nha_b200 import NHARingCache, fused_recurrent_nha_decode
    dev = 'cuda'
    g0 = torch.Generator().manual_seed(300 + W)
    r = lambda *s: torch.randn(*s, generator=g0)
    HQ = H * NG
    win_k = (r(B, T0, H, D) * D ** -0.5).bfloat16().to(dev)
    win_v = (r(B, T0, H, D) * D ** -0.5).bfloat16().to(dev)
    win_g = (F.logsigmoid(r(B, T0, H, M)) / 8).bfloat16().to(dev)
    hk = (r(B, H, D, M) * 0.5).to(dev)
    hv = (r(B, H, M, D) * 0.5).to(dev)
    cache = NHARingCache()
    cache.init_layer(0, win_k, win_v, win_g, W, (hk, hv), fused=fused)
    assert cache[0].head.shape == ((B, H) if fused else (B,))
    ref_k, ref_v, ref_g = win_k.clone(), win_v.clone(), win_g.clone()
    ref_hk, ref_hv = hk.clone(), hv.clone()
    for t in range(steps):
        q = (r(B, 1, HQ, D) * D ** -0.5).bfloat16().to(dev)
        k = (r(B, 1, H, D) * D ** -0.5).bfloat16().to(dev)
        v = (r(B, 1, H, D) * D ** -0.5).bfloat16().to(dev)
        g = (F.logsigmoid(r(B, 1, H, M)) / 8).bfloat16().to(dev)
        full = ref_k.shape[1] >= W
        pk, pv, pg = cache.get_pop_kvf(0, W)
        assert (pk is not None) == full
        if full:
            pop_k, pop_v, pop_g = ref_k[:, :1].contiguous(), ref_v[:, :1].contiguous(), ref_g[:, :1].contiguous()
            ref_k, ref_v, ref_g = ref_k[:, 1:], ref_v[:, 1:], ref_g[:, 1:]
        else:
            pop_k, pop_v, pop_g = torch.zeros_like(k), torch.zeros_like(v), torch.zeros_like(g)
        ref_k, ref_v, ref_g = torch.cat([ref_k, k], 1), torch.cat([ref_v, v], 1), torch.cat([ref_g, g], 1)
        wlen = ref_k.shape[1]
        cos, sin = gen.rope_tables(wlen, D, first_pos=T0 + t - wlen + 1)
        cos, sin = cos.to(dev), sin.to(dev)
        o_ref, (ref_hk, ref_hv) = fused_recurrent_nha_decode(q=q, k=pop_k, v=pop_v, g=pop_g, sw_k=ref_k.contiguous(),
                                                             sw_v=ref_v.contiguous(), cos=cos, sin=sin,
                                                             initial_state=(ref_hk, ref_hv), output_final_state=True)
        o = cache.decode(0, q, k, v, g, cos, sin)
        assert torch.equal(o, o_ref), f'step {t} (window {wlen}): output differs from the growing-window decode'
        assert torch.equal(cache[0].hk, ref_hk) and torch.equal(cache[0].hv, ref_hv), f'step {t}: state differs'
        if t == 0:
            want = orc.decode_step(q.cpu(), pop_k.cpu(), pop_v.cpu(), pop_g.cpu(), ref_k.cpu(), ref_v.cpu(), D ** -0.5,
                                   cos=cos.cpu(), sin=sin.cpu(), hk0=hk.cpu(), hv0=hv.cpu())
            assert_close(o, want[0], TOL_OUT, 'o (first step vs oracle)')
    ok, ov, og = cache[0].ordered()
    assert torch.equal(ok, ref_k) and torch.equal(ov, ref_v) and torch.equal(og, ref_g)


@pytest.mark.parametrize('B,H,NG,D,M,W,T0,steps', [(2, 2, 4, 64, 32, 64, 64, 70), (2, 4, 8, 128, 64, 256, 300, 20),
                                                   (2, 2, 4, 128, 64, 32, 7, 50), (1, 1, 1, 64, 64, 16, 0, 40)])
def test_ring_with_keys_rotated_on_entry_matches_raw_key_ring(B, H, NG, D, M, W, T0, steps):
    """Keys rotated once, when they enter the ring (absolute positions), against the shifted-window decode that
    rotates the whole raw window at every step with the tables of the same absolute positions: same bits, from
    full rings and from prompts shorter than the window."""
    from nha_b200 import NHARingCache, fused_recurrent_nha_decode
    dev = 'cuda'
    g0 = torch.Generator().manual_seed(500 + W)
    r = lambda *s: torch.randn(*s, generator=g0)
    HQ = H * NG
    pre_k = (r(B, T0, H, D) * D ** -0.5).bfloat16().to(dev)
    pre_v = (r(B, T0, H, D) * D ** -0.5).bfloat16().to(dev)
    pre_g = (F.logsigmoid(r(B, T0, H, M)) / 8).bfloat16().to(dev)
    hk = (r(B, H, D, M) * 0.5).to(dev)
    hv = (r(B, H, M, D) * 0.5).to(dev)
    cos_all, sin_all = gen.rope_tables(T0 + steps, D, first_pos=0)          # [1, T0 + steps, D], absolute positions
    cos_all, sin_all = cos_all.to(dev), sin_all.to(dev)
    cache = NHARingCache()
    cache.init_layer(0, pre_k, pre_v, pre_g, W, (hk, hv), rope=(cos_all[:, :T0], sin_all[:, :T0]))
    assert cache[0].ring_kr is not None
    ref_k, ref_v, ref_g = pre_k[:, -W:].clone(), pre_v[:, -W:].clone(), pre_g[:, -W:].clone()
    ref_hk, ref_hv = hk.clone(), hv.clone()
    for t in range(steps):
        pos = T0 + t
        q = (r(B, 1, HQ, D) * D ** -0.5).bfloat16().to(dev)
        k = (r(B, 1, H, D) * D ** -0.5).bfloat16().to(dev)
        v = (r(B, 1, H, D) * D ** -0.5).bfloat16().to(dev)
        g = (F.logsigmoid(r(B, 1, H, M)) / 8).bfloat16().to(dev)
        if ref_k.shape[1] >= W:
            pop_k, pop_v, pop_g = ref_k[:, :1].contiguous(), ref_v[:, :1].contiguous(), ref_g[:, :1].contiguous()
            ref_k, ref_v, ref_g = ref_k[:, 1:], ref_v[:, 1:], ref_g[:, 1:]
        else:
            pop_k, pop_v, pop_g = torch.zeros_like(k), torch.zeros_like(v), torch.zeros_like(g)
        ref_k, ref_v, ref_g = torch.cat([ref_k, k], 1), torch.cat([ref_v, v], 1), torch.cat([ref_g, g], 1)
        wlen = ref_k.shape[1]
        cos, sin = cos_all[:, pos - wlen + 1:pos + 1].contiguous(), sin_all[:, pos - wlen + 1:pos + 1].contiguous()
        o_ref, (ref_hk, ref_hv) = fused_recurrent_nha_decode(q=q, k=pop_k, v=pop_v, g=pop_g, sw_k=ref_k.contiguous(),
                                                             sw_v=ref_v.contiguous(), cos=cos, sin=sin,
                                                             initial_state=(ref_hk, ref_hv), output_final_state=True)
        o = cache.decode(0, q, k, v, g, cos[:, -1:], sin[:, -1:])
        assert torch.equal(o, o_ref), f'step {t} (window {wlen}): output differs'
        assert torch.equal(cache[0].hk, ref_hk) and torch.equal(cache[0].hv, ref_hv), f'step {t}: state differs'
    ok, ov, og = cache[0].ordered()
    assert torch.equal(ok, ref_k) and torch.equal(ov, ref_v) and torch.equal(og, ref_g)
