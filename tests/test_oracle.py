"""CPU: the oracle against the fixtures generated from the reference's own naive functions."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import nha_oracle as orc
from tests import inputs as gen

GOLD = os.path.join(os.path.dirname(__file__), 'golden')
MAN = json.load(open(os.path.join(GOLD, 'manifest.json')))
TOL = 1e-6   # fixtures are stored in fp32; the oracle is fp64


def _npz(name):
    return np.load(os.path.join(GOLD, name))


def _t(a):
    return torch.from_numpy(np.asarray(a))


@pytest.mark.parametrize('case', sorted(MAN['decode']))
def test_decode_matches_reference_fixture(case):
    c = MAN['decode'][case]
    z = _npz('decode.npz')
    d = gen.decode_inputs(c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'])
    assert gen.digest(d) == c['digest'], 'input generator drifted from the one that made the fixture'
    o, hk, hv, ps, pw = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'],
                                        s=d['s'], cos=d['cos'], sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    for got, key in ((o, 'o'), (hk, 'hkt'), (hv, 'hvt'), (ps, 'qv'), (pw, 'swp')):
        assert orc.rel_l2(got, _t(z[f'{case}/{key}'])) < TOL, key


@pytest.mark.parametrize('case', sorted(MAN['recurrent']))
def test_recurrent_matches_reference_fixture(case):
    c = MAN['recurrent'][case]
    z = _npz('recurrent.npz')
    d = gen.recurrent_inputs(c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'])
    assert gen.digest(d) == c['digest']
    o, pw, hk, hv = orc.recurrent_step(d['q'], d['k'], d['v'], d['sliding_window'], d['s'], d['g'], d['scale'],
                                       d['hk0'], d['hv0'])
    for got, key in ((o, 'o'), (pw, 'swa_score'), (hk, 'hkt'), (hv, 'hvt')):
        assert orc.rel_l2(got, _t(z[f'{case}/{key}'])) < TOL, key


@pytest.mark.parametrize('case', sorted(MAN['prefill']))
def test_prefill_matches_reference_fixture(case):
    c = MAN['prefill'][case]
    z = _npz('prefill.npz')
    d = gen.prefill_inputs(c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'], c['T'], c['with_state'])
    assert gen.digest(d) == c['digest']
    o, hk, hv = orc.prefill(d['q'], d['k'], d['v'], d['rotary_q'], d['rotary_k'], d['s'], d['g'], c['W'], d['scale'],
                            d.get('hk0'), d.get('hv0'))
    for got, key in ((o, 'o'), (hk, 'hkt'), (hv, 'hvt')):
        assert orc.rel_l2(got, _t(z[f'{case}/{key}'])) < TOL, key


def training_case(name):
    """Inputs, oracle outputs and oracle gradients of a stored training case."""
    c = MAN['training'][name]
    B, T, H, K, V, M = c['B'], c['T'], c['H'], c['K'], c['V'], c['M']
    d = gen.training_inputs(c['seed'], B, T, H, K, V, M)
    assert gen.digest(d) == c['digest']
    cu = c['cu'] if c['cu'] is not None else [i * T for i in range(B + 1)]
    N = len(cu) - 1
    hk0 = hv0 = None
    if c['with_state']:
        torch.manual_seed(c['seed'] + 50000)
        hk0 = (torch.randn(N, H, K, M) * 0.5).float()
        hv0 = (torch.randn(N, H, M, V) * 0.5).float()
    torch.manual_seed(c['seed'] + 70000)
    dlse = (torch.randn(B * T, H) * 0.1).double()
    return c, d, cu, hk0, hv0, dlse


@pytest.mark.parametrize('case', sorted(MAN['training']))
def test_training_matches_reference_replay_fixture(case):
    c, d, cu, hk0, hv0, dlse = training_case(case)
    z = _npz('training.npz')
    B, T = c['B'], c['T']
    names = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')
    xs = {n: d[n].reshape(B * T, *d[n].shape[2:]).double().requires_grad_(True) for n in names}
    st = []
    if hk0 is not None:
        st = [hk0.double().requires_grad_(True), hv0.double().requires_grad_(True)]
    o, ls, lg, hk, hv = orc.nha_varlen(xs['q_gsa'], xs['q_swa'], xs['k_gsa'], xs['k_swa'], xs['v'], xs['s'], xs['g'],
                                       cu, c['K'] ** -0.5, c['window_left'], c['shift'], *(st or [None, None]))
    do = d['do'].reshape(B * T, *d['do'].shape[2:]).double()
    ((o * do).sum() + (lg * dlse).sum()).backward()
    for got, key in ((o, 'o'), (ls, 'lse_swa'), (lg, 'lse_gsa'), (hk, 'hkt'), (hv, 'hvt')):
        assert orc.rel_l2(got, _t(z[f'{case}/{key}'])) < TOL, key
    for n in names:
        assert orc.rel_l2(xs[n].grad, _t(z[f'{case}/grad_{n}'])) < TOL, n
    if st:
        assert orc.rel_l2(st[0].grad, _t(z[f'{case}/grad_hk0'])) < TOL
        assert orc.rel_l2(st[1].grad, _t(z[f'{case}/grad_hv0'])) < TOL


def test_lse_merge_equals_joint_softmax():
    """The reference merges two branch outputs by log-sum-exp (nha_fla/ops/nha/chunk.py:458-470);
    the oracle takes one softmax over the concatenation.  Both must agree."""
    torch.manual_seed(1)
    T, H, K, V, M, W = 40, 2, 16, 16, 8, 6
    dd = torch.float64
    q, qs, k, ks = (torch.randn(T, H, K, dtype=dd) for _ in range(4))
    v = torch.randn(T, H, V, dtype=dd)
    g = torch.nn.functional.logsigmoid(torch.randn(T, H, M, dtype=dd))
    s = 1 - g.exp()
    o, ls, lg, hk, hv = orc.nha_sequence(q, qs, k, ks, v, s, g, 0.25, W, 0)
    # slot-only and window-only outputs recomputed separately
    hkc = torch.zeros(H, K, M, dtype=dd); hvc = torch.zeros(H, M, V, dtype=dd)
    for t in range(T):
        hkc, hvc = orc.gsa_step(hkc, hvc, k[t], v[t], s[t], g[t])
        ok = torch.einsum('hk,hkm->hm', q[t] * 0.25, hkc)
        og = torch.einsum('hm,hmv->hv', torch.softmax(ok, -1), hvc)
        lo = max(0, t - W)
        sw = torch.einsum('hk,whk->hw', qs[t] * 0.25, ks[lo:t + 1])
        osw = torch.einsum('hw,whv->hv', torch.softmax(sw, -1), v[lo:t + 1])
        mx = torch.maximum(ls[t], lg[t])
        ws, wg = (ls[t] - mx).exp(), (lg[t] - mx).exp()
        merged = (ws[:, None] * osw + wg[:, None] * og) / (ws + wg)[:, None]
        assert torch.allclose(merged, o[t], atol=1e-12)


def test_slot_gates_against_the_layer_chain():
    """The oracle's gate function against the layer's own three lines (nha_fla/layers/nha.py:229-231) run
    literally in fp64 and in bf16: identical in fp64, within bf16 rounding of the chain's three roundings in bf16."""
    import torch.nn.functional as F
    torch.manual_seed(3)
    f = torch.randn(4, 33, 2, 16, dtype=torch.float64) * 3
    for norm in (1.0, 8.0):
        g, s = orc.slot_gates(f, norm)
        f1 = F.logsigmoid(f) / norm                       # the chain, as written in the layer
        s1 = (1 - f1.exp()).to(f1.dtype)
        assert torch.allclose(g, f1, rtol=0, atol=1e-15) and torch.allclose(s, s1, rtol=0, atol=1e-14)
        fb = f.bfloat16()
        f2 = F.logsigmoid(fb) / norm
        s2 = (1 - f2.exp()).to(f2.dtype)
        gb, sb = orc.slot_gates(fb, norm)
        assert orc.rel_l2(f2.double(), gb) < 1e-2 and orc.rel_l2(s2.double(), sb) < 1e-2


def test_rotary_positions_against_fla_reference_and_rotate_half():
    """The oracle's rotary against the third-party PyTorch reference the layer's RotaryEmbedding stands on
    (fla.modules.rotary.rotary_embedding_ref, flash-linear-attention 0.5.1) and against the oracle's own HF-style
    rotate-half on duplicated-halves tables (scripts/verify_opt_parity.py:48-54)."""
    torch.manual_seed(4)
    T, H, K, P = 37, 3, 32, 64
    x = torch.randn(T, H, K, dtype=torch.float64)
    inv = 1.0 / (10000.0 ** (torch.arange(0, K, 2, dtype=torch.float64) / K))
    fr = torch.outer(torch.arange(P, dtype=torch.float64), inv)
    cos, sin = fr.cos(), fr.sin()
    pos = torch.arange(5, 5 + T)
    got = orc.rotary_positions(x, cos, sin, pos)
    hf = orc.rope_rotate_half(x, torch.cat([cos, cos], -1)[pos], torch.cat([sin, sin], -1)[pos])
    assert torch.allclose(got, hf, rtol=0, atol=1e-14)
    rot = pytest.importorskip('fla.modules.rotary')
    want = rot.rotary_embedding_ref(x[None], cos[pos], sin[pos])[0]
    assert torch.allclose(got, want, rtol=0, atol=1e-14)


def test_gsa_aux_against_the_layer_chain():
    """The oracle's aux-loss function against the layer's own lines run literally
    (nha_fla/layers/nha.py:257-259, 291-292, 308-312)."""
    import torch.nn.functional as F
    torch.manual_seed(5)
    ls = torch.randn(3, 50, 4, dtype=torch.float64) * 3
    lg = (torch.randn(3, 50, 4, dtype=torch.float64) * 3).requires_grad_(True)
    loss, ratio = orc.gsa_aux(ls, lg, 0.3)
    lse_max = torch.maximum(ls, lg)
    w_swa, w_gsa = torch.exp(ls - lse_max), torch.exp(lg - lse_max)
    want_ratio = (w_gsa / (w_swa + w_gsa)).mean()
    delta = lg - ls.detach()                        # the layer writes .float() here: its lse tensors are fp32
    want = F.binary_cross_entropy_with_logits(delta, torch.full_like(delta, 0.3), reduction='mean')
    assert torch.allclose(loss, want, rtol=0, atol=1e-14) and torch.allclose(ratio, want_ratio.detach(), rtol=0, atol=1e-14)
    (g1,) = torch.autograd.grad(loss, lg, retain_graph=True)
    lg2 = lg.detach().clone().requires_grad_(True)
    d2 = lg2 - ls
    (g2,) = torch.autograd.grad(F.binary_cross_entropy_with_logits(d2, torch.full_like(d2, 0.3)), lg2)
    assert torch.allclose(g1, g2, rtol=0, atol=1e-15)


def test_layer_activations_and_norm_against_fla_references():
    """The oracle's feature map / value activation and its silu + RMS norm against the layer's own lines
    (nha_fla/layers/nha.py:219-223, 277-278) written with the third-party pieces they call: torch's silu / relu (the
    swish feature map of flash-linear-attention 0.5.1 is x * sigmoid(x)) and fla.modules.layernorm.rms_norm_ref."""
    import torch.nn.functional as F
    torch.manual_seed(11)
    q, k, v = (torch.randn(2, 9, 3, 16, dtype=torch.float64) * 2 for _ in range(3))
    qg, kg, va = orc.feature_maps(q, k, v, 'swish')
    assert torch.allclose(qg, F.silu(q), atol=1e-15) and torch.allclose(kg, F.silu(k), atol=1e-15)
    assert torch.allclose(va, F.silu(v), atol=1e-15)
    qr, kr, _ = orc.feature_maps(q, k, v, 'relu')
    assert torch.equal(qr, F.relu(q)) and torch.equal(kr, F.relu(k))
    o = torch.randn(7, 256, dtype=torch.float64) * 3
    w, b = torch.rand(256, dtype=torch.float64) + 0.5, torch.randn(256, dtype=torch.float64) * 0.1
    got = orc.silu_rms_norm(o, w, b, 1e-5)
    ln = pytest.importorskip('fla.modules.layernorm')
    want = ln.rms_norm_ref(F.silu(o), w, b, eps=1e-5)
    assert torch.allclose(got, want, rtol=0, atol=1e-13)
    assert torch.allclose(orc.silu_rms_norm(o, w, None, 1e-5), ln.rms_norm_ref(F.silu(o), w, None, eps=1e-5), atol=1e-13)
