"""GPU: chunk_nha forward and backward through the C ABI against the oracle (autograd in fp64)."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import nha_oracle as orc
from tests import inputs as gen
from tests.gpu_util import TOL_GRAD, TOL_OUT, assert_close
from tests.test_oracle import training_case

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), 'golden')
MAN = json.load(open(os.path.join(GOLD, 'manifest.json')))
NAMES = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')


def run_oracle(x, cu, scale, wl, shift, hk0, hv0, do, dlse, dhk=None, dhv=None):
    xs = {n: x[n].double().requires_grad_(True) for n in NAMES}
    st = [None, None]
    if hk0 is not None:
        st = [hk0.double().requires_grad_(True), hv0.double().requires_grad_(True)]
    o, ls, lg, hk, hv = orc.nha_varlen(xs['q_gsa'], xs['q_swa'], xs['k_gsa'], xs['k_swa'], xs['v'], xs['s'], xs['g'],
                                       cu, scale, wl, shift, st[0], st[1])
    loss = (o * do.double()).sum()
    if dlse is not None:
        loss = loss + (lg * dlse.double()).sum()
    if dhk is not None:
        loss = loss + (hk * dhk.double()).sum() + (hv * dhv.double()).sum()
    loss.backward()
    grads = {n: xs[n].grad for n in NAMES}
    if hk0 is not None:
        grads['hk0'], grads['hv0'] = st[0].grad, st[1].grad
    return (o, ls, lg, hk, hv), grads


def run_gpu(x, cu, T, scale, wl, shift, hk0, hv0, do, dlse, dhk=None, dhv=None, batched_B=None):
    from nha_b200 import chunk_nha
    dev = 'cuda'
    xs = {n: x[n].to(dev).requires_grad_(True) for n in NAMES}
    st = None
    if hk0 is not None:
        st = (hk0.to(dev).requires_grad_(True), hv0.to(dev).requires_grad_(True))
    if batched_B is not None:
        B = batched_B
        args = {n: xs[n].view(B, -1, *xs[n].shape[1:]) for n in NAMES}
        kw = {}
    else:
        args = {n: xs[n][None] for n in NAMES}
        kw = dict(cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), max_seqlen=T)
    wl_a = torch.tensor(wl, dtype=torch.int32, device=dev) if isinstance(wl, (list, tuple)) else wl
    sh_a = torch.tensor(shift, dtype=torch.int32, device=dev) if isinstance(shift, (list, tuple)) else shift
    out = chunk_nha(args['q_swa'], args['k_swa'], args['q_gsa'], args['k_gsa'], args['v'], args['s'], args['g'],
                    scale=scale, window_size_left=wl_a, window_size_right=0, gsa_kv_shift=sh_a, initial_state=st,
                    output_final_state=True, **kw)
    o, ls, lg, (hk, hv) = out
    Ttot = x['q_swa'].shape[0]
    loss = (o.reshape(Ttot, *o.shape[2:]).float() * do.to(dev).float()).sum()
    if dlse is not None:
        loss = loss + (lg.reshape(Ttot, -1) * dlse.to(dev).float()).sum()
    if dhk is not None:
        loss = loss + (hk * dhk.to(dev)).sum() + (hv * dhv.to(dev)).sum()
    loss.backward()
    grads = {n: xs[n].grad for n in NAMES}
    if st is not None:
        grads['hk0'], grads['hv0'] = st[0].grad, st[1].grad
    flat = lambda t: t.reshape(Ttot, *t.shape[2:])
    return (flat(o), flat(ls), flat(lg), hk, hv), grads


def compare(outs_g, grads_g, outs_o, grads_o, check_grads=True):
    for got, want, name in zip(outs_g, outs_o, ('o', 'lse_swa', 'lse_gsa', 'hkt', 'hvt')):
        assert_close(got, want, TOL_OUT, name)
    if check_grads:
        for n in grads_o:
            assert grads_g[n] is not None, f'no gradient for {n}'
            assert torch.isfinite(grads_g[n].float()).all(), f'non-finite gradient for {n}'
            assert_close(grads_g[n], grads_o[n], TOL_GRAD, f'grad_{n}')


def flat_inputs(d, B, T):
    return {n: d[n].reshape(B * T, *d[n].shape[2:]) for n in NAMES}


# the reference's training shapes (scripts/verify_opt_parity.py:539-544), window_size_left = 63
@pytest.mark.parametrize('B,T,H,K,M,cu', [(2, 128, 4, 64, 32, None), (1, 300, 8, 64, 64, [0, 100, 300]),
                                          (2, 96, 4, 128, 16, None)])
def test_training_shapes_of_the_reference(B, T, H, K, M, cu):
    d = gen.training_inputs(4000 + T, B, T, H, K, K, M)
    x = flat_inputs(d, B, T)
    cul = cu if cu is not None else [i * T for i in range(B + 1)]
    do = d['do'].reshape(B * T, H, K)
    o_o, g_o = run_oracle(x, cul, K ** -0.5, 63, 0, None, None, do, None)
    o_g, g_g = run_gpu(x, cul, T, K ** -0.5, 63, 0, None, None, do, None, batched_B=B if cu is None else None)
    compare(o_g, g_g, o_o, g_o)


@pytest.mark.parametrize('case', sorted(MAN['training']))
def test_training_against_reference_replay_fixture(case):
    c, d, cu, hk0, hv0, dlse = training_case(case)
    z = np.load(os.path.join(GOLD, 'training.npz'))
    B, T = c['B'], c['T']
    x = flat_inputs(d, B, T)
    do = d['do'].reshape(B * T, *d['do'].shape[2:])
    o_g, g_g = run_gpu(x, cu, T, c['K'] ** -0.5, c['window_left'], c['shift'], hk0, hv0, do, dlse.float(),
                       batched_B=B if c['cu'] is None else None)
    for got, key in zip(o_g, ('o', 'lse_swa', 'lse_gsa', 'hkt', 'hvt')):
        assert_close(got, torch.from_numpy(z[f'{case}/{key}']), TOL_OUT, key)
    for n in NAMES + (('hk0', 'hv0') if c['with_state'] else ()):
        assert_close(g_g[n], torch.from_numpy(z[f'{case}/grad_{n}']), TOL_GRAD, f'grad_{n}')


@pytest.mark.parametrize('wl,shift', [(64, 0), (63, 64), (200, 0), (-1, 0), (5, 130), (0, 1)])
def test_window_and_shift_conventions(wl, shift):
    """Overlapping (layer) and disjoint (hybrid model) conventions, a window wider than a chunk,
    an unbounded window, a shift longer than a chunk, and the one-key window."""
    B, T, HQ, H, K, M = 1, 330, 4, 2, 64, 32
    d = gen.layer_inputs(600 + wl + shift, B, T, HQ, H, K, K, M, gate_div=1.0, val_scale=1.0)
    x = flat_inputs(d, B, T)
    torch.manual_seed(9)
    hk0 = torch.randn(1, H, K, M) * 0.5
    hv0 = torch.randn(1, H, M, K) * 0.5
    dlse = torch.randn(T, HQ) * 0.1
    dhk, dhv = torch.randn(1, H, K, M) * 0.1, torch.randn(1, H, M, K) * 0.1
    do = d['do'].reshape(T, HQ, K).float()
    o_o, g_o = run_oracle(x, [0, T], K ** -0.5, wl, shift, hk0, hv0, do, dlse, dhk, dhv)
    o_g, g_g = run_gpu(x, [0, T], T, K ** -0.5, wl, shift, hk0, hv0, do, dlse, dhk, dhv)
    compare(o_g, g_g, o_o, g_o)


def test_varlen_with_per_sequence_windows():
    """Packed sequences of ragged lengths (the reference's varlen smoke cases, tests/test_varlen.py:60-73,
    include length-1 and length-2 sequences) with a different window and shift per sequence."""
    lens = [1, 200, 3, 50, 4, 300, 2, 7, 64, 65]
    wls = [31, 63, 127, 255, 511, 31, 63, 15, 63, 7]
    shs = [w + 1 for w in wls]
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    T = cu[-1]
    HQ = H = 2
    K, M = 64, 64
    d = gen.layer_inputs(31337, 1, T, HQ, H, K, K, M, gate_div=1.0)
    x = flat_inputs(d, 1, T)
    do = d['do'].reshape(T, HQ, K).float()
    o_o, g_o = run_oracle(x, cu, K ** -0.5, wls, shs, None, None, do, None)
    o_g, g_g = run_gpu(x, cu, max(lens), K ** -0.5, wls, shs, None, None, do, None)
    compare(o_g, g_g, o_o, g_o)


# every tensor-memory backward instantiation (rows, columns and window-columns kernels): tile of 64 rows (one query
# head per kv head) or 128 rows (two heads of a group), head dim 64 or 128; M = 64 selects those kernels
UMMA_SHAPES = [(2, 2, 64), (4, 2, 64), (2, 2, 128), (8, 2, 128)]


@pytest.mark.parametrize('no_umma', ['0', '1'])
@pytest.mark.parametrize('HQ,H,K', UMMA_SHAPES)
def test_backward_of_every_tile_shape(HQ, H, K, no_umma, monkeypatch):
    """Gradients (all seven inputs, both initial states) for grouped query heads and head dim 128 with 64 slots: a
    window wider than a chunk, a packing that holds a one-token sequence, initial states, gradients arriving on
    lse_gsa and on the final states; with the tensor-memory kernels and with the general kernels forced."""
    monkeypatch.setenv('NHA_B200_NO_UMMA', no_umma)
    lens = [150, 1, 70]
    cu = [0, 150, 151, 221]
    T, N, M = cu[-1], len(lens), 64
    d = gen.layer_inputs(7700 + HQ + K, 1, T, HQ, H, K, K, M, gate_div=2.0, val_scale=1.0)
    x = flat_inputs(d, 1, T)
    torch.manual_seed(HQ * K)
    hk0 = torch.randn(N, H, K, M) * 0.5
    hv0 = torch.randn(N, H, M, K) * 0.5
    dlse = torch.randn(T, HQ) * 0.1
    dhk, dhv = torch.randn(N, H, K, M) * 0.1, torch.randn(N, H, M, K) * 0.1
    do = d['do'].reshape(T, HQ, K).float()
    for wl, shift in ((100, 0), (95, 96)):
        o_o, g_o = run_oracle(x, cu, K ** -0.5, wl, shift, hk0, hv0, do, dlse, dhk, dhv)
        o_g, g_g = run_gpu(x, cu, max(lens), K ** -0.5, wl, shift, hk0, hv0, do, dlse, dhk, dhv)
        compare(o_g, g_g, o_o, g_o)


@pytest.mark.parametrize('HQ,H,K', [(2, 2, 64), (4, 2, 128)])
def test_backward_with_strong_gates(HQ, H, K):
    """Gates of about -3 nats per token: most chunks decay by more than the single-reference tensor-memory kernels
    accept, so the forward flags them and the general kernels (one reference per 16 rows) produce their outputs AND
    gradients; chunks of the same call that stay below the bound take the tensor-memory kernels."""
    T, M = 260, 64
    d = gen.layer_inputs(8800 + K, 1, T, HQ, H, K, K, M, gate_div=1.0, val_scale=1.0)
    g = d['g'].float() * 3.0 - 1.0
    g[:, 64:128] = d['g'][:, 64:128].float() / 8.0                  # one chunk with weak gates in the middle
    d['g'] = g.to(torch.bfloat16)
    d['s'] = (1 - d['g'].float().exp()).to(torch.bfloat16)
    x = flat_inputs(d, 1, T)
    do = d['do'].reshape(T, HQ, K).float()
    o_o, g_o = run_oracle(x, [0, T], K ** -0.5, 63, 64, None, None, do, None)
    o_g, g_g = run_gpu(x, [0, T], T, K ** -0.5, 63, 64, None, None, do, None)
    for n in NAMES:
        assert torch.isfinite(g_g[n].float()).all(), n
    compare(o_g, g_g, o_o, g_o)


def test_headline_shape_slice():
    """The fwd+bwd workload's shape (H=16, D=64, M=64, W=64, gates logsigmoid(N(0,1)), values N(0,1)/8)
    on a slice short enough for the oracle, both window conventions."""
    B, T, H, K, M = 2, 256, 16, 64, 64
    d = gen.layer_inputs(2024, B, T, H, H, K, K, M, gate_div=1.0)
    x = flat_inputs(d, B, T)
    cu = [0, T, 2 * T]
    do = d['do'].reshape(B * T, H, K).float()
    for wl, shift in ((64, 0), (63, 64)):
        o_o, g_o = run_oracle(x, cu, K ** -0.5, wl, shift, None, None, do, None)
        o_g, g_g = run_gpu(x, cu, T, K ** -0.5, wl, shift, None, None, do, None, batched_B=B)
        compare(o_g, g_g, o_o, g_o)


def test_api_errors():
    from nha_b200 import chunk_nha
    x = torch.zeros(1, 8, 2, 64, device='cuda', dtype=torch.bfloat16)
    sg = torch.zeros(1, 8, 2, 16, device='cuda', dtype=torch.bfloat16)
    with pytest.raises(DeprecationWarning):
        chunk_nha(x, x, x, x, x, sg, sg, head_first=True)
    with pytest.raises(AssertionError):
        chunk_nha(x[0], x[0], x[0], x[0], x[0], sg[0], sg[0])
    out = chunk_nha(x, x, x, x, x, sg, sg, window_size_left=4, window_size_right=0)
    assert len(out) == 3 and out[0].shape == (1, 8, 2, 64) and out[1].dtype == torch.float32


def test_many_tiny_sequences_in_one_packing():
    """More (sequence, kv head) pairs than a grid's y dimension holds (65535): 4200 sequences of 1-3 tokens with 16 kv
    heads.  Forward and backward must run (the scans put the pairs in the grid's x dimension) and a handful of the
    sequences are checked against the oracle."""
    from nha_b200 import chunk_nha
    N, H, K, M = 4200, 16, 64, 16
    g0 = torch.Generator().manual_seed(77)
    lens = torch.randint(1, 4, (N,), generator=g0).tolist()
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    T = cu[-1]
    d = gen.layer_inputs(7001, 1, T, H, H, K, K, M, gate_div=1.0)
    x = flat_inputs(d, 1, T)
    dev = 'cuda'
    xs = {n: x[n][None].to(dev).requires_grad_(True) for n in NAMES}
    o, ls, lg = chunk_nha(xs['q_swa'], xs['k_swa'], xs['q_gsa'], xs['k_gsa'], xs['v'], xs['s'], xs['g'],
                          cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), max_seqlen=3, scale=K ** -0.5,
                          window_size_left=1, window_size_right=0, gsa_kv_shift=1)
    o.float().sum().backward()
    assert torch.isfinite(o.float()).all() and all(torch.isfinite(xs[n].grad.float()).all() for n in NAMES)
    for n in (0, 1, 2099, N - 1):
        a, b = cu[n], cu[n + 1]
        sl = {k: x[k][a:b].double() for k in NAMES}
        want = orc.nha_varlen(sl['q_gsa'], sl['q_swa'], sl['k_gsa'], sl['k_swa'], sl['v'], sl['s'], sl['g'], [0, b - a],
                              K ** -0.5, 1, 1, None, None)
        assert_close(o[0, a:b], want[0], TOL_OUT, f'o of sequence {n}')
