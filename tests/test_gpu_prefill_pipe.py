"""GPU: the warp-specialised output pass (head dim 128, query heads in groups of four) against the oracle.

The kernel differs from the other output-pass kernels in everything but the mathematics (TMA-fed operand ring, one
thread per row, one-sweep softmax with a lazily raised reference and rescaling of the accumulator in tensor memory),
so it gets its own cases: windows from one key to unbounded, ragged and one-token sequences in a packing, initial
states, eight query heads per kv head, rows whose window logits dwarf their slot logits (forces the rescaling path)
and chunks with gates strong enough to be handed to the general kernel.  NHA_B200_NO_PIPE=1 selects the older kernel;
both must agree with the oracle and with each other.
"""
import pytest
import torch

from oracle import nha_oracle as orc
from tests import inputs as gen
from tests.gpu_util import TOL_OUT, assert_close

pytestmark = pytest.mark.gpu
NAMES = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')


def _run(x, cu, maxlen, scale, wl, shift, hk0, hv0):
    from nha_b200 import chunk_nha
    dev = 'cuda'
    a = {n: x[n][None].to(dev) for n in NAMES}
    st = None if hk0 is None else (hk0.to(dev), hv0.to(dev))
    wl_a = torch.tensor(wl, dtype=torch.int32, device=dev) if isinstance(wl, (list, tuple)) else wl
    sh_a = torch.tensor(shift, dtype=torch.int32, device=dev) if isinstance(shift, (list, tuple)) else shift
    o, ls, lg, (hk, hv) = chunk_nha(a['q_swa'], a['k_swa'], a['q_gsa'], a['k_gsa'], a['v'], a['s'], a['g'],
                                    cu_seqlens=torch.tensor(cu, dtype=torch.int32, device=dev), max_seqlen=maxlen,
                                    scale=scale, window_size_left=wl_a, window_size_right=0, gsa_kv_shift=sh_a,
                                    initial_state=st, output_final_state=True)
    return o[0], ls[0], lg[0]


def _check(x, cu, scale, wl, shift, hk0, hv0, monkeypatch, tol=TOL_OUT):
    xs = {n: x[n].double() for n in NAMES}
    want = orc.nha_varlen(xs['q_gsa'], xs['q_swa'], xs['k_gsa'], xs['k_swa'], xs['v'], xs['s'], xs['g'], cu, scale, wl,
                          shift, None if hk0 is None else hk0.double(), None if hv0 is None else hv0.double())
    maxlen = max(b - a for a, b in zip(cu[:-1], cu[1:]))
    outs = {}
    for off in ('0', '1'):
        monkeypatch.setenv('NHA_B200_NO_PIPE', off)
        got = _run(x, cu, maxlen, scale, wl, shift, hk0, hv0)
        for g_, w_, name in zip(got, want[:3], ('o', 'lse_swa', 'lse_gsa')):
            assert torch.isfinite(g_.float()).all(), f'{name} (no_pipe={off})'
            assert_close(g_, w_, tol, f'{name} (no_pipe={off})')
        outs[off] = got
    assert_close(outs['0'][0], outs['1'][0].float().cpu(), 1e-2, 'pipelined vs non-pipelined o')


@pytest.mark.parametrize('wl,shift', [(511, 512), (63, 64), (64, 0), (0, 1), (200, 0), (-1, 0), (130, 70)])
def test_windows_and_shifts(wl, shift, monkeypatch):
    T, HQ, H, K, M = 700, 4, 1, 128, 64
    d = gen.layer_inputs(4100 + wl + shift, 1, T, HQ, H, K, K, M, gate_div=8.0, val_scale=1.0)
    x = {n: d[n][0] for n in NAMES}
    torch.manual_seed(wl + 7)
    hk0, hv0 = torch.randn(1, H, K, M) * 0.5, torch.randn(1, H, M, K) * 0.5
    _check(x, [0, T], K ** -0.5, wl, shift, hk0, hv0, monkeypatch)


def test_packed_ragged_sequences_with_their_own_windows(monkeypatch):
    lens = [1, 130, 64, 3, 257, 65, 2, 191]
    wls = [31, 63, 127, 15, 255, 511, 7, 100]
    shs = [w + 1 for w in wls[:4]] + [0, 0, 0, 0]
    cu = [0]
    for L in lens:
        cu.append(cu[-1] + L)
    T, HQ, H, K, M = cu[-1], 8, 2, 128, 64
    d = gen.layer_inputs(4242, 1, T, HQ, H, K, K, M, gate_div=4.0, val_scale=1.0)
    x = {n: d[n][0] for n in NAMES}
    _check(x, cu, K ** -0.5, wls, shs, None, None, monkeypatch)


def test_eight_query_heads_per_kv_head(monkeypatch):
    T, HQ, H, K, M = 300, 16, 2, 128, 64
    d = gen.layer_inputs(4343, 1, T, HQ, H, K, K, M, gate_div=8.0, val_scale=1.0)
    x = {n: d[n][0] for n in NAMES}
    _check(x, [0, 100, T], K ** -0.5, 127, 128, None, None, monkeypatch)


def test_window_logits_far_above_slot_logits(monkeypatch):
    """Queries and window keys ten times larger than the slot branch's: the reference of every row is raised (and its
    accumulator rescaled) when the first window tile arrives, and again where an older tile holds the row's maximum."""
    T, HQ, H, K, M = 400, 4, 1, 128, 64
    d = gen.layer_inputs(4444, 1, T, HQ, H, K, K, M, gate_div=8.0, val_scale=1.0)
    x = {n: d[n][0] for n in NAMES}
    x['q_swa'] = (x['q_swa'].float() * 3.0).to(torch.bfloat16)
    x['k_swa'] = (x['k_swa'].float() * 3.0).to(torch.bfloat16)
    # a few keys far in the past with a very large norm: the maximum of later rows sits in an old tile
    x['k_swa'][5] = (x['k_swa'][5].float() * 4.0).to(torch.bfloat16)
    x['k_swa'][70] = (x['k_swa'][70].float() * 4.0).to(torch.bfloat16)
    _check(x, [0, T], K ** -0.5, 300, 0, None, None, monkeypatch)


def test_strong_gates_are_left_to_the_general_kernel(monkeypatch):
    T, HQ, H, K, M = 260, 4, 1, 128, 64
    d = gen.layer_inputs(4545, 1, T, HQ, H, K, K, M, gate_div=1.0, val_scale=1.0)
    g = d['g'].float() * 3.0 - 1.0
    g[:, 64:128] = d['g'][:, 64:128].float() / 8.0
    d['g'] = g.to(torch.bfloat16)
    d['s'] = (1 - d['g'].float().exp()).to(torch.bfloat16)
    x = {n: d[n][0] for n in NAMES}
    _check(x, [0, T], K ** -0.5, 63, 64, None, None, monkeypatch)
