"""GPU: fused decode step / recurrent step through the C ABI against the oracle and the fixtures."""
import json
import os

import numpy as np
import pytest
import torch

from oracle import nha_oracle as orc
from tests import inputs as gen
from tests.gpu_util import TOL_OUT, assert_close, cuda

pytestmark = pytest.mark.gpu
GOLD = os.path.join(os.path.dirname(__file__), 'golden')
MAN = json.load(open(os.path.join(GOLD, 'manifest.json')))

# the reference's decode grid (scripts/verify_opt_parity.py:322-329), incl. the non-power-of-two M = 80
GRID = [(NG, M, W, K, B) for NG in (1, 4, 8) for M in (16, 64, 80) for W in (32, 64) for K in (64, 128) for B in (1, 4)]


def _seed(i):
    return 2000 + i


@pytest.mark.parametrize('idx', range(len(GRID)))
def test_decode_grid(idx):
    from nha_b200 import fused_recurrent_nha_decode
    NG, M, W, K, B = GRID[idx]
    d = gen.decode_inputs(_seed(idx), B, 2, NG, K, K, M, W)
    ref_o, ref_hk, ref_hv, _, _ = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'],
                                                  s=d['s'], cos=d['cos'], sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    c = cuda(d)
    # in-kernel rotary, s recomputed from g in-kernel
    ref2 = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'],
                           cos=d['cos'], sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'],
                                             cos=c['cos'], sin=c['sin'],
                                             initial_state=(c['hk0'].clone(), c['hv0'].clone()),
                                             output_final_state=True, scale=d['scale'])
    assert_close(o, ref2[0], TOL_OUT, 'o (rotary)')
    assert_close(hk, ref2[1], 1e-5, 'hkt (rotary)')
    assert_close(hv, ref2[2], 1e-5, 'hvt (rotary)')
    # pre-rotated query/keys and caller-supplied s
    hk0, hv0 = c['hk0'].clone(), c['hv0'].clone()
    o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], sq=c['sq'], k=c['k'], v=c['v'], g=c['g'], s=c['s'],
                                             sw_k=c['sk'], sw_v=c['vw'], initial_state=(hk0, hv0),
                                             output_final_state=True, scale=d['scale'])
    assert_close(o, ref_o, TOL_OUT, 'o (eager)')
    assert_close(hk, ref_hk, 1e-5, 'hkt (eager)')
    assert_close(hv, ref_hv, 1e-5, 'hvt (eager)')
    assert hk.data_ptr() == hk0.data_ptr(), 'state must be updated in place'
    # no final state requested: the caller's state must stay untouched
    keep = c['hk0'].clone()
    o2, st = fused_recurrent_nha_decode(q=c['q'], sq=c['sq'], k=c['k'], v=c['v'], g=c['g'], s=c['s'], sw_k=c['sk'],
                                        sw_v=c['vw'], initial_state=(keep, c['hv0'].clone()), scale=d['scale'])
    assert st == (None, None) and torch.equal(keep, c['hk0'])
    assert torch.equal(o2, o)


@pytest.mark.parametrize('idx', range(0, len(GRID), 3))
def test_recurrent_grid(idx):
    from nha_b200 import fused_recurrent_nha
    NG, M, W, K, B = GRID[idx]
    d = gen.recurrent_inputs(1000 + idx, B, 2, NG, K, K, M, W)
    ref_o, ref_pw, ref_hk, ref_hv = orc.recurrent_step(d['q'], d['k'], d['v'], d['sliding_window'], d['s'], d['g'],
                                                       d['scale'], d['hk0'], d['hv0'])
    c = cuda(d)
    o, pw, (hk, hv) = fused_recurrent_nha(c['q'], c['k'], c['v'], c['sliding_window'], c['s'], c['g'],
                                          scale=d['scale'], initial_state=(c['hk0'].clone(), c['hv0'].clone()),
                                          output_final_state=True)
    assert_close(o, ref_o, TOL_OUT, 'o')
    assert_close(pw, ref_pw, TOL_OUT, 'swa_score')
    assert_close(hk, ref_hk, 1e-5, 'hkt')
    assert_close(hv, ref_hv, 1e-5, 'hvt')


@pytest.mark.parametrize('case', sorted(MAN['decode']))
def test_decode_against_reference_fixture(case):
    from nha_b200 import fused_recurrent_nha_decode
    c = MAN['decode'][case]
    z = np.load(os.path.join(GOLD, 'decode.npz'))
    d = gen.decode_inputs(c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'])
    assert gen.digest(d) == c['digest']
    g = cuda(d)
    o, (hk, hv) = fused_recurrent_nha_decode(q=g['q'], k=g['k'], v=g['v'], g=g['g'], s=g['s'], sw_k=g['sw_k_raw'],
                                             sw_v=g['vw'], cos=g['cos'], sin=g['sin'],
                                             initial_state=(g['hk0'].clone(), g['hv0'].clone()),
                                             output_final_state=True, scale=d['scale'])
    assert_close(o, torch.from_numpy(z[f'{case}/o']), TOL_OUT, 'o')
    assert_close(hk, torch.from_numpy(z[f'{case}/hkt']), 1e-5, 'hkt')
    assert_close(hv, torch.from_numpy(z[f'{case}/hvt']), 1e-5, 'hvt')


def test_decode_edge_cases():
    """Zero state, a window shorter than 16 keys, a dummy popped entry, T != 1 and autograd misuse."""
    from nha_b200 import fused_recurrent_nha, fused_recurrent_nha_decode
    d = gen.decode_inputs(77, 2, 2, 4, 64, 64, 32, 5)
    d['k'].zero_(); d['v'].zero_(); d['g'].zero_()
    ref = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'], cos=d['cos'], sin=d['sin'])
    c = cuda(d)
    o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'],
                                             cos=c['cos'], sin=c['sin'], initial_state=(None, None),
                                             output_final_state=True)
    assert_close(o, ref[0], TOL_OUT, 'o')
    assert float(hk.abs().max()) == 0.0 and float(hv.abs().max()) == 0.0
    with pytest.raises(ValueError):
        fused_recurrent_nha(c['q'].repeat(1, 2, 1, 1), c['k'], c['v'], c['sliding_window'], c['s'], c['g'])
    with pytest.raises(AssertionError):
        fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'])


def test_decode_headline_shape():
    """One layer of the batched-decode workload: HQ=32, H=4, D=128, M=64, W=512, rotary in-kernel."""
    from nha_b200 import fused_recurrent_nha_decode
    torch.manual_seed(5)
    B, H, NG, K, M, W = 3, 4, 8, 128, 64, 512
    d = gen.decode_inputs(5, B, H, NG, K, K, M, W)
    d['cos'], d['sin'] = gen.rope_tables(W, K, first_pos=32768 - W + 1)
    ref = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'], cos=d['cos'],
                          sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    c = cuda(d)
    o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'],
                                             cos=c['cos'], sin=c['sin'], initial_state=(c['hk0'], c['hv0']),
                                             output_final_state=True)
    assert_close(o, ref[0], TOL_OUT, 'o')
    assert_close(hk, ref[1], 1e-5, 'hkt')
    assert_close(hv, ref[2], 1e-5, 'hvt')


@pytest.mark.parametrize('B', [1, 3, 40])
def test_decode_general_kernel_matches_streaming_kernel(B, monkeypatch):
    """K == V in {64, 128} normally takes the streaming kernel; NHA_B200_DECODE_GENERAL=1 forces the
    general one.  Both must agree with the oracle on the headline layer shape at batch sizes that give
    different split counts (few sequences: many splits per kv head; many: none)."""
    from nha_b200 import fused_recurrent_nha_decode
    H, NG, K, M, W = 4, 8, 128, 64, 512
    d = gen.decode_inputs(70 + B, B, H, NG, K, K, M, W)
    d['cos'], d['sin'] = gen.rope_tables(W, K, first_pos=32768 - W + 1)
    ref = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'], cos=d['cos'],
                          sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    c = cuda(d)
    outs = []
    for force in ('0', '1'):
        monkeypatch.setenv('NHA_B200_DECODE_GENERAL', force)
        o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'],
                                                 sw_v=c['vw'], cos=c['cos'], sin=c['sin'],
                                                 initial_state=(c['hk0'].clone(), c['hv0'].clone()),
                                                 output_final_state=True)
        assert_close(o, ref[0], TOL_OUT, f'o (general={force})')
        assert_close(hk, ref[1], 1e-5, f'hkt (general={force})')
        assert_close(hv, ref[2], 1e-5, f'hvt (general={force})')
        outs.append(o.float())
    assert (outs[0] - outs[1]).abs().max() < 2e-2


@pytest.mark.parametrize('B', [2, 32])
def test_decode_cluster_merge_matches_workspace_merge(B, monkeypatch):
    """The splits of a (sequence, kv head) merge through the cluster's shared memory; NHA_B200_DECODE_NO_CLUSTER=1
    makes the same kernel merge through the workspace (the path taken when a cluster cannot be launched or the
    split count is not 2, 4 or 8).  Same partial results, so the states agree bit for bit and the outputs to
    rounding of the merge weights."""
    from nha_b200 import fused_recurrent_nha_decode
    H, NG, K, M, W = 4, 8, 128, 64, 512
    d = gen.decode_inputs(90 + B, B, H, NG, K, K, M, W)
    d['cos'], d['sin'] = gen.rope_tables(W, K, first_pos=32768 - W + 1)
    ref = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'], cos=d['cos'],
                          sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    c = cuda(d)
    res = []
    for off in ('0', '1'):
        monkeypatch.setenv('NHA_B200_DECODE_NO_CLUSTER', off)
        o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'],
                                                 sw_v=c['vw'], cos=c['cos'], sin=c['sin'],
                                                 initial_state=(c['hk0'].clone(), c['hv0'].clone()),
                                                 output_final_state=True)
        assert_close(o, ref[0], TOL_OUT, f'o (no_cluster={off})')
        res.append((o.float(), hk, hv))
    monkeypatch.setenv('NHA_B200_DECODE_NO_CLUSTER', '0')
    assert torch.equal(res[0][1], res[1][1]) and torch.equal(res[0][2], res[1][2])
    assert (res[0][0] - res[1][0]).abs().max() < 1e-2


@pytest.mark.parametrize('B', [2, 48])
def test_decode_with_a_2048_key_window(B):
    """The window of the model classes' wide layers (2048 keys), few and many sequences: the streaming kernel splits a
    (sequence, kv head) until a split holds at most 512 keys, whatever the batch."""
    from nha_b200 import fused_recurrent_nha_decode
    H, NG, K, M, W = 2, 4, 128, 64, 2048
    d = gen.decode_inputs(500 + B, B, H, NG, K, K, M, W)
    d['cos'], d['sin'] = gen.rope_tables(W, K, first_pos=5000)
    ref = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'], cos=d['cos'],
                          sin=d['sin'], hk0=d['hk0'], hv0=d['hv0'])
    c = cuda(d)
    o, (hk, hv) = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'],
                                             cos=c['cos'], sin=c['sin'], initial_state=(c['hk0'], c['hv0']),
                                             output_final_state=True)
    assert_close(o, ref[0], TOL_OUT, 'o')
    assert_close(hk, ref[1], 1e-5, 'hkt')
    assert_close(hv, ref[2], 1e-5, 'hvt')


@pytest.mark.parametrize('B,H,NG,K,M,W', [(3, 2, 4, 128, 64, 256), (32, 4, 8, 128, 64, 512), (2, 1, 1, 64, 64, 130),
                                          (1, 1, 2, 64, 32, 64)])
def test_decode_with_bf16_slot_memory(B, H, NG, K, M, W):
    """The slot memory kept in bf16 (an extension; the reference keeps it in fp32): three steps in a row on the same
    window with the state carried in bf16, against the oracle stepping in fp64 from the same bf16-rounded start state.
    Outputs to the usual bar; states to bf16 rounding (one rounding per step and element)."""
    from nha_b200 import fused_recurrent_nha_decode_bf16_state
    d = gen.decode_inputs(700 + B, B, H, NG, K, K, M, W)
    d['cos'], d['sin'] = gen.rope_tables(W, K, first_pos=900)
    c = cuda(d)
    hk = c['hk0'].bfloat16().contiguous()
    hv = c['hv0'].bfloat16().contiguous()
    rk, rv = hk.double().cpu(), hv.double().cpu()
    for step in range(3):
        ref = orc.decode_step(d['q'], d['k'], d['v'], d['g'], d['sw_k_raw'], d['vw'], d['scale'], cos=d['cos'],
                              sin=d['sin'], hk0=rk, hv0=rv)
        o, (hk2, hv2) = fused_recurrent_nha_decode_bf16_state(
            q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'], cos=c['cos'], sin=c['sin'],
            initial_state=(hk, hv), output_final_state=True)
        assert hk2.dtype == torch.bfloat16 and hk2.data_ptr() == hk.data_ptr(), 'bf16 states are updated in place'
        assert_close(o, ref[0], TOL_OUT, f'step {step} o')
        assert_close(hk2, ref[1], 6e-3 * (step + 1), f'step {step} hkt')
        assert_close(hv2, ref[2], 6e-3 * (step + 1), f'step {step} hvt')
        rk, rv = ref[1], ref[2]


def test_bf16_slot_memory_is_refused_without_the_streaming_kernel():
    from nha_b200 import fused_recurrent_nha_decode_bf16_state
    from nha_b200._lib import NHALibraryError
    d = gen.decode_inputs(710, 1, 1, 1, 32, 32, 16, 16)                      # K = 32: general kernel only
    d['cos'], d['sin'] = gen.rope_tables(16, 32, first_pos=0)
    c = cuda(d)
    with pytest.raises(NHALibraryError):
        fused_recurrent_nha_decode_bf16_state(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'], sw_v=c['vw'],
                                              cos=c['cos'], sin=c['sin'], initial_state=(c['hk0'], c['hv0']),
                                              output_final_state=True)


@pytest.fixture
def pdl_mode():
    """Sets the dependent-launch mode of the streaming decode kernel for a test and restores the default."""
    from nha_b200 import _lib
    lib = _lib.load()
    before = lib.nha_decode_get_pdl()
    yield lambda m: _lib.check(lib.nha_decode_set_pdl(m), 'nha_decode_set_pdl')
    lib.nha_decode_set_pdl(before)


@pytest.mark.parametrize('B', [3, 32])
def test_dependent_launch_modes_agree_on_a_stack_of_layers(B, pdl_mode):
    """Six layers with their own slot memory and window, decoded back to back for two tokens: plain launches (0),
    dependent launches that wait before their first read (1), and dependent launches that request the layer's state
    and window before the wait (2; allowed here because the kernel in front belongs to another layer).  Layer 0 of
    the first token is checked against the oracle; all modes must give the same bits."""
    from nha_b200 import NHARingCache, fused_recurrent_nha_decode
    H, NG, K, M, W, L, STEPS = 4, 8, 128, 64, 512, 6, 2
    layers = [gen.decode_inputs(300 + i, B, H, NG, K, K, M, W) for i in range(L)]
    cos, sin = gen.rope_tables(W, K, first_pos=32768 - W + 1)
    d0 = layers[0]
    ref = orc.decode_step(d0['q'], d0['k'], d0['v'], d0['g'], d0['sw_k_raw'], d0['vw'], d0['scale'], cos=cos, sin=sin,
                          hk0=d0['hk0'], hv0=d0['hv0'])
    cl = [cuda(d) for d in layers]
    cosd, sind = cos.cuda(), sin.cuda()
    results = {}
    for mode in (0, 1, 2):
        pdl_mode(mode)
        st = [(c['hk0'].clone(), c['hv0'].clone()) for c in cl]
        outs = []
        for _ in range(STEPS):
            for i, c in enumerate(cl):
                o, st[i] = fused_recurrent_nha_decode(q=c['q'], k=c['k'], v=c['v'], g=c['g'], sw_k=c['sw_k_raw'],
                                                      sw_v=c['vw'], cos=cosd, sin=sind, initial_state=st[i],
                                                      output_final_state=True)
                outs.append(o)
        # the same stack on ring caches (decode + append per layer)
        cache = NHARingCache()
        for i, c in enumerate(cl):
            cache.init_layer(i, c['sw_k_raw'], c['vw'], (c['g'].expand(B, W, H, M) * 0.5).contiguous(), W,
                             (c['hk0'], c['hv0']))
        routs = []
        for _ in range(STEPS + 1):
            for i, c in enumerate(cl):
                routs.append(cache.decode(i, c['q'], c['k'], c['v'], c['g'], cosd, sind))
        torch.cuda.synchronize()
        results[mode] = (outs, [x for pair in st for x in pair], routs, [cache[i].hk for i in range(L)])
    assert_close(results[0][0][0], ref[0], TOL_OUT, 'o of layer 0 (plain launches)')
    for mode in (1, 2):
        for part in range(4):
            for a, b in zip(results[0][part], results[mode][part]):
                assert torch.equal(a, b), f'mode {mode} differs from plain launches'
