"""GPU: chunked forward (state pass + output pass) through the C ABI against the oracle."""
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

# the reference's prefill grid (scripts/verify_opt_parity.py:437-444); B = 4 only where the oracle stays fast
GRID = [(T, B, W, M) for T in (63, 128, 257, 1000) for B in (1, 4) for W in (32, 64) for M in (16, 64)
        if not (B == 4 and T == 1000)]


@pytest.mark.parametrize('T,B,W,M', GRID)
def test_prefill_grid(T, B, W, M):
    from nha_b200 import fused_chunk_nha_prefill
    d = gen.prefill_inputs(3000 + T + 7 * W + M + B, B, 2, 4, 64, 64, M, W, T, with_state=(T == 128))
    ref_o, ref_hk, ref_hv = orc.prefill(d['q'], d['k'], d['v'], d['rotary_q'], d['rotary_k'], d['s'], d['g'], W,
                                        d['scale'], d.get('hk0'), d.get('hv0'))
    c = cuda(d)
    o, (hk, hv) = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'], rotary_k=c['rotary_k'],
                                          window_size=W, s=c['s'], g=c['g'],
                                          initial_state=(c['hk0'], c['hv0']) if 'hk0' in c else None,
                                          output_final_state=True, scale=None)
    assert_close(o, ref_o, TOL_OUT, 'o')
    assert_close(hk, ref_hk, TOL_OUT, 'hkt')
    assert_close(hv, ref_hv, TOL_OUT, 'hvt')
    o2, st = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'], rotary_k=c['rotary_k'],
                                     window_size=W, s=c['s'], g=c['g'],
                                     initial_state=(c['hk0'], c['hv0']) if 'hk0' in c else None)
    assert st == (None, None) and torch.equal(o2, o)


@pytest.mark.parametrize('case', sorted(MAN['prefill']))
def test_prefill_against_reference_fixture(case):
    from nha_b200 import fused_chunk_nha_prefill
    c = MAN['prefill'][case]
    z = np.load(os.path.join(GOLD, 'prefill.npz'))
    d = gen.prefill_inputs(c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'], c['T'], c['with_state'])
    assert gen.digest(d) == c['digest']
    g = cuda(d)
    o, (hk, hv) = fused_chunk_nha_prefill(q=g['q'], k=g['k'], v=g['v'], rotary_q=g['rotary_q'], rotary_k=g['rotary_k'],
                                          window_size=c['W'], s=g['s'], g=g['g'],
                                          initial_state=(g['hk0'], g['hv0']) if c['with_state'] else None,
                                          output_final_state=True)
    assert_close(o, torch.from_numpy(z[f'{case}/o']), TOL_OUT, 'o')
    assert_close(hk, torch.from_numpy(z[f'{case}/hkt']), TOL_OUT, 'hkt')
    assert_close(hv, torch.from_numpy(z[f'{case}/hvt']), TOL_OUT, 'hvt')


@pytest.mark.parametrize('K,M,W,T,NG', [(128, 64, 512, 700, 4), (128, 32, 100, 300, 2), (64, 64, 200, 500, 1),
                                         (32, 16, 8, 150, 2)])
def test_prefill_wide_window_and_head_dims(K, M, W, T, NG):
    """Windows wider than a chunk (the long-context shape: D=128, W=512, GQA) and other head dims."""
    from nha_b200 import fused_chunk_nha_prefill
    d = gen.prefill_inputs(9000 + K + W, 1, 2, NG, K, K, M, W, T, with_state=True)
    ref_o, ref_hk, ref_hv = orc.prefill(d['q'], d['k'], d['v'], d['rotary_q'], d['rotary_k'], d['s'], d['g'], W,
                                        d['scale'], d['hk0'], d['hv0'])
    c = cuda(d)
    o, (hk, hv) = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'], rotary_k=c['rotary_k'],
                                          window_size=W, s=c['s'], g=c['g'], initial_state=(c['hk0'], c['hv0']),
                                          output_final_state=True)
    assert_close(o, ref_o, TOL_OUT, 'o')
    assert_close(hk, ref_hk, TOL_OUT, 'hkt')
    assert_close(hv, ref_hv, TOL_OUT, 'hvt')


def test_chunk_start_states_against_the_oracle():
    """The state pass alone: the chunk-start states it leaves for the output pass and the backward are the
    oracle's slot memory at every 64th token (bf16 storage), and the final states its fp32 end value."""
    from nha_b200.chunk import chunk_forward
    B, T, H, K, M, W = 2, 300, 2, 64, 32, 16
    d = gen.prefill_inputs(4242, B, H, 2, K, K, M, W, T, with_state=True)
    c = cuda(d)
    flat = lambda x: x.reshape(B * T, *x.shape[2:]).contiguous()
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device='cuda')
    o, ls, lg, hk, hv, saved = chunk_forward(flat(c['q']), flat(c['rotary_q']), flat(c['k']), flat(c['rotary_k']),
                                             flat(c['v']), flat(c['s']), flat(c['g']), cu, T, d['scale'], W - 1, W,
                                             c['hk0'], c['hv0'], True)
    nc = (T + 63) // 64
    for b in range(B):
        hk_r, hv_r = d['hk0'][b].double(), d['hv0'][b].double()
        for t in range(T + 1):
            if t % 64 == 0 and t < T:
                ci = b * nc + t // 64
                assert_close(saved['hk_chunks'][ci], hk_r, TOL_OUT, f'hk_chunks[{b},{t // 64}]')
                assert_close(saved['hv_chunks'][ci], hv_r, TOL_OUT, f'hv_chunks[{b},{t // 64}]')
            j = t - W
            if t < T and j >= 0:
                hk_r, hv_r = orc.gsa_step(hk_r, hv_r, d['k'][b, j].double(), d['v'][b, j].double(),
                                          d['s'][b, j].double(), d['g'][b, j].double())
        assert_close(hk[b], hk_r, TOL_OUT, 'hkt')
        assert_close(hv[b], hv_r, TOL_OUT, 'hvt')


def test_strong_gates_stay_finite_and_exact():
    """Gates of -3 nats per token (192 nats per chunk): the per-row-block decay references must
    keep every factor in range, where a single per-chunk reference would overflow."""
    from nha_b200 import fused_chunk_nha_prefill
    d = gen.prefill_inputs(5151, 1, 2, 2, 64, 64, 32, 32, 300, with_state=True)
    d['g'] = (d['g'].float() * 24.0 - 1.0).to(torch.bfloat16)
    d['s'] = (1 - d['g'].float().exp()).to(torch.bfloat16)
    ref_o, ref_hk, ref_hv = orc.prefill(d['q'], d['k'], d['v'], d['rotary_q'], d['rotary_k'], d['s'], d['g'], 32,
                                        d['scale'], d['hk0'], d['hv0'])
    c = cuda(d)
    o, (hk, hv) = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'], rotary_k=c['rotary_k'],
                                          window_size=32, s=c['s'], g=c['g'], initial_state=(c['hk0'], c['hv0']),
                                          output_final_state=True)
    assert torch.isfinite(o.float()).all()
    assert_close(o, ref_o, TOL_OUT, 'o')
    assert_close(hk, ref_hk, TOL_OUT, 'hkt')
