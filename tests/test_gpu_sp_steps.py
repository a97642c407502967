"""GPU, one device: the arithmetic of the sequence-parallel prefill with the ranks emulated one after another.

The exchange steps (halo, all-gather) are host plumbing that the gloo test covers; what needs a GPU is the engine the
ranks run: one state pass from a zero start, the start state folded into the chunk-start states afterwards
(nha_chunk_apply_state_prefix), and an output pass whose query tensors start W positions later than its kv-head tensors
(q_offset).  Here every emulated rank builds its halo-extended kv tensors from the full inputs, the summaries are
stacked as the all-gather would stack them, and the outputs of all ranks are compared with the single-call op and the
oracle.  The long-context layer shape takes the three-step path, the other shape the fallback (halo-extended queries).
"""
import pytest
import torch

from oracle import nha_oracle as orc
from tests import inputs as gen
from tests.gpu_util import TOL_OUT, assert_close, cuda

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize('K,M,NG,W,T,world,with_state', [(128, 64, 4, 128, 1152, 3, True), (128, 64, 2, 64, 640, 2, False),
                                                         (64, 32, 2, 32, 400, 2, True)])
def test_emulated_ranks_match_the_single_call(K, M, NG, W, T, world, with_state):
    from nha_b200 import fused_chunk_nha_prefill
    from nha_b200.sharding import CudaEngine
    H = 2
    d = gen.prefill_inputs(6000 + K + W, 1, H, NG, K, K, M, W, T, with_state)
    ref_o, ref_hk, ref_hv = orc.prefill(d['q'], d['k'], d['v'], d['rotary_q'], d['rotary_k'], d['s'], d['g'], W,
                                        d['scale'], d.get('hk0'), d.get('hv0'))
    c = cuda(d)
    st = (c['hk0'], c['hv0']) if with_state else None
    one_o, (one_hk, one_hv) = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'],
                                                      rotary_k=c['rotary_k'], s=c['s'], g=c['g'], window_size=W,
                                                      initial_state=st, output_final_state=True)
    bounds = [T * r // world // 64 * 64 for r in range(world)] + [T]
    engines, packs = [], []
    for r in range(world):
        a, b = bounds[r], bounds[r + 1]
        lo = a - W if r > 0 else a
        seg = lambda x: x[:, a:b].contiguous()
        ext = lambda x: x[:, lo:b].contiguous()
        eng = CudaEngine(seg(c['q']), seg(c['rotary_q']), ext(c['k']), ext(c['rotary_k']), ext(c['v']), ext(c['s']),
                         ext(c['g']), W, d['scale'], a - lo)
        if K == 128:
            assert eng.steps is not None, 'the long-context shape must take the three-step path'
        engines.append(eng)
        if r % 2 == 1:
            # the early start (per-chunk terms of the chunks that do not read the halo rows) followed by the rest must
            # give the same message as the state pass in one go
            want = eng.summary().clone()
            eng.start()
            got = eng.summary().clone()
            assert torch.equal(got, want), 'split state pass differs from the one-call state pass'
        packs.append(eng.summary().clone())
    allp = torch.stack(packs, 0)                       # [world, B, P], as the all-gather leaves it
    outs = []
    for r in range(world):
        o, hk, hv = engines[r].finish(allp, r, st)
        outs.append(o)
    o = torch.cat(outs, 1)
    assert_close(o, ref_o, TOL_OUT, 'o vs oracle')
    assert_close(hk, ref_hk, TOL_OUT, 'final hk vs oracle')
    assert_close(hv, ref_hv, TOL_OUT, 'final hv vs oracle')
    assert_close(o, one_o.float().cpu(), 1e-2, 'o vs single call')
    assert_close(hk, one_hk.cpu(), 5e-3, 'final hk vs single call')
