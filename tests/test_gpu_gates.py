"""GPU: the fused slot-gate kernels against the oracle's fp64 gate chain (nha_fla/layers/nha.py:229-231)."""
import ctypes

import pytest
import torch
import torch.nn.functional as F

from oracle import nha_oracle as orc
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu

# one bf16 rounding per output against fp64: 2^-9 relative per element
TOL_GATE = 4e-3
TOL_GATE_GRAD = 6e-3


@pytest.mark.parametrize('shape,norm', [((2, 160, 4, 64), 8.0), ((1, 2048, 16, 64), 1.0), ((3, 7, 5), 8.0), ((8,), 2.0),
                                        ((0, 4, 16), 8.0)])
def test_slot_gates_forward_backward(shape, norm):
    from nha_b200 import slot_gates
    gen = torch.Generator().manual_seed(17)
    f = (torch.randn(*shape, generator=gen) * 3).bfloat16()
    dg = torch.randn(*shape, generator=gen).bfloat16()
    ds = torch.randn(*shape, generator=gen).bfloat16()
    fx = f.cuda().requires_grad_(True)
    g, s = slot_gates(fx, norm)
    assert g.dtype == torch.bfloat16 and g.shape == f.shape and s.shape == f.shape
    fo = f.double().requires_grad_(True)
    go, so = orc.slot_gates(fo, norm)
    if f.numel() == 0:
        return
    assert_close(g, go, TOL_GATE, 'g')
    assert_close(s, so, TOL_GATE, 's')
    assert (g.float() <= 0).all() and (s.float() >= 0).all() and (s.float() <= 1).all()
    # s is computed from the ROUNDED g, so the pair the operator sees is consistent: at most the last bf16 bit apart
    # from 1 - exp(g) evaluated on the bf16 g
    want_s = -torch.expm1(g.double())
    assert ((s.double() - want_s).abs() <= want_s * 2.0 ** -7 + 1e-30).all()
    torch.autograd.backward([g, s], [dg.cuda(), ds.cuda()])
    torch.autograd.backward([go, so], [dg.double(), ds.double()])
    assert_close(fx.grad, fo.grad, TOL_GATE_GRAD, 'df')


def test_slot_gates_one_sided_gradients_and_extremes():
    from nha_b200 import slot_gates
    f = torch.tensor([-80.0, -20.0, -1.0, 0.0, 1.0, 20.0, 80.0, 3.0] * 5 + [0.5, -0.5, 7.0]).bfloat16()
    for which in (0, 1):
        fx = f.cuda().requires_grad_(True)
        out = slot_gates(fx, 8.0)
        fo = f.double().requires_grad_(True)
        ref = orc.slot_gates(fo, 8.0)
        assert torch.isfinite(out[0].float()).all() and torch.isfinite(out[1].float()).all()
        assert_close(out[which], ref[which], TOL_GATE, 'output')
        out[which].sum().backward()
        ref[which].sum().backward()
        assert torch.isfinite(fx.grad.float()).all()
        assert_close(fx.grad, fo.grad, TOL_GATE_GRAD, 'df (one output used)')


def test_slot_gates_feed_the_operator():
    """g, s from the fused kernel give the same operator output as g, s from the layer's torch chain, up to the
    chain's extra bf16 roundings."""
    from nha_b200 import chunk_nha, slot_gates
    from tests import inputs as gen
    d = gen.layer_inputs(5, 2, 192, 2, 2, 64, 64, 64)
    gtor = torch.Generator().manual_seed(9)
    f = torch.randn(2, 192, 2, 64, generator=gtor).bfloat16().cuda()
    g, s = slot_gates(f, 8.0)
    g_t = F.logsigmoid(f) / 8.0
    s_t = (1 - g_t.exp()).to(g_t.dtype)
    x = {n: d[n].cuda() for n in ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v')}
    o1 = chunk_nha(x['q_swa'], x['k_swa'], x['q_gsa'], x['k_gsa'], x['v'], s, g, window_size_left=64,
                   window_size_right=0)[0]
    o2 = chunk_nha(x['q_swa'], x['k_swa'], x['q_gsa'], x['k_gsa'], x['v'], s_t, g_t, window_size_left=64,
                   window_size_right=0)[0]
    assert_close(o1, o2.double().cpu(), 2e-2, 'operator output on fused gates vs torch-chain gates')


def test_slot_gates_rejects_bad_arguments():
    from nha_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(64, dtype=torch.bfloat16, device='cuda')
    assert lib.nha_slot_gates_fwd(None, x.data_ptr(), x.data_ptr(), 64, 8.0, None) == 1
    assert lib.nha_slot_gates_fwd(x.data_ptr(), x.data_ptr(), x.data_ptr(), 64, 0.0, None) == 1
    assert lib.nha_slot_gates_fwd(x.data_ptr() + 2, x.data_ptr(), x.data_ptr(), 8, 8.0, None) == 1
    assert lib.nha_slot_gates_bwd(x.data_ptr(), None, None, x.data_ptr(), 64, 8.0, None) == 1
