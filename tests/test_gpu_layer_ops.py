"""GPU: the layer-side element-wise kernels around the operator against the fp64 oracle - feature map of q and k with
silu(v) in one launch (nha_fla/layers/nha.py:219-223) and silu + RMS norm in front of the output projection
(nha_fla/layers/nha.py:277-278), forward and backward."""
import pytest
import torch

from oracle import nha_oracle as orc

pytestmark = pytest.mark.gpu


def _rel(a, b):
    return orc.rel_l2(a.double().cpu(), b.double().cpu())


@pytest.mark.parametrize('fmap', ['swish', 'relu', None])
@pytest.mark.parametrize('shape', [(2, 130, 4, 64), (1, 7, 3, 20)])        # the second is not a multiple of 8 elements
def test_feature_maps_forward_and_backward(fmap, shape):
    from nha_b200 import feature_maps
    torch.manual_seed(5)
    B, T, H, D = shape
    q, k = (torch.randn(B, T, H, D) * 2).bfloat16(), (torch.randn(B, T, H, D) * 2).bfloat16()
    v = (torch.randn(B, T, max(1, H // 2), D) * 2).bfloat16()                   # v may have another shape than q and k
    dq, dk, dv = (torch.randn_like(x.float()).bfloat16() for x in (q, k, v))
    xs = [x.cuda().requires_grad_(True) for x in (q, k, v)]
    outs = feature_maps(*xs, feature_map=fmap)
    ref_in = [x.double().requires_grad_(True) for x in (q, k, v)]
    if fmap is None:
        ref = (ref_in[0], ref_in[1], orc.feature_maps(*ref_in, 'swish')[2])
    else:
        ref = orc.feature_maps(*ref_in, fmap)
    for got, want, name in zip(outs, ref, 'qkv'):
        assert got.dtype == torch.bfloat16 and _rel(got, want.detach()) < 5e-3, name
    torch.autograd.backward(list(outs), [g.cuda() for g in (dq, dk, dv)])
    torch.autograd.backward(list(ref), [g.double() for g in (dq, dk, dv)])
    for x, r, name in zip(xs, ref_in, 'qkv'):
        assert _rel(x.grad, r.grad) < 6e-3, f'd{name}'


@pytest.mark.parametrize('rows,cols,bias', [(300, 1024, True), (37, 256, False), (64, 2048, True), (5, 1280, True)])
def test_silu_rms_norm_linear_forward_and_backward(rows, cols, bias):
    from nha_b200 import silu_rms_norm, silu_rms_norm_linear
    torch.manual_seed(6)
    o = (torch.randn(rows, cols) * 2).bfloat16()
    w = torch.rand(cols) + 0.5
    b = torch.randn(cols) * 0.1 if bias else None
    dy = torch.randn(rows, cols).bfloat16()
    oc = o.cuda().requires_grad_(True)
    wc = w.cuda().requires_grad_(True)
    bc = b.cuda().requires_grad_(True) if bias else None
    y = silu_rms_norm(oc, wc, bc, 1e-5)
    o64 = o.double().requires_grad_(True)
    w64 = w.double().requires_grad_(True)
    b64 = b.double().requires_grad_(True) if bias else None
    want = orc.silu_rms_norm(o64, w64, b64, 1e-5)
    assert y.dtype == torch.bfloat16 and _rel(y, want.detach()) < 5e-3
    y.backward(dy.cuda())
    want.backward(dy.double())
    assert _rel(oc.grad, o64.grad) < 1e-2, 'd_o'
    assert _rel(wc.grad, w64.grad) < 1e-2, 'd_weight'
    if bias:
        assert _rel(bc.grad, b64.grad) < 1e-2, 'd_bias'
    # with the projection behind it, as the layer calls it
    W = (torch.randn(96, cols) / cols ** 0.5).bfloat16()
    got = silu_rms_norm_linear(o.cuda(), w.cuda(), None if b is None else b.cuda(), W.cuda(), None)
    ref = orc.silu_rms_norm(o, w, b, 1e-5) @ W.double().t()
    assert _rel(got, ref) < 1e-2


def test_silu_rms_norm_refuses_widths_without_a_kernel():
    from nha_b200 import silu_rms_norm
    from nha_b200._lib import NHALibraryError
    with pytest.raises(NHALibraryError):
        silu_rms_norm(torch.zeros(4, 200, device='cuda', dtype=torch.bfloat16), torch.ones(200, device='cuda'))
