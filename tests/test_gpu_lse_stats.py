"""GPU: the fused aux loss / compression statistic of the training layer against the oracle
(nha_fla/layers/nha.py:255-264, 288-323)."""
import pytest
import torch

from oracle import nha_oracle as orc

pytestmark = pytest.mark.gpu

TOL = 1e-5            # fp32 sums of up to 2^19 terms against fp64, relative


@pytest.mark.parametrize('shape,target', [((2, 100, 4), 0.3), ((16, 2048, 16), 0.1), ((1, 1, 1), 0.5), ((1, 4097, 3), 0.9)])
def test_gsa_aux_loss_matches_oracle_and_is_repeatable(shape, target):
    from nha_b200 import gsa_aux_loss
    gen = torch.Generator().manual_seed(41)
    ls = torch.randn(*shape, generator=gen) * 4 + 1
    lg = torch.randn(*shape, generator=gen) * 4
    lgx = lg.cuda().requires_grad_(True)
    loss, ratio = gsa_aux_loss(ls.cuda(), lgx, target)
    assert loss.dim() == 0 and ratio.dim() == 0 and not ratio.requires_grad
    lgo = lg.double().requires_grad_(True)
    wl, wr = orc.gsa_aux(ls, lgo, target)
    assert abs(loss.item() - wl.item()) <= TOL * abs(wl.item()) + 1e-7
    assert abs(ratio.item() - wr.item()) <= TOL * abs(wr.item()) + 1e-7
    (loss * 0.25).backward()
    (wl * 0.25).backward()
    assert orc.rel_l2(lgx.grad.cpu(), lgo.grad) < 1e-5
    # fixed summation order: a second call (same scratch, ticket reset by the first) gives the same bits
    loss2, ratio2 = gsa_aux_loss(ls.cuda(), lg.cuda(), target)
    assert torch.equal(loss2, loss.detach()) and torch.equal(ratio2, ratio)


def test_gsa_aux_loss_extreme_logits_stay_finite():
    from nha_b200 import gsa_aux_loss
    ls = torch.tensor([0.0, 200.0, -200.0, 5.0] * 16).cuda()
    lg = torch.tensor([0.0, -200.0, 200.0, 5.0] * 16).cuda().requires_grad_(True)
    loss, ratio = gsa_aux_loss(ls, lg, 0.2)
    wl, wr = orc.gsa_aux(ls.cpu(), lg.detach().cpu(), 0.2)
    assert torch.isfinite(loss) and abs(loss.item() - wl.item()) < 1e-4 * wl.item()
    assert abs(ratio.item() - wr.item()) < 1e-6
    loss.backward()
    assert torch.isfinite(lg.grad).all()


def test_aux_gradient_feeds_the_operator():
    """loss = aux(lse of chunk_nha): the gradient reaches the operator's inputs through d_lse_gsa."""
    from nha_b200 import chunk_nha, gsa_aux_loss
    from tests import inputs as gen
    d = gen.layer_inputs(6, 1, 128, 2, 2, 64, 64, 64)
    names = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')
    xs = {n: d[n].cuda().requires_grad_(True) for n in names}
    o, ls, lg = chunk_nha(xs['q_swa'], xs['k_swa'], xs['q_gsa'], xs['k_gsa'], xs['v'], xs['s'], xs['g'],
                          window_size_left=64, window_size_right=0)
    loss, _ = gsa_aux_loss(ls, lg, 0.3)
    loss.backward()
    ys = {n: d[n].double().requires_grad_(True) for n in names}
    _, lso, lgo, _, _ = orc.nha_batched(ys['q_gsa'], ys['q_swa'], ys['k_gsa'], ys['k_swa'], ys['v'], ys['s'], ys['g'],
                                        64 ** -0.5, 64, 0)
    orc.gsa_aux(lso, lgo, 0.3)[0].backward()
    assert abs(loss.item() - orc.gsa_aux(lso, lgo, 0.3)[0].item()) < 2e-2
    for n in ('q_gsa', 'k_gsa', 's', 'g'):
        assert orc.rel_l2(xs[n].grad.float().cpu(), ys[n].grad) < 3e-2, n
    assert xs['q_swa'].grad is None or xs['q_swa'].grad.abs().max().item() == 0.0   # lse_swa is detached
