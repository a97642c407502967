"""GPU: the fused rotary kernel (q and k in one launch) against the oracle's fp64 rotary, batch and packed input."""
import pytest
import torch

from oracle import nha_oracle as orc
from tests.gpu_util import assert_close

pytestmark = pytest.mark.gpu

TOL_ROPE = 4e-3        # one bf16 rounding per element against fp64


def _tables(P, K, dup):
    inv = 1.0 / (10000.0 ** (torch.arange(0, K, 2, dtype=torch.float32) / K))
    fr = torch.outer(torch.arange(P, dtype=torch.float32), inv)
    if dup:
        fr = torch.cat([fr, fr], -1)
    return fr.cos().bfloat16(), fr.sin().bfloat16()


@pytest.mark.parametrize('B,T,HQ,H,K,off,dup', [(2, 100, 4, 2, 64, 0, False), (1, 333, 8, 8, 128, 77, True),
                                                 (3, 17, 2, 1, 32, 5, False), (1, 1, 1, 1, 16, 0, False)])
def test_rotary_pair_batch(B, T, HQ, H, K, off, dup):
    from nha_b200 import rotary_pair
    gen = torch.Generator().manual_seed(31)
    q = torch.randn(B, T, HQ, K, generator=gen).bfloat16()
    k = torch.randn(B, T, H, K, generator=gen).bfloat16()
    dq = torch.randn(B, T, HQ, K, generator=gen).bfloat16()
    dk = torch.randn(B, T, H, K, generator=gen).bfloat16()
    cos, sin = _tables(off + T + 3, K, dup)
    qx, kx = q.cuda().requires_grad_(True), k.cuda().requires_grad_(True)
    qr, kr = rotary_pair(qx, kx, cos.cuda(), sin.cuda(), seqlen_offset=off)
    pos = torch.arange(off, off + T)
    qo, ko = q.double().requires_grad_(True), k.double().requires_grad_(True)
    wq = torch.stack([orc.rotary_positions(qo[b], cos, sin, pos) for b in range(B)])
    wk = torch.stack([orc.rotary_positions(ko[b], cos, sin, pos) for b in range(B)])
    assert_close(qr, wq, TOL_ROPE, 'q_rot')
    assert_close(kr, wk, TOL_ROPE, 'k_rot')
    torch.autograd.backward([qr, kr], [dq.cuda(), dk.cuda()])
    torch.autograd.backward([wq, wk], [dq.double(), dk.double()])
    assert_close(qx.grad, qo.grad, TOL_ROPE, 'dq')
    assert_close(kx.grad, ko.grad, TOL_ROPE, 'dk')


def test_rotary_pair_packed_sequences_restart_positions():
    from nha_b200 import rotary_pair
    gen = torch.Generator().manual_seed(32)
    lens = [1, 70, 64, 129, 5]
    Ttot, HQ, H, K, off = sum(lens), 4, 2, 64, 3
    q = torch.randn(1, Ttot, HQ, K, generator=gen).bfloat16()
    k = torch.randn(1, Ttot, H, K, generator=gen).bfloat16()
    cos, sin = _tables(off + max(lens), K, False)
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32)
    qr, kr = rotary_pair(q.cuda(), k.cuda(), cos.cuda(), sin.cuda(), seqlen_offset=off, cu_seqlens=cu.cuda())
    pos = torch.cat([torch.arange(off, off + n) for n in lens])
    assert_close(qr[0], orc.rotary_positions(q[0], cos, sin, pos), TOL_ROPE, 'q_rot packed')
    assert_close(kr[0], orc.rotary_positions(k[0], cos, sin, pos), TOL_ROPE, 'k_rot packed')
    # a packed sequence equals the same sequence rotated alone, bit for bit
    a, b = lens[0] + lens[1], lens[0] + lens[1] + lens[2]
    q1, k1 = rotary_pair(q[:, a:b].cuda(), k[:, a:b].cuda(), cos.cuda(), sin.cuda(), seqlen_offset=off)
    assert torch.equal(q1, qr[:, a:b]) and torch.equal(k1, kr[:, a:b])


def test_rotary_pair_rejects_bad_arguments():
    from nha_b200 import _lib
    lib = _lib.load()
    x = torch.zeros(4 * 2 * 64, dtype=torch.bfloat16, device='cuda')
    t = torch.zeros(8 * 32, dtype=torch.bfloat16, device='cuda')
    args = lambda K, cs: (x.data_ptr(), x.data_ptr(), x.data_ptr(), x.data_ptr(), t.data_ptr(), t.data_ptr(), cs, 8, None,
                          0, 4, 4, 2, 2, K, 0, 0, None)
    assert lib.nha_rope_pair(*args(64, 32)) == 0
    assert lib.nha_rope_pair(*args(24, 32)) == 2          # head dim not a multiple of 16
    assert lib.nha_rope_pair(*args(64, 16)) == 2          # table rows shorter than K/2
    assert lib.nha_rope_pair(None, None, x.data_ptr(), None, t.data_ptr(), t.data_ptr(), 32, 8, None, 0, 4, 4, 2, 2, 64, 0,
                             0, None) == 1
