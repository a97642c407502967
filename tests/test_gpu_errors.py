"""GPU: the bounded waits end, and the ops read the device error words.

Every wait of the tensor-core kernels on a completion barrier polls a limited number of times and then sets an error
word instead of spinning.  The self test launches a wait on a barrier that nothing completes, with a short limit:
the call must come back and the word must be set (no trap, no fault; the context stays usable).  tests/conftest.py
sets NHA_B200_CHECK=1, so every op of every GPU test also reads its kernels' word and raises if it is non-zero.
"""
import ctypes

import pytest
import torch

from tests import inputs as gen

pytestmark = pytest.mark.gpu


def test_a_wait_that_nothing_completes_runs_out_and_reports():
    from nha_b200 import _lib
    lib = _lib.load()
    word = torch.zeros(1, dtype=torch.int32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.nha_selftest_bounded_wait(word.data_ptr(), 64, stream) == 0
    torch.cuda.synchronize()
    assert int(word.item()) == 1
    assert lib.nha_selftest_bounded_wait(word.data_ptr(), 0, stream) == 1          # bad argument, nothing launched
    # the context is still usable
    assert float((torch.ones(4, device='cuda') * 2).sum().item()) == 8.0


def test_ops_raise_when_the_device_word_is_set(monkeypatch):
    """The check the ops run after every call (NHA_B200_CHECK=1): clean after a normal call, raising once the plan's
    error word is non-zero (set here by hand on the plan of a finished forward, then read through the same path)."""
    from nha_b200 import _lib
    from nha_b200.chunk import _fill_desc, chunk_forward
    monkeypatch.setenv('NHA_B200_CHECK', '1')
    lib = _lib.load()
    B, T, H, K, M = 1, 130, 2, 64, 64
    d = gen.layer_inputs(5, B, T, H, H, K, K, M)
    x = {n: d[n].reshape(B * T, *d[n].shape[2:]).cuda() for n in ('q_gsa', 'q_swa', 'k_gsa', 'k_swa', 'v', 's', 'g')}
    cu = torch.tensor([0, T], dtype=torch.int32, device='cuda')
    o, ls, lg, _, _, saved = chunk_forward(x['q_gsa'], x['q_swa'], x['k_gsa'], x['k_swa'], x['v'], x['s'], x['g'], cu, T,
                                           K ** -0.5, 63, 64)
    geo = saved['geo']
    desc = _fill_desc(geo, dict(x, cu_seqlens=cu), K ** -0.5, None, 63, None, 64)
    stream = torch.cuda.current_stream().cuda_stream
    assert lib.nha_chunk_device_error(ctypes.byref(desc), stream) == 0
    _lib.check_chunk_device(lib, ctypes.byref(desc), stream, 'clean')
    word = int(geo.N + 1 + geo.ncb + geo.ncb * geo.H)
    geo.plan[word] = 1
    with pytest.raises(_lib.NHALibraryError):
        _lib.check_chunk_device(lib, ctypes.byref(desc), stream, 'marked')


def test_the_fold_of_the_peer_exchange_gives_up_on_a_summary_that_never_arrives():
    """nha_sp_fold_wait on a mailbox whose flag nothing raises (the rank before 'never publishes'): the wait is bounded,
    the kernel sets the error word and returns, the context stays usable; with the flag raised the same call folds the
    summary in the mailbox.  One GPU, no peer involved: the mailbox is ordinary device memory here."""
    from nha_b200 import _lib
    lib = _lib.load()
    H, K, M, V, world, depth, rank = 1, 16, 16, 16, 2, 3, 1
    nk, nv = H * K * M, H * M * V
    P = nk + nv + H * M
    box = torch.zeros(depth, world, P, device='cuda')
    flag = torch.zeros(depth, world, dtype=torch.int32, device='cuda')
    ctr = torch.tensor([1, 0], dtype=torch.int32, device='cuda')             # call number 1 -> slot 1
    sk, sv = torch.full((1, H, K, M), 7.0, device='cuda'), torch.full((1, H, M, V), 7.0, device='cuda')
    err = torch.zeros(1, dtype=torch.int32, device='cuda')
    stream = torch.cuda.current_stream().cuda_stream
    call = lambda: lib.nha_sp_fold_wait(box.data_ptr(), flag.data_ptr(), ctr.data_ptr(), world, rank, depth, H, K, M, V, None,
                                        None, sk.data_ptr(), sv.data_ptr(), err.data_ptr(), stream)
    assert call() == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 1 and float(sk.min().item()) == 7.0, 'the wait must run out and leave the outputs alone'
    assert float((torch.ones(4, device='cuda') * 2).sum().item()) == 8.0      # the context is still usable
    # the summary of rank 0 arrives: end state 2.0 everywhere, log decay 0
    err.zero_()
    box[1, 0, :nk + nv] = 2.0
    flag[1, 0] = 1
    assert call() == 0
    torch.cuda.synchronize()
    assert int(err.item()) == 0
    assert torch.equal(sk, torch.full_like(sk, 2.0)) and torch.equal(sv, torch.full_like(sv, 2.0))
