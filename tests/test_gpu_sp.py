"""GPU, 2 ranks over NCCL (skipped on a single-GPU box): sequence-parallel prefill against the
single-device op on the same inputs.  Ranks only exchange the halo and the segment summaries."""
import os
import socket

import pytest
import torch

pytestmark = pytest.mark.gpu


def _worker(rank, world, port, out):
    import faulthandler
    import torch.distributed as dist
    faulthandler.dump_traceback_later(240, exit=True)        # a rank that waits for a lost peer reports where and leaves
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    try:
        from nha_b200 import fused_chunk_nha_prefill
        from nha_b200.sharding import sequence_parallel_prefill
        from oracle import nha_oracle as orc
        from tests import inputs as gen
        T, W = 1024, 64
        d = gen.prefill_inputs(4321, 1, 2, 4, 64, 64, 64, W, T, True)
        c = {k: (v.cuda() if torch.is_tensor(v) else v) for k, v in d.items()}
        ref_o, (ref_hk, ref_hv) = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'],
                                                          rotary_k=c['rotary_k'], s=c['s'], g=c['g'], window_size=W,
                                                          initial_state=(c['hk0'], c['hv0']), output_final_state=True)
        a, b = T * rank // world, T * (rank + 1) // world
        seg = lambda x: x[:, a:b].contiguous()
        o, (hk, hv) = sequence_parallel_prefill(seg(c['q']), seg(c['k']), seg(c['v']), seg(c['rotary_q']),
                                                seg(c['rotary_k']), seg(c['s']), seg(c['g']), W,
                                                initial_state=(c['hk0'], c['hv0']))
        err = orc.rel_l2(o.float().cpu(), ref_o[:, a:b].float().cpu())
        if rank == world - 1:
            err = max(err, orc.rel_l2(hk.cpu(), ref_hk.cpu()), orc.rel_l2(hv.cpu(), ref_hv.cpu()))
        out[rank] = err
    finally:
        dist.destroy_process_group()


def _graph_worker(rank, world, port, out):
    """The captured form at the shape the pipelined kernels serve: two different inputs through one graph."""
    import faulthandler
    import torch.distributed as dist
    faulthandler.dump_traceback_later(240, exit=True)        # a rank that waits for a lost peer reports where and leaves
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    os.environ['NCCL_NVLS_ENABLE'] = '0'
    torch.cuda.set_device(rank)
    dist.init_process_group('nccl', rank=rank, world_size=world, device_id=torch.device('cuda', rank))
    graphed = None
    try:
        from nha_b200 import fused_chunk_nha_prefill
        from nha_b200.sharding import GraphedPrefill
        from oracle import nha_oracle as orc
        from tests import inputs as gen
        T, W = 2048, 128
        names = ('q', 'k', 'v', 'rotary_q', 'rotary_k', 's', 'g')
        a, b = T * rank // world, T * (rank + 1) // world
        static, worst = None, 0.0
        for seed in (99, 100):
            d = gen.prefill_inputs(seed, 1, 2, 4, 128, 128, 64, W, T, False)
            c = {k: v.cuda() for k, v in d.items() if torch.is_tensor(v)}
            ref_o, (ref_hk, ref_hv) = fused_chunk_nha_prefill(q=c['q'], k=c['k'], v=c['v'], rotary_q=c['rotary_q'],
                                                              rotary_k=c['rotary_k'], s=c['s'], g=c['g'], window_size=W,
                                                              output_final_state=True)
            if static is None:
                static = {n: c[n][:, a:b].contiguous() for n in names}
                graphed = GraphedPrefill(*(static[n] for n in names), W)
            else:
                # the graph's inputs: q and rotary_q as passed, the kv-head tensors as the object holds them
                for n in names:
                    getattr(graphed, n).copy_(c[n][:, a:b])
            o, (hk, hv) = graphed()
            torch.cuda.synchronize()
            err = orc.rel_l2(o.float().cpu(), ref_o[:, a:b].float().cpu())
            if rank == world - 1:
                err = max(err, orc.rel_l2(hk.cpu(), ref_hk.cpu()), orc.rel_l2(hv.cpu(), ref_hv.cpu()))
            worst = max(worst, err)
        out[rank] = worst
    finally:
        graphed = None                  # the graph holds NCCL work: it must be gone before the group is destroyed
        torch.cuda.synchronize()
        dist.destroy_process_group()


def _spawn(worker):
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(worker, args=(2, port, out), nprocs=2, join=True)
        return dict(out)


def test_graphed_sequence_parallel_prefill_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    out = _spawn(_graph_worker)
    for r in range(2):
        assert out[r] < 1e-2, f'rank {r}: rel-L2 {out[r]:.2e}'


def test_sequence_parallel_prefill_two_gpus():
    if torch.cuda.device_count() < 2:
        pytest.skip('needs 2 GPUs')
    import torch.multiprocessing as mp
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        port = s.getsockname()[1]
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(2, port, out), nprocs=2, join=True)
        for r in range(2):
            assert out[r] < 1e-2, f'rank {r}: rel-L2 {out[r]:.2e}'
