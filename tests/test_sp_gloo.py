"""CPU, world_size 2 and 3 over gloo: the host logic of the sequence-parallel prefill (halo exchange,
segment summaries, cross-rank scan) with the oracle standing in for the CUDA arithmetic."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

from oracle import nha_oracle as orc
from tests import inputs as gen


class OracleEngine:
    """CPU stand-in for the CUDA arithmetic of the sequence-parallel prefill (same two calls)."""

    def __init__(self, q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset):
        self.a = (q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset)
        self.dims = (k_e.shape[2], k_e.shape[3], s_e.shape[3], v_e.shape[3])

    def summary(self):
        from nha_b200.sharding import pack_summary
        q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset = self.a
        z = torch.zeros(k_e.shape[0], k_e.shape[1], k_e.shape[2], k_e.shape[3])
        _, hk, hv = orc.prefill(z, k_e, v_e, z, k_e, s_e, g_e, W, 1.0)
        return pack_summary(hk.float(), hv.float(), g_e, W)

    def finish(self, allp, rank, initial_state=None):
        from nha_b200.sharding import fold_start_state
        q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset = self.a
        Sk, Sv = fold_start_state(allp, rank, self.dims, initial_state)
        zq = torch.zeros(q.shape[0], q_offset, *q.shape[2:])
        o, hk, hv = orc.prefill(torch.cat([zq, q], 1), k_e, v_e, torch.cat([zq, rq], 1), rk_e, s_e, g_e, W, scale, Sk, Sv)
        return o[:, q_offset:].float(), hk.float(), hv.float()


def _worker(rank, world, port, T, W, with_state, out, B=2, room=False):
    os.environ['MASTER_ADDR'] = '127.0.0.1'
    os.environ['MASTER_PORT'] = str(port)
    dist.init_process_group('gloo', rank=rank, world_size=world)
    try:
        from nha_b200.sharding import sequence_parallel_prefill
        d = gen.prefill_inputs(777, B, 2, 2, 16, 16, 8, W, T, with_state)
        d = {k: (v.float() if torch.is_tensor(v) else v) for k, v in d.items()}
        bounds = [T * r // world for r in range(world + 1)]
        a, b = bounds[rank], bounds[rank + 1]
        seg = lambda x: x[:, a:b].contiguous()
        st = (d['hk0'], d['hv0']) if with_state else None
        kv = {n: seg(d[n]) for n in ('k', 'rotary_k', 'v', 's', 'g')}
        halo_room = None
        if room and rank > 0:
            # the caller keeps its kv tensors in buffers with W free rows in front: the halo lands there, nothing is copied
            halo_room = [torch.cat([torch.full_like(kv[n][:, :W], float('nan')), kv[n]], 1) for n in ('k', 'rotary_k', 'v', 's', 'g')]
            kv = {n: e[:, W:] for n, e in zip(('k', 'rotary_k', 'v', 's', 'g'), halo_room)}
        o, (hk, hv) = sequence_parallel_prefill(seg(d['q']), kv['k'], kv['v'], seg(d['rotary_q']), kv['rotary_k'], kv['s'],
                                                kv['g'], W, initial_state=st, scale=d['scale'], engine=OracleEngine,
                                                halo_room=halo_room)
        ref_o, ref_hk, ref_hv = orc.prefill(d['q'], d['k'], d['v'], d['rotary_q'], d['rotary_k'], d['s'], d['g'], W,
                                            d['scale'], d.get('hk0'), d.get('hv0'))
        err = orc.rel_l2(o, ref_o[:, a:b])
        if rank == world - 1:
            err = max(err, orc.rel_l2(hk, ref_hk), orc.rel_l2(hv, ref_hv))
        out[rank] = err
    finally:
        dist.destroy_process_group()


def _free_port():
    with socket.socket() as s:
        s.bind(('127.0.0.1', 0))
        return s.getsockname()[1]


@pytest.mark.parametrize('world,T,W,with_state,B,room', [(2, 96, 8, False, 2, False), (3, 150, 16, True, 2, False),
                                                         (2, 64, 32, True, 2, False), (3, 144, 16, True, 1, False),
                                                         (2, 96, 8, False, 1, True)])
def test_sequence_parallel_prefill_matches_single_process(world, T, W, with_state, B, room):
    """Batches (halo received into temporaries and concatenated), one sequence (halo received straight into the extended
    tensors) and one sequence whose kv tensors already sit in buffers with room for the halo (nothing copied)."""
    with mp.Manager() as mgr:
        out = mgr.dict()
        mp.spawn(_worker, args=(world, _free_port(), T, W, with_state, out, B, room), nprocs=world, join=True)
        assert len(out) == world
        for r in range(world):
            assert out[r] < 1e-5, f'rank {r}: rel-L2 {out[r]:.2e}'
