"""Multi-GPU use of the NHA ops: one process per GPU, ``torch.distributed`` for the plumbing.

Two modes, following how the operator shards:

* Batch / head sharding needs no code here: sequences and kv heads are independent, so every rank
  simply calls the ops on its own rows (no collective).
* Sequence-parallel prefill (one long sequence cut into contiguous segments, rank r owning tokens
  ``[r*T/P, (r+1)*T/P)``) has exactly one exchange step, implemented by
  :func:`sequence_parallel_prefill`:

    1. halo: rank r receives from rank r-1 the last ``W`` tokens of ``k, rotary_k, v, s, g`` (the
       keys/values its first queries still see, and the tokens that enter its slot memory late
       because of the shift by ``W``) - one point-to-point message;
    2. every rank summarises its segment: the slot memory it would end with from a zero start,
       ``L_r``, and the total log decay ``G_r`` of the tokens that enter - the recurrence is linear,
       so ``S_start(r+1) = S_start(r) * exp(G_r) + L_r``;
    3. one all-gather of ``(L_r, G_r)``; every rank folds the ranks before it;
    4. the rank's forward runs from its true start state, fully parallel with the other ranks.

  The reference has no distributed code at all (its long-context story is the O(1) state plus
  ``initial_state`` resumption, nha_fla/ops/nha/chunk_fused.py:337-342); the single-device op is the
  oracle for this function.

The arithmetic sits behind an ``engine`` (``summary`` / ``finish``) so the host logic can be exercised on CPU ranks
with the ``gloo`` backend; the default engine runs the CUDA ops of this package: ONE state pass per rank from a zero
start (it yields the chunk-start states and the segment summary together), the true start state folded into the
chunk-start states afterwards (``nha_chunk_apply_state_prefix``), and an output pass whose query tensors are NOT
extended by the halo (``q_offset``: only the kv-head tensors, a quarter of the bytes, are concatenated with it).
"""
from __future__ import annotations

from typing import Optional, Tuple

import torch
import torch.distributed as dist

_BF16 = torch.bfloat16


class PeerMailbox:
    """Symmetric mailboxes for the segment summaries: every rank holds ``box [depth, world, P]`` floats and ``flag
    [depth, world]`` words that every other rank of the group can address over NVLink (``torch.distributed``'s symmetric
    memory supplies the allocation and the peer pointers; the stores, flags and waits are this package's kernels,
    ``nha_sp_publish`` / ``nha_sp_fold_wait``).  One object per (group, message size); made by the first eager call of
    :func:`sequence_parallel_prefill` (a collective: all ranks create it together), never inside a graph capture."""

    _cache = {}

    def __init__(self, P: int, device, group=None):
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        self.depth, self.P = self.world + 1, int(P)
        pg = group if group is not None else dist.group.WORLD
        try:                                             # older releases want the group registered first
            import warnings
            with warnings.catch_warnings():
                warnings.simplefilter('ignore')
                symm.enable_symm_mem_for_group(pg.group_name)
        except Exception:                                # noqa: BLE001
            pass
        self.box = symm.empty(self.depth * self.world * self.P, dtype=torch.float32, device=device)
        self.flag = symm.empty(self.depth * self.world, dtype=torch.int32, device=device)
        self.box.zero_()
        self.flag.zero_()
        self._hb = symm.rendezvous(self.box, pg.group_name)
        self._hf = symm.rendezvous(self.flag, pg.group_name)
        self.box_ptrs, self.flag_ptrs = int(self._hb.buffer_ptrs_dev), int(self._hf.buffer_ptrs_dev)
        self.ctr = torch.zeros(2, dtype=torch.int32, device=device)
        torch.cuda.synchronize(device)
        dist.barrier(group)                              # every rank's flags are zero before anybody publishes

    @staticmethod
    def key(P: int, device, group=None):
        pg = group if group is not None else dist.group.WORLD
        return (pg.group_name, int(P), device.index)

    @classmethod
    def get(cls, P: int, device, group=None):
        """The mailbox of this (group, message size, device), or None when peer memory cannot be set up here (the
        exchange then goes through the collective library).  Collective on first use."""
        import os
        if os.environ.get('NHA_B200_SP_NCCL') == '1' or device.type != 'cuda' or torch.cuda.is_current_stream_capturing():
            return None
        key = cls.key(P, device, group)
        if key not in cls._cache:
            try:
                box = cls(P, device, group)
            except Exception:                            # noqa: BLE001 - no peer access / no symmetric memory: NCCL path
                box = None
            ok = torch.tensor([1 if box is not None else 0], device=device)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)           # every rank takes the same path
            cls._cache[key] = box if int(ok.item()) == 1 else None
        return cls._cache[key]

    def publish(self, pack: torch.Tensor):
        from . import _lib
        lib = _lib.load()
        with torch.cuda.device(pack.device):
            _lib.check(lib.nha_sp_publish(pack.data_ptr(), self.P, self.box_ptrs, self.flag_ptrs, self.ctr.data_ptr(), self.world,
                                          self.rank, self.depth, torch.cuda.current_stream(pack.device).cuda_stream),
                       'nha_sp_publish')


class PeerHalo:
    """Halo-extended kv tensors in symmetric memory, so that the rank before can store its last window straight into
    their first ``W`` rows (``nha_sp_halo_push`` / ``_wait`` / ``_ack``): for callers that keep their kv inputs in
    these buffers, i.e. :class:`GraphedPrefill`.  Construction is a collective of the group."""

    def __init__(self, own, W: int, group=None):
        import ctypes
        import torch.distributed._symmetric_memory as symm
        self.world, self.rank = dist.get_world_size(group), dist.get_rank(group)
        pg = group if group is not None else dist.group.WORLD
        dev = own[0].device
        self.W, self.Tr = int(W), own[0].shape[1]
        self.ext, handles = [], []
        for x in own:
            e = symm.empty((self.W + self.Tr) * x[0, 0].numel(), dtype=x.dtype, device=dev)
            handles.append(symm.rendezvous(e, pg.group_name))
            e = e.view(1, self.W + self.Tr, *x.shape[2:])
            e[:, self.W:].copy_(x)
            self.ext.append(e)
        self.flags = symm.empty(4, dtype=torch.int32, device=dev)            # [0] data flag, [1] acknowledgement
        self.flags.zero_()
        hf = symm.rendezvous(self.flags, pg.group_name)
        self._handles = handles + [hf]
        self.ctr_push = torch.zeros(2, dtype=torch.int32, device=dev)
        self.ctr_recv = torch.zeros(1, dtype=torch.int32, device=dev)
        self.err = torch.zeros(1, dtype=torch.int32, device=dev)
        self.side = torch.cuda.Stream(dev)
        nxt, prv = self.rank + 1, self.rank - 1
        rows = [self.W * x[0, 0].numel() * x.element_size() for x in own]     # bytes of W rows
        if nxt < self.world:
            self._src = (ctypes.c_void_p * 5)(*[e[:, self.Tr:].data_ptr() for e in self.ext])
            self._dst = (ctypes.c_void_p * 5)(*[int(h.buffer_ptrs[nxt]) for h in handles])
            self._bytes = (ctypes.c_int64 * 5)(*rows)
            self._flag_peer = int(hf.buffer_ptrs[nxt])
        if prv >= 0:
            self._ack_peer = int(hf.buffer_ptrs[prv]) + 4
        torch.cuda.synchronize(dev)
        dist.barrier(group)                              # every rank's flags are zero before anybody pushes

    def _st(self):
        return torch.cuda.current_stream(self.flags.device).cuda_stream

    def push(self):
        from . import _lib
        with torch.cuda.device(self.flags.device):
            _lib.check(_lib.load().nha_sp_halo_push(self._src, self._dst, self._bytes, 5, self._flag_peer,
                                                    self.flags.data_ptr() + 4, self.ctr_push.data_ptr(), self.err.data_ptr(),
                                                    self._st()), 'nha_sp_halo_push')

    def wait(self):
        from . import _lib
        with torch.cuda.device(self.flags.device):
            _lib.check(_lib.load().nha_sp_halo_wait(self.flags.data_ptr(), self.ctr_recv.data_ptr(), self.err.data_ptr(),
                                                    self._st()), 'nha_sp_halo_wait')

    def ack(self):
        from . import _lib
        with torch.cuda.device(self.flags.device):
            _lib.check(_lib.load().nha_sp_halo_ack(self._ack_peer, self.ctr_recv.data_ptr(), self._st()), 'nha_sp_halo_ack')


class CudaEngine:
    """Default arithmetic of :func:`sequence_parallel_prefill` on this rank's GPU: ``summary()`` gives the rank's message
    to the others, ``finish()`` turns everybody's messages into this rank's outputs."""

    def __init__(self, q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset):
        from .chunk import SegmentForward
        self.args = (q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset)
        B = k_e.shape[0]
        K, V, M = k_e.shape[-1], v_e.shape[-1], s_e.shape[-1]
        NG = q.shape[2] // k_e.shape[2]
        self.dims = (k_e.shape[2], K, M, V)
        # the three-step path needs the pipelined output pass (it alone knows late-starting queries)
        self.steps = None
        if B == 1 and K == 128 and V == 128 and M == 64 and NG % 2 == 0 and q_offset % 64 == 0:
            f = lambda x: x[0].to(_BF16).contiguous()
            self.steps = SegmentForward(f(q), f(rq), f(k_e), f(rk_e), f(v_e), f(s_e), f(g_e), scale, W - 1, W, q_offset)

    def start(self):
        """What can run before the halo has arrived: the per-chunk state terms of the chunks that read only this rank's
        own rows."""
        if self.steps is not None:
            self.steps.start()

    def summary(self):
        """``[B, H*K*M + H*M*V + H*M]`` fp32: zero-start end state of the (halo-extended) segment and the total log
        decay of the tokens that enter its slot memory."""
        if self.steps is not None:
            return self.steps.summary()
        from .chunk import chunk_final_state
        q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset = self.args
        B, T = k_e.shape[0], k_e.shape[1]
        flat = lambda x: x.reshape(B * T, *x.shape[2:]).to(_BF16).contiguous()
        cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=k_e.device)
        Lk, Lv = chunk_final_state(flat(k_e), flat(v_e), flat(s_e), flat(g_e), cu, T, W)
        return pack_summary(Lk, Lv, g_e, W)

    def finish(self, allp, rank, initial_state=None, mailbox=None):
        """Outputs of the rank's own tokens and the slot memory at the end of its segment, from ``allp [world, B, P]`` or,
        with ``mailbox`` (the three-step path only), from the summaries the other ranks put there."""
        q, rq, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset = self.args
        if self.steps is not None:
            if mailbox is not None:
                Sk, Sv = self.steps.fold_from_mailbox(mailbox, rank, initial_state)
            else:
                Sk, Sv = self.steps.fold(allp[:, 0], rank, initial_state)
            self.steps.apply_prefix(Sk, Sv)
            o, _, _, hk, hv = self.steps.output_pass()
            return o[None].to(q.dtype), hk, hv
        from .chunk_fused import fused_chunk_nha_prefill
        Sk, Sv = fold_start_state(allp, rank, self.dims, initial_state)
        if q_offset:
            zq = q.new_zeros(q.shape[0], q_offset, *q.shape[2:])
            q, rq = torch.cat([zq, q], 1), torch.cat([zq, rq], 1)
        o, (hk, hv) = fused_chunk_nha_prefill(q=q, k=k_e, v=v_e, rotary_q=rq, rotary_k=rk_e, s=s_e, g=g_e, window_size=W,
                                              initial_state=(Sk, Sv), output_final_state=True, scale=scale)
        return o[:, q_offset:], hk, hv


def _mailbox_for(pack: torch.Tensor, group):
    """The peer-memory mailbox for messages like ``pack``.  Inside a graph capture only a mailbox made earlier (by an
    eager call with the same group and message size) can be used."""
    if torch.cuda.is_current_stream_capturing():
        return PeerMailbox._cache.get(PeerMailbox.key(pack.shape[1], pack.device, group))
    return PeerMailbox.get(pack.shape[1], pack.device, group)


def _halo_done(halo_peer, rank, world, dev):
    """End of a call that used a :class:`PeerHalo`: the receiver tells the sender that the halo rows have been read for
    the last time, the sender's store stream joins the caller's."""
    if halo_peer is None:
        return
    if rank > 0:
        halo_peer.ack()
    if rank + 1 < world:
        torch.cuda.current_stream(dev).wait_stream(halo_peer.side)


def pack_summary(Lk, Lv, g_e: torch.Tensor, W: int):
    """One rank's message to the others from its zero-start end state and its gates: the total log decay of the tokens
    that enter its slot memory is all of the halo-extended segment but its last ``W`` rows, summed from the gates as the
    kernels see them (rounded to bf16).  ``[B, H*K*M + H*M*V + H*M]`` fp32."""
    B = g_e.shape[0]
    G = g_e[:, :g_e.shape[1] - W].to(_BF16).float().sum(1)                # [B,H,M]
    return torch.cat([Lk.reshape(B, -1).float(), Lv.reshape(B, -1).float(), G.reshape(B, -1)], 1).contiguous()


def fold_start_state(allp: torch.Tensor, rank: int, dims, initial_state=None):
    """Start state of rank ``rank`` from the summaries ``allp [world, B, P]`` of all ranks: the recurrence is linear, so
    ``S_start = S_0 * exp(sum_{r<rank} G_r) + sum_{r<rank} L_r * exp(sum_{r<r'<rank} G_r')`` - a fixed number of
    tensor operations whatever the rank."""
    H, K, M, V = dims
    B, dev = allp.shape[1], allp.device
    nk, nv = H * K * M, H * M * V
    if initial_state is not None and initial_state != (None, None):
        Sk, Sv = initial_state[0].float(), initial_state[1].float()
    else:
        Sk = torch.zeros(B, H, K, M, dtype=torch.float32, device=dev)
        Sv = torch.zeros(B, H, M, V, dtype=torch.float32, device=dev)
    if rank > 0:
        before = allp[:rank]
        Gs = before[:, :, nk + nv:].reshape(rank, B, H, M)
        wgt = (Gs.flip(0).cumsum(0).flip(0) - Gs).exp()                   # decay through the ranks between r and this one
        tot = Gs.sum(0).exp()
        Sk = Sk * tot[:, :, None, :] + (before[:, :, :nk].reshape(rank, B, H, K, M) * wgt[:, :, :, None, :]).sum(0)
        Sv = Sv * tot[:, :, :, None] + (before[:, :, nk:nk + nv].reshape(rank, B, H, M, V) * wgt[..., None]).sum(0)
    return Sk, Sv


def sequence_parallel_prefill(
    q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, rotary_q: torch.Tensor, rotary_k: torch.Tensor,
    s: torch.Tensor, g: torch.Tensor, window_size: int,
    initial_state: Optional[Tuple[torch.Tensor, torch.Tensor]] = None,
    scale: Optional[float] = None,
    group: Optional[dist.ProcessGroup] = None,
    engine=CudaEngine,
    halo_room=None,
    halo_peer=None,
):
    """``fused_chunk_nha_prefill`` over a sequence sharded along tokens.

    Every rank passes ITS segment: ``q, rotary_q [B,Tr,HQ,K]``, ``k, rotary_k [B,Tr,H,K]``,
    ``v [B,Tr,H,V]``, ``s, g [B,Tr,H,M]`` (segments in rank order, each at least ``window_size``
    tokens long), plus on every rank the same ``initial_state`` of the whole sequence (or None).
    Returns ``(o [B,Tr,HQ,V], (hk, hv))`` where the state is the slot memory at the END of this
    rank's segment (the last rank holds the final state of the sequence).

    ``halo_room`` (one sequence, ranks > 0): five tensors ``[1, W + Tr, H, *]`` whose rows ``W:`` ARE the ``k,
    rotary_k, v, s, g`` passed (views of them); the halo is then received into their first ``W`` rows and nothing is
    copied.  ``halo_peer``: a :class:`PeerHalo` whose ``ext`` tensors are ``halo_room``: the halo then travels over peer
    memory (a store kernel on the sender, a flag wait on the receiver) instead of a send / receive pair.
    """
    W = int(window_size)
    rank, world = dist.get_rank(group), dist.get_world_size(group)
    B, Tr = k.shape[0], k.shape[1]
    assert Tr >= W, f'every segment must hold at least window_size={W} tokens, got {Tr}'
    if scale is None:
        scale = q.shape[-1] ** -0.5
    dev = k.device

    # ---- 1. halo of W tokens from the left neighbour (kv-head tensors only) ---------------------------
    # The extended tensors are allocated first and the halo is received straight into their first W rows (contiguous
    # for one sequence), while this rank's own rows are copied behind them - or nothing is copied at all when the caller
    # keeps its kv tensors in buffers with W free rows in front (halo_room).
    own = (k, rotary_k, v, s, g)
    send = [x[:, Tr - W:].contiguous() for x in own] if halo_peer is None else []
    q_offset = W if rank > 0 else 0
    direct = rank > 0 and B == 1
    ext = None
    if direct:
        ext = halo_room if halo_room is not None else \
            [torch.empty(B, Tr + W, *x.shape[2:], dtype=x.dtype, device=dev) for x in own]
        recv = [e[:, :W] for e in ext]
    else:
        recv = [torch.empty_like(x[:, Tr - W:]) for x in own]
    ops = []
    peer = lambda r: dist.get_global_rank(group, r) if group else r
    if halo_peer is not None:
        assert B == 1 and (rank == 0 or halo_room is not None)
        if rank + 1 < world:
            # on a stream of its own: the store kernel first waits for the receiver's acknowledgement of the call before,
            # and this rank's kernels need not wait with it (joined at the end of the call)
            cur = torch.cuda.current_stream(dev)
            halo_peer.side.wait_stream(cur)
            with torch.cuda.stream(halo_peer.side):
                halo_peer.push()                         # the last W rows of this rank's kv tensors into the next rank's
    else:
        if rank + 1 < world:
            ops += [dist.P2POp(dist.isend, x, peer(rank + 1), group) for x in send]
        if rank > 0:
            ops += [dist.P2POp(dist.irecv, x, peer(rank - 1), group) for x in recv]
    works = dist.batch_isend_irecv(ops) if ops else []
    if direct and halo_room is None:
        for e, x in zip(ext, own):
            e[:, W:].copy_(x)
    eng = None
    if direct or rank == 0:
        # ---- 2a. everything that does not need the halo runs while it is on the wire --------------------------
        k_e, rk_e, v_e, s_e, g_e = ext if direct else own
        eng = engine(q, rotary_q, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset)
        if hasattr(eng, 'start'):
            eng.start()
    for w in works:
        w.wait()
    if halo_peer is not None and rank > 0:
        halo_peer.wait()
    if eng is None:
        k_e, rk_e, v_e, s_e, g_e = (torch.cat([h_, x], 1) for h_, x in zip(recv, own))
        eng = engine(q, rotary_q, k_e, rk_e, v_e, s_e, g_e, W, scale, q_offset)

    # ---- 2b. segment summary from a zero start ------------------------------------------------------------
    pack = eng.summary()

    # ---- 3. exchange of the summaries: over peer memory where the engine and the system allow it (each rank stores its
    #         summary into the mailboxes of the ranks after it; the fold kernel waits for the ranks before it), else one
    #         all-gather ------------------------------------------------------------------------------------------
    mailbox = None
    if getattr(eng, 'steps', None) is not None and B == 1:
        mailbox = _mailbox_for(pack, group)
    if mailbox is not None:
        mailbox.publish(pack)
        o, hk, hv = eng.finish(None, rank, initial_state, mailbox=mailbox)
        _halo_done(halo_peer, rank, world, dev)
        return o, (hk, hv)
    allp = torch.empty(world * B, pack.shape[1], dtype=pack.dtype, device=dev)
    dist.all_gather_into_tensor(allp, pack, group=group)

    # ---- 4. fold the ranks before this one, outputs of the rank's own tokens from its true start state ------------
    o, hk, hv = eng.finish(allp.view(world, B, -1), rank, initial_state)
    _halo_done(halo_peer, rank, world, dev)
    return o, (hk, hv)


class GraphedPrefill:
    """:func:`sequence_parallel_prefill` for one fixed segment shape, captured once as a CUDA graph - the rank's kernels,
    its halo messages and the all-gather - and replayed per call.  A call then costs the host one graph launch instead of
    some sixty launches, copies and NCCL calls; from eight ranks on that host work is longer than the rank's kernels.

    The graph's inputs are the attributes ``q, rotary_q`` (the tensors passed to the constructor) and ``k, rotary_k, v, s,
    g``: for one sequence these are views of buffers that keep ``window_size`` free rows in front for the halo of the
    rank before (initialised from the tensors passed in), so that nothing is copied per call.  Write the next segment
    into them in place, call the object, read ``(o, (hk, hv))`` (the same output tensors every call).  Every rank of the
    group must construct the object and call it the same number of times (the graph contains collectives), and must
    drop it before the process group is destroyed (``destroy_process_group`` waits for ever on a communicator that a
    live graph still uses).  The constructor runs the eager function ``warmup`` times first (communicators and kernel
    attributes are set up outside the capture)."""

    def __init__(self, q, k, v, rotary_q, rotary_k, s, g, window_size, initial_state=None, scale=None, group=None,
                 warmup: int = 2):
        import os
        W = int(window_size)
        self.q, self.rotary_q = q, rotary_q
        room, halo = None, None
        rank = dist.get_rank(group)
        if k.shape[0] == 1 and dist.get_world_size(group) > 1:
            # kv inputs in buffers with W free rows in front; in symmetric memory where the system has it, so that the
            # halo is a store by the rank before instead of a send / receive pair (every rank takes the same path)
            if os.environ.get('NHA_B200_SP_NCCL') != '1':
                try:
                    halo = PeerHalo((k, rotary_k, v, s, g), W, group)
                except Exception:                        # noqa: BLE001 - no symmetric memory here
                    halo = None
                ok = torch.tensor([1 if halo is not None else 0], device=k.device)
                dist.all_reduce(ok, op=dist.ReduceOp.MIN, group=group)
                if int(ok.item()) != 1:
                    halo = None
            if halo is not None:
                room = halo.ext
            elif rank > 0:
                room = []
                for x in (k, rotary_k, v, s, g):
                    e = torch.empty(1, W + x.shape[1], *x.shape[2:], dtype=x.dtype, device=x.device)
                    e[:, W:].copy_(x)
                    room.append(e)
            if room is not None:
                k, rotary_k, v, s, g = (e[:, W:] for e in room)
        self.k, self.rotary_k, self.v, self.s, self.g = k, rotary_k, v, s, g
        self.halo = halo
        run = lambda: sequence_parallel_prefill(q, k, v, rotary_q, rotary_k, s, g, W, initial_state=initial_state,
                                                scale=scale, group=group, halo_room=room if rank > 0 else None,
                                                halo_peer=halo)
        cur = torch.cuda.current_stream(k.device)
        side = torch.cuda.Stream(k.device)
        side.wait_stream(cur)
        with torch.cuda.stream(side):
            for _ in range(max(1, warmup)):
                run()
        cur.wait_stream(side)
        torch.cuda.synchronize(k.device)
        self.graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.graph, capture_error_mode='thread_local'):
            self.out = run()

    def __call__(self):
        self.graph.replay()
        if self.halo is not None:
            from . import _lib
            if _lib.check_device_words() and int(self.halo.err.item()) != 0:
                raise _lib.NHALibraryError('sequence-parallel prefill: a bounded wait of the peer-memory halo ran out; the '
                                           'outputs of this call are invalid')
        return self.out
