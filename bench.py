#!/usr/bin/env python
"""Benchmark of the NHA attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference]

Workload (config.workload): fused NHA attention forward + backward at the
340M-layer shape, B=16 T=2048 H=16 head_dim=64 M=64 slots window=64 chunk 64,
bf16, q/k/v ~ N(0,1)/8, gate logits ~ N(0,1) through logsigmoid, upstream
gradients ~ N(0,1), synthetic seeded inputs.  A step is one forward + backward
over one such batch.  With N > 1 (launched by torchrun) every rank runs the
same batch shape on its own GPU (sequences are independent: batch sharding, no
collective); `value` is the tokens all ranks processed per second of the
slowest rank.

One JSON line is printed by rank 0.  `value` times the C-ABI calls with inputs
resident in HBM; `e2e` times the public `chunk_nha` call + autograd backward
with pinned HOST buffers (host->device of the 8 inputs and device->host of the
output, both LSEs and the 7 gradients inside the timed region).  `roofline`
is the whole step against the HBM roof: algorithmic bytes (every input read
once per pass, every output written once, no intermediates: 49,344 B per token)
divided by the step time; it names the kernel with the largest share, and
`kernels` lists every stage timed on its own with CUDA events together with the
bytes that stage moves by design (`stage_bytes`, hand-over scratch included).
`cpu_baseline` is the CPU oracle (a port of the reference's naive PyTorch path)
timed on this box's host cores on a bounded slice.  A timed region is repeated
back to back until it lasts about half a second (`inner_repeats`), so that the
sampled clocks describe it; `ms_per_step` stays the time of one step.

`--impl reference` times that CPU oracle alone (rank 0 only), same metric/unit.
"""
from __future__ import annotations

import argparse
import json
import math
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

import torch  # noqa: E402
import torch.nn.functional as F  # noqa: E402

METRIC = 'NHA attn fwd+bwd tokens/s (bf16)'
UNIT = 'tokens/s'
CFG = dict(B=16, T=2048, H=16, D=64, M=64, W=64, shift=0)
WORKLOAD = 'nha_attn_fwd_bwd B16 T2048 H16 D64 M64 W64 chunk64 bf16 (340M-layer shape)'
CPU_SLICE_T = 512                             # tokens of the B=1 slice both CPU measurements run (cost grows with T)
# dram__bytes_read.sum + dram__bytes_write.sum of all kernels of one step per token, from the committed ncu captures
NCU_STEP_TRAFFIC_PER_TOKEN = 1104.2e6 / 8192       # profiles/step_traffic_chunk_fwd_bwd_B4_T2048.md
ALG_BYTES_PER_TOKEN = 16512 + 32832          # forward + backward, all 16 heads (each input read once per pass)
NAMES = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')


def peaks():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        d = json.load(open(p))
        return float(d['hbm_gbs']), 'measured'
    return 6650.0, 'fallback'


def gen_inputs(seed, B, T, H, D, M, pin=False):
    """CPU-generated fp32 -> bf16, like the reference's generators."""
    g = torch.Generator().manual_seed(seed)
    sc = D ** -0.5
    out = {}
    for n in ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v'):
        out[n] = (torch.randn(B, T, H, D, generator=g) * sc).to(torch.bfloat16)
    gl = F.logsigmoid(torch.randn(B, T, H, M, generator=g))
    out['g'] = gl.to(torch.bfloat16)
    out['s'] = (1 - gl.exp()).to(torch.bfloat16)
    out['do'] = torch.randn(B, T, H, D, generator=g).to(torch.bfloat16)
    if pin:
        out = {k: v.pin_memory() for k, v in out.items()}
    return out


# ---------------------------------------------------------------------------------------------
class ClockSampler:
    """Samples SM clocks and throttle reasons of one GPU with nvidia-smi while a region runs."""
    Q = ('clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,'
         'clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,'
         'clocks_event_reasons.sw_power_cap,utilization.gpu')

    def __init__(self, index):
        self.index, self.rows, self.proc = index, [], None

    def __enter__(self):
        try:
            self.proc = subprocess.Popen(['nvidia-smi', f'--query-gpu={self.Q}', '--format=csv,noheader,nounits',
                                          '-lms', '100', '-i', str(self.index)], stdout=subprocess.PIPE, text=True)
            self.th = threading.Thread(target=self._read, daemon=True)
            self.th.start()
        except Exception:
            self.proc = None
        return self

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append([x.strip() for x in line.split(',')])

    def __exit__(self, *a):
        if self.proc is not None:
            time.sleep(0.15)
            self.proc.terminate()
            try:
                self.proc.wait(timeout=2)
            except Exception:
                self.proc.kill()

    def summary(self):
        sm, mx, reasons = [], 0.0, set()
        loaded = [r for r in self.rows if len(r) > 7 and r[7].replace('.', '').isdigit() and float(r[7]) >= 50]
        for r in (loaded or self.rows):                  # samples taken under load (GPU utilisation >= 50 %)
            try:
                sm.append(float(r[0])); mx = max(mx, float(r[1]))
            except Exception:
                continue
            for name, val in zip(('hw_slowdown', 'hw_thermal_slowdown', 'sw_thermal_slowdown', 'sw_power_cap'), r[3:7]):
                if val.lower().startswith('active'):
                    reasons.add(name)
        busy = [x for x in sm if x > 0]
        return {'sm_mhz': statistics.median(busy) if busy else None, 'sm_max_mhz': mx or None,
                'reasons': sorted(reasons), 'samples': len(sm)}

    def start(self):
        return self.__enter__()

    def stop(self):
        self.__exit__()


# ---------------------------------------------------------------------------------------------
def cpu_oracle_tokens_per_s(T, repeats=1):
    """fwd+bwd of the CPU oracle on a B=1, T-token slice of the workload (all heads)."""
    from oracle import nha_oracle as orc
    torch.set_num_threads(os.cpu_count())
    c = CFG
    d = gen_inputs(0, 1, T, c['H'], c['D'], c['M'])
    best = None
    for _ in range(repeats):
        xs = {n: d[n][0].double().requires_grad_(True) for n in NAMES}
        t0 = time.perf_counter()
        o, ls, lg, hk, hv = orc.nha_sequence(xs['q_gsa'], xs['q_swa'], xs['k_gsa'], xs['k_swa'], xs['v'], xs['s'],
                                             xs['g'], c['D'] ** -0.5, c['W'], c['shift'])
        (o * d['do'][0].double()).sum().backward()
        dt = time.perf_counter() - t0
        best = dt if best is None else min(best, dt)
    return T / best, best


def run_reference(args):
    """`--impl reference`: the reference's CPU path for this op is its naive PyTorch functions
    (scripts/verify_opt_parity.py:147-191); they cannot travel to the GPU box, so the oracle port,
    pinned against them by tests/golden, is timed instead."""
    rank = int(os.environ.get('RANK', '0'))
    if rank != 0:
        return
    T = CPU_SLICE_T
    for _ in range(min(args.warmup, 3)):
        cpu_oracle_tokens_per_s(T)
    t0 = time.perf_counter()
    for _ in range(args.steps):
        cpu_oracle_tokens_per_s(T)
    dt = time.perf_counter() - t0
    val = T * args.steps / dt
    sample = f'B=1 T={T} slice of the workload (H16 D64 M64 W64), fp64 oracle fwd + autograd bwd per step'
    line = {
        'metric': METRIC, 'value': val, 'unit': UNIT, 'n_gpus': args.gpus, 'steps': args.steps, 'warmup': args.warmup,
        'ms_per_step': 1e3 * dt / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
        'dtype': 'f64', 'data': 'synthetic', 'impl': 'reference',
        'config': {'workload': WORKLOAD, 'sample': sample},
        'cpu_baseline': {'value': val, 'unit': UNIT, 'cores': os.cpu_count(), 'kind': 'port', 'sample': sample},
        'e2e': {'value': val, 'unit': UNIT, 'h2d_bytes_per_step': 0, 'd2h_bytes_per_step': 0},
        'gpu_launches': 0,
    }
    emit(line)



# ---------------------------------------------------------------------------------------------
def bench_decode(lib, dev, rank, world, timed, peak):
    """Batched decode in a Qwen3-MoE-style stack: 48 layers, 32 sequences per GPU (256 over 8 GPUs), HQ=32, H=4,
    D=128, M=64 slots, W=512 window with in-kernel rotary; one fused step per layer, 48 C-ABI calls back to back.
    Attention only (projections and MoE are outside the operator).  Batch-sharded: no collective."""
    B, H, NG, K, M, W, LAYERS = 32, 4, 8, 128, 64, 512, 48
    g = torch.Generator(device='cpu').manual_seed(99 + rank)
    mk = lambda *sh: torch.randn(*sh, generator=g).to(dev)
    layers = []
    for _ in range(LAYERS):
        layers.append(dict(q=mk(B, H * NG, K).bfloat16(), k=mk(B, H, K).bfloat16(), v=mk(B, H, K).bfloat16(),
                           g=(F.logsigmoid(mk(B, H, M)) / 8).bfloat16(), sw_k=mk(B, W, H, K).bfloat16(),
                           sw_v=mk(B, W, H, K).bfloat16(), hk=mk(B, H, K, M) * 0.5, hv=mk(B, H, M, K) * 0.5,
                           o=torch.empty(B, H * NG, K, device=dev, dtype=torch.bfloat16)))
    inv = 1.0 / (10000.0 ** (torch.arange(0, K, 2, dtype=torch.float32) / K))
    fr = torch.outer(torch.arange(32768 - W + 1, 32768 + 1, dtype=torch.float32), inv)
    emb = torch.cat([fr, fr], -1)
    cos, sin = emb.cos().bfloat16()[None], emb.sin().bfloat16()[None]
    cos, sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
    ws = torch.zeros(int(lib.nha_decode_workspace_bytes(B, H * NG, H, K, W)), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def step(stream=stream):
        for d in layers:
            st = lib.nha_decode_step(d['q'].data_ptr(), None, d['k'].data_ptr(), d['v'].data_ptr(), d['g'].data_ptr(), None,
                                     d['sw_k'].data_ptr(), d['sw_v'].data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                     cos.stride(1), None, d['hk'].data_ptr(), d['hv'].data_ptr(), 0, d['o'].data_ptr(), None,
                                     ws.data_ptr(), ws.numel(), B, H * NG, H, K, K, M, W, K ** -0.5, stream)
            assert st == 0
    # programmatic dependent launch: 0 = plain launches, 1 = wait before the first read (the library's default),
    # 2 = the layer's state and window are requested before the wait (valid for this stack: the kernel in front on
    # the stream belongs to another layer and writes neither)
    by_mode = {}
    for mode in (0, 1, 2):
        assert lib.nha_decode_set_pdl(mode) == 0
        for _ in range(3):
            step()
        by_mode[mode] = timed(step, 200) / 200
    ms = by_mode[2]
    # the same 48 launches captured once as a CUDA graph and replayed (the dependent-launch edges are kept by the capture)
    graph_us = None
    try:
        graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(graph):
            step(torch.cuda.current_stream(dev).cuda_stream)
        for _ in range(3):
            graph.replay()
        graph_us = 1e3 * (timed(graph.replay, 200) / 200) / LAYERS
        del graph
    except Exception as e:                                       # noqa: BLE001 - reported, the eager figure stands
        print(f'[bench] rank {rank}: decode graph capture failed: {e}', file=sys.stderr)
    per_seq_layer = H * (2 * (K * M + M * K) * 4 + 2 * W * K * 2) + (2 * H * NG * K + H * (2 * K + M)) * 2
    gbs = per_seq_layer * B * LAYERS / (ms * 1e-3) / 1e9
    # the slot memory kept in bf16 (an extension; the reference keeps fp32 states): half the state bytes per step
    for d in layers:
        d['hk16'], d['hv16'] = d['hk'].bfloat16(), d['hv'].bfloat16()

    def step_bf16_state():
        for d in layers:
            st = lib.nha_decode_step_bf16_state(d['q'].data_ptr(), None, d['k'].data_ptr(), d['v'].data_ptr(),
                                                d['g'].data_ptr(), None, d['sw_k'].data_ptr(), d['sw_v'].data_ptr(),
                                                cos.data_ptr(), sin.data_ptr(), 0, cos.stride(1), d['hk16'].data_ptr(),
                                                d['hv16'].data_ptr(), 0, d['o'].data_ptr(), ws.data_ptr(), ws.numel(), B,
                                                H * NG, H, K, K, M, W, K ** -0.5, stream)
            assert st == 0
    for _ in range(3):
        step_bf16_state()
    ms16 = timed(step_bf16_state, 200) / 200
    per_seq_layer16 = per_seq_layer - H * (K * M + M * K) * 4
    bf16_state = {'us_per_layer': 1e3 * ms16 / LAYERS, 'tokens_per_s': world * B / (ms16 * 1e-3),
                  'gbs': per_seq_layer16 * B * LAYERS / (ms16 * 1e-3) / 1e9,
                  'frac': per_seq_layer16 * B * LAYERS / (ms16 * 1e-3) / 1e9 / peak,
                  'algorithmic_bytes_per_launch': per_seq_layer16 * B,
                  'note': 'slot memory in bf16 (nha_decode_step_bf16_state): not the reference\'s numerics, reported beside '
                          'the fp32-state figure'}
    # the same stack with the cache maintenance of one generated token inside the timed region: the reference's
    # NHACache shifts each layer's window with torch.cat (keys, values, gate rows) and pops the oldest entry; the
    # ring cache replaces that with nha_decode_step_ring + nha_ring_append
    gnew = [(F.logsigmoid(mk(B, H, M)) / 8).bfloat16() for _ in range(LAYERS)]
    gwin = [(F.logsigmoid(mk(B, W, H, M)) / 8).bfloat16() for _ in range(LAYERS)]

    def step_shift():
        for d, gn, li in zip(layers, gnew, range(LAYERS)):
            pk, pv, pg = d['sw_k'][:, :1].contiguous(), d['sw_v'][:, :1].contiguous(), gwin[li][:, :1].contiguous()
            d['sw_k'] = torch.cat([d['sw_k'][:, 1:], d['k'][:, None]], 1)
            d['sw_v'] = torch.cat([d['sw_v'][:, 1:], d['v'][:, None]], 1)
            gwin[li] = torch.cat([gwin[li][:, 1:], gn[:, None]], 1)
            st = lib.nha_decode_step(d['q'].data_ptr(), None, pk.data_ptr(), pv.data_ptr(), pg.data_ptr(), None,
                                     d['sw_k'].data_ptr(), d['sw_v'].data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                     cos.stride(1), None, d['hk'].data_ptr(), d['hv'].data_ptr(), 0, d['o'].data_ptr(), None,
                                     ws.data_ptr(), ws.numel(), B, H * NG, H, K, K, M, W, K ** -0.5, stream)
            assert st == 0
    heads = [torch.zeros(B, dtype=torch.int32, device=dev) for _ in range(LAYERS)]

    def step_ring():
        for d, gn, gw, hd in zip(layers, gnew, gwin, heads):
            st = lib.nha_decode_step_ring(d['q'].data_ptr(), d['k'].data_ptr(), d['v'].data_ptr(), d['sw_k'].data_ptr(),
                                          d['sw_v'].data_ptr(), gw.data_ptr(), hd.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                          0, cos.stride(1), d['hk'].data_ptr(), d['hv'].data_ptr(), d['o'].data_ptr(),
                                          ws.data_ptr(), ws.numel(), B, H * NG, H, K, K, M, W, W, K ** -0.5, stream)
            assert st == 0
            st = lib.nha_ring_append(d['sw_k'].data_ptr(), d['sw_v'].data_ptr(), gw.data_ptr(), d['k'].data_ptr(),
                                     d['v'].data_ptr(), gn.data_ptr(), hd.data_ptr(), B, H, K, K, M, W, W, stream)
            assert st == 0
    heads_kv = [torch.zeros(B, H, dtype=torch.int32, device=dev) for _ in range(LAYERS)]

    def step_ring_fused():
        # one launch per layer: the decode kernel stores the step's token over the entry that left the window
        for d, gn, gw, hd in zip(layers, gnew, gwin, heads_kv):
            st = lib.nha_decode_step_ring_fused(d['q'].data_ptr(), d['k'].data_ptr(), d['v'].data_ptr(), gn.data_ptr(),
                                                d['sw_k'].data_ptr(), d['sw_v'].data_ptr(), gw.data_ptr(), hd.data_ptr(),
                                                cos.data_ptr(), sin.data_ptr(), 0, cos.stride(1), d['hk'].data_ptr(),
                                                d['hv'].data_ptr(), d['o'].data_ptr(), ws.data_ptr(), ws.numel(), B, H * NG,
                                                H, K, K, M, W, W, K ** -0.5, stream)
            assert st == 0
    # rings whose keys were rotated when they entered (absolute positions): the step rotates only its own token
    kr = [torch.empty_like(d['sw_k']) for d in layers]
    for d, x in zip(layers, kr):
        assert lib.nha_ring_rotate_rows(d['sw_k'].data_ptr(), x.data_ptr(), cos.data_ptr(), sin.data_ptr(), 0,
                                        cos.stride(1), B, H, K, W, W, stream) == 0
    cosq, sinq = cos[:, -1].contiguous(), sin[:, -1].contiguous()

    def step_ring_rot(append=True):
        for d, x, gn, gw, hd in zip(layers, kr, gnew, gwin, heads):
            st = lib.nha_decode_step_ring_rot(d['q'].data_ptr(), d['k'].data_ptr(), d['v'].data_ptr(), d['sw_k'].data_ptr(),
                                              x.data_ptr(), d['sw_v'].data_ptr(), gw.data_ptr(), hd.data_ptr(),
                                              cosq.data_ptr(), sinq.data_ptr(), 0, d['hk'].data_ptr(), d['hv'].data_ptr(),
                                              d['o'].data_ptr(), ws.data_ptr(), ws.numel(), B, H * NG, H, K, K, M, W, W,
                                              K ** -0.5, stream)
            assert st == 0
            if append:
                st = lib.nha_ring_append_rot(d['sw_k'].data_ptr(), x.data_ptr(), d['sw_v'].data_ptr(), gw.data_ptr(),
                                             d['k'].data_ptr(), d['v'].data_ptr(), gn.data_ptr(), cosq.data_ptr(),
                                             sinq.data_ptr(), 0, hd.data_ptr(), B, H, K, K, M, W, W, stream)
                assert st == 0
    for _ in range(2):
        step_shift()
        step_ring()
        step_ring_fused()
        step_ring_rot()
    ms_shift = timed(step_shift, 10) / 10
    ms_ring = timed(step_ring, 50) / 50
    ms_fused = timed(step_ring_fused, 100) / 100
    ms_rot = timed(step_ring_rot, 50) / 50
    ms_rot_only = timed(lambda: step_ring_rot(False), 50) / 50
    with_cache = {'shifted_window_us_per_layer': 1e3 * ms_shift / LAYERS, 'ring_us_per_layer': 1e3 * ms_ring / LAYERS,
                  'ring_tokens_per_s': world * B / (ms_ring * 1e-3),
                  'ring_fused_us_per_layer': 1e3 * ms_fused / LAYERS,
                  'ring_fused_tokens_per_s': world * B / (ms_fused * 1e-3),
                  'ring_rotated_keys_us_per_layer': 1e3 * ms_rot / LAYERS,
                  'ring_rotated_keys_tokens_per_s': world * B / (ms_rot * 1e-3),
                  'ring_rotated_keys_decode_only_us_per_layer': 1e3 * ms_rot_only / LAYERS,
                  'ring_rotated_keys_decode_only_gbs': per_seq_layer * B * LAYERS / (ms_rot_only * 1e-3) / 1e9,
                  'note': 'one generated token per sequence including the window cache update of every layer'}
    return {'workload': 'decode 48 layers x 32 seq/GPU HQ32 H4 D128 M64 W512 bf16, fp32 state', 'ms_per_token_step': ms,
            'with_cache_update': with_cache,
            'tokens_per_s': world * B / (ms * 1e-3), 'us_per_layer': 1e3 * ms / LAYERS,
            'bf16_state': bf16_state,
            'dependent_launch': {'us_per_layer_plain': 1e3 * by_mode[0] / LAYERS,
                                 'us_per_layer_wait_first': 1e3 * by_mode[1] / LAYERS,
                                 'us_per_layer_early_requests': 1e3 * by_mode[2] / LAYERS,
                                 'us_per_layer_early_requests_cuda_graph': graph_us,
                                 'headline_mode': 'early requests (mode 2), eager launches'},
            'roofline': {'bound': 'hbm', 'achieved': gbs, 'peak': peak, 'unit': 'GB/s', 'frac': gbs / peak,
                         'algorithmic_bytes_per_launch': per_seq_layer * B}, 'gpu_launches_per_step': LAYERS}


def bench_prefill(dev, rank, world, dist, timed):
    """Long-context prefill, Llama-3-8B attention shape: B=1 T=131072 HQ=32 H=8 D=128 M=64 W=512 bf16, forward.
    With N > 1 the sequence is cut into N contiguous segments (sequence parallel: halo + all-gather of state summaries)."""
    import nha_b200
    from nha_b200.sharding import sequence_parallel_prefill
    T, HQ, H, K, M, W = 131072, 32, 8, 128, 64, 512
    Tr = T // world
    g = torch.Generator(device='cpu').manual_seed(7 + rank)
    mk = lambda *sh: torch.randn(*sh, generator=g).bfloat16().to(dev)
    q, rq = mk(1, Tr, HQ, K), mk(1, Tr, HQ, K)
    k, rk, v = mk(1, Tr, H, K), mk(1, Tr, H, K), mk(1, Tr, H, K)
    gl = F.logsigmoid(torch.randn(1, Tr, H, M, generator=g)) / 8
    gg, ss = gl.bfloat16().to(dev), (1 - gl.exp()).bfloat16().to(dev)

    def step():
        if world == 1:
            return nha_b200.fused_chunk_nha_prefill(q=q, k=k, v=v, rotary_q=rq, rotary_k=rk, s=ss, g=gg, window_size=W,
                                                    output_final_state=True)
        return sequence_parallel_prefill(q, k, v, rq, rk, ss, gg, W)
    # values first (N > 1): a short sequence (the same on every rank) cut into the ranks' segments must reproduce the
    # single-GPU op on this rank's segment and, on the last rank, its final state
    check = None
    if world > 1:
        Ts = 1024 * world
        gs = torch.Generator(device='cpu').manual_seed(4242)
        mks = lambda *sh: torch.randn(*sh, generator=gs).bfloat16().to(dev)
        sq, srq, sk, srk, sv = mks(1, Ts, HQ, K), mks(1, Ts, HQ, K), mks(1, Ts, H, K), mks(1, Ts, H, K), mks(1, Ts, H, K)
        sgl = F.logsigmoid(torch.randn(1, Ts, H, M, generator=gs)) / 8
        sgg, sss = sgl.bfloat16().to(dev), (1 - sgl.exp()).bfloat16().to(dev)
        ref_o, (ref_hk, ref_hv) = nha_b200.fused_chunk_nha_prefill(q=sq, k=sk, v=sv, rotary_q=srq, rotary_k=srk, s=sss, g=sgg,
                                                                   window_size=W, output_final_state=True)
        a, b = Ts * rank // world, Ts * (rank + 1) // world
        seg = lambda x: x[:, a:b].contiguous()
        so, (shk, shv) = sequence_parallel_prefill(seg(sq), seg(sk), seg(sv), seg(srq), seg(srk), seg(sss), seg(sgg), W)
        rel = lambda x, y: float((x.float() - y.float()).norm() / y.float().norm().clamp_min(1e-30))
        e = rel(so, ref_o[:, a:b])
        if rank == world - 1:
            e = max(e, rel(shk, ref_hk), rel(shv, ref_hv))
        te = torch.tensor([e], device=dev)
        dist.all_reduce(te, op=dist.ReduceOp.MAX)
        check = {'tokens': Ts, 'rel_l2_vs_single_gpu_max_over_ranks': float(te.item()), 'bound': 1e-2}
    for _ in range(2):
        step()
    ms = timed(step, 30) / 30
    ms_eager, captured = ms, False
    if world > 1:
        # the same call captured once as a CUDA graph (kernels, halo messages, all-gather): a rank's host work per call
        # shrinks to one graph launch.  Every rank must take the same branch, so the outcome of the capture is agreed on.
        from nha_b200.sharding import GraphedPrefill
        graphed = None
        try:
            graphed = GraphedPrefill(q, k, v, rq, rk, ss, gg, W)
        except Exception as e:                                   # noqa: BLE001 - reported, the eager figure stands
            print(f'[bench] rank {rank}: graph capture failed: {e}', file=sys.stderr)
        ok = torch.tensor([1 if graphed is not None else 0], device=dev)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if int(ok.item()) == 1:
            for _ in range(3):
                graphed()
            ms, captured = timed(graphed, 30) / 30, True
    flops = T * 9699328.0
    return {'workload': f'prefill fwd B1 T131072 HQ32 H8 D128 M64 W512 bf16, sequence-parallel x{world}', 'ms': ms,
            'ms_eager_calls': ms_eager, 'captured_as_graph': captured,
            'sequence_parallel_check': check,
            'tokens_per_s': T / (ms * 1e-3), 'tflops': flops / (ms * 1e-3) / 1e12,
            'roofline': {'bound': 'tensor', 'achieved': flops / (ms * 1e-3) / 1e12 / world,
                         'peak': tensor_peak(), 'unit': 'TFLOP/s per GPU',
                         'frac': flops / (ms * 1e-3) / 1e12 / world / tensor_peak()}}


def bench_varlen(dev, rank, timed):
    """Varlen packed forward + backward: 32768 tokens per GPU, sequence lengths uniform[128, 8192], per-sequence
    window from {32, 64, 128, 256, 512}, H16 D64 M64, through the public chunk_nha op."""
    import nha_b200
    H, D, M, total = 16, 64, 64, 32768
    g = torch.Generator().manual_seed(7 + rank)
    lens = []
    while sum(lens) < total:
        lens.append(int(torch.randint(128, 8193, (1,), generator=g)))
    lens[-1] -= sum(lens) - total
    if lens[-1] < 1:
        lens[-2] += lens[-1] - 1
        lens[-1] = 1
    wins = [int([32, 64, 128, 256, 512][int(torch.randint(0, 5, (1,), generator=g))]) for _ in lens]
    cu = torch.tensor([0] + list(torch.tensor(lens).cumsum(0)), dtype=torch.int32, device=dev)
    wl = torch.tensor(wins, dtype=torch.int32, device=dev)
    sh = torch.zeros(len(lens), dtype=torch.int32, device=dev)
    gd = torch.Generator(device=dev).manual_seed(17 + rank)
    r = lambda *s: torch.randn(*s, generator=gd, device=dev)
    x = {n: (r(1, total, H, D) * D ** -0.5).bfloat16().requires_grad_(True) for n in ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v')}
    gg = F.logsigmoid(r(1, total, H, M)).bfloat16()
    x['s'] = (1 - gg.float().exp()).bfloat16().detach().requires_grad_(True)
    x['g'] = gg.detach().requires_grad_(True)
    do = r(1, total, H, D).bfloat16()

    def step():
        for t in x.values():
            t.grad = None
        o, _, _ = nha_b200.chunk_nha(x['q_swa'], x['k_swa'], x['q_gsa'], x['k_gsa'], x['v'], x['s'], x['g'], cu_seqlens=cu,
                                     max_seqlen=max(lens), scale=D ** -0.5, window_size_left=wl, window_size_right=0,
                                     gsa_kv_shift=sh)
        o.backward(do)
    for _ in range(3):
        step()
    ms = timed(step, 100) / 100
    return {'workload': f'varlen fwd+bwd, {total} packed tokens in {len(lens)} sequences of 128-8192, windows 32-512, '
                        f'H16 D64 M64 bf16', 'ms': ms, 'tokens_per_s_per_gpu': total / (ms * 1e-3)}


def bench_gates(lib, dev, rank, timed, peak):
    """The callers' gate chain at the bench workload's gate shape (B16 T2048 H16 M64): g = logsigmoid(f) / 8 and
    s = 1 - exp(g) from one pass over f (nha_slot_gates_fwd) and df from dg, ds (nha_slot_gates_bwd), beside the
    layer's own chain of element-wise torch kernels (nha_fla/layers/nha.py:229-231) with autograd."""
    n = 16 * 2048 * 16 * 64
    gd = torch.Generator(device=dev).manual_seed(23 + rank)
    f = (torch.randn(n, generator=gd, device=dev) * 2).bfloat16()
    dg = torch.randn(n, generator=gd, device=dev).bfloat16()
    ds = torch.randn(n, generator=gd, device=dev).bfloat16()
    g, s, df = torch.empty_like(f), torch.empty_like(f), torch.empty_like(f)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def fwd():
        assert lib.nha_slot_gates_fwd(f.data_ptr(), g.data_ptr(), s.data_ptr(), n, 8.0, stream) == 0

    def bwd():
        assert lib.nha_slot_gates_bwd(f.data_ptr(), dg.data_ptr(), ds.data_ptr(), df.data_ptr(), n, 8.0, stream) == 0
    ft = f.clone().requires_grad_(True)

    def chain():
        ft.grad = None
        g1 = F.logsigmoid(ft) / 8.0
        s1 = (1 - g1.exp()).to(g1.dtype)
        torch.autograd.backward([g1, s1], [dg, ds])
    for fn in (fwd, bwd, chain):
        for _ in range(3):
            fn()
    ms_f, ms_b, ms_c = timed(fwd, 20) / 20, timed(bwd, 20) / 20, timed(chain, 10) / 10
    bytes_f, bytes_b = n * 6, n * 8                       # f read, g and s written; f, dg, ds read, df written
    return {'workload': 'slot gates g = logsigmoid(f)/8, s = 1 - exp(g): B16 T2048 H16 M64 bf16 (201 MB forward, 268 MB '
                        'backward: larger than L2)',
            'fwd_ms': ms_f, 'bwd_ms': ms_b, 'torch_chain_fwd_bwd_ms': ms_c, 'gpu_launches_fwd_bwd': 2,
            'roofline': {'bound': 'hbm', 'achieved': (bytes_f + bytes_b) / ((ms_f + ms_b) * 1e-3) / 1e9, 'peak': peak,
                         'unit': 'GB/s', 'frac': (bytes_f + bytes_b) / ((ms_f + ms_b) * 1e-3) / 1e9 / peak,
                         'fwd_gbs': bytes_f / (ms_f * 1e-3) / 1e9, 'bwd_gbs': bytes_b / (ms_b * 1e-3) / 1e9}}


def bench_rotary(lib, dev, rank, timed, peak):
    """The layer's rotary call at the bench workload's shape (B16 T2048 H16 D64): q and k rotated by one launch
    (nha_rope_pair), 268 MB read + written."""
    B, T, H, K = 16, 2048, 16, 64
    gd = torch.Generator(device=dev).manual_seed(29 + rank)
    q = torch.randn(B * T, H, K, generator=gd, device=dev).bfloat16()
    k = torch.randn(B * T, H, K, generator=gd, device=dev).bfloat16()
    qo, ko = torch.empty_like(q), torch.empty_like(k)
    inv = 1.0 / (10000.0 ** (torch.arange(0, K, 2, dtype=torch.float32) / K))
    fr = torch.outer(torch.arange(T, dtype=torch.float32), inv)
    cos, sin = fr.cos().bfloat16().to(dev).contiguous(), fr.sin().bfloat16().to(dev).contiguous()
    stream = torch.cuda.current_stream(dev).cuda_stream

    def step():
        assert lib.nha_rope_pair(q.data_ptr(), k.data_ptr(), qo.data_ptr(), ko.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                 cos.stride(0), T, None, 0, T, B * T, H, H, K, 0, 0, stream) == 0
    for _ in range(3):
        step()
    ms = timed(step, 20) / 20
    nbytes = 4 * q.numel() * 2
    return {'workload': 'rotary of q and k, B16 T2048 H16 D64 bf16, one launch (268 MB: larger than L2)', 'ms': ms,
            'gpu_launches': 1,
            'roofline': {'bound': 'hbm', 'achieved': nbytes / (ms * 1e-3) / 1e9, 'peak': peak, 'unit': 'GB/s',
                         'frac': nbytes / (ms * 1e-3) / 1e9 / peak}}


def bench_layer_ops(lib, dev, rank, timed, peak):
    """The layer's element-wise work around the operator at the bench workload's shape (B16 T2048 H16 D64, hidden 1024):
    feature map of q and k with silu(v) in one launch (nha_fla/layers/nha.py:219-223) and silu + RMS norm in front of the
    output projection (nha_fla/layers/nha.py:277-278), forward and backward through the C ABI, beside the same lines in
    torch with autograd."""
    import ctypes
    import torch.nn.functional as F
    B, T, H, K = 16, 2048, 16, 64
    gd = torch.Generator(device=dev).manual_seed(41 + rank)
    mk = lambda *sh: torch.randn(*sh, generator=gd, device=dev).bfloat16()
    stream = torch.cuda.current_stream(dev).cuda_stream
    xs = [mk(B * T, H, K) for _ in range(3)]
    dys = [mk(B * T, H, K) for _ in range(3)]
    ys = [torch.empty_like(x) for x in xs]
    arr = lambda ts: (ctypes.c_void_p * 3)(*[t.data_ptr() for t in ts])
    n3 = (ctypes.c_int64 * 3)(*[x.numel() for x in xs])

    def fm_fwd():
        assert lib.nha_act3_fwd(arr(xs), arr(ys), n3, None, 3, stream) == 0

    def fm_bwd():
        assert lib.nha_act3_bwd(arr(xs), arr(dys), arr(ys), n3, None, 3, stream) == 0
    xg = [x.clone().requires_grad_(True) for x in xs]

    def fm_torch():
        torch.autograd.backward([F.silu(x) for x in xg], dys)
    rows, cols = B * T, H * K
    o, dy, y, d_o = mk(rows, cols), mk(rows, cols), torch.empty(rows, cols, dtype=torch.bfloat16, device=dev), None
    d_o = torch.empty_like(o)
    w = torch.rand(cols, generator=gd, device=dev) + 0.5
    bias = torch.zeros(cols, device=dev)
    rstd = torch.empty(rows, device=dev)
    nparts = int(lib.nha_silu_rmsnorm_bwd_ctas(rows))
    pw, pb = torch.empty(nparts, cols, device=dev), torch.empty(nparts, cols, device=dev)

    def nm_fwd():
        assert lib.nha_silu_rmsnorm_fwd(o.data_ptr(), w.data_ptr(), bias.data_ptr(), y.data_ptr(), rstd.data_ptr(), rows, cols,
                                        1e-5, stream) == 0

    def nm_bwd():
        assert lib.nha_silu_rmsnorm_bwd(o.data_ptr(), w.data_ptr(), rstd.data_ptr(), dy.data_ptr(), d_o.data_ptr(),
                                        pw.data_ptr(), pb.data_ptr(), rows, cols, stream) == 0
        pw.sum(0), pb.sum(0)
    og, wg, bg = o.clone().requires_grad_(True), w.clone().requires_grad_(True), bias.clone().requires_grad_(True)

    def nm_torch():
        x = F.silu(og).float()
        (x * torch.rsqrt(x.pow(2).mean(-1, keepdim=True) + 1e-5) * wg + bg).to(og.dtype).backward(dy)
    res = {}
    for name, fn in (('fm_fwd', fm_fwd), ('fm_bwd', fm_bwd), ('fm_torch', fm_torch), ('nm_fwd', nm_fwd), ('nm_bwd', nm_bwd),
                     ('nm_torch', nm_torch)):
        for _ in range(3):
            fn()
        res[name] = timed(fn, 20) / 20
    e3, eo = 3 * xs[0].numel() * 2, o.numel() * 2
    gbs = lambda nbytes, ms: nbytes / (ms * 1e-3) / 1e9
    return {'workload': 'feature map of q, k + silu(v) (B16 T2048 H16 D64: 201 MB per tensor set) and silu + RMS norm over '
                        'hidden 1024 (67 MB), bf16; every pass larger than L2',
            'feature_maps': {'fwd_ms': res['fm_fwd'], 'bwd_ms': res['fm_bwd'], 'torch_fwd_bwd_ms': res['fm_torch'],
                             'fwd_gbs': gbs(2 * e3, res['fm_fwd']), 'bwd_gbs': gbs(3 * e3, res['fm_bwd']), 'gpu_launches': 2},
            'silu_rms_norm': {'fwd_ms': res['nm_fwd'], 'bwd_ms': res['nm_bwd'], 'torch_fwd_bwd_ms': res['nm_torch'],
                              'fwd_gbs': gbs(2 * eo, res['nm_fwd']), 'bwd_gbs': gbs(3 * eo, res['nm_bwd']),
                              'gpu_launches': '1 forward; 1 + two small column sums backward'},
            'roofline': {'bound': 'hbm', 'peak': peak, 'unit': 'GB/s',
                         'achieved': gbs(5 * e3, res['fm_fwd'] + res['fm_bwd']),
                         'frac': gbs(5 * e3, res['fm_fwd'] + res['fm_bwd']) / peak,
                         'silu_rms_norm_achieved': gbs(5 * eo, res['nm_fwd'] + res['nm_bwd']),
                         'silu_rms_norm_frac': gbs(5 * eo, res['nm_fwd'] + res['nm_bwd']) / peak}}


def bench_lse_stats(lib, dev, rank, timed):
    """The training layer's aux loss and compression statistic at the bench shape (T*HQ = 524288 log-sum-exp pairs,
    4 MB): one launch for both means plus one for the gradient, beside the layer's chain of torch kernels with
    autograd and its .item() (nha_fla/layers/nha.py:255-264, 288-323)."""
    n = 16 * 2048 * 16
    gd = torch.Generator(device=dev).manual_seed(37 + rank)
    ls = torch.randn(n, generator=gd, device=dev) * 3
    lg = torch.randn(n, generator=gd, device=dev) * 3
    out, d = torch.empty(2, device=dev), torch.empty(n, device=dev)
    one = torch.ones(1, device=dev)
    scratch = torch.zeros(int(lib.nha_lse_stats_scratch_bytes()), dtype=torch.uint8, device=dev)
    stream = torch.cuda.current_stream(dev).cuda_stream

    def ours():
        assert lib.nha_lse_stats(ls.data_ptr(), lg.data_ptr(), n, 0.3, out.data_ptr(), scratch.data_ptr(), stream) == 0
        assert lib.nha_lse_aux_grad(ls.data_ptr(), lg.data_ptr(), one.data_ptr(), n, 0.3, d.data_ptr(), stream) == 0
    lgt = lg.clone().requires_grad_(True)

    def chain():
        lgt.grad = None
        mx = torch.maximum(ls, lgt)
        w_swa, w_gsa = torch.exp(ls - mx), torch.exp(lgt - mx)
        with torch.no_grad():
            (w_gsa / (w_swa + w_gsa)).mean().item()
        delta = lgt.float() - ls.detach().float()
        F.binary_cross_entropy_with_logits(delta, torch.full_like(delta, 0.3), reduction='mean').backward()
    for fn in (ours, chain):
        for _ in range(3):
            fn()
    return {'workload': 'aux loss + slot-branch share from 524288 lse pairs, forward and gradient', 'ms': timed(ours, 20) / 20,
            'torch_chain_ms': timed(chain, 10) / 10, 'gpu_launches': 2}


def tensor_peak():
    p = os.path.join(ROOT, 'MEASURED_PEAKS.json')
    if os.path.exists(p):
        return float(json.load(open(p))['bf16_tflops'])
    return 1590.0


_RESULT_OUT = None


def claim_stdout():
    """Keep the process's stdout for the one JSON line: file descriptor 1 is pointed at stderr, so that
    whatever a library writes there (NCCL's version banner, for one) cannot land beside the result."""
    global _RESULT_OUT
    if _RESULT_OUT is None:
        sys.stdout.flush()
        _RESULT_OUT = os.fdopen(os.dup(1), 'w')
        os.dup2(2, 1)
    return _RESULT_OUT


def emit(line):
    out = claim_stdout()
    out.write(json.dumps(line) + '\n')
    out.flush()


# ---------------------------------------------------------------------------------------------
def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--gpus', type=int, default=1)
    ap.add_argument('--steps', type=int, default=20)
    ap.add_argument('--warmup', type=int, default=3)
    ap.add_argument('--impl', default='ours')
    ap.add_argument('--no-cpu-baseline', action='store_true')
    ap.add_argument('--no-e2e', action='store_true')
    ap.add_argument('--no-extras', action='store_true', help='skip the decode and long-context prefill side measurements')
    ap.add_argument('--small', action='store_true', help='B=4 instead of 16 (profiling captures)')
    ap.add_argument('--no-repeat', action='store_true', help='time each region once, without the inner repeats that '
                    'stretch it to half a second (profiling captures: few launches)')
    ap.add_argument('--pre-op', action='store_true', help='only the slot-gate and rotary side measurements (profiling '
                    'captures of those kernels; prints their JSON, not the bench line)')
    args = ap.parse_args()
    claim_stdout()
    args.warmup = max(args.warmup, 3)
    if args.impl == 'reference':
        return run_reference(args)

    world = int(os.environ.get('WORLD_SIZE', '1'))
    rank = int(os.environ.get('RANK', '0'))
    local = int(os.environ.get('LOCAL_RANK', '0'))
    dist = None
    if world > 1:
        import torch.distributed as dist
        os.environ.setdefault('MASTER_ADDR', '127.0.0.1')
        os.environ.setdefault('NCCL_DEBUG_FILE', '/tmp/nccl_debug.%h.%p')   # keep stdout to the one JSON line
        dist.init_process_group('nccl', device_id=torch.device('cuda', local))
    torch.cuda.set_device(local)
    dev = torch.device('cuda', local)

    import nha_b200
    from nha_b200 import _lib
    from nha_b200.chunk import _Geometry, _fill_desc, chunk_backward, chunk_forward
    lib = _lib.load()

    c = dict(CFG)
    if args.small:
        c['B'] = 4
    B, T, H, D, M, W, shift = c['B'], c['T'], c['H'], c['D'], c['M'], c['W'], c['shift']
    scale = D ** -0.5
    host = gen_inputs(1234 + rank, B, T, H, D, M, pin=not args.no_e2e)
    flat = lambda x: x.reshape(B * T, *x.shape[2:])
    x = {n: flat(host[n]).to(dev) for n in NAMES}
    do = flat(host['do']).to(dev)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=dev)
    tokens = B * T

    def step():
        o, ls, lg, _, _, saved = chunk_forward(x['q_gsa'], x['q_swa'], x['k_gsa'], x['k_swa'], x['v'], x['s'], x['g'],
                                               cu, T, scale, W, shift)
        return chunk_backward(x['q_gsa'], x['q_swa'], x['k_gsa'], x['k_swa'], x['v'], x['s'], x['g'], cu, scale, saved,
                              o, ls, lg, do)

    def barrier():
        if dist is not None:
            dist.barrier()
        torch.cuda.synchronize()

    def timed(fn, steps):
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        barrier()
        e0.record()
        for _ in range(steps):
            fn()
        e1.record()
        barrier()
        ms = e0.elapsed_time(e1)
        if dist is not None:
            t = torch.tensor([ms], device=dev)
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
            ms = float(t.item())
        return ms

    if args.pre_op:
        pk = peaks()[0]
        out = {'gates': bench_gates(lib, dev, rank, timed, pk), 'rotary': bench_rotary(lib, dev, rank, timed, pk),
               'lse_stats': bench_lse_stats(lib, dev, rank, timed), 'layer_ops': bench_layer_ops(lib, dev, rank, timed, pk)}
        if rank == 0:
            emit(out)
        return 0

    # clocks and throttle reasons are sampled from the warm-up to the last measurement of this process (the timed
    # region itself lasts tens of milliseconds, less than one sampling period)
    clk = ClockSampler(local).start()
    for _ in range(args.warmup):
        step()
    # K steps are timed once to size the region, then K x inner_repeats steps back to back (about half a second, so
    # that the clock samples fall inside it); `ms` is the time of K steps
    ms_cal = timed(step, args.steps)
    reps = 1 if args.no_repeat else max(1, int(math.ceil(500.0 / max(ms_cal, 1e-3))))
    if dist is not None:
        t_r = torch.tensor([reps], device=dev)
        dist.all_reduce(t_r, op=dist.ReduceOp.MAX)
        reps = int(t_r.item())
    ms = timed(step, args.steps * reps) / reps
    value = world * tokens * args.steps / (ms * 1e-3)

    def timed_avg(fn, min_ms=250.0):
        """ms per call of `fn`, measured over a region of at least `min_ms`."""
        cal = timed(fn, args.steps) / args.steps
        if args.no_repeat:
            return cal
        n = max(args.steps, int(math.ceil(min_ms / max(cal, 1e-4))))
        if dist is not None:
            t_n = torch.tensor([n], device=dev)
            dist.all_reduce(t_n, op=dist.ReduceOp.MAX)
            n = int(t_n.item())
        return timed(fn, n) / n
    # plan, state pass (2), output pass (2), backward: rows (2), window columns (1), slot (1), state-gradient terms +
    # scan + gate carry + columns + general inter-chunk kernel (5); the general kernels run gated on the chunk flags
    launches_per_step = 14

    # ---- per-kernel timing: every kernel of a step on its own, CUDA events on the launching stream ----
    kernels = {}
    o, ls, lg, _, _, saved = chunk_forward(x['q_gsa'], x['q_swa'], x['k_gsa'], x['k_swa'], x['v'], x['s'], x['g'], cu, T,
                                           scale, W, shift)
    geo = saved['geo']
    t = dict(x, cu_seqlens=cu, o=o, lse_swa=ls, lse_gsa=lg, hk_chunks=saved['hk_chunks'], hv_chunks=saved['hv_chunks'],
             d_o=do)
    for n in NAMES:
        t['d' + n] = torch.empty_like(x[n])
    d0 = _fill_desc(geo, t, scale, None, W, None, shift)
    t['workspace'] = torch.empty(max(16, int(lib.nha_chunk_bwd_workspace_bytes(d0))), dtype=torch.uint8, device=dev)
    desc = _fill_desc(geo, t, scale, None, W, None, shift)
    stream = torch.cuda.current_stream(dev).cuda_stream
    import ctypes
    calls = {
        'state_pass': lambda: lib.nha_chunk_state_pass(ctypes.byref(desc), stream),
        'output_pass': lambda: lib.nha_chunk_output_pass(ctypes.byref(desc), stream),
        'bwd_rows': lambda: lib.nha_chunk_bwd_stage(ctypes.byref(desc), 0, stream),
        'bwd_window_cols': lambda: lib.nha_chunk_bwd_stage(ctypes.byref(desc), 1, stream),
        'bwd_slot_general': lambda: lib.nha_chunk_bwd_stage(ctypes.byref(desc), 2, stream),
        'bwd_state_scan': lambda: lib.nha_chunk_bwd_stage(ctypes.byref(desc), 3, stream),
        'bwd_cols': lambda: lib.nha_chunk_bwd_stage(ctypes.byref(desc), 4, stream),
    }
    # compulsory bytes of each stage per token (all heads): what its kernels must read once and write once,
    # scratch that one kernel hands to the next included (e = bf16, f = fp32; states per 64-token chunk)
    e, f = 2, 4
    st = 2 * D * M / 64
    per_tok = {
        # k', v, s, g in; per-chunk terms out (fp32) and back in; chunk-start states out (bf16)
        'state_pass': H * ((2 * D + 2 * M) * e + st * (2 * f + e)),
        # q_gsa, q_swa, k_gsa, k_swa, v, s, g, states in; o and both log-sum-exps out
        'output_pass': H * ((5 * D + 2 * M) * e + st * e + D * e + 2 * f),
        # q_gsa, q_swa, do, o, k_gsa, k_swa, v, s, g, states, log-sum-exps in; dq_gsa, dq_swa, delta, joint LSE,
        # gate terms (fp32), two bf16 copies of dz / p, the chunk's state-gradient terms (fp32) out
        'bwd_rows': H * ((7 * D + 2 * M) * e + st * e + 2 * f + 2 * D * e + 2 * f + M * f + 2 * M * e + st * f),
        # k_swa, v, q_swa, do, joint LSE, delta in; dk_swa and the fp32 window part of dv out
        'bwd_window_cols': H * (4 * D * e + 2 * f + D * e + D * f),
        # general kernel of the slot branch: runs only on chunks flagged by the forward (none here)
        'bwd_slot_general': H * ((4 * D + 2 * M) * e + st * e + 4 * f + D * e + (2 * D + 2 * M) * f + 2 * M * e),
        # in-place scan of the chunks' fp32 state-gradient terms
        'bwd_state_scan': H * (st * 2 * f),
        # gate carry (fp32 state gradients and next states in, bf16 copies out), columns pass (q_gsa, do, k_gsa, v,
        # s, g, dz / p copies, bf16 state gradients, gate terms, window dv in; dk_gsa, dv, ds, dg out)
        'bwd_cols': H * (st * (f + 2 * e) + (4 * D + 4 * M) * e + st * e + M * f + D * f + (2 * D + 2 * M) * e),
    }
    for name, fn in calls.items():
        for _ in range(3):
            assert fn() == 0
        kms = timed_avg(fn)
        kernels[name] = {'ms': kms, 'stage_bytes': per_tok[name] * tokens, 'gbs': per_tok[name] * tokens / (kms * 1e-3) / 1e9}
    top = max(kernels, key=lambda k: kernels[k]['ms'])
    stage_sum = sum(k['ms'] for k in kernels.values())
    peak, how = peaks()
    # DRAM bytes of one step: dram__bytes_read.sum + dram__bytes_write.sum of every kernel of a step, one ncu capture
    # per kernel on the B=4 case (8192 tokens; traffic grows in proportion to the tokens), summed; the per-kernel
    # figures are in profiles/step_traffic_chunk_fwd_bwd_B4_T2048.md
    traffic = NCU_STEP_TRAFFIC_PER_TOKEN * tokens if NCU_STEP_TRAFFIC_PER_TOKEN else None
    step_gbs = ALG_BYTES_PER_TOKEN * tokens * args.steps / (ms * 1e-3) / 1e9
    roofline = {'bound': 'hbm', 'achieved': step_gbs, 'peak': peak, 'unit': 'GB/s', 'frac': step_gbs / peak,
                'traffic': traffic, 'peak_source': how, 'algorithmic_bytes_per_step': ALG_BYTES_PER_TOKEN * tokens,
                'scope': 'one forward + backward step (all kernels), algorithmic bytes = inputs once per pass + outputs once',
                'kernel': top, 'kernel_share': kernels[top]['ms'] / stage_sum,
                'stage_bytes_per_step': sum(k['stage_bytes'] for k in kernels.values())}

    # ---- end to end through the public API with host buffers -------------------------------------------
    # Every step copies its inputs from pinned host memory, runs chunk_nha forward + backward through the public
    # op, and reads o, both log-sum-exps and all seven gradients back to pinned host memory.  The three parts run
    # on three streams with the inputs double-buffered, so the copy-in of step i + 1 and the read-back of step
    # i - 1 overlap the compute of step i (PCIe is full duplex); every copy of every step is inside the timed
    # region.
    e2e = None
    if not args.no_e2e:
        s_in, s_cmp, s_out = (torch.cuda.Stream(dev) for _ in range(3))
        dbuf = [{n: torch.empty(B, T, *host[n].shape[2:], dtype=torch.bfloat16, device=dev) for n in NAMES + ('do',)}
                for _ in range(2)]
        out_host = {n: torch.empty_like(host[n]).pin_memory() for n in NAMES}
        o_host = torch.empty(B, T, H, D, dtype=torch.bfloat16).pin_memory()
        lse_host = torch.empty(2, B, T, H, dtype=torch.float32).pin_memory()
        ev_in = [torch.cuda.Event() for _ in range(2)]
        ev_cmp = [torch.cuda.Event() for _ in range(2)]

        def e2e_run(steps):
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record(s_in)
            for i in range(steps):
                sl = i % 2
                with torch.cuda.stream(s_in):
                    if i >= 2:
                        s_in.wait_event(ev_cmp[sl])          # the compute that read this input buffer has finished
                    for n in NAMES + ('do',):
                        dbuf[sl][n].copy_(host[n], non_blocking=True)
                    ev_in[sl].record(s_in)
                with torch.cuda.stream(s_cmp):
                    s_cmp.wait_event(ev_in[sl])
                    leaves = {n: dbuf[sl][n].detach().requires_grad_(True) for n in NAMES}
                    o, ls, lg = nha_b200.chunk_nha(leaves['q_swa'], leaves['k_swa'], leaves['q_gsa'], leaves['k_gsa'],
                                                   leaves['v'], leaves['s'], leaves['g'], scale=scale,
                                                   window_size_left=W, window_size_right=0, gsa_kv_shift=shift)
                    o.backward(dbuf[sl]['do'])
                    ev_cmp[sl].record(s_cmp)
                with torch.cuda.stream(s_out):
                    s_out.wait_event(ev_cmp[sl])
                    results = [o.detach(), ls, lg] + [leaves[n].grad for n in NAMES]
                    for r in results:
                        r.record_stream(s_out)
                    o_host.copy_(results[0], non_blocking=True)
                    lse_host[0].copy_(ls, non_blocking=True)
                    lse_host[1].copy_(lg, non_blocking=True)
                    for n in NAMES:
                        out_host[n].copy_(leaves[n].grad, non_blocking=True)
            e1.record(s_out)
            e1.synchronize()
            torch.cuda.synchronize()
            ems_ = e0.elapsed_time(e1)
            if dist is not None:
                tt = torch.tensor([ems_], device=dev)
                dist.all_reduce(tt, op=dist.ReduceOp.MAX)
                ems_ = float(tt.item())
            return ems_

        e2e_run(3)
        ems = e2e_run(args.steps)
        h2d = sum(host[n].numel() * 2 for n in NAMES + ('do',))
        d2h = o_host.numel() * 2 + lse_host.numel() * 4 + sum(out_host[n].numel() * 2 for n in NAMES)
        e2e = {'value': world * tokens * args.steps / (ems * 1e-3), 'unit': UNIT, 'h2d_bytes_per_step': h2d,
               'd2h_bytes_per_step': d2h, 'ms_per_step': ems / args.steps,
               'overlap': 'copy-in, compute and read-back on three streams, inputs double-buffered'}

    # ---- side measurements (not the headline): batched decode and long-context prefill ---------------------
    extras = None
    if not args.no_extras and not args.small:
        extras = {'decode': bench_decode(lib, dev, rank, world, timed, peak),
                  'prefill': bench_prefill(dev, rank, world, dist, timed),
                  'varlen': bench_varlen(dev, rank, timed),
                  'gates': bench_gates(lib, dev, rank, timed, peak),
                  'rotary': bench_rotary(lib, dev, rank, timed, peak),
                  'lse_stats': bench_lse_stats(lib, dev, rank, timed),
                  'layer_ops': bench_layer_ops(lib, dev, rank, timed, peak)}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        Ts = CPU_SLICE_T
        tps, secs = cpu_oracle_tokens_per_s(Ts, repeats=3)
        cpu = {'value': tps, 'unit': UNIT, 'cores': os.cpu_count(), 'kind': 'port',
               'sample': f'B=1 T={Ts} slice of the workload, fp64 oracle fwd + autograd bwd, {secs:.1f} s'}

    clk.stop()
    if rank == 0:
        line = {
            'metric': METRIC, 'value': value, 'unit': UNIT, 'n_gpus': world, 'steps': args.steps, 'warmup': args.warmup,
            'ms_per_step': ms / args.steps, 'higher_is_better': True, 'scaling': 'weak', 'vs_baseline': None,
            'dtype': 'bf16', 'data': 'synthetic',
            'config': {'workload': WORKLOAD if not args.small else WORKLOAD.replace('B16', 'B4'),
                       'tokens_per_gpu_per_step': tokens, 'window_left': W, 'gsa_kv_shift': shift,
                       'parallelism': f'batch-sharded x{world}, no collective',
                       'l2': 'inputs of one step (0.54 GB) exceed the 126 MB L2; no flush between steps'},
            'inner_repeats': reps, 'roofline': roofline, 'kernels': kernels,
            'cpu_baseline': cpu, 'e2e': e2e, 'gpu_launches': launches_per_step * args.steps, 'extras': extras,
            'clocks': clk.summary(),
        }
        emit(line)
    if dist is not None:
        dist.destroy_process_group()


if __name__ == '__main__':
    main()
