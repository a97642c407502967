"""Generate the golden fixtures of tests/golden/ from the reference itself.

Run where the reference checkout is readable (it is not needed, and not read,
by any test):

    python tests/golden/make_golden.py --reference /path/to/NHA

What it does
  1. imports the reference's fp64 naive functions ``ref_decode``,
     ``ref_fused_recurrent`` and ``ref_prefill`` (scripts/verify_opt_parity.py)
     and its input generators, forced onto the CPU;
  2. checks the oracle restatement (oracle/nha_oracle.py) against them on the
     reference's FULL case grids (decode/recurrent: NG x M x W x K x B, prefill:
     T x B x W x M) and prints the worst relative L2 error per family;
  3. checks tests/inputs.py reproduces the reference generators bit for bit;
  4. stores the reference functions' outputs for a subset of the grid
     (``decode.npz``, ``recurrent.npz``, ``prefill.npz`` + ``manifest.json``);
  5. for ``chunk_nha`` (no CPU implementation exists in the reference) replays
     nha_fla/ops/nha/chunk.py:401-470 on the CPU from the reference's own shift
     helpers, ``fla.ops.gsa.naive.naive_recurrent_gsa`` and a masked softmax,
     differentiates it with autograd, checks the oracle against it and stores
     outputs and gradients (``training.npz``).
"""
from __future__ import annotations

import argparse
import json
import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
sys.path.insert(0, ROOT)

from oracle import nha_oracle as orc          # noqa: E402
from tests import inputs as gen               # noqa: E402


def rel(a, b):
    return orc.rel_l2(a, b)


def same_inputs(mine, ref):
    for key, x in ref.items():
        if torch.is_tensor(x):
            assert torch.equal(mine[key].float(), x.float()), f'input generator mismatch on {key}'


# ---------------------------------------------------------------------------
def grid_decode():
    seed = 2000
    for NG in (1, 4, 8):
        for M in (16, 64, 80):
            for W in (32, 64):
                for K in (64, 128):
                    for B in (1, 4):
                        yield dict(seed=seed, B=B, H=2, NG=NG, K=K, V=K, M=M, W=W)
                        seed += 1


def grid_recurrent():
    for c in grid_decode():
        c = dict(c)
        c['seed'] -= 1000
        yield c


def grid_prefill():
    seed = 3000
    for T in (63, 128, 257, 1000):
        for B in (1, 4):
            for W in (32, 64):
                for M in (16, 64):
                    yield dict(seed=seed, B=B, H=2, NG=4, K=64, V=64, M=M, W=W, T=T, with_state=(T == 128))
                    seed += 1


def name_of(prefix, c):
    parts = [prefix] + [f'{k.lower()}{int(v)}' for k, v in c.items() if k not in ('seed', 'H', 'V', 'with_state')]
    return '_'.join(parts)


def run_decode(vp, store):
    worst = 0.0
    out, man = {}, {}
    for c in grid_decode():
        args = (c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'])
        ref_in = vp.gen_decode_inputs(*args)
        mine = gen.decode_inputs(*args)
        same_inputs(mine, ref_in)
        ref = vp.ref_decode(ref_in)
        o, hk, hv, ps, pw = orc.decode_step(
            mine['q'], mine['k'], mine['v'], mine['g'], mine['sw_k_raw'], mine['vw'], mine['scale'],
            s=mine['s'], cos=mine['cos'], sin=mine['sin'], hk0=mine['hk0'], hv0=mine['hv0'])
        errs = [rel(o, ref['o']), rel(hk, ref['hkt']), rel(hv, ref['hvt']), rel(ps, ref['qv']), rel(pw, ref['swp'])]
        worst = max(worst, *errs)
        if store(c):
            n = name_of('dc', c)
            man[n] = dict(c, digest=gen.digest(mine))
            for key in ('o', 'hkt', 'hvt', 'qv', 'swp'):
                out[f'{n}/{key}'] = ref[key].float().numpy()
    return worst, out, man


def run_recurrent(vp, store):
    worst = 0.0
    out, man = {}, {}
    for c in grid_recurrent():
        args = (c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'])
        ref_in = vp.gen_recurrent_inputs(*args)
        mine = gen.recurrent_inputs(*args)
        same_inputs(mine, ref_in)
        ref = vp.ref_fused_recurrent(ref_in)
        o, pw, hk, hv = orc.recurrent_step(mine['q'], mine['k'], mine['v'], mine['sliding_window'], mine['s'],
                                           mine['g'], mine['scale'], mine['hk0'], mine['hv0'])
        errs = [rel(o, ref['o']), rel(pw, ref['swa_score']), rel(hk, ref['hkt']), rel(hv, ref['hvt'])]
        worst = max(worst, *errs)
        if store(c):
            n = name_of('fr', c)
            man[n] = dict(c, digest=gen.digest(mine))
            for key in ('o', 'swa_score', 'hkt', 'hvt'):
                out[f'{n}/{key}'] = ref[key].float().numpy()
    return worst, out, man


def run_prefill(vp, store):
    worst = 0.0
    out, man = {}, {}
    for c in grid_prefill():
        args = (c['seed'], c['B'], c['H'], c['NG'], c['K'], c['V'], c['M'], c['W'], c['T'], c['with_state'])
        ref_in = vp.gen_prefill_inputs(*args)
        mine = gen.prefill_inputs(*args)
        same_inputs(mine, ref_in)
        ref = vp.ref_prefill(ref_in)
        o, hk, hv = orc.prefill(mine['q'], mine['k'], mine['v'], mine['rotary_q'], mine['rotary_k'], mine['s'],
                                mine['g'], c['W'], mine['scale'], mine.get('hk0'), mine.get('hv0'))
        errs = [rel(o, ref['o']), rel(hk, ref['hkt']), rel(hv, ref['hvt'])]
        worst = max(worst, *errs)
        if store(c):
            n = name_of('pf', c)
            man[n] = dict(c, digest=gen.digest(mine))
            for key in ('o', 'hkt', 'hvt'):
                out[f'{n}/{key}'] = ref[key].float().numpy()
        print(f'  prefill {name_of("pf", c)} err {max(errs):.2e}', flush=True)
    return worst, out, man


# ---------------------------------------------------------------------------
def swa_masked(q, k, v, cu, scale, wl):
    """Causal sliding-window softmax attention per packed sequence with flash-attn's
    conventions (keys ``[t-wl, t]``), returning the output and the natural-log LSE."""
    outs, lses = [], []
    for a, b in zip(cu[:-1], cu[1:]):
        qq, kk, vv = q[a:b], k[a:b], v[a:b]
        T = b - a
        sc = torch.einsum('thk,whk->htw', qq, kk) * scale
        i = torch.arange(T)[:, None]
        j = torch.arange(T)[None, :]
        ok = (j <= i) & ((j >= i - wl) if wl >= 0 else torch.ones_like(j, dtype=torch.bool))
        sc = sc.masked_fill(~ok[None], float('-inf'))
        lses.append(torch.logsumexp(sc, dim=-1).transpose(0, 1))
        outs.append(torch.einsum('htw,whv->thv', torch.softmax(sc, dim=-1), vv))
    return torch.cat(outs), torch.cat(lses)


def gsa_lse(q, k, s, g, cu, scale, hk0):
    """logsumexp of the slot logits, the quantity chunk_gsa_fwd_with_lse adds
    (nha_fla/ops/nha/chunk_gsa.py:47); loop as in fla/ops/gsa/naive.py:47-53."""
    res = []
    for n, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        H, K, M = q.shape[1], q.shape[2], s.shape[-1]
        hk = torch.zeros(H, K, M, dtype=q.dtype) if hk0 is None else hk0[n].to(q.dtype)
        for t in range(a, b):
            hk = hk * g[t].exp()[:, None, :] + k[t][:, :, None] * s[t][:, None, :]
            res.append(torch.logsumexp(torch.einsum('hk,hkm->hm', q[t] * scale, hk), dim=-1))
    return torch.stack(res)


def replay_chunk_nha(ref_chunk, naive_gsa, x, cu, scale, wl, shift, hk0=None, hv0=None):
    """CPU replay of ChunkNativeHybridAttentionFunction.forward (nha_fla/ops/nha/chunk.py:401-470)
    on flat ``[Ttot,H,*]`` fp64 tensors; autograd supplies the backward."""
    q_swa, k_swa, q_gsa, k_gsa, v, s, g = x
    cu_t = torch.tensor(cu, dtype=torch.int32)
    if shift > 0:
        k_g = ref_chunk._packed_shift_right(k_gsa, cu_t, shift)
        v_g = ref_chunk._packed_shift_right(v, cu_t, shift)
        s_g = ref_chunk._packed_shift_right(s, cu_t, shift)
        g_g = ref_chunk._packed_shift_right(g, cu_t, shift)
    else:
        k_g, v_g, s_g, g_g = k_gsa, v, s, g
    out_swa, lse_swa = swa_masked(q_swa, k_swa, v, cu, scale, wl)
    ovs, hks, hvs = [], [], []
    for n, (a, b) in enumerate(zip(cu[:-1], cu[1:])):
        init = None if hk0 is None else (hk0[n][None].double(), hv0[n][None].double())
        ov, (hkt, hvt) = naive_gsa_f64(naive_gsa, q_gsa[a:b][None], k_g[a:b][None], v_g[a:b][None], s_g[a:b][None],
                                       g_g[a:b][None], scale, init)
        ovs.append(ov[0]); hks.append(hkt[0]); hvs.append(hvt[0])
    out_gsa = torch.cat(ovs)
    lse_gsa = gsa_lse(q_gsa, k_g, s_g, g_g, cu, scale, hk0)
    lse_max = torch.maximum(lse_swa, lse_gsa)
    w_swa = torch.exp(lse_swa - lse_max)
    w_gsa = torch.exp(lse_gsa - lse_max)
    den = w_swa + w_gsa
    out = (w_swa.unsqueeze(-1) * out_swa + w_gsa.unsqueeze(-1) * out_gsa) / den.unsqueeze(-1)
    return out, lse_swa, lse_gsa, torch.stack(hks), torch.stack(hvs)


def naive_gsa_f64(naive_gsa, q, k, v, s, g, scale, init):
    """fla's naive recurrent GSA with its internal ``.float()`` casts lifted to fp64."""
    orig_float = torch.Tensor.float
    orig_zeros = torch.zeros

    def zeros64(*a, **kw):
        if kw.get('dtype') is torch.float:
            kw['dtype'] = torch.float64
        return orig_zeros(*a, **kw)

    torch.Tensor.float = lambda self: self.double()
    torch.zeros = zeros64
    try:
        return naive_gsa(q, k, v, s, g, scale=scale, initial_state=init, output_final_state=True)
    finally:
        torch.Tensor.float = orig_float
        torch.zeros = orig_zeros


TRAIN_CASES = [
    # name, seed, B, T, H, K, V, M, cu (None = batched), window_left, shift, with_state
    # the reference's training shapes (scripts/verify_opt_parity.py:539-544) with fewer heads,
    # plus the overlapping (wl=W, shift=0) and disjoint (wl=W-1, shift=W) conventions
    ('tr_b2_t128_h2_k64_m32_wl63_sh0', 4000, 2, 128, 2, 64, 64, 32, None, 63, 0, False),
    ('tr_vl_t300_h1_k64_m64_wl63_sh0', 4001, 1, 300, 1, 64, 64, 64, [0, 100, 300], 63, 0, False),
    ('tr_b1_t96_h1_k128_m16_wl63_sh0', 4002, 1, 96, 1, 128, 128, 16, None, 63, 0, False),
    ('tr_b1_t160_h2_k64_m32_wl64_sh0', 4100, 1, 160, 2, 64, 64, 32, None, 64, 0, False),
    ('tr_b1_t200_h1_k64_m64_wl31_sh32', 4101, 1, 200, 1, 64, 64, 64, None, 31, 32, True),
    ('tr_vl_t260_h1_k64_m16_wl63_sh64', 4102, 1, 260, 1, 64, 64, 16, [0, 50, 51, 260], 63, 64, False),
]


def run_training(ref_chunk, naive_gsa):
    worst_f, worst_b = 0.0, 0.0
    out, man = {}, {}
    names = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')
    for (name, seed, B, T, H, K, V, M, cu, wl, shift, with_state) in TRAIN_CASES:
        d = gen.training_inputs(seed, B, T, H, K, V, M)
        flat = lambda t: t.reshape(B * T, *t.shape[2:])
        cu_l = cu if cu is not None else [i * T for i in range(B + 1)]
        N = len(cu_l) - 1
        scale = K ** -0.5
        hk0 = hv0 = None
        if with_state:
            torch.manual_seed(seed + 50000)
            hk0 = (torch.randn(N, H, K, M) * 0.5).float()
            hv0 = (torch.randn(N, H, M, V) * 0.5).float()
        torch.manual_seed(seed + 70000)
        dlse = (torch.randn(B * T, H) * 0.1).double()
        do = flat(d['do']).double()

        def leaves():
            xs = [flat(d[n]).double().clone().requires_grad_(True) for n in names]
            st = [None, None] if hk0 is None else [hk0.double().clone().requires_grad_(True),
                                                    hv0.double().clone().requires_grad_(True)]
            return xs, st

        # reference replay
        xs, st = leaves()
        o_r, ls_r, lg_r, hk_r, hv_r = replay_chunk_nha(ref_chunk, naive_gsa, xs, cu_l, scale, wl, shift, st[0], st[1])
        ((o_r * do).sum() + (lg_r * dlse).sum()).backward()
        g_r = [x.grad for x in xs] + [t.grad for t in st if t is not None]
        # oracle
        ys, st2 = leaves()
        o_o, ls_o, lg_o, hk_o, hv_o = orc.nha_varlen(ys[2], ys[0], ys[3], ys[1], ys[4], ys[5], ys[6], cu_l, scale,
                                                      wl, shift, st2[0], st2[1])
        ((o_o * do).sum() + (lg_o * dlse).sum()).backward()
        g_o = [y.grad for y in ys] + [t.grad for t in st2 if t is not None]
        ef = max(rel(o_o, o_r), rel(ls_o, ls_r), rel(lg_o, lg_r), rel(hk_o, hk_r), rel(hv_o, hv_r))
        eb = max(rel(a, b) for a, b in zip(g_o, g_r))
        worst_f, worst_b = max(worst_f, ef), max(worst_b, eb)
        print(f'  training {name}: fwd err {ef:.2e} grad err {eb:.2e}', flush=True)
        man[name] = dict(seed=seed, B=B, T=T, H=H, K=K, V=V, M=M, cu=cu, window_left=wl, shift=shift,
                         with_state=with_state, digest=gen.digest(d))
        out[f'{name}/o'] = o_r.detach().float().numpy()
        out[f'{name}/lse_swa'] = ls_r.detach().float().numpy()
        out[f'{name}/lse_gsa'] = lg_r.detach().float().numpy()
        out[f'{name}/hkt'] = hk_r.detach().float().numpy()
        out[f'{name}/hvt'] = hv_r.detach().float().numpy()
        for n, gr in zip(names + (('hk0', 'hv0') if with_state else ()), g_r):
            out[f'{name}/grad_{n}'] = gr.float().numpy()
    return worst_f, worst_b, out, man


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument('--reference', required=True, help='path of a checkout of the reference project')
    ap.add_argument('--skip-grids', action='store_true')
    args = ap.parse_args()
    sys.path.insert(0, os.path.join(args.reference, 'scripts'))
    sys.path.insert(0, args.reference)
    import verify_opt_parity as vp
    vp.DEVICE = 'cpu'
    torch.set_num_threads(os.cpu_count())

    manifest, report = {}, {}
    small = lambda c: (c['B'] == 1 and c['K'] == 64 and c['W'] == 32) or (c['NG'] == 4 and c['M'] == 80 and c['W'] == 64 and c['B'] == 1)
    w, out, man = run_decode(vp, small)
    report['decode_grid_worst_rel_l2'] = w
    np.savez(os.path.join(HERE, 'decode.npz'), **out); manifest['decode'] = man
    print(f'decode grid: oracle vs ref_decode worst rel-L2 {w:.3e} ({len(man)} cases stored)')
    w, out, man = run_recurrent(vp, small)
    report['recurrent_grid_worst_rel_l2'] = w
    np.savez(os.path.join(HERE, 'recurrent.npz'), **out); manifest['recurrent'] = man
    print(f'recurrent grid: oracle vs ref_fused_recurrent worst rel-L2 {w:.3e} ({len(man)} cases stored)')
    keep_pf = lambda c: (c['B'] == 1 and c['T'] <= 128 and c['W'] + c['M'] in (48, 128)) or (c['B'] == 1 and c['T'] == 257 and c['W'] == 64 and c['M'] == 16)
    w, out, man = run_prefill(vp, keep_pf)
    report['prefill_grid_worst_rel_l2'] = w
    np.savez(os.path.join(HERE, 'prefill.npz'), **out); manifest['prefill'] = man
    print(f'prefill grid: oracle vs ref_prefill worst rel-L2 {w:.3e} ({len(man)} cases stored)')

    import nha_fla.ops.nha.chunk as ref_chunk
    from fla.ops.gsa.naive import naive_recurrent_gsa
    wf, wb, out, man = run_training(ref_chunk, naive_recurrent_gsa)
    report['training_replay_worst_fwd'] = wf
    report['training_replay_worst_grad'] = wb
    np.savez(os.path.join(HERE, 'training.npz'), **out); manifest['training'] = man
    print(f'training replay: oracle vs chunk.py replay worst fwd {wf:.3e} grad {wb:.3e}')
    manifest['_report'] = report
    manifest['_torch'] = torch.__version__
    with open(os.path.join(HERE, 'manifest.json'), 'w') as f:
        json.dump(manifest, f, indent=1)


if __name__ == '__main__':
    main()
