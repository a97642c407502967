"""GPU: the benchmark configurations at FULL size, checked through properties that need no oracle run.

The fp64 oracle takes minutes to hours at these sizes, so the checks are size independent:
  * two independent implementations agree: the tcgen05 kernels against the general (wmma) kernels, which
    share no device code beyond the state pass (NHA_B200_NO_UMMA=1 forces the latter);
  * sequences do not interact: a sequence gives bit-identical results inside a batch / a packed buffer and
    on its own;
  * causality and the state hand-off: the long prefill cut in two, with the first half's final state as the
    second half's initial state and the last W tokens as its halo, reproduces the one-piece run.
Inputs follow the value distributions of the workloads (q/k/v ~ N(0,1)/sqrt(D), gates logsigmoid(N(0,1))).
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu
NAMES = ('q_swa', 'k_swa', 'q_gsa', 'k_gsa', 'v', 's', 'g')


def _inputs(seed, Ttot, HQ, H, D, M):
    g = torch.Generator(device='cuda').manual_seed(seed)
    r = lambda *s: torch.randn(*s, generator=g, device='cuda')
    x = {
        'q_swa': (r(Ttot, HQ, D) * D ** -0.5).bfloat16(), 'k_swa': (r(Ttot, H, D) * D ** -0.5).bfloat16(),
        'q_gsa': (r(Ttot, HQ, D) * D ** -0.5).bfloat16(), 'k_gsa': (r(Ttot, H, D) * D ** -0.5).bfloat16(),
        'v': (r(Ttot, H, D) * D ** -0.5).bfloat16(),
    }
    x['g'] = F.logsigmoid(r(Ttot, H, M)).bfloat16()
    x['s'] = (1 - x['g'].float().exp()).bfloat16()
    do = r(Ttot, HQ, D).bfloat16()
    return x, do


def _run(x, do, cu, max_len, wl, shift, rows=None):
    """chunk_nha forward + backward on packed inputs (optionally only the rows `rows` = (start, stop))."""
    from nha_b200 import chunk_nha
    sl = slice(None) if rows is None else slice(*rows)
    leaves = {n: x[n][sl].detach().clone().requires_grad_(True) for n in NAMES}
    o, ls, lg = chunk_nha(leaves['q_swa'][None], leaves['k_swa'][None], leaves['q_gsa'][None], leaves['k_gsa'][None],
                          leaves['v'][None], leaves['s'][None], leaves['g'][None], cu_seqlens=cu, max_seqlen=max_len,
                          scale=x['q_swa'].shape[-1] ** -0.5, window_size_left=wl, window_size_right=0,
                          gsa_kv_shift=shift)
    o.backward(do[sl][None])
    torch.cuda.synchronize()
    return dict(o=o[0], lse_swa=ls[0], lse_gsa=lg[0], **{'d' + n: leaves[n].grad for n in NAMES})


def _rel(a, b):
    a, b = a.detach().double(), b.detach().double()
    return float((a - b).norm() / b.norm().clamp_min(1e-30))


def test_headline_full_size_two_implementations_and_batch_independence(monkeypatch):
    """B16 T2048 H16 D64 M64 W64, forward + backward."""
    B, T, H, D, M, W = 16, 2048, 16, 64, 64, 64
    x, do = _inputs(11, B * T, H, H, D, M)
    cu = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device='cuda')
    monkeypatch.setenv('NHA_B200_NO_UMMA', '0')
    fast = _run(x, do, cu, T, W, 0)
    monkeypatch.setenv('NHA_B200_NO_UMMA', '1')
    general = _run(x, do, cu, T, W, 0)
    monkeypatch.setenv('NHA_B200_NO_UMMA', '0')
    for name in fast:
        assert torch.isfinite(fast[name].float()).all(), name
        tol = 2e-2 if name in ('o', 'lse_swa', 'lse_gsa') else 3e-2
        assert _rel(fast[name], general[name]) <= tol, (name, _rel(fast[name], general[name]))
    # sequence 5 on its own: the same kernels on the same data, bit for bit
    one = _run(x, do, torch.tensor([0, T], dtype=torch.int32, device='cuda'), T, W, 0, rows=(5 * T, 6 * T))
    for name in one:
        assert torch.equal(one[name], fast[name][5 * T:6 * T]), name


def test_varlen_full_size_sequences_do_not_interact():
    """32768 packed tokens, lengths uniform[128, 8192], per-sequence windows from {32, ..., 512}; H16 D64 M64."""
    H, D, M, total = 16, 64, 64, 32768
    g = torch.Generator().manual_seed(3)
    lens = []
    while sum(lens) < total:
        lens.append(int(torch.randint(128, 8193, (1,), generator=g)))
    lens[-1] -= sum(lens) - total
    if lens[-1] < 1:
        lens[-2] += lens[-1] - 1
        lens[-1] = 1
    assert sum(lens) == total and min(lens) >= 1
    wins = [int([32, 64, 128, 256, 512][int(torch.randint(0, 5, (1,), generator=g))]) for _ in lens]
    cu_l = [0]
    for L in lens:
        cu_l.append(cu_l[-1] + L)
    x, do = _inputs(12, total, H, H, D, M)
    cu = torch.tensor(cu_l, dtype=torch.int32, device='cuda')
    wl = torch.tensor(wins, dtype=torch.int32, device='cuda')
    sh = torch.zeros(len(lens), dtype=torch.int32, device='cuda')
    packed = _run(x, do, cu, max(lens), wl, sh)
    for name in packed:
        assert torch.isfinite(packed[name].float()).all(), name
    for n in (0, len(lens) // 2, len(lens) - 1):
        a, b = cu_l[n], cu_l[n + 1]
        one = _run(x, do, torch.tensor([0, b - a], dtype=torch.int32, device='cuda'), b - a, wins[n], 0, rows=(a, b))
        for name in one:
            assert torch.equal(one[name], packed[name][a:b]), (n, name)


def test_long_prefill_full_size_cut_in_two(monkeypatch):
    """B1 T131072 HQ32 H8 D128 M64 W512 (forward): one piece against two pieces with state and halo hand-off,
    with the window tiles fetched by TMA and by the zero-filling fallback."""
    from nha_b200 import fused_chunk_nha_prefill
    T, HQ, H, D, M, W = 131072, 32, 8, 128, 64, 512
    g = torch.Generator(device='cuda').manual_seed(13)
    r = lambda *s: torch.randn(*s, generator=g, device='cuda')
    q, rq = (r(1, T, HQ, D) * D ** -0.5).bfloat16(), (r(1, T, HQ, D) * D ** -0.5).bfloat16()
    k, rk = (r(1, T, H, D) * D ** -0.5).bfloat16(), (r(1, T, H, D) * D ** -0.5).bfloat16()
    v = (r(1, T, H, D) * D ** -0.5).bfloat16()
    gg = (F.logsigmoid(r(1, T, H, M)) / 8).bfloat16()
    ss = (1 - gg.float().exp()).bfloat16()
    full = {}
    for tma in ('0', '1'):
        monkeypatch.setenv('NHA_B200_NO_TMA', tma)
        o, (hk, hv) = fused_chunk_nha_prefill(q=q, k=k, v=v, rotary_q=rq, rotary_k=rk, s=ss, g=gg, window_size=W,
                                              output_final_state=True)
        torch.cuda.synchronize()
        assert torch.isfinite(o.float()).all()
        full[tma] = (o, hk, hv)
    assert _rel(full['0'][0], full['1'][0]) <= 1e-3         # same arithmetic, different copy engines
    monkeypatch.setenv('NHA_B200_NO_TMA', '0')
    o, hk, hv = full['0']
    # first half alone: causal, so identical to the first half of the one-piece run
    cut = T // 2
    a = lambda t, lo, hi: t[:, lo:hi].contiguous()
    o1, (hk1, hv1) = fused_chunk_nha_prefill(q=a(q, 0, cut), k=a(k, 0, cut), v=a(v, 0, cut), rotary_q=a(rq, 0, cut),
                                             rotary_k=a(rk, 0, cut), s=a(ss, 0, cut), g=a(gg, 0, cut), window_size=W,
                                             output_final_state=True)
    assert torch.equal(o1, o[:, :cut])
    # second half as the sequence-parallel composition runs it: halo of W tokens in front (its outputs dropped;
    # with the shift by W nothing enters the slot memory during the halo), start state = the first half's end state
    lo = cut - W
    o2, (hk2, hv2) = fused_chunk_nha_prefill(q=a(q, lo, T), k=a(k, lo, T), v=a(v, lo, T), rotary_q=a(rq, lo, T),
                                             rotary_k=a(rk, lo, T), s=a(ss, lo, T), g=a(gg, lo, T), window_size=W,
                                             initial_state=(hk1, hv1), output_final_state=True)
    assert _rel(o2[:, W:], o[:, cut:]) <= 5e-3
    assert _rel(hk2, hk) <= 5e-3 and _rel(hv2, hv) <= 5e-3
