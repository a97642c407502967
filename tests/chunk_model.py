"""Host-side model of the chunked arithmetic the CUDA kernels use (TEST INFRASTRUCTURE).

The kernels do not run the token-by-token recurrence of the oracle: they use a
chunked reformulation (chunk = 64 tokens) with a state pass, per-chunk
factorised decays around a per-slot reference exponent, a joint softmax over
[slots | window keys], and a backward made of a chunk-parallel pass plus a
reverse march.  This file states that reformulation in plain fp64 PyTorch, one
sequence and one kv head at a time, so that CPU tests can prove it equal to the
oracle (forward and gradients) independently of any CUDA code.  The names
follow the kernels' (state pass, output pass, backward pass 1, reverse march).
"""
from __future__ import annotations

import torch

C = 64          # chunk length
CLAMP = 75.0    # exponent clamp of the factorised decays


def _shifted(x, shift):
    y = torch.zeros_like(x)
    if x.shape[0] > shift:
        y[shift:] = x[:x.shape[0] - shift]
    return y


BC = 16         # row block inside a chunk: one decay reference per (row block, slot)


def _chunk_decays(gp):
    """gp [c,M] shifted log gates of one chunk -> (G, Gend, be) with G the inclusive cumsum."""
    G = gp.cumsum(0)
    Gend = G[-1]
    be = (Gend - G).exp()
    return G, Gend, be


def _block_refs(G, i0, i1):
    """Decay factors of row block [i0,i1): rows t use a[t] = exp(G_t - R), columns i < i1 use
    b[i] = exp(R - G_i), R = midpoint of the block's own cumulative-gate range (per slot).
    Every valid pair (i <= t) has a*b = exp(G_t - G_i) <= 1 and each factor stays inside
    exp(+-CLAMP) as long as one block decays by less than 2*CLAMP nats per slot."""
    Gn = G[i0 - 1] if i0 > 0 else torch.zeros_like(G[0])
    R = 0.5 * (Gn + G[i1 - 1])
    a = (G[i0:i1] - R).clamp(-CLAMP, CLAMP).exp()
    b = (R - G[:i1]).clamp(-CLAMP, CLAMP).exp()
    return a, b


def state_pass(kp, vp, sp, gp, hk0, hv0):
    """Chunk-start states of one (sequence, kv head): lists hk[c] [K,M], hv[c] [M,V], plus final."""
    T = kp.shape[0]
    hk, hv = hk0.clone(), hv0.clone()
    hks, hvs = [], []
    for c0 in range(0, T, C):
        hks.append(hk); hvs.append(hv)
        sl = slice(c0, min(T, c0 + C))
        G, Gend, be = _chunk_decays(gp[sl])
        sbe = sp[sl] * be
        hk = hk * Gend.exp()[None, :] + kp[sl].T @ sbe
        hv = hv * Gend.exp()[:, None] + sbe.T @ vp[sl]
    return hks, hvs, hk, hv


def _window(c0, c1, wl):
    w0 = 0 if wl < 0 else max(0, c0 - wl)
    rows = torch.arange(c0, c1)[:, None]
    cols = torch.arange(w0, c1)[None, :]
    mask = (cols <= rows) & ((cols >= rows - wl) if wl >= 0 else True)
    return w0, mask


def _slot_logits(q, kp_c, sp_c, G, Hk, scale):
    """ok [n,M] of one chunk and query head, row block by row block, plus the per-block
    (a, SB = s' * b, tril A) the other passes reuse."""
    n = q.shape[0]
    ok = scale * G.exp() * (q @ Hk)
    blocks = []
    for i0 in range(0, n, BC):
        i1 = min(n, i0 + BC)
        a, b = _block_refs(G, i0, i1)
        SB = sp_c[:i1] * b
        A = q[i0:i1] @ kp_c[:i1].T
        A = A * (torch.arange(i1)[None, :] <= torch.arange(i0, i1)[:, None])
        ok[i0:i1] += scale * a * (A @ SB)
        blocks.append((i0, i1, a, b, SB, A))
    return ok, blocks


def forward(q_gsa, q_swa, k_gsa, k_swa, v, s, g, scale, wl, shift, hk0=None, hv0=None):
    """One sequence, one kv head: q_* [T,NG,K]; k_*, v, s, g [T,*].  Returns o, lse_swa, lse_gsa,
    hkt, hvt and the per-chunk states (what the forward saves for the backward)."""
    dd = torch.float64
    q_gsa, q_swa, k_gsa, k_swa, v, s, g = (x.to(dd) for x in (q_gsa, q_swa, k_gsa, k_swa, v, s, g))
    T, NG, K = q_gsa.shape
    M, V = s.shape[-1], v.shape[-1]
    hk0 = torch.zeros(K, M, dtype=dd) if hk0 is None else hk0.to(dd)
    hv0 = torch.zeros(M, V, dtype=dd) if hv0 is None else hv0.to(dd)
    kp, vp, sp, gp = (_shifted(x, shift) for x in (k_gsa, v, s, g))
    hks, hvs, hkt, hvt = state_pass(kp, vp, sp, gp, hk0, hv0)
    o = torch.zeros(T, NG, V, dtype=dd)
    lse_s = torch.zeros(T, NG, dtype=dd)
    lse_g = torch.zeros(T, NG, dtype=dd)
    for ci, c0 in enumerate(range(0, T, C)):
        c1 = min(T, c0 + C)
        sl = slice(c0, c1)
        G, Gend, be = _chunk_decays(gp[sl])
        w0, wmask = _window(c0, c1, wl)
        for h in range(NG):
            ok, blocks = _slot_logits(q_gsa[sl, h], kp[sl], sp[sl], G, hks[ci], scale)
            sw = scale * (q_swa[sl, h] @ k_swa[w0:c1].T)
            sw = sw.masked_fill(~wmask, float('-inf'))
            p = torch.softmax(torch.cat([ok, sw], dim=1), dim=1)
            ps = p[:, :M]
            oc = (ps * G.exp()) @ hvs[ci] + p[:, M:] @ v[w0:c1]
            for (i0, i1, a, b, SB, A) in blocks:
                Bv = (ps[i0:i1] * a) @ SB.T
                Bv = Bv * (torch.arange(i1)[None, :] <= torch.arange(i0, i1)[:, None])
                oc[i0:i1] += Bv @ vp[sl][:i1]
            o[sl, h] = oc
            lse_g[sl, h] = torch.logsumexp(ok, dim=1)
            lse_s[sl, h] = torch.logsumexp(sw, dim=1)
    return o, lse_s, lse_g, hkt, hvt, (hks, hvs)


def backward(q_gsa, q_swa, k_gsa, k_swa, v, s, g, scale, wl, shift, saved, o, lse_s, lse_g, do, dlse_g=None,
             dhkt=None, dhvt=None, hkt=None, hvt=None):
    """Backward pass 1 (chunk-parallel) followed by the reverse march.  Returns grads for
    q_swa, k_swa, q_gsa, k_gsa, v, s, g, hk0, hv0."""
    dd = torch.float64
    q_gsa, q_swa, k_gsa, k_swa, v, s, g, o, do = (x.to(dd) for x in (q_gsa, q_swa, k_gsa, k_swa, v, s, g, o, do))
    hks, hvs = saved
    T, NG, K = q_gsa.shape
    M, V = s.shape[-1], v.shape[-1]
    kp, vp, sp, gp = (_shifted(x, shift) for x in (k_gsa, v, s, g))
    L = torch.logaddexp(lse_s, lse_g)
    dq_swa = torch.zeros_like(q_swa); dq_gsa = torch.zeros_like(q_gsa)
    dk_swa = torch.zeros_like(k_swa); dv = torch.zeros_like(v)
    dkp = torch.zeros_like(kp); dvp = torch.zeros_like(vp); dsp = torch.zeros_like(sp)
    dgA = torch.zeros_like(gp)
    dzg_all = torch.zeros(T, NG, M, dtype=dd); pg_all = torch.zeros(T, NG, M, dtype=dd)
    # ---- pass 1: everything that stays inside a chunk, plus the window gradients
    for ci, c0 in enumerate(range(0, T, C)):
        c1 = min(T, c0 + C)
        sl = slice(c0, c1)
        G, Gend, be = _chunk_decays(gp[sl])
        eG = G.exp()
        Hk, Hv = hks[ci], hvs[ci]
        w0, wmask = _window(c0, c1, wl)
        kc, vc, sc = kp[sl], vp[sl], sp[sl]
        for h in range(NG):
            q, qs, d_o = q_gsa[sl, h], q_swa[sl, h], do[sl, h]
            ok, blocks = _slot_logits(q, kc, sc, G, Hk, scale)
            sw = (scale * (qs @ k_swa[w0:c1].T)).masked_fill(~wmask, float('-inf'))
            Lr = L[sl, h][:, None]
            ps, pw = (ok - Lr).exp(), (sw - Lr).exp()
            dps = eG * (d_o @ Hv.T)
            Avs = []
            for (i0, i1, a, b, SB, A) in blocks:
                Av = d_o[i0:i1] @ vc[:i1].T
                Av = Av * (torch.arange(i1)[None, :] <= torch.arange(i0, i1)[:, None])
                dps[i0:i1] += a * (Av @ SB)
                Avs.append(Av)
            dpw = d_o @ v[w0:c1].T
            delta = (d_o * o[sl, h]).sum(1, keepdim=True)
            dzs = ps * (dps - delta)
            if dlse_g is not None:
                dzs = dzs + dlse_g[sl, h][:, None] * (ok - lse_g[sl, h][:, None]).exp()
            dzw = pw * (dpw - delta)
            dq_swa[sl, h] = scale * dzw @ k_swa[w0:c1]
            dk_swa[w0:c1] += scale * dzw.T @ qs
            dv[w0:c1] += pw.T @ d_o
            dqg = scale * ((dzs * eG) @ Hk.T)
            for (i0, i1, a, b, SB, A), Av in zip(blocks, Avs):
                tri = (torch.arange(i1)[None, :] <= torch.arange(i0, i1)[:, None])
                dza, pa = dzs[i0:i1] * a, ps[i0:i1] * a
                E = (dza @ SB.T) * tri
                Bv = (pa @ SB.T) * tri
                dqg[i0:i1] += scale * E @ kc[:i1]
                dkp[c0:c0 + i1] += scale * E.T @ q[i0:i1]
                dvp[c0:c0 + i1] += Bv.T @ d_o[i0:i1]
                dsp[c0:c0 + i1] += b * (scale * A.T @ dza + Av.T @ pa)
            dq_gsa[sl, h] = dqg
            dgA[sl] += ok * dzs + ps * dps
            dzg_all[sl, h], pg_all[sl, h] = dzs * eG, ps * eG
    # ---- reverse march: inter-chunk terms, gate gradient, state gradients
    DK = torch.zeros(K, M, dtype=dd) if dhkt is None else dhkt.to(dd).clone()
    DV = torch.zeros(M, V, dtype=dd) if dhvt is None else dhvt.to(dd).clone()
    cg = torch.zeros(M, dtype=dd)
    if dhkt is not None:
        cg = cg + (dhkt.to(dd) * hkt.to(dd)).sum(0) + (dhvt.to(dd) * hvt.to(dd)).sum(1)
    dgp = torch.zeros_like(gp)
    starts = list(range(0, T, C))
    for ci in reversed(range(len(starts))):
        c0 = starts[ci]
        c1 = min(T, c0 + C)
        sl = slice(c0, c1)
        G, Gend, be = _chunk_decays(gp[sl])
        if ci < len(starts) - 1:
            # carry of all later chunks rebuilt from the state at this chunk's end and its gradient
            # (equal to the running sum of dgraw over the later tokens, without its rounding noise)
            cg = (DK * hks[ci + 1]).sum(0) + (DV * hvs[ci + 1]).sum(1)
        sbe = sp[sl] * be
        dkp[sl] += sbe @ DK.T
        dvp[sl] += sbe @ DV
        dsp[sl] += be * (kp[sl] @ DK + vp[sl] @ DV.T)
        dgraw = dgA[sl] - sp[sl] * dsp[sl]
        rc = dgraw.flip(0).cumsum(0).flip(0)
        dgp[sl] = rc + cg[None, :]
        cg = cg + dgraw.sum(0)
        DK = DK * Gend.exp()[None, :]
        DV = DV * Gend.exp()[:, None]
        for h in range(NG):
            DK = DK + scale * q_gsa[sl, h].T @ dzg_all[sl, h]
            DV = DV + pg_all[sl, h].T @ do[sl, h]

    def unshift(x):
        y = torch.zeros_like(x)
        if T > shift:
            y[:T - shift] = x[shift:]
        return y

    return dq_swa, dk_swa, dq_gsa, unshift(dkp), dv + unshift(dvp), unshift(dsp), unshift(dgp), DK, DV
