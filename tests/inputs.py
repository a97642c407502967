"""Seeded synthetic inputs for the NHA parity tests.

The generators reproduce, draw for draw, the streams of the reference's
procedural fixtures (scripts/verify_opt_parity.py:198-256 and :535-562): CPU
``torch.randn`` in fp32 after ``torch.manual_seed(seed)``, scaled, then cast to
bf16.  ``tests/golden/make_golden.py`` asserts bit-equality with the
reference's own generators before it writes fixtures, so a fixture only has to
store the seed, the shape and the expected outputs.
"""
from __future__ import annotations

import hashlib

import torch
import torch.nn.functional as F

BF16 = torch.bfloat16


def _draw(*shape, dtype=BF16, scale=1.0):
    return (torch.randn(*shape, dtype=torch.float32) * scale).to(dtype)


def recurrent_inputs(seed, B, H, NG, K, V, M, W):
    """Inputs of ``fused_recurrent_nha`` (reference generator :202-216)."""
    torch.manual_seed(seed)
    HQ = H * NG
    d = {
        'q': _draw(B, 1, HQ, K),
        'k': _draw(B, 1, H, K),
        'v': _draw(B, 1, H, V),
        'sliding_window': _draw(B, 1, HQ, W),
        'hk0': _draw(B, H, K, M, dtype=torch.float32, scale=0.5),
        'hv0': _draw(B, H, M, V, dtype=torch.float32, scale=0.5),
    }
    d['g'] = F.logsigmoid(torch.randn(B, 1, H, M)).to(BF16) / 8.0
    d['s'] = (1 - d['g'].exp()).to(BF16)
    d['scale'] = K ** -0.5
    return d


def rope_tables(W, K, first_pos=100, theta=10000.0):
    inv_freq = 1.0 / (theta ** (torch.arange(0, K, 2, dtype=torch.float32) / K))
    pos = torch.arange(first_pos, first_pos + W, dtype=torch.float32)
    freqs = torch.outer(pos, inv_freq)
    emb = torch.cat([freqs, freqs], dim=-1)
    return emb.cos().to(BF16)[None], emb.sin().to(BF16)[None]


def eager_rope(x, cos, sin):
    x1, x2 = x.chunk(2, dim=-1)
    rot = torch.cat([-x2, x1], dim=-1)
    return x * cos.unsqueeze(-2) + rot * sin.unsqueeze(-2)


def decode_inputs(seed, B, H, NG, K, V, M, W):
    """Inputs of ``fused_recurrent_nha_decode`` (reference generator :219-236)."""
    d = recurrent_inputs(seed, B, H, NG, K, V, M, W)
    d['sw_k_raw'] = _draw(B, W, H, K)
    d['vw'] = _draw(B, W, H, V)
    d['cos'], d['sin'] = rope_tables(W, K)
    d['sq'] = eager_rope(d['q'], d['cos'][:, -1:], d['sin'][:, -1:])
    d['sk'] = eager_rope(d['sw_k_raw'], d['cos'], d['sin'])
    return d


def prefill_inputs(seed, B, H, NG, K, V, M, W, T, with_state):
    """Inputs of ``fused_chunk_nha_prefill`` (reference generator :239-256)."""
    torch.manual_seed(seed)
    HQ = H * NG
    d = {
        'q': _draw(B, T, HQ, K),
        'k': _draw(B, T, H, K),
        'v': _draw(B, T, H, V),
        'rotary_q': _draw(B, T, HQ, K),
        'rotary_k': _draw(B, T, H, K),
        'W': W,
        'scale': K ** -0.5,
    }
    d['g'] = F.logsigmoid(torch.randn(B, T, H, M)).to(BF16) / 8.0
    d['s'] = (1 - d['g'].exp()).to(BF16)
    if with_state:
        d['hk0'] = _draw(B, H, K, M, dtype=torch.float32, scale=0.5)
        d['hv0'] = _draw(B, H, M, V, dtype=torch.float32, scale=0.5)
    return d


def training_inputs(seed, B, T, H, K, V, M, gate_div=8.0, val_scale=1.0):
    """Inputs of ``chunk_nha`` fwd+bwd in the order of the reference's training dump (:549-559)."""
    torch.manual_seed(seed)
    d = {
        'q_swa': _draw(B, T, H, K, scale=val_scale),
        'k_swa': _draw(B, T, H, K, scale=val_scale),
        'q_gsa': _draw(B, T, H, K, scale=val_scale),
        'k_gsa': _draw(B, T, H, K, scale=val_scale),
        'v': _draw(B, T, H, V, scale=val_scale),
        's': _draw(B, T, H, M),
    }
    d['g'] = F.logsigmoid(torch.randn(B, T, H, M)).to(BF16) / gate_div
    d['do'] = _draw(B, T, H, V, dtype=torch.float32)
    return d


def layer_inputs(seed, B, T, HQ, H, K, V, M, gate_div=1.0, val_scale=None, dtype=BF16):
    """Inputs with the value distributions of the headline workloads: q/k/v ~ N(0,1)*val_scale
    (default 1/sqrt(K)), gate logits ~ N(0,1) through logsigmoid, ``s = 1 - exp(g)``."""
    torch.manual_seed(seed)
    vs = K ** -0.5 if val_scale is None else val_scale
    d = {
        'q_swa': _draw(B, T, HQ, K, scale=vs, dtype=dtype),
        'k_swa': _draw(B, T, H, K, scale=vs, dtype=dtype),
        'q_gsa': _draw(B, T, HQ, K, scale=vs, dtype=dtype),
        'k_gsa': _draw(B, T, H, K, scale=vs, dtype=dtype),
        'v': _draw(B, T, H, V, scale=vs, dtype=dtype),
    }
    d['g'] = (F.logsigmoid(torch.randn(B, T, H, M)) / gate_div).to(dtype)
    d['s'] = (1 - d['g'].float().exp()).to(dtype)
    d['do'] = _draw(B, T, HQ, V, dtype=dtype)
    return d


def digest(d) -> str:
    """Order-independent checksum of the tensors of an input dict (fp32 bytes)."""
    h = hashlib.sha256()
    for name in sorted(d):
        x = d[name]
        if torch.is_tensor(x):
            h.update(name.encode())
            h.update(x.detach().float().contiguous().numpy().tobytes())
    return h.hexdigest()[:16]
