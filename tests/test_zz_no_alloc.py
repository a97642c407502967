"""GPU: the allocation-free state pass (scratch inside the library) against the regular one.

For hosts that cannot allocate device memory the library offers nha_chunk_state_pass_static,
which takes its per-chunk scratch from a fixed array in the library's own device image.  This
test drives it through the C ABI on a problem of several chunks per sequence, twice in a row with different
inputs (the second call finds the first call's leftovers in the shared array), and requires
the chunk-start and final states to be identical to those of nha_chunk_state_pass with a
caller-provided workspace.  It also checks that an oversized problem is refused.  The file
name makes pytest collect it last, so a failure here cannot hide one elsewhere.
"""
import ctypes

import pytest
import torch

from tests import inputs as gen

pytestmark = pytest.mark.gpu


def _states(seed, static, T=700, B=2, H=2, K=64, M=32):
    from nha_b200 import _lib
    from nha_b200.chunk import _Geometry, _fill_desc
    lib = _lib.load()
    dev = 'cuda'
    d = gen.prefill_inputs(seed, B, H, 1, K, K, M, 16, T, with_state=True)
    flat = lambda x: x.reshape(B * T, *x.shape[2:]).to(dev).contiguous()
    t = dict(q_gsa=flat(d['q']), q_swa=flat(d['rotary_q']), k_gsa=flat(d['k']), k_swa=flat(d['rotary_k']),
             v=flat(d['v']), s=flat(d['s']), g=flat(d['g']), hk0=d['hk0'].to(dev), hv0=d['hv0'].to(dev))
    t['cu_seqlens'] = torch.arange(0, (B + 1) * T, T, dtype=torch.int32, device=dev)
    geo = _Geometry(t['q_gsa'], t['k_gsa'], t['v'], t['s'], t['cu_seqlens'], T, 0)
    t['hk_chunks'] = torch.zeros(geo.ncb, H, K, M, dtype=torch.bfloat16, device=dev)
    t['hv_chunks'] = torch.zeros(geo.ncb, H, M, K, dtype=torch.bfloat16, device=dev)
    t['hkt'] = torch.zeros(B, H, K, M, dtype=torch.float32, device=dev)
    t['hvt'] = torch.zeros(B, H, M, K, dtype=torch.float32, device=dev)
    desc = _fill_desc(geo, t, K ** -0.5, None, 15, None, 16)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(lib.nha_chunk_plan(ctypes.byref(desc), stream), 'plan')
    if static:
        st = lib.nha_chunk_state_pass_static(ctypes.byref(desc), stream)
    else:
        nbytes = int(lib.nha_chunk_fwd_workspace_bytes(ctypes.byref(desc)))
        assert nbytes > 0, 'the case must need scratch memory'
        t['workspace'] = torch.empty(nbytes, dtype=torch.uint8, device=dev)
        desc = _fill_desc(geo, t, K ** -0.5, None, 15, None, 16)
        st = lib.nha_chunk_state_pass(ctypes.byref(desc), stream)
    _lib.check(st, 'state pass')
    torch.cuda.synchronize()
    nchunks = B * ((T + 63) // 64)
    return t['hk_chunks'][:nchunks].float(), t['hv_chunks'][:nchunks].float(), t['hkt'], t['hvt']


def test_static_scratch_state_pass_matches_workspace_version_twice():
    for seed in (901, 902):            # two calls in a row; the second reuses a dirty array
        want = _states(seed, static=False)
        got = _states(seed, static=True)
        for a, b, name in zip(got, want, ('hk_chunks', 'hv_chunks', 'hkt', 'hvt')):
            assert torch.isfinite(a).all(), name
            assert torch.allclose(a, b, rtol=0, atol=0), f'{name} differs from the workspace version'


def test_static_scratch_refuses_oversized_problem():
    from nha_b200 import _lib
    from nha_b200.chunk import _Geometry, _fill_desc
    lib = _lib.load()
    assert lib.nha_chunk_state_pass_static_max_bytes() == 16 << 20
    dev = 'cuda'
    B, T, H, K, M = 1, 64 * 400, 8, 128, 64          # 400 chunks of 8 heads: > 16 MiB of scratch
    z = lambda *s: torch.zeros(*s, dtype=torch.bfloat16, device=dev)
    t = dict(q_gsa=z(T, H, K), q_swa=z(T, H, K), k_gsa=z(T, H, K), k_swa=z(T, H, K), v=z(T, H, K), s=z(T, H, M),
             g=z(T, H, M), cu_seqlens=torch.tensor([0, T], dtype=torch.int32, device=dev))
    geo = _Geometry(t['q_gsa'], t['k_gsa'], t['v'], t['s'], t['cu_seqlens'], T, 0)
    t['hk_chunks'] = z(geo.ncb, H, K, M)
    t['hv_chunks'] = z(geo.ncb, H, M, K)
    desc = _fill_desc(geo, t, 0.1, None, 15, None, 16)
    st = lib.nha_chunk_state_pass_static(ctypes.byref(desc), torch.cuda.current_stream().cuda_stream)
    assert st == 6
    assert b'static' in lib.nha_status_string(st)
