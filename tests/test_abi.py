"""CPU: the C-ABI library builds, loads and exports every symbol include/nha_b200.h declares."""
import ctypes
import os
import re

from nha_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    text = open(os.path.join(ROOT, 'include', 'nha_b200.h')).read()
    text = re.sub(r'/\*.*?\*/', '', text, flags=re.S)
    return set(re.findall(r'\b(nha_[a-z_0-9]+)\s*\(', text))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = declared_symbols()
    assert names, 'no declarations parsed from the header'
    for name in names:
        assert hasattr(lib, name), f'{name} declared in include/nha_b200.h but not exported'
    assert names == set(_lib.SYMBOLS), 'binding table and header disagree'


def test_desc_layout_and_status_strings():
    lib = _lib.load()
    assert lib.nha_chunk_desc_size() == ctypes.sizeof(_lib.ChunkDesc)
    assert lib.nha_abi_version() >= 1
    assert lib.nha_status_string(0) == b'ok'
    assert b'unsupported' in lib.nha_status_string(2)
    assert lib.nha_chunk_count_bound(130, 2) == 3 + 2
    # offsets, chunk -> sequence, flags, error word, padded to a multiple of four ints, then 4 ints per chunk
    assert lib.nha_chunk_plan_ints(130, 2, 3) == (3 + 5 + 5 * 3 + 4 + 3) // 4 * 4 + 4 * 5


def test_argument_validation_needs_no_gpu():
    lib = _lib.load()
    # null pointers are rejected before any CUDA call
    st = lib.nha_decode_step(None, None, None, None, None, None, None, None, None, None, 0, 0, None, None, None, 0,
                             None, None, None, 0, 1, 4, 2, 64, 64, 16, 8, 0.125, None)
    assert st == 1
    d = _lib.ChunkDesc()
    assert lib.nha_chunk_fwd(ctypes.byref(d), None) == 1


def test_operator_signatures_equal_the_reference():
    """Parameter names, kinds and defaults of the four public ops against those of the reference's ops, read from its
    sources by tests/golden/make_boundary.py (nha_fla/ops/nha/chunk.py:568-585, chunk_fused.py:291-303,
    fused_recurrent.py:431-445, :588-598).  Callers pass keywords, so names and defaults are the contract."""
    import inspect
    import json
    import nha_b200
    want = json.load(open(os.path.join(ROOT, 'tests', 'golden', 'boundary.json')))['signatures']
    assert set(want) == {'chunk_nha', 'fused_chunk_nha_prefill', 'fused_recurrent_nha', 'fused_recurrent_nha_decode'}
    for name, params in want.items():
        got = [[p.name, str(p.kind), None if p.default is inspect.Parameter.empty else repr(p.default)]
               for p in inspect.signature(getattr(nha_b200, name)).parameters.values()]
        assert got == params, f'{name}: {got} != {params}'


def test_patch_reference_rebinds_every_import_site():
    """With the reference package importable, patch_reference() must reach every module that bound an operator by
    name, including the hybrid model file that imports fused_chunk_nha_prefill from its defining module."""
    import pytest
    nha_fla = pytest.importorskip('nha_fla', reason='reference package not importable here')
    import nha_b200
    done = nha_b200.patch_reference()
    try:
        import nha_fla.layers.nha as layer
        import nha_fla.ops.nha as ops
        assert layer.chunk_nha is nha_b200.chunk_nha and ops.chunk_nha is nha_b200.chunk_nha
        assert ops.fused_recurrent_nha_decode is nha_b200.fused_recurrent_nha_decode
        import nha_fla.models.qwen3_moe_nha.qwennha as moe
        assert moe.fused_chunk_nha_prefill is nha_b200.fused_chunk_nha_prefill
        assert moe.fused_recurrent_nha_decode is nha_b200.fused_recurrent_nha_decode
        assert 'nha_fla.ops.nha.chunk_fused' in done['fused_chunk_nha_prefill']
    finally:
        nha_b200.unpatch_reference()
    import nha_fla.ops.nha as ops
    assert ops.chunk_nha is not nha_b200.chunk_nha


def test_wide_window_layers_pass_the_reference_gates():
    """route_wide_windows() makes a layer with window_size > 64 take the branches the reference reserves for
    window_size <= 64 (its gates are literal comparisons with 64), while the value stays usable as the integer it is."""
    import torch
    import nha_b200

    class Attn(torch.nn.Module):               # the attributes the reference's attention classes carry
        def __init__(self, w):
            super().__init__()
            self.window_size, self.num_slots = w, 64

        def takes_nha_path(self):
            # the reference's gate expressions (nha_fla/models/qwen3_moe_nha/qwennha.py:185, 219, 274, 345)
            return (not (self.window_size > 64)) and self.window_size <= 64

    model = torch.nn.ModuleList([Attn(64), Attn(2048), Attn(512)])
    assert [m.takes_nha_path() for m in model] == [True, False, False]
    assert nha_b200.route_wide_windows(model) == ['1', '2']
    assert all(m.takes_nha_path() for m in model)
    w = model[1].window_size
    assert w == 2048 and w - 1 == 2047 and int(w) == 2048 and list(range(3000))[-w:][0] == 952
    assert w <= 4096 and not (w <= 100) and w > 100                  # other comparisons are the integer's
    # the cache's bookkeeping (nha_fla/models/nha_cache.py:86-104): sizes compared with and sliced by window_size
    x = torch.zeros(1, 3000, 4)
    assert x.shape[-2] > w and x[..., -w:, :].shape[-2] == 2048 and (x[..., -w:, :].shape[-2] == w)
    assert nha_b200.route_wide_windows(model) == []                  # idempotent
