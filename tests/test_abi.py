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
