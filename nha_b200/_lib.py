"""ctypes binding of ``libnha_b200.so`` (the C ABI declared in ``include/nha_b200.h``).

The library is the only implementation: loading fails loudly when it is
missing and cannot be built, and every op raises when the library reports a
non-zero status.  Nothing here falls back to PyTorch arithmetic.
"""
from __future__ import annotations

import ctypes as C
import os
import threading

from . import build as _build

_lock = threading.Lock()
_lib = None

c_void_p = C.c_void_p


class ChunkDesc(C.Structure):
    """Mirror of ``nha_chunk_desc`` (include/nha_b200.h); field order and types must match."""
    _fields_ = [
        ('q_gsa', c_void_p), ('q_swa', c_void_p), ('k_gsa', c_void_p), ('k_swa', c_void_p), ('v', c_void_p),
        ('s', c_void_p), ('g', c_void_p), ('cu_seqlens', c_void_p), ('window_left', c_void_p), ('shift', c_void_p),
        ('hk0', c_void_p), ('hv0', c_void_p),
        ('o', c_void_p), ('lse_swa', c_void_p), ('lse_gsa', c_void_p), ('hkt', c_void_p), ('hvt', c_void_p),
        ('hk_chunks', c_void_p), ('hv_chunks', c_void_p),
        ('plan', c_void_p), ('workspace', c_void_p), ('workspace_bytes', C.c_size_t),
        ('d_o', c_void_p), ('d_lse_gsa', c_void_p), ('d_hkt', c_void_p), ('d_hvt', c_void_p),
        ('dq_gsa', c_void_p), ('dq_swa', c_void_p), ('dk_gsa', c_void_p), ('dk_swa', c_void_p), ('dv', c_void_p),
        ('ds', c_void_p), ('dg', c_void_p), ('dhk0', c_void_p), ('dhv0', c_void_p),
        ('Ttot', C.c_int32), ('N', C.c_int32), ('HQ', C.c_int32), ('H', C.c_int32), ('K', C.c_int32),
        ('V', C.c_int32), ('M', C.c_int32), ('max_seqlen', C.c_int32), ('window_left_all', C.c_int32),
        ('shift_all', C.c_int32), ('q_offset', C.c_int32), ('scale', C.c_float),
    ]


#: every symbol include/nha_b200.h declares -> (restype, argtypes)
SYMBOLS = {
    'nha_status_string': (C.c_char_p, [C.c_int]),
    'nha_last_cuda_error': (C.c_char_p, []),
    'nha_abi_version': (C.c_int, []),
    'nha_selftest_bounded_wait': (C.c_int, [c_void_p, C.c_int, c_void_p]),
    'nha_decode_workspace_bytes': (C.c_int64, [C.c_int] * 5),
    'nha_decode_step': (C.c_int, [c_void_p] * 10 + [C.c_int64, C.c_int64, c_void_p, c_void_p, c_void_p, C.c_int,
                                                     c_void_p, c_void_p, c_void_p, C.c_int64] + [C.c_int] * 7
                        + [C.c_float, c_void_p]),
    'nha_decode_step_bf16_state': (C.c_int, [c_void_p] * 10 + [C.c_int64, C.c_int64, c_void_p, c_void_p, C.c_int, c_void_p,
                                                                c_void_p, C.c_int64] + [C.c_int] * 7 + [C.c_float, c_void_p]),
    'nha_decode_device_error': (C.c_int, [c_void_p, C.c_int, C.c_int, c_void_p]),
    'nha_decode_set_pdl': (C.c_int, [C.c_int]),
    'nha_decode_get_pdl': (C.c_int, []),
    'nha_decode_step_ring': (C.c_int, [c_void_p] * 9 + [C.c_int64, C.c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                       C.c_int64] + [C.c_int] * 8 + [C.c_float, c_void_p]),
    'nha_ring_append': (C.c_int, [c_void_p] * 7 + [C.c_int] * 7 + [c_void_p]),
    'nha_decode_step_ring_fused': (C.c_int, [c_void_p] * 10 + [C.c_int64, C.c_int64, c_void_p, c_void_p, c_void_p, c_void_p,
                                             C.c_int64] + [C.c_int] * 8 + [C.c_float, c_void_p]),
    'nha_ring_rotate_rows': (C.c_int, [c_void_p] * 4 + [C.c_int64, C.c_int64] + [C.c_int] * 5 + [c_void_p]),
    'nha_decode_step_ring_rot': (C.c_int, [c_void_p] * 10 + [C.c_int64, c_void_p, c_void_p, c_void_p, c_void_p, C.c_int64]
                                 + [C.c_int] * 8 + [C.c_float, c_void_p]),
    'nha_ring_append_rot': (C.c_int, [c_void_p] * 9 + [C.c_int64, c_void_p] + [C.c_int] * 7 + [c_void_p]),
    'nha_chunk_desc_size': (C.c_int64, []),
    'nha_chunk_count_bound': (C.c_int64, [C.c_int64, C.c_int64]),
    'nha_chunk_plan_ints': (C.c_int64, [C.c_int64, C.c_int64, C.c_int64]),
    'nha_chunk_device_error': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_fwd_workspace_bytes': (C.c_int64, [C.POINTER(ChunkDesc)]),
    'nha_chunk_bwd_workspace_bytes': (C.c_int64, [C.POINTER(ChunkDesc)]),
    'nha_chunk_plan': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_state_pass': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_state_terms': (C.c_int, [C.POINTER(ChunkDesc), C.c_int, C.c_int, c_void_p]),
    'nha_chunk_state_scan': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_output_pass': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_apply_state_prefix': (C.c_int, [C.POINTER(ChunkDesc), c_void_p, c_void_p, c_void_p]),
    'nha_chunk_gate_totals': (C.c_int, [C.POINTER(ChunkDesc), C.POINTER(c_void_p)]),
    'nha_sp_fold_start_state': (C.c_int, [c_void_p] + [C.c_int] * 6 + [c_void_p] * 5),
    'nha_sp_publish': (C.c_int, [c_void_p, C.c_int64, c_void_p, c_void_p, c_void_p, C.c_int, C.c_int, C.c_int, c_void_p]),
    'nha_sp_fold_wait': (C.c_int, [c_void_p, c_void_p, c_void_p] + [C.c_int] * 7 + [c_void_p] * 6),
    'nha_sp_halo_push': (C.c_int, [c_void_p, c_void_p, c_void_p, C.c_int, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p]),
    'nha_sp_halo_wait': (C.c_int, [c_void_p, c_void_p, c_void_p, c_void_p]),
    'nha_sp_halo_ack': (C.c_int, [c_void_p, c_void_p, c_void_p]),
    'nha_chunk_fwd': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_bwd': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_state_pass_static_max_bytes': (C.c_int64, []),
    'nha_chunk_state_pass_static': (C.c_int, [C.POINTER(ChunkDesc), c_void_p]),
    'nha_chunk_bwd_stage': (C.c_int, [C.POINTER(ChunkDesc), C.c_int, c_void_p]),
    'nha_slot_gates_fwd': (C.c_int, [c_void_p, c_void_p, c_void_p, C.c_int64, C.c_float, c_void_p]),
    'nha_act3_fwd': (C.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, C.c_int, c_void_p]),
    'nha_act3_bwd': (C.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, C.c_int, c_void_p]),
    'nha_silu_rmsnorm_fwd': (C.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, C.c_int64, C.c_int, C.c_float,
                                       c_void_p]),
    'nha_silu_rmsnorm_bwd_ctas': (C.c_int, [C.c_int64]),
    'nha_silu_rmsnorm_bwd': (C.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, c_void_p, C.c_int64,
                                       C.c_int, c_void_p]),
    'nha_rope_pair': (C.c_int, [c_void_p] * 6 + [C.c_int64, C.c_int, c_void_p, C.c_int, C.c_int, C.c_int64] + [C.c_int] * 5
                      + [c_void_p]),
    'nha_lse_stats_scratch_bytes': (C.c_int64, []),
    'nha_lse_stats': (C.c_int, [c_void_p, c_void_p, C.c_int64, C.c_float, c_void_p, c_void_p, c_void_p]),
    'nha_lse_aux_grad': (C.c_int, [c_void_p, c_void_p, c_void_p, C.c_int64, C.c_float, c_void_p, c_void_p]),
    'nha_slot_gates_bwd': (C.c_int, [c_void_p, c_void_p, c_void_p, c_void_p, C.c_int64, C.c_float, c_void_p]),
}


class NHALibraryError(RuntimeError):
    pass


def lib_path() -> str:
    return _build.LIB


def load():
    """Load (building first if needed) the CUDA library and bind every declared symbol."""
    global _lib
    if _lib is not None:
        return _lib
    with _lock:
        if _lib is not None:
            return _lib
        path = _build.LIB
        if _build.is_stale():
            if _build.nvcc_path() is not None and os.environ.get('NHA_B200_NO_BUILD') != '1':
                _build.build()
            elif not os.path.exists(path):
                raise NHALibraryError(f'{path} is missing and nvcc is unavailable; nha_b200 has no fallback path')
        lib = C.CDLL(path)
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(lib, name)          # AttributeError if the library lacks a declared symbol
            fn.restype = res
            fn.argtypes = args
        if lib.nha_chunk_desc_size() != C.sizeof(ChunkDesc):
            raise NHALibraryError('nha_chunk_desc layout mismatch between the binding and the library')
        _lib = lib
        return lib


def check(status: int, what: str):
    if status != 0:
        lib = load()
        msg = lib.nha_status_string(status).decode()
        detail = lib.nha_last_cuda_error().decode()
        raise NHALibraryError(f'{what}: {msg}' + (f' [{detail}]' if detail and status == 4 else ''))


def check_device_words() -> bool:
    """True when ``NHA_B200_CHECK=1``: the ops then read the kernels' device error word after every call (a bounded
    wait that ran out leaves it non-zero) and raise.  Reading it synchronises the stream, so it is off by default, and
    it is skipped while the stream is being captured into a CUDA graph (a capture cannot be synchronised)."""
    if os.environ.get('NHA_B200_CHECK') != '1':
        return False
    import torch
    return not torch.cuda.is_current_stream_capturing()


def check_chunk_device(lib, desc, stream, what: str):
    if check_device_words():
        e = lib.nha_chunk_device_error(desc, stream)
        if e != 0:
            raise NHALibraryError(f'{what}: device error word {e} (a bounded wait on a tensor-core completion ran out; '
                                  f'the outputs of this call are invalid)')


def check_decode_device(lib, ws, B, H, stream, what: str):
    if ws is not None and check_device_words():
        e = lib.nha_decode_device_error(ws.data_ptr(), B, H, stream)
        if e != 0:
            raise NHALibraryError(f'{what}: device error word {e} (a bounded wait in the decode kernel ran out; '
                                  f'the outputs of this call are invalid)')


def ptr(t):
    """Device pointer of a tensor (or NULL for None)."""
    return None if t is None else t.data_ptr()
