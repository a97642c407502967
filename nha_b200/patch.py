"""Rebinding of the reference package's operator names to this package.

``patch_reference()`` makes an installed ``nha_fla`` (JusenD/NHA) call the sm_100a kernels without an edit to its
sources: every module attribute of ``nha_fla`` that IS one of the reference's four operator functions is rebound to
the function of the same name here.  That covers the re-exports (``nha_fla/ops/__init__.py:3-11``,
``nha_fla/ops/nha/__init__.py:3-10``), the defining modules (``ops/nha/chunk.py``, ``ops/nha/fused_recurrent.py``,
``ops/nha/chunk_fused.py``) and the names the callers imported with ``from ... import``
(``nha_fla/layers/nha.py:17``; ``nha_fla/models/llama3_nha/llamanha.py:13``;
``nha_fla/models/{qwen2_nha,qwen3_nha}/qwennha.py:12``; ``nha_fla/models/qwen3_moe_nha/qwennha.py:12-13``, which takes
``fused_chunk_nha_prefill`` from ``nha_fla.ops.nha.chunk_fused`` directly).
"""
from __future__ import annotations

import importlib
import sys
from typing import Dict, List

OP_NAMES = ('chunk_nha', 'fused_chunk_nha_prefill', 'fused_recurrent_nha', 'fused_recurrent_nha_decode')

#: (module of the reference, attribute) that defines each operator
_DEFINED_IN = {
    'chunk_nha': 'nha_fla.ops.nha.chunk',
    'fused_chunk_nha_prefill': 'nha_fla.ops.nha.chunk_fused',
    'fused_recurrent_nha': 'nha_fla.ops.nha.fused_recurrent',
    'fused_recurrent_nha_decode': 'nha_fla.ops.nha.fused_recurrent',
}

#: caller modules that bind the operators by name at import time
_CALLERS = ('nha_fla.ops', 'nha_fla.ops.nha', 'nha_fla.layers.nha', 'nha_fla.models.llama3_nha.llamanha',
            'nha_fla.models.qwen2_nha.qwennha', 'nha_fla.models.qwen3_nha.qwennha',
            'nha_fla.models.qwen3_moe_nha.qwennha')

_undo: List[tuple] = []


def patch_reference(import_callers: bool = True) -> Dict[str, List[str]]:
    """Rebind the reference's operator names to ``nha_b200``'s.  Returns ``{operator: [module names patched]}``.

    Raises ``ImportError`` when ``nha_fla`` is not importable.  ``import_callers=False`` patches only the modules
    that are already imported (plus the defining ones).  ``unpatch_reference()`` restores the originals."""
    import nha_b200
    originals = {}
    for name, mod in _DEFINED_IN.items():
        m = importlib.import_module(mod)
        originals[name] = getattr(m, name)
    if import_callers:
        for mod in _CALLERS:
            try:
                importlib.import_module(mod)
            except ImportError:                      # an optional dependency of that caller is absent
                continue
    done: Dict[str, List[str]] = {n: [] for n in OP_NAMES}
    for modname, m in list(sys.modules.items()):
        if m is None or not (modname == 'nha_fla' or modname.startswith('nha_fla.')):
            continue
        for name, ref_fn in originals.items():
            if getattr(m, name, None) is ref_fn:
                setattr(m, name, getattr(nha_b200, name))
                _undo.append((m, name, ref_fn))
                done[name].append(modname)
    return done


def unpatch_reference() -> None:
    while _undo:
        m, name, fn = _undo.pop()
        setattr(m, name, fn)


class WideWindow(int):
    """A window size that passes the reference models' ``window_size <= 64`` gates.

    The hybrid model classes send a layer through the NHA ops (slot memory + window) only when ``self.window_size <= 64``
    (``nha_fla/models/qwen3_moe_nha/qwennha.py:185, 219, 274, 345``; ``llama3_nha/llamanha.py:183, 218``;
    ``qwen2_nha/qwennha.py:202, 236``; ``qwen3_nha/qwennha.py:190, 225``); wider layers fall to plain sliding-window /
    full attention without slots, because the reference's fused kernels stop at 64 keys
    (``nha_fla/ops/nha/chunk_fused.py:332``).  The kernels here take any window, so a layer whose ``window_size`` is a
    ``WideWindow`` answers those comparisons with 64 as "not wider" and is otherwise the plain integer (arithmetic,
    slicing, equality, the cache's ``window_size`` bookkeeping)."""

    def __le__(self, other):
        return True if other == 64 else int.__le__(self, other)

    def __gt__(self, other):
        return False if other == 64 else int.__gt__(self, other)

    def __lt__(self, other):
        return True if other == 65 else int.__lt__(self, other)

    def __ge__(self, other):
        return False if other == 65 else int.__ge__(self, other)


def route_wide_windows(model, max_window: int = 1 << 20) -> List[str]:
    """Send the wide-window attention layers of a reference model through the NHA ops as well: every sub-module that has
    an integer ``window_size`` above 64 and slot parameters (``num_slots``) gets a :class:`WideWindow` of the same value.
    Call :func:`patch_reference` too, so that those ops are this package's.  Returns the names of the modules changed.

    This changes what such a layer computes (it now reads the slot memory, like the narrow layers), which is the point
    of the routing; it needs weights trained for it."""
    changed = []
    for name, m in model.named_modules():
        w = getattr(m, 'window_size', None)
        if isinstance(w, int) and not isinstance(w, WideWindow) and 64 < w <= max_window and hasattr(m, 'num_slots'):
            m.window_size = WideWindow(w)
            changed.append(name)
    return changed
