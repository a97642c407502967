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
