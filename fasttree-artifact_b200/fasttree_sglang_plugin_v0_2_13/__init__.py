"""SGLang v0.2.13 plugin: radix-cache decode attention on the B200 engine.

Same public surface as the reference package
(sglang_v0.2.13_bench/fasttree_sglang_plugin_v0_2_13/__init__.py:1-5)."""
import os as _os
import sys as _sys

_PKG = _os.path.dirname(_os.path.dirname(_os.path.abspath(__file__)))
if _PKG not in _sys.path:
    _sys.path.insert(0, _PKG)

from .plugin import load_fasttree_plugin  # noqa: E402

__all__ = ["load_fasttree_plugin"]
