"""Install the B200 kernels behind the reference package's own names, without editing the reference.

The reference binds the entry point at import time (``from semicat.jvp_utils.functional import
safe_sdpa_jvp`` in semicat/net/duo.py:15, dit.py, song.py, mysong.py), so both the defining module and
every module that already imported the name are re-pointed.  ``uninstall()`` restores the originals.
"""
from __future__ import annotations

import importlib
import sys

from . import functional as _ours

_CALLERS = ("semicat.net.duo", "semicat.net.dit", "semicat.net.song", "semicat.net.mysong")
_saved: dict = {}


def install(strict: bool = False) -> list[str]:
    """Re-point ``sdpa_jvp`` / ``safe_sdpa_jvp`` of an importable ``semicat`` package at this library.
    Returns the names of the modules that were patched.  With ``strict`` a missing ``semicat`` raises."""
    patched = []
    try:
        ref = importlib.import_module("semicat.jvp_utils.functional")
    except Exception:
        if strict:
            raise
        return patched
    for name in ("sdpa_jvp", "safe_sdpa_jvp"):
        _saved.setdefault((ref.__name__, name), getattr(ref, name))
        setattr(ref, name, getattr(_ours, name))
    patched.append(ref.__name__)
    for modname in _CALLERS:
        mod = sys.modules.get(modname)
        if mod is None:
            try:
                mod = importlib.import_module(modname)
            except Exception:
                continue  # optional dependencies of that network are missing; nothing to patch
        for name in ("sdpa_jvp", "safe_sdpa_jvp"):
            if hasattr(mod, name):
                _saved.setdefault((modname, name), getattr(mod, name))
                setattr(mod, name, getattr(_ours, name))
        patched.append(modname)
    return patched


def uninstall() -> None:
    for (modname, name), fn in list(_saved.items()):
        mod = sys.modules.get(modname)
        if mod is not None:
            setattr(mod, name, fn)
    _saved.clear()
