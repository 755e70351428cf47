"""Loading of the native extensions (built in-tree by ``_build.py``).

``core()`` returns the host-only module, ``cuda()`` the sm_100a module.  Nothing falls back to
Python: if a module is missing and cannot be built, the call raises.
"""
from __future__ import annotations

import importlib
import threading

_lock = threading.Lock()
_mods: dict[str, object] = {}


def _load(name: str):
    with _lock:
        if name in _mods:
            return _mods[name]
        try:
            mod = importlib.import_module(f"sharedtensor_b200.{name}")
        except ImportError:
            from . import _build

            (_build.build_core if name == "_core" else _build.build_cuda)()
            importlib.invalidate_caches()
            mod = importlib.import_module(f"sharedtensor_b200.{name}")
        _mods[name] = mod
        return mod


def core():
    return _load("_core")


def cuda():
    return _load("_cuda")
