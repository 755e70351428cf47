"""Checkpoint / resume.

The reference keeps its state in process memory only; "resume" there means joining again and being streamed the
state by the parent.  Here a replica's values can be written to disk and a tree can be re-founded from the file:
the first process that calls ``createOrFetch`` with the loaded tensor becomes the master, later ones join it as
usual.  A running replica can also be overwritten in place (``load_state_dict``); the difference to its previous
values propagates like any other update.
"""
from __future__ import annotations

import os
import tempfile
from typing import Any

import torch


def save(shared: Any, path: str, extra: dict | None = None) -> None:
    """Writes ``shared.state_dict()`` atomically.  The state is the replica's values.  Mirrors are not part of it: a
    mirror says what one particular neighbour holds, and a replica that comes back from a file meets new neighbours,
    whose links start from a snapshot (GPU edges) or from zero (TCP edges, as in the reference)."""
    state = {"state": shared.state_dict(), "numel": shared.numel, "shape": tuple(shared.shape), "extra": extra or {}}
    d = os.path.dirname(os.path.abspath(path))
    fd, tmp = tempfile.mkstemp(dir=d, suffix=".tmp")
    os.close(fd)
    try:
        torch.save(state, tmp)
        os.replace(tmp, path)
    finally:
        if os.path.exists(tmp):
            os.remove(tmp)


def load_values(path: str, device: str | torch.device = "cpu") -> tuple[torch.Tensor, dict]:
    """Returns ``(values shaped like the saved tensor, extra)`` for a fresh ``createOrFetch``."""
    state = torch.load(path, map_location="cpu")
    v = state["state"]["values"].view(state["shape"]).to(device)
    return v, state.get("extra", {})


def restore_into(shared: Any, path: str) -> dict:
    """Overwrites a live replica with the saved values."""
    state = torch.load(path, map_location="cpu")
    if state["numel"] != shared.numel:
        raise ValueError("Not the right size!")
    shared.load_state_dict(state["state"])
    return state.get("extra", {})
