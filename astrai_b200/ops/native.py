"""Loader of the in-tree sm_100a extension (``_C.so``) and its ``torch.ops.astrai_b200`` namespace.

The reference loads one pybind module per kernel from ``astrai/extension/lib`` and silently falls back to
torch when a module is missing (``astrai/extension/loader.py:23-54``).  Here a CUDA tensor never falls back
silently: if the library cannot be loaded on a machine that has a GPU, the first native call raises.
"""

from __future__ import annotations

import os
import threading
from pathlib import Path

import torch

_LIB = Path(__file__).resolve().parent / "_C.so"
_lock = threading.Lock()
_state = {"loaded": False, "error": None}


def lib_path() -> Path:
    return _LIB


def load(build_if_missing: bool = True) -> bool:
    """Load ``_C.so`` (building it first if it is absent and nvcc exists).  Returns True on success."""
    if _state["loaded"]:
        return True
    with _lock:
        if _state["loaded"]:
            return True
        try:
            if not _LIB.exists() and build_if_missing and os.environ.get("ASTRAI_B200_NO_BUILD") != "1":
                from astrai_b200.ops.build import build

                build()
            torch.ops.load_library(str(_LIB))
            _state["loaded"] = True
            _state["error"] = None
        except Exception as exc:  # noqa: BLE001 - reported by require()
            _state["error"] = exc
        return _state["loaded"]


def is_available() -> bool:
    return load()


def require():
    """Return ``torch.ops.astrai_b200`` or raise with the reason the library is missing."""
    if not load():
        raise RuntimeError(
            f"astrai_b200 native extension is not available ({_state['error']!r}); "
            "run `python -m astrai_b200.ops.build` (needs nvcc with sm_100a support)"
        )
    return torch.ops.astrai_b200


def kernel_status(device) -> int:
    """Largest error code recorded by a kernel whose bounded wait expired (0 = none).  Synchronises."""
    like = torch.empty(0, device=device)
    return int(require().kernel_status(like).max().item())


def launch_count() -> int:
    """Kernels of this library launched by this process so far."""
    return int(require().launch_count())


def _op_names():
    """Names under ``torch.ops.astrai_b200``, read from the binding source (one ``m.def("name(...)")`` per operator)."""
    import re

    src = Path(__file__).resolve().parent / "csrc" / "bindings.cpp"
    try:
        return tuple(sorted(set(re.findall(r'm\.def\("([A-Za-z0-9_]+)\(', src.read_text()))))
    except OSError:
        return ()


KERNEL_NAMES = _op_names()


def kernel_available(name: str = "") -> bool:
    """True if the extension is loaded and (when ``name`` is given) has that operator; never raises, never builds."""
    if name and name not in KERNEL_NAMES:
        return False
    if not _state["loaded"] and not _LIB.exists():
        return False
    return load(build_if_missing=False)


def get_module(name: str):
    """The loaded operator ``torch.ops.astrai_b200.<name>``, or ``None`` when the extension (or that operator) is not there -
    the lookup of the reference's loader (``astrai/extension/loader.py:51-54``), one namespace instead of one module per
    kernel."""
    if not kernel_available(name):
        return None
    return getattr(torch.ops.astrai_b200, name, None)
