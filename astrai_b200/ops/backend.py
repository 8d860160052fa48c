"""Attention backend selection.

The reference exposes ``ATTN_BACKEND`` (torch_native / cuda / flash), a context manager ``attn_backend(...)``, the
``ASTR_BACKEND`` environment override and ``get_backend()`` (``astrai/extension/backend/attention.py:61-303``).  This
framework has one architecture, so the choice is between the hand-written sm_100a kernels (``TCGEN05``, the default on
CUDA: flash forward / backward, ragged prefill, paged decode) and the plain-PyTorch statement (``TORCH_NATIVE``:
SDPA, the only choice on CPU and the oracle / baseline on GPU).  The reference's names ``cuda`` and ``flash`` are
accepted as aliases of ``TCGEN05``.  Selection order, as in the reference (``attention.py:204-217``): the process-wide
``ASTR_BACKEND`` (or ``ASTRAI_B200_ATTN``) > the innermost ``attn_backend(...)`` context > default; a call the kernels do not cover (arbitrary boolean mask, head dim outside 64 / 128 for dense attention) falls
back to ``TORCH_NATIVE`` unless the backend was chosen explicitly, in which case it raises.
"""

from __future__ import annotations

import contextlib
import contextvars
import enum
import os
from typing import Optional, Union


class ATTN_BACKEND(enum.Enum):
    TORCH_NATIVE = "torch_native"
    TCGEN05 = "tcgen05"

    @classmethod
    def parse(cls, value: Union[str, "ATTN_BACKEND"]) -> "ATTN_BACKEND":
        if isinstance(value, cls):
            return value
        name = str(value).strip().lower()
        aliases = {"cuda": cls.TCGEN05, "flash": cls.TCGEN05, "tcgen05": cls.TCGEN05, "native": cls.TCGEN05,
                   "torch": cls.TORCH_NATIVE, "torch_native": cls.TORCH_NATIVE, "sdpa": cls.TORCH_NATIVE}
        if name not in aliases:
            raise ValueError(f"unknown attention backend {value!r}; choose from {sorted(aliases)}")
        return aliases[name]


_current: contextvars.ContextVar[Optional[ATTN_BACKEND]] = contextvars.ContextVar("astrai_b200_attn_backend", default=None)


def _environment() -> Optional[ATTN_BACKEND]:
    raw = os.environ.get("ASTR_BACKEND") or os.environ.get("ASTRAI_B200_ATTN")
    return ATTN_BACKEND.parse(raw) if raw else None


def get_backend(device_type: str = "cuda", use_default: bool = True) -> Optional[ATTN_BACKEND]:
    """The backend a call on ``device_type`` would use right now.  ``use_default=False`` returns only what the
    environment or a context named (``None`` if neither did)."""
    chosen = _environment() or _current.get()
    if not use_default:
        return chosen
    if device_type != "cuda":
        return ATTN_BACKEND.TORCH_NATIVE
    return chosen or ATTN_BACKEND.TCGEN05


def explicit() -> bool:
    """True when the caller (context or environment) named a backend: no silent fallback then."""
    return _current.get() is not None or _environment() is not None


@contextlib.contextmanager
def attn_backend(backend: Union[str, ATTN_BACKEND]):
    token = _current.set(ATTN_BACKEND.parse(backend))
    try:
        yield
    finally:
        _current.reset(token)


def is_available(backend: Union[str, ATTN_BACKEND] = ATTN_BACKEND.TCGEN05) -> bool:
    b = ATTN_BACKEND.parse(backend)
    if b is ATTN_BACKEND.TORCH_NATIVE:
        return True
    import torch

    from astrai_b200.ops import native

    return torch.cuda.is_available() and native.is_available()
