"""Attention backend selection.

The reference exposes ``ATTN_BACKEND`` (torch_native / cuda / flash), a context manager ``attn_backend(...)``, the
``ASTR_BACKEND`` environment override and ``get_backend()`` (``astrai/extension/backend/attention.py:61-303``).  This
framework has one architecture, so the choice is between the hand-written sm_100a kernels (``TCGEN05``, the default on
CUDA: flash forward / backward, ragged prefill, paged decode) and the plain-PyTorch statement (``TORCH_NATIVE``:
SDPA, the only choice on CPU and the oracle / baseline on GPU).  The reference's names ``cuda`` and ``flash`` are
accepted as aliases of ``TCGEN05``.  Selection order, as in the reference (``attention.py:204-217``): the process-wide
``ASTR_BACKEND`` (or ``ASTRAI_B200_ATTN``) > the innermost ``attn_backend(...)`` context > default; a call the kernels
do not cover (arbitrary boolean mask, head dim outside 64 / 128 for dense attention) falls
back to ``TORCH_NATIVE`` unless the backend was chosen explicitly, in which case it raises.
"""

from __future__ import annotations

import contextlib
import contextvars
import enum
import os
from typing import Optional, Union

from astrai_b200.factory import BaseFactory


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


_current: contextvars.ContextVar[Optional[object]] = contextvars.ContextVar("astrai_b200_attn_backend", default=None)


class AttentionBackend:
    """Base class of attention back ends (the reference's ``AttentionBackend``, ``attention.py:306-396``).

    The two built-in ones select between this package's kernels and the plain-PyTorch statement.  A subclass of its own
    implements :meth:`fwd_prefill` (training when ``kv_cache`` is ``None``: dense ``[B, S, H, D]`` in and out; serving:
    packed ``[T, H, D]`` tensors plus the KV cache struct) and :meth:`fwd_decode` (one token per request), is registered
    in :class:`AttentionBackendFactory`, and receives every attention call made while it is selected
    (``with attn_backend(MyBackend()):``, ``with MyBackend():``, ``InferenceScheduler(backend=...)`` or ``ASTR_BACKEND``).
    """

    kind: Optional[ATTN_BACKEND] = None  # built-in back ends: the enum member they stand for

    def __enter__(self) -> "AttentionBackend":
        self._token = _current.set(self.kind if self.kind is not None else self)
        return self

    def __exit__(self, *exc) -> None:
        _current.reset(self._token)

    def forward(self, q, k, v, kv_cache=None, layer_id: int = 0, attn_mask=None, is_causal: bool = False, fwd: Optional[str] = None):
        if fwd == "decode":
            return self.fwd_decode(q, k, v, kv_cache, layer_id, attn_mask, is_causal)
        if fwd == "prefill" or fwd is None:
            return self.fwd_prefill(q, k, v, kv_cache, layer_id, attn_mask, is_causal)
        raise ValueError(f"unsupported attention forward mode: {fwd}")

    def fwd_decode(self, q, k, v, kv_cache, layer_id: int, attn_mask=None, is_causal: bool = False):
        raise NotImplementedError

    def fwd_prefill(self, q, k, v, kv_cache, layer_id: int, attn_mask=None, is_causal: bool = False):
        raise NotImplementedError

    @staticmethod
    def supports(**kwargs) -> bool:
        return True

    @staticmethod
    def supports_graph() -> bool:
        """Whether decode steps under this back end may be captured into CUDA graphs."""
        return False


class AttentionBackendFactory(BaseFactory[AttentionBackend]):
    """Registered attention back ends by name."""


class _BuiltIn(AttentionBackend):
    """A built-in back end runs the package's own attention entry under its selection."""

    def _run(self, q, k, v, kv_cache, layer_id, attn_mask, is_causal, fwd):
        from astrai_b200.ops.attention import attention

        with self:
            return attention(q, k, v, kv_cache, layer_id, attn_mask, is_causal, fwd)

    def fwd_decode(self, q, k, v, kv_cache, layer_id: int, attn_mask=None, is_causal: bool = False):
        return self._run(q, k, v, kv_cache, layer_id, attn_mask, is_causal, "decode")

    def fwd_prefill(self, q, k, v, kv_cache, layer_id: int, attn_mask=None, is_causal: bool = False):
        return self._run(q, k, v, kv_cache, layer_id, attn_mask, is_causal, None if kv_cache is None else "prefill")


@AttentionBackendFactory.register("torch_native")
class TorchNativeBackend(_BuiltIn):
    """PyTorch's scaled-dot-product attention (with per-request gathers from the KV pool when serving)."""

    kind = ATTN_BACKEND.TORCH_NATIVE


@AttentionBackendFactory.register("tcgen05")
class Tcgen05Backend(_BuiltIn):
    """The sm_100a kernels: flash forward / backward, ragged prefill over the paged pool, paged decode."""

    kind = ATTN_BACKEND.TCGEN05

    @staticmethod
    def supports(**kwargs) -> bool:
        return is_available(ATTN_BACKEND.TCGEN05)

    @staticmethod
    def supports_graph() -> bool:
        return True


@AttentionBackendFactory.register("cuda")
class CudaBackend(Tcgen05Backend):
    """The tcgen05 back end under the name of the reference's own-kernel back end."""


@AttentionBackendFactory.register("flash")
class FlashAttnBackend(Tcgen05Backend):
    """The tcgen05 back end under the name of the reference's flash-attention back end."""


Selection = Union[str, ATTN_BACKEND, AttentionBackend, type]


def resolve(backend: Selection):
    """What a selection stands for: an :class:`ATTN_BACKEND` member for the built-in back ends (under any of their
    names, as enum, class or instance), else the instance of a registered or given back end of its own."""
    if isinstance(backend, ATTN_BACKEND):
        return backend
    if isinstance(backend, type) and issubclass(backend, AttentionBackend):
        backend = backend()
    if isinstance(backend, AttentionBackend):
        return backend.kind if backend.kind is not None else backend
    if isinstance(backend, str):
        try:
            return ATTN_BACKEND.parse(backend)
        except ValueError:
            name = backend.strip().lower()
            if name in AttentionBackendFactory.list_registered():
                return resolve(AttentionBackendFactory.create(name))
            raise
    raise ValueError(f"unknown attention backend {backend!r}")


_env_cache = {"raw": None, "chosen": None}


def _environment():
    raw = os.environ.get("ASTR_BACKEND") or os.environ.get("ASTRAI_B200_ATTN")
    if not raw:
        return None
    if raw != _env_cache["raw"]:  # a registered back end of its own is built once per value of the variable
        _env_cache["raw"], _env_cache["chosen"] = raw, resolve(raw)
    return _env_cache["chosen"]


def get_backend(device_type: str = "cuda", use_default: bool = True):
    """The back end a call on ``device_type`` would use right now: an :class:`ATTN_BACKEND` member, or the instance of a
    back end of its own.  ``use_default=False`` returns only what the environment or a context named (``None`` if
    neither did)."""
    chosen = _environment() or _current.get()
    if not use_default:
        return chosen
    if isinstance(chosen, AttentionBackend):
        return chosen
    if device_type != "cuda":
        return ATTN_BACKEND.TORCH_NATIVE
    return chosen or ATTN_BACKEND.TCGEN05


def current_custom() -> Optional[AttentionBackend]:
    """The selected back end if it is one that computes attention itself (not one of the two built-in ones)."""
    chosen = _environment() or _current.get()
    return chosen if isinstance(chosen, AttentionBackend) else None


def explicit() -> bool:
    """True when the caller (context or environment) named a backend: no silent fallback then."""
    return _current.get() is not None or _environment() is not None


@contextlib.contextmanager
def attn_backend(backend: Selection):
    """Select the attention back end for the calls made inside (per thread): a name, an :class:`ATTN_BACKEND` member, an
    :class:`AttentionBackend` class or an instance."""
    token = _current.set(resolve(backend))
    try:
        yield
    finally:
        _current.reset(token)


def is_available(backend: Union[str, ATTN_BACKEND] = ATTN_BACKEND.TCGEN05) -> bool:
    b = resolve(backend)
    if b is ATTN_BACKEND.TORCH_NATIVE:
        return True
    if isinstance(b, AttentionBackend):
        return bool(b.supports())
    import torch

    from astrai_b200.ops import native

    return torch.cuda.is_available() and native.is_available()
