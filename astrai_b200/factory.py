"""Name -> class registries used by every pluggable part of the framework.

Parity target: ``astrai/factory.py:63-153`` of the reference (``BaseFactory``):
decorator registration, base-class validation, duplicate rejection, and
``create`` that drops keyword arguments the target constructor cannot take.
"""

from __future__ import annotations

import inspect
import sys
import typing
from typing import Callable, ClassVar, Dict, Generic, List, Optional, Type, TypeVar

T = TypeVar("T")


def _lookup_base(type_arg, owner: type) -> Optional[type]:
    """Turn the ``T`` of ``BaseFactory[T]`` into a class (or None if unknown)."""
    if isinstance(type_arg, type):
        return type_arg
    if isinstance(type_arg, typing.ForwardRef):
        type_arg = type_arg.__forward_arg__
    if not isinstance(type_arg, str):
        return None
    namespace = vars(sys.modules.get(owner.__module__, object()))
    found = namespace.get(type_arg) if isinstance(namespace, dict) else None
    return found if isinstance(found, type) else None


class BaseFactory(Generic[T]):
    """Registry keyed by string.  Subclass as ``class XFactory(BaseFactory[XBase])``."""

    _entries: ClassVar[Dict[str, type]]
    _component_base: ClassVar[Optional[type]] = None
    _pending_base: ClassVar[object] = None

    def __init_subclass__(cls, **kw):
        super().__init_subclass__(**kw)
        for base in getattr(cls, "__orig_bases__", ()):
            if typing.get_origin(base) is BaseFactory:
                (arg,) = typing.get_args(base)
                cls._entries = {}
                cls._pending_base = arg
                cls._component_base = _lookup_base(arg, cls)
                break

    @classmethod
    def _base(cls) -> Optional[type]:
        # A forward reference may only become resolvable after the module body ran.
        if cls._component_base is None and cls._pending_base is not None:
            cls._component_base = _lookup_base(cls._pending_base, cls)
        return cls._component_base

    @classmethod
    def register(cls, name: str) -> Callable[[Type[T]], Type[T]]:
        def deco(klass: Type[T]) -> Type[T]:
            base = cls._base()
            if base is not None and not (isinstance(klass, type) and issubclass(klass, base)):
                raise TypeError(f"{getattr(klass, '__name__', klass)} must inherit from {base.__name__}")
            if name in cls._entries:
                raise ValueError(f"Component '{name}' is already registered")
            cls._entries[name] = klass
            return klass

        return deco

    @classmethod
    def get_component_class(cls, name: str) -> Type[T]:
        try:
            return cls._entries[name]
        except KeyError:
            raise ValueError(
                f"Unknown component: '{name}'. Supported types: {sorted(cls._entries)}"
            ) from None

    @classmethod
    def create(cls, name: str, *args, **kwargs) -> T:
        klass = cls.get_component_class(name)
        params = inspect.signature(klass.__init__).parameters
        if not any(p.kind is inspect.Parameter.VAR_KEYWORD for p in params.values()):
            kwargs = {k: v for k, v in kwargs.items() if k in params and k != "self"}
        return klass(*args, **kwargs)

    @classmethod
    def list_registered(cls) -> List[str]:
        return sorted(cls._entries)

    @classmethod
    def is_registered(cls, name: str) -> bool:
        return name in cls._entries
