"""Packaging: ``pip install .`` (or ``-e .``) compiles the sm_100a extension in the source tree first.

The metadata lives in ``pyproject.toml``.  The native extension is not a setuptools ``Extension``: it is built by
``astrai_b200/ops/build.py`` (nvcc for ``sm_100a`` only, objects cached by source hash) into ``astrai_b200/ops/_C.so``
and shipped as package data.  ``ASTRAI_B200_BUILD_EXT=0`` skips the build (a CPU-only install: everything that does not
launch a kernel still works); ``=1`` makes a failed build an error; unset, the build runs when ``nvcc`` is on the path
and a failure is a warning.
"""

import os
import shutil
import sys
import warnings
from pathlib import Path

from setuptools import Distribution, setup
from setuptools.command.build_py import build_py as _build_py

ROOT = Path(__file__).resolve().parent


def want_extension() -> bool:
    flag = os.environ.get("ASTRAI_B200_BUILD_EXT", "").strip().lower()
    if flag in ("0", "false", "no", "off"):
        return False
    if flag in ("1", "true", "yes", "on"):
        return True
    return shutil.which("nvcc") is not None or os.path.exists("/usr/local/cuda/bin/nvcc")


def build_extension() -> None:
    sys.path.insert(0, str(ROOT))
    try:
        from astrai_b200.ops.build import build

        print("built", build())
    except Exception as exc:  # noqa: BLE001 - a CPU-only install is still useful
        if os.environ.get("ASTRAI_B200_BUILD_EXT", "").strip().lower() in ("1", "true", "yes", "on"):
            raise
        warnings.warn(f"the sm_100a extension was not built ({exc}); CUDA ops will refuse to run until "
                      "`python -m astrai_b200.ops.build` succeeds")
    finally:
        sys.path.pop(0)


class build_py(_build_py):
    def run(self):
        if want_extension():
            build_extension()
        super().run()


def _carries_extension() -> bool:
    return (ROOT / "astrai_b200" / "ops" / "_C.so").exists() or want_extension()


class PlatformDistribution(Distribution):
    """Makes the wheel a platform wheel (files installed as platform-specific) when it carries ``_C.so``."""

    def has_ext_modules(self):
        return _carries_extension()


def _commands():
    commands = {"build_py": build_py}
    try:
        from setuptools.command.bdist_wheel import bdist_wheel as _bdist_wheel
    except ImportError:  # older setuptools: the command lives in the `wheel` package
        try:
            from wheel.bdist_wheel import bdist_wheel as _bdist_wheel
        except ImportError:
            return commands

    class bdist_wheel(_bdist_wheel):
        """A wheel that carries ``_C.so`` is tied to the platform (not to a Python version: the library is loaded with
        ``torch.ops.load_library``, it is not an import module)."""

        def finalize_options(self):
            super().finalize_options()
            if _carries_extension():
                self.root_is_pure = False

        def get_tag(self):
            python, abi, plat = super().get_tag()
            return ("py3", "none", plat) if not self.root_is_pure else (python, abi, plat)

    commands["bdist_wheel"] = bdist_wheel
    return commands


if __name__ == "__main__":
    setup(cmdclass=_commands(), distclass=PlatformDistribution)
