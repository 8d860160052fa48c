"""Packaging metadata: every console script resolves, the version is the package's, the extension build switch works."""

import importlib
import importlib.util
import os
import subprocess
import sys
import tomllib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _pyproject():
    with open(os.path.join(ROOT, "pyproject.toml"), "rb") as fh:
        return tomllib.load(fh)


def test_console_scripts_resolve_to_callables():
    scripts = _pyproject()["project"]["scripts"]
    assert {"astrai-b200-train", "astrai-b200-serve", "astrai-b200-generate", "astrai-b200-preprocess", "astrai-b200-benchmark",
            "astrai-b200-build"} <= set(scripts)
    for name, target in scripts.items():
        module, attr = target.split(":")
        assert callable(getattr(importlib.import_module(module), attr)), name


def test_version_and_name_come_from_the_package():
    import astrai_b200

    out = subprocess.run([sys.executable, "setup.py", "--name", "--version"], cwd=ROOT, capture_output=True, text=True, timeout=120)
    assert out.returncode == 0, out.stderr[-2000:]
    assert out.stdout.split()[-2:] == ["astrai_b200", astrai_b200.__version__]


def test_dependencies_cover_what_the_package_imports_at_the_top_level():
    deps = {d.split(">")[0].split("=")[0].split("[")[0].strip().replace("-", "_").lower() for d in _pyproject()["project"]["dependencies"]}
    assert {"torch", "tokenizers", "safetensors", "pydantic", "fastapi", "click", "pyyaml", "jinja2"} <= deps


def test_extension_build_switch(monkeypatch):
    spec = importlib.util.spec_from_file_location("_setup_under_test", os.path.join(ROOT, "setup.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)  # guarded by __main__: nothing is set up
    monkeypatch.setenv("ASTRAI_B200_BUILD_EXT", "0")
    assert mod.want_extension() is False
    monkeypatch.setenv("ASTRAI_B200_BUILD_EXT", "1")
    assert mod.want_extension() is True


def test_build_tool_rejects_unknown_options(capsys):
    from astrai_b200.ops import build

    assert build.main(["--bogus"]) == 2
    assert "usage:" in capsys.readouterr().err
