"""Host-side ``runtime:`` sections of the YAML configs, turned into shell exports for container wrappers.

A training or serving YAML may carry a ``runtime:`` mapping that the Python entry points ignore and the launch scripts
read.  ``python -m astrai_b200.cli.runtime train cfg.yaml`` prints ``export KEY=value`` lines; with a third argument
``environment`` it prints the ``runtime.environment`` mapping as NUL-separated ``NAME=value`` records (for ``env -0``
style consumers).  Two spellings of the section are understood:

* flat keys (``image``, ``gpus``, ``data_dir``, ``param_dir``, ``ckpt_dir``, ``shm_size``, ``auto_resume``, ``max_hours``,
  ``container_name``, ``nprocs`` for training; ``image``, ``gpus``, ``param_dir``, ``port``, ``container_name``,
  ``restart``, ``shm_size`` for serving);
* the nested layout of the reference's YAML files (``job_name``, ``port``, ``paths: {data, model, checkpoints | param}``,
  ``gpu: {enabled, devices, parallel_mode}``, ``container: {max_duration_hours, ipc, ...}``, ``environment: {...}``), with
  the reference's consistency rules (``scripts/tools/train_runtime.py:32-152``, ``serve_runtime.py:45-154``): a port is
  1..65535, ``gpu.devices`` is ``all`` or a list of distinct non-negative integers (exactly one for serving, whose engine
  is single-GPU), a disabled GPU needs ``server.device: cpu``, the parallel mode must fit the device count, relative
  paths are resolved against the config file.

Both spellings end up in the same ``ASTRAI_*`` variables, so one set of wrappers serves either.
"""

from __future__ import annotations

import math
import re
import shlex
import sys
from pathlib import Path
from typing import Any, Dict, List, Optional

from astrai_b200.cli.common import load_yaml

TRAIN_KEYS = {"image": "ASTRAI_IMAGE", "gpus": "ASTRAI_GPUS", "data_dir": "ASTRAI_DATA_DIR", "param_dir": "ASTRAI_PARAM_DIR",
              "ckpt_dir": "ASTRAI_CKPT_DIR", "shm_size": "ASTRAI_SHM_SIZE", "auto_resume": "ASTRAI_AUTO_RESUME",
              "max_hours": "ASTRAI_MAX_HOURS", "container_name": "ASTRAI_CONTAINER", "nprocs": "ASTRAI_NPROCS"}
SERVE_KEYS = {"image": "ASTRAI_IMAGE", "gpus": "ASTRAI_GPUS", "param_dir": "ASTRAI_PARAM_DIR", "port": "ASTRAI_PORT",
              "container_name": "ASTRAI_CONTAINER", "restart": "ASTRAI_RESTART", "shm_size": "ASTRAI_SHM_SIZE"}
NESTED_SECTIONS = ("paths", "gpu", "container", "environment", "job_name")
NAME = re.compile(r"[A-Za-z0-9][A-Za-z0-9._-]*")
ENV_NAME = re.compile(r"[A-Za-z_][A-Za-z0-9_]*")
# what a parallel mode needs from the number of visible devices
MIN_DEVICES = {"auto": 1, "none": 1, "ddp": 2, "fsdp": 2, "tp": 2, "cp": 2, "ep": 2}


def _render(value: Any) -> str:
    if isinstance(value, bool):
        return "1" if value else "0"
    if isinstance(value, (list, tuple)):
        return ",".join(str(v) for v in value)
    return str(value)


def _section(parent: Dict[str, Any], key: str) -> Dict[str, Any]:
    value = parent.get(key)
    if value is None:
        return {}
    if not isinstance(value, dict):
        raise ValueError(f"runtime.{key} must be a mapping")
    return value


def _port(value: Any, where: str) -> int:
    if isinstance(value, bool) or not isinstance(value, int):
        raise ValueError(f"{where} must be an integer")
    if not 1 <= value <= 65535:
        raise ValueError(f"{where} must be between 1 and 65535")
    return value


def _devices(gpu: Dict[str, Any]) -> Optional[List[str]]:
    """``None`` for "all", else the device ids as strings."""
    devices = gpu.get("devices", "all")
    if devices == "all":
        return None
    if not isinstance(devices, list) or not devices:
        raise ValueError("runtime.gpu.devices must be 'all' or a non-empty list such as [0, 1]")
    ids = [str(d) for d in devices]
    if not all(i.isdigit() for i in ids):
        raise ValueError("runtime.gpu.devices entries must be non-negative integers")
    if len(set(ids)) != len(ids):
        raise ValueError("runtime.gpu.devices must not contain duplicates")
    return ids


def _resolved(value: Any, what: str, base: Optional[Path]) -> str:
    if not isinstance(value, str) or not value.strip():
        raise ValueError(f"runtime.paths.{what} is required")
    path = Path(value).expanduser()
    if not path.is_absolute() and base is not None:
        path = base / path
    return str(path.resolve()) if base is not None else str(path)


def _job_name(runtime: Dict[str, Any], required: bool) -> Optional[str]:
    name = runtime.get("job_name")
    if name in (None, "") and not required:
        return None
    if not isinstance(name, str) or not NAME.fullmatch(name):
        raise ValueError("runtime.job_name must use letters, numbers, dot, underscore, or dash")
    return name


def environment_of(config: Dict[str, Any]) -> Dict[str, str]:
    """``runtime.environment`` as strings (``None`` becomes the empty string); names and values are checked."""
    runtime = config.get("runtime") or {}
    env = _section(runtime, "environment") if isinstance(runtime, dict) else {}
    out: Dict[str, str] = {}
    for name, value in env.items():
        if not isinstance(name, str) or not ENV_NAME.fullmatch(name):
            raise ValueError(f"invalid runtime.environment name: {name!r}")
        if value is not None and not isinstance(value, (str, int, float, bool)):
            raise ValueError(f"runtime.environment.{name} must be a scalar")
        out[name] = "" if value is None else str(value)
    return out


def _nested(kind: str, config: Dict[str, Any], base: Optional[Path]) -> Dict[str, Any]:
    """The reference's nested ``runtime:`` layout as this package's flat keys."""
    runtime = config["runtime"]
    paths, gpu, container = _section(runtime, "paths"), _section(runtime, "gpu"), _section(runtime, "container")
    environment_of(config)  # validated here, printed by the `environment` command
    known = set(NESTED_SECTIONS) | {"port", "image"}
    unknown = sorted(set(runtime) - known)
    if unknown:
        raise ValueError(f"unknown runtime key(s): {', '.join(unknown)}")
    flat: Dict[str, Any] = {}
    if runtime.get("image") is not None:
        flat["image"] = runtime["image"]
    ids = _devices(gpu)
    if kind == "train":
        flat["container_name"] = _job_name(runtime, required=True)
        flat["data_dir"] = _resolved(paths.get("data"), "data", base)
        flat["param_dir"] = _resolved(paths.get("model"), "model", base)
        flat["ckpt_dir"] = _resolved(paths.get("checkpoints"), "checkpoints", base)
        mode = str(gpu.get("parallel_mode", "auto"))
        if mode not in MIN_DEVICES:
            raise ValueError(f"runtime.gpu.parallel_mode must be one of {', '.join(MIN_DEVICES)}")
        if ids is not None:
            if mode == "none" and len(ids) != 1:
                raise ValueError("parallel_mode none requires exactly one GPU")
            if len(ids) < MIN_DEVICES[mode]:
                raise ValueError(f"parallel_mode {mode} requires at least two GPUs")
            flat["gpus"], flat["nprocs"] = ids, len(ids)
        hours = container.get("max_duration_hours", 0)
        try:
            hours = float(hours) if hours else 0.0
        except (TypeError, ValueError):
            raise ValueError("runtime.container.max_duration_hours must be a number") from None
        if hours < 0 or math.isnan(hours):
            raise ValueError("runtime.container.max_duration_hours must not be negative")
        if hours:
            flat["max_hours"] = hours
        if "shm_size" in container:
            flat["shm_size"] = container["shm_size"]
        return flat
    name = _job_name(runtime, required=False)
    if name:
        flat["container_name"] = name
    flat["port"] = _port(runtime.get("port", 8000), "runtime.port")
    server = config.get("server") or {}
    if not isinstance(server, dict):
        raise ValueError("server must be a mapping")
    if "port" in server:
        _port(server["port"], "server.port")
    device = server.get("device", "cuda")
    if not isinstance(device, str) or not device.strip():
        raise ValueError("server.device must be a string")
    enabled = gpu.get("enabled", True)
    if not isinstance(enabled, bool):
        raise ValueError("runtime.gpu.enabled must be a boolean")
    if enabled:
        if ids is not None:
            if len(ids) != 1:
                raise ValueError("runtime.gpu.devices must be 'all' or a single-device list such as [0]")
            flat["gpus"] = ids
    else:
        if ids is not None:
            raise ValueError("runtime.gpu.devices is ignored when runtime.gpu.enabled is false")
        if device != "cpu":
            raise ValueError("server.device must be 'cpu' when runtime.gpu.enabled is false")
        flat["gpus"] = "none"
    flat["param_dir"] = _resolved(paths.get("param", "./params"), "param", base)
    if "restart" in container:
        flat["restart"] = container["restart"]
    return flat


def exports(kind: str, config: Dict[str, Any], config_dir: Optional[Path] = None) -> List[str]:
    table = TRAIN_KEYS if kind == "train" else SERVE_KEYS
    runtime = config.get("runtime") or {}
    if not isinstance(runtime, dict):
        raise ValueError("runtime: must be a mapping")
    if any(k in runtime for k in NESTED_SECTIONS):
        runtime = _nested(kind, config, config_dir)
    else:
        unknown = sorted(set(runtime) - set(table))
        if unknown:
            raise ValueError(f"unknown runtime key(s): {', '.join(unknown)}")
        if runtime.get("port") is not None:
            _port(runtime["port"], "runtime.port")
    return [f"export {table[k]}={shlex.quote(_render(v))}" for k, v in runtime.items() if v is not None and k in table]


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) not in (2, 3) or argv[0] not in ("train", "serve") or (len(argv) == 3 and argv[2] not in ("exports", "environment")):
        print("usage: python -m astrai_b200.cli.runtime {train|serve} CONFIG.yaml [exports|environment]", file=sys.stderr)
        return 2
    try:
        config = load_yaml(argv[1])
        if len(argv) == 3 and argv[2] == "environment":
            for name, value in environment_of(config).items():
                sys.stdout.write(f"{name}={value}\0")
            return 0
        for line in exports(argv[0], config, Path(argv[1]).resolve().parent):
            print(line)
    except (ValueError, OSError) as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
