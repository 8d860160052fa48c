"""Host-side ``runtime:`` sections of the YAML configs, turned into shell exports for container wrappers.

A training or serving YAML may carry a ``runtime:`` mapping (image, GPUs, mounts, restart policy ...) that the
Python entry points ignore and the launch scripts read.  ``python -m astrai_b200.cli.runtime train cfg.yaml`` prints
``export KEY=value`` lines - the role of ``scripts/tools/train_runtime.py:32-152`` and ``serve_runtime.py:45-154`` in
the reference.
"""

from __future__ import annotations

import shlex
import sys
from typing import Any, Dict, List

from astrai_b200.cli.common import load_yaml

TRAIN_KEYS = {"image": "ASTRAI_IMAGE", "gpus": "ASTRAI_GPUS", "data_dir": "ASTRAI_DATA_DIR", "param_dir": "ASTRAI_PARAM_DIR",
              "ckpt_dir": "ASTRAI_CKPT_DIR", "shm_size": "ASTRAI_SHM_SIZE", "auto_resume": "ASTRAI_AUTO_RESUME",
              "max_hours": "ASTRAI_MAX_HOURS", "container_name": "ASTRAI_CONTAINER", "nprocs": "ASTRAI_NPROCS"}
SERVE_KEYS = {"image": "ASTRAI_IMAGE", "gpus": "ASTRAI_GPUS", "param_dir": "ASTRAI_PARAM_DIR", "port": "ASTRAI_PORT",
              "container_name": "ASTRAI_CONTAINER", "restart": "ASTRAI_RESTART", "shm_size": "ASTRAI_SHM_SIZE"}


def _render(value: Any) -> str:
    if isinstance(value, bool):
        return "1" if value else "0"
    if isinstance(value, (list, tuple)):
        return ",".join(str(v) for v in value)
    return str(value)


def exports(kind: str, config: Dict[str, Any]) -> List[str]:
    table = TRAIN_KEYS if kind == "train" else SERVE_KEYS
    runtime = config.get("runtime") or {}
    if not isinstance(runtime, dict):
        raise ValueError("runtime: must be a mapping")
    unknown = sorted(set(runtime) - set(table))
    if unknown:
        raise ValueError(f"unknown runtime key(s): {', '.join(unknown)}")
    return [f"export {table[k]}={shlex.quote(_render(v))}" for k, v in runtime.items() if v is not None]


def main(argv=None) -> int:
    argv = list(sys.argv[1:] if argv is None else argv)
    if len(argv) != 2 or argv[0] not in ("train", "serve"):
        print("usage: python -m astrai_b200.cli.runtime {train|serve} CONFIG.yaml", file=sys.stderr)
        return 2
    try:
        for line in exports(argv[0], load_yaml(argv[1])):
            print(line)
    except ValueError as exc:
        print(f"error: {exc}", file=sys.stderr)
        return 1
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
