#!/usr/bin/env bash
# Helpers shared by the host wrappers (train.sh, serve.sh, docker.sh): messages, YAML runtime exports, compose call,
# and the checkpoint queries that the wrappers and the container entry point agree on.
set -euo pipefail

DEPLOY_DIR="$(cd -- "$(dirname -- "${BASH_SOURCE[0]}")" && pwd)"
REPO_DIR="$(dirname -- "${DEPLOY_DIR}")"

say()  { printf '[astrai_b200] %s\n' "$*"; }
fail() { printf '[astrai_b200] error: %s\n' "$*" >&2; exit 1; }
need() { command -v "$1" >/dev/null 2>&1 || fail "'$1' is not on PATH"; }

# load_runtime KIND CONFIG: export the `runtime:` section of a YAML file (ASTRAI_* variables)
load_runtime() {
    local kind=$1 cfg=$2
    [[ -f "${cfg}" ]] || fail "config not found: ${cfg}"
    need python3
    local lines
    lines="$(cd "${REPO_DIR}" && python3 -m astrai_b200.cli.runtime "${kind}" "${cfg}")" || fail "cannot read runtime: section of ${cfg}"
    eval "${lines}"
    CONFIG_PATH="$(cd "$(dirname "${cfg}")" && pwd)/$(basename "${cfg}")"
}

compose() { (cd "${DEPLOY_DIR}" && docker compose "$@"); }

# complete_checkpoints DIR: every checkpoint directory that a resume can use, oldest first
complete_checkpoints() {
    local root=$1
    [[ -d "${root}" ]] || return 0
    (cd "${REPO_DIR}" && python3 - "${root}" <<'PY'
import sys
from pathlib import Path
from astrai_b200.serialization import is_complete

def key(p):
    parts = p.name.split("_")
    try:
        return int(parts[1]), int(parts[3])
    except (IndexError, ValueError):
        return (-1, -1)

for d in sorted((p for p in Path(sys.argv[1]).iterdir() if p.is_dir() and p.name.startswith("epoch_")), key=key):
    if is_complete(d):
        print(d)
PY
    )
}

latest_checkpoint() { complete_checkpoints "$1" | tail -n 1; }
