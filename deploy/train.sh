#!/usr/bin/env bash
# Host wrapper: `deploy/train.sh cfg.yaml [extra train options]` exports the YAML's `runtime:` section and starts the
# compose `train` service; ASTRAI_MAX_HOURS (if set) stops it gracefully after that many hours.
set -euo pipefail
cfg=${1:?usage: deploy/train.sh CONFIG.yaml [train options]}
shift || true
eval "$(python -m astrai_b200.cli.runtime train "$cfg")"
export ASTRAI_TRAIN_ARGS="--config /workspace/astrai_b200/${cfg} $*"
cd "$(dirname "$0")"
if [[ -n "${ASTRAI_MAX_HOURS:-}" ]]; then
  ( sleep "$(python -c "print(int(float('${ASTRAI_MAX_HOURS}') * 3600))")"; docker compose stop train ) &
fi
docker compose run --rm --name "${ASTRAI_CONTAINER:-astrai_b200_train}" train
