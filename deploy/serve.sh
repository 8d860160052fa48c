#!/usr/bin/env bash
# Host wrapper: `deploy/serve.sh cfg.yaml {up|down|logs|status}` for the compose `serve` service.
set -euo pipefail
cfg=${1:?usage: deploy/serve.sh CONFIG.yaml [up|down|logs|status]}
action=${2:-up}
eval "$(python -m astrai_b200.cli.runtime serve "$cfg")"
cd "$(dirname "$0")"
case "$action" in
  up) docker compose up -d serve ;;
  down) docker compose stop serve ;;
  logs) docker compose logs -f serve ;;
  status) docker compose ps serve ;;
  *) echo "unknown action $action" >&2; exit 2 ;;
esac
