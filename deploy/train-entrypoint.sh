#!/usr/bin/env bash
# Container entry point for training: resumes from the newest COMPLETE checkpoint under /checkpoint when
# ASTRAI_AUTO_RESUME=1 (a checkpoint is complete when meta.json, config.json, model.safetensors, optimizer.pt and
# scheduler.pt all exist and are non-empty), otherwise starts from /params.  Extra options: $ASTRAI_TRAIN_ARGS.
set -euo pipefail
param_path=/params
resume=()
if [[ "${ASTRAI_AUTO_RESUME:-0}" == "1" ]]; then
  latest=$(python - <<'PY'
from astrai_b200.serialization import latest_complete
print(latest_complete("/checkpoint") or "")
PY
)
  if [[ -n "$latest" ]]; then
    echo "resuming from $latest"
    param_path="$latest"
    resume=(--resume)
  fi
fi
# shellcheck disable=SC2086
exec python -m astrai_b200.cli.train --param_path "$param_path" --data_root_path /data --ckpt_dir /checkpoint \
  --nprocs "${ASTRAI_NPROCS:-1}" "${resume[@]}" ${ASTRAI_TRAIN_ARGS:-}
