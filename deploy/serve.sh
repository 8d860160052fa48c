#!/usr/bin/env bash
# Serving control on a Docker host.
#
#   deploy/serve.sh COMMAND [CONFIG.yaml]                   (CONFIG defaults to ./serve.yaml)
#
#   preflight   check docker, the compose file and the parameter directory (config.json, weights, tokenizer.json)
#   build       build the image
#   up          start the OpenAI / Anthropic compatible server in the background and wait until GET /health answers
#   down        stop it
#   restart     down, then up
#   logs        follow its output
#   status      container state, /health and the queue / latency counters of /stats
#   smoke       one short chat completion against the running server
source "$(dirname -- "${BASH_SOURCE[0]}")/lib.sh"

usage() { sed -n '2,13p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; }

cmd=${1:-help}
shift || true
cfg=serve.yaml
if [[ $# -gt 0 && "$1" != -* ]]; then cfg=$1; shift; fi
case "${cmd}" in help|-h|--help) usage; exit 0 ;; esac
load_runtime serve "${cfg}"
base="http://127.0.0.1:${ASTRAI_PORT:-8000}"

preflight() {
    need docker
    docker info >/dev/null 2>&1 || fail "the docker daemon does not answer"
    local p=${ASTRAI_PARAM_DIR:-${DEPLOY_DIR}/params}
    for f in config.json tokenizer.json; do [[ -s "${p}/${f}" ]] || fail "missing ${p}/${f}"; done
    [[ -s "${p}/model.safetensors" || -s "${p}/model.safetensors.index.json" ]] || fail "no model weights under ${p}"
    compose config --quiet
    say "preflight passed (GPU ${ASTRAI_GPUS:-0}, port ${ASTRAI_PORT:-8000})"
}

wait_healthy() {
    need curl
    local deadline=$(( $(date +%s) + ${ASTRAI_START_TIMEOUT:-600} ))
    until curl -fsS "${base}/health" 2>/dev/null | grep -q '"model_loaded": *true'; do
        (( $(date +%s) < deadline )) || fail "the server did not become healthy in time (see: deploy/serve.sh logs ${cfg})"
        sleep 2
    done
    say "serving at ${base}"
}

case "${cmd}" in
    preflight) preflight ;;
    build) compose build serve ;;
    up) preflight; compose up --detach serve; wait_healthy ;;
    down) compose stop serve ;;
    restart) compose stop serve; preflight; compose up --detach serve; wait_healthy ;;
    logs) compose logs --follow serve ;;
    status)
        compose ps serve
        need curl
        curl -fsS "${base}/health" || say "/health does not answer"
        echo
        curl -fsS "${base}/stats" || true
        echo ;;
    smoke)
        need curl
        curl -fsS "${base}/v1/chat/completions" -H 'content-type: application/json' \
             -d '{"messages": [{"role": "user", "content": "Say hello."}], "max_tokens": 16, "temperature": 0}'
        echo ;;
    *) usage >&2; exit 2 ;;
esac
