#!/usr/bin/env bash
# Training job control on a Docker host.
#
#   deploy/train.sh COMMAND [CONFIG.yaml] [options]        (CONFIG defaults to ./train.yaml)
#
#   init        create the data / parameter / checkpoint directories named in the config's runtime: section
#   preflight   check docker, the compose file, the directories and (without a checkpoint to resume) the parameters
#   build       build the image
#   start       start or resume training in the background (--foreground keeps the terminal; `-- ARGS` go to the trainer)
#   stop        ask the trainer to stop: SIGTERM -> emergency checkpoint -> exit 0 (compose waits up to 10 minutes)
#   restart     stop, then start
#   logs        follow the trainer's output
#   status      container state and checkpoint summary
#   latest      print the newest complete checkpoint
#   list        print every complete checkpoint, oldest first
#   clean       remove old checkpoints: --keep N (default 3) newest complete ones stay; a preview unless --force
#
# `runtime.max_hours` in the config schedules an automatic `stop`; `runtime.auto_resume: true` makes every start pick up
# the newest complete checkpoint (meta.json, config.json, model.safetensors, optimizer.pt, scheduler.pt all non-empty).
source "$(dirname -- "${BASH_SOURCE[0]}")/lib.sh"

usage() { sed -n '2,19p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; }

cmd=${1:-help}
shift || true
cfg=train.yaml
if [[ $# -gt 0 && "$1" != -* ]]; then cfg=$1; shift; fi

job_name()   { printf '%s\n' "${ASTRAI_CONTAINER:-astrai_b200_train}"; }
ckpt_root()  { printf '%s\n' "${ASTRAI_CKPT_DIR:-${DEPLOY_DIR}/checkpoint}"; }
timer_file() { printf '/tmp/%s.stop-timer.pid\n' "$(job_name)"; }

cancel_timer() {
    local f pid
    f="$(timer_file)"
    [[ -f "$f" ]] || return 0
    pid="$(<"$f")"
    [[ "${pid}" =~ ^[0-9]+$ ]] && kill "${pid}" 2>/dev/null || true
    rm -f -- "$f"
}

arm_timer() {
    [[ -n "${ASTRAI_MAX_HOURS:-}" ]] || return 0
    cancel_timer
    local seconds
    seconds="$(python3 -c "print(int(float('${ASTRAI_MAX_HOURS}') * 3600))")"
    (( seconds > 0 )) || return 0
    ( sleep "${seconds}"; "${BASH_SOURCE[0]}" stop "${CONFIG_PATH}" ) >/dev/null 2>&1 &
    echo $! >"$(timer_file)"
    say "automatic stop in ${seconds} s"
}

do_init() {
    mkdir -p "${ASTRAI_DATA_DIR:-${DEPLOY_DIR}/data}" "${ASTRAI_PARAM_DIR:-${DEPLOY_DIR}/params}" "$(ckpt_root)"
    say "data:        ${ASTRAI_DATA_DIR:-${DEPLOY_DIR}/data}"
    say "parameters:  ${ASTRAI_PARAM_DIR:-${DEPLOY_DIR}/params}"
    say "checkpoints: $(ckpt_root)"
}

do_preflight() {
    need docker
    docker info >/dev/null 2>&1 || fail "the docker daemon does not answer"
    [[ -d "${ASTRAI_DATA_DIR:-${DEPLOY_DIR}/data}" ]] || fail "data directory missing (run: deploy/train.sh init ${cfg})"
    mkdir -p "$(ckpt_root)"
    [[ -w "$(ckpt_root)" ]] || fail "checkpoint directory is not writable: $(ckpt_root)"
    local last
    last="$(latest_checkpoint "$(ckpt_root)")"
    if [[ -n "${last}" && "${ASTRAI_AUTO_RESUME:-0}" == "1" ]]; then
        say "will resume from ${last}"
    else
        local p=${ASTRAI_PARAM_DIR:-${DEPLOY_DIR}/params}
        [[ -s "${p}/config.json" ]] || fail "no model config at ${p}/config.json"
        [[ -s "${p}/model.safetensors" || -s "${p}/model.safetensors.index.json" ]] || fail "no model weights under ${p}"
    fi
    compose config --quiet
    say "preflight passed (GPUs: ${ASTRAI_GPUS:-all}, ranks: ${ASTRAI_NPROCS:-1})"
}

do_start() {
    local foreground=0 extra=()
    while [[ $# -gt 0 ]]; do
        case "$1" in
            --foreground) foreground=1 ;;
            --) shift; extra=("$@"); break ;;
            *) fail "unknown option for start: $1" ;;
        esac
        shift
    done
    do_preflight
    export ASTRAI_TRAIN_ARGS="--config /workspace/astrai_b200/$(realpath --relative-to="${REPO_DIR}" "${CONFIG_PATH}") ${extra[*]:-}"
    arm_timer
    if (( foreground )); then
        compose run --rm --name "$(job_name)" train
    else
        compose run --detach --rm --name "$(job_name)" train >/dev/null
        say "started $(job_name); follow it with: deploy/train.sh logs ${cfg}"
    fi
}

do_stop() {
    cancel_timer
    if docker ps --format '{{.Names}}' | grep -qx "$(job_name)"; then
        say "stopping $(job_name) (it writes a checkpoint first)"
        docker stop --time 600 "$(job_name)" >/dev/null
    else
        say "$(job_name) is not running"
    fi
}

do_status() {
    docker ps --all --filter "name=^$(job_name)$" --format 'container {{.Names}}: {{.Status}}' || true
    local all
    all="$(complete_checkpoints "$(ckpt_root)")"
    say "complete checkpoints: $(printf '%s\n' "${all}" | grep -c . || true)"
    [[ -z "${all}" ]] || say "latest: $(printf '%s\n' "${all}" | tail -n 1)"
}

do_clean() {
    local keep=3 force=0
    while [[ $# -gt 0 ]]; do
        case "$1" in
            --keep) keep=$2; shift ;;
            --force) force=1 ;;
            *) fail "unknown option for clean: $1" ;;
        esac
        shift
    done
    [[ "${keep}" =~ ^[0-9]+$ ]] || fail "--keep takes a number"
    local all victims
    all="$(complete_checkpoints "$(ckpt_root)")"
    victims="$(printf '%s\n' "${all}" | grep . | head -n "-${keep}" || true)"
    if [[ -z "${victims}" ]]; then say "nothing to remove"; return 0; fi
    while IFS= read -r dir; do
        if (( force )); then rm -rf -- "${dir}" "${dir}.shards"; say "removed ${dir}"; else say "would remove ${dir}"; fi
    done <<<"${victims}"
    (( force )) || say "preview only; repeat with --force to delete"
}

case "${cmd}" in
    help|-h|--help) usage; exit 0 ;;
esac
load_runtime train "${cfg}"
case "${cmd}" in
    init) do_init ;;
    preflight) do_preflight ;;
    build) compose build train ;;
    start) do_start "$@" ;;
    stop) do_stop ;;
    restart) do_stop; do_start "$@" ;;
    logs) docker logs --follow "$(job_name)" ;;
    status) do_status ;;
    latest) latest_checkpoint "$(ckpt_root)" ;;
    list) complete_checkpoints "$(ckpt_root)" ;;
    clean) do_clean "$@" ;;
    *) usage >&2; exit 2 ;;
esac
