#!/usr/bin/env bash
# Image helper: deploy/docker.sh {build|shell|test|push|prune} [TAG]
#
#   build   build the image (CUDA >= 12.8 toolchain inside: the sm_100a extension is compiled during the build)
#   shell   an interactive shell in the image with the repository mounted and all GPUs visible
#   test    run the CPU test suite inside the image
#   push    push TAG to its registry
#   prune   remove dangling images left by rebuilds
source "$(dirname -- "${BASH_SOURCE[0]}")/lib.sh"
cmd=${1:-help}
tag=${2:-${ASTRAI_IMAGE:-astrai_b200:latest}}
need docker
case "${cmd}" in
    build) docker build --file "${DEPLOY_DIR}/Dockerfile" --tag "${tag}" "${REPO_DIR}" ;;
    shell) docker run --rm -it --gpus all --shm-size 16g -v "${REPO_DIR}:/workspace/astrai_b200" --entrypoint bash "${tag}" ;;
    test)  docker run --rm --entrypoint python "${tag}" -m pytest tests -x -q -m "not gpu" ;;
    push)  docker push "${tag}" ;;
    prune) docker image prune --force ;;
    *) sed -n '2,8p' "${BASH_SOURCE[0]}" | sed 's/^# \{0,1\}//'; [[ "${cmd}" == help ]] || exit 2 ;;
esac
