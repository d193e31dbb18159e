#!/usr/bin/env bash
# Start an interactive container with all GPUs, host IPC and the source tree mounted (counterpart of the reference's
# docker/run.sh).  Usage: docker/run.sh [image] [command...]
set -euo pipefail
cd "$(dirname "$0")/.."
image="${1:-iris_b200:dev}"
shift || true
exec docker run --rm -it --gpus all --ipc=host --shm-size=16g --ulimit memlock=-1 \
  -v "$PWD":/workspace/iris_b200 -w /workspace/iris_b200 "$image" "${@:-bash}"
