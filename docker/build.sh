#!/usr/bin/env bash
# Build the development image (counterpart of the reference's docker/build.sh).
set -euo pipefail
cd "$(dirname "$0")/.."
docker build -f docker/Dockerfile -t "${1:-iris_b200:dev}" .
