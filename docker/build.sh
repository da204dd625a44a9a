#!/usr/bin/env bash
# Build the container image (CUDA 12.9 toolchain + PyTorch, kernels compiled for sm_100a at build time).
#   docker/build.sh [image-tag]
set -euo pipefail
cd "$(dirname "$0")/.."
docker build -t "${1:-ironcore-b200:latest}" -f Dockerfile .
