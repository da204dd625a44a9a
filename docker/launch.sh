#!/usr/bin/env bash
# Run a command of the framework inside the container with all GPUs of the host.
#   docker/launch.sh train --config configs/baseline_llama7b_tp8.yaml        (one process, one GPU)
#   NPROC=8 docker/launch.sh train --config configs/baseline_llama7b_tp8.yaml
set -euo pipefail
IMAGE="${IMAGE:-ironcore-b200:latest}"
NPROC="${NPROC:-1}"
DATA_DIR="${DATASET_DIR:-$PWD/data}"
if [ "$NPROC" -gt 1 ]; then
  ENTRY=(python -m torch.distributed.run --nnodes=1 --nproc-per-node "$NPROC" --master-addr 127.0.0.1 -m ironcore_b200)
else
  ENTRY=(python -m ironcore_b200)
fi
exec docker run --rm --gpus all --ipc=host --ulimit memlock=-1 --ulimit stack=67108864 \
  -v "$DATA_DIR":/workspace/data -e DATASET_DIR=/workspace/data \
  --entrypoint "${ENTRY[0]}" "$IMAGE" "${ENTRY[@]:1}" "$@"
