#!/bin/bash
# Shared launcher: 1 GPU runs in-process, G > 1 GPUs through torch.distributed.run (one process per GPU).
HERE="$(cd "$(dirname "${BASH_SOURCE[0]}")" && pwd)"
ROOT="$(cd "$HERE/../.." && pwd)"
GPUS="${GPUS:-1}"
run_train () {
  if [ "$GPUS" -gt 1 ]; then
    python -m torch.distributed.run --nnodes=1 --nproc-per-node "$GPUS" --master-addr 127.0.0.1 "$ROOT/examples/train.py" "$@"
  else
    python "$ROOT/examples/train.py" "$@"
  fi
}
