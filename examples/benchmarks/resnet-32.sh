#!/bin/bash
# ResNet-32 / CIFAR-10 workload of the reference (scripts/benchmarks/resnet-32.sh:75-173): SMA alpha 0.1, lr 0.1,
# momentum 0.9, weight decay 1e-4, multistep 80,120 epochs x0.1, wpc = replicas x GPUs, direct scheduling.
source "$(dirname "$0")/common.sh"
REPLICAS="${REPLICAS:-1}"; BATCH="${BATCH:-512}"; EPOCHS="${EPOCHS:-140}"
run_train --model resnet32 --gpu true --cpu false --number-of-gpu-models "$REPLICAS" --batch-size "$BATCH" \
  --wpc "$((REPLICAS * GPUS))" --update-model SMA --alpha 0.1 --learning-rate 0.1 --momentum 0.9 --weight-decay 0.0001 \
  --learning-rate-decay-policy multistep --step-values 80,120 --learning-rate-step-unit epochs --gamma 0.1 \
  --direct-scheduling true --number-of-task-handlers 8 --number-of-callback-handlers 8 --display-interval 100 \
  --N "$EPOCHS" --training-unit epochs "$@"
