#!/bin/bash
# ResNet-50 / ImageNet-shaped workload (scripts/benchmarks/resnet-50.sh:71-146): batch 16, 2 replicas per GPU, SMA
# alpha 0.1, lr 0.1, momentum 0.9, wd 1e-4, steps 30,60,80 epochs.  The reference sets wpc = k*G*1e6 (effectively never
# synchronising within a run); here wpc = replicas x GPUs (the work per clock counts the tasks of the whole job), i.e. every replica synchronises after each of its tasks.
source "$(dirname "$0")/common.sh"
REPLICAS="${REPLICAS:-2}"; BATCH="${BATCH:-16}"; EPOCHS="${EPOCHS:-90}"
run_train --model resnet50 --gpu true --cpu false --number-of-gpu-models "$REPLICAS" --batch-size "$BATCH" \
  --wpc "$((REPLICAS * GPUS))" --update-model SMA --alpha 0.1 --learning-rate 0.1 --momentum 0.9 --weight-decay 0.0001 \
  --learning-rate-decay-policy multistep --step-values 30,60,80 --learning-rate-step-unit epochs --gamma 0.1 \
  --reuse-memory true --number-of-task-handlers 8 --number-of-callback-handlers 8 --display-interval 100 \
  --N "$EPOCHS" --training-unit epochs "$@"
