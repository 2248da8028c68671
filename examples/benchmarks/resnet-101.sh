#!/bin/bash
# ResNet-101, batch 32, 1 replica per GPU, synchronous SGD (scripts/benchmarks/resnet-101.sh:76-108).
source "$(dirname "$0")/common.sh"
run_train --model resnet101 --gpu true --cpu false --number-of-gpu-models 1 --batch-size "${BATCH:-32}" --wpc "$GPUS" \
  --update-model WORKER --learning-rate 0.1 --momentum 0.9 --weight-decay 0.0001 --learning-rate-decay-policy multistep \
  --step-values 30,60,80 --learning-rate-step-unit epochs --gamma 0.1 --N "${EPOCHS:-90}" --training-unit epochs "$@"
