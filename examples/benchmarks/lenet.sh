#!/bin/bash
# LeNet / MNIST (scripts/benchmarks/lenet.sh:67-103): batch 1, lr 0.001, 100 epochs.
source "$(dirname "$0")/common.sh"
run_train --model lenet --gpu "${GPU:-true}" --cpu false --number-of-gpu-models 1 --batch-size "${BATCH:-1}" --wpc 1 \
  --update-model DEFAULT --learning-rate 0.001 --learning-rate-decay-policy fixed --N "${EPOCHS:-100}" --training-unit epochs "$@"
