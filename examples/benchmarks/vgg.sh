#!/bin/bash
# VGG-16 / CIFAR-10 (scripts/benchmarks/vgg.sh:68-102): batch 256, synchronous EAMSGD (= the SMA code path) alpha 0.2,
# lr halved every 20 epochs, weight decay 5e-4, 250 epochs.
source "$(dirname "$0")/common.sh"
run_train --model vgg16 --gpu true --cpu false --number-of-gpu-models "${REPLICAS:-1}" --batch-size "${BATCH:-256}" \
  --wpc "$(( ${REPLICAS:-1} * GPUS ))" --update-model SYNCHRONOUSEAMSGD --alpha 0.2 --learning-rate 0.1 --momentum 0.9 --weight-decay 0.0005 \
  --learning-rate-decay-policy step --step-size 20 --learning-rate-step-unit epochs --gamma 0.5 \
  --N "${EPOCHS:-250}" --training-unit epochs "$@"
