#!/bin/bash
# ImageNet TFRecords -> record files of JPEGs for the decoding data set (the reference's scripts/datasets/imagenet/
# prepare-imagenet.sh + parse-records.py; no TensorFlow needed here).
#   ./prepare-imagenet.sh <input directory with train-*-of-* and validation-*-of-*> <output directory>
set -e
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
if [ $# -ne 2 ]; then
  echo "usage: prepare-imagenet.sh [input directory] [output directory]"
  exit 1
fi
cd "$ROOT"
python -m crossbow_b200.data.convert imagenet --subset train      --input "$1/train-*-of-*"      -o "$2"
python -m crossbow_b200.data.convert imagenet --subset validation --input "$1/validation-*-of-*" -o "$2"
