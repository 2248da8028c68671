#!/bin/bash
# CIFAR-10 -> binary partitions (the reference's scripts/datasets/cifar-10/{download,preprocess,prepare}-cifar-10.sh).
#   ./prepare-cifar-10.sh [batch size] [data directory]       output: <data>/cifar-10/b-NNN/cifar-{train,test}.metadata (+ mean image)
# cifar-10-binary.tar.gz is downloaded and unpacked into <data>/cifar-10/original unless the batches are already there.
set -e
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
BATCH="${1:-1}"; DATA="${2:-$ROOT/data}"
ORIG="$DATA/cifar-10/original"; OUT="$(printf "%s/cifar-10/b-%03d" "$DATA" "$BATCH")"
if [ ! -f "$ORIG/data_batch_1.bin" ]; then
  mkdir -p "$DATA/cifar-10"
  echo "[Download]"
  (cd "$DATA/cifar-10" && { [ -f cifar-10-binary.tar.gz ] || wget --no-check-certificate https://www.cs.toronto.edu/~kriz/cifar-10-binary.tar.gz; }) \
    || { echo "error: cannot download cifar-10-binary.tar.gz; unpack it to $ORIG"; exit 1; }
  echo "[Untar]"
  (cd "$DATA/cifar-10" && tar zxf cifar-10-binary.tar.gz && mv cifar-10-batches-bin original)
fi
[ -d "$OUT" ] && { echo "error: $OUT already exists"; exit 1; }
cd "$ROOT"
python -m crossbow_b200.data.convert cifar10 --input "$ORIG"/data_batch_{1,2,3,4,5}.bin -o "$OUT" --name cifar-train -b "$BATCH"
python -m crossbow_b200.data.convert cifar10 --input "$ORIG/test_batch.bin" -o "$OUT" --name cifar-test -b "$BATCH"
echo "Bye."
