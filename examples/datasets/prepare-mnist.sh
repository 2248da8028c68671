#!/bin/bash
# MNIST -> binary partitions (the reference's scripts/datasets/mnist/{download,preprocess,prepare}-mnist.sh).
#   ./prepare-mnist.sh [batch size] [data directory]          output: <data>/mnist/b-NNN/mnist-{train,test}.metadata
# The four idx files are downloaded into <data>/mnist/original unless they are already there (no network: put them there).
set -e
ROOT="$(cd "$(dirname "${BASH_SOURCE[0]}")/../.." && pwd)"
BATCH="${1:-1}"; DATA="${2:-$ROOT/data}"
ORIG="$DATA/mnist/original"; OUT="$(printf "%s/mnist/b-%03d" "$DATA" "$BATCH")"
mkdir -p "$ORIG"
for f in train-images-idx3-ubyte train-labels-idx1-ubyte t10k-images-idx3-ubyte t10k-labels-idx1-ubyte; do
  if [ ! -f "$ORIG/$f" ] && [ ! -f "$ORIG/$f.gz" ]; then
    echo "[Download] $f.gz"
    (cd "$ORIG" && wget --no-check-certificate "https://ossci-datasets.s3.amazonaws.com/mnist/$f.gz") || { echo "error: cannot download $f.gz; place it under $ORIG"; exit 1; }
  fi
done
[ -d "$OUT" ] && { echo "error: $OUT already exists"; exit 1; }
pick () { [ -f "$ORIG/$1" ] && echo "$ORIG/$1" || echo "$ORIG/$1.gz"; }
cd "$ROOT"
python -m crossbow_b200.data.convert mnist --images "$(pick train-images-idx3-ubyte)" --labels "$(pick train-labels-idx1-ubyte)" -o "$OUT" --name mnist-train -b "$BATCH"
python -m crossbow_b200.data.convert mnist --images "$(pick t10k-images-idx3-ubyte)" --labels "$(pick t10k-labels-idx1-ubyte)" -o "$OUT" --name mnist-test -b "$BATCH"
echo "Bye."
