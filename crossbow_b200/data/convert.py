"""Converters from the public data-set files to the binary partition format (``DatasetWriter``): what the reference's
pre-processing encoders do (src/test/java/.../preprocess/{mnist/MNISTEncoder.java, cifar/CifarEncoder.java,
ratings/RatingsEncoder.java, yahoomusic/YahooMusicEncoder.java, random/RandomEncoder.java}).

    python -m crossbow_b200.data.convert mnist   --images train-images-idx3-ubyte --labels train-labels-idx1-ubyte -o out --name mnist-train -b 128
    python -m crossbow_b200.data.convert cifar10 --input data_batch_1.bin data_batch_2.bin ... -o out --name cifar-train -b 64
    python -m crossbow_b200.data.convert ratings --input ratings.txt -o out --name ratings-train -b 1024
    python -m crossbow_b200.data.convert random  --shape 3,32,32 --classes 10 --count 1024 -o out --name random-train -b 64
    python -m crossbow_b200.data.convert imagenet --input 'train-*-of-*' --subset train -o out     (TFRecords -> record files,
        scripts/datasets/imagenet/parse-records.py; see tfrecords.py)

Pixel handling follows the reference: MNIST pixels are scaled by 1/256 (its default ``-s 0.00390625``), CIFAR pixels go to
[-1, 1] (``p / 127.5 - 1``) and the mean image of the converted set is written beside it (``<name>.mean``, raw fp32) for
the DataTransform operator.  An incomplete last batch is completed by the writer with examples from the start of the set.
"""
from __future__ import annotations

import argparse
import gzip
import os
import struct
from typing import Iterable, Optional, Sequence

import numpy as np

from .native import DatasetWriter


def _open(path):
    return gzip.open(path, "rb") if str(path).endswith(".gz") else open(path, "rb")


def _write(directory, name, shape, batch, examples: np.ndarray, labels: np.ndarray, partition_bytes=None) -> str:
    n = len(examples)
    w = DatasetWriter(directory, name, shape, batch, partition_bytes=partition_bytes)
    step = max(batch, (4096 // batch) * batch)
    for i in range(0, n, step):
        j = min(n, i + step)
        w.append(examples[i:j], labels[i:j])
    return w.close()


def convert_mnist(images: str, labels: str, directory: str, name: str, batch: int, scale: float = 0.00390625) -> str:
    """IDX files (magic 2051 / 2049, big-endian header) -> [1, H, W] fp32 examples scaled by `scale`, int32 labels."""
    with _open(images) as f:
        magic, count, h, w = struct.unpack(">iiii", f.read(16))
        if magic != 2051:
            raise ValueError("error: invalid magic number in the image file")
        px = np.frombuffer(f.read(count * h * w), dtype=np.uint8).reshape(count, 1, h, w)
    with _open(labels) as f:
        magic, lcount = struct.unpack(">ii", f.read(8))
        if magic != 2049:
            raise ValueError("error: invalid magic number in the label file")
        lab = np.frombuffer(f.read(lcount), dtype=np.uint8)
    if lcount != count:
        raise ValueError("error: image and label counts differ")
    return _write(directory, name, (1, h, w), batch, px.astype(np.float32) * np.float32(scale), lab.astype(np.int32))


def _convert_cifar(files: Iterable[str], directory, name, batch, label_bytes, label_index) -> str:
    rec = label_bytes + 3072
    raw = np.concatenate([np.frombuffer(_open(p).read(), dtype=np.uint8) for p in files])
    if raw.size % rec:
        raise ValueError("error: the input is not a whole number of CIFAR records")
    raw = raw.reshape(-1, rec)
    lab = raw[:, label_index].astype(np.int32)
    px = raw[:, label_bytes:].reshape(-1, 3, 32, 32).astype(np.float32) / np.float32(127.5) - np.float32(1.0)
    meta = _write(directory, name, (3, 32, 32), batch, px, lab)
    px.mean(axis=0, dtype=np.float64).astype(np.float32).tofile(os.path.join(directory, f"{name}.mean"))
    return meta


def convert_cifar10(files: Sequence[str], directory: str, name: str, batch: int) -> str:
    """CIFAR-10 binary batches: 1 label byte + 3072 pixel bytes (channel-major) per record."""
    return _convert_cifar(files, directory, name, batch, 1, 0)


def convert_cifar100(files: Sequence[str], directory: str, name: str, batch: int, coarse: bool = False) -> str:
    """CIFAR-100 binary files: coarse label byte, fine label byte, 3072 pixel bytes."""
    return _convert_cifar(files, directory, name, batch, 2, 0 if coarse else 1)


def convert_ratings(path: str, directory: str, name: str, batch: int) -> str:
    """Lines "row column rating" -> examples [row, column] (as fp32 indices), labels = rating (integer stars), the input of
    the matrix-factorisation model."""
    rows = []
    with _open(path) as f:
        for line in f:
            parts = line.split()
            if len(parts) >= 3:
                rows.append((float(parts[0]), float(parts[1]), float(parts[2])))
    a = np.asarray(rows, dtype=np.float32).reshape(-1, 3)
    return _write(directory, name, (2,), batch, a[:, :2].copy(), np.rint(a[:, 2]).astype(np.int32))


def convert_random(shape: Sequence[int], classes: int, count: int, directory: str, name: str, batch: int, seed: int = 0) -> str:
    """Normal(0, 1) examples and uniform labels (random/RandomEncoder.java, used by the benchmark scripts without data)."""
    g = np.random.default_rng(seed)
    return _write(directory, name, tuple(shape), batch, g.standard_normal((count, *shape), dtype=np.float32),
                  g.integers(0, classes, size=count, dtype=np.int32))


def main(argv: Optional[Sequence[str]] = None) -> int:
    ap = argparse.ArgumentParser(description="convert public data-set files to binary partitions")
    ap.add_argument("kind", choices=["mnist", "cifar10", "cifar100", "ratings", "yahoomusic", "random", "imagenet"])
    ap.add_argument("--images"), ap.add_argument("--labels")
    ap.add_argument("--input", nargs="*", default=[])
    ap.add_argument("-o", "--output", required=True)
    ap.add_argument("--name", default=None)
    ap.add_argument("-b", "--batch", type=int, default=0, help="examples per batch (every kind but imagenet: record files hold single images)")
    ap.add_argument("--subset", default="train", help="imagenet: train or validation (part of the output file names)")
    ap.add_argument("--records-per-file", type=int, default=2048)
    ap.add_argument("--scale", type=float, default=0.00390625)
    ap.add_argument("--coarse", action="store_true")
    ap.add_argument("--shape", default="3,32,32"), ap.add_argument("--classes", type=int, default=10)
    ap.add_argument("--count", type=int, default=1024), ap.add_argument("--seed", type=int, default=0)
    a = ap.parse_args(argv)
    if a.kind == "imagenet":
        from .tfrecords import convert_imagenet
        for path in convert_imagenet(a.input, a.output, a.subset, a.records_per_file):
            print(path)
        return 0
    if a.batch <= 0 or not a.name:
        ap.error("--batch and --name are required")
    if a.kind == "mnist":
        meta = convert_mnist(a.images, a.labels, a.output, a.name, a.batch, a.scale)
    elif a.kind == "cifar10":
        meta = convert_cifar10(a.input, a.output, a.name, a.batch)
    elif a.kind == "cifar100":
        meta = convert_cifar100(a.input, a.output, a.name, a.batch, a.coarse)
    elif a.kind in ("ratings", "yahoomusic"):           # the same "row column rating" lines (yahoomusic/YahooMusicEncoder.java:47-56)
        meta = convert_ratings(a.input[0], a.output, a.name, a.batch)
    else:
        meta = convert_random([int(v) for v in a.shape.split(",")], a.classes, a.count, a.output, a.name, a.batch, a.seed)
    print(meta)
    return 0


if __name__ == "__main__":
    raise SystemExit(main())
