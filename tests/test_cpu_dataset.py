"""C++ data-set pipeline on the host: writer -> partition files + metadata, mapped sliding window, slot ring, and the
native scheduler pulling batches straight from the ring."""
import os

import numpy as np
import pytest
import torch

from crossbow_b200.data.native import BasicDataset, DatasetWriter, LightDataset
from crossbow_b200.runtime import Runtime


def _write(tmp_path, n=70, batch=8, shape=(3, 5, 5), partition_bytes=3 * 4096):
    g = np.random.default_rng(0)
    x = g.standard_normal((n,) + shape).astype(np.float32)
    y = g.integers(0, 10, n).astype(np.int32)
    w = DatasetWriter(str(tmp_path), "toy-train", shape, batch, partition_bytes=partition_bytes)
    w.append(x[:30], y[:30]).append(x[30:], y[30:])
    return w.close(), x, y


def test_writer_layout_and_metadata(tmp_path):
    meta, x, y = _write(tmp_path)
    text = open(meta).read()
    assert "batch size   : 8" in text and "example shape: [3, 5, 5]" in text and "elements     : 72" in text   # 70 refilled to 72
    files = sorted(f for f in os.listdir(tmp_path) if "examples" in f)
    assert len(files) == 3 and files[0].endswith("examples.1")
    # every batch starts on a page boundary
    first = np.fromfile(os.path.join(tmp_path, files[0]), dtype=np.float32)
    per_batch = 4096 // 4
    assert first.size == 3 * per_batch
    assert np.array_equal(first[:8 * 75].reshape(8, 3, 5, 5), x[:8])
    assert np.all(first[8 * 75:per_batch] == 0)


def test_basic_dataset_batches_and_window(tmp_path):
    meta, x, y = _write(tmp_path)
    ds = BasicDataset(meta, window=2)
    assert ds.number_of_examples() == 72 and ds.example_shape == (3, 5, 5) and ds.partitions == 3
    for b in range(9):
        ex, lab = ds.batch(b)
        lo = b * 8
        exp_x = np.concatenate([x[lo:lo + 8], x[:max(0, lo + 8 - 70)]])[:8]
        assert np.array_equal(ex.numpy(), exp_x), b
        assert ds.resident_partitions() <= 2
    ex, _ = ds.batch(9)          # wraps around to the first batch
    assert np.array_equal(ex.numpy(), x[:8])
    ds.close()


def test_light_dataset_ring(tmp_path):
    meta, x, y = _write(tmp_path)
    ds = LightDataset(meta, slots=3, copiers=2)
    for b in range(12):
        ex, lab = ds.batch(b)
        lo = (b % 9) * 8
        exp_y = np.concatenate([y[lo:lo + 8], y[:max(0, lo + 8 - 70)]])[:8]
        assert np.array_equal(lab.numpy(), exp_y), b
    ds.close()


def test_scheduler_pulls_from_ring(tmp_path):
    meta, x, y = _write(tmp_path)
    ds = LightDataset(meta, slots=4, copiers=1)
    rt = Runtime(learners=2, wpc=2, task_timeout_s=5)
    rt.attach_fake(2, task_us=300)
    rt.set_data_source(ds.source(stride=1, offset=0, timeout_s=5))
    assert rt.train(40) == 40          # 40 tasks through a 4-slot ring: slots are recycled by the callback handlers
    rt.drain(10)
    assert rt.tasks_completed() == 40
    rt.close()
    ds.close()


def test_converters_mnist_cifar_ratings_random(tmp_path):
    import gzip
    import struct
    from crossbow_b200.data import convert
    g = np.random.default_rng(3)
    # MNIST: IDX files, big-endian headers, pixels scaled by 1/256
    px = g.integers(0, 256, (20, 28, 28), dtype=np.uint8)
    lab = g.integers(0, 10, 20, dtype=np.uint8)
    with gzip.open(tmp_path / "img.gz", "wb") as f:
        f.write(struct.pack(">iiii", 2051, 20, 28, 28) + px.tobytes())
    (tmp_path / "lab").write_bytes(struct.pack(">ii", 2049, 20) + lab.tobytes())
    meta = convert.convert_mnist(str(tmp_path / "img.gz"), str(tmp_path / "lab"), str(tmp_path / "m"), "mnist-train", 8)
    ds = BasicDataset(meta)
    ex, lb = ds.batch(1)
    assert ds.example_shape == (1, 28, 28) and np.array_equal(lb.numpy(), lab[8:16].astype(np.int32))
    assert np.array_equal(ex.numpy(), px[8:16, None].astype(np.float32) / 256.0)
    ds.close()
    with pytest.raises(ValueError, match="magic"):
        convert.convert_mnist(str(tmp_path / "lab"), str(tmp_path / "lab"), str(tmp_path / "bad"), "x", 8)
    # CIFAR-10 / CIFAR-100 records, pixels to [-1, 1], mean image beside the partitions
    rec = np.concatenate([g.integers(0, 10, (16, 1), dtype=np.uint8), g.integers(0, 256, (16, 3072), dtype=np.uint8)], axis=1)
    (tmp_path / "b1.bin").write_bytes(rec[:8].tobytes())
    (tmp_path / "b2.bin").write_bytes(rec[8:].tobytes())
    meta = convert.main(["cifar10", "--input", str(tmp_path / "b1.bin"), str(tmp_path / "b2.bin"), "-o", str(tmp_path / "c"), "--name", "cifar-train", "-b", "8"])
    ds = BasicDataset(str(tmp_path / "c" / "cifar-train.metadata"))
    ex, lb = ds.batch(1)
    want = rec[8:, 1:].reshape(8, 3, 32, 32).astype(np.float32) / 127.5 - 1.0
    assert np.allclose(ex.numpy(), want, atol=1e-6) and np.array_equal(lb.numpy(), rec[8:, 0].astype(np.int32))
    mean = np.fromfile(tmp_path / "c" / "cifar-train.mean", dtype=np.float32).reshape(3, 32, 32)
    assert np.allclose(mean, (rec[:, 1:].reshape(16, 3, 32, 32).astype(np.float32) / 127.5 - 1.0).mean(0), atol=1e-5)
    ds.close()
    rec100 = np.concatenate([g.integers(0, 20, (8, 1), dtype=np.uint8), g.integers(0, 100, (8, 1), dtype=np.uint8),
                             g.integers(0, 256, (8, 3072), dtype=np.uint8)], axis=1)
    (tmp_path / "c100.bin").write_bytes(rec100.tobytes())
    ds = BasicDataset(convert.convert_cifar100([str(tmp_path / "c100.bin")], str(tmp_path / "c100"), "c100", 8))
    assert np.array_equal(ds.batch(0)[1].numpy(), rec100[:, 1].astype(np.int32))          # fine labels
    ds.close()
    # ratings: "row column rating" lines
    (tmp_path / "r.txt").write_text("".join(f"{i} {2 * i} {i % 5 + 1}\n" for i in range(8)))
    ds = BasicDataset(convert.convert_ratings(str(tmp_path / "r.txt"), str(tmp_path / "r"), "ratings", 4))
    ex, lb = ds.batch(1)
    assert np.array_equal(ex.numpy(), np.array([[4, 8], [5, 10], [6, 12], [7, 14]], dtype=np.float32)) and list(lb.numpy()) == [5, 1, 2, 3]
    ds.close()
    # random
    ds = BasicDataset(convert.convert_random([3, 8, 8], 10, 32, str(tmp_path / "rnd"), "random-train", 16, seed=1))
    assert ds.number_of_examples() == 32 and ds.example_shape == (3, 8, 8)
    ds.close()
