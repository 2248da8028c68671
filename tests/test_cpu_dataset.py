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
