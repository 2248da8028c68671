"""Batch sources that hand out page-locked host memory, ready for an asynchronous host-to-device copy.

The reference memory-maps pre-batched binary files and registers the mapped pages with CUDA
(data/Dataset.java:51-126, clib-multigpu/dataset.c); tasks are then (offset, length) ranges of that memory.  The
same contract is kept: ``batch(i)`` returns the host ADDRESSES of the examples and labels of task ``i``; nothing
is copied on the way to the device except the DMA itself.
"""
from __future__ import annotations

from typing import Sequence, Tuple

import numpy as np
import torch


def _pinned(shape, dtype):
    try:
        return torch.empty(shape, dtype=dtype, pin_memory=torch.cuda.is_available())
    except RuntimeError:
        return torch.empty(shape, dtype=dtype)


class Dataset:
    """Interface: fixed batch size, ``number_of_examples``, ``batch(task) -> (examples, labels)`` pinned tensors."""

    batch_size: int
    example_shape: Tuple[int, ...]

    def number_of_examples(self) -> int:
        raise NotImplementedError

    def number_of_batches(self) -> int:
        return self.number_of_examples() // self.batch_size

    def batch(self, task: int):
        raise NotImplementedError

    def batch_bytes(self) -> int:
        n = self.batch_size
        return 4 * n * int(np.prod(self.example_shape)) + 4 * n


class ArrayDataset(Dataset):
    """Examples [N, ...] float32 and labels [N] int32 held in pinned memory, cut into consecutive batches.
    The tail that does not fill a batch is dropped unless ``refill`` wraps it around with examples from the start
    (DatasetMetadata.java:441-458 refills the last batch the same way)."""

    def __init__(self, examples, labels, batch_size: int, refill=False):
        examples = torch.as_tensor(np.asarray(examples), dtype=torch.float32)
        labels = torch.as_tensor(np.asarray(labels)).to(torch.int32)
        n = examples.shape[0]
        if refill and n % batch_size:
            pad = batch_size - n % batch_size
            examples = torch.cat([examples, examples[:pad]])
            labels = torch.cat([labels, labels[:pad]])
            n += pad
        nb = n // batch_size
        self.batch_size = batch_size
        self.example_shape = tuple(examples.shape[1:])
        self.examples = _pinned((nb, batch_size) + self.example_shape, torch.float32)
        self.labels = _pinned((nb, batch_size), torch.int32)
        self.examples.copy_(examples[: nb * batch_size].reshape(self.examples.shape))
        self.labels.copy_(labels[: nb * batch_size].reshape(self.labels.shape))

    def number_of_examples(self):
        return self.examples.shape[0] * self.batch_size

    def batch(self, task: int):
        i = task % self.examples.shape[0]
        return self.examples[i], self.labels[i]


class SyntheticDataset(ArrayDataset):
    """Random examples of a given shape (N(0,1) or U[0,1)) and uniform labels, generated once from a seed."""

    def __init__(self, example_shape: Sequence[int], classes: int, batch_size: int, batches: int = 8, seed: int = 0,
                 distribution: str = "normal"):
        g = np.random.default_rng(seed)
        n = batches * batch_size
        if distribution == "normal":
            x = g.standard_normal((n,) + tuple(example_shape), dtype=np.float32)
        else:
            x = g.random((n,) + tuple(example_shape), dtype=np.float32)
        y = g.integers(0, classes, size=n, dtype=np.int32)
        super().__init__(x, y, batch_size)
        self.classes = classes
