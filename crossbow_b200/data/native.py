"""Binary data sets on disk, served by the C++ pipeline (csrc/data/dataset.cpp).

``DatasetWriter``  - encoder: cuts (example, label) tuples into page-padded batches and partition files + a metadata
                     file (the job of the reference's Java encoders, preprocess/*).
``BasicDataset``   - memory-mapped partitions with a sliding window of locked (and, on a GPU box, CUDA-registered)
                     partitions; a batch is two addresses inside the mappings.
``LightDataset``   - fixed ring of page-locked slots filled ahead of time by copier threads.
Both implement the ``Dataset`` interface of ``dataset.py`` and can also feed the native scheduler directly
(``source()``), in which case no Python runs per task.
"""
from __future__ import annotations

import ctypes as C
import os
from typing import Optional, Sequence

import numpy as np
import torch

from ..runtime import load as _load
from .dataset import Dataset


def _tensor(ptr: int, shape, dtype):
    n = int(np.prod(shape))
    ctype = C.c_float if dtype == torch.float32 else C.c_int32
    buf = (ctype * n).from_address(ptr)
    return torch.frombuffer(buf, dtype=dtype).reshape(tuple(shape))


class DatasetWriter:
    def __init__(self, directory: str, name: str, example_shape: Sequence[int], batch_size: int,
                 partition_bytes: Optional[int] = None, pad_to_page: bool = True):
        """`partition_bytes`: size limit of one partition file (default: `--file-partition-size`)."""
        if partition_bytes is None:
            from ..conf import SystemConf
            partition_bytes = SystemConf.getInstance().file_partition_size
        self.lib = _load()
        os.makedirs(directory, exist_ok=True)
        self.meta_path = os.path.join(directory, f"{name}.metadata")
        shape = (C.c_longlong * len(example_shape))(*example_shape)
        self.example_shape = tuple(example_shape)
        self.h = self.lib.ds_writer_create(self.meta_path.encode(), os.path.join(directory, f"{name}-examples").encode(),
                                           os.path.join(directory, f"{name}-labels").encode(), batch_size, shape, len(example_shape),
                                           partition_bytes, int(pad_to_page))

    def append(self, examples, labels):
        x = np.ascontiguousarray(np.asarray(examples, dtype=np.float32)).reshape((-1,) + self.example_shape)
        y = np.ascontiguousarray(np.asarray(labels, dtype=np.int32)).reshape(-1)
        if x.shape[0] != y.shape[0]:
            raise ValueError("examples and labels differ in count")
        if self.lib.ds_writer_append(self.h, x.ctypes.data, y.ctypes.data, x.shape[0]) != 0:
            raise IOError("could not write the data set partition")
        return self

    def close(self) -> str:
        if self.lib.ds_writer_close(self.h) != 0:
            raise IOError("could not finish the data set")
        self.h = None
        return self.meta_path


class _NativeDataset(Dataset):
    kind = 0

    def _read_meta(self, path):
        lib = self.lib
        m = lib.ds_meta_load(path.encode())
        if not m:
            raise FileNotFoundError(f"error: cannot read data set metadata {path}")
        g = lambda i: lib.ds_meta_get(m, i)
        self.partitions, self.elements, self.batch_size = g(0), g(1), g(2)
        self.example_shape = tuple(lib.ds_meta_shape(m, i) for i in range(g(7)))
        self.nbatches = g(8)
        lib.ds_meta_free(m)

    def number_of_examples(self):
        return self.nbatches * self.batch_size

    def source(self, stride: int = 1, offset: int = 0, timeout_s: float = 30.0) -> int:
        """Handle for ``Runtime.set_data_source`` (task t reads batch t*stride+offset)."""
        self._source = self.lib.ds_source_create(self.h, self.kind, stride, offset, timeout_s)
        return self._source


class BasicDataset(_NativeDataset):
    kind = 0

    def __init__(self, metadata_path: str, window: Optional[int] = None, register_with_cuda: bool = False, timeout_s: float = 30.0):
        """`window`: partitions kept mapped at a time (default: `--mapped-partitions-window`)."""
        if window is None:
            from ..conf import SystemConf
            window = SystemConf.getInstance().mapped_partitions_window
        self.lib = _load()
        self._read_meta(metadata_path)
        reg = unreg = None
        if register_with_cuda:
            from ..ops import lib as L
            cl = L.load()
            reg = C.cast(cl.xb_host_register, C.c_void_p).value
            unreg = C.cast(cl.xb_host_unregister, C.c_void_p).value
        self.h = self.lib.ds_basic_open(metadata_path.encode(), window, reg, unreg)
        if not self.h:
            raise IOError(f"error: cannot open the partitions of {metadata_path}")
        self.timeout_s = timeout_s

    def batch(self, task: int):
        e, l = C.c_void_p(), C.c_void_p()
        if self.lib.ds_basic_batch(self.h, task, C.byref(e), C.byref(l), self.timeout_s) != 0:
            raise TimeoutError("partition did not become resident in time")
        return _tensor(e.value, (self.batch_size,) + self.example_shape, torch.float32), _tensor(l.value, (self.batch_size,), torch.int32)

    def resident_partitions(self):
        return self.lib.ds_basic_resident_partitions(self.h)

    def close(self):
        if self.h:
            self.lib.ds_basic_close(self.h)
            self.h = None


class LightDataset(_NativeDataset):
    kind = 1

    def __init__(self, metadata_path: str, slots: int = 8, copiers: Optional[int] = None, register_with_cuda: bool = False,
                 timeout_s: float = 30.0):
        """`copiers`: threads that fill the slot ring from the partition files (default: `--number-of-file-handlers`)."""
        if copiers is None:
            from ..conf import SystemConf
            copiers = max(1, SystemConf.getInstance().number_of_file_handlers)
        self.lib = _load()
        self._read_meta(metadata_path)
        self.h = self.lib.ds_light_open(metadata_path.encode(), slots, copiers)
        if not self.h:
            raise IOError(f"error: cannot open the partitions of {metadata_path}")
        self.timeout_s, self.slots = timeout_s, slots
        self._held = {}
        if register_with_cuda:
            from ..ops import lib as L
            cl = L.load()
            for which in (0, 1):
                n = C.c_longlong()
                p = self.lib.ds_light_ring(self.h, which, C.byref(n))
                L.check(cl.xb_host_register(p, n.value), "cudaHostRegister of the slot ring")

    def batch(self, task: int):
        """Tasks must be taken in order; the slot of task t is released when task t+slots-1 is requested, or via release()."""
        e, l = C.c_void_p(), C.c_void_p()
        for old in [t for t in self._held if t <= task - self.slots + 1]:
            self.release(old)
        slot = self.lib.ds_light_take(self.h, task, C.byref(e), C.byref(l), self.timeout_s)
        if slot < 0:
            raise TimeoutError("slot was not filled in time")
        self._held[task] = slot
        return _tensor(e.value, (self.batch_size,) + self.example_shape, torch.float32), _tensor(l.value, (self.batch_size,), torch.int32)

    def release(self, task: int):
        slot = self._held.pop(task, None)
        if slot is not None:
            self.lib.ds_light_release(self.h, slot)

    def close(self):
        if self.h:
            self.lib.ds_light_close(self.h)
            self.h = None
