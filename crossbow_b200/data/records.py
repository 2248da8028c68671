"""Record files (JPEG + label + bounding boxes) and the double-buffered, multi-threaded decoding data set
(csrc/data/record.cpp): the ImageNet path of the reference (RecordDataset.java:59-99, clib-multigpu/recorddataset.c,
doublebuffer.c, image/*.c)."""
from __future__ import annotations

import ctypes as C
from typing import Sequence

import numpy as np
import torch

from ..runtime import load as _load
from .dataset import Dataset
from .native import _tensor

_ready = False


def _lib():
    global _ready
    lib = _load()
    if not _ready:
        P, I, L, F = C.c_void_p, C.c_int, C.c_longlong, C.c_float
        V = C.POINTER(C.c_void_p)
        lib.rec_jpeg_decode.restype, lib.rec_jpeg_decode.argtypes = I, [P, L, P, L, C.POINTER(I), C.POINTER(I)]
        lib.rec_process.restype, lib.rec_process.argtypes = I, [P, L, C.POINTER(F), I, I, I, C.c_ulonglong, P]
        lib.rec_plan.restype, lib.rec_plan.argtypes = None, [I, I, C.POINTER(F), I, I, C.c_ulonglong, C.POINTER(I)]
        lib.rec_writer_open.restype, lib.rec_writer_open.argtypes = P, [C.c_char_p]
        lib.rec_writer_append.restype, lib.rec_writer_append.argtypes = I, [P, P, L, I, C.POINTER(F), I, I, I]
        lib.rec_writer_close.restype, lib.rec_writer_close.argtypes = I, [P]
        lib.rec_dataset_open.restype = P
        lib.rec_dataset_open.argtypes = [C.POINTER(C.c_char_p), I, I, I, I, I, I, C.c_ulonglong]
        lib.rec_dataset_buffer.restype, lib.rec_dataset_buffer.argtypes = P, [P, I, I, C.POINTER(L)]
        lib.rec_dataset_take.restype, lib.rec_dataset_take.argtypes = I, [P, L, V, V, C.c_double]
        lib.rec_dataset_release.restype, lib.rec_dataset_release.argtypes = None, [P, I]
        for n in ("rec_dataset_examples", "rec_dataset_failures", "rec_dataset_images"):
            getattr(lib, n).restype, getattr(lib, n).argtypes = L, [P]
        lib.rec_dataset_close.restype, lib.rec_dataset_close.argtypes = None, [P]
        lib.rec_source_create.restype, lib.rec_source_create.argtypes = P, [P, L, L, C.c_double]
        _ready = True
    return lib


def decode_jpeg(data: bytes) -> np.ndarray:
    """JPEG (sequential or progressive; grey, YCbCr, RGB, CMYK / YCCK) -> uint8 RGB array [H, W, 3]."""
    lib = _lib()
    w, h = C.c_int(), C.c_int()
    out = np.zeros(1, dtype=np.uint8)
    rc = lib.rec_jpeg_decode(data, len(data), out.ctypes.data, 0, C.byref(w), C.byref(h))
    if rc not in (0, -3):
        raise ValueError(f"JPEG decoder error {rc} ({'unsupported coding process' if rc == -2 else 'malformed stream'})")
    out = np.zeros((h.value, w.value, 3), dtype=np.uint8)
    rc = lib.rec_jpeg_decode(data, len(data), out.ctypes.data, out.size, C.byref(w), C.byref(h))
    if rc != 0:
        raise ValueError(f"JPEG decoder error {rc}")
    return out


def preprocess(data: bytes, boxes: Sequence[Sequence[float]] = (), training: bool = True, size: int = 224, seed: int = 0) -> np.ndarray:
    """One record through the train / test pipeline -> float32 [3, size, size] in [-1, 1]."""
    lib = _lib()
    b = np.asarray(boxes, dtype=np.float32).reshape(-1, 4)
    out = np.empty((3, size, size), dtype=np.float32)
    rc = lib.rec_process(data, len(data), b.ctypes.data_as(C.POINTER(C.c_float)), b.shape[0], int(training), size, seed, out.ctypes.data)
    if rc != 0:
        raise ValueError(f"JPEG decoder error {rc}")
    return out


def crop_plan(width: int, height: int, boxes: Sequence[Sequence[float]] = (), training: bool = True, seed: int = 0):
    """(x0, y0, crop width, crop height, flip) the pipeline uses for a decoded ``width`` x ``height`` image: the sampled
    distorted bounding box and mirror flag of a training example, or the centre crop of a test example."""
    lib = _lib()
    b = np.asarray(boxes, dtype=np.float32).reshape(-1, 4)
    plan = (C.c_int * 5)()
    lib.rec_plan(width, height, b.ctypes.data_as(C.POINTER(C.c_float)), b.shape[0], int(training), seed, plan)
    return tuple(int(v) for v in plan)


def preprocess_batch_gpu(images: Sequence[np.ndarray], plans: Sequence[Sequence[int]], size: int = 224, device=None, stream: int = 0) -> torch.Tensor:
    """Decoded uint8 RGB images [H, W, 3] + their crop plans -> float32 [N, 3, size, size] in [-1, 1] ON THE GPU, in one
    kernel launch (csrc/kernels/image.cu): crop, mirror, bilinear resize, x / 127.5 - 1, planar layout.  Bit-identical to
    ``preprocess`` for the same plan; the host only uploads 3 bytes per source pixel."""
    from ..ops import lib as L
    cl = L.load()
    device = device if device is not None else torch.device("cuda", torch.cuda.current_device())
    n = len(images)
    if n == 0 or n != len(plans):
        raise ValueError("one crop plan per image is required")
    desc = np.zeros((n, cl.xb_image_desc_size() // 4), dtype=np.int32)
    offsets, total = [], 0
    for img in images:
        if img.dtype != np.uint8 or img.ndim != 3 or img.shape[2] != 3:
            raise ValueError("images must be uint8 arrays of shape [H, W, 3]")
        offsets.append(total)
        total += (img.size + 15) // 16 * 16
    packed = torch.empty(total, dtype=torch.uint8).pin_memory() if torch.cuda.is_available() else torch.empty(total, dtype=torch.uint8)
    pk = packed.numpy()
    for i, (img, plan) in enumerate(zip(images, plans)):
        h, w = img.shape[:2]
        x0, y0, cw, ch, flip = [int(v) for v in plan]
        if not (0 <= x0 and 0 <= y0 and cw >= 1 and ch >= 1 and x0 + cw <= w and y0 + ch <= h):
            raise ValueError(f"crop window {plan} does not fit a {w} x {h} image")
        pk[offsets[i]:offsets[i] + img.size] = np.ascontiguousarray(img).reshape(-1)
        desc[i].view(np.int64)[0] = offsets[i]
        desc[i, 2:9] = (w, h, x0, y0, cw, ch, flip)
    d_rgb = packed.to(device, non_blocking=True)
    d_desc = torch.from_numpy(desc).to(device)
    out = torch.empty((n, 3, size, size), dtype=torch.float32, device=device)
    s = stream or torch.cuda.current_stream(device).cuda_stream
    L.check(cl.xb_image_crop_resize(d_rgb.data_ptr(), d_desc.data_ptr(), n, size, out.data_ptr(), s), "image crop / resize")
    out._keep = (d_rgb, d_desc)          # the kernel may still be reading them when this returns
    return out


class RecordWriter:
    def __init__(self, path: str):
        self.lib = _lib()
        self.h = self.lib.rec_writer_open(path.encode())
        if not self.h:
            raise IOError(f"cannot create {path}")

    def append(self, jpeg: bytes, label: int, boxes: Sequence[Sequence[float]] = (), height: int = 0, width: int = 0):
        b = np.asarray(boxes, dtype=np.float32).reshape(-1, 4)
        self.lib.rec_writer_append(self.h, jpeg, len(jpeg), label, b.ctypes.data_as(C.POINTER(C.c_float)), b.shape[0], height, width)
        return self

    def close(self) -> int:
        n = self.lib.rec_writer_close(self.h)
        self.h = None
        return n


class RecordDataset(Dataset):
    """Two page-locked halves of ``batches_per_half`` batches; ``workers`` threads decode + augment into the idle half."""

    def __init__(self, paths: Sequence[str], batch_size: int, batches_per_half: int = 32, image_size: int = 224, workers: int = 4,
                 training: bool = True, seed: int = 0, register_with_cuda: bool = False, timeout_s: float = 60.0):
        self.lib = _lib()
        arr = (C.c_char_p * len(paths))(*[p.encode() for p in paths])
        self.h = self.lib.rec_dataset_open(arr, len(paths), batch_size, batches_per_half, image_size, workers, int(training), seed)
        if not self.h:
            raise IOError("cannot open the record files")
        self.batch_size, self.example_shape, self.nb, self.timeout_s = batch_size, (3, image_size, image_size), batches_per_half, timeout_s
        self._held = []
        if register_with_cuda:
            from ..ops import lib as L
            cl = L.load()
            for half in (0, 1):
                for which in (0, 1):
                    n = C.c_longlong()
                    p = self.lib.rec_dataset_buffer(self.h, half, which, C.byref(n))
                    L.check(cl.xb_host_register(p, n.value), "cudaHostRegister of the double buffer")

    def number_of_examples(self):
        n = self.lib.rec_dataset_examples(self.h)
        return n // self.batch_size * self.batch_size

    def batch(self, task: int):
        """Batches must be requested in increasing order; earlier batches are released when the next half is entered."""
        e, l = C.c_void_p(), C.c_void_p()
        while self._held and self._held[0][0] // self.nb < task // self.nb:
            self.lib.rec_dataset_release(self.h, self._held.pop(0)[1])
        half = self.lib.rec_dataset_take(self.h, task, C.byref(e), C.byref(l), self.timeout_s)
        if half < 0:
            raise TimeoutError("the decoders did not refill the buffer in time")
        self._held.append((task, half))
        return _tensor(e.value, (self.batch_size,) + self.example_shape, torch.float32), _tensor(l.value, (self.batch_size,), torch.int32)

    def decode_failures(self):
        return self.lib.rec_dataset_failures(self.h)

    def source(self, stride: int = 1, offset: int = 0, timeout_s: float = 60.0) -> int:
        self._source = self.lib.rec_source_create(self.h, stride, offset, timeout_s)
        return self._source

    def close(self):
        for _, half in self._held:
            self.lib.rec_dataset_release(self.h, half)
        self._held = []
        if self.h:
            self.lib.rec_dataset_close(self.h)
            self.h = None
