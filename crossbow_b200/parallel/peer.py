"""Peer-visible device buffers for one-process-per-GPU jobs.

Each rank allocates its communication buffers with plain ``cudaMalloc`` (through the native library, so the
allocation is a whole one and can be exported), publishes a CUDA IPC handle through the ``torch.distributed``
process group, and maps every peer's buffer into its own address space.  Kernels then address a peer's memory with
ordinary loads / stores over NVLink.  The reference is a single process that drives all GPUs and never needs this
(clib-multigpu/executioncontext.c:185-201 creates in-process NCCL communicators instead).
"""
from __future__ import annotations

import ctypes as C
import os
from typing import List, Optional

import torch

from ..ops import lib as L


def dist_info():
    """(rank, world, local_rank) from torch.distributed if initialised, else from the launcher's environment."""
    import torch.distributed as dist
    if dist.is_available() and dist.is_initialized():
        return dist.get_rank(), dist.get_world_size(), int(os.environ.get("LOCAL_RANK", dist.get_rank()))
    return int(os.environ.get("RANK", 0)), int(os.environ.get("WORLD_SIZE", 1)), int(os.environ.get("LOCAL_RANK", 0))


def init_process_group(backend: Optional[str] = None, timeout_s: float = 600.0):
    """Join the job described by RANK / WORLD_SIZE / MASTER_ADDR / MASTER_PORT (no-op for a single process)."""
    import datetime
    import torch.distributed as dist
    world = int(os.environ.get("WORLD_SIZE", 1))
    if world <= 1 or dist.is_initialized():
        return
    os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
    os.environ.setdefault("MASTER_PORT", "29500")
    if backend is None:
        backend = "nccl" if torch.cuda.is_available() else "gloo"
    if backend == "nccl":
        torch.cuda.set_device(int(os.environ.get("LOCAL_RANK", 0)))
    dist.init_process_group(backend=backend, timeout=datetime.timedelta(seconds=timeout_s))


class PeerBuffer:
    """A device buffer of ``nbytes`` on every rank; ``ptrs[g]`` is rank g's buffer as seen from this process."""

    def __init__(self, nbytes: int, rank: int, world: int, group=None):
        import torch.distributed as dist
        lib = L.load()
        self.lib, self.rank, self.world, self.nbytes = lib, rank, world, nbytes
        self.local = lib.xb_device_alloc(max(256, nbytes))
        if not self.local:
            raise L.CudaError(f"cudaMalloc of {nbytes} bytes for a peer buffer failed")
        self.ptrs: List[int] = [0] * world
        self.ptrs[rank] = self.local
        self._imported: List[int] = []
        if world > 1:
            handle = (C.c_char * 64)()
            L.check(lib.xb_ipc_export(self.local, handle), "cudaIpcGetMemHandle")
            mine = bytes(handle)
            gathered: List[Optional[bytes]] = [None] * world
            dist.all_gather_object(gathered, mine, group=group)
            for g in range(world):
                if g == rank:
                    continue
                buf = (C.c_char * 64).from_buffer_copy(gathered[g])
                p = lib.xb_ipc_import(buf)
                if not p:
                    raise L.CudaError(f"cudaIpcOpenMemHandle failed for rank {g}'s buffer")
                self.ptrs[g] = p
                self._imported.append(p)

    def as_tensor(self, numel: int, device=None) -> torch.Tensor:
        """This rank's buffer as a float32 tensor (no copy; the buffer must outlive the tensor)."""
        class _Raw:
            pass
        raw = _Raw()
        raw.__cuda_array_interface__ = {"shape": (int(numel),), "typestr": "<f4", "data": (int(self.local), False), "version": 2}
        self._keep = raw
        return torch.as_tensor(raw, device=device if device is not None else torch.device("cuda", torch.cuda.current_device()))

    def close(self):
        for p in self._imported:
            self.lib.xb_ipc_close(p)
        self._imported = []
        if self.local:
            self.lib.xb_device_free(self.local)
            self.local = 0
