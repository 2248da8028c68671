"""Philox4x32-10 counter-based random numbers, bit-identical to the device implementation.

The reference draws dropout masks and crop/mirror randoms from stateful cuRAND / cuDNN generators
(cudnndropout.cu:4-75, datatransform.cu:78-193), which cannot be reproduced on a CPU.  Here every random
number is a pure function of (seed, stream, offset, element index), so the CPU oracle and the CUDA kernels
agree bit for bit and a task can be replayed.

Counter layout: c0 = element_index // 4, c1 = offset (task id), c2 = stream (operator id), c3 = 0;
key = (seed low 32 bits, seed high 32 bits).  Element ``i`` takes lane ``i % 4`` of the 4-word output.
"""
from __future__ import annotations

import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32(c0, c1, c2, c3, k0, k1):
    """Vectorised Philox4x32-10. Counters are uint64 arrays holding 32-bit values; keys are Python ints."""
    c0, c1, c2, c3 = (np.asarray(c, dtype=np.uint64) for c in (c0, c1, c2, c3))
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
        n0 = hi1 ^ c1 ^ np.uint64(k0)
        n2 = hi0 ^ c3 ^ np.uint64(k1)
        c0, c1, c2, c3 = n0, lo1, n2, lo0
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return c0, c1, c2, c3


def philox_uint32(n: int, seed: int, stream: int = 0, offset: int = 0) -> np.ndarray:
    """``n`` uint32 values for elements 0..n-1."""
    groups = (n + 3) // 4
    idx = np.arange(groups, dtype=np.uint64)
    z = np.zeros(groups, dtype=np.uint64)
    out = philox4x32(idx, z + np.uint64(offset & 0xFFFFFFFF), z + np.uint64(stream & 0xFFFFFFFF), z,
                     seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    return np.stack(out, axis=1).reshape(-1)[:n].astype(np.uint32)


def philox_uniform(n: int, seed: int, stream: int = 0, offset: int = 0) -> np.ndarray:
    """Uniform [0,1) floats with 24 random bits: (x >> 8) * 2^-24, exactly representable in fp32."""
    return (philox_uint32(n, seed, stream, offset) >> np.uint32(8)).astype(np.float32) * np.float32(1.0 / 16777216.0)
