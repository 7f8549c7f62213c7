"""Philox4x32-10 counter-based RNG, bit-identical to the device code in
``csrc/philox.cuh``.

Convention shared by every stochastic kernel of this package:

* key     = (seed_lo, seed_hi)
* counter = (group_lo, group_hi, step, stream)

``group`` is the index of a group of four consecutive flat elements, ``step``
the exchange sequence number of the tensor and ``stream`` a small constant that
separates independent draws inside one kernel.  Element ``4*group + j`` uses
output word ``j``; a uniform in ``[0, 1)`` is ``(word >> 8) * 2**-24`` (exact in
fp32).  The result does not depend on grid shape, which is what lets a NumPy
restatement check a kernel bit for bit.
"""
from __future__ import annotations

import numpy as np

_M0 = np.uint64(0xD2511F53)
_M1 = np.uint64(0xCD9E8D57)
_W0 = 0x9E3779B9
_W1 = 0xBB67AE85
_MASK = np.uint64(0xFFFFFFFF)


def philox4x32(c0, c1, c2, c3, k0: int, k1: int):
    """Vectorised Philox4x32-10.  ``c*`` are uint32 arrays (or scalars)."""
    c0 = np.asarray(c0, dtype=np.uint64)
    c1 = np.broadcast_to(np.asarray(c1, dtype=np.uint64), c0.shape).copy()
    c2 = np.broadcast_to(np.asarray(c2, dtype=np.uint64), c0.shape).copy()
    c3 = np.broadcast_to(np.asarray(c3, dtype=np.uint64), c0.shape).copy()
    c0 = c0.copy()
    k0 = int(k0) & 0xFFFFFFFF
    k1 = int(k1) & 0xFFFFFFFF
    for _ in range(10):
        p0 = _M0 * c0
        p1 = _M1 * c2
        hi0, lo0 = p0 >> np.uint64(32), p0 & _MASK
        hi1, lo1 = p1 >> np.uint64(32), p1 & _MASK
        n0 = (hi1 ^ c1 ^ np.uint64(k0)) & _MASK
        n1 = lo1
        n2 = (hi0 ^ c3 ^ np.uint64(k1)) & _MASK
        n3 = lo0
        c0, c1, c2, c3 = n0, n1, n2, n3
        k0 = (k0 + _W0) & 0xFFFFFFFF
        k1 = (k1 + _W1) & 0xFFFFFFFF
    return (c0.astype(np.uint32), c1.astype(np.uint32), c2.astype(np.uint32), c3.astype(np.uint32))


def random_words(numel: int, seed: int, step: int, stream: int = 0) -> np.ndarray:
    """uint32 word for every flat element index in ``[0, numel)``."""
    groups = (numel + 3) // 4
    g = np.arange(groups, dtype=np.uint64)
    w = philox4x32(g & _MASK, g >> np.uint64(32), step & 0xFFFFFFFF, stream & 0xFFFFFFFF,
                   seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF)
    return np.stack(w, axis=1).reshape(-1)[:numel]


def uniform(numel: int, seed: int, step: int, stream: int = 0) -> np.ndarray:
    """fp32 uniforms in [0, 1) for every flat element index."""
    return (random_words(numel, seed, step, stream) >> np.uint32(8)).astype(np.float32) * np.float32(2.0 ** -24)
