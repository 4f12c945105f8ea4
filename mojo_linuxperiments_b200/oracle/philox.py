"""NumPy statement of the Philox-4x32-10 stream used by the fill+reduce workload (host C++, CUDA and this file agree)."""
import numpy as np

_M0, _M1 = np.uint64(0xD2511F53), np.uint64(0xCD9E8D57)
_W0, _W1 = 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter: np.ndarray, seed: int) -> np.ndarray:
    """counter: uint64 array -> uint32 array [..., 4]."""
    counter = np.asarray(counter, dtype=np.uint64)
    mask = np.uint64(0xFFFFFFFF)
    c0, c1 = counter & mask, counter >> np.uint64(32)
    c2 = np.zeros_like(c0)
    c3 = np.zeros_like(c0)
    k0, k1 = seed & 0xFFFFFFFF, (seed >> 32) & 0xFFFFFFFF
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        hi0, lo0, hi1, lo1 = p0 >> np.uint64(32), p0 & mask, p1 >> np.uint64(32), p1 & mask
        c0, c1, c2, c3 = hi1 ^ c1 ^ np.uint64(k0), lo1, hi0 ^ c3 ^ np.uint64(k1), lo0
        k0, k1 = (k0 + _W0) & 0xFFFFFFFF, (k1 + _W1) & 0xFFFFFFFF
    return np.stack([c0, c1, c2, c3], axis=-1).astype(np.uint32)


def uniform_pm1(n: int, seed: int, start: int = 0) -> np.ndarray:
    """Elements start..start+n of the uniform[-1,1) float32 stream of ``seed``."""
    idx = np.arange(start, start + n, dtype=np.uint64)
    blocks = philox4x32_10(idx >> np.uint64(2), seed)
    lane = (idx & np.uint64(3)).astype(np.int64)
    x = blocks[np.arange(n), lane]
    return ((x >> np.uint32(8)).astype(np.float32) * np.float32(2.0 / 16777216.0) - np.float32(1.0)).astype(np.float32)
