"""Counter-based random inputs shared by tests, fixtures and the benchmark.

Every element is a pure function of (seed, tensor id, element index): SplitMix64 hashes the
three into two 32-bit uniforms and Box-Muller turns those into one N(0,1) sample.  The same
call gives the same bytes everywhere, whatever the shape of the loop that asks, so the CPU
checkers and the GPU path are fed identical data.
"""
import numpy as np

# fixed tensor ids
X, WQ, WK, WV, WO, DOUT, BQ, BK, BV, BO, KEY, VALUE = range(12)

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(z):
    with np.errstate(over="ignore"):
        z = (z + np.uint64(0x9E3779B97F4A7C15)) & _M64
        z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
        z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
        return z ^ (z >> np.uint64(31))


def normal(seed, tensor_id, shape, std=1.0, offset=0, dtype=np.float32):
    """N(0, std^2) samples for elements offset .. offset+prod(shape)-1 of tensor `tensor_id`."""
    n = int(np.prod(shape))
    out = np.empty(n, dtype=np.float32)
    key = _splitmix64(np.uint64(seed) ^ _splitmix64(np.uint64(tensor_id + 1)))
    step = 1 << 22
    for s in range(0, n, step):
        idx = np.arange(s + offset, min(n, s + step) + offset, dtype=np.uint64)
        with np.errstate(over="ignore"):
            h = _splitmix64(idx * np.uint64(0xD1342543DE82EF95) + key)
        u1 = ((h >> np.uint64(32)).astype(np.float64) + 1.0) / 4294967296.0      # (0, 1]
        u2 = (h & np.uint64(0xFFFFFFFF)).astype(np.float64) / 4294967296.0       # [0, 1)
        out[s:s + len(idx)] = (np.sqrt(-2.0 * np.log(u1)) * np.cos(2.0 * np.pi * u2) * std).astype(np.float32)
    return out.reshape(shape).astype(dtype, copy=False)


def bf16_round(a):
    """Round FP32 values to the nearest BF16 (ties to even), returned as FP32."""
    u = np.ascontiguousarray(a, dtype=np.float32).view(np.uint32).astype(np.uint64)
    r = ((u + np.uint64(0x7FFF) + ((u >> np.uint64(16)) & np.uint64(1))) >> np.uint64(16)) << np.uint64(16)
    return (r & np.uint64(0xFFFFFFFF)).astype(np.uint32).view(np.float32).reshape(np.shape(a))


def to_bf16_bits(a):
    """FP32 array -> uint16 array of BF16 bit patterns (round to nearest even)."""
    return (bf16_round(a).view(np.uint32) >> np.uint32(16)).astype(np.uint16)


def from_bf16_bits(b):
    """uint16 BF16 bit patterns -> FP32 array."""
    return (np.ascontiguousarray(b, dtype=np.uint16).astype(np.uint32) << np.uint32(16)).view(np.float32)
