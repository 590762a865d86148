"""Exactly reproducible synthetic inputs for fixtures and parity tests.

Integer-only generator (splitmix64 counters, sum of twelve 16-bit uniforms, the
Irwin-Hall approximation of N(0,1)), so the same (seed, shape) gives the same
bits on every machine and numpy version, with no libm involved.
"""
import numpy as np

_M64 = np.uint64(0xFFFFFFFFFFFFFFFF)


def _splitmix64(x):
    x = (x + np.uint64(0x9E3779B97F4A7C15)) & _M64
    z = x
    z = ((z ^ (z >> np.uint64(30))) * np.uint64(0xBF58476D1CE4E5B9)) & _M64
    z = ((z ^ (z >> np.uint64(27))) * np.uint64(0x94D049BB133111EB)) & _M64
    return z ^ (z >> np.uint64(31))


def normal(seed, shape, sigma=1.0, stream=0):
    """float32 array of approximately N(0, sigma^2) values, exact in fp32."""
    n = int(np.prod(shape))
    with np.errstate(over="ignore"):
        base = np.arange(n, dtype=np.uint64) * np.uint64(3) + (
            np.uint64(seed) * np.uint64(0x100000001B3) + np.uint64(stream) * np.uint64(0x9E3779B1)) * np.uint64(0x10001)
        total = np.zeros(n, dtype=np.int64)
        for t in range(3):
            w = _splitmix64(base + np.uint64(t))
            for s in (0, 16, 32, 48):
                total += ((w >> np.uint64(s)) & np.uint64(0xFFFF)).astype(np.int64)
    x = (total * 2 - 12 * 65535).astype(np.float64) / 131072.0
    return (x * sigma).astype(np.float32).reshape(shape)


def round_to(x, dtype_name):
    """Round an fp32 array to fp16/bf16 (round-to-nearest-even) and back."""
    import torch
    dt = {"float16": torch.float16, "bfloat16": torch.bfloat16}[dtype_name]
    return torch.from_numpy(np.ascontiguousarray(x)).to(dt).float().numpy()


def qkv(seed, B, H, Nq, Nk, d, dtype_name, sigma=1.0):
    q = round_to(normal(seed, (B, H, Nq, d), sigma, 0), dtype_name)
    k = round_to(normal(seed, (B, H, Nk, d), sigma, 1), dtype_name)
    v = round_to(normal(seed, (B, H, Nk, d), sigma, 2), dtype_name)
    return q, k, v


def alibi_slopes(H):
    return np.array([2.0 ** (-8.0 * (h + 1) / H) for h in range(H)], dtype=np.float32)
