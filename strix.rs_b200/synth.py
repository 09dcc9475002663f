"""Seeded synthetic GGUF tensors and activations for the tests and the bench.

No model file or dataset is involved anywhere: every input is drawn here from
the distributions the benchmark configurations state (block scales as f16 of a
uniform, codes uniform over their range, activations standard normal), from a
PCG64 stream keyed by (seed, tensor name). Outputs are raw GGUF block bytes,
row-major ``[out_dim][in_dim/blk][blk_bytes]``, exactly what a model hands to
``upload_*``.
"""
import zlib

import numpy as np

Q4_0, Q4_1, Q8_0, Q6_K = 2, 3, 8, 14
BLOCK_ELEMS = {Q4_0: 32, Q4_1: 32, Q8_0: 32, Q6_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q8_0: 34, Q6_K: 210}


def rng(seed, name):
    return np.random.Generator(np.random.PCG64([int(seed) & 0xFFFFFFFF, zlib.crc32(name.encode())]))


def _f16_bytes(g, shape, lo, hi):
    d = g.uniform(lo, hi, size=shape).astype(np.float16)
    return d.view(np.uint8).reshape(shape + (2,))


def q4_0(seed, name, out_dim, in_dim, d_lo=0.002, d_hi=0.02):
    """Q4_0: d = f16(U(d_lo, d_hi)), 16 code bytes with nibbles U{0..15}."""
    nb = in_dim // 32
    g = rng(seed, name)
    a = np.empty((out_dim, nb, 18), dtype=np.uint8)
    a[:, :, 0:2] = _f16_bytes(g, (out_dim, nb), d_lo, d_hi)
    a[:, :, 2:] = g.integers(0, 256, size=(out_dim, nb, 16), dtype=np.uint8)
    return a.reshape(-1)


def q4_1(seed, name, out_dim, in_dim, d_lo=0.002, d_hi=0.02):
    """Q4_1: d = f16(U(d_lo, d_hi)), m = f16(U(-8 d_hi, 0)) (what an asymmetric quantiser of centred
    weights produces), 16 code bytes with nibbles U{0..15}; value = d * code + m."""
    nb = in_dim // 32
    g = rng(seed, name)
    a = np.empty((out_dim, nb, 20), dtype=np.uint8)
    a[:, :, 0:2] = _f16_bytes(g, (out_dim, nb), d_lo, d_hi)
    a[:, :, 2:4] = _f16_bytes(g, (out_dim, nb), -8.0 * d_hi, 0.0)
    a[:, :, 4:] = g.integers(0, 256, size=(out_dim, nb, 16), dtype=np.uint8)
    return a.reshape(-1)


def q8_0(seed, name, out_dim, in_dim, d_lo=1e-4, d_hi=1e-3):
    """Q8_0: d = f16(U(d_lo, d_hi)), 32 int8 codes U[-127, 127]."""
    nb = in_dim // 32
    g = rng(seed, name)
    a = np.empty((out_dim, nb, 34), dtype=np.uint8)
    a[:, :, 0:2] = _f16_bytes(g, (out_dim, nb), d_lo, d_hi)
    a[:, :, 2:] = g.integers(-127, 128, size=(out_dim, nb, 32), dtype=np.int8).view(np.uint8)
    return a.reshape(-1)


def q6_k(seed, name, out_dim, in_dim, d_lo=1e-4, d_hi=1e-3):
    """Q6_K: uniform ql/qh bytes (q6 U{0..63}), 16 int8 sub-scales U[-32, 31], d = f16(U)."""
    nb = in_dim // 256
    g = rng(seed, name)
    a = np.empty((out_dim, nb, 210), dtype=np.uint8)
    a[:, :, 0:192] = g.integers(0, 256, size=(out_dim, nb, 192), dtype=np.uint8)
    a[:, :, 192:208] = g.integers(-32, 32, size=(out_dim, nb, 16), dtype=np.int8).view(np.uint8)
    a[:, :, 208:210] = _f16_bytes(g, (out_dim, nb), d_lo, d_hi)
    return a.reshape(-1)


def quant(ty, seed, name, out_dim, in_dim):
    return {Q4_0: q4_0, Q4_1: q4_1, Q8_0: q8_0, Q6_K: q6_k}[ty](seed, name, out_dim, in_dim)


def normal(seed, name, *shape):
    return rng(seed, name).standard_normal(size=shape, dtype=np.float32)


def norm_weight(seed, name, n):
    """RMSNorm weights ~ 1 + N(0, 0.02)."""
    return (1.0 + 0.02 * rng(seed, name).standard_normal(size=n)).astype(np.float32)


def gguf_bytes(ty, out_dim, in_dim):
    return out_dim * (in_dim // BLOCK_ELEMS[ty]) * BLOCK_BYTES[ty]


def lcg_q4_0(out_dim, in_dim):
    """The tensor recipe of the reference's own device test
    (crates/strix-backend-rocm/src/lib.rs:132-152): one LCG stream, seed 0xA5A5_1234,
    ``s = s * 6364136223846793005 + 1``, draw = ``(s >> 33) as u32``; per block one draw
    for the scale ``f16(0.03 + (draw % 32) * 0.003)`` then four draws for the four
    code words; ``x[i] = sin(0.017 i) * 0.5`` in f32. Returns (GGUF Q4_0 bytes, x)."""
    nb = in_dim // 32
    total = out_dim * nb
    n = total * 5
    draws = np.empty(n, dtype=np.uint32)
    mul = np.uint64(6364136223846793005)
    B = 8192
    A = np.empty(B, dtype=np.uint64)   # s_{i+j} = A[j-1] * s_i + Cc[j-1]
    Cc = np.empty(B, dtype=np.uint64)
    with np.errstate(over="ignore"):
        a_, c_ = np.uint64(1), np.uint64(0)
        for j in range(B):
            a_ = a_ * mul
            c_ = c_ * mul + np.uint64(1)
            A[j], Cc[j] = a_, c_
        state = np.uint64(0xA5A51234)
        for at in range(0, n, B):
            m = min(B, n - at)
            s = A[:m] * state + Cc[:m]
            draws[at:at + m] = (s >> np.uint64(33)).astype(np.uint32)
            state = s[m - 1]
    draws = draws.reshape(total, 5)
    a = np.empty((total, 18), dtype=np.uint8)
    d = (np.float32(0.03) + (draws[:, 0] % 32).astype(np.float32) * np.float32(0.003)).astype(np.float16)
    a[:, 0:2] = d.view(np.uint8).reshape(total, 2)
    a[:, 2:] = np.ascontiguousarray(draws[:, 1:5]).view(np.uint8).reshape(total, 16)
    x = (np.sin(np.arange(in_dim, dtype=np.float32) * np.float32(0.017)) * np.float32(0.5)).astype(np.float32)
    return a.reshape(-1), x
