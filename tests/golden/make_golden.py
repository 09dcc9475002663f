"""Generates tests/golden/dequant_golden.npz.

The reference is Rust and cannot be run here, so these fixtures come from an
independent numpy restatement of its block codecs (this file), written from the
format description in crates/strix-models/src/ggml_quant.rs:240-262, 404-430,
separately from the C oracle. The fixtures pin the C oracle and, through it, the
CUDA path. Run ``python tests/golden/make_golden.py`` to regenerate.
"""
import os

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def f16(b):
    return np.ascontiguousarray(b).view(np.float16).astype(np.float32)


def np_dequant_q4_0(raw):
    blk = raw.reshape(-1, 18)
    d = f16(blk[:, 0:2]).reshape(-1, 1)
    qs = blk[:, 2:]
    lo = (qs & 0x0F).astype(np.int32) - 8
    hi = (qs >> 4).astype(np.int32) - 8
    return (d * np.concatenate([lo, hi], axis=1).astype(np.float32)).reshape(-1)


def np_dequant_q8_0(raw):
    blk = raw.reshape(-1, 34)
    d = f16(blk[:, 0:2]).reshape(-1, 1)
    return (d * blk[:, 2:].view(np.int8).astype(np.float32)).reshape(-1)


def np_dequant_q6_k(raw):
    blk = raw.reshape(-1, 210)
    n = blk.shape[0]
    ql = blk[:, 0:128].reshape(n, 2, 64)
    qh = blk[:, 128:192].reshape(n, 2, 32)
    sc = blk[:, 192:208].view(np.int8).reshape(n, 2, 8).astype(np.float32)
    d = f16(blk[:, 208:210]).reshape(n, 1, 1)
    out = np.empty((n, 2, 4, 32), dtype=np.float32)
    l = np.arange(32)
    for quarter in range(4):
        lowsrc = ql[:, :, l + (32 if quarter in (1, 3) else 0)]
        low = (lowsrc & 0x0F) if quarter < 2 else (lowsrc >> 4)
        high = (qh[:, :, l] >> (2 * quarter)) & 3
        q = (low | (high << 4)).astype(np.int32) - 32
        s = sc[:, :, (l // 16) + 2 * quarter]          # [n,2,32]
        ds = (d * s).astype(np.float32)                 # first rounding: d*sc
        out[:, :, quarter, :] = ds * q.astype(np.float32)  # second rounding
    return out.reshape(-1)


def special_scales():
    # zero, smallest subnormal, a subnormal, smallest normal, -1, max finite, typical
    return np.array([0x0000, 0x0001, 0x01FF, 0x0400, 0xBC00, 0x7BFF, 0x2E66, 0x9EB8], dtype=np.uint16)


def main():
    g = np.random.Generator(np.random.PCG64(20240607))
    out = {}
    sp = special_scales()
    # Q4_0: 24 blocks
    a = np.empty((24, 18), dtype=np.uint8)
    a[:, 2:] = g.integers(0, 256, size=(24, 16), dtype=np.uint8)
    d = g.uniform(0.002, 0.02, size=24).astype(np.float16).view(np.uint16)
    d[:8] = sp
    a[:, 0:2] = d.view(np.uint8).reshape(24, 2)
    out["q4_0_raw"], out["q4_0_f32"] = a.reshape(-1), np_dequant_q4_0(a)
    # Q8_0: 24 blocks (include -128 deliberately: the codec treats it as a plain i8)
    a = np.empty((24, 34), dtype=np.uint8)
    a[:, 2:] = g.integers(-128, 128, size=(24, 32), dtype=np.int8).view(np.uint8)
    d = g.uniform(1e-4, 1e-3, size=24).astype(np.float16).view(np.uint16)
    d[:8] = sp
    a[:, 0:2] = d.view(np.uint8).reshape(24, 2)
    out["q8_0_raw"], out["q8_0_f32"] = a.reshape(-1), np_dequant_q8_0(a)
    # Q6_K: 12 super-blocks, sub-scales over the full i8 range
    a = np.empty((12, 210), dtype=np.uint8)
    a[:, 0:192] = g.integers(0, 256, size=(12, 192), dtype=np.uint8)
    a[:, 192:208] = g.integers(-128, 128, size=(12, 16), dtype=np.int8).view(np.uint8)
    d = g.uniform(1e-4, 1e-3, size=12).astype(np.float16).view(np.uint16)
    d[:8] = sp
    a[:, 208:210] = d.view(np.uint8).reshape(12, 2)
    out["q6_k_raw"], out["q6_k_f32"] = a.reshape(-1), np_dequant_q6_k(a)
    np.savez_compressed(os.path.join(HERE, "dequant_golden.npz"), **out)
    print({k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
