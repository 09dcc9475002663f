"""ctypes binding of the CPU oracle (oracle/strix_oracle.c).

Test infrastructure only: imported by tests/, by ``__graft_entry__.smoke()`` and
by ``bench.py``'s CPU-baseline legs as the checker / the timed CPU baseline. The
shipped backend never imports it.
"""
import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_SO = os.path.join(_HERE, "libstrix_oracle.so")

Q4_0, Q4_1, Q8_0, Q6_K = 2, 3, 8, 14
BLOCK_ELEMS = {Q4_0: 32, Q4_1: 32, Q8_0: 32, Q6_K: 256}
BLOCK_BYTES = {Q4_0: 18, Q4_1: 20, Q8_0: 34, Q6_K: 210}


def build(force=False):
    src = os.path.join(_HERE, "strix_oracle.c")
    if force or not os.path.exists(_SO) or os.path.getmtime(_SO) < os.path.getmtime(src):
        subprocess.check_call(["make", "-s", "-C", _HERE] + (["-B"] if force else []))
    return _SO


_lib = None


def lib():
    global _lib
    if _lib is None:
        build()
        L = C.CDLL(_SO)
        u8p, f32p, i8p, i32p = (C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.POINTER(C.c_int8),
                                C.POINTER(C.c_int32))
        L.so_f16_to_f32.restype = C.c_float
        L.so_f16_to_f32.argtypes = [C.c_uint16]
        L.so_dequantize_into.restype = C.c_int
        L.so_dequantize_into.argtypes = [C.c_int, u8p, C.c_size_t, f32p, C.c_size_t]
        L.so_dot_f32.restype = C.c_float
        L.so_dot_f32.argtypes = [f32p, f32p, C.c_size_t]
        L.so_qmatmul.restype = C.c_int
        L.so_qmatmul.argtypes = [f32p, f32p, u8p, C.c_int, C.c_size_t, C.c_size_t, C.c_int]
        L.so_qmatmul_batch.restype = C.c_int
        L.so_qmatmul_batch.argtypes = [f32p, f32p, C.c_size_t, u8p, C.c_int, C.c_size_t, C.c_size_t, C.c_int]
        L.so_rmsnorm.restype = None
        L.so_rmsnorm.argtypes = [f32p, f32p, f32p, C.c_size_t, C.c_float]
        L.so_swiglu.restype = None
        L.so_swiglu.argtypes = [f32p, f32p, C.c_size_t]
        L.so_geglu.restype = None
        L.so_geglu.argtypes = [f32p, f32p, f32p, C.c_size_t]
        L.so_xquant8.restype = C.c_size_t
        L.so_xquant8.argtypes = [f32p, C.c_size_t, i8p, f32p]
        L.so_idot_gemm.restype = C.c_int
        L.so_idot_gemm.argtypes = [f32p, u8p, C.c_int, i8p, f32p, C.c_size_t, C.c_size_t, C.c_size_t,
                                   i32p, C.c_int]
        _lib = L
    return _lib


def _p(a, ty):
    return a.ctypes.data_as(C.POINTER(ty))


def _u8(b):
    a = np.frombuffer(b, dtype=np.uint8) if not isinstance(b, np.ndarray) else b
    return np.ascontiguousarray(a, dtype=np.uint8)


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def default_threads():
    return os.cpu_count() or 1


def f16_to_f32(h):
    return float(lib().so_f16_to_f32(int(h) & 0xFFFF))


def dequantize(ty, data, n):
    """ggml_quant.rs dequantize(): raises ValueError on the reference's error cases."""
    b = _u8(data)
    out = np.zeros(n, dtype=np.float32)
    rc = lib().so_dequantize_into(ty, _p(b, C.c_uint8), b.size, _p(out, C.c_float), n)
    if rc != 0:
        raise ValueError({-1: "element count not a multiple of the block size",
                          -2: "too few bytes", -3: "unsupported type"}[rc])
    return out


def dot_f32(a, b):
    a, b = _f32(a), _f32(b)
    return float(lib().so_dot_f32(_p(a, C.c_float), _p(b, C.c_float), min(a.size, b.size)))


def qmatmul(x, data, ty, in_dim, out_dim, threads=None):
    x, b = _f32(x), _u8(data)
    assert x.size == in_dim
    out = np.empty(out_dim, dtype=np.float32)
    rc = lib().so_qmatmul(_p(out, C.c_float), _p(x, C.c_float), _p(b, C.c_uint8), ty, in_dim, out_dim,
                          threads or default_threads())
    if rc != 0:
        raise ValueError("bad shape")
    return out


def qmatmul_batch(xs, m, data, ty, in_dim, out_dim, threads=None):
    xs, b = _f32(xs).reshape(-1), _u8(data)
    assert xs.size == m * in_dim
    out = np.empty((m, out_dim), dtype=np.float32)
    rc = lib().so_qmatmul_batch(_p(out, C.c_float), _p(xs, C.c_float), m, _p(b, C.c_uint8), ty, in_dim,
                                out_dim, threads or default_threads())
    if rc != 0:
        raise ValueError("bad shape")
    return out


def rmsnorm(x, w, eps):
    x, w = _f32(x), _f32(w)
    out = np.empty_like(x)
    lib().so_rmsnorm(_p(out, C.c_float), _p(x, C.c_float), _p(w, C.c_float), x.size, eps)
    return out


def swiglu(gate, up):
    g, u = _f32(gate).copy(), _f32(up)
    lib().so_swiglu(_p(g, C.c_float), _p(u, C.c_float), g.size)
    return g


def geglu(gate, up):
    g, u = _f32(gate), _f32(up)
    out = np.empty_like(g)
    lib().so_geglu(_p(out, C.c_float), _p(g, C.c_float), _p(u, C.c_float), g.size)
    return out


def xquant8(x):
    """Returns (q int8[n], d f32[n/32], ties)."""
    x = _f32(x).reshape(-1)
    assert x.size % 32 == 0
    q = np.empty(x.size, dtype=np.int8)
    d = np.empty(x.size // 32, dtype=np.float32)
    ties = lib().so_xquant8(_p(x, C.c_float), x.size, _p(q, C.c_int8), _p(d, C.c_float))
    return q, d, int(ties)


def idot_gemm(data, ty, xq, xd, m, in_dim, out_dim, want_isums=False, threads=None):
    """Integer-dot GEMV (m=1) / W8A8 GEMM. Returns y[m][out] (and isums[m][out][in/32])."""
    b = _u8(data)
    xq = np.ascontiguousarray(xq, dtype=np.int8).reshape(-1)
    xd = _f32(xd).reshape(-1)
    assert xq.size == m * in_dim and xd.size == m * in_dim // 32
    y = np.empty((m, out_dim), dtype=np.float32)
    isums = np.empty((m, out_dim, in_dim // 32), dtype=np.int32) if want_isums else None
    rc = lib().so_idot_gemm(_p(y, C.c_float), _p(b, C.c_uint8), ty, _p(xq, C.c_int8), _p(xd, C.c_float), m,
                            in_dim, out_dim, _p(isums, C.c_int32) if want_isums else None,
                            threads or default_threads())
    if rc != 0:
        raise ValueError("bad shape or type")
    return (y, isums) if want_isums else y


def argmax_f32(x):
    """Greedy argmax with the reference kernel's semantics (crates/strix-backend-rocm/src/kernels.rs:2088-2110):
    the running best starts at (-3.0e38, index 0) and is replaced only by a GREATER value, so NaN never
    wins and a row with nothing above -3.0e38 gives 0; ties resolve to the lowest index. Pure numpy."""
    x = _f32(x).reshape(-1)
    with np.errstate(invalid="ignore"):
        ok = x > np.float32(-3.0e38)          # False for NaN
    if not ok.any():
        return 0
    masked = np.where(ok, x, -np.inf)
    return int(np.argmax(masked))             # numpy returns the first (lowest) index of the maximum


# ---- single-token attention of the dense Qwen3 forward (crates/strix-backend-cpu/src/qwen3.rs) ----
def rmsnorm_inplace(v, w, eps):
    """qwen3.rs:117-124: v * (1 / sqrt(mean(v^2) + eps)) * w, over one head."""
    v = _f32(v)
    ss = np.float32(0.0)
    for x in v:                      # the reference's sequential f32 sum
        ss = np.float32(ss + x * x)
    scale = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(v.size) + np.float32(eps)))
    return (v * scale * _f32(w)).astype(np.float32)


def rope_neox(vec, pos, n_dims, freq_base):
    """qwen3.rs:126-138: pairs (k, k + half); theta starts at pos and is multiplied by
    freq_base^(-2/n_dims) once per pair, all in f32."""
    vec = _f32(vec).copy()
    half = n_dims // 2
    theta_scale = np.float32(np.power(np.float32(freq_base), np.float32(-2.0) / np.float32(n_dims)))
    theta = np.float32(pos)
    for k in range(half):
        s, c = np.float32(np.sin(theta)), np.float32(np.cos(theta))
        x0, x1 = vec[k], vec[k + half]
        vec[k] = x0 * c - x1 * s
        vec[k + half] = x0 * s + x1 * c
        theta = np.float32(theta * theta_scale)
    return vec


def attention_token(q, k, v, q_norm, k_norm, pos, kc, vc, n_heads, n_kv, hd, eps, freq_base):
    """One token of qwen3.rs:823-873: per-head QK-norm then rope, append k / v to the caches (python
    lists of rows, one per position), softmax(q k^T / sqrt(hd)) v per head with grouped-query sharing.
    q_norm / k_norm None = no QK-norm. Returns attn[n_heads * hd]."""
    q, k, v = _f32(q).copy(), _f32(k).copy(), _f32(v)
    for hh in range(n_heads):
        qh = q[hh * hd:(hh + 1) * hd]
        if q_norm is not None:
            qh = rmsnorm_inplace(qh, q_norm, eps)
        q[hh * hd:(hh + 1) * hd] = rope_neox(qh, pos, hd, freq_base)
    for kh in range(n_kv):
        kk = k[kh * hd:(kh + 1) * hd]
        if k_norm is not None:
            kk = rmsnorm_inplace(kk, k_norm, eps)
        k[kh * hd:(kh + 1) * hd] = rope_neox(kk, pos, hd, freq_base)
    assert len(kc) == pos and len(vc) == pos
    kc.append(k)
    vc.append(v.copy())
    K = np.stack(kc).reshape(pos + 1, n_kv, hd)
    V = np.stack(vc).reshape(pos + 1, n_kv, hd)
    scale = np.float32(1.0) / np.sqrt(np.float32(hd))
    groups = n_heads // n_kv
    out = np.zeros(n_heads * hd, dtype=np.float32)
    for hh in range(n_heads):
        kvh = hh // groups
        qh = q[hh * hd:(hh + 1) * hd]
        scores = np.array([dot_f32(qh, K[t, kvh]) for t in range(pos + 1)], dtype=np.float32) * scale
        e = np.exp(scores - scores.max()).astype(np.float32)
        o = np.zeros(hd, dtype=np.float32)
        for t in range(pos + 1):
            o += e[t] * V[t, kvh]
        out[hh * hd:(hh + 1) * hd] = o * (np.float32(1.0) / e.sum(dtype=np.float32))
    return out


# ---- the other attention flavours: SmolLM3 (smollm3.rs), Gemma (gemma.rs, ops.rs), f16 KV cache (kernels.rs) ----
def rope_adjacent(vec, pos, n_dims, freq_base):
    """smollm3.rs:126-138: pairs (2k, 2k + 1); the angle chain of rope_neox."""
    vec = _f32(vec).copy()
    half = n_dims // 2
    theta_scale = np.float32(np.power(np.float32(freq_base), np.float32(-2.0) / np.float32(n_dims)))
    theta = np.float32(pos)
    for k in range(half):
        s, c = np.float32(np.sin(theta)), np.float32(np.cos(theta))
        x0, x1 = vec[2 * k], vec[2 * k + 1]
        vec[2 * k] = x0 * c - x1 * s
        vec[2 * k + 1] = x0 * s + x1 * c
        theta = np.float32(theta * theta_scale)
    return vec


def rope_pow(vec, pos, theta, freq_factors=None):
    """ops.rs:159-176 rope_in_place_ff: pairs (j, j + half), inv_freq = theta^(-(2 j) / head_dim), divided by
    freq_factors[j] where given, angle = pos * inv_freq, all in f32."""
    vec = _f32(vec).copy()
    hd = vec.size
    half = hd // 2
    for j in range(half):
        ex = np.float32(-(np.float32(2.0) * np.float32(j))) / np.float32(hd)
        inv = np.float32(np.power(np.float32(theta), ex))
        if freq_factors is not None:
            inv = np.float32(inv / np.float32(freq_factors[j]))
        ang = np.float32(np.float32(pos) * inv)
        s, c = np.float32(np.sin(ang)), np.float32(np.cos(ang))
        x1, x2 = vec[j], vec[j + half]
        vec[j] = x1 * c - x2 * s
        vec[j + half] = x2 * c + x1 * s
    return vec


def softcap(x, cap):
    """ops.rs:127-135 softcap_inplace: cap * tanh(x * (1 / cap)); cap <= 0 leaves x alone."""
    x = _f32(x)
    if cap <= 0:
        return x.copy()
    inv = np.float32(1.0) / np.float32(cap)
    return (np.float32(cap) * np.tanh(x * inv)).astype(np.float32)


def addnorm(h, x, w, eps, out_scale=1.0):
    """gemma.rs:268-275 norm, then the sandwich residual gemma.rs:876-879 / 896-906:
    (h + x * (1 / sqrt(mean(x^2) + eps)) * w) * out_scale."""
    on = rmsnorm_inplace(x, w, eps)
    return ((_f32(h) + on).astype(np.float32) * np.float32(out_scale)).astype(np.float32)


def f32_to_f16_cache(x):
    """f2h of the reference's f16 KV cache (kernels.rs:18-32): to nearest, a tie AWAY from zero (numpy's own
    conversion rounds ties to even), overflow and NaN to infinity. Returns uint16 words."""
    b = _f32(x).view(np.uint32).astype(np.uint64)
    sign = (b >> 16) & 0x8000
    a = b & 0x7FFFFFFF
    normal = ((a + 0x1000) >> 13) - (112 << 10)
    mant = (a & 0x7FFFFF) | 0x800000
    shift = np.clip(125 - (a >> 23).astype(np.int64), 0, 63).astype(np.uint64)
    sub = ((mant >> shift) + 1) >> 1
    h = np.where(a >= 0x47800000, 0x7C00, np.where(a >= 0x38800000, normal, np.where(a < 0x33000000, 0, sub)))
    return (sign | h).astype(np.uint16)


def f16_cache_to_f32(hw):
    """h2f (kernels.rs:8-16): exact."""
    return np.asarray(hw, dtype=np.uint16).view(np.float16).astype(np.float32)


def attention_token_flavour(q, k, v, q_norm, k_norm, pos, kc, vc, n_heads, n_kv, hd, eps, rope, adjacent=False,
                            norm_v=False, window=0, scale=None, kv_f16=False):
    """One token of attention in the flavours of smollm3.rs:590-648 and gemma.rs:779-872.
    v None: the layer shares K and V, V is the RAW k (gemma.rs:796-803). q_norm / k_norm None: no QK-norm.
    rope: None | ("chain", base) (qwen3.rs / smollm3.rs) | ("pow", theta, freq_factors or None) (ops.rs:159-176).
    norm_v: V RMS-normed per head without a weight (gemma.rs:804-813). window > 0: only the last `window` cached
    rows are attended to (gemma.rs:840-851). kv_f16: rows pass through the f16 cache (kernels.rs:1984-1995, KVLD).
    kc / vc: python lists of cached rows (already rounded when kv_f16), one per position. Returns attn[n_heads * hd]."""
    q, k = _f32(q).copy(), _f32(k).copy()
    vv = k.copy() if v is None else _f32(v).copy()
    if norm_v:
        ones = np.ones(hd, dtype=np.float32)
        for kh in range(n_kv):
            vv[kh * hd:(kh + 1) * hd] = rmsnorm_inplace(vv[kh * hd:(kh + 1) * hd], ones, eps)

    def rot(x):
        if rope is None:
            return x
        if rope[0] == "chain":
            return rope_adjacent(x, pos, hd, rope[1]) if adjacent else rope_neox(x, pos, hd, rope[1])
        assert not adjacent
        return rope_pow(x, pos, rope[1], rope[2])

    for hh in range(n_heads):
        qh = q[hh * hd:(hh + 1) * hd]
        if q_norm is not None:
            qh = rmsnorm_inplace(qh, q_norm, eps)
        q[hh * hd:(hh + 1) * hd] = rot(qh)
    for kh in range(n_kv):
        kk = k[kh * hd:(kh + 1) * hd]
        if k_norm is not None:
            kk = rmsnorm_inplace(kk, k_norm, eps)
        k[kh * hd:(kh + 1) * hd] = rot(kk)
    if kv_f16:
        k, vv = f16_cache_to_f32(f32_to_f16_cache(k)), f16_cache_to_f32(f32_to_f16_cache(vv))
    assert len(kc) == pos and len(vc) == pos
    kc.append(k)
    vc.append(vv)
    length = pos + 1
    first = length - min(length, window) if window > 0 else 0
    K = np.stack(kc[first:]).reshape(length - first, n_kv, hd)
    V = np.stack(vc[first:]).reshape(length - first, n_kv, hd)
    sc = np.float32(1.0) / np.sqrt(np.float32(hd)) if scale is None else np.float32(scale)
    groups = n_heads // n_kv
    out = np.zeros(n_heads * hd, dtype=np.float32)
    for hh in range(n_heads):
        kvh = hh // groups
        qh = q[hh * hd:(hh + 1) * hd]
        scores = np.array([dot_f32(qh, K[t, kvh]) for t in range(length - first)], dtype=np.float32) * sc
        e = np.exp(scores - scores.max()).astype(np.float32)          # ops.rs:50-72 softmax_inplace
        e = (e * (np.float32(1.0) / e.sum(dtype=np.float32))).astype(np.float32)
        o = np.zeros(hd, dtype=np.float32)
        for t in range(length - first):
            o += e[t] * V[t, kvh]
        out[hh * hd:(hh + 1) * hd] = o
    return out


# ---- mixture-of-experts FFN (crates/strix-backend-cpu/src/mellum.rs:1582-1663) ----
def topk_router(logits, k):
    """mellum.rs:1590-1609: p = exp(l - max) then p /= sum (sequential f32 sum), the k largest by a STABLE
    descending sort (a tie keeps the lower index first), weights p[e] / (sum of the chosen p, in that order).
    Returns (ids int32[k], weights f32[k])."""
    l = _f32(logits)
    mx = l.max()
    p = np.exp((l - mx).astype(np.float32)).astype(np.float32)
    s = np.float32(0.0)
    for v in p:
        s = np.float32(s + v)
    p = (p / s).astype(np.float32)
    idx = sorted(range(p.size), key=lambda e: -float(p[e]))[:k]      # python's sort is stable
    ws = np.float32(0.0)
    for e in idx:
        ws = np.float32(ws + p[e])
    return np.array(idx, dtype=np.int32), np.array([p[e] / ws for e in idx], dtype=np.float32)


def moe_expert_bytes(ty, hidden, eff):
    """Bytes of one expert's gate (= up) matrix and of its down matrix (mellum.rs:1620-1622)."""
    be, bb = BLOCK_ELEMS[ty], BLOCK_BYTES[ty]
    return (hidden // be) * bb * eff, (eff // be) * bb * hidden


def moe_expert_ffn(x, gate, up, down, ty, hidden, eff, e, int8=False):
    """mellum.rs:1629-1654 for expert e and one token: down_e(silu(gate_e x) * up_e x); the expert's blocks are the
    e-th slice of the layer's tensors. int8: activations through the per-32 int8 quantiser before each matmul
    (the reference's q8i_moe_* kernels)."""
    gb, db = moe_expert_bytes(ty, hidden, eff)

    def mm(data, xv, k, n):
        if int8:
            xq, xd, _ = xquant8(xv)
            return idot_gemm(data, ty, xq, xd, 1, k, n)[0]
        return qmatmul(xv, data, ty, k, n)

    g = mm(_u8(gate)[e * gb:(e + 1) * gb], x, hidden, eff)
    u = mm(_u8(up)[e * gb:(e + 1) * gb], x, hidden, eff)
    return mm(_u8(down)[e * db:(e + 1) * db], swiglu(g, u), eff, hidden)


def moe_ffn(x, gate, up, down, ty, hidden, eff, ids, wexp, int8=False):
    """mellum.rs:1624-1660: out += wexp[i] * expert_{ids[i]}(x), in the order given, multiply then add in f32."""
    out = np.zeros(hidden, dtype=np.float32)
    for e, w in zip(ids, _f32(wexp)):
        dy = moe_expert_ffn(x, gate, up, down, ty, hidden, eff, int(e), int8)
        out = (out + (np.float32(w) * dy).astype(np.float32)).astype(np.float32)
    return out
