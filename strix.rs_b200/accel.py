"""Python mirror of the reference's ``WeightAccel`` trait over the C ABI.

Method names, argument meaning and the None/False "declined" convention follow
``crates/strix-core/src/accel.rs:147-507`` so that tests read like calls into the
reference: ``upload_q4_0(key, bytes, in_dim, out_dim) -> bool``,
``gemv(key, x) -> array | None``, ...  Every method goes through
``libstrix_cuda.so``; nothing is computed in Python and there is no CPU fallback:
if the library is missing, loading raises.
"""
import ctypes as C
import os

import numpy as np

ACT_F32, ACT_Q8DOT = 0, 1
PRE_NONE, PRE_RMSNORM, PRE_SWIGLU, PRE_GEGLU = 0, 1, 2, 3

_HERE = os.path.dirname(os.path.abspath(__file__))


class StrixCudaError(RuntimeError):
    pass


def library_path():
    return os.path.join(_HERE, "lib", "libstrix_cuda.so")


class _Opts(C.Structure):
    _fields_ = [("rank", C.c_int), ("world", C.c_int), ("profile", C.c_int), ("reserved", C.c_int * 5)]


class _LayerCfg(C.Structure):
    _fields_ = [("head_dim", C.c_uint32), ("n_kv", C.c_uint32), ("k_eq_v", C.c_int), ("rope_theta", C.c_float),
                ("is_local", C.c_int), ("output_scale", C.c_float), ("no_rope", C.c_int), ("rope_norm", C.c_int)]


class _DecodeCfg(C.Structure):
    _fields_ = [("hidden", C.c_uint32), ("n_heads", C.c_uint32), ("ffn", C.c_uint32), ("vocab", C.c_uint32),
                ("n_layers", C.c_uint32), ("eps", C.c_float), ("final_softcap", C.c_float), ("attn_rsqrt", C.c_int),
                ("norm_v", C.c_int), ("qk_norm", C.c_int), ("post_norm", C.c_int), ("act_gelu", C.c_int),
                ("gpu_prefill", C.c_int), ("n_swa", C.c_uint32), ("max_seq", C.c_uint32),
                ("layers", C.POINTER(_LayerCfg)), ("attn_standin_q", C.c_int), ("act", C.c_int)]


_lib = None


def load_library():
    """Loads libstrix_cuda.so and declares every entry point of include/strix_cuda.h."""
    global _lib
    if _lib is not None:
        return _lib
    path = library_path()
    if not os.path.exists(path):
        raise StrixCudaError("%s is missing: run strix.rs_b200/build.py (there is no fallback path)" % path)
    L = C.CDLL(path)
    H = C.c_void_p
    u8p, f32p, sz = C.POINTER(C.c_uint8), C.POINTER(C.c_float), C.c_size_t
    szp = C.POINTER(C.c_size_t)

    def sig(name, res, *args):
        f = getattr(L, name)
        f.restype, f.argtypes = res, list(args)

    sig("strix_cuda_create", C.c_int, C.c_int, C.POINTER(_Opts), C.POINTER(H))
    sig("strix_cuda_destroy", None, H)
    sig("strix_cuda_last_error", C.c_char_p, H)
    sig("strix_cuda_create_error", C.c_char_p)
    sig("strix_cuda_name", C.c_char_p, H)
    sig("strix_cuda_resident_count", sz, H)
    for q in ("q4_0", "q8_0", "q6_k", "q4_1"):
        sig("strix_cuda_upload_" + q, C.c_int, H, C.c_char_p, u8p, sz, sz, sz)
    sig("strix_cuda_upload_f32", C.c_int, H, C.c_char_p, f32p, sz)
    sig("strix_cuda_weight_info", C.c_int, H, C.c_char_p, szp, szp, szp, szp, C.POINTER(C.c_int))
    sig("strix_cuda_gemv", C.c_int, H, C.c_char_p, f32p, sz, f32p, sz, C.c_int)
    sig("strix_cuda_gemv_batch", C.c_int, H, sz, C.POINTER(C.c_char_p), C.POINTER(C.c_void_p), szp, C.POINTER(C.c_void_p), szp,
        C.c_int, C.POINTER(C.c_int))
    sig("strix_cuda_gemv_batch_dev", C.c_int, H, sz, C.POINTER(C.c_char_p), C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_int,
        C.c_void_p)
    sig("strix_cuda_profile_dump", C.c_size_t, H, C.c_char_p, C.c_size_t)
    sig("strix_cuda_gemv_batch_peers_dev", C.c_int, H, sz, C.POINTER(C.c_char_p), C.POINTER(C.c_void_p), C.c_int,
        C.POINTER(C.c_void_p), C.c_int, C.c_void_p)
    sig("strix_cuda_gemv_dev", C.c_int, H, C.c_int, C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p, C.c_float,
        C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_void_p)
    sig("strix_cuda_gemv_res_dev", C.c_int, H, C.c_int, C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p, C.c_float,
        C.c_int, C.c_int, C.POINTER(C.c_void_p), C.POINTER(C.c_void_p), C.c_void_p)
    sig("strix_cuda_gemv_peers_dev", C.c_int, H, C.c_int, C.POINTER(C.c_char_p), C.c_void_p, C.c_void_p, C.c_float,
        C.c_int, C.c_int, C.POINTER(C.c_void_p), C.c_int, C.POINTER(C.c_void_p), C.c_void_p)
    sig("strix_cuda_enable_peer_access", C.c_int, H, C.c_int)
    sig("strix_cuda_ipc_open", C.c_int, H, C.c_char_p, sz, C.POINTER(C.c_void_p))
    sig("strix_cuda_ipc_close", C.c_int, H, C.c_void_p)
    sig("strix_cuda_ipc_export", C.c_int, H, C.c_void_p, C.c_char_p, sz)
    sig("strix_cuda_peek_u32", C.c_int, H, C.c_void_p, C.POINTER(C.c_uint32))
    sig("strix_cuda_poke_u32", C.c_int, H, C.c_void_p, C.c_uint32)
    sig("strix_cuda_peer_barrier_dev", C.c_int, H, C.c_void_p, C.c_void_p, C.POINTER(C.c_void_p), C.c_void_p)
    sig("strix_cuda_prefill_q8_gemm", C.c_int, H, C.c_char_p, f32p, sz, f32p, sz)
    sig("strix_cuda_prefill_q8_gemm_dev", C.c_int, H, C.c_char_p, C.c_void_p, sz, C.c_void_p, C.c_void_p)
    sig("strix_cuda_prefill_q8_gemm_noalloc", C.c_int, H, C.c_char_p, C.c_void_p, sz, C.c_void_p, C.c_void_p)
    sig("strix_cuda_noalloc_scratch_bytes", sz)
    sig("strix_cuda_debug_block_isums", C.c_int, H, C.c_char_p, f32p, sz, C.POINTER(C.c_int32), sz)
    sig("strix_cuda_configure_decode", C.c_int, H, C.POINTER(_DecodeCfg))
    sig("strix_cuda_decode_step", C.c_int, H, f32p, sz, f32p, sz)
    sig("strix_cuda_decode_chain_dev", C.c_int, H, C.c_void_p, C.c_void_p, C.c_void_p)
    sig("strix_cuda_decode_step_argmax", C.c_int, H, f32p, sz, C.POINTER(C.c_uint32))
    sig("strix_cuda_prefill", C.c_int, H, f32p, sz, sz, f32p, sz)
    sig("strix_cuda_verify", C.c_int, H, f32p, sz, sz, f32p, sz)
    sig("strix_cuda_prefill_max", sz, H)
    sig("strix_cuda_seed_decode_kv", C.c_int, H, sz, f32p, f32p, sz)
    sig("strix_cuda_lm_head_argmax_rows", C.c_int, H, C.c_char_p, f32p, sz, sz, C.c_int, C.POINTER(C.c_uint32), f32p)
    sig("strix_cuda_argmax_dev", C.c_int, H, C.c_void_p, sz, sz, sz, C.c_void_p, C.c_void_p, C.c_void_p)
    sig("strix_cuda_gemv_rows", C.c_int, H, C.c_char_p, f32p, sz, f32p, sz, C.c_int)
    sig("strix_cuda_gemv_rows_dev", C.c_int, H, C.c_int, C.POINTER(C.c_char_p), C.c_void_p, sz, C.c_int,
        C.POINTER(C.c_void_p), C.c_void_p)
    sig("strix_cuda_device_status", C.c_int, H, C.c_void_p, C.POINTER(C.c_uint32))
    sig("strix_cuda_clear_device_status", C.c_int, H, C.c_void_p)
    sig("strix_cuda_dequant_to_f32", C.c_int, H, C.c_char_p, f32p, sz)
    sig("strix_cuda_xquant8", C.c_int, H, f32p, sz, C.POINTER(C.c_int8), f32p)
    sig("strix_cuda_fold_argmax_shards", None, sz, sz, C.POINTER(C.c_uint32), f32p, C.POINTER(C.c_uint32), f32p)
    sig("strix_cuda_prefill_q4_gemm", C.c_int, H, C.c_char_p, f32p, sz, f32p, sz)
    sig("strix_cuda_prefill_q4_gemm_dev", C.c_int, H, C.c_char_p, C.c_void_p, sz, C.c_void_p, C.c_void_p)
    i32p = C.POINTER(C.c_int32)
    for nm in ("strix_cuda_upload_moe_q8", "strix_cuda_upload_moe_q6"):
        sig(nm, C.c_int, H, sz, u8p, sz, u8p, sz, u8p, sz, sz, sz, sz)
    sig("strix_cuda_moe_ffn", C.c_int, H, sz, i32p, f32p, sz, f32p, sz, C.c_float, C.c_int, f32p, sz)
    sig("strix_cuda_moe_ffn_dev", C.c_int, H, sz, C.c_void_p, C.c_void_p, sz, C.c_void_p, C.c_float, C.c_int, C.c_void_p, C.c_void_p)
    sig("strix_cuda_moe_expert_ffn", C.c_int, H, sz, sz, f32p, sz, C.c_int, f32p, sz)
    sig("strix_cuda_moe_layer_ffn", C.c_int, H, sz, i32p, sz, f32p, sz, C.c_int, f32p, sz)
    sig("strix_cuda_topk_router", C.c_int, H, f32p, sz, sz, i32p, f32p)
    sig("strix_cuda_topk_router_dev", C.c_int, H, C.c_void_p, sz, sz, C.c_void_p, C.c_void_p, C.c_void_p)
    sig("strix_cuda_debug_gemm_isums", C.c_int, H, C.c_char_p, f32p, sz, C.c_uint32, C.POINTER(C.c_int32), sz)
    sig("strix_cuda_debug_gemm_mode_dev", C.c_int, H, C.c_char_p, C.c_void_p, sz, C.c_void_p, C.c_int, C.c_int, C.c_void_p)
    sig("strix_cuda_decode_exchange_info", C.c_int, H, C.POINTER(C.c_void_p), szp)
    sig("strix_cuda_decode_set_peers", C.c_int, H, C.c_int, C.POINTER(C.c_void_p))
    sig("strix_cuda_set_option", C.c_int, H, C.c_char_p, C.c_longlong)
    sig("strix_cuda_decode_trace", C.c_int, H, C.POINTER(C.c_uint64), sz)
    _lib = L
    return L


def shard_begin(rows, world, r):
    """First row of rank r's shard (contiguous shards, sizes differ by at most one)."""
    if world <= 1:
        return 0 if r <= 0 else rows
    q, rem = divmod(rows, world)
    return r * q + min(r, rem)


def _u8(b):
    a = b if isinstance(b, np.ndarray) else np.frombuffer(b, dtype=np.uint8)
    return np.ascontiguousarray(a.reshape(-1), dtype=np.uint8)


def _f32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.float32).reshape(-1))


def _fp(a):
    return a.ctypes.data_as(C.POINTER(C.c_float))


def fold_argmax_shards(ids, vals):
    """Fold the per-shard winners of ``lm_head_argmax_rows`` (one (ids[m], vals[m]) pair per row shard, in
    rank order) into the winners over the whole weight (strix_cuda_fold_argmax_shards: the device kernel's rule)."""
    L = load_library()
    ids = np.ascontiguousarray(np.asarray(ids, dtype=np.uint32))
    vals = np.ascontiguousarray(np.asarray(vals, dtype=np.float32))
    n, m = ids.shape
    out = np.zeros(m, dtype=np.uint32)
    L.strix_cuda_fold_argmax_shards(n, m, ids.ctypes.data_as(C.POINTER(C.c_uint32)), _fp(vals),
                                    out.ctypes.data_as(C.POINTER(C.c_uint32)), None)
    return out


class CudaWeightAccel:
    """``impl WeightAccel`` for one CUDA device (the hot-path methods only)."""

    def __init__(self, device=0, rank=0, world=1, profile=False):
        self._L = load_library()
        self._h = C.c_void_p()
        o = _Opts(rank=rank, world=world, profile=int(profile))
        rc = self._L.strix_cuda_create(device, C.byref(o), C.byref(self._h))
        if rc != 1:
            self._h = None
            raise StrixCudaError(self._L.strix_cuda_create_error().decode())
        self.device, self.rank, self.world = device, rank, world

    # -- lifetime ---------------------------------------------------------
    def close(self):
        if getattr(self, "_h", None):
            self._L.strix_cuda_destroy(self._h)
            self._h = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    def _check(self, rc):
        if rc < 0:
            raise StrixCudaError(self._L.strix_cuda_last_error(self._h).decode())
        return rc

    # -- trait methods ----------------------------------------------------
    def name(self):
        return self._L.strix_cuda_name(self._h).decode()

    def resident_count(self):
        return int(self._L.strix_cuda_resident_count(self._h))

    def _upload(self, fn, key, data, in_dim, out_dim):
        self._rows = {}
        b = _u8(data)
        rc = fn(self._h, key.encode(), b.ctypes.data_as(C.POINTER(C.c_uint8)), b.size, in_dim, out_dim)
        return self._check(rc) == 1

    def upload_q4_0(self, key, data, in_dim, out_dim):
        return self._upload(self._L.strix_cuda_upload_q4_0, key, data, in_dim, out_dim)

    def upload_q4_1(self, key, data, in_dim, out_dim):
        return self._upload(self._L.strix_cuda_upload_q4_1, key, data, in_dim, out_dim)

    def upload_q8_0(self, key, data, in_dim, out_dim):
        return self._upload(self._L.strix_cuda_upload_q8_0, key, data, in_dim, out_dim)

    def upload_q6_k(self, key, data, in_dim, out_dim):
        return self._upload(self._L.strix_cuda_upload_q6_k, key, data, in_dim, out_dim)

    def upload_f32(self, key, data):
        a = _f32(data)
        self._check(self._L.strix_cuda_upload_f32(self._h, key.encode(), _fp(a), a.size))

    def weight_info(self, key):
        """None, or dict(in_dim, out_dim, row0, rows, ggml_type) for an adopted weight."""
        v = [C.c_size_t() for _ in range(4)]
        t = C.c_int()
        rc = self._check(self._L.strix_cuda_weight_info(self._h, key.encode(), *[C.byref(x) for x in v], C.byref(t)))
        if rc == 0:
            return None
        return dict(in_dim=v[0].value, out_dim=v[1].value, row0=v[2].value, rows=v[3].value, ggml_type=t.value)

    def gemv(self, key, x, act=ACT_F32):
        """y = W x, or None when `key` is not resident or len(x) != in_dim."""
        info = self.weight_info(key)
        if info is None:
            return None
        xa = _f32(x)
        y = np.empty(info["rows"], dtype=np.float32)
        rc = self._check(self._L.strix_cuda_gemv(self._h, key.encode(), _fp(xa), xa.size, _fp(y), y.size, act))
        return y if rc == 1 else None

    def gemv_batch(self, calls, act=ACT_F32):
        """calls = [(key, x), ...] -> [array | None, ...] with one device sync."""
        n = len(calls)
        if n == 0:
            return []
        # What depends on the keys only (their C strings, the rows each weight holds here, the capacity array) is
        # kept until the next upload: a token step repeats the same batch.
        plans = getattr(self, "_rows", None)
        if plans is None:
            plans = self._rows = {}
        names = tuple(k for k, _ in calls)
        plan = plans.get(names)
        if plan is None:
            infos = [self.weight_info(k) for k in names]
            nrows = [i["rows"] if i else None for i in infos]
            plan = plans[names] = (nrows, (C.c_char_p * n)(*[k.encode() for k in names]),
                                   (C.c_size_t * n)(*[r or 0 for r in nrows]), (C.c_int * n)())
        nrows, keys, yc, st = plan
        xs = [_f32(x) for _, x in calls]
        ys = [np.empty(r or 0, dtype=np.float32) for r in nrows]
        xp = (C.c_void_p * n)(*[x.ctypes.data for x in xs])
        yp = (C.c_void_p * n)(*[y.ctypes.data for y in ys])
        ks = (C.c_size_t * n)(*[x.size for x in xs])
        self._check(self._L.strix_cuda_gemv_batch(self._h, n, keys, xp, ks, yp, yc, act, st))
        return [ys[i] if (nrows[i] is not None and st[i] == 1) else None for i in range(n)]

    def gemv_rows(self, key, xs, b, act=ACT_F32):
        """ys[b][rows] = W xs[b][in_dim]: b activation rows, one pass over the weights. None if not resident."""
        info = self.weight_info(key)
        xa = _f32(xs)
        if info is None or xa.size != b * info["in_dim"]:
            return None
        y = np.empty((b, info["rows"]), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_gemv_rows(self._h, key.encode(), _fp(xa), b, _fp(y), y.size, act))
        return y if rc == 1 else None

    def gemv_rows_dev(self, keys, d_xs, b, d_ys, act=ACT_F32, stream=0):
        n = len(keys)
        kk = (C.c_char_p * n)(*[k.encode() for k in keys])
        yy = (C.c_void_p * n)(*[int(p) for p in d_ys])
        rc = self._check(self._L.strix_cuda_gemv_rows_dev(self._h, n, kk, C.c_void_p(int(d_xs)), b, act, yy,
                                                         C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def prefill_q8_gemm(self, key, xs, m):
        """y[m][out] = W8A8 GEMM on a resident Q8_0 weight, or None (unknown key / not Q8_0 / bad length)."""
        info = self.weight_info(key)
        xa = _f32(xs)
        if info is None or xa.size != m * info["in_dim"]:
            return None
        y = np.empty((m, info["rows"]), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_prefill_q8_gemm(self._h, key.encode(), _fp(xa), m, _fp(y), y.size))
        return y if rc == 1 else None

    def prefill_q4_gemm(self, key, xs, m):
        """The prefill GEMM with a resident Q4_0 weight (q4_gemm_w, kernels.rs:443-601): [m][rows] f32 or None."""
        info = self.weight_info(key)
        xa = _f32(xs)
        if info is None or xa.size != m * info["in_dim"]:
            return None
        y = np.empty((m, info["rows"]), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_prefill_q4_gemm(self._h, key.encode(), _fp(xa), m, _fp(y), y.size))
        return y if rc == 1 else None

    # ---- mixture-of-experts layers (accel.rs:167-246) ----
    def _upload_moe(self, fn, layer, gate, up, down, hidden, eff, ne):
        self._rows = {}
        g, u, d = (np.ascontiguousarray(np.frombuffer(b, dtype=np.uint8) if not isinstance(b, np.ndarray) else b.view(np.uint8))
                   for b in (gate, up, down))
        u8 = lambda a: a.ctypes.data_as(C.POINTER(C.c_uint8))
        rc = self._check(fn(self._h, layer, u8(g), g.size, u8(u), u.size, u8(d), d.size, hidden, eff, ne))
        if rc == 1:
            self._moe = getattr(self, "_moe", {})
            self._moe[layer] = (hidden, eff, ne)
        return rc == 1

    def upload_moe_q8(self, layer, gate, up, down, hidden, eff, ne):
        """Adopt a layer's experts in native Q8_0 blocks (accel.rs:167-181)."""
        return self._upload_moe(self._L.strix_cuda_upload_moe_q8, layer, gate, up, down, hidden, eff, ne)

    def upload_moe_q6(self, layer, gate, up, down, hidden, eff, ne):
        """Adopt a layer's experts in native Q6_K super-blocks (accel.rs:183-196)."""
        return self._upload_moe(self._L.strix_cuda_upload_moe_q6, layer, gate, up, down, hidden, eff, ne)

    def moe_ffn(self, layer, ids, wexp, x, sgate=0.0, act=ACT_F32):
        """y[hidden] of one token over its routed experts, or None (accel.rs:198-211)."""
        dims = getattr(self, "_moe", {}).get(layer)
        if dims is None:
            return None
        ia = np.ascontiguousarray(ids, dtype=np.int32)
        wa, xa = _f32(wexp), _f32(x)
        if ia.size != wa.size:
            return None
        y = np.empty(dims[0], dtype=np.float32)
        rc = self._check(self._L.strix_cuda_moe_ffn(self._h, layer, ia.ctypes.data_as(C.POINTER(C.c_int32)), _fp(wa), ia.size,
                                                     _fp(xa), xa.size, float(sgate), act, _fp(y), y.size))
        return y if rc == 1 else None

    def moe_expert_ffn(self, layer, e, xs, m, act=ACT_F32):
        """y[m][hidden]: m grouped tokens through expert e, or None (accel.rs:220-223)."""
        dims = getattr(self, "_moe", {}).get(layer)
        xa = _f32(xs)
        if dims is None or xa.size != m * dims[0] or m == 0:
            return None
        y = np.empty((m, dims[0]), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_moe_expert_ffn(self._h, layer, e, _fp(xa), m, act, _fp(y), y.size))
        return y if rc == 1 else None

    def moe_layer_ffn(self, layer, plan, xs, rows, act=ACT_F32):
        """plan: [(expert, row count)]; xs[rows][hidden] gathered expert-major -> y[rows][hidden], or None (accel.rs:236-246)."""
        dims = getattr(self, "_moe", {}).get(layer)
        xa = _f32(xs)
        if dims is None or xa.size != rows * dims[0] or rows == 0:
            return None
        pa = np.ascontiguousarray(np.asarray(plan, dtype=np.int32).reshape(-1))
        y = np.empty((rows, dims[0]), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_moe_layer_ffn(self._h, layer, pa.ctypes.data_as(C.POINTER(C.c_int32)), pa.size // 2,
                                                           _fp(xa), rows, act, _fp(y), y.size))
        return y if rc == 1 else None

    def topk_router(self, logits, k):
        """(ids[k], weights[k]) of the router's softmax top-k, or None."""
        la = _f32(logits)
        ids, w = np.zeros(k, dtype=np.int32), np.zeros(k, dtype=np.float32)
        rc = self._check(self._L.strix_cuda_topk_router(self._h, _fp(la), la.size, k, ids.ctypes.data_as(C.POINTER(C.c_int32)), _fp(w)))
        return (ids, w) if rc == 1 else None

    def prefill_q8_gemm_dev(self, key, d_xs, m, d_y, stream=0):
        rc = self._check(self._L.strix_cuda_prefill_q8_gemm_dev(self._h, key.encode(), C.c_void_p(int(d_xs)), m,
                                                               C.c_void_p(int(d_y)),
                                                               C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def prefill_q8_gemm_noalloc(self, key, d_xs, m, d_y, stream=0):
        """The GEMM with all scratch in the library's fixed device array: for callers that cannot
        allocate device memory. Raises StrixCudaError when the shape needs more than the array holds."""
        rc = self._check(self._L.strix_cuda_prefill_q8_gemm_noalloc(self._h, key.encode(), C.c_void_p(int(d_xs)), m,
                                                                   C.c_void_p(int(d_y)),
                                                                   C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def noalloc_scratch_bytes(self):
        return int(self._L.strix_cuda_noalloc_scratch_bytes())

    def debug_block_isums(self, key, xs, m):
        """int32 [m][rows][in_dim/32] block sums of the GEMM (bit-exact tier)."""
        info = self.weight_info(key)
        xa = _f32(xs)
        if info is None or xa.size != m * info["in_dim"]:
            return None
        out = np.empty((m, info["rows"], info["in_dim"] // 32), dtype=np.int32)
        rc = self._check(self._L.strix_cuda_debug_block_isums(self._h, key.encode(), _fp(xa), m,
                                                             out.ctypes.data_as(C.POINTER(C.c_int32)), out.size))
        return out if rc == 1 else None

    def debug_gemm_isums(self, key, xs, m, splits=0):
        """The same block sums as the tcgen05 GEMM kernel itself produces them (splits: split-K slices, 0 = as
        prefill_q8_gemm picks)."""
        info = self.weight_info(key)
        xa = _f32(xs)
        if info is None or xa.size != m * info["in_dim"]:
            return None
        out = np.empty((m, info["rows"], info["in_dim"] // 32), dtype=np.int32)
        rc = self._check(self._L.strix_cuda_debug_gemm_isums(self._h, key.encode(), _fp(xa), m, splits,
                                                            out.ctypes.data_as(C.POINTER(C.c_int32)), out.size))
        return out if rc == 1 else None

    def debug_gemm_mode_dev(self, key, d_xs, m, d_y, mode, reps, stream=0):
        """Measurement: quantise once, then `reps` launches of the GEMM kernel in `mode` (0 product, 2 no drain,
        3 no drain and no loads)."""
        rc = self._check(self._L.strix_cuda_debug_gemm_mode_dev(self._h, key.encode(), C.c_void_p(int(d_xs)), m,
                                                               C.c_void_p(int(d_y)), mode, reps,
                                                               C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def configure_decode(self, hidden, n_heads, ffn, vocab, n_layers, eps=1e-6, act_gelu=False, act=ACT_Q8DOT,
                         attn_standin_q=True, post_norm=False, final_softcap=0.0, head_dim=0, n_kv=0,
                         rope_theta=1e6, max_seq=0, qk_norm=True, layer_overrides=None, attn_rsqrt=True,
                         norm_v=False, n_swa=0, layers=None):
        """GpuDecodeConfig -> bool (accel.rs:417). attn_standin_q=True: the projection chain alone (Wo is
        fed with q). False: real attention (QK-norm, rope, KV cache of max_seq rows, grouped-query softmax);
        head_dim / n_kv / rope_theta describe every layer unless `layers` (a list of dicts with the GpuLayerCfg
        fields, accel.rs:19-39) gives them per layer; layer_overrides: {layer: {field: value}} on top of either.
        A post_norm model with the stand-in takes its output scales from `layers` too (default 1)."""
        lay = None
        if not attn_standin_q or layers is not None:
            lay = (_LayerCfg * n_layers)()
            for il in range(n_layers):
                f = dict(head_dim=head_dim, n_kv=n_kv, k_eq_v=0, rope_theta=rope_theta, is_local=0,
                         output_scale=1.0, no_rope=0, rope_norm=0)
                if layers is not None:
                    f.update(layers[il])
                f.update((layer_overrides or {}).get(il, {}))
                lay[il] = _LayerCfg(**f)
        c = _DecodeCfg(hidden=hidden, n_heads=n_heads, ffn=ffn, vocab=vocab, n_layers=n_layers, eps=eps,
                       final_softcap=final_softcap, attn_rsqrt=int(attn_rsqrt), norm_v=int(norm_v), qk_norm=int(qk_norm),
                       post_norm=int(post_norm), act_gelu=int(act_gelu), n_swa=n_swa, max_seq=max_seq,
                       layers=lay if lay is not None else None,
                       attn_standin_q=int(attn_standin_q), act=act)
        rc = self._check(self._L.strix_cuda_configure_decode(self._h, C.byref(c)))
        self._vocab = vocab if rc == 1 else None
        self._kvdims = [int(l.head_dim) * int(l.n_kv) for l in lay] if (rc == 1 and not attn_standin_q) else []
        self._kvdim = self._kvdims[0] if self._kvdims else 0
        return rc == 1

    def decode_step(self, h, pos=0):
        """logits[vocab] or None (accel.rs:433). A row-sharded accelerator returns its shard of the logits."""
        if not getattr(self, "_vocab", None):
            return None
        ha = _f32(h)
        out = np.empty(self._vocab, dtype=np.float32)
        rc = self._check(self._L.strix_cuda_decode_step(self._h, _fp(ha), pos, _fp(out), out.size))
        if rc != 1:
            return None
        if self.world > 1:
            return out[:shard_begin(self._vocab, self.world, self.rank + 1) - shard_begin(self._vocab, self.world, self.rank)]
        return out

    def decode_exchange_info(self):
        """(device address, bytes) of this accelerator's exchange block (row-sharded decode), or None."""
        base, n = C.c_void_p(), C.c_size_t()
        rc = self._check(self._L.strix_cuda_decode_exchange_info(self._h, C.byref(base), C.byref(n)))
        return (base.value, n.value) if rc == 1 else None

    def decode_set_peers(self, blocks):
        """blocks[r]: rank r's exchange block as mapped into this process (0 / None for this rank's own)."""
        arr = (C.c_void_p * len(blocks))(*[int(b) if b else None for b in blocks])
        return self._check(self._L.strix_cuda_decode_set_peers(self._h, len(blocks), arr)) == 1

    def prefill(self, hs, start_pos, m):
        """Logits of the last of m tokens, KV cache filled for start_pos .. start_pos+m-1, or None (accel.rs:464-473)."""
        if not getattr(self, "_vocab", None):
            return None
        ha = _f32(hs)
        out = np.empty(self._vocab, dtype=np.float32)
        rc = self._check(self._L.strix_cuda_prefill(self._h, _fp(ha), start_pos, m, _fp(out), out.size))
        return out if rc == 1 else None

    def verify(self, hs, start_pos, m):
        """Logits [m][vocab] of all m tokens, or None (accel.rs:500-506)."""
        if not getattr(self, "_vocab", None):
            return None
        ha = _f32(hs)
        out = np.empty((max(m, 1), self._vocab), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_verify(self._h, _fp(ha), start_pos, m, _fp(out), out.size))
        return out[:m] if rc == 1 else None

    def prefill_max(self):
        return int(self._L.strix_cuda_prefill_max(self._h))

    def seed_decode_kv(self, il, k, v):
        ka, va = _f32(k), _f32(v)
        kvdims = getattr(self, "_kvdims", [])
        kvdim = kvdims[il] if il < len(kvdims) else 0
        if not kvdim or ka.size != va.size or ka.size % kvdim:
            return False
        return self._check(self._L.strix_cuda_seed_decode_kv(self._h, il, _fp(ka), _fp(va), ka.size // kvdim)) == 1

    def decode_step_argmax(self, h, pos=0):
        """Greedy token id of one decode step, argmax on the device, or None (accel.rs:437-442)."""
        if not getattr(self, "_vocab", None):
            return None
        ha = _f32(h)
        out = C.c_uint32(0)
        rc = self._check(self._L.strix_cuda_decode_step_argmax(self._h, _fp(ha), pos, C.byref(out)))
        return int(out.value) if rc == 1 else None

    def lm_head_argmax_rows(self, key, xs, m, act=ACT_F32, with_values=False):
        """ids[m] = argmax over the rows of W xs[t], or None (unknown key, bad length, m > 16) (accel.rs:216-219)."""
        xa = _f32(xs)
        ids = np.zeros(max(m, 1), dtype=np.uint32)
        vals = np.zeros(max(m, 1), dtype=np.float32)
        rc = self._check(self._L.strix_cuda_lm_head_argmax_rows(
            self._h, key.encode(), _fp(xa), xa.size, m, act, ids.ctypes.data_as(C.POINTER(C.c_uint32)), _fp(vals)))
        if rc != 1:
            return None
        return (ids[:m], vals[:m]) if with_values else ids[:m]

    def argmax_dev(self, d_x, n, stride, rows, d_ids=0, d_vals=0, stream=0):
        rc = self._check(self._L.strix_cuda_argmax_dev(
            self._h, C.c_void_p(int(d_x)), n, stride, rows, C.c_void_p(int(d_ids)) if d_ids else None,
            C.c_void_p(int(d_vals)) if d_vals else None, C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def decode_chain_dev(self, d_h, d_logits, stream=0):
        rc = self._check(self._L.strix_cuda_decode_chain_dev(self._h, C.c_void_p(int(d_h)), C.c_void_p(int(d_logits)),
                                                            C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    # -- device-resident form (pointers are ints: torch ``tensor.data_ptr()``) ----
    def gemv_dev(self, keys, d_a, d_ys, d_b=0, eps=0.0, pre=PRE_NONE, act=ACT_F32, stream=0, d_res=None):
        """d_res: per-weight device pointers (0 = none) of residual vectors added to the outputs."""
        n = len(keys)
        kk = (C.c_char_p * n)(*[k.encode() for k in keys])
        yy = (C.c_void_p * n)(*[int(p) for p in d_ys])
        if d_res is not None:
            rr = (C.c_void_p * n)(*[int(p) if p else None for p in d_res])
            rc = self._check(self._L.strix_cuda_gemv_res_dev(self._h, n, kk, C.c_void_p(int(d_a)),
                                                            C.c_void_p(int(d_b)) if d_b else None, float(eps), pre, act,
                                                            yy, rr, C.c_void_p(int(stream)) if stream else None))
            return rc == 1
        rc = self._check(self._L.strix_cuda_gemv_dev(self._h, n, kk, C.c_void_p(int(d_a)),
                                                    C.c_void_p(int(d_b)) if d_b else None, float(eps), pre, act, yy,
                                                    C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def profile_dump(self):
        """Per-kernel totals since the last call (set_option("profile", 1) first), as text; resets them."""
        n = self._L.strix_cuda_profile_dump(self._h, None, 0)
        buf = C.create_string_buffer(n + 1)
        self._L.strix_cuda_profile_dump(self._h, buf, n + 1)
        return buf.value.decode()

    def gemv_batch_dev(self, keys, d_xs, d_ys, act=ACT_F32, stream=0):
        """n independent GEMVs on device vectors (ys[i] = W(keys[i]) xs[i]); the small ones run side by side in one launch."""
        n = len(keys)
        kk = (C.c_char_p * n)(*[k.encode() for k in keys])
        xx = (C.c_void_p * n)(*[int(p) for p in d_xs])
        yy = (C.c_void_p * n)(*[int(p) for p in d_ys])
        rc = self._check(self._L.strix_cuda_gemv_batch_dev(self._h, n, kk, xx, yy, act, C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def gemv_batch_peers_dev(self, keys, d_xs, peer_ys, act=ACT_F32, stream=0):
        """Row-sharded gemv_batch_dev: peer_ys[i] = the device pointers of item i's FULL output vector on every
        accelerator of the group (own copy included); the kernels store this shard's rows into all of them."""
        n, npeer = len(keys), len(peer_ys[0])
        kk = (C.c_char_p * n)(*[k.encode() for k in keys])
        xx = (C.c_void_p * n)(*[int(p) for p in d_xs])
        pp = (C.c_void_p * (n * npeer))(*[int(p) for ys in peer_ys for p in ys])
        rc = self._check(self._L.strix_cuda_gemv_batch_peers_dev(self._h, n, kk, xx, npeer, pp, act,
                                                                C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def gemv_peers_dev(self, keys, d_a, peer_ys, d_b=0, eps=0.0, pre=PRE_NONE, act=ACT_F32, stream=0, d_res=None):
        """Row-sharded form: peer_ys[m] = the device pointers of weight m's FULL output vector on every
        accelerator of the group (own copy included); rows land at row0 + r in each of them."""
        n, npeer = len(keys), len(peer_ys[0])
        kk = (C.c_char_p * n)(*[k.encode() for k in keys])
        pp = (C.c_void_p * (n * npeer))(*[int(p) for ys in peer_ys for p in ys])
        rr = (C.c_void_p * n)(*[int(p) if p else None for p in d_res]) if d_res is not None else None
        rc = self._check(self._L.strix_cuda_gemv_peers_dev(self._h, n, kk, C.c_void_p(int(d_a)),
                                                          C.c_void_p(int(d_b)) if d_b else None, float(eps), pre, act,
                                                          rr, npeer, pp, C.c_void_p(int(stream)) if stream else None))
        return rc == 1

    def enable_peer_access(self, peer_device):
        return self._check(self._L.strix_cuda_enable_peer_access(self._h, int(peer_device))) == 1

    def ipc_open(self, handle):
        """Base address (int) of memory another process exported (64-byte CUDA IPC handle), mapped for this device."""
        out = C.c_void_p()
        self._check(self._L.strix_cuda_ipc_open(self._h, bytes(handle), len(handle), C.byref(out)))
        return int(out.value)

    def poke_u32(self, d_ptr, value):
        return self._check(self._L.strix_cuda_poke_u32(self._h, C.c_void_p(int(d_ptr)), int(value))) == 1

    def ipc_export(self, d_ptr):
        """The 64-byte CUDA IPC handle of the device allocation that starts at d_ptr."""
        buf = C.create_string_buffer(64)
        self._check(self._L.strix_cuda_ipc_export(self._h, C.c_void_p(int(d_ptr)), buf, 64))
        return bytes(buf.raw)

    def peek_u32(self, d_ptr):
        out = C.c_uint32()
        self._check(self._L.strix_cuda_peek_u32(self._h, C.c_void_p(int(d_ptr)), C.byref(out)))
        return out.value

    def ipc_close(self, base):
        self._check(self._L.strix_cuda_ipc_close(self._h, C.c_void_p(int(base))))

    def peer_barrier_dev(self, d_epoch, d_local_flags, peer_flags, stream=0):
        pf = (C.c_void_p * len(peer_flags))(*[int(p) for p in peer_flags])
        self._check(self._L.strix_cuda_peer_barrier_dev(self._h, C.c_void_p(int(d_epoch)), C.c_void_p(int(d_local_flags)),
                                                        pf, C.c_void_p(int(stream)) if stream else None))

    def device_status(self, stream=0):
        s = C.c_uint32()
        self._check(self._L.strix_cuda_device_status(self._h, C.c_void_p(int(stream)) if stream else None, C.byref(s)))
        return s.value

    # -- test / measurement extras ---------------------------------------
    def clear_device_status(self, stream=0):
        return self._check(self._L.strix_cuda_clear_device_status(self._h, C.c_void_p(int(stream)) if stream else None)) == 1

    def set_option(self, name, value):
        """Planning / measurement knob by name (see strix_cuda_set_option); False for an unknown name."""
        return self._check(self._L.strix_cuda_set_option(self._h, name.encode(), int(value))) == 1

    def decode_trace(self, max_steps=4096):
        """Per-step words [steps][6] of the last decode-chain launch after set_option("chain_trace", 1), or None
        (see strix_cuda_decode_trace)."""
        buf = np.zeros(6 * max_steps, np.uint64)
        n = self._check(self._L.strix_cuda_decode_trace(self._h, buf.ctypes.data_as(C.POINTER(C.c_uint64)), buf.size))
        return buf[:6 * n].reshape(n, 6).copy() if n > 0 else None

    def dequant_to_f32(self, key):
        info = self.weight_info(key)
        if info is None:
            return None
        out = np.empty((info["rows"], info["in_dim"]), dtype=np.float32)
        self._check(self._L.strix_cuda_dequant_to_f32(self._h, key.encode(), _fp(out), out.size))
        return out

    def xquant8(self, x):
        xa = _f32(x)
        q = np.empty(xa.size, dtype=np.int8)
        d = np.empty(xa.size // 32, dtype=np.float32)
        self._check(self._L.strix_cuda_xquant8(self._h, _fp(xa), xa.size, q.ctypes.data_as(C.POINTER(C.c_int8)),
                                               _fp(d)))
        return q, d
