"""GGUF files on the way to the accelerator.

``GgufFile`` mirrors the reference's ``GgufFile`` (crates/strix-models/src/gguf.rs:104-269) over the
C-ABI of ``include/strix_gguf.h``: open / parse, metadata getters with the reference's widening
rules, the tensor index, borrowed raw tensor bytes, and the hand-over of tensors to a
``CudaWeightAccel``. The parser itself is the C++ code in ``csrc/gguf.cpp``; nothing is parsed here.

``write_gguf`` writes a GGUF v3 file from Python values (synthetic models for tests and benchmarks:
there are no model files in this environment). It follows the published container layout the
reference's own test builds by hand (gguf.rs:385-430).
"""
import ctypes as C
import struct

import numpy as np

from .accel import StrixCudaError, load_library

GGML_F32, GGML_F16, GGML_Q4_0, GGML_Q4_1, GGML_Q8_0, GGML_Q6_K = 0, 1, 2, 3, 8, 14
_MAGIC = 0x46554747


class _Tensor(C.Structure):
    _fields_ = [("name", C.c_char_p), ("n_dims", C.c_uint32), ("dims", C.c_uint64 * 4), ("ggml_type", C.c_uint32),
                ("offset", C.c_uint64), ("data", C.POINTER(C.c_uint8)), ("nbytes", C.c_size_t)]


_declared = False


def _lib():
    global _declared
    L = load_library()
    if not _declared:
        G, sz = C.c_void_p, C.c_size_t

        def sig(name, res, *args):
            f = getattr(L, name)
            f.restype, f.argtypes = res, list(args)

        sig("strix_gguf_open", C.c_int, C.c_char_p, C.POINTER(G))
        sig("strix_gguf_open_memory", C.c_int, C.c_void_p, sz, C.POINTER(G))
        sig("strix_gguf_close", None, G)
        sig("strix_gguf_last_error", C.c_char_p)
        sig("strix_gguf_version", C.c_uint32, G)
        sig("strix_gguf_alignment", sz, G)
        sig("strix_gguf_data_offset", sz, G)
        sig("strix_gguf_tensor_count", sz, G)
        sig("strix_gguf_meta_count", sz, G)
        sig("strix_gguf_tensor_at", C.c_int, G, sz, C.POINTER(_Tensor))
        sig("strix_gguf_find_tensor", C.c_int, G, C.c_char_p, C.POINTER(_Tensor))
        sig("strix_gguf_meta_u64", C.c_int, G, C.c_char_p, C.POINTER(C.c_uint64))
        sig("strix_gguf_meta_f32", C.c_int, G, C.c_char_p, C.POINTER(C.c_float))
        sig("strix_gguf_meta_str", C.c_int, G, C.c_char_p, C.POINTER(C.c_char_p), C.POINTER(sz))
        sig("strix_gguf_meta_array_len", C.c_int, G, C.c_char_p, C.POINTER(C.c_uint64), C.POINTER(C.c_uint32))
        sig("strix_gguf_meta_key_at", C.c_int, G, sz, C.POINTER(C.c_char_p), C.POINTER(C.c_uint32))
        sig("strix_gguf_advise_dontneed", None, G, C.c_char_p)
        sig("strix_ggml_block_elems", sz, C.c_uint32)
        sig("strix_ggml_block_bytes", sz, C.c_uint32)
        sig("strix_cuda_upload_gguf_tensor", C.c_int, C.c_void_p, G, C.c_char_p, C.c_int)
        sig("strix_cuda_upload_gguf", C.c_int, C.c_void_p, G, C.c_int, C.POINTER(sz), C.POINTER(sz))
        _declared = True
    return L


class GgufError(StrixCudaError):
    pass


def block_elems(ggml_type):
    return int(_lib().strix_ggml_block_elems(ggml_type))


def block_bytes(ggml_type):
    return int(_lib().strix_ggml_block_bytes(ggml_type))


class GgufFile:
    """A parsed GGUF file: memory-mapped from ``path`` or parsed from ``data`` (bytes, kept alive here)."""

    def __init__(self, path=None, data=None):
        self._L = _lib()
        self._g = C.c_void_p()
        self._keep = None
        if (path is None) == (data is None):
            raise ValueError("give a path or the file's bytes")
        if path is not None:
            rc = self._L.strix_gguf_open(str(path).encode(), C.byref(self._g))
        else:
            self._keep = (C.c_uint8 * max(len(data), 1)).from_buffer_copy(bytes(data) or b"\0")
            rc = self._L.strix_gguf_open_memory(C.addressof(self._keep), len(data), C.byref(self._g))
        if rc != 1:
            self._g = None
            raise GgufError(self._L.strix_gguf_last_error().decode())

    def close(self):
        if getattr(self, "_g", None):
            self._L.strix_gguf_close(self._g)
            self._g = None

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()

    # -- header ---------------------------------------------------------------
    @property
    def version(self):
        return int(self._L.strix_gguf_version(self._g))

    @property
    def alignment(self):
        return int(self._L.strix_gguf_alignment(self._g))

    @property
    def data_offset(self):
        return int(self._L.strix_gguf_data_offset(self._g))

    # -- metadata (MetaValue::as_u64 / as_f32 / as_str, gguf.rs:43-80) -------------
    def meta_keys(self):
        out = []
        for i in range(self._L.strix_gguf_meta_count(self._g)):
            k, ty = C.c_char_p(), C.c_uint32()
            self._L.strix_gguf_meta_key_at(self._g, i, C.byref(k), C.byref(ty))
            out.append((k.value.decode(), int(ty.value)))
        return out

    def meta_u64(self, key):
        v = C.c_uint64()
        return int(v.value) if self._L.strix_gguf_meta_u64(self._g, key.encode(), C.byref(v)) == 1 else None

    def meta_f32(self, key):
        v = C.c_float()
        return float(v.value) if self._L.strix_gguf_meta_f32(self._g, key.encode(), C.byref(v)) == 1 else None

    def meta_str(self, key):
        p, n = C.c_char_p(), C.c_size_t()
        if self._L.strix_gguf_meta_str(self._g, key.encode(), C.byref(p), C.byref(n)) != 1:
            return None
        return C.string_at(p, n.value).decode("utf-8", "replace")

    def meta_array_len(self, key):
        n, ty = C.c_uint64(), C.c_uint32()
        if self._L.strix_gguf_meta_array_len(self._g, key.encode(), C.byref(n), C.byref(ty)) != 1:
            return None
        return int(n.value), int(ty.value)

    def architecture(self):
        return self.meta_str("general.architecture")

    # -- tensors ----------------------------------------------------------------
    @staticmethod
    def _info(t):
        return {"name": t.name.decode(), "dims": [int(t.dims[d]) for d in range(t.n_dims)], "ggml_type": int(t.ggml_type),
                "offset": int(t.offset), "nbytes": int(t.nbytes)}

    def tensors(self):
        out = []
        for i in range(self._L.strix_gguf_tensor_count(self._g)):
            t = _Tensor()
            if self._L.strix_gguf_tensor_at(self._g, i, C.byref(t)) != 1:
                raise GgufError(self._L.strix_gguf_last_error().decode())
            out.append(self._info(t))
        return out

    def tensor_info(self, name):
        t = _Tensor()
        rc = self._L.strix_gguf_find_tensor(self._g, name.encode(), C.byref(t))
        if rc < 0:
            raise GgufError(self._L.strix_gguf_last_error().decode())
        return self._info(t) if rc == 1 else None

    def tensor_bytes(self, name):
        """Raw block bytes of a tensor as a numpy view into the map (valid until close)."""
        t = _Tensor()
        rc = self._L.strix_gguf_find_tensor(self._g, name.encode(), C.byref(t))
        if rc < 0:
            raise GgufError(self._L.strix_gguf_last_error().decode())
        if rc == 0:
            raise GgufError("GGUF tensor `%s` not found" % name)
        if t.nbytes == 0:
            return np.zeros(0, dtype=np.uint8)
        return np.ctypeslib.as_array(t.data, shape=(t.nbytes,))

    def advise_dontneed(self, name):
        self._L.strix_gguf_advise_dontneed(self._g, name.encode())

    # -- hand-over to the accelerator ------------------------------------------------
    def upload_tensor(self, accel, name, drop_pages=False):
        """True = adopted, False = declined (no kernel for the type / rank)."""
        accel._rows = {}  # (the mirror's per-key row counts: a key may be replaced)
        rc = self._L.strix_cuda_upload_gguf_tensor(accel._h, self._g, name.encode(), int(drop_pages))
        if rc < 0:
            msg = accel._L.strix_cuda_last_error(accel._h).decode() or self._L.strix_gguf_last_error().decode()
            raise GgufError(msg)
        return rc == 1

    def upload_all(self, accel, drop_pages=False):
        """Returns (adopted, declined) tensor counts."""
        a, d = C.c_size_t(), C.c_size_t()
        accel._rows = {}
        rc = self._L.strix_cuda_upload_gguf(accel._h, self._g, int(drop_pages), C.byref(a), C.byref(d))
        if rc < 0:
            msg = accel._L.strix_cuda_last_error(accel._h).decode() or self._L.strix_gguf_last_error().decode()
            raise GgufError(msg)
        return int(a.value), int(d.value)


# ---------------------------------------------------------------------------- writer
_SCALAR_FMT = {0: "<B", 1: "<b", 2: "<H", 3: "<h", 4: "<I", 5: "<i", 6: "<f", 7: "<B", 10: "<Q", 11: "<q", 12: "<d"}


class Typed:
    """A metadata value with an explicit GGUF value type (0..12), e.g. ``Typed(4, 7)`` = u32 7;
    arrays: ``Typed(9, [..], elem_type=8)``."""

    def __init__(self, ty, value, elem_type=None):
        self.ty, self.value, self.elem_type = ty, value, elem_type


def _wstr(s):
    b = s.encode() if isinstance(s, str) else bytes(s)
    return struct.pack("<Q", len(b)) + b


def _wvalue(ty, v, elem_type=None):
    if ty in _SCALAR_FMT:
        return struct.pack(_SCALAR_FMT[ty], v)
    if ty == 8:
        return _wstr(v)
    if ty == 9:
        out = struct.pack("<IQ", elem_type, len(v))
        for e in v:
            out += _wvalue(e.ty, e.value, e.elem_type) if isinstance(e, Typed) else _wvalue(elem_type, e)
        return out
    raise ValueError("GGUF value type %r" % ty)


def _auto(v):
    if isinstance(v, Typed):
        return v
    if isinstance(v, bool):
        return Typed(7, int(v))
    if isinstance(v, int):
        return Typed(4, v) if 0 <= v < 2 ** 32 else Typed(11, v)
    if isinstance(v, float):
        return Typed(6, v)
    if isinstance(v, str):
        return Typed(8, v)
    if isinstance(v, (list, tuple)):
        et = _auto(v[0]).ty if len(v) else 4
        return Typed(9, list(v), elem_type=et)
    raise ValueError("no GGUF value type for %r" % (v,))


def gguf_bytes(meta, tensors, version=3, alignment=None):
    """meta: dict key -> value (or Typed). tensors: list of (name, dims (GGUF order: in_dim first),
    ggml_type, raw bytes). Returns the file's bytes. ``alignment`` also writes general.alignment."""
    meta = dict(meta)
    if alignment is not None:
        meta["general.alignment"] = Typed(4, alignment)
    align = alignment if alignment is not None else 32
    head = struct.pack("<IIQQ", _MAGIC, version, len(tensors), len(meta))
    for k, v in meta.items():
        t = _auto(v)
        head += _wstr(k) + struct.pack("<I", t.ty) + _wvalue(t.ty, t.value, t.elem_type)
    off, offs = 0, []
    for _, _, _, raw in tensors:
        offs.append(off)
        off += len(raw)
        if align:
            off = -(-off // align) * align
    for (name, dims, ty, _), o in zip(tensors, offs):
        head += _wstr(name) + struct.pack("<I", len(dims)) + b"".join(struct.pack("<Q", d) for d in dims)
        head += struct.pack("<IQ", ty, o)
    if align:
        head += b"\0" * (-len(head) % align)
    body = bytearray(off)
    for (_, _, _, raw), o in zip(tensors, offs):
        body[o:o + len(raw)] = bytes(raw)
    return bytes(head) + bytes(body)


def write_gguf(path, meta, tensors, version=3, alignment=None):
    with open(path, "wb") as f:
        f.write(gguf_bytes(meta, tensors, version=version, alignment=alignment))
