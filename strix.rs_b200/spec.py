"""Speculative-decoding callers of the batched verify path over the C ABI (include/strix_spec.h): the n-gram
lookup proposer, greedy acceptance, the lookup loop's utility gate and the draft-model round
(crates/strix-cli/src/commands/generate.rs:597-668, 848-899). Nothing is computed here."""
import ctypes as C

import numpy as np

from .accel import StrixCudaError, load_library

EMBED_FN = C.CFUNCTYPE(None, C.c_void_p, C.c_uint32, C.POINTER(C.c_float))


class Gate(C.Structure):
    """strix_spec_gate."""
    _fields_ = [("zero_rounds", C.c_uint32), ("plain_left", C.c_uint32)]


_ready = False


def _lib():
    global _ready
    L = load_library()
    if not _ready:
        u32p, sz = C.POINTER(C.c_uint32), C.c_size_t
        L.strix_spec_propose_ngram.restype, L.strix_spec_propose_ngram.argtypes = sz, [u32p, sz, sz, u32p]
        L.strix_spec_accept.restype, L.strix_spec_accept.argtypes = sz, [u32p, sz, u32p, sz, u32p]
        L.strix_spec_gate_plain.restype, L.strix_spec_gate_plain.argtypes = C.c_int, [C.POINTER(Gate)]
        L.strix_spec_gate_round.restype, L.strix_spec_gate_round.argtypes = None, [C.POINTER(Gate), sz]
        L.strix_cuda_spec_round.restype = C.c_int
        L.strix_cuda_spec_round.argtypes = [C.c_void_p, C.c_void_p, EMBED_FN, C.c_void_p, EMBED_FN, C.c_void_p, sz, sz,
                                            C.c_uint32, sz, sz, u32p, u32p]
        L.strix_cuda_verify_argmax.restype = C.c_int
        L.strix_cuda_verify_argmax.argtypes = [C.c_void_p, C.POINTER(C.c_float), sz, sz, u32p]
        _ready = True
    return L


def _u32(a):
    return np.ascontiguousarray(np.asarray(a, dtype=np.uint32))


def propose_ngram(ctx, gamma):
    """Proposed continuation (list of token ids, possibly empty) of the context from its own history."""
    c = _u32(ctx)
    out = np.zeros(max(gamma, 1), dtype=np.uint32)
    n = _lib().strix_spec_propose_ngram(c.ctypes.data_as(C.POINTER(C.c_uint32)), c.size, gamma,
                                        out.ctypes.data_as(C.POINTER(C.c_uint32)))
    return [int(t) for t in out[:n]]


def accept(proposal, argmax, room):
    """(accepted count, next token): argmax has len(proposal) + 1 entries."""
    p, a = _u32(proposal), _u32(argmax)
    assert a.size == p.size + 1
    nxt = C.c_uint32()
    n = _lib().strix_spec_accept(p.ctypes.data_as(C.POINTER(C.c_uint32)), p.size, a.ctypes.data_as(C.POINTER(C.c_uint32)),
                                 room, C.byref(nxt))
    return int(n), int(nxt.value)


def gate_plain(g):
    return _lib().strix_spec_gate_plain(C.byref(g)) == 1


def gate_round(g, accepted):
    _lib().strix_spec_gate_round(C.byref(g), accepted)


def verify_argmax(accel, hs, start_pos, m):
    """Greedy tokens of m verified rows (argmax on the device), or None."""
    L = _lib()
    ha = np.ascontiguousarray(np.asarray(hs, dtype=np.float32).reshape(-1))
    ids = np.zeros(m, dtype=np.uint32)
    rc = L.strix_cuda_verify_argmax(accel._h, ha.ctypes.data_as(C.POINTER(C.c_float)), start_pos, m,
                                    ids.ctypes.data_as(C.POINTER(C.c_uint32)))
    if rc < 0:
        raise StrixCudaError(accel._L.strix_cuda_last_error(accel._h).decode())
    return ids if rc == 1 else None


def spec_round(target, draft, embed_target, embed_draft, cur, pos, gamma):
    """One draft-model round: embed_*: arrays [vocab][hidden] of the two models. Returns (tokens to emit, next token)."""
    L = _lib()
    et = np.ascontiguousarray(embed_target, dtype=np.float32)
    ed = np.ascontiguousarray(embed_draft, dtype=np.float32)

    def mk(table):
        hidden = table.shape[1]

        def fn(_user, token, out):
            C.memmove(out, table[int(token)].ctypes.data, hidden * 4)
        return EMBED_FN(fn)
    ft, fd = mk(et), mk(ed)
    out = np.zeros(gamma + 1, dtype=np.uint32)
    nxt = C.c_uint32()
    rc = L.strix_cuda_spec_round(target._h, draft._h, ft, None, fd, None, et.shape[1], ed.shape[1], int(cur), pos, gamma,
                                 out.ctypes.data_as(C.POINTER(C.c_uint32)), C.byref(nxt))
    if rc < 0:
        for a in (target, draft):
            msg = a._L.strix_cuda_last_error(a._h).decode()
            if msg:
                raise StrixCudaError(msg)
        raise StrixCudaError("spec_round failed")
    if rc == 0:
        return None
    return [int(t) for t in out[:rc]], int(nxt.value)
