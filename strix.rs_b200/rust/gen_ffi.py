"""Writes strix-backend-cuda/src/ffi.rs from the C headers under include/: one `extern "C"` declaration per
STRIX_API function, so that the Rust binding cannot drift from the ABI (tests/test_abi.py runs this in check mode).

    python strix.rs_b200/rust/gen_ffi.py            # rewrite ffi.rs
    python strix.rs_b200/rust/gen_ffi.py --check    # exit 1 if ffi.rs is out of date

The crate is not compiled in this repository's build image (no Rust toolchain); the C ABI it binds is."""
import os
import re
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
ROOT = os.path.dirname(os.path.dirname(HERE))
OUT = os.path.join(HERE, "strix-backend-cuda", "src", "ffi.rs")

BASE = {"void": "c_void", "char": "c_char", "int": "c_int", "float": "f32", "size_t": "usize", "uint8_t": "u8",
        "int8_t": "i8", "uint32_t": "u32", "int32_t": "i32", "uint64_t": "u64", "long long": "c_longlong",
        "unsigned long long": "u64", "strix_cuda": "StrixCuda", "strix_cuda_opts": "StrixCudaOpts",
        "strix_gpu_decode_config": "StrixGpuDecodeConfig", "strix_gguf": "StrixGguf",
        "strix_gguf_tensor": "StrixGgufTensor", "strix_spec_gate": "StrixSpecGate", "strix_embed_fn": "StrixEmbedFn"}


def rust_type(c):
    """'const float *const *' -> '*const *const f32' (the name, if any, is already removed)."""
    c = c.strip()
    parts = [p.strip() for p in c.split("*")]
    base = parts[0]
    base_const = bool(re.search(r"\bconst\b", base))
    base = re.sub(r"\bconst\b", "", base).strip()
    base = re.sub(r"\s+", " ", base)
    if base not in BASE:
        raise SystemExit("gen_ffi: unknown C type `%s` in `%s`" % (base, c))
    t = BASE[base]
    consts = [base_const] + ["const" in p for p in parts[1:]]
    # pointer level i points at something whose constness is consts[i]
    for i in range(len(parts) - 1):
        t = ("*const " if consts[i] else "*mut ") + t
    return t


def declarations():
    out = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if not fn.endswith(".h"):
            continue
        txt = open(os.path.join(ROOT, "include", fn)).read()
        txt = re.sub(r"/\*.*?\*/", "", txt, flags=re.S)
        for m in re.finditer(r"STRIX_API\s+([^;{]*?)\b(strix_\w+)\s*\(([^;]*?)\)\s*;", txt, flags=re.S):
            ret, name, params = m.group(1).strip(), m.group(2), " ".join(m.group(3).split())
            args = []
            if params not in ("", "void"):
                for p in params.split(","):
                    p = p.strip()
                    mm = re.match(r"^(.*?)(\w+)$", p)
                    ctype, pname = mm.group(1), mm.group(2)
                    if pname in ("type", "fn", "in", "box", "loop", "match", "move", "ref", "self", "use"):
                        pname += "_"
                    args.append("%s: %s" % (pname, rust_type(ctype)))
            r = "" if ret == "void" else " -> " + rust_type(ret)
            out.append((fn, "    pub fn %s(%s)%s;" % (name, ", ".join(args), r)))
    return out


HEAD = '''//! Raw bindings to libstrix_cuda.so. GENERATED from include/*.h by strix.rs_b200/rust/gen_ffi.py: do not edit.
//! Not compiled in the repository's build image (no Rust toolchain there); the C ABI itself is compiled and
//! tested, and tests/test_abi.py checks that this file declares every exported entry point.
#![allow(non_camel_case_types, clippy::too_many_arguments)]
use std::os::raw::{c_char, c_int, c_longlong, c_void};

#[repr(C)]
pub struct StrixCuda { _private: [u8; 0] }
#[repr(C)]
pub struct StrixGguf { _private: [u8; 0] }

/// strix_cuda_opts
#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct StrixCudaOpts { pub rank: c_int, pub world: c_int, pub profile: c_int, pub reserved: [c_int; 5] }

/// strix_gpu_layer_cfg: plain-data mirror of strix_core::accel::GpuLayerCfg (accel.rs:19-40)
#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct StrixGpuLayerCfg {
    pub head_dim: u32, pub n_kv: u32, pub k_eq_v: c_int, pub rope_theta: f32, pub is_local: c_int,
    pub output_scale: f32, pub no_rope: c_int, pub rope_norm: c_int,
}

/// strix_gpu_decode_config: plain-data mirror of GpuDecodeConfig (accel.rs:42-72) plus the two fields the
/// reference does not have (attn_standin_q, act)
#[repr(C)]
#[derive(Clone, Copy)]
pub struct StrixGpuDecodeConfig {
    pub hidden: u32, pub n_heads: u32, pub ffn: u32, pub vocab: u32, pub n_layers: u32,
    pub eps: f32, pub final_softcap: f32,
    pub attn_rsqrt: c_int, pub norm_v: c_int, pub qk_norm: c_int, pub post_norm: c_int, pub act_gelu: c_int,
    pub gpu_prefill: c_int,
    pub n_swa: u32, pub max_seq: u32,
    pub layers: *const StrixGpuLayerCfg,
    pub attn_standin_q: c_int, pub act: c_int,
}

/// strix_gguf_tensor
#[repr(C)]
pub struct StrixGgufTensor {
    pub name: *const c_char, pub n_dims: u32, pub dims: [u64; 4], pub ggml_type: u32, pub offset: u64,
    pub data: *const u8, pub nbytes: usize,
}

/// strix_spec_gate
#[repr(C)]
#[derive(Default, Clone, Copy)]
pub struct StrixSpecGate { pub zero_rounds: u32, pub plain_left: u32 }

pub type StrixEmbedFn = Option<unsafe extern "C" fn(user: *mut c_void, token: u32, hidden_out: *mut f32)>;

pub const ACT_F32: c_int = 0;
pub const ACT_Q8DOT: c_int = 1;
pub const PRE_NONE: c_int = 0;
pub const PRE_RMSNORM: c_int = 1;
pub const PRE_SWIGLU: c_int = 2;
pub const PRE_GEGLU: c_int = 3;

#[link(name = "strix_cuda")]
extern "C" {
'''


def render():
    lines, last = [HEAD], None
    for fn, decl in declarations():
        if fn != last:
            lines.append("    // ---- include/%s\n" % fn)
            last = fn
        lines.append(decl + "\n")
    lines.append("}\n")
    return "".join(lines)


if __name__ == "__main__":
    txt = render()
    if "--check" in sys.argv:
        cur = open(OUT).read() if os.path.exists(OUT) else ""
        sys.exit(0 if cur == txt else 1)
    open(OUT, "w").write(txt)
    print("wrote", OUT, "(%d functions)" % len(declarations()))
