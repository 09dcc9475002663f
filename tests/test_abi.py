"""The C-ABI library loads without a GPU and exports every symbol the header declares."""
import ctypes
import os
import re

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def declared_symbols():
    names = []
    for fn in sorted(os.listdir(os.path.join(ROOT, "include"))):
        if fn.endswith(".h"):
            txt = open(os.path.join(ROOT, "include", fn)).read()
            names += re.findall(r"STRIX_API[^;(]*?\b(strix_(?:cuda|gguf|ggml|spec)_\w+)\s*\(", txt)
    return names


def test_header_declares_the_trait_surface():
    names = set(declared_symbols())
    for must in ("strix_cuda_create", "strix_cuda_destroy", "strix_cuda_upload_q4_0", "strix_cuda_upload_q6_k",
                 "strix_cuda_upload_q8_0", "strix_cuda_gemv", "strix_cuda_gemv_batch", "strix_cuda_resident_count",
                 "strix_cuda_name", "strix_cuda_upload_f32"):
        assert must in names


def test_library_exports_every_declared_symbol(pkg):
    lib = ctypes.CDLL(pkg.library_path())
    missing = [n for n in declared_symbols() if not hasattr(lib, n)]
    assert not missing, missing


def test_create_fails_loudly_without_a_device(pkg):
    import torch
    if torch.cuda.is_available():
        return  # covered by the gpu tests
    try:
        pkg.CudaWeightAccel(0)
    except pkg.StrixCudaError as e:
        assert str(e)  # a real message, not a silent fallback
    else:
        raise AssertionError("create succeeded without a CUDA device")


def test_rust_ffi_is_generated_from_the_headers():
    """strix-backend-cuda/src/ffi.rs (the Rust side of the boundary, uncompiled here) declares exactly what
    include/*.h declares: it is generated, and this checks that it is current."""
    import subprocess
    import sys
    gen = os.path.join(ROOT, "strix.rs_b200", "rust", "gen_ffi.py")
    assert subprocess.run([sys.executable, gen, "--check"]).returncode == 0, "run strix.rs_b200/rust/gen_ffi.py"
    txt = open(os.path.join(ROOT, "strix.rs_b200", "rust", "strix-backend-cuda", "src", "ffi.rs")).read()
    for name in declared_symbols():
        assert "pub fn %s(" % name in txt, name


def test_every_option_name_is_documented_in_the_header():
    """strix_cuda_set_option answers 0 for a name it does not know; every name it does know must be described in
    include/strix_cuda.h, which is all a binder has to go by."""
    src = open(os.path.join(ROOT, "strix.rs_b200", "csrc", "accel.cu")).read()
    body = src[src.index("int strix_cuda_set_option("):]
    body = body[:body.index("\n}\n")]
    names = re.findall(r'n == "([a-z0-9_]+)"', body)
    assert len(names) >= 10
    hdr = open(os.path.join(ROOT, "include", "strix_cuda.h")).read()
    assert [n for n in names if '"%s"' % n not in hdr] == []
