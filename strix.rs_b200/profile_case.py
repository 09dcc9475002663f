"""Small driver for profiling one kernel on one shape (what the ncu summaries under profiles/ ran).

    python strix.rs_b200/profile_case.py gemv <ggml type 2|8|14> <rows> <in_dim> <act 0|1> [launches]
    python strix.rs_b200/profile_case.py gemm <tokens> <in_dim> <rows> [launches]

Uploads one seeded synthetic weight through the C ABI and launches the device-resident entry
point a few times on cuda:0. Run it plain first, then under ncu with ``-k regex:gemv_kernel``
(or ``gemm_w8a8``), ``-s 1 -c 1`` and ``--clock-control none``.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402


def main():
    import torch
    pkg = entry.load_package()
    from strix_rs_b200 import synth
    kind = sys.argv[1]
    acc = pkg.CudaWeightAccel(0)
    dev = torch.device("cuda:0")
    s = torch.cuda.current_stream().cuda_stream
    if kind == "gemv":
        ty, n, k, act = (int(a) for a in sys.argv[2:6])
        reps = int(sys.argv[6]) if len(sys.argv) > 6 else 3
        gen = min(n, 8192)
        base = synth.quant(ty, 1, "w", gen, k).reshape(gen, -1)
        w = np.ascontiguousarray(base[np.arange(n) % gen]).reshape(-1)
        assert {2: acc.upload_q4_0, 8: acc.upload_q8_0, 14: acc.upload_q6_k}[ty]("w", w, k, n)
        x = torch.randn(k, device=dev)
        y = torch.empty(n, device=dev)
        for _ in range(reps):
            acc.gemv_dev(["w"], x.data_ptr(), [y.data_ptr()], act=act, stream=s)
    else:
        m, k, n = (int(a) for a in sys.argv[2:5])
        reps = int(sys.argv[5]) if len(sys.argv) > 5 else 3
        assert acc.upload_q8_0("w", synth.q8_0(1, "w", n, k), k, n)
        x = torch.randn(m, k, device=dev)
        y = torch.empty(m, n, device=dev)
        for _ in range(reps):
            acc.prefill_q8_gemm_dev("w", x.data_ptr(), m, y.data_ptr(), stream=s)
    torch.cuda.synchronize()
    print("status", acc.device_status(s), "checksum", float(y.abs().sum()))
    acc.close()


if __name__ == "__main__":
    main()
