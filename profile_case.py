"""Small driver for profiling one kernel on one shape (what the ncu summaries under profiles/ ran).

    python profile_case.py gemv <ggml type 2|8|14> <rows> <in_dim> <act 0|1> [launches]
    python profile_case.py gemm <tokens> <in_dim> <rows> [launches]
    python profile_case.py attn <context> [steps]
    python profile_case.py chain <layers> [tokens]
    python profile_case.py multi <act 0|1> [launches]

`multi`: the four small weights of the benchmark step (Q8_0 and Q6_K, 2560 -> 9728 and 9728 -> 2560) as one
gemv_batch_dev call, i.e. side by side in one launch (``-k regex:gemv_multi_kernel``).

`chain`: the decode configuration's layer shapes (hidden 2560, q 4096, k/v 1024, ffn 9728, Q4_0; Q6_K head over
151936 rows) with <layers> layers, integer-dot form, run as the persistent chain kernel (``-k regex:chain_kernel``).

`attn`: a two-layer model with the benchmark's attention geometry (32 query heads, 8 KV heads of 128,
hidden 2560) and a KV cache seeded up to <context>; runs decode_step at that position (``-k regex:sdpa_split``).

Uploads one seeded synthetic weight through the C ABI and launches the device-resident entry
point a few times on cuda:0. Run it plain first, then under ncu with ``-k regex:gemv_kernel``
(or ``gemm_w8a8``), ``-s 1 -c 1`` and ``--clock-control none``.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
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
    elif kind == "multi":
        act = int(sys.argv[2])
        reps = int(sys.argv[3]) if len(sys.argv) > 3 else 3
        keys, xs, ys = [], [], []
        for ty, k, n in ((8, 2560, 9728), (8, 9728, 2560), (14, 2560, 9728), (14, 9728, 2560)):
            key = "w.%d.%d.%d" % (ty, k, n)
            assert {8: acc.upload_q8_0, 14: acc.upload_q6_k}[ty](key, synth.quant(ty, 1, key, n, k), k, n)
            keys.append(key)
            xs.append(torch.randn(k, device=dev))
            ys.append(torch.empty(n, device=dev))
        flush = torch.empty(256 << 20, dtype=torch.uint8, device=dev)
        for _ in range(reps):
            flush.zero_()   # (the 94 MB of weights would otherwise sit in L2 from the launch before)
            assert acc.gemv_batch_dev(keys, [x.data_ptr() for x in xs], [y_.data_ptr() for y_ in ys], act=act, stream=s)
        y = ys[0]
    elif kind == "chain":
        n_layers = int(sys.argv[2])
        reps = int(sys.argv[3]) if len(sys.argv) > 3 else 3
        hidden, qdim, kvdim, ffn, vocab = 2560, 4096, 1024, 9728, 151936
        shapes = {"attn_q": (qdim, hidden), "attn_k": (kvdim, hidden), "attn_v": (kvdim, hidden), "attn_output": (hidden, qdim),
                  "ffn_gate": (ffn, hidden), "ffn_up": (ffn, hidden), "ffn_down": (hidden, ffn)}
        base = {nm: synth.q4_0(1, nm, n_, k_) for nm, (n_, k_) in shapes.items()}
        for il in range(n_layers):
            for nm, (n_, k_) in shapes.items():
                assert acc.upload_q4_0("blk.%d.%s.weight" % (il, nm), base[nm], k_, n_)
            for nn in ("attn_norm", "ffn_norm"):
                acc.upload_f32("blk.%d.%s.weight" % (il, nn), synth.norm_weight(1, nn, hidden))
        gen = 8192
        hb = synth.q6_k(1, "head", gen, hidden).reshape(gen, -1)
        assert acc.upload_q6_k("output.weight", np.ascontiguousarray(hb[np.arange(vocab) % gen]).reshape(-1), hidden, vocab)
        acc.upload_f32("output_norm.weight", synth.norm_weight(1, "on", hidden))
        acc.set_option("decode_chain", 1)
        assert acc.configure_decode(hidden, 32, ffn, vocab, n_layers, eps=1e-6, act=pkg.ACT_Q8DOT)
        h0 = synth.normal(1, "h0", hidden)
        for i in range(reps):
            y = torch.from_numpy(acc.decode_step(h0, i))
    elif kind == "attn":
        ctx = int(sys.argv[2])
        reps = int(sys.argv[3]) if len(sys.argv) > 3 else 3
        hidden, hd, n_heads, n_kv, ffn, vocab, n_layers = 2560, 128, 32, 8, 1024, 2048, 2
        shapes = {"attn_q": (n_heads * hd, hidden), "attn_k": (n_kv * hd, hidden), "attn_v": (n_kv * hd, hidden),
                  "attn_output": (hidden, n_heads * hd), "ffn_gate": (ffn, hidden), "ffn_up": (ffn, hidden),
                  "ffn_down": (hidden, ffn)}
        for il in range(n_layers):
            for nm, (n, k) in shapes.items():
                assert acc.upload_q4_0("blk.%d.%s.weight" % (il, nm), synth.q4_0(1, nm, n, k), k, n)
            for nn in ("attn_norm", "ffn_norm"):
                acc.upload_f32("blk.%d.%s.weight" % (il, nn), synth.norm_weight(1, nn, hidden))
            for nn in ("attn_q_norm", "attn_k_norm"):
                acc.upload_f32("blk.%d.%s.weight" % (il, nn), synth.norm_weight(1, nn, hd))
        assert acc.upload_q6_k("output.weight", synth.q6_k(1, "head", vocab, hidden), hidden, vocab)
        acc.upload_f32("output_norm.weight", synth.norm_weight(1, "on", hidden))
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, eps=1e-6, act=pkg.ACT_Q8DOT,
                                    attn_standin_q=False, head_dim=hd, n_kv=n_kv, rope_theta=1e6, max_seq=ctx + 1)
        rows = synth.normal(1, "kv", (ctx + 1) * n_kv * hd).reshape(ctx + 1, n_kv * hd)
        for il in range(n_layers):
            assert acc.seed_decode_kv(il, rows, rows)
        h0 = synth.normal(1, "h0", hidden)
        for _ in range(reps):
            y = torch.from_numpy(acc.decode_step(h0, ctx))
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
