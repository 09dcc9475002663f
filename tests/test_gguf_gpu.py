"""A synthetic GGUF model file flows through the reader into the accelerator: every tensor the
accelerator has a kernel for is adopted under its GGUF name, the rest is declined, and the decode
chain built from the file matches the oracle chain on the same bytes."""
import numpy as np
import pytest

from test_decode_gpu import oracle_chain, rel_l2

pytestmark = pytest.mark.gpu


def test_model_file_to_decode_step(pkg, orc, synth, tmp_path):
    from strix_rs_b200 import gguf
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 768, 256, 1536, 3000, 2, 1e-6
    W, ts = {}, []

    def add(name, ty, n, k):
        w = synth.quant(ty, 70, name, n, k)
        W[name] = (w, ty, k, n)
        ts.append((name, [k, n], ty, w.tobytes()))          # GGUF order: in_dim first (qwen3.rs:772-774)

    for il in range(n_layers):
        b = "blk.%d." % il
        for nm, n, k in (("attn_q", qdim, hidden), ("attn_k", kvdim, hidden), ("attn_v", kvdim, hidden),
                         ("attn_output", hidden, qdim), ("ffn_gate", ffn, hidden), ("ffn_up", ffn, hidden)):
            add(b + nm + ".weight", synth.Q4_0, n, k)
        add(b + "ffn_down.weight", synth.Q4_1 if il == 0 else synth.Q8_0, hidden, ffn)  # mixed formats in one file
        for nn in ("attn_norm.weight", "ffn_norm.weight"):
            W[b + nn] = synth.norm_weight(70, b + nn, hidden)
            ts.append((b + nn, [hidden], gguf.GGML_F32, W[b + nn].tobytes()))
    add("output.weight", synth.Q6_K, vocab, hidden)
    W["output_norm.weight"] = synth.norm_weight(70, "output_norm", hidden)
    ts.append(("output_norm.weight", [hidden], gguf.GGML_F32, W["output_norm.weight"].tobytes()))
    # tensors the accelerator has no kernel for: F16 matrix, Q4_K matrix, 2-D F32
    ts.append(("token_embd.weight", [hidden, 8], gguf.GGML_F16, np.zeros(hidden * 8, np.float16).tobytes()))
    ts.append(("blk.0.q4k.weight", [256, 4], 12, bytes(4 * 144)))
    ts.append(("rope_freqs", [4, 4], gguf.GGML_F32, bytes(64)))
    path = tmp_path / "model.gguf"
    gguf.write_gguf(path, {"general.architecture": "qwen3", "qwen3.block_count": n_layers,
                           "qwen3.embedding_length": hidden, "qwen3.feed_forward_length": ffn,
                           "qwen3.attention.layer_norm_rms_epsilon": eps}, ts)

    acc = pkg.CudaWeightAccel(0)
    try:
        with gguf.GgufFile(path=path) as g:
            assert g.meta_u64("qwen3.block_count") == n_layers
            adopted, declined = g.upload_all(acc, drop_pages=True)
            assert declined == 3 and adopted == len(ts) - 3
            assert g.upload_tensor(acc, "token_embd.weight") is False
            with pytest.raises(gguf.GgufError):
                g.upload_tensor(acc, "no.such.tensor")
            eps_f = g.meta_f32("qwen3.attention.layer_norm_rms_epsilon")
        # the file is closed: the accelerator copied what it adopted (bytes are borrowed for the call only)
        assert acc.resident_count() == 7 * n_layers + 1
        info = acc.weight_info("blk.1.ffn_down.weight")
        assert info["in_dim"] == ffn and info["rows"] == hidden
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, eps=eps_f, act=pkg.ACT_F32)
        h0 = synth.normal(71, "h0", hidden)
        got = acc.decode_step(h0, 0)
        want = oracle_chain(orc, W, h0, n_layers, eps, False)
        assert rel_l2(got, want) <= 1e-3
        assert acc.decode_step_argmax(h0, 0) == orc.argmax_f32(got)
        # bit-exact weight tier through the file: dequantised resident bytes == oracle dequant of the file's bytes
        w, ty, k, n = W["output.weight"]
        np.testing.assert_array_equal(acc.dequant_to_f32("output.weight").reshape(-1).view(np.uint32),
                                      orc.dequantize(ty, w, n * k).reshape(-1).view(np.uint32))
    finally:
        acc.close()
