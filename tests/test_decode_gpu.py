"""GPU parity of the resident decode step (projection chain) against the CPU oracle chain."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def build_model(accel, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed=80, gate_ty=None):
    """Uploads a random-init Q4_0 model with a Q6_K head under the reference's tensor names."""
    W = {}

    def up(name, ty, n, k):
        w = synth.quant(ty, seed, name, n, k)
        ok = {synth.Q4_0: accel.upload_q4_0, synth.Q6_K: accel.upload_q6_k, synth.Q8_0: accel.upload_q8_0}[ty](name, w, k, n)
        assert ok, name
        W[name] = (w, ty, k, n)

    for il in range(n_layers):
        b = "blk.%d." % il
        up(b + "attn_q.weight", synth.Q4_0, qdim, hidden)
        up(b + "attn_k.weight", synth.Q4_0, kvdim, hidden)
        up(b + "attn_v.weight", synth.Q4_0, kvdim, hidden)
        up(b + "attn_output.weight", synth.Q4_0, hidden, qdim)
        up(b + "ffn_gate.weight", synth.Q4_0, ffn, hidden)
        up(b + "ffn_up.weight", synth.Q4_0, ffn, hidden)
        up(b + "ffn_down.weight", synth.Q4_0, hidden, ffn)
        for nn in ("attn_norm.weight", "ffn_norm.weight"):
            W[b + nn] = synth.norm_weight(seed, b + nn, hidden)
            accel.upload_f32(b + nn, W[b + nn])
    up("output.weight", synth.Q6_K, vocab, hidden)
    W["output_norm.weight"] = synth.norm_weight(seed, "output_norm", hidden)
    accel.upload_f32("output_norm.weight", W["output_norm.weight"])
    return W


def oracle_chain(orc, W, h0, n_layers, eps, int8, gelu=False):
    """qwen3.rs:818-899 without attention: Wo is fed with q (the stand-in this path defines)."""
    def mm(name, x):
        w, ty, k, n = W[name]
        if int8:
            xq, xd, _ = orc.xquant8(x)
            return orc.idot_gemm(w, ty, xq, xd, 1, k, n)[0]
        return orc.qmatmul(x, w, ty, k, n)

    h = h0.astype(np.float32).copy()
    for il in range(n_layers):
        b = "blk.%d." % il
        n_ = orc.rmsnorm(h, W[b + "attn_norm.weight"], eps)
        q = mm(b + "attn_q.weight", n_)
        mm(b + "attn_k.weight", n_)
        mm(b + "attn_v.weight", n_)
        h = (h + mm(b + "attn_output.weight", q)).astype(np.float32)
        n_ = orc.rmsnorm(h, W[b + "ffn_norm.weight"], eps)
        g, u = mm(b + "ffn_gate.weight", n_), mm(b + "ffn_up.weight", n_)
        a = orc.geglu(g, u) if gelu else orc.swiglu(g, u)
        h = (h + mm(b + "ffn_down.weight", a)).astype(np.float32)
    return mm("output.weight", orc.rmsnorm(h, W["output_norm.weight"], eps))


@pytest.mark.parametrize("chain_kernel", ["0", "1"])
@pytest.mark.parametrize("int8", [False, True])
def test_decode_step_matches_oracle_chain(pkg, orc, synth, int8, chain_kernel, monkeypatch):
    """chain_kernel = "1": the whole chain as one cooperative kernel; "0": one launch per step."""
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 768, 256, 1536, 3000, 3, 1e-6
    monkeypatch.setenv("STRIX_DECODE_CHAIN", chain_kernel)
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers)
        act = pkg.ACT_Q8DOT if int8 else pkg.ACT_F32
        assert acc.decode_step(np.zeros(hidden, np.float32)) is None            # not configured yet -> None
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, eps=eps, act=act)
        h0 = synth.normal(81, "h0", hidden)
        want = oracle_chain(orc, W, h0, n_layers, eps, int8)
        got = acc.decode_step(h0, 0)
        r = rel_l2(got, want)
        print("decode chain int8=%s rel-L2 %.2e max-abs %.2e" % (int8, r, np.abs(got - want).max()))
        if int8:
            # Every projection re-quantises its input to int8. The GPU's fused rmsnorm / SwiGLU differ
            # from the CPU's in the last ulp (summation order, expf), which moves a few codes across a
            # rounding boundary at each of the 13 quantisers of this chain; one code is 1/127 of a block's
            # amax, so end-of-chain agreement is bounded by quantisation noise, not by the 1e-3 kernel
            # tolerance. The kernel-level contract (same codes in -> rel-L2 <= 1e-3) is checked per
            # projection, with CPU-computed inputs, in test_gemv_gpu.py.
            assert r <= 5e-2
            want_f32 = oracle_chain(orc, W, h0, n_layers, eps, False)
            print("   vs f32-activation chain: rel-L2 %.2e" % rel_l2(got, want_f32))
            assert rel_l2(got, want_f32) <= 1e-1
        else:
            assert r <= REL_L2_TOL
        got2 = acc.decode_step(h0, 1)                                            # graph replay: bit-identical
        np.testing.assert_array_equal(got, got2)
        # declined configurations: real attention, post-norm
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, attn_standin_q=False) is False
        assert acc.decode_step(h0) is None
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, post_norm=True) is False
        # a missing weight declines too
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers + 1) is False
    finally:
        acc.close()


def oracle_chain_attn(orc, W, h0, n_layers, eps, kc, vc, pos, n_heads, n_kv, hd, base, int8=False):
    """qwen3.rs:818-899 for one token at `pos`; kc / vc: per-layer python lists that grow by one row."""
    def mm(name, x):
        w, ty, k, n = W[name]
        if int8:
            xq, xd, _ = orc.xquant8(x)
            return orc.idot_gemm(w, ty, xq, xd, 1, k, n)[0]
        return orc.qmatmul(x, w, ty, k, n)

    h = h0.astype(np.float32).copy()
    for il in range(n_layers):
        b = "blk.%d." % il
        n_ = orc.rmsnorm(h, W[b + "attn_norm.weight"], eps)
        q, k, v = mm(b + "attn_q.weight", n_), mm(b + "attn_k.weight", n_), mm(b + "attn_v.weight", n_)
        a = orc.attention_token(q, k, v, W.get(b + "attn_q_norm.weight"), W.get(b + "attn_k_norm.weight"), pos,
                                kc[il], vc[il], n_heads, n_kv, hd, eps, base)
        h = (h + mm(b + "attn_output.weight", a)).astype(np.float32)
        n_ = orc.rmsnorm(h, W[b + "ffn_norm.weight"], eps)
        g, u = mm(b + "ffn_gate.weight", n_), mm(b + "ffn_up.weight", n_)
        h = (h + mm(b + "ffn_down.weight", orc.swiglu(g, u))).astype(np.float32)
    return mm("output.weight", orc.rmsnorm(h, W["output_norm.weight"], eps))


@pytest.mark.parametrize("qk_norm", [True, False])
def test_decode_step_with_real_attention(pkg, orc, synth, qk_norm):
    """Dense Qwen3 step: QK-norm, NEOX rope, KV cache, grouped-query softmax; several positions, the
    positions cross several softmax splits (64 cached tokens each) so that the fold of the splits is exercised."""
    hidden, hd, n_heads, n_kv, ffn, vocab, n_layers, eps, base = 256, 64, 6, 2, 512, 1000, 2, 1e-6, 1e6
    qdim, kvdim, max_seq = n_heads * hd, n_kv * hd, 300
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed=83)
        if qk_norm:
            for il in range(n_layers):
                for nn in ("attn_q_norm.weight", "attn_k_norm.weight"):
                    W["blk.%d.%s" % (il, nn)] = synth.norm_weight(83, "blk.%d.%s" % (il, nn), hd)
                    acc.upload_f32("blk.%d.%s" % (il, nn), W["blk.%d.%s" % (il, nn)])
        kw = dict(eps=eps, act=pkg.ACT_F32, attn_standin_q=False, head_dim=hd, n_kv=n_kv, rope_theta=base,
                  max_seq=max_seq, qk_norm=qk_norm)
        # declined: sliding-window layer, shared K = V, GPT-J style rope, a head size that does not match the weights
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, layer_overrides={1: {"is_local": 1}}, **kw) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, layer_overrides={0: {"k_eq_v": 1}}, **kw) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, layer_overrides={0: {"rope_norm": 1}}, **kw) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, **dict(kw, head_dim=32)) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, **kw)
        kc, vc = [[] for _ in range(n_layers)], [[] for _ in range(n_layers)]
        worst = 0.0
        n_tok = 262
        for pos in range(n_tok):
            h0 = synth.normal(84, "h.%d" % pos, hidden)
            got = acc.decode_step(h0, pos)
            # the oracle's own cache must grow at every position; compare at a few
            want = oracle_chain_attn(orc, W, h0, n_layers, eps, kc, vc, pos, n_heads, n_kv, hd, base)
            if pos < 4 or pos in (17, 100, 255, 256, 257, n_tok - 1):
                r = rel_l2(got, want)
                worst = max(worst, r)
                assert r <= REL_L2_TOL, (pos, r)
        print("real attention qk_norm=%s: worst rel-L2 over checked positions %.2e" % (qk_norm, worst))
        # a position is re-playable: same input, same position, same cache rows below it -> same bits
        h0 = synth.normal(84, "h.%d" % (n_tok - 1), hidden)
        np.testing.assert_array_equal(acc.decode_step(h0, n_tok - 1), got)
        assert acc.decode_step_argmax(h0, n_tok - 1) == orc.argmax_f32(got)
        with pytest.raises(pkg.StrixCudaError, match="beyond max_seq"):
            acc.decode_step(h0, max_seq)
        assert acc.device_status() == 0
    finally:
        acc.close()


@pytest.mark.parametrize("int8", [False, True])
def test_prefill_verify_and_seeded_cache(pkg, orc, synth, int8):
    """prefill / verify push m tokens through the chain in one pass over the weights (batched GEMV rows,
    causal attention row after row); the cache they leave behind is the one token-at-a-time decoding
    would have built, and seed_decode_kv can install the same rows from outside."""
    hidden, hd, n_heads, n_kv, ffn, vocab, n_layers, eps, base = 256, 64, 4, 2, 512, 700, 2, 1e-6, 1e4
    qdim, kvdim, max_seq = n_heads * hd, n_kv * hd, 64
    act = pkg.ACT_Q8DOT if int8 else pkg.ACT_F32
    tol = 5e-2 if int8 else REL_L2_TOL      # int8: re-quantisation noise along the chain (see the chain test above)
    acc = pkg.CudaWeightAccel(0)
    try:
        assert acc.prefill_max() == 0                                   # nothing configured
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed=85)
        for il in range(n_layers):
            for nn in ("attn_q_norm.weight", "attn_k_norm.weight"):
                W["blk.%d.%s" % (il, nn)] = synth.norm_weight(85, "blk.%d.%s" % (il, nn), hd)
                acc.upload_f32("blk.%d.%s" % (il, nn), W["blk.%d.%s" % (il, nn)])
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, eps=eps, act=act, attn_standin_q=False,
                                    head_dim=hd, n_kv=n_kv, rope_theta=base, max_seq=max_seq)
        assert acc.prefill_max() == 8
        hs = synth.normal(86, "hs", 13 * hidden).reshape(13, hidden)
        kc, vc = [[] for _ in range(n_layers)], [[] for _ in range(n_layers)]
        want = [oracle_chain_attn(orc, W, hs[t], n_layers, eps, kc, vc, t, n_heads, n_kv, hd, base, int8=int8)
                for t in range(13)]
        # prompt of 5 tokens: prefill returns the last token's logits
        got = acc.prefill(hs[:5], 0, 5)
        assert rel_l2(got, want[4]) <= tol
        # speculative verify of 4 rows at positions 5..8: all logits
        gv = acc.verify(hs[5:9], 5, 4)
        assert gv.shape == (4, vocab)
        for t in range(4):
            assert rel_l2(gv[t], want[5 + t]) <= tol, t
        # rejected draft: positions 7, 8 are decoded again one at a time over the same cache rows
        for t in (7, 8, 9):
            assert rel_l2(acc.decode_step(hs[t], t), want[t]) <= tol
        # a full chunk of 8 rows re-verifies positions 2..9 (rows are rewritten with the same values)
        g8 = acc.verify(hs[2:10], 2, 8)
        for t in range(8):
            assert rel_l2(g8[t], want[2 + t]) <= tol
        # guards: more than prefill_max rows / zero rows -> None; positions past the cache -> error
        assert acc.verify(hs[:9], 0, 9) is None and acc.prefill(hs[:1], 0, 0) is None
        with pytest.raises(pkg.StrixCudaError, match="beyond max_seq"):
            acc.verify(hs[:4], max_seq - 2, 4)
        # a cache seeded from outside (the oracle's rows 0..9) continues identically at position 10
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, eps=eps, act=act, attn_standin_q=False,
                                    head_dim=hd, n_kv=n_kv, rope_theta=base, max_seq=max_seq)
        for il in range(n_layers):
            assert acc.seed_decode_kv(il, np.stack(kc[il][:10]), np.stack(vc[il][:10]))
        assert acc.seed_decode_kv(n_layers, np.zeros(kvdim, np.float32), np.zeros(kvdim, np.float32)) is False
        for t in (10, 11, 12):
            assert rel_l2(acc.decode_step(hs[t], t), want[t]) <= tol
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_verify_rows_with_the_attention_standin(pkg, orc, synth):
    """Without real attention (the benchmark's projection chain) verify rows are independent of one another."""
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 768, 256, 1536, 900, 2, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed=87)
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, eps=eps, act=pkg.ACT_F32)
        hs = synth.normal(88, "hs", 6 * hidden).reshape(6, hidden)
        gv = acc.verify(hs, 0, 6)
        for t in range(6):
            assert rel_l2(gv[t], oracle_chain(orc, W, hs[t], n_layers, eps, False)) <= REL_L2_TOL
        assert rel_l2(acc.prefill(hs, 0, 6), oracle_chain(orc, W, hs[5], n_layers, eps, False)) <= REL_L2_TOL
        assert acc.seed_decode_kv(0, np.zeros(kvdim, np.float32), np.zeros(kvdim, np.float32)) is False
    finally:
        acc.close()
