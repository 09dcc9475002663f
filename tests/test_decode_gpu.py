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


@pytest.mark.parametrize("chain_kernel", [0, 1])
@pytest.mark.parametrize("int8", [False, True])
def test_decode_step_matches_oracle_chain(pkg, orc, synth, int8, chain_kernel):
    """chain_kernel = 1: the whole chain as one persistent kernel (integer-dot form); 0: one launch per step."""
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 768, 256, 1536, 3000, 3, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        assert acc.set_option("decode_chain", chain_kernel)
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


def build_model_types(accel, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed, ty_attn, ty_ffn, ty_down, ty_head):
    """A random-init model with a weight format per projection family (the chain kernel walks steps of
    different formats in one launch)."""
    W = {}
    ups = {synth.Q4_0: accel.upload_q4_0, synth.Q4_1: accel.upload_q4_1, synth.Q6_K: accel.upload_q6_k,
           synth.Q8_0: accel.upload_q8_0}

    def up(name, ty, n, k):
        w = synth.quant(ty, seed, name, n, k)
        assert ups[ty](name, w, k, n), name
        W[name] = (w, ty, k, n)

    for il in range(n_layers):
        b = "blk.%d." % il
        up(b + "attn_q.weight", ty_attn, qdim, hidden)
        up(b + "attn_k.weight", ty_attn, kvdim, hidden)
        up(b + "attn_v.weight", ty_attn, kvdim, hidden)
        up(b + "attn_output.weight", ty_attn, hidden, qdim)
        up(b + "ffn_gate.weight", ty_ffn, ffn, hidden)
        up(b + "ffn_up.weight", ty_ffn, ffn, hidden)
        up(b + "ffn_down.weight", ty_down, hidden, ffn)
        for nn in ("attn_norm.weight", "ffn_norm.weight"):
            W[b + nn] = synth.norm_weight(seed, b + nn, hidden)
            accel.upload_f32(b + nn, W[b + nn])
    up("output.weight", ty_head, vocab, hidden)
    W["output_norm.weight"] = synth.norm_weight(seed, "output_norm", hidden)
    accel.upload_f32("output_norm.weight", W["output_norm.weight"])
    return W


@pytest.mark.parametrize("gelu", [False, True])
@pytest.mark.parametrize("fmts", ["q4_0+q6_k", "q8_0+q8_0", "q4_1 down+q4_0", "q6_k ffn"])
def test_chain_kernel_formats_and_ragged_shapes(pkg, orc, synth, fmts, gelu):
    """The persistent chain kernel against the oracle chain on shapes that are not multiples of anything
    convenient: row counts that leave a ragged last row group (k / v 264, vocab 2999), odd numbers of row
    groups (q 50, ffn 66), fewer row
    groups than SMs in some steps and more than the 12 waiting slots in others, a step list that mixes
    formats, and both gate activations. The launch-per-step path must agree with it to quantiser noise."""
    T = {"q4_0+q6_k": (synth.Q4_0, synth.Q4_0, synth.Q4_0, synth.Q6_K),
         "q8_0+q8_0": (synth.Q8_0, synth.Q8_0, synth.Q8_0, synth.Q8_0),
         "q4_1 down+q4_0": (synth.Q4_0, synth.Q4_0, synth.Q4_1, synth.Q4_0),
         "q6_k ffn": (synth.Q4_0, synth.Q6_K, synth.Q6_K, synth.Q6_K)}[fmts]
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 800, 264, 1024 if T[2] == synth.Q6_K else 1056, 2999, 2, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model_types(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, 95, *T)
        h0 = synth.normal(96, "h0", hidden)
        want = oracle_chain(orc, W, h0, n_layers, eps, True, gelu=gelu)
        outs = {}
        for chain in (1, 0):
            assert acc.set_option("decode_chain", chain)
            assert acc.configure_decode(hidden, qdim // 8, ffn, vocab, n_layers, eps=eps, act=pkg.ACT_Q8DOT, act_gelu=gelu)
            outs[chain] = acc.decode_step(h0, 0)
            again = acc.decode_step(h0, 1)
            np.testing.assert_array_equal(outs[chain], again)           # replay: bit-identical (epochs move on)
            assert acc.device_status() == 0
        r1, r0, r10 = rel_l2(outs[1], want), rel_l2(outs[0], want), rel_l2(outs[1], outs[0])
        print("%s gelu=%s: chain kernel vs oracle %.2e, launches vs oracle %.2e, chain vs launches %.2e" % (fmts, gelu, r1, r0, r10))
        # end-of-chain agreement of integer-dot chains is bounded by quantiser noise (a code that lands on the
        # other side of a rounding boundary moves a block by 1/127 of its amax), see the test above
        assert r1 <= 5e-2 and r0 <= 5e-2 and r10 <= 5e-2
    finally:
        acc.close()


def test_chain_kernel_first_layer_steps_at_kernel_tolerance(pkg, orc, synth):
    """One layer, where every step's input can be replayed on the CPU from the step before it with the chain
    kernel's own outputs: the kernel-level contract (same activation in -> rel-L2 <= 1e-3 against the integer
    oracle) for the steps of the chain kernel, q/k/v (RMSNorm prologue), o (residual), down (SwiGLU from the
    gate|up epilogue, residual), head."""
    import torch
    hidden, qdim, kvdim, ffn, vocab, eps = 768, 1024, 256, 2048, 4000, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, 1, seed=97)
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, 1, eps=eps, act=pkg.ACT_Q8DOT)
        h0 = synth.normal(98, "h0", hidden)
        dev = torch.device("cuda:0")
        d_h = torch.from_numpy(h0).to(dev)
        d_logits = torch.zeros(vocab, device=dev)
        assert acc.decode_chain_dev(d_h.data_ptr(), d_logits.data_ptr(), stream=torch.cuda.current_stream().cuda_stream)
        torch.cuda.synchronize()
        assert acc.device_status() == 0
        h_out, logits = d_h.cpu().numpy(), d_logits.cpu().numpy()      # hidden state after the layer, logits

        def mm(name, x):
            w, ty, k, n = W[name]
            xq, xd, _ = orc.xquant8(x)
            return orc.idot_gemm(w, ty, xq, xd, 1, k, n)[0]
        b = "blk.0."
        n_ = orc.rmsnorm(h0, W[b + "attn_norm.weight"], eps)
        q = mm(b + "attn_q.weight", n_)
        h1 = (h0 + mm(b + "attn_output.weight", q)).astype(np.float32)
        n2 = orc.rmsnorm(h1, W[b + "ffn_norm.weight"], eps)
        a = orc.swiglu(mm(b + "ffn_gate.weight", n2), mm(b + "ffn_up.weight", n2))
        h2 = (h1 + mm(b + "ffn_down.weight", a)).astype(np.float32)
        r_h = rel_l2(h_out, h2)
        # the head from the KERNEL's hidden state: isolates the last step
        r_head = rel_l2(logits, mm("output.weight", orc.rmsnorm(h_out, W["output_norm.weight"], eps)))
        print("one layer: hidden state rel-L2 %.2e, head step rel-L2 %.2e" % (r_h, r_head))
        assert r_head <= REL_L2_TOL
        assert r_h <= 5e-3      # four quantisers deep: a handful of flipped codes
    finally:
        acc.close()


def test_sharded_chain_wait_runs_out_and_the_handle_recovers(pkg, orc, synth):
    """Failure detection without a fault: rank 0 of a group of two, alone on the GPU, never receives the other
    rank's rows. Its waits on the exchange vectors are bounded (here ~2000 polls), the kernel runs to its end,
    the status word shows the time-out, the call reports it, and the handle works afterwards."""
    hidden, qdim, kvdim, ffn, vocab, eps = 512, 768, 256, 1536, 1000, 1e-6
    acc = pkg.CudaWeightAccel(0, rank=0, world=2)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, 1, seed=99)
        assert acc.set_option("poll_limit", 2000)
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, 1, eps=eps, act=pkg.ACT_F32) is False   # sharded: integer-dot chain only
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, 1, eps=eps, act=pkg.ACT_Q8DOT)
        base, nbytes = acc.decode_exchange_info()
        assert base and nbytes >= 8 * (qdim + 2 * hidden + ffn)
        h0 = synth.normal(99, "h0", hidden)
        with pytest.raises(pkg.StrixCudaError) as ei:
            acc.decode_step(h0, 0)
        assert "bounded wait ran out" in str(ei.value)
        assert acc.device_status() == 0                                  # reported once, then cleared
        # the handle is still good: a plain GEMV on its shard of a weight agrees with the oracle
        w, ty, k, n = W["blk.0.attn_q.weight"]
        x = synth.normal(100, "x", k)
        got = acc.gemv("blk.0.attn_q.weight", x)
        want = orc.qmatmul(x, w, ty, k, n)[:len(got)]
        assert rel_l2(got, want) <= REL_L2_TOL
        assert acc.device_status() == 0
    finally:
        acc.close()


@pytest.mark.parametrize("int8", [False, True])
def test_decode_chain_config3_full_size(pkg, orc, synth, int8):
    """The decode configuration at its own size: 36 layers, hidden 2560, q 4096, k/v 1024, ffn 9728, Q4_0
    projections, Q6_K head over 151936 rows. End of chain against the oracle chain (f32 form at the kernel
    tolerance; the integer-dot chain kernel at quantiser noise), and every projection of the LAST layer and the
    head on CPU-computed inputs at the kernel tolerance."""
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 2560, 4096, 1024, 9728, 151936, 36, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed=3)
        act = pkg.ACT_Q8DOT if int8 else pkg.ACT_F32
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, eps=eps, act=act)
        h0 = synth.normal(3, "h0", hidden)
        got = acc.decode_step(h0, 0)
        assert acc.device_status() == 0
        # oracle chain, keeping the inputs of the last layer's projections
        inputs = {}

        def mm(name, x, keep=False):
            w, ty, k, n = W[name]
            if keep:
                inputs[name] = x.copy()
            if int8:
                xq, xd, _ = orc.xquant8(x)
                return orc.idot_gemm(w, ty, xq, xd, 1, k, n)[0]
            return orc.qmatmul(x, w, ty, k, n)
        h = h0.copy()
        for il in range(n_layers):
            b, last = "blk.%d." % il, il == n_layers - 1
            n_ = orc.rmsnorm(h, W[b + "attn_norm.weight"], eps)
            q = mm(b + "attn_q.weight", n_, last)
            mm(b + "attn_k.weight", n_, last)
            mm(b + "attn_v.weight", n_, last)
            h = (h + mm(b + "attn_output.weight", q, last)).astype(np.float32)
            n_ = orc.rmsnorm(h, W[b + "ffn_norm.weight"], eps)
            g, u = mm(b + "ffn_gate.weight", n_, last), mm(b + "ffn_up.weight", n_, last)
            h = (h + mm(b + "ffn_down.weight", orc.swiglu(g, u), last)).astype(np.float32)
        want = mm("output.weight", orc.rmsnorm(h, W["output_norm.weight"], eps), True)
        r = rel_l2(got, want)
        print("config 3 full size int8=%s: end of chain rel-L2 %.2e max-abs %.2e, argmax %d vs %d" %
              (int8, r, np.abs(got - want).max(), int(np.argmax(got)), int(np.argmax(want))))
        assert np.isfinite(got).all()
        # 36 layers deep: the f32 form accumulates rounding only; the integer form 145 quantisers' worth of noise
        assert r <= (1e-1 if int8 else REL_L2_TOL)
        for name, x in inputs.items():
            w, ty, k, n = W[name]
            g1 = acc.gemv(name, x, act=act)
            if int8:
                xq, xd, _ = orc.xquant8(x)
                w1 = orc.idot_gemm(w, ty, xq, xd, 1, k, n)[0]
            else:
                w1 = orc.qmatmul(x, w, ty, k, n)
            r1 = rel_l2(g1, w1)
            print("   %s on the CPU's input: rel-L2 %.2e max-abs %.2e" % (name, r1, np.abs(g1 - w1).max()))
            assert r1 <= REL_L2_TOL
    finally:
        acc.close()
