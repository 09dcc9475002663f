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
        # declined: a head size that does not match the weights, one beyond the kernels' limit, heads that do not group
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, **dict(kw, head_dim=32)) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, layer_overrides={1: {"head_dim": 516}}, **kw) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, layer_overrides={0: {"n_kv": 4}}, **kw) is False
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, layer_overrides={0: {"rope_theta": 0.0}}, **kw) is False
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


def build_model_flavour(acc, synth, hidden, n_heads, layers, ffn, vocab, seed, post_norm=False, qk_norm=False, freq_hd=0):
    """A random-init Q4_0 model with per-layer head sizes; layers: dicts with head_dim, n_kv, k_eq_v (no V weight then)."""
    W = {}

    def up(name, ty, n, k):
        w = synth.quant(ty, seed, name, n, k)
        ok = {synth.Q4_0: acc.upload_q4_0, synth.Q6_K: acc.upload_q6_k}[ty](name, w, k, n)
        assert ok, name
        W[name] = (w, ty, k, n)

    def f32(name, n, lo=None):
        W[name] = synth.norm_weight(seed, name, n) if lo is None else lo
        acc.upload_f32(name, W[name])

    for il, lc in enumerate(layers):
        b, hd = "blk.%d." % il, lc["head_dim"]
        up(b + "attn_q.weight", synth.Q4_0, n_heads * hd, hidden)
        up(b + "attn_k.weight", synth.Q4_0, lc["n_kv"] * hd, hidden)
        if not lc.get("k_eq_v"):
            up(b + "attn_v.weight", synth.Q4_0, lc["n_kv"] * hd, hidden)
        up(b + "attn_output.weight", synth.Q4_0, hidden, n_heads * hd)
        up(b + "ffn_gate.weight", synth.Q4_0, ffn, hidden)
        up(b + "ffn_up.weight", synth.Q4_0, ffn, hidden)
        up(b + "ffn_down.weight", synth.Q4_0, hidden, ffn)
        for nn in ("attn_norm.weight", "ffn_norm.weight"):
            f32(b + nn, hidden)
        if post_norm:
            for nn in ("post_attention_norm.weight", "post_ffw_norm.weight"):
                f32(b + nn, hidden)
        if qk_norm:
            for nn in ("attn_q_norm.weight", "attn_k_norm.weight"):
                f32(b + nn, hd)
    up("output.weight", synth.Q6_K, vocab, hidden)
    f32("output_norm.weight", hidden)
    if freq_hd:
        # proportional-rope frequency factors of the global layers (gemma.rs:367, 819-829): > 0, around 1 .. 8
        f32("rope_freqs.weight", freq_hd // 2, (1.0 + 7.0 * np.linspace(0.0, 1.0, freq_hd // 2) ** 2).astype(np.float32))
    return W


def oracle_chain_flavour(orc, W, h0, layers, eps, kc, vc, pos, n_heads, cfg, int8=False):
    """One token of smollm3.rs:557-680 / gemma.rs:772-925 over the oracle's pieces. cfg: post_norm, act_gelu, norm_v,
    attn_rsqrt, n_swa, final_softcap, kv_f16, qk_norm; layers: the GpuLayerCfg fields per layer. Returns RAW logits
    (the caller applies the soft-cap where it wants it)."""
    def mm(name, x):
        w, ty, k, n = W[name]
        if int8:
            xq, xd, _ = orc.xquant8(x)
            return orc.idot_gemm(w, ty, xq, xd, 1, k, n)[0]
        return orc.qmatmul(x, w, ty, k, n)

    h = h0.astype(np.float32).copy()
    for il, lc in enumerate(layers):
        b, hd = "blk.%d." % il, lc["head_dim"]
        n_ = orc.rmsnorm(h, W[b + "attn_norm.weight"], eps)
        q, k = mm(b + "attn_q.weight", n_), mm(b + "attn_k.weight", n_)
        v = None if lc.get("k_eq_v") else mm(b + "attn_v.weight", n_)
        if lc.get("no_rope"):
            rope = None
        elif cfg.get("post_norm"):
            rope = ("pow", lc["rope_theta"], None if lc.get("is_local") else W.get("rope_freqs.weight"))
        else:
            rope = ("chain", lc["rope_theta"])
        a = orc.attention_token_flavour(
            q, k, v, W.get(b + "attn_q_norm.weight") if cfg.get("qk_norm") else None,
            W.get(b + "attn_k_norm.weight") if cfg.get("qk_norm") else None, pos, kc[il], vc[il], n_heads, lc["n_kv"], hd, eps,
            rope, adjacent=bool(lc.get("rope_norm")), norm_v=bool(cfg.get("norm_v")),
            window=cfg.get("n_swa", 0) if lc.get("is_local") else 0,
            scale=None if cfg.get("attn_rsqrt", True) else 1.0, kv_f16=bool(cfg.get("kv_f16")))
        o = mm(b + "attn_output.weight", a)
        if cfg.get("post_norm"):
            h = orc.addnorm(h, o, W[b + "post_attention_norm.weight"], eps)
        else:
            h = (h + o).astype(np.float32)
        n_ = orc.rmsnorm(h, W[b + "ffn_norm.weight"], eps)
        g, u = mm(b + "ffn_gate.weight", n_), mm(b + "ffn_up.weight", n_)
        dn = mm(b + "ffn_down.weight", orc.geglu(g, u) if cfg.get("act_gelu") else orc.swiglu(g, u))
        if cfg.get("post_norm"):
            h = orc.addnorm(h, dn, W[b + "post_ffw_norm.weight"], eps, lc.get("output_scale", 1.0))
        else:
            h = (h + dn).astype(np.float32)
    return mm("output.weight", orc.rmsnorm(h, W["output_norm.weight"], eps))


def test_decode_step_smollm3_flavour(pkg, orc, synth):
    """smollm3.rs:557-680: no QK-norm, adjacent-pair rope (the Llama-permuted layout), every second layer without rope."""
    hidden, hd, n_heads, n_kv, ffn, vocab, eps, base, max_seq = 256, 64, 4, 2, 512, 800, 1e-6, 5e6, 160
    layers = [dict(head_dim=hd, n_kv=n_kv, rope_theta=base, rope_norm=1, no_rope=int(il % 2 == 1)) for il in range(2)]
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model_flavour(acc, synth, hidden, n_heads, layers, ffn, vocab, seed=301)
        assert acc.configure_decode(hidden, n_heads, ffn, vocab, 2, eps=eps, act=pkg.ACT_F32, attn_standin_q=False,
                                    max_seq=max_seq, qk_norm=False, layers=layers)
        kc, vc = [[], []], [[], []]
        worst = 0.0
        for pos in range(131):
            h0 = synth.normal(302, "h.%d" % pos, hidden)
            got = acc.decode_step(h0, pos)
            want = oracle_chain_flavour(orc, W, h0, layers, eps, kc, vc, pos, n_heads, dict(qk_norm=False))
            if pos < 3 or pos in (63, 64, 65, 130):
                r = rel_l2(got, want)
                worst = max(worst, r)
                assert r <= REL_L2_TOL, (pos, r)
        print("smollm3 flavour: worst rel-L2 %.2e" % worst)
        assert acc.device_status() == 0
    finally:
        acc.close()


GEMMA_LAYERS = [
    # local layer: its own head size, sliding window, rope base 1e4, no frequency factors
    dict(head_dim=64, n_kv=2, k_eq_v=0, rope_theta=1e4, is_local=1, output_scale=0.75),
    # global layer: wider heads, one KV head shared by all, V = raw K, rope base 1e6 with frequency factors
    dict(head_dim=128, n_kv=1, k_eq_v=1, rope_theta=1e6, is_local=0, output_scale=1.25),
    dict(head_dim=64, n_kv=2, k_eq_v=0, rope_theta=1e4, is_local=1, output_scale=0.9),
]
GEMMA_CFG = dict(post_norm=True, act_gelu=True, norm_v=True, attn_rsqrt=False, n_swa=40, final_softcap=30.0, qk_norm=True)


def gemma_configure(pkg, acc, hidden, n_heads, ffn, vocab, eps, max_seq, act, cfg=GEMMA_CFG):
    return acc.configure_decode(hidden, n_heads, ffn, vocab, len(GEMMA_LAYERS), eps=eps, act=act, attn_standin_q=False,
                                max_seq=max_seq, qk_norm=True, layers=GEMMA_LAYERS, post_norm=True, act_gelu=True,
                                norm_v=cfg["norm_v"], attn_rsqrt=cfg["attn_rsqrt"], n_swa=cfg["n_swa"],
                                final_softcap=cfg["final_softcap"])


@pytest.mark.parametrize("kv_f16", [False, True])
def test_decode_step_gemma_flavour(pkg, orc, synth, kv_f16):
    """gemma.rs:772-925: per-layer head sizes, shared K = V on the global layer, weightless V-norm, QK-norm, rope with
    frequency factors on the global layer, a sliding window of 40 rows on the local layers (positions run past it and
    past a softmax split), scale 1.0, GeGLU, sandwich post-norms with per-layer output scales, final soft-cap.
    kv_f16: the cache keeps f16 rows rounded as the reference's cache stores round (kernels.rs:18-35)."""
    hidden, n_heads, ffn, vocab, eps, max_seq = 256, 4, 512, 900, 1e-6, 128
    cfg = dict(GEMMA_CFG, kv_f16=kv_f16)
    acc = pkg.CudaWeightAccel(0)
    try:
        assert acc.set_option("kv_f16", int(kv_f16))
        W = build_model_flavour(acc, synth, hidden, n_heads, GEMMA_LAYERS, ffn, vocab, seed=311, post_norm=True, qk_norm=True,
                                freq_hd=128)
        assert gemma_configure(pkg, acc, hidden, n_heads, ffn, vocab, eps, max_seq, pkg.ACT_F32)
        kc, vc = [[] for _ in GEMMA_LAYERS], [[] for _ in GEMMA_LAYERS]
        worst = 0.0
        for pos in range(100):
            h0 = synth.normal(312, "h.%d" % pos, hidden)
            got = acc.decode_step(h0, pos)
            raw = oracle_chain_flavour(orc, W, h0, GEMMA_LAYERS, eps, kc, vc, pos, n_heads, cfg)
            if pos < 3 or pos in (39, 40, 41, 63, 64, 65, 99):
                want = orc.softcap(raw, cfg["final_softcap"])
                r = rel_l2(got, want)
                worst = max(worst, r)
                # f16 rows: a GPU value one f32 ulp from the oracle's can round to the neighbouring f16 code
                assert r <= (3e-3 if kv_f16 else REL_L2_TOL), (pos, r)
                assert np.abs(got).max() <= cfg["final_softcap"]
        print("gemma flavour kv_f16=%s: worst rel-L2 %.2e" % (kv_f16, worst))
        # the greedy entry point skips the soft-cap (monotone): same winner
        h0 = synth.normal(312, "h.99", hidden)
        assert acc.decode_step_argmax(h0, 99) == orc.argmax_f32(got)
        assert acc.device_status() == 0
    finally:
        acc.close()


@pytest.mark.parametrize("kv_f16", [False, True])
def test_prefill_verify_gemma_flavour_and_seeded_f16_cache(pkg, orc, synth, kv_f16):
    """The batched rows (prefill / verify) of the Gemma flavour against token-at-a-time oracle steps, with the
    integer-dot projections; then a cache seeded from outside (f32 rows in, rounded to f16 by the library when the
    cache is f16) continues like the one decoding built."""
    hidden, n_heads, ffn, vocab, eps, max_seq = 256, 4, 512, 900, 1e-6, 64
    cfg = dict(GEMMA_CFG, n_swa=6, kv_f16=kv_f16)
    acc = pkg.CudaWeightAccel(0)
    try:
        assert acc.set_option("kv_f16", int(kv_f16))
        W = build_model_flavour(acc, synth, hidden, n_heads, GEMMA_LAYERS, ffn, vocab, seed=321, post_norm=True, qk_norm=True,
                                freq_hd=128)
        assert gemma_configure(pkg, acc, hidden, n_heads, ffn, vocab, eps, max_seq, pkg.ACT_Q8DOT, cfg)
        hs = synth.normal(322, "hs", 14 * hidden).reshape(14, hidden)
        kc, vc = [[] for _ in GEMMA_LAYERS], [[] for _ in GEMMA_LAYERS]
        want = [orc.softcap(oracle_chain_flavour(orc, W, hs[t], GEMMA_LAYERS, eps, kc, vc, t, n_heads, cfg, int8=True), 30.0)
                for t in range(14)]
        # re-quantisation noise along an integer-dot chain of 13 quantisers (a code that flips moves a value by 1/127
        # of its block's amax; with f16 rows a flip of a cache code adds to it); the flavours themselves are held to
        # 1e-3 with f32 activations in test_decode_step_gemma_flavour
        tol = 8e-2
        assert rel_l2(acc.prefill(hs[:5], 0, 5), want[4]) <= tol
        gv = acc.verify(hs[5:12], 5, 7)                    # rows 5..11 run past the window of 6
        for t in range(7):
            assert rel_l2(gv[t], want[5 + t]) <= tol, t
        assert rel_l2(acc.decode_step(hs[12], 12), want[12]) <= tol
        from strix_rs_b200 import spec
        ids = spec.verify_argmax(acc, hs[5:12], 5, 7)
        assert list(ids) == [orc.argmax_f32(gv[t]) for t in range(7)]
        # a cache seeded from outside continues identically
        assert gemma_configure(pkg, acc, hidden, n_heads, ffn, vocab, eps, max_seq, pkg.ACT_Q8DOT, cfg)
        for il in range(len(GEMMA_LAYERS)):
            assert acc.seed_decode_kv(il, np.stack(kc[il][:13]), np.stack(vc[il][:13]))
        assert rel_l2(acc.decode_step(hs[13], 13), want[13]) <= tol
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_post_norm_chain_with_the_attention_standin(pkg, orc, synth):
    """The sandwich post-norm residuals on the projection chain alone (stand-in attention): launch path, f32."""
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 768, 256, 1536, 1100, 2, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        W = build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers, seed=331)
        for il in range(n_layers):
            for nn in ("post_attention_norm.weight", "post_ffw_norm.weight"):
                W["blk.%d.%s" % (il, nn)] = synth.norm_weight(331, "blk.%d.%s" % (il, nn), hidden)
                acc.upload_f32("blk.%d.%s" % (il, nn), W["blk.%d.%s" % (il, nn)])
        scales = [0.5, 1.5]
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, eps=eps, act=pkg.ACT_F32, post_norm=True,
                                    final_softcap=20.0, layers=[dict(output_scale=s) for s in scales])
        h0 = synth.normal(332, "h0", hidden)

        def mm(name, x):
            w, ty, k, n = W[name]
            return orc.qmatmul(x, w, ty, k, n)
        h = h0.copy()
        for il in range(n_layers):
            b = "blk.%d." % il
            n_ = orc.rmsnorm(h, W[b + "attn_norm.weight"], eps)
            q = mm(b + "attn_q.weight", n_)
            h = orc.addnorm(h, mm(b + "attn_output.weight", q), W[b + "post_attention_norm.weight"], eps)
            n_ = orc.rmsnorm(h, W[b + "ffn_norm.weight"], eps)
            a = orc.swiglu(mm(b + "ffn_gate.weight", n_), mm(b + "ffn_up.weight", n_))
            h = orc.addnorm(h, mm(b + "ffn_down.weight", a), W[b + "post_ffw_norm.weight"], eps, scales[il])
        want = orc.softcap(mm("output.weight", orc.rmsnorm(h, W["output_norm.weight"], eps)), 20.0)
        assert rel_l2(acc.decode_step(h0, 0), want) <= REL_L2_TOL
        gv = acc.verify(np.stack([h0, h0]), 0, 2)
        assert rel_l2(gv[1], want) <= REL_L2_TOL
    finally:
        acc.close()
