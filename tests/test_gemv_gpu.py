"""GPU parity of upload/repack and the dequant-GEMV family against the CPU oracle,
through the C ABI. Tier 1 (bit-exact): dequantised weights, the activation
quantiser. Tier 2: f32 outputs within rel-L2 1e-3 (max-abs printed)."""
import os

import numpy as np
import pytest

pytestmark = pytest.mark.gpu

HERE = os.path.dirname(os.path.abspath(__file__))
REL_L2_TOL = 1e-3   # the tolerance the benchmark contract states for floating-point outputs


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def uploader(accel, synth, ty):
    return {synth.Q4_0: accel.upload_q4_0, synth.Q4_1: accel.upload_q4_1, synth.Q8_0: accel.upload_q8_0,
            synth.Q6_K: accel.upload_q6_k}[ty]


# ------------------------------------------------------------------ tier 1
@pytest.mark.parametrize("name,ty", [("q4_0", 2), ("q8_0", 8), ("q6_k", 14)])
def test_dequant_golden_bit_exact(accel, name, ty, synth):
    g = np.load(os.path.join(HERE, "golden", "dequant_golden.npz"))
    raw, want = g[name + "_raw"], g[name + "_f32"]
    be = synth.BLOCK_ELEMS[ty]
    rows = 4
    in_dim = want.size // rows
    assert in_dim % be == 0
    assert uploader(accel, synth, ty)("golden." + name, raw, in_dim, rows)
    got = accel.dequant_to_f32("golden." + name).reshape(-1)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


@pytest.mark.parametrize("ty,shapes", [
    (2, [(1, 32), (7, 64), (9, 2560), (33, 4096), (8, 9728), (5, 16384)]),
    (8, [(1, 32), (7, 96), (9, 2560), (33, 4096), (8, 9728), (3, 16384)]),
    (14, [(1, 256), (7, 512), (9, 2560), (33, 4096), (8, 9728), (3, 16384)]),
    (3, [(1, 32), (7, 64), (9, 2560), (33, 4096), (8, 9728), (5, 16384)]),
])
def test_dequant_matches_oracle_bit_exact(accel, orc, synth, ty, shapes):
    for out_dim, in_dim in shapes:
        w = synth.quant(ty, 21, "dq", out_dim, in_dim)
        key = "dq.%d.%d.%d" % (ty, out_dim, in_dim)
        assert uploader(accel, synth, ty)(key, w, in_dim, out_dim)
        got = accel.dequant_to_f32(key)
        want = orc.dequantize(ty, w, out_dim * in_dim).reshape(out_dim, in_dim)
        np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_xquant8_bit_exact(accel, orc, synth):
    x = synth.normal(22, "xq", 4 * 9728)
    x[0:32] = 0.0                                # an all-zero block: d = 0, q = 0
    x[32:40] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5]   # ties, |amax| = 127
    x[40:64] = 0.0
    q, d = accel.xquant8(x)
    wq, wd, ties = orc.xquant8(x)
    assert ties >= 7
    np.testing.assert_array_equal(d.view(np.uint32), wd.view(np.uint32))
    np.testing.assert_array_equal(q, wq)


# ------------------------------------------------------------------ boundary behaviour
def test_upload_declines_like_the_reference(accel, synth):
    w = synth.q4_0(1, "d", 4, 64)
    assert accel.upload_q4_0("bad.k", w, 48, 4) is False          # in_dim % 32 != 0  (decode.rs:2492-2494)
    assert accel.upload_q4_0("bad.len", w[:-1], 64, 4) is False   # len mismatch       (decode.rs:2497-2499)
    assert accel.upload_q6_k("bad.k6", w, 128, 4) is False        # in_dim % 256 != 0  (decode.rs:2630-2632)
    assert accel.upload_q4_1("q41", w, 64, 4) is False            # 18-byte blocks are not Q4_1's 20 (decode.rs:2594-2596)
    assert accel.upload_q4_1("q41", synth.q4_1(1, "d", 4, 64), 48, 4) is False   # in_dim % 32 != 0 (decode.rs:2589-2591)
    assert accel.weight_info("bad.k") is None and accel.weight_info("bad.len") is None


def test_gemv_none_for_unknown_key_or_bad_length(accel, synth):
    w = synth.q8_0(1, "n", 8, 64)
    assert accel.upload_q8_0("none.w", w, 64, 8)
    assert accel.gemv("no.such.key", np.zeros(64, np.float32)) is None     # decode.rs:3898 falls to None
    assert accel.gemv("none.w", np.zeros(32, np.float32)) is None          # x.len() != in_dim
    assert accel.gemv("none.w", np.zeros(64, np.float32)) is not None


def test_resident_count_and_name(accel, synth):
    n0 = accel.resident_count()
    assert accel.upload_q8_0("cnt.a", synth.q8_0(1, "c", 2, 32), 32, 2)
    assert accel.resident_count() == n0 + 1
    assert accel.upload_q8_0("cnt.a", synth.q8_0(2, "c", 2, 32), 32, 2)   # same key replaces
    assert accel.resident_count() == n0 + 1
    assert "B200" in accel.name() or "sm_100" in accel.name()


# ------------------------------------------------------------------ tier 2: GEMV
GEMV_CASES = [
    # (ggml type, out_dim, in_dim)            edge shapes then the benchmark shapes
    (2, 1, 32), (2, 7, 64), (2, 9, 96), (2, 257, 2560), (2, 4096, 4096), (2, 2560, 9728), (2, 100, 16384),
    (8, 1, 32), (8, 8, 64), (8, 9, 3840), (8, 9728, 2560), (8, 2560, 9728), (8, 64, 16384),
    (14, 1, 256), (14, 7, 512), (14, 17, 3840), (14, 9728, 2560), (14, 2560, 9728), (14, 40, 16384),
    # Q4_1 (llama.cpp keeps early-layer ffn_down in it): value = d * code + m
    (3, 1, 32), (3, 7, 64), (3, 9, 96), (3, 257, 2560), (3, 2560, 9728), (3, 50, 16384), (3, 19, 20480),
    # rows longer than the activation prologue keeps in registers (6 float4 x 768 threads = 18432 values):
    # the rest of the row is re-read; and the widest FFN of the reference's model zoo (27648)
    (2, 33, 20480), (8, 20, 27648), (14, 18, 20480),
]


@pytest.mark.parametrize("ty,out_dim,in_dim", GEMV_CASES)
def test_gemv_f32_and_q8dot_match_oracle(accel, orc, synth, pkg, ty, out_dim, in_dim):
    w = synth.quant(ty, 31, "gv", out_dim, in_dim)
    x = synth.normal(31, "gv.x", in_dim)
    key = "gv.%d.%d.%d" % (ty, out_dim, in_dim)
    assert uploader(accel, synth, ty)(key, w, in_dim, out_dim)
    want = orc.qmatmul(x, w, ty, in_dim, out_dim)
    got = accel.gemv(key, x)
    assert got.shape == (out_dim,) and np.isfinite(got).all()
    r = rel_l2(got, want)
    print("f32   ty=%d %dx%d rel-L2 %.2e max-abs %.2e" % (ty, out_dim, in_dim, r, np.abs(got - want).max()))
    assert r <= REL_L2_TOL
    # integer-dot variant: tolerance applies against the integer oracle (same quantised operands)
    xq, xd, _ = orc.xquant8(x)
    want_i = orc.idot_gemm(w, ty, xq, xd, 1, in_dim, out_dim)[0]
    got_i = accel.gemv(key, x, act=pkg.ACT_Q8DOT)
    ri = rel_l2(got_i, want_i)
    rf = rel_l2(got_i, want)
    print("q8dot ty=%d %dx%d rel-L2 vs int oracle %.2e (max-abs %.2e), vs f32 oracle %.2e"
          % (ty, out_dim, in_dim, ri, np.abs(got_i - want_i).max(), rf))
    assert ri <= REL_L2_TOL
    if in_dim >= 512:          # a handful of blocks is too few for the statistical bound to hold
        assert rf <= 2e-2      # activation quantisation error; the reference's own dp4a bound
    assert accel.device_status() == 0


@pytest.mark.parametrize("rule", [0, 2])
@pytest.mark.parametrize("out_dim,in_dim", [(300, 256), (1030, 2560), (64, 9728)])
def test_q6k_f32_forms_agree(accel, orc, synth, rule, out_dim, in_dim):
    """Q6_K with one f32 row runs either on f16 tensor-core tiles (activation split hi + lo) or on int8
    tiles (activation as three base-254 digits). The option "q6k_digits" picks: 0 = never the digit form,
    2 = whenever it fits. Both must sit at f32 rounding level from the f64 product of the dequantised
    weight, far inside the contract's tolerance."""
    assert accel.set_option("q6k_digits", rule)
    w = synth.quant(14, 41, "dg", out_dim, in_dim)
    assert accel.upload_q6_k("dg", w, in_dim, out_dim)
    W = accel.dequant_to_f32("dg").reshape(out_dim, in_dim).astype(np.float64)
    for seed, scale in ((1, 1.0), (2, 1e-4), (3, 3e3)):
        x = (synth.normal(seed, "dg.x", in_dim) * scale).astype(np.float32)
        x[::7] = 0.0                      # zeros inside blocks
        x[32:64] = 0.0                    # an all-zero block
        got = accel.gemv("dg", x)
        assert rel_l2(got, W @ x.astype(np.float64)) <= 2e-6
        assert rel_l2(got, orc.qmatmul(x, w, 14, in_dim, out_dim)) <= REL_L2_TOL
    assert accel.device_status() == 0
    assert accel.set_option("q6k_digits", 1)
    assert accel.set_option("no_such_knob", 1) is False


@pytest.mark.parametrize("rule", [0, 2])
@pytest.mark.parametrize("fmt", ["q8_0", "q4_0"])
@pytest.mark.parametrize("out_dim,in_dim", [(300, 256), (1030, 2560), (64, 9728)])
def test_q8_0_and_q4_0_f32_forms_agree(accel, orc, synth, fmt, rule, out_dim, in_dim):
    """Q8_0 and Q4_0 with one f32 row, like Q6_K: f16 tensor-core tiles (rule 0) or the three-digit int8 form
    (rule 2 = whenever it fits; the default takes it up to 8192 elements). Both at f32 rounding level from the f64
    product of the dequantised weight, and inside the contract against the oracle."""
    ty = synth.Q8_0 if fmt == "q8_0" else synth.Q4_0
    opt = fmt + "_digits"
    assert accel.set_option(opt, rule)
    try:
        key = "dg." + fmt
        w = synth.quant(ty, 43, key, out_dim, in_dim)
        assert uploader(accel, synth, ty)(key, w, in_dim, out_dim)
        W = accel.dequant_to_f32(key).reshape(out_dim, in_dim).astype(np.float64)
        for seed, scale in ((1, 1.0), (2, 1e-4), (3, 3e3)):
            x = (synth.normal(seed, key + ".x", in_dim) * scale).astype(np.float32)
            x[::7] = 0.0                      # zeros inside blocks
            x[32:64] = 0.0                    # an all-zero block
            got = accel.gemv(key, x)
            assert rel_l2(got, W @ x.astype(np.float64)) <= 2e-6
            assert rel_l2(got, orc.qmatmul(x, w, ty, in_dim, out_dim)) <= REL_L2_TOL
        assert accel.device_status() == 0
    finally:
        assert accel.set_option(opt, 1)


def test_lm_head_shapes(accel, orc, synth):
    # the 2560 -> 151936 lm_head of the benchmark, Q8_0 and Q6_K; every row must be written
    # (the reference once left half the rows unwritten through a grid-size slip, README.md:125-128)
    in_dim, out_dim = 2560, 151936
    x = synth.normal(32, "lm.x", in_dim)
    for ty in (synth.Q8_0, synth.Q6_K):
        w = synth.quant(ty, 32, "lm", out_dim, in_dim)
        assert uploader(accel, synth, ty)("lm.%d" % ty, w, in_dim, out_dim)
        want = orc.qmatmul(x, w, ty, in_dim, out_dim)
        got = accel.gemv("lm.%d" % ty, x)
        assert rel_l2(got, want) <= REL_L2_TOL
        # per-row check so that an unwritten stretch cannot hide inside a norm
        assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()
    accel.upload_q8_0("lm.8", synth.q8_0(1, "tiny", 1, 32), 32, 1)      # release the big buffers
    accel.upload_q6_k("lm.14", synth.q6_k(1, "tiny", 1, 256), 256, 1)


def test_reference_device_test_recipe(accel, orc, synth):
    # crates/strix-backend-rocm/src/lib.rs:132-232: 3840 x 15360 Q4_0 from the LCG,
    # asserted there as max_err / max|cpu| < 1e-3
    out_dim, in_dim = 3840, 15360
    w, x = synth.lcg_q4_0(out_dim, in_dim)
    assert accel.upload_q4_0("lcg", w, in_dim, out_dim)
    want = orc.qmatmul(x, w, synth.Q4_0, in_dim, out_dim)
    got = accel.gemv("lcg", x)
    assert np.abs(got - want).max() / np.abs(want).max() < 1e-3


def test_gemv_batch_one_sync(accel, orc, synth):
    calls, wants = [], []
    for i, (ty, n, k) in enumerate([(8, 100, 256), (8, 33, 512), (2, 65, 128), (14, 17, 512)]):
        w = synth.quant(ty, 40 + i, "b", n, k)
        assert uploader(accel, synth, ty)("batch.%d" % i, w, k, n)
        x = synth.normal(40 + i, "b.x", k)
        calls.append(("batch.%d" % i, x))
        wants.append(orc.qmatmul(x, w, ty, k, n))
    calls.insert(2, ("batch.missing", np.zeros(8, np.float32)))
    wants.insert(2, None)
    got = accel.gemv_batch(calls)
    for g, wv in zip(got, wants):
        if wv is None:
            assert g is None
        else:
            assert rel_l2(g, wv) <= REL_L2_TOL


def test_sharded_accelerators_cover_all_rows(pkg, orc, synth):
    # rank r of `world` adopts a contiguous row shard; shards concatenate to the full result
    in_dim, out_dim, world = 512, 101, 4
    w = synth.q6_k(50, "sh", out_dim, in_dim)
    x = synth.normal(50, "sh.x", in_dim)
    want = orc.qmatmul(x, w, synth.Q6_K, in_dim, out_dim)
    parts = []
    for r in range(world):
        a = pkg.CudaWeightAccel(0, rank=r, world=world)
        try:
            assert a.upload_q6_k("sh", w, in_dim, out_dim)
            info = a.weight_info("sh")
            assert info["row0"] == pkg.shard_begin(out_dim, world, r) and info["out_dim"] == out_dim
            parts.append(a.gemv("sh", x))
        finally:
            a.close()
    got = np.concatenate(parts)
    assert got.size == out_dim and rel_l2(got, want) <= REL_L2_TOL


def test_peer_store_form_fills_full_vectors_on_every_peer(pkg, orc, synth):
    """The multi-GPU epilogue on one GPU: the "peers" are two full-length buffers of this device. Each rank
    handle (run one after the other: nothing here waits on another rank) stores its row shard at its row
    offset into both; after all ranks both buffers hold the whole product. The residual is the shard's rows."""
    import torch
    dev = torch.device("cuda:0")
    in_dim, out_dim, world = 512, 208, 2
    w = synth.q4_0(51, "peer", out_dim, in_dim)
    x = synth.normal(51, "peer.x", in_dim)
    res = synth.normal(51, "peer.res", out_dim)
    want = orc.qmatmul(x, w, synth.Q4_0, in_dim, out_dim) + res
    d_x, d_res = torch.from_numpy(x).to(dev), torch.from_numpy(res).to(dev)
    full = [torch.full((out_dim,), float("nan"), device=dev) for _ in range(2)]
    s = torch.cuda.current_stream().cuda_stream
    for r in range(world):
        a = pkg.CudaWeightAccel(0, rank=r, world=world)
        try:
            assert a.upload_q4_0("peer", w, in_dim, out_dim)
            row0 = a.weight_info("peer")["row0"]
            assert a.gemv_peers_dev(["peer"], d_x.data_ptr(), [[f.data_ptr() for f in full]], stream=s,
                                    d_res=[d_res.data_ptr() + 4 * row0])
            torch.cuda.synchronize()
            assert a.device_status(s) == 0
        finally:
            a.close()
    for f in full:
        assert rel_l2(f.cpu().numpy(), want) <= REL_L2_TOL


def test_peer_barrier_wait_runs_out_without_the_other_rank(pkg, orc, synth):
    """Failure detection without a fault: rank 0 of a group of two runs the cross-GPU barrier alone, so the flag
    word of rank 1 is never raised. The wait is bounded (here 10^4 polls): the kernel returns, the status word
    shows the time-out, and after it is cleared the handle computes as before."""
    import torch
    dev = torch.device("cuda:0")
    a = pkg.CudaWeightAccel(0, rank=0, world=2)
    try:
        assert a.set_option("poll_limit", 10000)
        epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        flags0, flags1 = torch.zeros(8, dtype=torch.int32, device=dev), torch.zeros(8, dtype=torch.int32, device=dev)
        s = torch.cuda.current_stream().cuda_stream
        a.peer_barrier_dev(epoch.data_ptr(), flags0.data_ptr(), [flags0.data_ptr(), flags1.data_ptr()], stream=s)
        torch.cuda.synchronize()
        assert a.device_status(s) == 1                     # STATUS_WAIT_TIMEOUT
        assert int(flags0[0].item()) == 1 and int(flags1[0].item()) == 1 and int(flags0[1].item()) == 0
        assert a.clear_device_status(s) and a.device_status(s) == 0
        in_dim, out_dim = 512, 64
        w = synth.q8_0(53, "after", out_dim, in_dim)
        x = synth.normal(53, "after.x", in_dim)
        assert a.upload_q8_0("after", w, in_dim, out_dim)
        got = a.gemv("after", x)
        assert rel_l2(got, orc.qmatmul(x, w, synth.Q8_0, in_dim, out_dim)[:len(got)]) <= REL_L2_TOL
        assert a.device_status(s) == 0
    finally:
        a.close()


def test_peer_barrier_single_rank(pkg):
    """world = 1: the barrier bumps its epoch and finds its own flag; no other rank is involved."""
    import torch
    dev = torch.device("cuda:0")
    a = pkg.CudaWeightAccel(0)
    try:
        epoch = torch.zeros(1, dtype=torch.int32, device=dev)
        flags = torch.zeros(8, dtype=torch.int32, device=dev)
        s = torch.cuda.current_stream().cuda_stream
        for _ in range(3):
            a.peer_barrier_dev(epoch.data_ptr(), flags.data_ptr(), [flags.data_ptr()], stream=s)
        torch.cuda.synchronize()
        assert int(epoch.item()) == 3 and int(flags[0].item()) == 3 and a.device_status(s) == 0
    finally:
        a.close()


# ------------------------------------------------------------------ device-resident form + fused prologues
def test_gemv_dev_prologues_and_fused_weights(accel, orc, synth, pkg):
    import torch
    dev = torch.device("cuda:0")
    hidden, ffn = 2560, 9728
    wq = synth.q4_0(60, "q", 4096, hidden)
    wk = synth.q4_0(60, "k", 1024, hidden)
    wv = synth.q4_0(60, "v", 1024, hidden)
    wd = synth.q4_0(60, "down", hidden, ffn)
    for k_, w_, n_, i_ in (("f.q", wq, 4096, hidden), ("f.k", wk, 1024, hidden), ("f.v", wv, 1024, hidden),
                           ("f.down", wd, hidden, ffn)):
        assert accel.upload_q4_0(k_, w_, i_, n_)
    h = synth.normal(60, "h", hidden)
    nw = synth.norm_weight(60, "nw", hidden)
    gate = synth.normal(60, "gate", ffn)
    up = synth.normal(60, "up", ffn)
    s = torch.cuda.current_stream().cuda_stream
    d_h, d_nw = torch.from_numpy(h).to(dev), torch.from_numpy(nw).to(dev)
    d_g, d_u = torch.from_numpy(gate).to(dev), torch.from_numpy(up).to(dev)
    yq, yk, yv = (torch.full((n,), float("nan"), device=dev) for n in (4096, 1024, 1024))
    yd = torch.full((hidden,), float("nan"), device=dev)
    yg = torch.full((hidden,), float("nan"), device=dev)
    n_cpu = orc.rmsnorm(h, nw, 1e-6)
    for act in (pkg.ACT_F32, pkg.ACT_Q8DOT):
        # rmsnorm prologue + q|k|v in one launch
        assert accel.gemv_dev(["f.q", "f.k", "f.v"], d_h.data_ptr(), [yq.data_ptr(), yk.data_ptr(), yv.data_ptr()],
                              d_b=d_nw.data_ptr(), eps=1e-6, pre=pkg.PRE_RMSNORM, act=act, stream=s)
        # swiglu / geglu prologue + down
        assert accel.gemv_dev(["f.down"], d_g.data_ptr(), [yd.data_ptr()], d_b=d_u.data_ptr(), pre=pkg.PRE_SWIGLU,
                              act=act, stream=s)
        assert accel.gemv_dev(["f.down"], d_g.data_ptr(), [yg.data_ptr()], d_b=d_u.data_ptr(), pre=pkg.PRE_GEGLU,
                              act=act, stream=s)
        assert accel.device_status(s) == 0
        tol = REL_L2_TOL if act == pkg.ACT_F32 else 2e-2   # vs the f32 oracle; int path adds quantisation error
        for y, w_, n_ in ((yq, wq, 4096), (yk, wk, 1024), (yv, wv, 1024)):
            assert rel_l2(y.cpu().numpy(), orc.qmatmul(n_cpu, w_, synth.Q4_0, hidden, n_)) <= tol
        assert rel_l2(yd.cpu().numpy(), orc.qmatmul(orc.swiglu(gate, up), wd, synth.Q4_0, ffn, hidden)) <= tol
        assert rel_l2(yg.cpu().numpy(), orc.qmatmul(orc.geglu(gate, up), wd, synth.Q4_0, ffn, hidden)) <= tol
        # fused residual: h + W_down swiglu(gate, up), accumulated in place (the o / down projections of the chain)
        acc_h = d_h.clone()
        assert accel.gemv_dev(["f.down"], d_g.data_ptr(), [acc_h.data_ptr()], d_b=d_u.data_ptr(), pre=pkg.PRE_SWIGLU,
                              act=act, stream=s, d_res=[acc_h.data_ptr()])
        want = h + orc.qmatmul(orc.swiglu(gate, up), wd, synth.Q4_0, ffn, hidden)
        assert rel_l2(acc_h.cpu().numpy(), want) <= tol


# ------------------------------------------------------------------ batched rows (speculative verify)
@pytest.mark.parametrize("ty,out_dim,in_dim", [(2, 257, 3840), (2, 100, 15360), (8, 64, 2560), (14, 33, 3840), (2, 9, 64),
                                               (3, 257, 3840), (3, 40, 15360)])
@pytest.mark.parametrize("b", [1, 2, 4, 8])
def test_gemv_rows_matches_oracle(accel, orc, synth, pkg, ty, out_dim, in_dim, b):
    w = synth.quant(ty, 33, "rows", out_dim, in_dim)
    xs = synth.normal(33, "rows.x", b, in_dim)
    key = "rows.%d.%d.%d" % (ty, out_dim, in_dim)
    assert uploader(accel, synth, ty)(key, w, in_dim, out_dim)
    want = orc.qmatmul_batch(xs, b, w, ty, in_dim, out_dim)
    got = accel.gemv_rows(key, xs, b)
    assert got.shape == (b, out_dim)
    assert rel_l2(got, want) <= REL_L2_TOL
    for t in range(b):      # each activation row on its own, so that a swapped row cannot hide
        assert rel_l2(got[t], want[t]) <= REL_L2_TOL
    xq, xd, _ = orc.xquant8(xs)
    want_i = orc.idot_gemm(w, ty, xq, xd, b, in_dim, out_dim)
    got_i = accel.gemv_rows(key, xs, b, act=pkg.ACT_Q8DOT)
    for t in range(b):
        assert rel_l2(got_i[t], want_i[t]) <= REL_L2_TOL
    assert accel.device_status() == 0


@pytest.mark.parametrize("out_dim,in_dim", [(15360, 3840), (3840, 15360)])
def test_gemv_rows_at_the_verify_configuration(accel, orc, synth, pkg, out_dim, in_dim):
    """The speculative-verify configuration's own FFN shapes (3840 -> 15360 and 15360 -> 3840, Q4_0), every
    batch width, both activation forms, each activation row checked on its own."""
    w = synth.q4_0(34, "vr", out_dim, in_dim)
    key = "vr.%d.%d" % (out_dim, in_dim)
    assert accel.upload_q4_0(key, w, in_dim, out_dim)
    xs8 = synth.normal(34, "vr.x", 8, in_dim)
    want8 = orc.qmatmul_batch(xs8, 8, w, synth.Q4_0, in_dim, out_dim)
    xq, xd, _ = orc.xquant8(xs8)
    want8_i = orc.idot_gemm(w, synth.Q4_0, xq, xd, 8, in_dim, out_dim)
    for b in (1, 2, 4, 8):
        got = accel.gemv_rows(key, xs8[:b], b)
        got_i = accel.gemv_rows(key, xs8[:b], b, act=pkg.ACT_Q8DOT)
        for t in range(b):
            assert rel_l2(got[t], want8[t]) <= REL_L2_TOL, (b, t)
            assert rel_l2(got_i[t], want8_i[t]) <= REL_L2_TOL, (b, t)
    assert accel.device_status() == 0
    accel.upload_q4_0(key, synth.q4_0(1, "tiny", 1, 32), 32, 1)


@pytest.mark.parametrize("pre", ["rmsnorm", "swiglu", "geglu"])
def test_fused_prologue_integer_form_at_the_contract(accel, orc, synth, pkg, pre):
    """RMSNorm / SwiGLU / GeGLU -> per-32 int8 -> GEMV in ONE launch against the INTEGER oracle on the CPU's
    own codes (rmsnorm_xquant / silu_xquant / geglu_xquant, kernels.rs:101-226), at the 1e-3 contract.
    The launch-per-step kernel quantises x * w and applies 1/rms to the outputs (the product is linear in
    it), so where (x / rms) * w sits within an f32 rounding of a .5 boundary its code can differ from the
    CPU's by one; the count of such codes is computed here on the host, from the two operand orders, and
    printed next to the error."""
    import torch
    dev = torch.device("cuda:0")
    hidden, ffn = 2560, 9728
    s = torch.cuda.current_stream().cuda_stream
    if pre == "rmsnorm":
        K, N = hidden, 4096
        a, b_ = synth.normal(61, "h", K), synth.norm_weight(61, "nw", K)
        x_cpu = orc.rmsnorm(a, b_, 1e-6)
        code, eps = pkg.PRE_RMSNORM, 1e-6
        # the kernel's operand order on the host: codes of x * w (scale-free) against codes of (x / rms) * w
        xw = (a * b_).astype(np.float32)
        flips = int((orc.xquant8(xw)[0] != orc.xquant8(x_cpu)[0]).sum())
    else:
        K, N = ffn, hidden
        a, b_ = synth.normal(61, "gate", K), synth.normal(61, "up", K)
        x_cpu = orc.swiglu(a, b_) if pre == "swiglu" else orc.geglu(a, b_)
        code, eps, flips = (pkg.PRE_SWIGLU if pre == "swiglu" else pkg.PRE_GEGLU), 0.0, None
    w = synth.q4_0(61, "fp." + pre, N, K)
    key = "fp." + pre
    assert accel.upload_q4_0(key, w, K, N)
    d_a, d_b = torch.from_numpy(a).to(dev), torch.from_numpy(b_).to(dev)
    y = torch.full((N,), float("nan"), device=dev)
    assert accel.gemv_dev([key], d_a.data_ptr(), [y.data_ptr()], d_b=d_b.data_ptr(), eps=eps, pre=code,
                          act=pkg.ACT_Q8DOT, stream=s)
    assert accel.device_status(s) == 0
    xq, xd, _ = orc.xquant8(x_cpu)
    want = orc.idot_gemm(w, synth.Q4_0, xq, xd, 1, K, N)[0]
    got = y.cpu().numpy()
    r = rel_l2(got, want)
    print("fused %s + int8 + GEMV vs integer oracle: rel-L2 %.2e max-abs %.2e; codes moved by the operand order: %s of %d"
          % (pre, r, np.abs(got - want).max(), flips, K))
    assert r <= REL_L2_TOL


@pytest.mark.parametrize("act_name", ["f32", "q8dot"])
def test_gemv_batch_small_items_side_by_side(pkg, orc, synth, act_name):
    """gemv_batch_dev / gemv_batch: independent items; the small ones run side by side in one launch (its CTAs dealt
    out among them), the large ones as a launch each. Every result against the oracle at the contract and against
    the item's own launch; with the option off; under stream capture; with an unknown key; after a weight of the
    batch was replaced by one of another format (the cached graph must go)."""
    import torch
    act = pkg.ACT_F32 if act_name == "f32" else pkg.ACT_Q8DOT
    shapes = [(synth.Q8_0, 2560, 1200), (synth.Q6_K, 2560, 1000), (synth.Q4_0, 4096, 777), (synth.Q8_0, 9728, 640),
              (synth.Q6_K, 9728, 48), (synth.Q4_1, 1024, 331)]
    up_of = lambda acc: {synth.Q8_0: acc.upload_q8_0, synth.Q6_K: acc.upload_q6_k, synth.Q4_0: acc.upload_q4_0,
                         synth.Q4_1: acc.upload_q4_1}
    acc = pkg.CudaWeightAccel(0)
    try:
        dev = torch.device("cuda", 0)
        assert acc.set_option("batch_small_bytes", 8 << 20)       # items 0..2, 4, 5 are small, item 3 is not
        keys, hx, xs, ys, want, ws = [], [], [], [], [], []

        def oracle_of(i):
            ty, k, n = shapes[i]
            if act == pkg.ACT_F32:
                return orc.qmatmul(hx[i], ws[i], ty, k, n)
            xq, xd, _ = orc.xquant8(hx[i])
            return orc.idot_gemm(ws[i], ty, xq, xd, 1, k, n)[0]

        for i, (ty, k, n) in enumerate(shapes):
            key = "bd.%d" % i
            w = synth.quant(ty, 601, key, n, k)
            assert up_of(acc)[ty](key, w, k, n)
            x = synth.normal(602, key, k)
            keys.append(key); hx.append(x); ws.append(w)
            xs.append(torch.from_numpy(x).to(dev))
            ys.append(torch.zeros(n, device=dev))
            one = torch.zeros(n, device=dev)
            assert acc.gemv_dev([key], xs[-1].data_ptr(), [one.data_ptr()], act=act)
            torch.cuda.synchronize()
            want.append(one.cpu().numpy())
            assert rel_l2(want[-1], oracle_of(i)) <= REL_L2_TOL

        def check(got_list, tag):
            for i, g in enumerate(got_list):
                r1, r2 = rel_l2(g, oracle_of(i)), rel_l2(g, want[i])
                assert r1 <= REL_L2_TOL and r2 <= 1e-5, (tag, i, r1, r2)

        for mode, overlap in ((1, 1), (1, 0), (2, 1), (0, 1), (0, 0)):
            assert acc.set_option("batch_side_by_side", mode)
            assert acc.set_option("batch_overlap", overlap)   # later launches of the batch wait for nothing / as usual
            for y in ys:
                y.zero_()
            assert acc.gemv_batch_dev(keys, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys], act=act)
            torch.cuda.synchronize()
            check([y.cpu().numpy() for y in ys], "dev mode %d overlap %d" % (mode, overlap))
            got = acc.gemv_batch(list(zip(keys, hx)), act=act)
            check(got, "host mode %d" % mode)
            got = acc.gemv_batch(list(zip(keys, hx)), act=act)   # the cached graph
            check(got, "host mode %d again" % mode)
        assert acc.set_option("batch_side_by_side", 1)
        assert acc.set_option("batch_overlap", 1)
        st = torch.cuda.Stream(device=dev)
        with torch.cuda.stream(st):
            assert acc.gemv_batch_dev(keys, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys], act=act, stream=st.cuda_stream)
            torch.cuda.synchronize()
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=st):
                assert acc.gemv_batch_dev(keys, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys], act=act,
                                          stream=torch.cuda.current_stream().cuda_stream)
            for y in ys:
                y.zero_()
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
        check([y.cpu().numpy() for y in ys], "captured")
        assert acc.gemv_batch_dev(keys + ["nope"], [x.data_ptr() for x in xs] + [xs[0].data_ptr()],
                                  [y.data_ptr() for y in ys] + [ys[0].data_ptr()], act=act) is False
        got = acc.gemv_batch(list(zip(keys, hx)) + [("nope", hx[0])], act=act)
        assert got[-1] is None
        check(got[:-1], "host with an unknown key")
        # replace item 0 (Q8_0 2560 -> 1200) by a Q4_0 weight of the same shape: same key, possibly the same address
        ty, k, n = synth.Q4_0, 2560, 1200
        shapes[0] = (ty, k, n)
        ws[0] = synth.quant(ty, 603, keys[0], n, k)
        assert acc.upload_q4_0(keys[0], ws[0], k, n)
        one = torch.zeros(n, device=dev)
        assert acc.gemv_dev([keys[0]], xs[0].data_ptr(), [one.data_ptr()], act=act)
        torch.cuda.synchronize()
        want[0] = one.cpu().numpy()
        check(acc.gemv_batch(list(zip(keys, hx)), act=act), "host after the re-upload")
        assert acc.gemv_batch_dev(keys, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys], act=act)
        torch.cuda.synchronize()
        check([y.cpu().numpy() for y in ys], "dev after the re-upload")
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_profile_option_times_every_launch(pkg, synth):
    """opts.profile / set_option("profile", 1): the reference's STRIX_PROF (decode.rs:25-69). Every launch made
    outside a capture is bracketed by events; profile_dump names the kernels with their launch counts and
    resets; with the option off nothing is recorded."""
    acc = pkg.CudaWeightAccel(0)
    try:
        k, n = 1024, 640
        assert acc.upload_q8_0("p.a", synth.quant(synth.Q8_0, 611, "p.a", n, k), k, n)
        assert acc.upload_q6_k("p.b", synth.quant(synth.Q6_K, 611, "p.b", n, k), k, n)
        x = synth.normal(612, "p.x", k)
        assert "total kernel time 0.000" in acc.profile_dump()
        acc.gemv("p.a", x)                                   # option off: not recorded
        assert "gemv" not in acc.profile_dump()
        assert acc.set_option("profile", 1)
        for _ in range(3):
            acc.gemv("p.a", x)
        acc.gemv("p.b", x, act=pkg.ACT_Q8DOT)
        acc.gemv_batch([("p.a", x), ("p.b", x)])             # two small items: one side-by-side launch
        txt = acc.profile_dump()
        print(txt)
        lines = {ln.split()[0]: ln for ln in txt.splitlines()[1:]}
        assert "gemv.q8_0.f32_digits" in lines and " 3 calls" in lines["gemv.q8_0.f32_digits"]
        assert "gemv.q6_k.q8dot" in lines and " 1 calls" in lines["gemv.q6_k.q8dot"]
        assert "gemv_multi" in lines and " 1 calls" in lines["gemv_multi"]
        assert "total kernel time 0.000" in acc.profile_dump()   # reset by the dump
        assert acc.set_option("profile", 0)
        acc.gemv("p.a", x)
        assert "gemv" not in acc.profile_dump()
    finally:
        acc.close()


def test_gemv_batch_overlap_keeps_stream_order(pkg, synth):
    """The launches of a batch do not wait for one another, but the batch as a whole keeps its place in the stream:
    activations written by kernels enqueued just before the call (behind a long-running one) are the ones every item
    reads, and a reader enqueued just after the call sees every item's output. Two sets of activations alternate;
    the results must equal, bit for bit, those of the same batch run with every launch waiting."""
    import torch
    dev = torch.device("cuda", 0)
    shapes = [(synth.Q8_0, 2560, 9000), (synth.Q6_K, 2560, 7000), (synth.Q8_0, 1024, 640), (synth.Q4_0, 4096, 777),
              (synth.Q6_K, 2560, 331)]
    acc = pkg.CudaWeightAccel(0)
    try:
        assert acc.set_option("batch_small_bytes", 4 << 20)   # items 0 and 1: a launch each; 2..4 side by side
        keys = []
        for i, (ty, k, n) in enumerate(shapes):
            keys.append("so.%d" % i)
            up = {synth.Q8_0: acc.upload_q8_0, synth.Q6_K: acc.upload_q6_k, synth.Q4_0: acc.upload_q4_0}[ty]
            assert up(keys[-1], synth.quant(ty, 631, keys[-1], n, k), k, n)
        sets = [[torch.from_numpy(synth.normal(632 + v, keys[i], k)).to(dev) for i, (_, k, _) in enumerate(shapes)]
                for v in range(2)]
        xs = [torch.zeros(k, device=dev) for (_, k, _) in shapes]
        ys = [torch.zeros(n, device=dev) for (_, _, n) in shapes]
        s = torch.cuda.current_stream().cuda_stream
        ballast = torch.ones(32 << 20, device=dev)

        def run(v):
            ballast.mul_(1.0000001)                       # ~0.1 ms of work the copies queue behind
            for x, src in zip(xs, sets[v]):
                x.copy_(src)
            assert acc.gemv_batch_dev(keys, [x.data_ptr() for x in xs], [y.data_ptr() for y in ys], stream=s)
            return [y.clone() for y in ys]                # readers enqueued right behind the batch

        assert acc.set_option("batch_overlap", 0)
        want = [run(v) for v in range(2)]
        torch.cuda.synchronize()
        assert not any(torch.equal(a, b) for a, b in zip(want[0], want[1]))
        assert acc.set_option("batch_overlap", 1)
        for it in range(6):
            got = run(it & 1)
            torch.cuda.synchronize()
            for i, (g, w) in enumerate(zip(got, want[it & 1])):
                assert torch.equal(g, w), (it, i)
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_close_leaves_no_cuda_error_behind(pkg, synth):
    """A handle that is created, used and closed leaves no pending CUDA error for the next user of the runtime in
    the process (a runtime call that fails, a second free of one pointer for one, stays 'the last error' until someone
    asks for it, and the next library that checks after its own launch reports it as its own)."""
    import ctypes
    import torch
    rt = ctypes.CDLL("libcudart.so.12")
    rt.cudaPeekAtLastError.restype = ctypes.c_int
    torch.zeros(4, device="cuda:0")
    torch.cuda.synchronize()
    assert rt.cudaPeekAtLastError() == 0
    acc = pkg.CudaWeightAccel(0)
    k, n = 1024, 64
    assert acc.upload_q8_0("c.a", synth.quant(synth.Q8_0, 641, "c.a", n, k), k, n)
    x = synth.normal(642, "c.x", k)
    assert acc.gemv("c.a", x) is not None
    assert acc.gemv("c.a", x, act=pkg.ACT_Q8DOT) is not None
    acc.close()
    assert rt.cudaPeekAtLastError() == 0
    torch.full((4,), 1.0, device="cuda:0")
    torch.cuda.synchronize()


def test_gemv_batch_peers_dev_fills_every_ranks_full_vectors(pkg, orc, synth):
    """The row-sharded form of gemv_batch_dev: each of three row shards (three handles on one GPU, run one after
    the other: no kernel waits for another) stores its rows of every item into the full output vectors of both
    'accelerators' (two local buffers per item). One item runs as a launch of its own, the others side by side.
    Every element of every vector against the oracle."""
    import torch
    dev = torch.device("cuda:0")
    world = 3
    shapes = [(synth.Q8_0, 2560, 1203), (synth.Q6_K, 2560, 997), (synth.Q4_0, 4096, 777), (synth.Q8_0, 1024, 50)]
    ws = [synth.quant(ty, 621, "bp.%d" % i, n, k) for i, (ty, k, n) in enumerate(shapes)]
    xs = [synth.normal(622, "bp.x.%d" % i, k) for i, (ty, k, n) in enumerate(shapes)]
    want = [orc.qmatmul(xs[i], ws[i], ty, k, n) for i, (ty, k, n) in enumerate(shapes)]
    d_xs = [torch.from_numpy(x).to(dev) for x in xs]
    full = [[torch.full((n,), float("nan"), device=dev) for _ in range(2)] for (_, _, n) in shapes]
    s = torch.cuda.current_stream().cuda_stream
    keys = ["bp.%d" % i for i in range(len(shapes))]
    for r in range(world):
        a = pkg.CudaWeightAccel(0, rank=r, world=world)
        try:
            assert a.set_option("batch_small_bytes", 600 << 10)   # item 0's shard is above it: a launch of its own
            for i, (ty, k, n) in enumerate(shapes):
                up = {synth.Q8_0: a.upload_q8_0, synth.Q6_K: a.upload_q6_k, synth.Q4_0: a.upload_q4_0}[ty]
                assert up(keys[i], ws[i], k, n)
            assert a.gemv_batch_peers_dev(keys, [x.data_ptr() for x in d_xs], [[f.data_ptr() for f in fs] for fs in full],
                                          stream=s)
            torch.cuda.synchronize()
            assert a.device_status(s) == 0
            assert a.gemv_batch_peers_dev(keys + ["nope"], [x.data_ptr() for x in d_xs] + [d_xs[0].data_ptr()],
                                          [[f.data_ptr() for f in fs] for fs in full] + [[full[0][0].data_ptr()] * 2],
                                          stream=s) is False
        finally:
            a.close()
    for i, fs in enumerate(full):
        for f in fs:
            got = f.cpu().numpy()
            assert np.isfinite(got).all()
            assert rel_l2(got, want[i]) <= REL_L2_TOL, i
