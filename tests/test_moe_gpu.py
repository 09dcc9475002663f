"""GPU parity of the mixture-of-experts FFN family (accel.rs:167-246) against the CPU oracle (mellum.rs:1582-1663)."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def make_layer(synth, ty, seed, hidden, eff, ne):
    return (synth.quant(ty, seed, "moe.gate", ne * eff, hidden), synth.quant(ty, seed, "moe.up", ne * eff, hidden),
            synth.quant(ty, seed, "moe.down", ne * hidden, eff))


@pytest.mark.parametrize("fmt,hidden,eff,ne,k", [("q8_0", 2048, 896, 64, 8),     # the Mellum layer (mellum.rs:1585-1588)
                                                 ("q8_0", 256, 96, 5, 3),        # eff not a multiple of 64, odd counts
                                                 ("q6_k", 1024, 512, 12, 6),     # native Q6_K experts, two down chunks
                                                 ("q8_0", 512, 128, 40, 16)])    # the largest k
@pytest.mark.parametrize("int8", [False, True])
def test_moe_ffn_matches_oracle(pkg, orc, synth, fmt, hidden, eff, ne, k, int8):
    ty = synth.Q8_0 if fmt == "q8_0" else synth.Q6_K
    acc = pkg.CudaWeightAccel(0)
    try:
        gate, up, down = make_layer(synth, ty, 401, hidden, eff, ne)
        upload = acc.upload_moe_q8 if fmt == "q8_0" else acc.upload_moe_q6
        assert acc.moe_ffn(3, [0], [1.0], np.zeros(hidden, np.float32)) is None          # not adopted yet
        assert upload(3, gate, up, down, hidden, eff, ne)
        rng = np.random.default_rng(402)
        act = pkg.ACT_Q8DOT if int8 else pkg.ACT_F32
        for trial in range(3):
            x = synth.normal(403, "x.%d" % trial, hidden)
            logits = rng.standard_normal(ne).astype(np.float32) * 2
            ids, w = orc.topk_router(logits, k)
            got = acc.moe_ffn(3, ids, w, x, act=act)
            want = orc.moe_ffn(x, gate, up, down, ty, hidden, eff, ids, w, int8=int8)
            r = rel_l2(got, want)
            # integer form: the activation of the down projection is re-quantised from GPU-computed gate / up values,
            # a code or two can fall on the other side of a rounding boundary (as along the dense chain)
            assert r <= (2e-2 if int8 else REL_L2_TOL), (trial, r)
        print("moe_ffn %s k=%d int8=%s rel-L2 %.2e" % (fmt, k, int8, r))
        # the order of the selections is the order of the sum; a permutation changes only rounding
        perm = np.arange(k)[::-1]
        got_p = acc.moe_ffn(3, ids[perm], w[perm], x, act=act)
        assert rel_l2(got_p, got) <= 1e-5
        # None: wrong length, too many experts, an id out of range, weights / ids of different sizes
        assert acc.moe_ffn(3, ids, w, x[:-32], act=act) is None
        assert acc.moe_ffn(3, list(range(17)), [1.0 / 17] * 17, x) is None
        assert acc.moe_ffn(3, [ne], [1.0], x) is None and acc.moe_ffn(3, [-1], [1.0], x) is None
        assert acc.moe_ffn(3, ids, w[:-1], x) is None
        assert acc.moe_ffn(4, ids, w, x) is None
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_moe_upload_declines_like_the_reference(pkg, synth):
    """decode.rs:2727-2735, 2803-2811: whole blocks, hidden and eff <= 4096, exact lengths."""
    acc = pkg.CudaWeightAccel(0)
    try:
        hidden, eff, ne = 128, 64, 2
        gate, up, down = make_layer(synth, synth.Q8_0, 411, hidden, eff, ne)
        assert acc.upload_moe_q8(0, gate, up, down, hidden, eff, ne + 1) is False          # lengths do not match
        assert acc.upload_moe_q8(0, gate[:-34], up, down, hidden, eff, ne) is False
        assert acc.upload_moe_q8(0, gate, up, down, hidden + 16, eff, ne) is False         # not whole blocks
        assert acc.upload_moe_q6(0, gate, up, down, hidden, eff, ne) is False              # Q6_K wants multiples of 256
        big = np.zeros((8192 // 32) * 34 * 32, np.uint8)
        assert acc.upload_moe_q8(0, big, big, big, 8192, 32, 1) is False                   # hidden > 4096
        assert acc.upload_moe_q8(0, gate, up, down, hidden, eff, ne)
        assert acc.resident_count() == 3
    finally:
        acc.close()


def test_moe_shared_expert(pkg, orc, synth):
    """decode.rs:1820-1856 queue_shexp: out += sgate * down_sh(silu(gate_sh x) * up_sh x) over dense Q8_0 residents."""
    hidden, eff, ne, sff = 512, 128, 6, 256
    acc = pkg.CudaWeightAccel(0)
    try:
        gate, up, down = make_layer(synth, synth.Q8_0, 421, hidden, eff, ne)
        assert acc.upload_moe_q8(1, gate, up, down, hidden, eff, ne)
        x = synth.normal(422, "x", hidden)
        ids, w = np.array([4, 1], np.int32), np.array([0.7, 0.3], np.float32)
        assert acc.moe_ffn(1, ids, w, x, sgate=0.25) is None                               # shared expert not resident
        sh = {}
        for nm, n, kdim in (("ffn_gate_shexp", sff, hidden), ("ffn_up_shexp", sff, hidden), ("ffn_down_shexp", hidden, sff)):
            sh[nm] = synth.quant(synth.Q8_0, 423, nm, n, kdim)
            assert acc.upload_q8_0("blk.1.%s.weight" % nm, sh[nm], kdim, n)
        got = acc.moe_ffn(1, ids, w, x, sgate=0.25)
        g = orc.qmatmul(x, sh["ffn_gate_shexp"], synth.Q8_0, hidden, sff)
        u = orc.qmatmul(x, sh["ffn_up_shexp"], synth.Q8_0, hidden, sff)
        sd = orc.qmatmul(orc.swiglu(g, u), sh["ffn_down_shexp"], synth.Q8_0, sff, hidden)
        want = orc.moe_ffn(x, gate, up, down, synth.Q8_0, hidden, eff, ids, w) + np.float32(0.25) * sd
        assert rel_l2(got, want) <= REL_L2_TOL
    finally:
        acc.close()


@pytest.mark.parametrize("fmt", ["q8_0", "q6_k"])
def test_moe_grouped_tokens(pkg, orc, synth, fmt):
    """moe_expert_ffn / moe_layer_ffn (decode.rs:3299-3356, 3552-3630): tokens grouped by expert, the expert's weights
    read once per chunk of rows; 11 rows cross a chunk of 8, a plan entry of zero rows is skipped."""
    ty = synth.Q8_0 if fmt == "q8_0" else synth.Q6_K
    hidden, eff, ne = 512, 256, 7
    acc = pkg.CudaWeightAccel(0)
    try:
        gate, up, down = make_layer(synth, ty, 431, hidden, eff, ne)
        upload = acc.upload_moe_q8 if fmt == "q8_0" else acc.upload_moe_q6
        assert upload(0, gate, up, down, hidden, eff, ne)
        xs = synth.normal(432, "xs", 14 * hidden).reshape(14, hidden)
        y = acc.moe_expert_ffn(0, 5, xs[:11], 11)
        for t in range(11):
            assert rel_l2(y[t], orc.moe_expert_ffn(xs[t], gate, up, down, ty, hidden, eff, 5)) <= REL_L2_TOL, t
        plan = [(2, 3), (6, 0), (0, 9), (4, 2)]
        yl = acc.moe_layer_ffn(0, plan, xs, 14)
        row = 0
        for e, cnt in plan:
            for _ in range(cnt):
                assert rel_l2(yl[row], orc.moe_expert_ffn(xs[row], gate, up, down, ty, hidden, eff, e)) <= REL_L2_TOL, row
                row += 1
        assert acc.moe_layer_ffn(0, [(2, 3)], xs, 14) is None                              # counts do not add up
        assert acc.moe_layer_ffn(0, [(7, 14)], xs, 14) is None                             # expert out of range
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_topk_router_matches_oracle(pkg, orc):
    acc = pkg.CudaWeightAccel(0)
    try:
        rng = np.random.default_rng(441)
        for ne, k in ((64, 8), (128, 16), (5, 5), (33, 1)):
            for _ in range(5):
                logits = (rng.standard_normal(ne) * 3).astype(np.float32)
                ids, w = acc.topk_router(logits, k)
                wi, ww = orc.topk_router(logits, k)
                np.testing.assert_array_equal(ids, wi)
                np.testing.assert_allclose(w, ww, rtol=2e-6)
        logits = np.array([1.0, 3.0, 3.0, 0.0, 3.0], np.float32)                           # ties: the lower index first
        ids, w = acc.topk_router(logits, 3)
        assert list(ids) == [1, 2, 4]
        assert acc.topk_router(np.zeros(129, np.float32), 4) is None and acc.topk_router(np.zeros(4, np.float32), 5) is None
    finally:
        acc.close()
