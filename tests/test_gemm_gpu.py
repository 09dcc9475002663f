"""GPU parity of the W8A8 prefill GEMM against the integer oracle, through the C ABI.
Tier 1 (bit-exact): int32 block sums. Tier 2: scaled f32 output within rel-L2 1e-3."""
import numpy as np
import pytest

pytestmark = pytest.mark.gpu
REL_L2_TOL = 1e-3


def rel_l2(got, want):
    return float(np.linalg.norm(got.astype(np.float64) - want) / max(np.linalg.norm(want), 1e-30))


def oracle_gemm(orc, synth, w, xs, m, k, n, want_isums=False):
    xq, xd, _ = orc.xquant8(xs)
    return orc.idot_gemm(w, synth.Q8_0, xq, xd, m, k, n, want_isums=want_isums)


@pytest.mark.parametrize("m,n,k", [(1, 8, 32), (3, 37, 256), (17, 100, 96), (33, 129, 2560)])
def test_block_isums_bit_exact(accel, orc, synth, m, n, k):
    w = synth.q8_0(70, "gi", n, k)
    xs = synth.normal(70, "gi.x", m, k)
    assert accel.upload_q8_0("gi.%d.%d" % (n, k), w, k, n)
    got = accel.debug_block_isums("gi.%d.%d" % (n, k), xs, m)
    _, want = oracle_gemm(orc, synth, w, xs, m, k, n, want_isums=True)
    np.testing.assert_array_equal(got, want)


@pytest.mark.parametrize("m,n,k", [
    (1, 8, 32), (1, 128, 128), (5, 64, 96), (17, 100, 160), (128, 128, 512), (130, 257, 2560),
    (200, 2560, 4096),          # split-K territory: few output tiles, long K
    (512, 4096, 2560),          # q_proj shape of the benchmark
])
def test_gemm_matches_integer_oracle(accel, orc, synth, m, n, k):
    w = synth.q8_0(71, "gm", n, k)
    xs = synth.normal(71, "gm.x", m, k)
    key = "gm.%d.%d" % (n, k)
    assert accel.upload_q8_0(key, w, k, n)
    got = accel.prefill_q8_gemm(key, xs, m)
    assert got is not None and got.shape == (m, n) and np.isfinite(got).all()
    want = oracle_gemm(orc, synth, w, xs, m, k, n)
    r = rel_l2(got, want)
    print("gemm m=%d n=%d k=%d rel-L2 %.2e max-abs %.2e" % (m, n, k, r, np.abs(got - want).max()))
    assert r <= REL_L2_TOL
    # per-element bound too, so that a wrong tile cannot hide inside the norm
    assert np.abs(got - want).max() <= 1e-3 * np.abs(want).max()
    # and close to the f32-activation path (quantisation error only; the reference's dp4a bound)
    wf = orc.qmatmul_batch(xs, m, w, synth.Q8_0, k, n)
    if k >= 512:
        assert rel_l2(got, wf) <= 2e-2
    assert accel.device_status() == 0


def test_gemm_benchmark_shapes_on_sampled_tokens(accel, orc, synth):
    # full benchmark sizes: M = 2048 tokens; the oracle checks a sample of the token rows, which
    # is exact because every output row depends on its own token only
    for n, k in ((9728, 2560), (2560, 9728)):
        m = 2048
        w = synth.q8_0(72, "gb", n, k)
        xs = synth.normal(72, "gb.x", m, k)
        key = "gb.%d.%d" % (n, k)
        assert accel.upload_q8_0(key, w, k, n)
        got = accel.prefill_q8_gemm(key, xs, m)
        rows = np.array([0, 1, 127, 128, 777, 1024, 2046, 2047])
        want = oracle_gemm(orc, synth, w, xs[rows], len(rows), k, n)
        assert rel_l2(got[rows], want) <= REL_L2_TOL
        # rows outside the sample: same statistics, finite, non-zero
        assert np.isfinite(got).all() and (np.abs(got).max(axis=1) > 0).all()
        accel.upload_q8_0(key, synth.q8_0(1, "tiny", 1, 32), 32, 1)


def test_gemm_declines_like_the_reference(accel, synth):
    assert accel.upload_q4_0("gd.q4", synth.q4_0(1, "gd", 8, 64), 64, 8)
    assert accel.prefill_q8_gemm("gd.q4", np.zeros((2, 64), np.float32), 2) is None      # only the q8 map is searched
    assert accel.prefill_q8_gemm("gd.none", np.zeros((2, 64), np.float32), 2) is None
    assert accel.upload_q8_0("gd.q8", synth.q8_0(1, "gd8", 8, 64), 64, 8)
    assert accel.prefill_q8_gemm("gd.q8", np.zeros(100, np.float32), 2) is None           # xs.len() != m * in_dim
