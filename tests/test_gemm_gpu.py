"""GPU parity of the W8A8 prefill GEMM against the integer oracle, through the C ABI.
Tier 1 (bit-exact): int32 block sums, as the tcgen05 kernel itself produces them and from a plain
integer loop. Tier 2: scaled f32 output within rel-L2 1e-3."""
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


@pytest.mark.parametrize("m,n,k,splits", [
    (1, 8, 32, 0),               # one block, one row group
    (3, 37, 256, 0),             # ragged tile, two stages of four K-blocks
    (130, 257, 2560, 0),         # crosses token tiles (128), row tiles (128) and 20 stages: TMEM buffers re-armed 20 times
    (200, 2560, 4096, 0),        # the split-K shape (few output tiles, long K): slices as the product path picks them
    (200, 384, 4096, 3),         # forced uneven slices (32 stages over 3: 11 + 11 + 10)
    (129, 130, 160, 2),          # a last stage with one K-block, split in two
])
def test_gemm_kernel_block_isums_bit_exact(accel, orc, synth, m, n, k, splits):
    """north_star: "int32 GEMM accumulators must be bit-exact". The integers come out of the GEMM's own
    tcgen05 kernel (same TMA producer, same MMA issue and descriptor stepping, same TMEM buffers and
    re-arming; only the epilogue stores the block sum instead of folding it), q8w_gemm32's per-block
    accumulator (kernels.rs:1417-1428)."""
    w = synth.q8_0(73, "gk", n, k)
    xs = synth.normal(73, "gk.x", m, k)
    key = "gk.%d.%d" % (n, k)
    assert accel.upload_q8_0(key, w, k, n)
    got = accel.debug_gemm_isums(key, xs, m, splits)
    _, want = oracle_gemm(orc, synth, w, xs, m, k, n, want_isums=True)
    assert got.shape == want.shape
    np.testing.assert_array_equal(got, want)
    assert accel.device_status() == 0
    accel.upload_q8_0(key, synth.q8_0(1, "tiny", 1, 32), 32, 1)       # release the memory


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


@pytest.mark.parametrize("m,n,k", [
    (2048, 9728, 2560), (2048, 4096, 2560), (2048, 2560, 9728),      # gate/up, q_proj, ffn_down (split-K)
    (512, 9728, 2560), (512, 2560, 9728),
])
def test_gemm_benchmark_shapes_on_sampled_tokens(accel, orc, synth, m, n, k):
    """The benchmark's full sizes. The oracle checks 64 sampled token rows (every row of the first and the
    last token tile boundary among them), which is exact because an output row depends on its own token only."""
    w = synth.q8_0(72, "gb", n, k)
    xs = synth.normal(72, "gb.x", m, k)
    key = "gb.%d.%d" % (n, k)
    assert accel.upload_q8_0(key, w, k, n)
    got = accel.prefill_q8_gemm(key, xs, m)
    fixed = [0, 1, 127, 128, 129, 255, 256, m // 2, m - 129, m - 128, m - 2, m - 1]
    rows = np.unique(np.concatenate([np.array(fixed), np.random.default_rng(5).choice(m, 52, replace=False)]))
    want = oracle_gemm(orc, synth, w, xs[rows], len(rows), k, n)
    r = rel_l2(got[rows], want)
    print("gemm m=%d n=%d k=%d: %d sampled rows rel-L2 %.2e max-abs %.2e" % (m, n, k, len(rows), r, np.abs(got[rows] - want).max()))
    assert r <= REL_L2_TOL
    assert np.abs(got[rows] - want).max() <= 1e-3 * np.abs(want).max()
    # rows outside the sample: same statistics, finite, non-zero
    assert np.isfinite(got).all() and (np.abs(got).max(axis=1) > 0).all()
    accel.upload_q8_0(key, synth.q8_0(1, "tiny", 1, 32), 32, 1)


def test_gemm_declines_like_the_reference(accel, synth):
    assert accel.upload_q4_0("gd.q4", synth.q4_0(1, "gd", 8, 64), 64, 8)
    assert accel.prefill_q8_gemm("gd.q4", np.zeros((2, 64), np.float32), 2) is None      # only the q8 map is searched
    assert accel.prefill_q8_gemm("gd.none", np.zeros((2, 64), np.float32), 2) is None
    assert accel.upload_q8_0("gd.q8", synth.q8_0(1, "gd8", 8, 64), 64, 8)
    assert accel.prefill_q8_gemm("gd.q8", np.zeros(100, np.float32), 2) is None           # xs.len() != m * in_dim


@pytest.mark.parametrize("m,n,k", [(1, 8, 32), (17, 100, 160), (130, 257, 2560), (200, 3840, 15360), (256, 4096, 3840)])
def test_q4_gemm_matches_integer_oracle(accel, orc, synth, m, n, k):
    """The prefill GEMM with Q4_0 weights (q4_gemm_w / q4_gemm_w_sk, kernels.rs:443-601): int32 block sums
    sum((nibble - 8) * xq) bit-exact from the tensor-core kernel, scaled output at the 1e-3 contract. The last two
    shapes are the verify configuration's ffn_down (K = 15360: split-K, the reference splits from K >= 12288) and
    q projection at the reference's chunk size of 256 tokens."""
    w = synth.q4_0(74, "g4", n, k)
    xs = synth.normal(74, "g4.x", m, k)
    key = "g4.%d.%d" % (n, k)
    assert accel.upload_q4_0(key, w, k, n)
    xq, xd, _ = orc.xquant8(xs)
    if m * n * (k // 32) <= 20_000_000:
        want, want_i = orc.idot_gemm(w, synth.Q4_0, xq, xd, m, k, n, want_isums=True)
        np.testing.assert_array_equal(accel.debug_gemm_isums(key, xs, m), want_i)
    else:
        want = orc.idot_gemm(w, synth.Q4_0, xq, xd, m, k, n)
    got = accel.prefill_q4_gemm(key, xs, m)
    assert got is not None and got.shape == (m, n)
    r = rel_l2(got, want)
    print("q4 gemm m=%d n=%d k=%d rel-L2 %.2e max-abs %.2e" % (m, n, k, r, np.abs(got - want).max()))
    assert r <= REL_L2_TOL and np.abs(got - want).max() <= 1e-3 * np.abs(want).max()
    assert accel.prefill_q8_gemm(key, xs, m) is None          # the q8 entry point looks only at Q8_0 weights
    assert accel.device_status() == 0
    accel.upload_q4_0(key, synth.q4_0(1, "tiny", 1, 32), 32, 1)
