"""Pins the CPU oracle: the reference's own known-answer tests, the committed golden
fixtures, and independent numpy restatements. CPU only."""
import os

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def f16b(v):
    return np.array([v], dtype=np.float16).view(np.uint8)


# ---- the reference's known-answer tests, crates/strix-models/src/ggml_quant.rs ----
def test_ref_q8_0_scales_each_int(orc):
    # ggml_quant.rs:443-453: d = 0.5, q[i] = i - 4
    qs = (np.arange(32) - 4).astype(np.int8)
    raw = np.concatenate([f16b(0.5), qs.view(np.uint8)])
    y = orc.dequantize(orc.Q8_0, raw, 32)
    np.testing.assert_array_equal(y, 0.5 * (np.arange(32, dtype=np.float32) - 4.0))


def test_ref_q4_0_nibble_layout_and_bias(orc):
    # ggml_quant.rs:456-469: d = 2; byte0 = 0x80, byte1 = 0xF1
    qs = np.zeros(16, dtype=np.uint8)
    qs[0], qs[1] = 0x80, 0xF1
    y = orc.dequantize(orc.Q4_0, np.concatenate([f16b(2.0), qs]), 32)
    assert y[0] == -16.0 and y[16] == 0.0 and y[1] == -14.0 and y[17] == 14.0


def test_ref_q6_k_decodes_known_values(orc):
    # ggml_quant.rs:497-514: ql[0] = 5, qh[0] = 1, scales 1, d = 1
    blk = np.zeros(210, dtype=np.uint8)
    blk[0], blk[128] = 0x05, 0x01
    blk[192:208] = 1
    blk[208:210] = f16b(1.0)
    y = orc.dequantize(orc.Q6_K, blk, 256)
    assert y[0] == -11.0 and y[1] == -32.0 and y[32] == -32.0 and y.size == 256


def test_ref_rejects_bad_sizes(orc):
    # ggml_quant.rs:562-565
    with pytest.raises(ValueError):
        orc.dequantize(orc.Q8_0, np.zeros(34, np.uint8), 16)
    with pytest.raises(ValueError):
        orc.dequantize(orc.Q4_0, np.zeros(4, np.uint8), 32)
    # extra bytes are ignored (bytes.len() < need is the only length check, :151-157)
    assert orc.dequantize(orc.Q4_0, np.zeros(40, np.uint8), 32).size == 32


def test_block_geometry(orc):
    # ggml_quant.rs:88-124
    assert orc.BLOCK_BYTES == {orc.Q4_0: 18, orc.Q4_1: 20, orc.Q8_0: 34, orc.Q6_K: 210}
    assert orc.BLOCK_ELEMS[orc.Q6_K] == 256 and orc.BLOCK_ELEMS[orc.Q4_0] == 32


# ---- half 2.7.1 f16 -> f32, exhaustively against numpy's IEEE binary16 ----
def test_f16_widening_exhaustive(orc):
    bits = np.arange(65536, dtype=np.uint16)
    want = bits.view(np.float16).astype(np.float32)
    got = np.array([orc.f16_to_f32(int(b)) for b in bits], dtype=np.float32)
    finite = ~np.isnan(want)
    np.testing.assert_array_equal(got[finite].view(np.uint32), want[finite].view(np.uint32))
    assert np.isnan(got[~finite]).all()


# ---- committed golden fixtures (independent numpy restatement, tests/golden/make_golden.py) ----
@pytest.mark.parametrize("name,ty,be", [("q4_0", 2, 32), ("q8_0", 8, 32), ("q6_k", 14, 256)])
def test_golden_dequant(orc, name, ty, be):
    g = np.load(os.path.join(HERE, "golden", "dequant_golden.npz"))
    raw, want = g[name + "_raw"], g[name + "_f32"]
    got = orc.dequantize(ty, raw, want.size)
    np.testing.assert_array_equal(got.view(np.uint32), want.view(np.uint32))


def test_q4_1_multiply_then_add(orc):
    # ggml_quant.rs:264-275: y = d*q + m, two roundings
    qs = np.arange(16, dtype=np.uint8) | ((15 - np.arange(16, dtype=np.uint8)) << 4)
    raw = np.concatenate([f16b(0.1), f16b(-0.7), qs])
    y = orc.dequantize(orc.Q4_1, raw, 32)
    d, m = np.float32(np.float16(0.1)), np.float32(np.float16(-0.7))
    lo = (d * np.arange(16, dtype=np.float32)).astype(np.float32) + m
    hi = (d * (15 - np.arange(16)).astype(np.float32)).astype(np.float32) + m
    np.testing.assert_array_equal(y, np.concatenate([lo, hi]).astype(np.float32))


# ---- dot_f32: the 8-lane order of qwen3.rs:90-105 ----
def _dot8(a, b):
    a, b = a.astype(np.float32), b.astype(np.float32)
    acc = np.zeros(8, dtype=np.float32)
    n = a.size
    for c in range(n // 8):
        acc = (acc + a[8 * c:8 * c + 8] * b[8 * c:8 * c + 8]).astype(np.float32)
    s = np.float32(np.float32(np.float32(acc[0] + acc[1]) + np.float32(acc[2] + acc[3])) +
                   np.float32(np.float32(acc[4] + acc[5]) + np.float32(acc[6] + acc[7])))
    for i in range(n // 8 * 8, n):
        s = np.float32(s + np.float32(a[i] * b[i]))
    return s


@pytest.mark.parametrize("n", [0, 1, 7, 8, 9, 64, 259, 2560])
def test_dot_f32_lane_order(orc, n):
    g = np.random.default_rng(n)
    a = (g.standard_normal(n) * 10 ** g.uniform(-3, 3, n)).astype(np.float32)
    b = g.standard_normal(n).astype(np.float32)
    assert np.float32(orc.dot_f32(a, b)).view(np.uint32) == _dot8(a, b).view(np.uint32)


def test_qmatmul_is_row_dequant_then_dot(orc, synth):
    in_dim, out_dim = 512, 37
    for ty in (synth.Q4_0, synth.Q8_0, synth.Q6_K):
        w = synth.quant(ty, 3, "w%d" % ty, out_dim, in_dim)
        x = synth.normal(3, "x", in_dim)
        y = orc.qmatmul(x, w, ty, in_dim, out_dim, threads=3)
        bpr = in_dim // synth.BLOCK_ELEMS[ty] * synth.BLOCK_BYTES[ty]
        for o in (0, 17, 36):
            row = orc.dequantize(ty, w[o * bpr:(o + 1) * bpr], in_dim)
            assert np.float32(y[o]).view(np.uint32) == _dot8(row, x).view(np.uint32)
        # thread count must not change any bit (one thread owns a row)
        np.testing.assert_array_equal(y, orc.qmatmul(x, w, ty, in_dim, out_dim, threads=1))


def test_qmatmul_batch_matches_token_at_a_time(orc, synth):
    # mellum.rs:244-271: "each row's value is bit-identical to the token-at-a-time path"
    in_dim, out_dim, m = 256, 19, 5
    w = synth.q8_0(4, "w", out_dim, in_dim)
    xs = synth.normal(4, "xs", m, in_dim)
    yb = orc.qmatmul_batch(xs, m, w, synth.Q8_0, in_dim, out_dim)
    for t in range(m):
        np.testing.assert_array_equal(yb[t], orc.qmatmul(xs[t], w, synth.Q8_0, in_dim, out_dim))


# ---- norm / activations vs straight numpy in f32 ----
def test_rmsnorm_swiglu_geglu(orc):
    g = np.random.default_rng(5)
    x = g.standard_normal(2560).astype(np.float32)
    w = (1 + 0.02 * g.standard_normal(2560)).astype(np.float32)
    ss = np.float32(0)
    for v in x:
        ss = np.float32(ss + np.float32(v * v))
    scale = np.float32(1.0) / np.sqrt(np.float32(ss / np.float32(2560) + np.float32(1e-6)))
    np.testing.assert_array_equal(orc.rmsnorm(x, w, 1e-6), ((x * scale).astype(np.float32) * w).astype(np.float32))
    u = g.standard_normal(2560).astype(np.float32)
    want = x.astype(np.float64) / (1 + np.exp(-x.astype(np.float64))) * u
    np.testing.assert_allclose(orc.swiglu(x, u), want, rtol=2e-6, atol=1e-7)
    xd = x.astype(np.float64)
    wantg = 0.5 * xd * (1 + np.tanh(0.7978846 * (xd + 0.044715 * xd ** 3))) * u
    np.testing.assert_allclose(orc.geglu(x, u), wantg, rtol=3e-6, atol=1e-7)


# ---- activation quantiser (kernels.rs:864-876) ----
def test_xquant8_rule(orc):
    x = np.zeros(96, dtype=np.float32)
    # block 0: amax 127 -> d = 1, inv = 1: ties go to even, clamp at +-127
    x[0:8] = [127.0, 0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 126.5]
    # block 1: all zero -> d = 0, inv = 0, q = 0
    # block 2: negative amax
    x[64:68] = [-3.0, 1.0, 2.0, 3.0]
    q, d, ties = orc.xquant8(x)
    assert d[0] == 1.0 and list(q[0:8]) == [127, 0, 2, 2, 0, -2, -2, 126]
    assert ties == 7
    assert d[1] == 0.0 and not q[32:64].any()
    assert d[2] == np.float32(3.0) / np.float32(127.0) and q[64] == -127 and q[67] == 127


def test_xquant8_matches_numpy(orc, synth):
    x = synth.normal(9, "x", 9728)
    q, d, _ = orc.xquant8(x)
    xb = x.reshape(-1, 32)
    amax = np.abs(xb).max(axis=1)
    dd = (amax / np.float32(127.0)).astype(np.float32)
    inv = np.where(dd > 0, np.float32(1.0) / dd, np.float32(0)).astype(np.float32)
    qq = np.clip(np.rint((xb * inv[:, None]).astype(np.float32)), -127, 127).astype(np.int8)
    np.testing.assert_array_equal(d, dd)
    np.testing.assert_array_equal(q, qq.reshape(-1))


# ---- integer-dot GEMV / W8A8 GEMM ----
def _np_isums_q8(w, xq, m, in_dim, out_dim):
    blk = w.reshape(out_dim, in_dim // 32, 34)
    wq = blk[:, :, 2:].view(np.int8).astype(np.int32)           # [n, nb, 32]
    x = xq.reshape(m, in_dim // 32, 32).astype(np.int32)        # [m, nb, 32]
    return np.einsum("nbi,mbi->mnb", wq, x).astype(np.int32)


def test_idot_q8_isums_exact_and_scaled_sum(orc, synth):
    in_dim, out_dim, m = 256, 23, 3
    w = synth.q8_0(6, "w", out_dim, in_dim)
    xs = synth.normal(6, "xs", m, in_dim)
    xq, xd, _ = orc.xquant8(xs)
    y, isums = orc.idot_gemm(w, synth.Q8_0, xq, xd, m, in_dim, out_dim, want_isums=True)
    want_i = _np_isums_q8(w, xq, m, in_dim, out_dim)
    np.testing.assert_array_equal(isums, want_i)
    dw = w.reshape(out_dim, in_dim // 32, 34)[:, :, 0:2].copy().view(np.float16).astype(np.float32).reshape(out_dim, -1)
    acc = np.zeros((m, out_dim), dtype=np.float32)
    xdm = xd.reshape(m, -1)
    for b in range(in_dim // 32):
        sc = (dw[None, :, b] * xdm[:, None, b]).astype(np.float32)
        acc = (acc + (sc * want_i[:, :, b].astype(np.float32)).astype(np.float32)).astype(np.float32)
    np.testing.assert_array_equal(y, acc)


def test_idot_q4_equals_signed_nibble_dot(orc, synth):
    in_dim, out_dim = 128, 11
    w = synth.q4_0(7, "w", out_dim, in_dim)
    x = synth.normal(7, "x", in_dim)
    xq, xd, _ = orc.xquant8(x)
    _, isums = orc.idot_gemm(w, synth.Q4_0, xq, xd, 1, in_dim, out_dim, want_isums=True)
    blk = w.reshape(out_dim, in_dim // 32, 18)[:, :, 2:]
    codes = np.concatenate([blk & 0x0F, blk >> 4], axis=2).astype(np.int32) - 8   # element order j, j+16
    want = np.einsum("nbi,bi->nb", codes, xq.reshape(-1, 32).astype(np.int32))
    np.testing.assert_array_equal(isums[0], want)


def test_idot_close_to_f32_path(orc, synth):
    # integer-dot differs from the f32-activation result only by the activation's
    # quantisation error (the reference accepts rel < 2e-2 for its dp4a variant)
    in_dim, out_dim = 2560, 64
    x = synth.normal(8, "x", in_dim)
    xq, xd, _ = orc.xquant8(x)
    for ty in (synth.Q4_0, synth.Q8_0, synth.Q6_K):
        w = synth.quant(ty, 8, "w%d" % ty, out_dim, in_dim)
        yi = orc.idot_gemm(w, ty, xq, xd, 1, in_dim, out_dim)[0]
        yf = orc.qmatmul(x, w, ty, in_dim, out_dim)
        rel = np.linalg.norm(yi - yf) / np.linalg.norm(yf)
        assert rel < 2e-2, (ty, rel)
        # and exactly equals a float64 evaluation of the same quantised operands within f32 rounding
        deq = orc.dequantize(ty, w, in_dim * out_dim).reshape(out_dim, in_dim).astype(np.float64)
        xdeq = (xq.astype(np.float64).reshape(-1, 32) * xd.astype(np.float64)[:, None]).reshape(-1)
        ref = deq @ xdeq
        assert np.linalg.norm(yi - ref) / np.linalg.norm(ref) < 1e-5


def test_argmax_follows_the_reference_kernel(orc):
    # kernels.rs:2088-2110: start at (-3.0e38, 0), replace on GREATER only, lowest index on ties.
    # A scalar replay of that loop (one thread, ascending) is the known answer.
    def replay(x):
        bv, bi = np.float32(-3.0e38), 0
        for i, v in enumerate(x):
            if v > bv:
                bv, bi = v, i
        return bi

    rng = np.random.default_rng(5)
    cases = [np.array([1.0, 3.0, 3.0, 2.0], np.float32), np.array([np.nan, 2.0, np.nan, 2.0], np.float32),
             np.full(7, -np.inf, np.float32), np.array([-3.0e38, -3.0e38], np.float32),
             np.array([np.nan], np.float32), np.array([np.inf, np.inf, 1.0], np.float32)]
    cases += [rng.integers(-3, 4, 50).astype(np.float32) for _ in range(20)]
    for x in cases:
        with np.errstate(invalid="ignore"):
            assert orc.argmax_f32(x) == replay(x), x


def test_q4_1_integer_dot_follows_q4_1_gemv_dp(orc, synth):
    # kernels.rs:289-320: acc += xd * (d * (float)isum + m * (float)xsum), codes 0..15 not centred
    in_dim, out_dim = 256, 12
    w = synth.quant(synth.Q4_1, 9, "w41", out_dim, in_dim)
    x = synth.normal(9, "x41", in_dim)
    xq, xd, _ = orc.xquant8(x)
    y, isums = orc.idot_gemm(w, synth.Q4_1, xq, xd, 1, in_dim, out_dim, want_isums=True)
    blk = w.reshape(out_dim, in_dim // 32, 20)
    d = blk[:, :, 0:2].copy().view(np.float16)[:, :, 0].astype(np.float64)
    m = blk[:, :, 2:4].copy().view(np.float16)[:, :, 0].astype(np.float64)
    codes = np.concatenate([blk[:, :, 4:] & 0x0F, blk[:, :, 4:] >> 4], axis=2).astype(np.int64)   # element order j, j+16
    xb = xq.reshape(-1, 32).astype(np.int64)
    want_isum = np.einsum("nbi,bi->nb", codes, xb)
    np.testing.assert_array_equal(isums[0], want_isum)
    ref = ((d * want_isum + m * xb.sum(axis=1)[None, :]) * xd.astype(np.float64)[None, :]).sum(axis=1)
    assert np.linalg.norm(y[0] - ref) / np.linalg.norm(ref) < 1e-5
    # and close to the f32-activation path (activation quantisation error only)
    yf = orc.qmatmul(x, w, synth.Q4_1, in_dim, out_dim)
    assert np.linalg.norm(y[0] - yf) / np.linalg.norm(yf) < 2e-2


def test_attention_pieces_known_answers(orc):
    # rope_neox (qwen3.rs:126-138) at pos 0 is the identity; at pos p pair k is rotated by p * base^(-2k/n)
    v = np.arange(1, 9, dtype=np.float32)
    np.testing.assert_array_equal(orc.rope_neox(v, 0, 8, 10000.0), v)
    r = orc.rope_neox(v, 3, 8, 10000.0)
    for k in range(4):
        th = 3.0 * 10000.0 ** (-2.0 * k / 8)
        assert abs(r[k] - (v[k] * np.cos(th) - v[k + 4] * np.sin(th))) < 1e-5
        assert abs(r[k + 4] - (v[k] * np.sin(th) + v[k + 4] * np.cos(th))) < 1e-5
    # rmsnorm_inplace (qwen3.rs:117-124)
    x = np.array([3.0, 4.0], dtype=np.float32)
    np.testing.assert_allclose(orc.rmsnorm_inplace(x, np.array([1.0, 2.0], np.float32), 0.0),
                               [3.0 / np.sqrt(12.5), 8.0 / np.sqrt(12.5)], rtol=1e-6)
    # one head, two cached tokens, no norm, hd = 2: softmax over two scores, checked by hand in f64
    kc, vc = [], []
    a0 = orc.attention_token([1.0, 0.0], [1.0, 0.0], [5.0, 7.0], None, None, 0, kc, vc, 1, 1, 2, 1e-6, 10000.0)
    np.testing.assert_allclose(a0, [5.0, 7.0], rtol=1e-6)          # one token: its own value
    a1 = orc.attention_token([1.0, 0.0], [0.0, 0.0], [1.0, 1.0], None, None, 1, kc, vc, 1, 1, 2, 1e-6, 10000.0)
    q = np.array([np.cos(1.0), np.sin(1.0)])                        # rope at pos 1, pair (0, 1), theta = 1
    s = np.array([q @ np.array([1.0, 0.0]), 0.0]) / np.sqrt(2.0)
    w = np.exp(s - s.max()); w /= w.sum()
    np.testing.assert_allclose(a1, w[0] * np.array([5.0, 7.0]) + w[1] * np.array([1.0, 1.0]), rtol=1e-5)


def test_attention_flavour_known_answers(orc):
    """The known answers of the reference's own unit tests for these pieces (crates/strix-backend-cpu/src/ops.rs
    tests: rope at position 0, first-pair rotation, norm preservation, softcap bounds; attention.rs tests: a single
    position returns its value, equal scores average, a dominant key dominates, convexity), against the oracle."""
    # ops.rs rope_at_position_zero_is_identity / rope_rotates_first_pair_as_expected / rope_preserves_norm
    v = np.array([0.5, -1.0, 2.0, 0.25], dtype=np.float32)
    np.testing.assert_allclose(orc.rope_pow(v, 0, 10000.0), v, atol=1e-6)
    r = orc.rope_pow(np.array([1.0, 0.0], np.float32), 1, 10000.0)
    np.testing.assert_allclose(r, [np.cos(np.float32(1.0)), np.sin(np.float32(1.0))], atol=1e-6)
    v6 = np.array([0.3, 0.7, -1.2, 2.5, 0.1, -0.6], dtype=np.float32)
    for rot in (orc.rope_pow(v6, 7, 10000.0), orc.rope_adjacent(v6, 7, 6, 10000.0), orc.rope_neox(v6, 7, 6, 10000.0)):
        assert abs(float((rot * rot).sum()) - float((v6 * v6).sum())) < 1e-4
    # frequency factors divide the inverse frequency (ops.rs:166-168): a factor of 2 on pair 0 halves its angle
    r2 = orc.rope_pow(np.array([1.0, 0.0], np.float32), 1, 10000.0, np.array([2.0], np.float32))
    np.testing.assert_allclose(r2, [np.cos(0.5), np.sin(0.5)], atol=1e-6)
    # adjacent pairs (smollm3.rs:126-138): hd = 4 at pos 1: pair 0 = (x0, x1) by angle 1, pair 1 = (x2, x3) by base^(-1/2)
    ra = orc.rope_adjacent(np.array([1.0, 0.0, 1.0, 0.0], np.float32), 1, 4, 10000.0)
    np.testing.assert_allclose(ra, [np.cos(1.0), np.sin(1.0), np.cos(0.01), np.sin(0.01)], atol=1e-6)
    # ops.rs softcap_bounds_and_is_near_identity_for_small
    x = orc.softcap(np.array([1000.0, -1000.0, 0.5], np.float32), 30.0)
    assert 29.0 < x[0] <= 30.0 and -30.0 <= x[1] < -29.0
    assert abs(x[2] - 30.0 * np.tanh(np.float32(0.5) / np.float32(30.0))) < 1e-6
    np.testing.assert_array_equal(orc.softcap(np.array([3.0], np.float32), 0.0), [3.0])
    # attention.rs single_position_returns_that_value / equal_scores_average_values / dominant_key / convexity,
    # through the flavour entry point (no norm, no rope, one head)
    def attend(q, keys, values, hd, scale):
        kc, vc, out = [], [], None
        n = len(keys) // hd
        for t in range(n):
            out = orc.attention_token_flavour(q, keys[t * hd:(t + 1) * hd], values[t * hd:(t + 1) * hd], None, None, t,
                                              kc, vc, 1, 1, hd, 0.0, None, scale=scale)
        return out
    np.testing.assert_allclose(attend([0.3, -0.7], [1.0, 2.0], [5.0, -9.0], 2, 1 / np.sqrt(2.0)), [5.0, -9.0], atol=1e-6)
    np.testing.assert_allclose(attend([1.0, 1.0], [0.5] * 4, [2.0, 4.0, 6.0, 8.0], 2, 1 / np.sqrt(2.0)), [4.0, 6.0], atol=1e-6)
    np.testing.assert_allclose(attend([10.0, 0.0], [10.0, 0.0, -10.0, 0.0], [1.0, 1.0, 99.0, 99.0], 2, 1 / np.sqrt(2.0)),
                               [1.0, 1.0], atol=1e-3)
    o = attend([0.4], [0.1, 0.9, -0.3], [3.0, 7.0, 5.0], 1, 1.0)
    assert 3.0 - 1e-6 <= o[0] <= 7.0 + 1e-6
    # the sliding window (gemma.rs:840-851): with window 2 the third token no longer sees the first
    kc, vc = [], []
    for t, (k, val) in enumerate([([9.0], [100.0]), ([0.0], [1.0]), ([0.0], [3.0])]):
        o = orc.attention_token_flavour([1.0], k, val, None, None, t, kc, vc, 1, 1, 1, 0.0, None, window=2, scale=1.0)
    np.testing.assert_allclose(o, [2.0], atol=1e-6)
    # shared K = V takes the RAW k as value, before the K-norm (gemma.rs:796-803); V-norm has no weight (gemma.rs:804-813)
    o = orc.attention_token_flavour([1.0, 0.0], [3.0, 4.0], None, None, np.array([2.0, 2.0], np.float32), 0, [], [], 1, 1, 2,
                                    0.0, None, scale=1.0)
    np.testing.assert_allclose(o, [3.0, 4.0], atol=1e-6)
    o = orc.attention_token_flavour([1.0, 0.0], [3.0, 4.0], None, None, None, 0, [], [], 1, 1, 2, 0.0, None, norm_v=True, scale=1.0)
    np.testing.assert_allclose(o, np.array([3.0, 4.0]) / np.sqrt(12.5), rtol=1e-6)
    # sandwich residual (gemma.rs:268-275, 876-879, 896-906)
    np.testing.assert_allclose(orc.addnorm([1.0, 1.0], [3.0, 4.0], [1.0, 2.0], 0.0, 0.5),
                               0.5 * (1.0 + np.array([3.0, 8.0]) / np.sqrt(12.5)), rtol=1e-6)


def test_f16_cache_rounding_follows_the_reference_kernel(orc):
    """kernels.rs:18-32 f2h: to nearest, a tie away from zero (numpy rounds a tie to even); overflow -> infinity;
    below half the smallest subnormal -> zero; kernels.rs:8-16 h2f is exact."""
    x = np.array([1.0, 1.0 + 2.0 ** -11, 1.0 + 3 * 2.0 ** -11, -1.0 - 2.0 ** -11, 65519.0, 65520.0, 1e9, 2.0 ** -24,
                  2.0 ** -25, 2.0 ** -26, 2.0 ** -15 + 2.0 ** -25, 0.0, -0.0], dtype=np.float32)
    want = [0x3C00, 0x3C01, 0x3C02, 0xBC01, 0x7BFF, 0x7C00, 0x7C00, 0x0001, 0x0001, 0x0000, 0x0201, 0x0000, 0x8000]
    np.testing.assert_array_equal(orc.f32_to_f16_cache(x), np.array(want, dtype=np.uint16))
    # away from ties it is the IEEE conversion
    r = np.random.default_rng(5).standard_normal(50000).astype(np.float32)
    h = orc.f32_to_f16_cache(r)
    ties = (r.view(np.uint32) & 0x1FFF) == 0x1000
    np.testing.assert_array_equal(h[~ties], r.astype(np.float16).view(np.uint16)[~ties])
    np.testing.assert_array_equal(orc.f16_cache_to_f32(h), h.view(np.float16).astype(np.float32))


def test_moe_router_and_ffn_rules(orc, synth):
    """mellum.rs:1590-1609 router: softmax, the k most probable by a stable sort (a tie keeps the lower index),
    weights renormalised over the chosen; mellum.rs:1624-1660: the weighted sum of the experts' FFNs."""
    ids, w = orc.topk_router(np.array([0.0, 2.0, 2.0, -1.0, 1.0], np.float32), 3)
    assert list(ids) == [1, 2, 4]
    p = np.exp(np.array([2.0, 2.0, 1.0]) - 2.0)
    np.testing.assert_allclose(w, p / p.sum(), rtol=1e-6)
    assert abs(float(w.sum()) - 1.0) < 1e-6
    ids, w = orc.topk_router(np.zeros(8, np.float32), 8)            # all tied: index order, uniform weights
    assert list(ids) == list(range(8))
    np.testing.assert_allclose(w, np.full(8, 0.125), rtol=1e-6)
    # two experts, weights (1, 0) -> exactly the first expert's FFN; (0.5, 0.5) -> the mean
    hidden, eff, ne = 64, 32, 3
    gate = synth.quant(synth.Q8_0, 7, "moe.gate", ne * eff, hidden)
    up = synth.quant(synth.Q8_0, 7, "moe.up", ne * eff, hidden)
    down = synth.quant(synth.Q8_0, 7, "moe.down", ne * hidden, eff)
    x = synth.normal(8, "x", hidden)
    e0 = orc.moe_expert_ffn(x, gate, up, down, synth.Q8_0, hidden, eff, 2)
    e1 = orc.moe_expert_ffn(x, gate, up, down, synth.Q8_0, hidden, eff, 0)
    np.testing.assert_array_equal(orc.moe_ffn(x, gate, up, down, synth.Q8_0, hidden, eff, [2, 0], [1.0, 0.0]), e0)
    np.testing.assert_allclose(orc.moe_ffn(x, gate, up, down, synth.Q8_0, hidden, eff, [2, 0], [0.5, 0.5]), 0.5 * (e0 + e1), rtol=1e-6, atol=1e-7)
    # the expert slices are what a per-expert matmul on the slice gives (mellum.rs:1620-1622)
    gb, db = orc.moe_expert_bytes(synth.Q8_0, hidden, eff)
    assert gb == (hidden // 32) * 34 * eff and db == (eff // 32) * 34 * hidden
    g = orc.qmatmul(x, np.frombuffer(gate, np.uint8)[2 * gb:3 * gb], synth.Q8_0, hidden, eff)
    u = orc.qmatmul(x, np.frombuffer(up, np.uint8)[2 * gb:3 * gb], synth.Q8_0, hidden, eff)
    np.testing.assert_array_equal(e0, orc.qmatmul(orc.swiglu(g, u), np.frombuffer(down, np.uint8)[2 * db:3 * db], synth.Q8_0, eff, hidden))
