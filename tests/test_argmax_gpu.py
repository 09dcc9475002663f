"""GPU parity of the on-device greedy argmax and the two trait methods built on it
(lm_head_argmax_rows, decode_step_argmax) against the oracle. Index work: bit-exact."""
import numpy as np
import pytest

from test_decode_gpu import build_model

pytestmark = pytest.mark.gpu


def _dev_argmax(accel, x2d):
    import torch
    rows, n = x2d.shape
    d = torch.from_numpy(np.ascontiguousarray(x2d)).cuda()
    ids = torch.zeros(rows, dtype=torch.int32, device="cuda")
    vals = torch.zeros(rows, dtype=torch.float32, device="cuda")
    s = torch.cuda.current_stream().cuda_stream
    assert accel.argmax_dev(d.data_ptr(), n, n, rows, ids.data_ptr(), vals.data_ptr(), stream=s)
    torch.cuda.synchronize()
    return ids.cpu().numpy().astype(np.int64), vals.cpu().numpy()


@pytest.mark.parametrize("n", [1, 2, 5, 31, 1023, 1024, 1025, 4097, 151936, 262144 + 3])
def test_argmax_matches_oracle_on_ties_nan_and_floor(accel, orc, synth, n):
    rows = 5
    x = synth.normal(7, "am.%d" % n, rows * n).reshape(rows, n).copy()
    # row 1: the maximum repeated (lowest index must win); row 2: NaN and +inf mixed in;
    # row 3: nothing above the kernel's floor (-3.0e38) -> index 0; row 4: maximum at the very end
    if n > 2:
        m = x[1].max()
        x[1, n // 2] = m
        x[1, n - 1] = m
    x[2, ::3] = np.nan
    if n > 4:
        x[2, n // 3] = np.inf
        x[2, n // 3 + 1] = np.inf
    x[3, :] = -np.inf
    x[3, n // 2] = np.float32(-3.0e38)
    x[4, n - 1] = 100.0
    ids, vals = _dev_argmax(accel, x)
    for r in range(rows):
        want = orc.argmax_f32(x[r])
        assert ids[r] == want, (n, r)
        if r != 3 and not np.isnan(x[r, want]):
            assert vals[r] == x[r, want]
    # the scratch (tickets) is reusable: a second launch gives the same answer
    ids2, _ = _dev_argmax(accel, x)
    np.testing.assert_array_equal(ids, ids2)


def test_argmax_unaligned_rows_take_the_scalar_path(accel, orc, synth):
    import torch
    n, rows = 1001, 3                               # stride not a multiple of 4 floats
    x = synth.normal(8, "am.u", rows * n).reshape(rows, n)
    d = torch.from_numpy(np.ascontiguousarray(x)).cuda()
    ids = torch.zeros(rows, dtype=torch.int32, device="cuda")
    assert accel.argmax_dev(d.data_ptr(), n, n, rows, ids.data_ptr(), 0, stream=torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    for r in range(rows):
        assert int(ids[r]) == orc.argmax_f32(x[r])


@pytest.mark.parametrize("ty,out_dim,in_dim", [(8, 3000, 512), (14, 5003, 512), (2, 777, 256)])
def test_lm_head_argmax_rows(accel, orc, synth, pkg, ty, out_dim, in_dim):
    w = synth.quant(ty, 51, "lh", out_dim, in_dim)
    up = {2: accel.upload_q4_0, 8: accel.upload_q8_0, 14: accel.upload_q6_k}[ty]
    assert up("lh", w, in_dim, out_dim)
    for m in (1, 3, 8, 16):
        xs = synth.normal(52, "lh.x%d" % m, m * in_dim)
        ids, vals = accel.lm_head_argmax_rows("lh", xs, m, with_values=True)
        y = accel.gemv_rows("lh", xs, m)            # the same kernels' logits
        for t in range(m):
            assert ids[t] == orc.argmax_f32(y[t])   # bit-exact against the device logits
            assert vals[t] == y[t, ids[t]]
            # and the oracle's own logits put the same row on top (or within rounding of the top)
            want = orc.qmatmul(xs[t * in_dim:(t + 1) * in_dim], w, ty, in_dim, out_dim)
            assert want[ids[t]] >= want.max() - 1e-4 * np.abs(want).max()
        ids_i = accel.lm_head_argmax_rows("lh", xs, m, act=pkg.ACT_Q8DOT)
        yi = accel.gemv_rows("lh", xs, m, act=pkg.ACT_Q8DOT)
        for t in range(m):
            assert ids_i[t] == orc.argmax_f32(yi[t])
    # the reference's guards (decode.rs:3631-3635): unknown key, wrong length, m > 16 -> None
    assert accel.lm_head_argmax_rows("nope", np.zeros(in_dim, np.float32), 1) is None
    assert accel.lm_head_argmax_rows("lh", np.zeros(in_dim + 1, np.float32), 1) is None
    assert accel.lm_head_argmax_rows("lh", np.zeros(17 * in_dim, np.float32), 17) is None
    assert accel.device_status() == 0


@pytest.mark.parametrize("int8", [False, True])
def test_decode_step_argmax_equals_argmax_of_decode_step(pkg, orc, synth, int8):
    hidden, qdim, kvdim, ffn, vocab, n_layers, eps = 512, 768, 256, 1536, 3000, 2, 1e-6
    acc = pkg.CudaWeightAccel(0)
    try:
        assert acc.decode_step_argmax(np.zeros(hidden, np.float32)) is None      # not configured -> None
        build_model(acc, synth, hidden, qdim, kvdim, ffn, vocab, n_layers)
        act = pkg.ACT_Q8DOT if int8 else pkg.ACT_F32
        assert acc.configure_decode(hidden, qdim // 128, ffn, vocab, n_layers, eps=eps, act=act)
        for seed in (1, 2, 3):
            h0 = synth.normal(90 + seed, "h0", hidden)
            logits = acc.decode_step(h0, 0)
            tok = acc.decode_step_argmax(h0, 0)
            assert tok == orc.argmax_f32(logits)
        assert acc.device_status() == 0
    finally:
        acc.close()


def test_lm_head_argmax_rows_row_sharded(pkg, orc, synth):
    """Three row-sharded accelerators (on the one device): each returns the winner among its rows as a row
    index of the whole weight plus its value; the fold of the shards equals the unsharded answer."""
    in_dim, out_dim, m, world = 512, 3001, 5, 3
    w = synth.quant(14, 61, "lhs", out_dim, in_dim)
    xs = synth.normal(62, "lhs.x", m * in_dim)
    accs = [pkg.CudaWeightAccel(0, rank=r, world=world) for r in range(world)]
    whole = pkg.CudaWeightAccel(0)
    try:
        assert whole.upload_q6_k("lhs", w, in_dim, out_dim)
        want = whole.lm_head_argmax_rows("lhs", xs, m)
        ids, vals = [], []
        for a in accs:
            assert a.upload_q6_k("lhs", w, in_dim, out_dim)
            i, v = a.lm_head_argmax_rows("lhs", xs, m, with_values=True)
            info = a.weight_info("lhs")
            assert ((i >= info["row0"]) & (i < info["row0"] + info["rows"])).all()
            ids.append(i)
            vals.append(v)
        np.testing.assert_array_equal(pkg.fold_argmax_shards(ids, vals), want)
        for a in accs:
            assert a.decode_step_argmax(np.zeros(8, np.float32)) is None   # nothing configured on a shard
    finally:
        for a in accs + [whole]:
            a.close()
