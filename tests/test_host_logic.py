"""Host-side logic that needs no GPU: row sharding, synthetic tensors, and the
world-size-2 gather of row shards (gloo)."""
import os
import sys

import numpy as np
import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.mark.parametrize("rows,world", [(0, 1), (1, 1), (7, 2), (8, 8), (9, 8), (151936, 8), (2560, 3), (5, 8)])
def test_shard_begin_partitions_rows(pkg, rows, world):
    edges = [pkg.shard_begin(rows, world, r) for r in range(world + 1)]
    assert edges[0] == 0 and edges[-1] == rows
    sizes = np.diff(edges)
    assert (sizes >= 0).all() and sizes.max() - sizes.min() <= 1


def test_synth_is_seeded_and_sized(synth):
    for ty in (synth.Q4_0, synth.Q8_0, synth.Q6_K):
        a = synth.quant(ty, 1, "t", 5, 512)
        b = synth.quant(ty, 1, "t", 5, 512)
        c = synth.quant(ty, 2, "t", 5, 512)
        assert a.size == synth.gguf_bytes(ty, 5, 512)
        assert (a == b).all() and (a != c).any()
    w = synth.q8_0(1, "t", 64, 256).reshape(64, 8, 34)
    q = w[:, :, 2:].view(np.int8)
    assert q.min() >= -127 and q.max() <= 127
    d = w[:, :, 0:2].copy().view(np.float16).astype(np.float32)
    assert d.min() >= 9e-5 and d.max() <= 1.01e-3
    w6 = synth.q6_k(1, "t", 8, 512).reshape(8, 2, 210)
    sc = w6[:, :, 192:208].view(np.int8)
    assert sc.min() >= -32 and sc.max() <= 31


def test_lcg_recipe_first_draws(synth):
    # crates/strix-backend-rocm/src/lib.rs:140-152: seed, multiplier, increment, >> 33
    raw, x = synth.lcg_q4_0(2, 64)
    s = 0xA5A51234
    draws = []
    for _ in range(5):
        s = (s * 6364136223846793005 + 1) & 0xFFFFFFFFFFFFFFFF
        draws.append((s >> 33) & 0xFFFFFFFF)
    blk = raw[:18]
    d = np.array([0.03 + (draws[0] % 32) * 0.003], dtype=np.float32).astype(np.float16).view(np.uint8)
    assert (blk[0:2] == d).all()
    assert (blk[2:6] == np.array([draws[1]], dtype=np.uint32).view(np.uint8)).all()
    assert x[0] == 0 and abs(x[1] - 0.5 * np.sin(0.017)) < 1e-7


def _gloo_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()
    orc = entry.load_oracle()
    from strix_rs_b200 import synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        in_dim, out_dim = 256, 37   # 37 rows over 2 ranks: 19 + 18
        w = synth.q8_0(11, "w", out_dim, in_dim)
        x = synth.normal(11, "x", in_dim)
        r0, r1 = pkg.shard_begin(out_dim, world, rank), pkg.shard_begin(out_dim, world, rank + 1)
        bpr = in_dim // 32 * 34
        mine = orc.qmatmul(x, w[r0 * bpr:r1 * bpr], synth.Q8_0, in_dim, r1 - r0)
        # ragged all-gather of the row shards: pad to the largest shard
        cap = max(pkg.shard_begin(out_dim, world, r + 1) - pkg.shard_begin(out_dim, world, r) for r in range(world))
        buf = torch.zeros(cap)
        buf[:r1 - r0] = torch.from_numpy(mine)
        got = [torch.zeros(cap) for _ in range(world)]
        dist.all_gather(got, buf)
        full = np.concatenate([got[r].numpy()[:pkg.shard_begin(out_dim, world, r + 1) - pkg.shard_begin(out_dim, world, r)]
                               for r in range(world)])
        want = orc.qmatmul(x, w, synth.Q8_0, in_dim, out_dim)
        q.put((rank, bool((full == want).all())))
    finally:
        dist.destroy_process_group()


def test_row_shards_gather_to_the_unsharded_result_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + os.getpid() % 2000
    ps = [ctx.Process(target=_gloo_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(60)
    assert res == [(0, True), (1, True)]


def _gloo_argmax_worker(rank, world, port, q):
    sys.path.insert(0, ROOT)
    import torch.distributed as dist

    import __graft_entry__ as entry
    pkg = entry.load_package()
    orc = entry.load_oracle()
    from strix_rs_b200 import synth
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        # what a row-sharded lm_head_argmax_rows returns on each rank: the winner among ITS rows (global row
        # index) and its value; the caller gathers the pairs and folds them
        in_dim, out_dim, m = 256, 41, 3
        w = synth.q8_0(12, "w", out_dim, in_dim)
        xs = synth.normal(12, "xs", m * in_dim).reshape(m, in_dim)
        full = np.stack([orc.qmatmul(xs[t], w, synth.Q8_0, in_dim, out_dim) for t in range(m)])
        full[1, 7] = full[1, 30] = full[1].max() + 1.0      # a tie across the two shards: the lower row wins
        full[2, :] = np.nan                                  # nothing wins: row 0
        r0, r1 = pkg.shard_begin(out_dim, world, rank), pkg.shard_begin(out_dim, world, rank + 1)
        ids = [orc.argmax_f32(full[t, r0:r1]) + r0 for t in range(m)]
        vals = [float(full[t, i]) for t, i in enumerate(ids)]
        got = [None] * world
        dist.all_gather_object(got, (ids, vals))
        folded = pkg.fold_argmax_shards([g[0] for g in got], [g[1] for g in got])
        want = [orc.argmax_f32(full[t]) for t in range(m)]
        q.put((rank, [int(v) for v in folded] == want and want[1] == 7 and want[2] == 0))
    finally:
        dist.destroy_process_group()


def test_sharded_argmax_folds_to_the_unsharded_winner_gloo():
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + os.getpid() % 2000
    ps = [ctx.Process(target=_gloo_argmax_worker, args=(r, 2, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    res = sorted(q.get(timeout=120) for _ in ps)
    for p in ps:
        p.join(60)
    assert res == [(0, True), (1, True)]


def test_fold_argmax_shards_rule(pkg):
    """strix_cuda_fold_argmax_shards against the kernel's rule restated in numpy: greater wins, ties go to the
    lower row index, NaN never wins, nothing above the floor leaves (row 0, -3.0e38)."""
    import numpy as np
    rng = np.random.default_rng(11)
    for n_sh, m in ((1, 1), (3, 5), (8, 16)):
        ids = rng.integers(0, 1000, size=(n_sh, m)).astype(np.uint32)
        vals = rng.normal(size=(n_sh, m)).astype(np.float32)
        vals[0, 0] = np.nan
        if n_sh > 1:
            vals[1, m - 1] = vals[0, m - 1]                 # a tie: the lower index must win
        best_v = np.full(m, np.float32(-3.0e38)); best_i = np.zeros(m, np.int64)
        for r in range(n_sh):
            with np.errstate(invalid="ignore"):
                take = (vals[r] > best_v) | ((vals[r] == best_v) & (ids[r] < best_i))
            best_v = np.where(take, vals[r], best_v); best_i = np.where(take, ids[r], best_i)
        np.testing.assert_array_equal(pkg.fold_argmax_shards(ids, vals), best_i.astype(np.uint32))
    allnan = np.full((2, 3), np.nan, np.float32)
    np.testing.assert_array_equal(pkg.fold_argmax_shards(np.ones((2, 3), np.uint32), allnan), np.zeros(3, np.uint32))
