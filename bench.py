"""Benchmark of the quantized-matmul hot path on B200.

``python bench.py --gpus N --steps K --warmup W`` prints ONE JSON line.

Headline metric: dequant-GEMV HBM GB/s on the Q8_0 + Q6_K projection shapes of a
Qwen3-4B-class model (2560->9728, 9728->2560, 2560->151936), batch 1, f32
activations. One step = one pass over the six weights (six GEMV launches, 827.5 MB
of GGUF blocks, far larger than L2, so every step streams from HBM). Inputs are
seeded synthetic tensors (no model file, no dataset).

  value     whole-job GB/s with weights, x and y resident in HBM (CUDA graph of one
            step, replayed; CUDA events; max over ranks)
  e2e       the same metric through the public host API (gemv_batch with host
            buffers: H2D of every x and D2H of every y inside the timed region)
  roofline  the largest launch (Q8_0 2560->151936) timed alone against the measured
            HBM copy bandwidth
  cpu_baseline  the CPU oracle (the reference's qmatmul restated in C) on a bounded
            row sample, all host threads

With N > 1 (torchrun) every weight is row-sharded over the ranks and each GEMV is
followed by an NCCL all-gather of the output shards: strong scaling.

``--impl reference`` times the reference's CPU path (the oracle port: the Rust
reference cannot be built here) on a bounded sample of the same workload.
"""
import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
import __graft_entry__ as entry  # noqa: E402

Q8_0, Q6_K, Q4_0 = 8, 14, 2
SHAPES = [(2560, 9728), (9728, 2560), (2560, 151936)]          # (in_dim, out_dim)
WORKLOAD = [(ty, k, n) for ty in (Q8_0, Q6_K) for (k, n) in SHAPES]
BLOCK = {Q8_0: (32, 34), Q6_K: (256, 210), Q4_0: (32, 18)}
TYNAME = {Q8_0: "q8_0", Q6_K: "q6_k", Q4_0: "q4_0"}
GEN_ROWS = 8192   # synthetic rows generated per weight, tiled up to out_dim (keeps host set-up short)


WORKLOAD_NAME = "configs[1]: Q8_0+Q6_K dequant-GEMV, batch 1, 2560->9728, 9728->2560, 2560->151936"
REPLAYS = 64   # the GPU arm replays the step's CUDA graph this many times per timed step and divides (a step is 0.17 ms)


def bench_config():
    """The `config` object of both arms (the driver compares them)."""
    return {"workload": WORKLOAD_NAME,
            "l2": "inputs larger than L2 (827.5 MB of weights streamed per step)",
            "timing": "GPU arm: each timed step replays the step's CUDA graph %d times and divides, so that the timed "
                      "region lasts ~0.5 s; CPU arm: each step runs once on a bounded row sample" % REPLAYS}


def algo_bytes(ty, k, n):
    """Algorithmic bytes of one GEMV: GGUF blocks + f32 x + f32 y."""
    be, bb = BLOCK[ty]
    return n * (k // be) * bb + 4 * k + 4 * n


def make_weight(synth, ty, k, n, seed, name, row0=0, rows=None):
    """Rows [row0, row0+rows) of a seeded synthetic weight; big weights repeat a GEN_ROWS-row pattern."""
    rows = n if rows is None else rows
    be, bb = BLOCK[ty]
    bpr = k // be * bb
    base = synth.quant(ty, seed, name, min(n, GEN_ROWS), k).reshape(-1, bpr)
    idx = (np.arange(row0, row0 + rows) % base.shape[0])
    return np.ascontiguousarray(base[idx]).reshape(-1)


class ClockSampler:
    """Samples nvidia-smi clocks and throttle reasons while the timed region runs."""
    Q = ("clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.index, self.rows, self.p = index, [], None

    def start(self):
        try:
            self.p = subprocess.Popen(["nvidia-smi", "-i", str(self.index), "--query-gpu=" + self.Q,
                                       "--format=csv,noheader,nounits", "-lms", "100"],
                                      stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.t = threading.Thread(target=self._read, daemon=True)
            self.t.start()
        except OSError:
            self.p = None

    def _read(self):
        for line in self.p.stdout:
            self.rows.append([c.strip() for c in line.split(",")])

    def stop(self):
        if not self.p:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        time.sleep(0.15)
        self.p.terminate()
        try:
            self.p.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.p.kill()
        sm, mx, reasons = [], [], set()
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for r in self.rows:
            if len(r) < 6:
                continue
            try:
                sm.append(float(r[0]))
                mx.append(float(r[1]))
            except ValueError:
                continue
            for nm, v in zip(names, r[2:6]):
                if v.lower().startswith("active"):
                    reasons.add(nm)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": max(mx) if mx else None,
                "reasons": sorted(reasons), "samples": len(sm)}


def cpu_baseline(orc, synth, seconds=12.0):
    """The oracle's qmatmul on a bounded sample: the first rows of each of the six weights,
    sized from a calibration call so that the whole leg takes about `seconds`."""
    threads = orc.default_threads()
    x = {k: synth.normal(1, "cpu.x%d" % k, k) for k in (2560, 9728)}
    # calibrate on 512 rows of the first weight
    w = make_weight(synth, Q8_0, 2560, 9728, 1, "cpu.cal", 0, 512)
    t0 = time.perf_counter()
    orc.qmatmul(x[2560], w, Q8_0, 2560, 512, threads)
    per_byte = (time.perf_counter() - t0) / w.size
    budget_bytes = seconds / max(per_byte, 1e-12) / 2      # dequant cost varies by format; stay under budget
    total_full = sum(algo_bytes(ty, k, n) for ty, k, n in WORKLOAD)
    frac = min(1.0, budget_bytes / total_full)
    # when the whole workload fits the budget many times over, it is repeated (same rows) to fill it
    reps = 1 if frac < 1.0 else int(min(60, max(1, budget_bytes // total_full)))
    done_bytes, secs, sample = 0, 0.0, []
    for ty, k, n in WORKLOAD:
        rows = max(64, int(n * frac))
        rows = min(rows, n)
        w = make_weight(synth, ty, k, n, 1, "cpu.%d.%d.%d" % (ty, k, n), 0, rows)
        orc.qmatmul(x[k], w[: (k // BLOCK[ty][0]) * BLOCK[ty][1] * 8], ty, k, 8, threads)  # touch / warm
        t0 = time.perf_counter()
        for _ in range(reps):
            orc.qmatmul(x[k], w, ty, k, rows, threads)
        secs += time.perf_counter() - t0
        done_bytes += algo_bytes(ty, k, rows) * reps
        sample.append("%s %d->%d rows %d x%d" % (TYNAME[ty], k, n, rows, reps))
    return {"value": done_bytes / secs / 1e9, "unit": "GB/s", "cores": threads, "kind": "port",
            "sample": "first rows of each weight: " + "; ".join(sample), "seconds": round(secs, 2)}


def decode_chain_extra(pkg, synth, torch, device, stream):
    """configs[3]: Qwen3-4B-shaped projection chain (36 layers, hidden 2560, q 4096, kv 1024, ffn 9728,
    Q4_0 projections, Q6_K lm_head 2560->151936), batch 1; attention replaced by the q stand-in."""
    hidden, qdim, kvdim, ffn, vocab, n_layers = 2560, 4096, 1024, 9728, 151936, 36
    acc = pkg.CudaWeightAccel(device)
    out = {}
    try:
        shapes = {"attn_q": (qdim, hidden), "attn_k": (kvdim, hidden), "attn_v": (kvdim, hidden),
                  "attn_output": (hidden, qdim), "ffn_gate": (ffn, hidden), "ffn_up": (ffn, hidden),
                  "ffn_down": (hidden, ffn)}
        base = {nm: make_weight(synth, Q4_0, k, n, 3, "dc." + nm) for nm, (n, k) in shapes.items()}
        nbytes = 0
        for il in range(n_layers):
            for nm, (n, k) in shapes.items():
                # the same seeded bytes under every layer's name: the chain streams 36 distinct resident copies
                assert acc.upload_q4_0("blk.%d.%s.weight" % (il, nm), base[nm], k, n)
                nbytes += n * (k // 32) * 18
            for nn in ("attn_norm", "ffn_norm"):
                acc.upload_f32("blk.%d.%s.weight" % (il, nn), synth.norm_weight(3, "dc.%d.%s" % (il, nn), hidden))
        assert acc.upload_q6_k("output.weight", make_weight(synth, Q6_K, hidden, vocab, 3, "dc.head"), hidden, vocab)
        nbytes += vocab * (hidden // 256) * 210
        acc.upload_f32("output_norm.weight", synth.norm_weight(3, "dc.out_norm", hidden))
        h0 = synth.normal(3, "dc.h0", hidden)
        dev = torch.device("cuda", device)
        for act, name, chain in ((pkg.ACT_Q8DOT, "q8dot", 0), (pkg.ACT_Q8DOT, "q8dot_chain_kernel", 1), (pkg.ACT_F32, "f32", 0)):
            # chain = 1: the whole chain as ONE persistent launch (steps exchange {value, epoch} entries); 0: a launch per step
            acc.set_option("decode_chain", chain)
            acc.set_option("chain_trace", chain)
            assert acc.configure_decode(hidden, 32, ffn, vocab, n_layers, eps=1e-6, act=act)
            for _ in range(3):
                logits = acc.decode_step(h0, 0)
            t0 = time.perf_counter()
            reps = 20
            for i in range(reps):
                logits = acc.decode_step(h0, i)
            e2e_ms = (time.perf_counter() - t0) / reps * 1e3
            assert np.isfinite(logits).all()
            # greedy form: the argmax on the device, 4 bytes back instead of the logits
            tok = acc.decode_step_argmax(h0, 0)
            assert tok == int(np.argmax(logits))
            t0 = time.perf_counter()
            for i in range(reps):
                tok = acc.decode_step_argmax(h0, i)
            e2e_argmax_ms = (time.perf_counter() - t0) / reps * 1e3
            d_h = torch.from_numpy(h0).to(dev)
            d_h0 = d_h.clone()
            d_l = torch.empty(vocab, device=dev)
            with torch.cuda.stream(stream):
                s = stream.cuda_stream
                acc.decode_chain_dev(d_h.data_ptr(), d_l.data_ptr(), stream=s)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    d_h.copy_(d_h0)
                    acc.decode_chain_dev(d_h.data_ptr(), d_l.data_ptr(), stream=s)
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                a.record()
                for _ in range(reps):
                    g.replay()
                b.record()
                torch.cuda.synchronize()
                dev_ms = a.elapsed_time(b) / reps
            out[name] = {"ms_per_token": round(dev_ms, 4), "ms_per_token_e2e": round(e2e_ms, 4),
                         "ms_per_token_e2e_argmax": round(e2e_argmax_ms, 4),
                         "gbs": round(nbytes / dev_ms / 1e6, 1),
                         # (integer-dot form: the ffn-long row of every down projection is prepared by a launch of its own)
                         "launches_per_token": 1 if chain else 4 * n_layers + 1 + (n_layers if act == pkg.ACT_Q8DOT and ffn >= 8192 else 0)}
            tr = acc.decode_trace() if chain else None
            if tr is not None:
                # CTA 0's clocks per step: start, activations arrived, prologue done, last row group done, rows published
                tt = tr.astype(np.int64)
                phases = {}
                for kk, nm in enumerate(("qkv", "o", "gate_up", "down")):
                    idx = np.arange(kk + 4, len(tt) - 1, 4)
                    f = lambda a_, b_: round(float((tt[idx, b_] - tt[idx, a_]).mean()) / 1965.0, 2)  # noqa: E731
                    phases[nm] = {"wait_us": f(0, 1), "prologue_us": f(1, 2), "tiles_us": f(2, 3), "reduce_store_us": f(3, 4),
                                  "stalled_on_weights_us": round(float(tt[idx, 5].mean()) / 1965.0, 2)}
                out[name]["phases_cta0"] = phases
                out[name]["phases_note"] = "SM clocks of CTA 0 at 1965 MHz, mean over layers 1..35"
        acc.set_option("decode_chain", -1)
        acc.set_option("chain_trace", 0)
        out["bytes_per_token"] = nbytes
        # the same model as a real token step: QK-norm, NEOX rope, KV cache (32 heads, 8 KV heads of 128),
        # grouped-query softmax over the cache; the cache is seeded with random rows up to each position
        hd, n_kv, max_seq = 128, 8, 4096
        for il in range(n_layers):
            for nn in ("attn_q_norm", "attn_k_norm"):
                acc.upload_f32("blk.%d.%s.weight" % (il, nn), synth.norm_weight(3, "dc.%d.%s" % (il, nn), hd))
        if acc.configure_decode(hidden, 32, ffn, vocab, n_layers, eps=1e-6, act=pkg.ACT_Q8DOT, attn_standin_q=False,
                                head_dim=hd, n_kv=n_kv, rope_theta=1e6, max_seq=max_seq):
            real = []
            rows = synth.normal(3, "dc.kv", max_seq * kvdim).reshape(max_seq, kvdim)
            for il in range(n_layers):
                acc.seed_decode_kv(il, rows, rows)
            for pos in (0, 1024, max_seq - 1):
                for _ in range(3):
                    acc.decode_step_argmax(h0, pos)
                t0 = time.perf_counter()
                for _ in range(reps):
                    acc.decode_step_argmax(h0, pos)
                real.append({"pos": pos, "ms_per_token_e2e": round((time.perf_counter() - t0) / reps * 1e3, 4)})
            # speculative verify through the same model: 5 rows (gamma + 1) in one pass over the weights
            hs = synth.normal(3, "dc.hs", 5 * hidden)
            for _ in range(2):
                acc.verify(hs, 1024, 5)
            t0 = time.perf_counter()
            for _ in range(5):
                acc.verify(hs, 1024, 5)
            out["real_attention"] = {"q8dot_decode_step_argmax": real,
                                     "verify_5_rows_at_1024_ms": round((time.perf_counter() - t0) / 5 * 1e3, 4),
                                     "note": "whole token step through the host API (H2D of h, graph replay, "
                                             "argmax on the device, 4 bytes back); KV cache f32, 36 layers x 4096 rows"}
        out["note"] = "projection chain only; attention replaced by feeding Wo with q (no KV cache)"
    finally:
        acc.close()
    return out


def share_tensor(acc, dist, t, rank, world, opened):
    """Device pointers of every rank's copy of tensor t: the owner exports the CUDA IPC handle of the allocation
    (through torch, which knows its base) and the offset of t in it; the library opens each handle once, with this
    rank's device current. `opened`: (rank, handle) -> mapped base, shared between calls."""
    meta = t.untyped_storage()._share_cuda_()
    handle = bytes(meta[1])
    if len(handle) == 66 and handle[1:2] == b"c":
        handle = handle[2:]      # torch prefixes a version byte and a type byte ('c' = cudaMalloc)
    if len(handle) != 64:
        raise RuntimeError("torch exported a %d-byte handle: not a plain cudaMalloc allocation" % len(handle))
    mine = (handle, int(meta[3]) + t.storage_offset() * t.element_size())
    metas = [None] * world
    dist.all_gather_object(metas, mine)
    ptrs = []
    for r, (handle, offset) in enumerate(metas):
        if r == rank:
            ptrs.append(t.data_ptr())
            continue
        if (r, handle) not in opened:
            opened[(r, handle)] = acc.ipc_open(handle)
        ptrs.append(opened[(r, handle)] + offset)
    return ptrs


def check_peer_mappings(acc, dist, torch, named, ptrs, rank, world):
    """Every mapping is checked with a copy-engine read before any kernel stores through it: each rank leaves a mark
    in the last word of each of its buffers and reads its peers' marks. named: [(name, int32-viewable tensor)]."""
    marks = {}
    for i, (nm, t) in enumerate(named):
        marks[nm] = (t, 0x5EED0000 + 256 * i)
        t.view(torch.int32)[-1] = marks[nm][1] + rank
    torch.cuda.synchronize()
    dist.barrier()
    for nm, (t, mark) in marks.items():
        for r in range(world):
            got = acc.peek_u32(ptrs[nm][r] + 4 * (t.numel() - 1))
            if got != mark + r:
                raise RuntimeError("peer mapping of %s on rank %d reads %#x, expected %#x" % (nm, r, got, mark + r))
    dist.barrier()
    for nm, (t, mark) in marks.items():
        t.view(torch.int32)[-1] = 0
    torch.cuda.synchronize()
    dist.barrier()


def decode_chain_sharded_extra(pkg, synth, torch, dist, local, stream, rank, world):
    """configs[3] on `world` GPUs: every projection row-sharded, an NCCL all-gather after each sharded
    projection or group (q|k|v and gate|up gathered in one coalesced call each). Every rank runs this."""
    hidden, qdim, kvdim, ffn, vocab, n_layers = 2560, 4096, 1024, 9728, 151936, 36
    dev = torch.device("cuda", local)
    acc = pkg.CudaWeightAccel(local, rank=rank, world=world)
    out = {}
    try:
        shapes = {"attn_q": (qdim, hidden), "attn_k": (kvdim, hidden), "attn_v": (kvdim, hidden),
                  "attn_output": (hidden, qdim), "ffn_gate": (ffn, hidden), "ffn_up": (ffn, hidden),
                  "ffn_down": (hidden, ffn)}
        base = {nm: make_weight(synth, Q4_0, k, n, 3, "dc." + nm) for nm, (n, k) in shapes.items()}
        nbytes = 0
        norms = []
        for il in range(n_layers):
            for nm, (n, k) in shapes.items():
                assert acc.upload_q4_0("blk.%d.%s.weight" % (il, nm), base[nm], k, n)   # the library keeps its row shard
                nbytes += n * (k // 32) * 18
            nws = [synth.norm_weight(3, "dc.%d.%s" % (il, nn), hidden) for nn in ("attn_norm", "ffn_norm")]
            for nn, nw in zip(("attn_norm", "ffn_norm"), nws):
                acc.upload_f32("blk.%d.%s.weight" % (il, nn), nw)
            norms.append([torch.from_numpy(nw).to(dev) for nw in nws])
        assert acc.upload_q6_k("output.weight", make_weight(synth, Q6_K, hidden, vocab, 3, "dc.head"), hidden, vocab)
        nbytes += vocab * (hidden // 256) * 210
        out_norm_np = synth.norm_weight(3, "dc.out_norm", hidden)
        acc.upload_f32("output_norm.weight", out_norm_np)
        out_norm = torch.from_numpy(out_norm_np).to(dev)
        h0 = torch.from_numpy(synth.normal(3, "dc.h0", hidden)).to(dev)

        def full(n):
            return torch.zeros(n, device=dev)

        def shard(n):
            assert n % world == 0
            return torch.zeros(n // world, device=dev)

        h_full, q_full, k_full, v_full = full(hidden), full(qdim), full(kvdim), full(kvdim)
        g_full, u_full, lg_full = full(ffn), full(ffn), full(vocab)
        q_sh, k_sh, v_sh, h_sh, g_sh, u_sh, lg_sh = (shard(n) for n in (qdim, kvdim, kvdim, hidden, ffn, ffn, vocab))
        h_res = h_full[rank * (hidden // world):(rank + 1) * (hidden // world)]   # this rank's rows of the residual
        state = {"coalesce": True}

        def gather(pairs):
            if len(pairs) > 1 and state["coalesce"]:
                try:
                    with dist._coalescing_manager(device=dev):
                        for f, s_ in pairs:
                            dist.all_gather_into_tensor(f, s_)
                    return
                except Exception:
                    state["coalesce"] = False
            for f, s_ in pairs:
                dist.all_gather_into_tensor(f, s_)

        def chain(act):
            s = torch.cuda.current_stream().cuda_stream
            p = lambda t: t.data_ptr()  # noqa: E731
            for il in range(n_layers):
                b = "blk.%d." % il
                an, fn = norms[il]
                assert acc.gemv_dev([b + "attn_q.weight", b + "attn_k.weight", b + "attn_v.weight"], p(h_full),
                                    [p(q_sh), p(k_sh), p(v_sh)], d_b=p(an), eps=1e-6, pre=pkg.PRE_RMSNORM, act=act, stream=s)
                gather([(q_full, q_sh), (k_full, k_sh), (v_full, v_sh)])
                assert acc.gemv_dev([b + "attn_output.weight"], p(q_full), [p(h_sh)], act=act, stream=s, d_res=[p(h_res)])
                gather([(h_full, h_sh)])
                assert acc.gemv_dev([b + "ffn_gate.weight", b + "ffn_up.weight"], p(h_full), [p(g_sh), p(u_sh)],
                                    d_b=p(fn), eps=1e-6, pre=pkg.PRE_RMSNORM, act=act, stream=s)
                gather([(g_full, g_sh), (u_full, u_sh)])
                assert acc.gemv_dev([b + "ffn_down.weight"], p(g_full), [p(h_sh)], d_b=p(u_full), pre=pkg.PRE_SWIGLU,
                                    act=act, stream=s, d_res=[p(h_res)])
                gather([(h_full, h_sh)])
            assert acc.gemv_dev(["output.weight"], p(h_full), [p(lg_sh)], d_b=p(out_norm), eps=1e-6,
                                pre=pkg.PRE_RMSNORM, act=act, stream=s)
            gather([(lg_full, lg_sh)])

        # ---- fused form: the GEMV stores its rows into every rank's full vectors (peer-mapped memory), a
        #      flag barrier follows instead of a collective ----
        fused = {"ok": False, "why": ""}
        try:
            opened = {}

            def share(t):
                """device pointers of every rank's copy of tensor t: the owner exports the CUDA IPC handle of
                the allocation (through torch, which knows its base) and the offset of t in it; the library
                opens each handle once, with this rank's device current"""
                meta = t.untyped_storage()._share_cuda_()
                handle = bytes(meta[1])
                if len(handle) == 66 and handle[1:2] == b"c":
                    handle = handle[2:]      # torch prefixes a version byte and a type byte ('c' = cudaMalloc)
                if len(handle) != 64:
                    raise RuntimeError("torch exported a %d-byte handle: not a plain cudaMalloc allocation" % len(handle))
                mine = (handle, int(meta[3]) + t.storage_offset() * t.element_size())
                metas = [None] * world
                dist.all_gather_object(metas, mine)
                ptrs_ = []
                for r, (handle, offset) in enumerate(metas):
                    if r == rank:
                        ptrs_.append(t.data_ptr())
                        continue
                    if (r, handle) not in opened:
                        opened[(r, handle)] = acc.ipc_open(handle)
                    ptrs_.append(opened[(r, handle)] + offset)
                return ptrs_

            flags = torch.zeros(8, dtype=torch.int32, device=dev)
            epoch = torch.zeros(1, dtype=torch.int32, device=dev)
            ptrs = {nm: share(t) for nm, t in (("h", h_full), ("q", q_full), ("k", k_full), ("v", v_full),
                                               ("g", g_full), ("u", u_full), ("lg", lg_full), ("flags", flags))}
            # check every mapping with a copy-engine read before any kernel stores through it: each rank
            # leaves a mark in the last word of each of its buffers and reads its peers' marks
            marks = {}
            for i, (nm, t) in enumerate((("h", h_full), ("q", q_full), ("k", k_full), ("v", v_full), ("g", g_full),
                                         ("u", u_full), ("lg", lg_full), ("flags", flags))):
                marks[nm] = (t, 0x5EED0000 + 256 * i)
                t.view(torch.int32)[-1] = marks[nm][1] + rank
            torch.cuda.synchronize()
            dist.barrier()
            for nm, (t, mark) in marks.items():
                for r in range(world):
                    got = acc.peek_u32(ptrs[nm][r] + 4 * (t.numel() - 1))
                    if got != mark + r:
                        raise RuntimeError("peer mapping of %s on rank %d reads %#x, expected %#x" % (nm, r, got, mark + r))
            dist.barrier()
            for nm, (t, mark) in marks.items():
                t.view(torch.int32)[-1] = 0
            torch.cuda.synchronize()
            dist.barrier()
            fused["ok"] = True
        except Exception as ex:   # the NCCL form above stands on its own
            fused["why"] = "%s: %s" % (type(ex).__name__, ex)

        def chain_fused(act):
            s = torch.cuda.current_stream().cuda_stream
            p = lambda t: t.data_ptr()  # noqa: E731

            def bar():
                acc.peer_barrier_dev(p(epoch), p(flags), ptrs["flags"], stream=s)

            for il in range(n_layers):
                b = "blk.%d." % il
                an, fn = norms[il]
                assert acc.gemv_peers_dev([b + "attn_q.weight", b + "attn_k.weight", b + "attn_v.weight"], p(h_full),
                                          [ptrs["q"], ptrs["k"], ptrs["v"]], d_b=p(an), eps=1e-6, pre=pkg.PRE_RMSNORM,
                                          act=act, stream=s)
                bar()
                assert acc.gemv_peers_dev([b + "attn_output.weight"], p(q_full), [ptrs["h"]], act=act, stream=s,
                                          d_res=[p(h_res)])
                bar()
                assert acc.gemv_peers_dev([b + "ffn_gate.weight", b + "ffn_up.weight"], p(h_full), [ptrs["g"], ptrs["u"]],
                                          d_b=p(fn), eps=1e-6, pre=pkg.PRE_RMSNORM, act=act, stream=s)
                bar()
                assert acc.gemv_peers_dev([b + "ffn_down.weight"], p(g_full), [ptrs["h"]], d_b=p(u_full),
                                          pre=pkg.PRE_SWIGLU, act=act, stream=s, d_res=[p(h_res)])
                bar()
            assert acc.gemv_peers_dev(["output.weight"], p(h_full), [ptrs["lg"]], d_b=p(out_norm), eps=1e-6,
                                      pre=pkg.PRE_RMSNORM, act=act, stream=s)
            bar()

        # ---- chain-kernel form: ONE persistent launch per token and rank; every step publishes its rows into the
        #      exchange block of every rank (peer stores of {value, epoch} entries), no barrier, no collective ----
        ck = {"ok": False, "why": ""}
        try:
            if not acc.configure_decode(hidden, 32, ffn, vocab, n_layers, eps=1e-6, act=pkg.ACT_Q8DOT):
                raise RuntimeError("configure_decode declined on the sharded handle")
            base_ptr, nbytes_blk = acc.decode_exchange_info()
            metas = [None] * world
            dist.all_gather_object(metas, acc.ipc_export(base_ptr))
            blocks = [0 if r == rank else acc.ipc_open(metas[r]) for r in range(world)]
            # every mapping checked with a copy-engine read of a mark before any kernel stores through it
            acc.poke_u32(base_ptr + nbytes_blk - 4, 0x5EED7700 + rank)   # (the block's last 128 bytes are spare)
            dist.barrier()
            for r in range(world):
                if r != rank and acc.peek_u32(blocks[r] + nbytes_blk - 4) != 0x5EED7700 + r:
                    raise RuntimeError("exchange block of rank %d does not read back its mark" % r)
            dist.barrier()
            assert acc.decode_set_peers(blocks)
            ck["ok"] = True
        except Exception as ex:
            ck["why"] = "%s: %s" % (type(ex).__name__, ex)

        lg_ck = torch.zeros(vocab // world, device=dev)

        def chain_kernel(act):
            s = torch.cuda.current_stream().cuda_stream
            assert acc.decode_chain_dev(h_full.data_ptr(), lg_ck.data_ptr(), stream=s)

        variants = [("nccl", chain)] + ([("fused", chain_fused)] if fused["ok"] else []) + \
                   ([("chain_kernel", chain_kernel)] if ck["ok"] else [])
        logits_ref = None
        for vname, chain in variants:
          for act, name in ((pkg.ACT_Q8DOT, "q8dot"),):
            if rank == 0:
                sys.stderr.write("decode_chain_sharded: %s %s\n" % (vname, name))
                sys.stderr.flush()
            with torch.cuda.stream(stream):
                h_full.copy_(h0)
                chain(act)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    h_full.copy_(h0)
                    chain(act)
                for _ in range(3):
                    g.replay()
                torch.cuda.synchronize()
                dist.barrier()
                torch.cuda.synchronize()
                a, b2 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 20
                a.record()
                for _ in range(reps):
                    g.replay()
                b2.record()
                torch.cuda.synchronize()
                t = torch.tensor([a.elapsed_time(b2) / reps], device=dev)
                dist.all_reduce(t, op=dist.ReduceOp.MAX)
                ms = float(t.item())
            assert acc.device_status(stream.cuda_stream) == 0
            if vname == "chain_kernel":
                # another kernel (RMSNorm before the quantiser, SwiGLU in the epilogue): same integer-dot chain to
                # quantiser noise, this rank's shard of the logits against the NCCL form's
                mine = logits_ref[rank * (vocab // world):(rank + 1) * (vocab // world)]
                err = float((lg_ck - mine).norm() / mine.norm())
                assert bool(torch.isfinite(lg_ck).all()) and err < 2e-2, "chain kernel and NCCL chain disagree: %g" % err
                out["chain_kernel_vs_nccl_rel_l2"] = round(err, 6)
            else:
                assert bool(torch.isfinite(lg_full).all())
                if logits_ref is None:
                    logits_ref = lg_full.clone()
                else:   # same shards, same kernels: the two exchange forms must agree bit for bit
                    assert bool((lg_full == logits_ref).all()), "fused and NCCL chains disagree"
            phases = None
            if vname == "chain_kernel":
                # where a step's time goes on this many GPUs: rank 0's CTA 0 notes its clocks per step (a separate,
                # untimed pass: tracing costs ~10 %); all ranks run it, the chain needs everybody
                acc.set_option("chain_trace", 1)
                with torch.cuda.stream(stream):
                    for _ in range(3):
                        h_full.copy_(h0)
                        chain(act)
                    torch.cuda.synchronize()
                dist.barrier()
                tr = acc.decode_trace()
                acc.set_option("chain_trace", 0)
                if tr is not None and rank == 0:
                    tt = tr.astype(np.int64)
                    phases = {}
                    for kk, nm in enumerate(("qkv", "o", "gate_up", "down")):
                        idx = np.arange(kk + 4, len(tt) - 1, 4)
                        idx = idx[(tt[idx, 1] != 0) & (tt[idx, 2] != 0) & (tt[idx, 3] != 0)]   # steps in which CTA 0 had rows
                        if idx.size == 0:
                            phases[nm] = {"note": "CTA 0 of rank 0 holds no row group of this step on %d GPUs" % world}
                            continue
                        f = lambda a_, b_: round(float((tt[idx, b_] - tt[idx, a_]).mean()) / 1965.0, 2)  # noqa: E731
                        phases[nm] = {"wait_us": f(0, 1), "prologue_us": f(1, 2), "tiles_us": f(2, 3), "reduce_publish_us": f(3, 4),
                                      "step_us": f(0, 4)}
            out[vname + "_" + name] = {"ms_per_token": round(ms, 4), "gbs_aggregate": round(nbytes / ms / 1e6, 1),
                                       "gbs_per_gpu": round(nbytes / ms / 1e6 / world, 1),
                                       "launches_per_token": 1 if vname == "chain_kernel" else (4 * n_layers + 1) * (2 if vname == "fused" else 1),
                                       "collectives_per_token": 4 * n_layers + 1 if vname == "nccl" else 0}
            if phases:
                out[vname + "_" + name]["phases_cta0_rank0"] = phases
                out[vname + "_" + name]["phases_note"] = ("SM clocks of rank 0's CTA 0 at 1965 MHz, mean over layers 1..%d: waiting "
                                                          "for the step's activation row (all ranks' rows), quantising it, "
                                                          "this shard's tiles, reduction and stores to every rank" % (n_layers - 1))
        out["n_gpus"] = world
        out["bytes_per_token"] = nbytes
        out["note"] = ("row-sharded projections; nccl: all-gather after each projection or fused group (coalesced: %s); "
                       "fused: the GEMV stores its rows into every rank's vectors over peer memory, then a flag barrier "
                       "kernel (%s); chain_kernel: one persistent launch per token, steps publish {value, epoch} entries "
                       "into every rank's exchange block, consumers poll their own block (%s); attention replaced by "
                       "feeding Wo with q"
                       % (state["coalesce"], "ran" if fused["ok"] else "not run: " + fused["why"],
                          "ran" if ck["ok"] else "not run: " + ck["why"]))
    finally:
        acc.close()
    return out


def verify_rows_extra(pkg, synth, torch, device, stream, rank=0, world=1, bs=(1, 2, 4, 8)):
    """configs[4]: speculative-verify batched GEMV at Gemma-3-12B-class shapes (48 layers, hidden 3840,
    q 4096, kv 2048, ffn 15360, Q4_0), b activation rows; 6.05 GB of weights per step, row-sharded over
    `world` GPUs (every rank streams its shard of every weight; the rows are independent dot products, so this
    step has no exchange). Per-step latency is the slowest rank's; GB/s per GPU and aggregate."""
    hidden, qdim, kvdim, ffn, n_layers = 3840, 4096, 2048, 15360, 48
    acc = pkg.CudaWeightAccel(device, rank=rank, world=world)
    out = {"per_b": []}
    try:
        shapes = {"q": (qdim, hidden), "k": (kvdim, hidden), "v": (kvdim, hidden), "o": (hidden, qdim),
                  "gate": (ffn, hidden), "up": (ffn, hidden), "down": (hidden, ffn)}
        base = {nm: make_weight(synth, Q4_0, k, n, 4, "vr." + nm) for nm, (n, k) in shapes.items()}
        nbytes = 0
        for il in range(n_layers):
            for nm, (n, k) in shapes.items():
                assert acc.upload_q4_0("L%d.%s" % (il, nm), base[nm], k, n)     # the library keeps its row shard
                nbytes += n * (k // 32) * 18
        dev = torch.device("cuda", device)
        rows = {nm: acc.weight_info("L0." + nm)["rows"] for nm in shapes}
        for b in bs:
            xh = torch.randn(b, hidden, device=dev)
            xq_ = torch.randn(b, qdim, device=dev)
            xf = torch.randn(b, ffn, device=dev)
            y = {nm: torch.empty(b, max(rows[nm], 1), device=dev) for nm in shapes}

            def step(s):
                for il in range(n_layers):
                    p = "L%d." % il
                    acc.gemv_rows_dev([p + "q", p + "k", p + "v"], xh.data_ptr(), b,
                                      [y["q"].data_ptr(), y["k"].data_ptr(), y["v"].data_ptr()], act=pkg.ACT_Q8DOT, stream=s)
                    acc.gemv_rows_dev([p + "o"], xq_.data_ptr(), b, [y["o"].data_ptr()], act=pkg.ACT_Q8DOT, stream=s)
                    acc.gemv_rows_dev([p + "gate", p + "up"], xh.data_ptr(), b, [y["gate"].data_ptr(), y["up"].data_ptr()],
                                      act=pkg.ACT_Q8DOT, stream=s)
                    acc.gemv_rows_dev([p + "down"], xf.data_ptr(), b, [y["down"].data_ptr()], act=pkg.ACT_Q8DOT, stream=s)

            with torch.cuda.stream(stream):
                s = stream.cuda_stream
                step(s)
                torch.cuda.synchronize()
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=stream):
                    step(s)
                g.replay()
                torch.cuda.synchronize()
                if world > 1:
                    torch.distributed.barrier()
                    torch.cuda.synchronize()
                a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                reps = 5
                a.record()
                for _ in range(reps):
                    g.replay()
                e.record()
                torch.cuda.synchronize()
                ms = a.elapsed_time(e) / reps
                if world > 1:
                    tt = torch.tensor([ms], device=dev)
                    torch.distributed.all_reduce(tt, op=torch.distributed.ReduceOp.MAX)
                    ms = float(tt.item())
            out["per_b"].append({"b": b, "ms_per_step": round(ms, 4), "gbs_aggregate": round(nbytes / ms / 1e6, 1),
                                 "gbs_per_gpu": round(nbytes / ms / 1e6 / world, 1)})
        out["bytes_per_step"] = nbytes
        out["n_gpus"] = world
        assert acc.device_status() == 0
        out["note"] = ("int8-dot activations; projections only (4 launches per layer, plus one operand-preparation launch "
                       "each for b > 1), weights streamed once per step; row shards, no exchange")
    finally:
        acc.close()
    return out


def config0_extra(pkg, synth, torch, device, stream):
    """configs[0]: one Q4_0 dequant-GEMV, 4096 x 4096, batch 1 (9,469,952 algorithmic bytes). HBM figure: 40
    distinct resident copies of the weight (377 MB, three times L2) in rotation; L2 figure: one copy, repeated."""
    k = n = 4096
    copies = 40
    acc = pkg.CudaWeightAccel(device)
    out = {}
    try:
        w = make_weight(synth, Q4_0, k, n, 9, "c0")
        for i in range(copies):
            assert acc.upload_q4_0("c0.%d" % i, w, k, n)
        dev = torch.device("cuda", device)
        x = torch.from_numpy(synth.normal(9, "c0.x", k)).to(dev)
        y = torch.empty(n, device=dev)
        by = algo_bytes(Q4_0, k, n)
        for act, an in ((pkg.ACT_F32, "f32"), (pkg.ACT_Q8DOT, "q8dot")):
            for label, keys in (("hbm_40_copies", ["c0.%d" % i for i in range(copies)]), ("l2_resident", ["c0.0"] * copies)):
                with torch.cuda.stream(stream):
                    s = stream.cuda_stream
                    g = torch.cuda.CUDAGraph()
                    acc.gemv_dev([keys[0]], x.data_ptr(), [y.data_ptr()], act=act, stream=s)
                    torch.cuda.synchronize()
                    with torch.cuda.graph(g, stream=stream):
                        for kk in keys:
                            acc.gemv_dev([kk], x.data_ptr(), [y.data_ptr()], act=act, stream=s)
                    for _ in range(3):
                        g.replay()
                    torch.cuda.synchronize()
                    a, e = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
                    a.record()
                    for _ in range(10):
                        g.replay()
                    e.record()
                    torch.cuda.synchronize()
                    us = a.elapsed_time(e) * 1e3 / 10 / copies
                out["%s_%s" % (an, label)] = {"us_per_gemv": round(us, 3), "gbs": round(by / us / 1e3, 1)}
        out["algorithmic_bytes"] = by
        out["note"] = "back-to-back launches with programmatic dependent launch; one GEMV moves 9.4 MB (1.4 us of HBM time)"
    finally:
        acc.close()
    return out


def upload_extra(pkg, synth, device):
    """upload_q4_0 / upload_q8_0 / upload_q6_k of one 2560 -> 9728 weight: GGUF bytes per second of wall time
    (H2D of the borrowed host bytes + the repack kernel + the sync that ends the borrow)."""
    acc = pkg.CudaWeightAccel(device)
    out = {}
    try:
        for ty, up in ((Q4_0, acc.upload_q4_0), (Q8_0, acc.upload_q8_0), (Q6_K, acc.upload_q6_k)):
            w = make_weight(synth, ty, 2560, 9728, 8, "up.%d" % ty)
            up("up.%d" % ty, w, 2560, 9728)
            t0 = time.perf_counter()
            reps = 5
            for _ in range(reps):
                assert up("up.%d" % ty, w, 2560, 9728)
            dt = (time.perf_counter() - t0) / reps
            out[TYNAME[ty]] = {"mb": round(w.size / 1e6, 2), "ms": round(dt * 1e3, 3), "gbs": round(w.size / dt / 1e9, 2)}
        out["note"] = "host bytes are pageable numpy memory (as a caller's mmap slice would be)"
    finally:
        acc.close()
    return out


def run_reference(args):
    """--impl reference: the reference's CPU implementation of the path (oracle port), all host
    threads, each step a bounded row sample of the same six GEMVs."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    orc = entry.load_oracle()
    orc.build()
    entry.load_package()
    from strix_rs_b200 import synth
    threads = orc.default_threads()
    frac = 1.0 / 8.0   # ~100 MB per step: large enough that thread start-up does not weigh on the CPU's figure
    ws, xs = [], {k: synth.normal(1, "ref.x%d" % k, k) for k in (2560, 9728)}
    nbytes = 0
    for ty, k, n in WORKLOAD:
        rows = max(64, int(n * frac))
        ws.append((ty, k, rows, make_weight(synth, ty, k, n, 1, "ref.%d.%d.%d" % (ty, k, n), 0, rows)))
        nbytes += algo_bytes(ty, k, rows)

    def step():
        for ty, k, rows, w in ws:
            orc.qmatmul(xs[k], w, ty, k, rows, threads)

    for _ in range(args.warmup):
        step()
    t0 = time.perf_counter()
    for _ in range(args.steps):
        step()
    dt = (time.perf_counter() - t0) / args.steps
    val = nbytes / dt / 1e9
    sample = "rows/8 of each of the six weights per step (%d bytes)" % nbytes
    print(json.dumps({
        "impl": "reference", "metric": "dequant_gemv_hbm_gbs", "value": val, "unit": "GB/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt * 1e3, "higher_is_better": True,
        "scaling": "strong" if args.gpus > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": bench_config(), "sample": sample,
        "cpu_baseline": {"value": val, "unit": "GB/s", "cores": threads, "kind": "port", "sample": sample},
        "e2e": {"value": val, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3)
    if args.impl == "reference":
        return run_reference(args)

    import torch
    import torch.distributed as dist

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the backend has no CPU path")
    torch.cuda.set_device(local)
    dev = torch.device("cuda", local)
    cpu_group = None
    if world > 1:
        os.environ.setdefault("MASTER_ADDR", "127.0.0.1")
        # plain peer-to-peer NCCL: the gathers here are a few KB to 600 KB, and a rank that leaves while
        # its memory is bound to an NVLink multicast object can fault its peers
        os.environ.setdefault("NCCL_NVLS_ENABLE", "0")
        dist.init_process_group("nccl", device_id=dev)
        cpu_group = dist.new_group(backend="gloo")  # host-side rendezvous for the end of the run

    pkg = entry.load_package()
    from strix_rs_b200 import synth
    acc = pkg.CudaWeightAccel(local, rank=rank, world=world)

    # ---- set-up: upload this rank's row shard of the six weights -------------------------
    items = []
    for ty, k, n in WORKLOAD:
        key = "%s.%d.%d" % (TYNAME[ty], k, n)
        r0, r1 = pkg.shard_begin(n, world, rank), pkg.shard_begin(n, world, rank + 1)
        # the library slices its own shard out of the full tensor; hand it a buffer whose shard rows are real
        be, bb = BLOCK[ty]
        bpr = k // be * bb
        full = np.zeros(n * bpr, dtype=np.uint8) if world > 1 else None
        shard = make_weight(synth, ty, k, n, 1, key, r0, r1 - r0)
        if world > 1:
            full[r0 * bpr:r1 * bpr] = shard
        up = {Q8_0: acc.upload_q8_0, Q6_K: acc.upload_q6_k}[ty]
        assert up(key, full if world > 1 else shard, k, n), "upload declined: " + key
        del full, shard
        x_host = synth.normal(1, key + ".x", k)
        x = torch.from_numpy(x_host).to(dev)
        items.append(dict(key=key, ty=ty, k=k, n=n, x=x, x_host=x_host, rows=r1 - r0,
                          bytes=algo_bytes(ty, k, n)))
    step_bytes = sum(it["bytes"] for it in items)
    # The six outputs of a rank sit in ONE buffer (slots of ceil(n / world) floats), so that the step's
    # exchange is one all-gather: the six GEMVs of configs[1] do not depend on each other. (In the
    # decode chain every projection feeds the next one and is gathered on its own.)
    off = 0
    for it in items:
        it["off"] = off
        off += -(-it["n"] // world)
    y_mine = torch.zeros(off, device=dev)
    y_all = torch.zeros(world * off, device=dev) if world > 1 else y_mine
    for it in items:
        it["y"] = y_mine[it["off"]:it["off"] + it["rows"]]

    stream = torch.cuda.Stream(device=dev)

    # The six GEMVs do not depend on one another: the step is ONE gemv_batch_dev call (the trait's gemv_batch on
    # device vectors). The library runs a shard above 256 MiB as a launch of its own and the smaller ones side by
    # side in one launch (up to six problems; its CTAs dealt out among them). The same rule here, for the launch
    # count and the per-launch events: units = lists of items that share a launch.
    SMALL = 256 << 20
    def shard_bytes(it):
        be, bb = BLOCK[it["ty"]]
        return it["rows"] * (it["k"] // be) * bb
    small = [it for it in items if shard_bytes(it) <= SMALL]
    if len(small) < 2:
        small = []
    units = [[it] for it in items if not any(it is s_ for s_ in small)] + [small[i:i + 6] for i in range(0, len(small), 6)]

    def step_device(act=None):
        s = torch.cuda.current_stream().cuda_stream
        ok = acc.gemv_batch_dev([it["key"] for it in items], [it["x"].data_ptr() for it in items],
                                [it["y"].data_ptr() for it in items], act=pkg.ACT_F32 if act is None else act, stream=s)
        assert ok
        if world > 1:
            dist.all_gather_into_tensor(y_all, y_mine)

    def barrier():
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    # ---- resident-input throughput: one step captured in a CUDA graph, replayed ----------
    sampler = ClockSampler(local)

    def time_step(step_fn, sample_clocks):
        """ms per step of step_fn: W warm-up replays of its CUDA graph, then K x REPLAYS timed ones between barriers,
        CUDA events on the launching stream, the slowest rank's time."""
        with torch.cuda.stream(stream):
            for _ in range(2):
                step_fn()
            torch.cuda.synchronize()
            g_ = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g_, stream=stream):
                step_fn()
            for _ in range(args.warmup):
                g_.replay()
            barrier()
            if rank == 0 and sample_clocks:
                sampler.start()
            e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            barrier()
            e0.record()
            for _ in range(args.steps * REPLAYS):
                g_.replay()
            e1.record()
            barrier()
            ms_total = e0.elapsed_time(e1) / REPLAYS
        st_ = torch.tensor([acc.device_status()], device=dev)
        if world > 1:
            dist.all_reduce(st_, op=dist.ReduceOp.MAX)   # (every rank takes the same way out)
        if st_.item() != 0:
            if sample_clocks:
                raise SystemExit("device status word is non-zero: a bounded wait ran out")
            acc.clear_device_status()
            torch.cuda.synchronize()
            raise RuntimeError("a bounded wait ran out (device status %d)" % int(st_.item()))
        t = torch.tensor([ms_total], device=dev)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item()) / args.steps, g_

    ms_step, graph = time_step(step_device, True)
    exchange = None
    if world > 1:
        # The same step with the output exchange fused into the kernels: every rank's kernels store their rows
        # straight into the full output vectors of ALL ranks (plain stores into CUDA-IPC-mapped peer memory over
        # NVLink), and a one-warp flag barrier replaces the all-gather. Checked against the gathered result, bit
        # for bit; the faster form that checks out is the one reported as `value`.
        exchange = {"nccl_all_gather_ms_per_step": round(ms_step, 5), "peer_stores_ms_per_step": None, "form": "nccl all-gather"}
        try:
            foff, tot = [], 0
            for it in items:
                foff.append(tot)
                tot += (it["n"] + 31) & ~31
            y_full = torch.zeros(tot + 32, device=dev)
            flags = torch.zeros(8, dtype=torch.int32, device=dev)
            epoch = torch.zeros(1, dtype=torch.int32, device=dev)
            opened = {}
            ptrs = {"y": share_tensor(acc, dist, y_full, rank, world, opened),
                    "flags": share_tensor(acc, dist, flags, rank, world, opened)}
            check_peer_mappings(acc, dist, torch, [("y", y_full), ("flags", flags)], ptrs, rank, world)
            peer_ys = [[ptrs["y"][r] + 4 * foff[i] for r in range(world)] for i in range(len(items))]

            def step_peers():
                s = torch.cuda.current_stream().cuda_stream
                assert acc.gemv_batch_peers_dev([it["key"] for it in items], [it["x"].data_ptr() for it in items], peer_ys,
                                                act=pkg.ACT_F32, stream=s)
                acc.peer_barrier_dev(epoch.data_ptr(), flags.data_ptr(), ptrs["flags"], stream=s)

            ms_peers, graph_peers = time_step(step_peers, False)
            # the gathered result of the NCCL form, item by item, against what the peer stores left on this rank
            graph.replay()
            torch.cuda.synchronize()
            same = True
            for i, it in enumerate(items):
                per = -(-it["n"] // world)
                got = y_full[foff[i]:foff[i] + it["n"]]
                parts = [y_all[r * off + it["off"]:r * off + it["off"] + (pkg.shard_begin(it["n"], world, r + 1) - pkg.shard_begin(it["n"], world, r))]
                         for r in range(world)]
                same = same and bool(torch.equal(got, torch.cat(parts)))
                del per
            ok = torch.tensor([1 if same else 0], device=dev)
            dist.all_reduce(ok, op=dist.ReduceOp.MIN)
            exchange["peer_stores_ms_per_step"] = round(ms_peers, 5)
            exchange["peer_stores_equal_to_gathered"] = bool(ok.item())
            if ok.item() and ms_peers < ms_step:
                ms_step = ms_peers
                exchange["form"] = "peer stores + flag barrier"
            del graph_peers
        except Exception as ex:   # the NCCL form stands on its own
            exchange["why_not_peer_stores"] = "%s: %s" % (type(ex).__name__, ex)
    value = step_bytes / (ms_step * 1e-3) / 1e9

    # ---- end to end through the host API: host x in, host y out, one sync per step --------
    calls = [(it["key"], it["x_host"]) for it in items]
    # A quarter of a second of the same calls first: the loop then runs in the steady state of ITS OWN duty cycle (the
    # device idles while the host stages and copies), not in the power-capped state the replay region above leaves behind.
    t_warm = time.perf_counter()
    while time.perf_counter() - t_warm < 0.25:
        acc.gemv_batch(calls)
    barrier()
    t0 = time.perf_counter()
    e2e_steps = max(3, min(args.steps, 20))
    for _ in range(e2e_steps):
        ys = acc.gemv_batch(calls)
    dt = (time.perf_counter() - t0) / e2e_steps
    tt = torch.tensor([dt], device=dev)
    if world > 1:
        dist.all_reduce(tt, op=dist.ReduceOp.MAX)
    e2e_val = step_bytes / float(tt.item()) / 1e9
    h2d = sum(4 * it["k"] for it in items)
    d2h = sum(4 * int(y.size) for y in ys)
    clocks = sampler.stop() if rank == 0 else None

    # ---- per-launch durations inside the step (CUDA events around every launch) ---------------
    # The six launches run in the step's order, so each one finds L2 as it does in the timed region
    # (the 827 MB of the other weights have passed through it since its own last launch).
    roof = None
    detail = []
    if rank == 0:
        peaks = {}
        try:
            peaks = json.load(open(os.path.join(ROOT, "MEASURED_PEAKS.json")))
        except OSError:
            pass
        peak = float(peaks.get("hbm_gbs", 6650.0))
        peak_src = "measured" if "hbm_gbs" in peaks else "fallback"
        def unit_launch(u, s):
            ok = acc.gemv_batch_dev([it["key"] for it in u], [it["x"].data_ptr() for it in u], [it["y"].data_ptr() for it in u],
                                    act=pkg.ACT_F32, stream=s)
            assert ok
        with torch.cuda.stream(stream):
            s = stream.cuda_stream
            rounds = 20
            evs = [[(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in units]
                   for _ in range(rounds)]
            for _ in range(3):
                for u in units:
                    unit_launch(u, s)
            torch.cuda.synchronize()
            # (a few ms of device-side spinning first, so that the host has queued every launch before the
            # first one runs and no event pair includes a wait for the host)
            torch.cuda._sleep(20_000_000)
            for r in range(rounds):
                for i, u in enumerate(units):
                    evs[r][i][0].record()
                    unit_launch(u, s)
                    evs[r][i][1].record()
            torch.cuda.synchronize()
            for i, u in enumerate(units):
                by = sum(it["bytes"] * it["y"].numel() / it["n"] for it in u)
                us = statistics.median(evs[r][i][0].elapsed_time(evs[r][i][1]) for r in range(rounds)) * 1e3
                detail.append({"weight": " + ".join(it["key"] for it in u), "us": round(us, 2), "gbs": round(by / us / 1e3, 1)})
        # The kernels of the timed step: one instantiation of gemv_kernel per large weight (Q8_0 and Q6_K with the f32
        # row as int8 digits for K <= 8192, on f16 tiles beyond) and gemv_multi_kernel
        # for the weights that run side by side. The roofline is reported for the one with the largest share of the
        # step (these per-launch events; the ncu launch list under profiles/ gives the same order), on its largest
        # launch; the runner-up follows as second_kernel. DRAM traffic per launch from the ncu captures of
        # 65536-row cases, scaled by rows (traffic grows with rows).
        def kernel_of(u):
            if len(u) > 1:
                return "gemv_multi_kernel<%d weights side by side>" % len(u)
            it = u[0]
            if it["ty"] == Q8_0:
                return "gemv_kernel<Q8_0, f32 row as int8 digits>" if it["k"] <= 8192 else "gemv_kernel<Q8_0, f32 row on f16 tiles>"
            return "gemv_kernel<Q6_K, f32 row as int8 digits>" if it["k"] <= 8192 else "gemv_kernel<Q6_K, f32 row on f16 tiles>"
        share = {}
        for d, u in zip(detail, units):
            share[kernel_of(u)] = share.get(kernel_of(u), 0.0) + d["us"]
        order = sorted(share, key=lambda k_: -share[k_])
        traffic65536 = {Q8_0: 181.93e6, Q6_K: 141.15e6}   # dram__bytes_read.sum + dram__bytes_write.sum, 65536 x 2560

        def unit_bytes(u):
            return sum(it["bytes"] * it["y"].numel() / it["n"] for it in u)

        def roof_of(kname):
            cand = [(d, u) for d, u in zip(detail, units) if kernel_of(u) == kname]
            d, u = max(cand, key=lambda c: unit_bytes(c[1]))
            it = u[0]
            one = len(u) == 1 and world == 1 and it["k"] == 2560
            return {"kernel": "%s on %s, %s algorithmic bytes per launch" % (kname, d["weight"], format(int(unit_bytes(u)), ",")),
                    "achieved": d["gbs"], "frac": round(d["gbs"] / peak, 4),
                    "share_of_step": round(share[kname] / sum(share.values()), 3),
                    "traffic": int(traffic65536[it["ty"]] * it["n"] / 65536) if one else None}
        dom = roof_of(order[0])
        sec = roof_of(order[1]) if len(order) > 1 else None
        def frac_all(kname):
            """the instantiation over ALL its launches of the step: their algorithmic bytes / their summed durations"""
            cand = [(d, u) for d, u in zip(detail, units) if kernel_of(u) == kname]
            by = sum(unit_bytes(u) for _, u in cand)
            return round(by / sum(d["us"] for d, _ in cand) / 1e3 / peak, 4)
        roof = {"bound": "hbm", "achieved": dom["achieved"], "peak": peak, "unit": "GB/s", "frac": dom["frac"],
                "traffic": dom["traffic"], "kernel": dom["kernel"] + " (of %s peak)" % peak_src,
                "share_of_step": dom["share_of_step"], "frac_of_8tbs": round(dom["achieved"] / 8000.0, 4),
                "frac_over_all_launches_of_the_instantiation": frac_all(order[0]),
                "frac_of_the_whole_step": round(value / world / peak, 4),
                "second_kernel": dict(sec, frac_over_all_launches_of_the_instantiation=frac_all(order[1])) if sec else None,
                "launches_of_the_step": [{"kernel": kernel_of(u), "weights": d["weight"], "us": d["us"], "gbs": d["gbs"],
                                          "frac": round(d["gbs"] / peak, 4)} for d, u in zip(detail, units)]}

    # ---- extras on rank 0 at N=1: the integer-dot GEMV variant and the W8A8 GEMM (configs[2]) ----
    extras = None
    if rank == 0 and world == 1:
        extras = {"q8dot_gemv": [], "w8a8_gemm": []}
        with torch.cuda.stream(stream):
            s = stream.cuda_stream
            # The timed step once more as a 15 ms burst after a pause: the half-second timed region above runs at the
            # power cap (see `clocks`), where the step is bound by energy; the burst shows the same kernels at full clock.
            torch.cuda.synchronize()
            time.sleep(0.3)
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            for _ in range(3):
                graph.replay()
            a.record()
            for _ in range(100):
                graph.replay()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / 100
            extras["step_burst"] = {"ms_per_step": round(ms, 5), "gbs": round(step_bytes / ms / 1e6, 1),
                                    "frac_of_measured_peak": round(step_bytes / ms / 1e6 / peak, 4),
                                    "note": "the timed step, 100 graph replays after 0.3 s of idle (not power-capped)"}
            g = torch.cuda.CUDAGraph()
            with torch.cuda.graph(g, stream=stream):
                assert acc.gemv_batch_dev([it["key"] for it in items], [it["x"].data_ptr() for it in items],
                                          [it["y"].data_ptr() for it in items], act=pkg.ACT_Q8DOT, stream=s)
            for _ in range(3):
                g.replay()
            torch.cuda.synchronize()
            a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
            reps = 10
            a.record()
            for _ in range(reps):
                g.replay()
            b.record()
            torch.cuda.synchronize()
            ms = a.elapsed_time(b) / reps
            extras["q8dot_gemv"] = {"ms_per_step": round(ms, 5), "gbs": round(step_bytes / ms / 1e6, 1),
                                    "note": "same six weights, activation quantised per 32 to int8 inside the kernel"}
            for (k, n) in ((2560, 9728), (2560, 4096), (9728, 2560)):
                key = "gemm.%d.%d" % (k, n)
                assert acc.upload_q8_0(key, make_weight(synth, Q8_0, k, n, 2, key), k, n)
                for m in (512, 2048):
                    xg = torch.randn(m, k, device=dev)
                    yg = torch.empty(m, n, device=dev)
                    for _ in range(2):
                        acc.prefill_q8_gemm_dev(key, xg.data_ptr(), m, yg.data_ptr(), stream=s)
                    torch.cuda.synchronize()
                    gg = torch.cuda.CUDAGraph()
                    with torch.cuda.graph(gg, stream=stream):
                        for _ in range(10):
                            acc.prefill_q8_gemm_dev(key, xg.data_ptr(), m, yg.data_ptr(), stream=s)
                    gg.replay()
                    torch.cuda.synchronize()
                    a.record()
                    gg.replay()
                    b.record()
                    torch.cuda.synchronize()
                    us = a.elapsed_time(b) * 1e3 / 10
                    rec = {"M": m, "K": k, "N": n, "us": round(us, 1), "tops": round(2.0 * m * n * k / us / 1e6, 1)}
                    # the same kernel without the accumulator drain and loads (its hand-over loop alone), and the bare
                    # issue rate of tcgen05.mma kind::i8 (128 x 128 x 32 per instruction): the measured int8 peak
                    for mode, nm in ((3, "tops_handover_loop_only"), (4, "tops_mma_issue_only")):
                        acc.debug_gemm_mode_dev(key, xg.data_ptr(), m, yg.data_ptr(), mode, 2, stream=s)
                        torch.cuda.synchronize()
                        a.record()
                        acc.debug_gemm_mode_dev(key, xg.data_ptr(), m, yg.data_ptr(), mode, 10, stream=s)
                        b.record()
                        torch.cuda.synchronize()
                        rec[nm] = round(2.0 * m * n * k / (a.elapsed_time(b) * 1e3 / 10) / 1e6, 1)
                    extras["w8a8_gemm"].append(rec)
                    del xg, yg
        extras["w8a8_gemm_peaks"] = {
            "nominal_int8_dense_tops": 4500,
            "measured_mma_issue_only_tops": max(r["tops_mma_issue_only"] for r in extras["w8a8_gemm"]),
            "note": "tcgen05.mma kind::i8, 128 x 128 x 32 per instruction, operands in shared memory, issued back to back by "
                    "one thread per CTA: the rate the tensor pipe sustains at this instruction shape. The product needs a "
                    "fresh accumulator per 32 of K (per-block scales on both operands), and all of TMEM holds four of them"}
        extras["config0"] = config0_extra(pkg, synth, torch, local, stream)
        extras["upload"] = upload_extra(pkg, synth, local)
        extras["decode_chain"] = decode_chain_extra(pkg, synth, torch, local, stream)
        extras["verify_rows"] = verify_rows_extra(pkg, synth, torch, local, stream)
        if acc.device_status() != 0:
            raise SystemExit("device status word is non-zero after the extras")
        # the keys the N > 1 lines carry too, so that a curve over N can be read for them
        dc = extras["decode_chain"]
        extras["scaling_curve"] = {
            "decode_ms_per_token": min(dc["q8dot"]["ms_per_token"], dc["q8dot_chain_kernel"]["ms_per_token"]),
            "decode_form": "launch per step" if dc["q8dot"]["ms_per_token"] <= dc["q8dot_chain_kernel"]["ms_per_token"] else "chain kernel",
            "verify_rows": {"b%d" % r["b"]: r for r in extras["verify_rows"]["per_b"] if r["b"] in (1, 8)}}

    if world > 1:
        # configs[3] on all ranks: the row-sharded decode chain with an all-gather per projection
        sharded = decode_chain_sharded_extra(pkg, synth, torch, dist, local, stream, rank, world)
        vr = verify_rows_extra(pkg, synth, torch, local, stream, rank, world, bs=(1, 8))
        if rank == 0:
            forms = {k_: v_["ms_per_token"] for k_, v_ in sharded.items() if isinstance(v_, dict) and "ms_per_token" in v_}
            best = min(forms, key=forms.get)
            extras = {"decode_chain_sharded": sharded, "verify_rows_sharded": vr,
                      "scaling_curve": {"decode_ms_per_token": forms[best], "decode_form": best,
                                        "verify_rows": {"b%d" % r["b"]: r for r in vr["per_b"]}}}

    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        orc = entry.load_oracle()
        orc.build()
        cpu = cpu_baseline(orc, synth)

    if rank == 0:
        out = {
            "metric": "dequant_gemv_hbm_gbs", "value": round(value, 2), "unit": "GB/s", "n_gpus": world,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": round(ms_step, 5), "higher_is_better": True,
            "scaling": "strong" if world > 1 else "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
            "config": bench_config(), "bytes_per_step": step_bytes, "replays_per_step": REPLAYS,
            "parallelism": "rows sharded over %d GPU(s)%s" % (
                world, ", outputs exchanged once per step (%s)" % exchange["form"] if world > 1 else ""),
            "exchange": exchange,
            "e2e": {"value": round(e2e_val, 2), "unit": "GB/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": d2h},
            # (with the fused exchange the flag-barrier kernel is one more launch of ours per step)
            "gpu_launches": args.steps * REPLAYS * (len(units) + (1 if exchange and exchange["form"].startswith("peer") else 0)),
            "launches_per_step": len(units) + (1 if exchange and exchange["form"].startswith("peer") else 0),
            "clocks": clocks, "roofline": roof, "cpu_baseline": cpu, "per_weight": detail, "extras": extras,
            "frac_of_8tbs": round(value / 8000.0, 4),
        }
        print(json.dumps(out))
    sys.stdout.flush()
    if world > 1:
        # Leave together and without NCCL teardown: destroying the process group after CUDA graphs that
        # captured collectives have run was seen to block for ever on this stack. All GPU work is done
        # (synchronised above); the ranks meet on the host, then exit.
        del graph
        torch.cuda.synchronize()
        dist.barrier(group=cpu_group)
        sys.stderr.flush()
        os._exit(0)
    acc.close()


if __name__ == "__main__":
    main()
