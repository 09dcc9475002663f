"""The speculative-decoding callers (include/strix_spec.h) against a Python restatement of the reference's loops
(crates/strix-cli/src/commands/generate.rs:597-668 n-gram lookup; :848-899 draft model)."""
import numpy as np
import pytest


@pytest.fixture(scope="module")
def spec(pkg):
    import importlib
    return importlib.import_module("strix_rs_b200.spec")


def ref_propose(ctx, gamma):
    """generate.rs:621-638, line for line in Python."""
    for n in (3, 2, 1):
        if len(ctx) < n + 1:
            continue
        pat = ctx[len(ctx) - n:]
        for st in range(len(ctx) - n - 1, -1, -1):
            if ctx[st:st + n] == pat:
                cont = ctx[st + n:min(st + n + gamma, len(ctx) - 1)]
                if cont:
                    return cont
    return []


def test_ngram_proposer_matches_the_reference_loop(spec):
    rng = np.random.default_rng(3)
    assert spec.propose_ngram([], 3) == [] and spec.propose_ngram([5], 3) == []
    assert spec.propose_ngram([1, 2, 3, 1, 2, 3, 1, 2], 3) == [3, 1]              # trigram (3,1,2) seen at 2: what followed, cut before the last token
    assert spec.propose_ngram([7, 8, 9, 7], 3) == [8, 9]                          # unigram match, cut before the last token
    assert spec.propose_ngram([4, 4], 3) == []                                    # the only continuation would be the last token itself
    for _ in range(300):
        n = int(rng.integers(1, 60))
        ctx = [int(t) for t in rng.integers(0, 6, size=n)]                        # a small alphabet: many repeats
        gamma = int(rng.integers(1, 6))
        assert spec.propose_ngram(ctx, gamma) == ref_propose(ctx, gamma), (ctx, gamma)


def test_acceptance_and_gate(spec):
    assert spec.accept([5, 6, 7], [5, 6, 9, 1], 10) == (2, 9)                      # two agree, 9 corrects
    assert spec.accept([5, 6, 7], [5, 6, 7, 4], 10) == (3, 4)                      # all agree: the bonus token
    assert spec.accept([5, 6, 7], [1, 6, 7, 4], 10) == (0, 1)
    assert spec.accept([5, 6, 7], [5, 6, 7, 4], 1) == (1, 6)                       # room for one accepted token only
    assert spec.accept([], [3], 10) == (0, 3)
    g = spec.Gate()
    for _ in range(3):
        spec.gate_round(g, 0)
        assert not spec.gate_plain(g)
    spec.gate_round(g, 2)                                                           # an accepted token resets the count
    for _ in range(4):
        spec.gate_round(g, 0)
    assert sum(1 for _ in range(200) if spec.gate_plain(g)) == 96                   # 96 plain steps, then speculation again
    assert g.zero_rounds == 0 and g.plain_left == 0


def _model(pkg, synth, acc, seed, hidden, hd, n_heads, n_kv, ffn, vocab, n_layers, max_seq):
    qdim, kvdim = n_heads * hd, n_kv * hd
    for il in range(n_layers):
        b = "blk.%d." % il
        for nm, (n, k) in (("attn_q", (qdim, hidden)), ("attn_k", (kvdim, hidden)), ("attn_v", (kvdim, hidden)),
                           ("attn_output", (hidden, qdim)), ("ffn_gate", (ffn, hidden)), ("ffn_up", (ffn, hidden)),
                           ("ffn_down", (hidden, ffn))):
            assert acc.upload_q4_0(b + nm + ".weight", synth.q4_0(seed, b + nm, n, k), k, n)
        for nm, n in (("attn_norm", hidden), ("ffn_norm", hidden), ("attn_q_norm", hd), ("attn_k_norm", hd)):
            acc.upload_f32(b + nm + ".weight", synth.norm_weight(seed, b + nm, n))
    assert acc.upload_q8_0("output.weight", synth.q8_0(seed, "head", vocab, hidden, d_lo=0.01, d_hi=0.05), hidden, vocab)
    acc.upload_f32("output_norm.weight", synth.norm_weight(seed, "out_norm", hidden))
    assert acc.configure_decode(hidden, n_heads, ffn, vocab, n_layers, eps=1e-6, act=pkg.ACT_F32, attn_standin_q=False,
                                head_dim=hd, n_kv=n_kv, rope_theta=1e4, max_seq=max_seq)
    return synth.normal(seed, "embed", vocab, hidden)


@pytest.mark.gpu
@pytest.mark.parametrize("same_draft", [True, False])
def test_speculation_is_lossless(pkg, synth, spec, same_draft):
    """Greedy speculation must emit exactly the tokens plain greedy decoding of the target emits: with a draft equal
    to the target (everything accepted), with an unrelated draft (almost nothing accepted), and with the n-gram
    lookup proposer driving strix_cuda_verify_argmax."""
    hidden, hd, n_heads, n_kv, ffn, vocab, max_seq = 256, 64, 4, 2, 512, 300, 96
    target, draft, plain = pkg.CudaWeightAccel(0), pkg.CudaWeightAccel(0), pkg.CudaWeightAccel(0)
    try:
        Et = _model(pkg, synth, target, 21, hidden, hd, n_heads, n_kv, ffn, vocab, 2, max_seq)
        _model(pkg, synth, plain, 21, hidden, hd, n_heads, n_kv, ffn, vocab, 2, max_seq)
        Ed = _model(pkg, synth, draft, 21 if same_draft else 22, hidden, hd, n_heads, n_kv, ffn, vocab, 2 if same_draft else 1, max_seq)
        n_tokens, first = 40, 17
        # plain greedy decoding of the target
        want, t = [first], first
        for pos in range(n_tokens):
            t = plain.decode_step_argmax(Et[t], pos)
            want.append(t)
        # draft-model rounds
        got, cur, pos, rounds, accepted = [], first, 0, 0, 0
        gamma = 4
        while len(got) < n_tokens - gamma:
            toks, nxt = spec.spec_round(target, draft, Et, Ed, cur, pos, gamma)
            got += toks
            pos += len(toks)
            accepted += len(toks) - 1
            rounds += 1
            cur = nxt
        assert got == want[:len(got)], (got, want)
        print("draft %s: %d rounds, %d of %d drafts accepted" % ("= target" if same_draft else "unrelated", rounds, accepted, rounds * gamma))
        if same_draft:
            assert accepted == rounds * gamma
        # n-gram lookup rounds on a fresh cache: propose from history, verify in one batched pass, accept the agreeing prefix
        ctx, nxt, pos, out = [first], None, 0, []
        cur = first
        while len(out) < n_tokens - 4:
            prop = spec.propose_ngram(ctx, 3)
            cand = [cur] + prop
            am = spec.verify_argmax(plain, np.stack([Et[c] for c in cand]), pos, len(cand))
            n, nxt = spec.accept(prop, am, 100)
            out += [cur] + prop[:n]
            ctx += prop[:n] + [nxt]
            pos += n + 1
            cur = nxt
        assert out == want[:len(out)]
        assert target.device_status() == 0 and draft.device_status() == 0 and plain.device_status() == 0
    finally:
        target.close(); draft.close(); plain.close()
