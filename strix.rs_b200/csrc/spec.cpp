// Speculative-decoding callers of the batched verify path: the n-gram lookup proposer, greedy acceptance,
// the lookup loop's utility gate, and a draft-model round driven on two accelerators. Host code.
// Reference: crates/strix-cli/src/commands/generate.rs:597-668 (lookup), :848-899 (draft model).
#include <cstring>
#include <vector>

#include "strix_spec.h"

extern "C" {

size_t strix_spec_propose_ngram(const uint32_t *ctx, size_t n_ctx, size_t gamma, uint32_t *out) {
    if (!ctx || !out || gamma == 0) return 0;
    for (size_t n = 3; n >= 1; n--) {
        if (n_ctx < n + 1) continue;
        const uint32_t *pat = ctx + n_ctx - n;
        // candidate starts n_ctx - n - 1 down to 0: the latest earlier occurrence first
        for (size_t st = n_ctx - n; st-- > 0;) {
            if (memcmp(ctx + st, pat, n * sizeof(uint32_t)) != 0) continue;
            const size_t from = st + n;
            size_t to = from + gamma;
            if (to > n_ctx - 1) to = n_ctx - 1;  // never past the context's last token
            if (to > from) {
                memcpy(out, ctx + from, (to - from) * sizeof(uint32_t));
                return to - from;
            }
        }
    }
    return 0;
}

size_t strix_spec_accept(const uint32_t *proposal, size_t n_prop, const uint32_t *argmax, size_t room, uint32_t *next) {
    size_t acc = 0;
    while (acc < n_prop && acc < room && argmax[acc] == proposal[acc]) acc++;
    if (next) *next = argmax[acc];
    return acc;
}

int strix_spec_gate_plain(strix_spec_gate *g) {
    if (!g || g->plain_left == 0) return 0;
    g->plain_left--;
    return 1;
}

void strix_spec_gate_round(strix_spec_gate *g, size_t accepted) {
    if (!g) return;
    if (accepted == 0) {
        if (++g->zero_rounds >= 4) {
            g->zero_rounds = 0;
            g->plain_left = 96;
        }
    } else {
        g->zero_rounds = 0;
    }
}

int strix_cuda_spec_round(strix_cuda *target, strix_cuda *draft, strix_embed_fn embed_target, void *user_target,
                          strix_embed_fn embed_draft, void *user_draft, size_t hidden_target, size_t hidden_draft,
                          uint32_t cur, size_t pos, size_t gamma, uint32_t *out_tokens, uint32_t *next) {
    if (!target || !draft || !embed_target || !embed_draft || !out_tokens || !next || gamma == 0) return -1;
    if (gamma + 1 > strix_cuda_prefill_max(target)) return 0;
    std::vector<float> hd(hidden_draft), ht((gamma + 1) * hidden_target);
    std::vector<uint32_t> drafts(gamma), am(gamma + 1);
    // the draft proposes gamma tokens, forwarding cur, d0 .. d(gamma-2) into its cache
    uint32_t d = cur;
    for (size_t i = 0; i < gamma; i++) {
        embed_draft(user_draft, d, hd.data());
        const int rc = strix_cuda_decode_step_argmax(draft, hd.data(), pos + i, &d);
        if (rc <= 0) return rc;
        drafts[i] = d;
    }
    {   // ... and the last draft too (its successor is not needed: only the cache row)
        uint32_t ignored;
        embed_draft(user_draft, drafts[gamma - 1], hd.data());
        const int rc = strix_cuda_decode_step_argmax(draft, hd.data(), pos + gamma, &ignored);
        if (rc <= 0) return rc;
    }
    // the target verifies [cur, d0 .. d(gamma-1)] in one batched pass: gamma + 1 greedy tokens
    embed_target(user_target, cur, ht.data());
    for (size_t i = 0; i < gamma; i++) embed_target(user_target, drafts[i], ht.data() + (i + 1) * hidden_target);
    const int rc = strix_cuda_verify_argmax(target, ht.data(), pos, gamma + 1, am.data());
    if (rc <= 0) return rc;
    const size_t n = strix_spec_accept(drafts.data(), gamma, am.data(), gamma, next);
    out_tokens[0] = cur;
    for (size_t i = 0; i < n; i++) out_tokens[1 + i] = drafts[i];
    return (int)(n + 1);
}

}  // extern "C"
