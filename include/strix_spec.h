/*
 * strix_spec.h -- the speculative-decoding callers of the batched verify path (the reference keeps them in its
 * CLI: crates/strix-cli/src/commands/generate.rs:597-668 n-gram lookup, :848-899 draft model). Host-side logic
 * plus one driver that runs a draft-model round on two accelerators. Greedy, hence lossless: the tokens that
 * come out are the ones plain greedy decoding of the target would have produced.
 */
#ifndef STRIX_SPEC_H
#define STRIX_SPEC_H

#include <stddef.h>
#include <stdint.h>

#include "strix_cuda.h"

#ifdef __cplusplus
extern "C" {
#endif

/* n-gram lookup proposer (generate.rs:621-638): the longest suffix of ctx (3, then 2, then 1 tokens) that also
 * occurs earlier in ctx, latest occurrence first; the proposal is what followed it there, at most `gamma` tokens
 * and never past the context's last token. Returns the number of proposed tokens written to out (0 = none). */
STRIX_API size_t strix_spec_propose_ngram(const uint32_t *ctx, size_t n_ctx, size_t gamma, uint32_t *out);

/* Greedy acceptance (generate.rs:644-651, 873-878): argmax[i] is the target's greedy token after the i-th verified
 * row (row 0 = the current token, row i = proposal[i-1]), n_prop + 1 entries. The accepted prefix is the longest
 * one with argmax[i] == proposal[i], cut so that at most `room` tokens are accepted; *next receives argmax[accepted]
 * (the correction, or the bonus token when everything was accepted). Returns the number of accepted proposals. */
STRIX_API size_t strix_spec_accept(const uint32_t *proposal, size_t n_prop, const uint32_t *argmax, size_t room,
                                   uint32_t *next);

/* The lookup loop's utility gate (generate.rs:604-607, 659-667): four rounds in a row without an accepted token switch
 * speculation off for the next 96 tokens. Zero-initialise. */
typedef struct strix_spec_gate {
    uint32_t zero_rounds, plain_left;
} strix_spec_gate;
/* 1 = take a plain decode step now (and count it), 0 = speculate. */
STRIX_API int strix_spec_gate_plain(strix_spec_gate *g);
STRIX_API void strix_spec_gate_round(strix_spec_gate *g, size_t accepted);

/* Token -> embedded hidden state of a model (the accelerator's decode entry points take hidden states). */
typedef void (*strix_embed_fn)(void *user, uint32_t token, float *hidden_out);

/* One round of draft-model speculation (generate.rs:858-895). The draft decodes gamma tokens greedily starting from
 * `cur` at position pos (its cache receives cur, d0 .. d(gamma-1)), the target verifies [cur, d0 .. d(gamma-1)] in ONE
 * batched pass (strix_cuda_verify_argmax), the longest agreeing prefix is accepted. out_tokens receives cur followed by
 * the accepted drafts; *next the token that carries into the next round, which starts at position pos + returned count
 * (rows past it in both caches are simply written again). gamma + 1 <= strix_cuda_prefill_max(target).
 * Returns the number of tokens written to out_tokens (accepted + 1), 0 if an accelerator declined, <0 on error
 * (text on the handle that failed). */
STRIX_API int strix_cuda_spec_round(strix_cuda *target, strix_cuda *draft, strix_embed_fn embed_target, void *user_target,
                                    strix_embed_fn embed_draft, void *user_draft, size_t hidden_target,
                                    size_t hidden_draft, uint32_t cur, size_t pos, size_t gamma, uint32_t *out_tokens,
                                    uint32_t *next);

#ifdef __cplusplus
}
#endif
#endif /* STRIX_SPEC_H */
