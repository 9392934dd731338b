// Greedy speculative decoding with the draft loop, the verify pass and the cache reconciliation inside the library.
//
// The reference's round (crates/sapient-generate/src/speculative.rs:523-631) drafts k tokens with k single-token
// forwards of the draft model, scores them with one k-row forward of the target (forward_all_logits_cached), then
// appends the corrected / bonus token with one more single-token target forward and replays the committed tokens
// through the draft — every forward returning full-vocabulary logits to the host. With greedy sampling (the
// temperature-0 case of its accept rule: a draft is kept exactly when it is the target's arg-max, the corrected token
// is the target's arg-max) the same tokens come out of a cheaper schedule, which is what this file runs:
//   * the token committed last (`pending`) has not been fed to either model yet;
//   * draft: k steps of the device-resident greedy loop starting from `pending` (no logits leave the device);
//   * target: ONE forward of the k + 1 rows [pending, d1 .. dk] — each weight matrix is streamed once for all rows —
//     returning only the k + 1 arg-max ids a0 .. ak (last maximum wins, sampler.rs:161-168);
//   * accept the longest prefix with d(i+1) == a(i); commit those drafts and a(n), which becomes the next `pending`;
//   * roll both caches back to the committed tokens (truncate is O(1) on the paged cache); when every draft was
//     accepted the draft model consumes dk, which it had produced but not read.
// The committed stream equals the target's own greedy decoding token for token; per round the host sees k + (k + 1)
// token ids instead of 2k + 2 logit vectors.
#include <algorithm>
#include <vector>

#include "engine.h"

namespace sp {

int spec_greedy(Engine* target, Engine* draft, const uint32_t* prompt, size_t n_prompt, int k, size_t max_new, const uint32_t* eos,
                int n_eos, uint32_t* tokens_out, size_t* n_out, uint64_t* stats) {
    if (!target || !draft || !prompt || n_prompt == 0 || !tokens_out || !n_out) { set_error("spec_greedy: null or empty argument"); return SP_ERR_ARG; }
    if (k < 1 || k > 15) { set_error("spec_greedy: draft length must be in 1..15"); return SP_ERR_ARG; }
    if (target->d.vocab != draft->d.vocab) { set_error("spec_greedy: target and draft vocabularies differ"); return SP_ERR_ARG; }
    if (target->d.tp_size > 1 || draft->d.tp_size > 1) { set_error("spec_greedy: tensor-parallel engines are not supported"); return SP_ERR_ARG; }
    *n_out = 0;
    uint64_t rounds = 0, drafted = 0, accepted = 0;
    auto is_eos = [&](uint32_t t) { for (int i = 0; i < n_eos; ++i) if (eos[i] == t) return true; return false; };
    int st;
    if ((st = target->reset(0)) != SP_OK || (st = draft->reset(0)) != SP_OK) return st;
    std::vector<int32_t> zeros(std::max<size_t>(n_prompt, (size_t)k + 1), 0);
    // spec_prefill (:499-513): both models consume the prompt; the target's pick is the first generated token
    uint32_t pending = 0;
    if ((st = target->forward(prompt, zeros.data(), (int64_t)n_prompt, false, nullptr, &pending)) != SP_OK) return st;
    if ((st = draft->forward(prompt, zeros.data(), (int64_t)n_prompt, false, nullptr, nullptr)) != SP_OK) return st;
    size_t count = 0;
    if (max_new > 0) tokens_out[count++] = pending;
    bool stop = max_new == 0 || is_eos(pending);
    std::vector<uint32_t> d((size_t)k), rows((size_t)k + 1), picks((size_t)k + 1);
    const int32_t slot0 = 0;
    while (!stop && count < max_new) {
        const int L = target->seq_len[0];  // committed tokens held by both caches
        // room for pending + k drafts in both windows, else a shorter round
        int kk = std::min<int>(k, std::min(target->d.max_ctx, draft->d.max_ctx) - L - 1);
        if (kk < 1) { set_error("spec_greedy: KV cache full"); *n_out = count; return SP_ERR_KV_FULL; }
        if ((st = draft->decode_greedy(&pending, &slot0, 1, kk, d.data())) != SP_OK) return st;
        rows[0] = pending;
        for (int i = 0; i < kk; ++i) rows[(size_t)i + 1] = d[(size_t)i];
        if ((st = target->forward(rows.data(), zeros.data(), kk + 1, true, nullptr, picks.data())) != SP_OK) return st;
        int n = 0;
        while (n < kk && d[(size_t)n] == picks[(size_t)n]) ++n;
        ++rounds;
        drafted += (uint64_t)kk;
        accepted += (uint64_t)n;
        // commit d1 .. dn and the target's own pick after them
        for (int i = 0; i <= n && count < max_new && !stop; ++i) {
            const uint32_t t = i < n ? d[(size_t)i] : picks[(size_t)n];
            tokens_out[count++] = t;
            stop = is_eos(t);
        }
        pending = picks[(size_t)n];
        size_t kept = 0;
        if ((st = target->truncate(0, (size_t)(L + 1 + n), &kept)) != SP_OK) return st;
        if (n < kk) {
            if ((st = draft->truncate(0, (size_t)(L + 1 + n), &kept)) != SP_OK) return st;
        } else if (!stop && count < max_new) {
            // every draft accepted: the draft model has produced dk but not consumed it
            if ((st = draft->forward(&d[(size_t)kk - 1], zeros.data(), 1, false, nullptr, nullptr)) != SP_OK) return st;
        }
    }
    *n_out = count;
    if (stats) { stats[0] = rounds; stats[1] = drafted; stats[2] = accepted; }
    return SP_OK;
}

}  // namespace sp
