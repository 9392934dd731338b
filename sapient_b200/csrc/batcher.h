// Continuous batching over the paged KV cache: requests arrive at any time, are admitted into free sequence slots as
// soon as the page pool can hold them, prefill in bounded chunks between decode steps, decode together one token per
// step, and leave as they finish — the batch never waits for its slowest member. Prompt prefixes are shared: the pages
// of finished (and of running, already prefilled) sequences stay in a prefix index keyed by their token content, and a
// new request whose prompt starts with the same tokens becomes a reader of those pages instead of recomputing them.
//
// The reference serves one sequence per engine; its pipeline re-uses a prefix only against the previous prompt of the
// same conversation (crates/sapient-generate/src/pipeline.rs:818-830) and lists batching as future work
// (docs/ROADMAP.md:312). Sampling here is the greedy rule of its sampler (last maximum wins, sampler.rs:161-168), so a
// request's tokens equal what the engine produces for that prompt alone.
#pragma once
#include <stdint.h>

#include <deque>
#include <map>
#include <unordered_map>
#include <vector>

#include "page_pool.h"

namespace sp {

// What the scheduler needs from an engine. The CUDA engine implements it (batcher.cu); tests of the scheduling logic
// that run without a GPU use a host stand-in with the same page bookkeeping.
class SeqBackend {
  public:
    virtual ~SeqBackend() {}
    virtual int max_slots() const = 0;
    virtual int max_ctx() const = 0;
    virtual int max_step_rows() const = 0;  // rows one decode step may carry
    virtual PagePool& pool() = 0;
    virtual int seq_len(int slot) const = 0;
    // Appends ids[0..n) to `slot`; when argmax is not null it receives the greedy pick after the last token.
    virtual int prefill(int slot, const uint32_t* ids, int n, uint32_t* argmax) = 0;
    // One token for each of b distinct slots; argmax[b] receives the picks.
    virtual int decode(const uint32_t* ids, const int32_t* slots, int b, uint32_t* argmax) = 0;
    virtual int release(int slot) = 0;  // truncate to 0
    virtual int adopt_prefix(int slot, const int32_t* pages, int n) = 0;
};

struct BatcherStats {
    uint64_t submitted = 0, finished = 0, steps = 0;
    uint64_t prefill_tokens = 0;  // prompt tokens actually computed
    uint64_t shared_tokens = 0;   // prompt tokens taken from the prefix index instead
    uint64_t decode_tokens = 0;   // tokens produced by decode steps
    uint64_t decode_rows = 0;     // sum of decode batch sizes (= decode_tokens; kept apart from steps for occupancy)
    uint64_t evicted_pages = 0;
    uint64_t cached_pages = 0;    // pages the prefix index holds now
};

class Batcher {
  public:
    Batcher(SeqBackend* be, int prefill_chunk, bool prefix_cache);
    ~Batcher();
    // Queues a request. SP_ERR_KV_FULL when prompt + max_new cannot fit one sequence window or the whole pool.
    int submit(const uint32_t* prompt, size_t n, size_t max_new, const uint32_t* eos, int n_eos, uint64_t* id);
    // One scheduler iteration: admit, at most prefill_chunk prompt tokens, one decode step of every decoding sequence.
    int step(int* n_running, int* n_waiting);
    // Tokens generated so far for a request; *finished = 1 once it has left the batch. Finished requests stay readable
    // until forget().
    int poll(uint64_t id, uint32_t* out, size_t cap, size_t* n, int* finished) const;
    int cancel(uint64_t id);
    int forget(uint64_t id);
    const BatcherStats& stats() const { return stats_; }
    void drop_prefix_cache();

  private:
    enum State { WAITING, PREFILL, DECODE, DONE };
    struct Request {
        uint64_t id = 0;
        std::vector<uint32_t> prompt, out, eos;
        size_t max_new = 0;
        State state = WAITING;
        int slot = -1;
        size_t fed = 0;        // prompt tokens in the cache (shared or computed)
        int reserved = 0;      // pages this request may still take from the pool
        int indexed_pages = 0; // leading pages of this sequence already entered into the prefix index
    };
    struct CachedPage {
        int page = 0;
        uint64_t parent = 0;
        uint32_t tokens[POOL_PAGE_TOKENS];
        uint64_t last_use = 0;
        int children = 0;
    };
    static uint64_t chain(uint64_t parent, const uint32_t* tok);
    int match_prefix(const std::vector<uint32_t>& prompt, std::vector<int32_t>& pages_out);
    void index_sequence(Request& r);          // enter the full pages of r's sequence into the prefix index
    bool evict_one();
    int admit();
    int finish(Request& r);
    bool is_eos(const Request& r, uint32_t t) const;

    SeqBackend* be_;
    int chunk_;
    bool use_prefix_;
    uint64_t next_id_ = 1, clock_ = 0;
    std::map<uint64_t, Request> reqs_;
    std::deque<uint64_t> waiting_;
    std::vector<uint64_t> running_;  // admission order
    std::vector<int> free_slots_;
    int reserved_total_ = 0;
    std::unordered_map<uint64_t, CachedPage> index_;
    BatcherStats stats_;
};

// Host stand-in for tests: a deterministic "model" whose next token is a hash of the sequence so far, with the page
// bookkeeping of the real engine and a content check on every shared page (the KV of a page is modelled as the running
// hash at its end, so reading a page that belongs to other tokens changes the output).
SeqBackend* make_mock_backend(int vocab, int max_slots, int max_ctx, int n_pages);
class Engine;
SeqBackend* make_engine_backend(Engine* e);

}  // namespace sp
