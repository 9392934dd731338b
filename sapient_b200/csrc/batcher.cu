// Continuous batching scheduler (batcher.h): admission against the page pool, chunked prefill between decode steps,
// prefix sharing through reference-counted pages.
#include "batcher.h"

#include <algorithm>
#include <cstring>

#include "engine.h"

namespace sp {

namespace {
constexpr uint64_t CHAIN_ROOT = 0x9E3779B97F4A7C15ull;
inline uint64_t mix64(uint64_t h, uint64_t v) {
    h ^= v + 0x9E3779B97F4A7C15ull + (h << 6) + (h >> 2);
    h *= 0xFF51AFD7ED558CCDull;
    h ^= h >> 33;
    return h;
}
}  // namespace

uint64_t Batcher::chain(uint64_t parent, const uint32_t* tok) {
    uint64_t h = parent;
    for (int i = 0; i < POOL_PAGE_TOKENS; ++i) h = mix64(h, tok[i]);
    return h ? h : 1;
}

Batcher::Batcher(SeqBackend* be, int prefill_chunk, bool prefix_cache) : be_(be), chunk_(std::max(1, prefill_chunk)), use_prefix_(prefix_cache) {
    for (int s = be_->max_slots() - 1; s >= 0; --s) free_slots_.push_back(s);
}

Batcher::~Batcher() {
    for (auto& kv : reqs_)
        if (kv.second.slot >= 0) be_->release(kv.second.slot);
    drop_prefix_cache();
}

void Batcher::drop_prefix_cache() {
    for (auto& kv : index_) be_->pool().release(kv.second.page);
    index_.clear();
    stats_.cached_pages = 0;
}

bool Batcher::is_eos(const Request& r, uint32_t t) const {
    return std::find(r.eos.begin(), r.eos.end(), t) != r.eos.end();
}

int Batcher::submit(const uint32_t* prompt, size_t n, size_t max_new, const uint32_t* eos, int n_eos, uint64_t* id) {
    if (!prompt || n == 0 || max_new == 0 || !id || (n_eos > 0 && !eos)) { set_error("batcher: empty prompt, zero max_new or null argument"); return SP_ERR_ARG; }
    if (n + max_new > (size_t)be_->max_ctx() || PagePool::pages_for((int64_t)(n + max_new)) > be_->pool().n_pages()) {
        set_error("batcher: prompt + max_new exceeds the sequence window or the page pool");
        return SP_ERR_KV_FULL;
    }
    Request r;
    r.id = next_id_++;
    r.prompt.assign(prompt, prompt + n);
    r.max_new = max_new;
    if (n_eos > 0) r.eos.assign(eos, eos + n_eos);
    *id = r.id;
    waiting_.push_back(r.id);
    reqs_.emplace(r.id, std::move(r));
    ++stats_.submitted;
    return SP_OK;
}

// Longest indexed prefix of the prompt in whole pages. At least one prompt token is always left to compute: its
// logits choose the first generated token.
int Batcher::match_prefix(const std::vector<uint32_t>& prompt, std::vector<int32_t>& pages_out) {
    pages_out.clear();
    if (!use_prefix_) return 0;
    const int max_pages = (int)((prompt.size() - 1) / POOL_PAGE_TOKENS);
    uint64_t h = CHAIN_ROOT;
    for (int j = 0; j < max_pages; ++j) {
        const uint32_t* tok = prompt.data() + (size_t)j * POOL_PAGE_TOKENS;
        const uint64_t hj = chain(h, tok);
        auto it = index_.find(hj);
        if (it == index_.end() || it->second.parent != h || std::memcmp(it->second.tokens, tok, sizeof(it->second.tokens)) != 0) break;
        it->second.last_use = ++clock_;
        pages_out.push_back(it->second.page);
        h = hj;
    }
    return (int)pages_out.size();
}

// Enters the full pages of r's sequence (prompt, then the generated tokens that have been fed back) into the index.
void Batcher::index_sequence(Request& r) {
    if (!use_prefix_ || r.slot < 0) return;
    const int len = be_->seq_len(r.slot);
    const int full = len / POOL_PAGE_TOKENS;
    if (full <= r.indexed_pages) return;
    auto token_at = [&](size_t i) { return i < r.prompt.size() ? r.prompt[i] : r.out[i - r.prompt.size()]; };
    uint64_t h = CHAIN_ROOT;
    uint32_t tok[POOL_PAGE_TOKENS];
    for (int j = 0; j < full; ++j) {
        for (int i = 0; i < POOL_PAGE_TOKENS; ++i) tok[i] = token_at((size_t)j * POOL_PAGE_TOKENS + i);
        const uint64_t hj = chain(h, tok);
        if (j >= r.indexed_pages) {
            auto it = index_.find(hj);
            if (it == index_.end()) {
                CachedPage c;
                c.page = be_->pool().page_of(r.slot, j);
                c.parent = h;
                std::memcpy(c.tokens, tok, sizeof(tok));
                c.last_use = ++clock_;
                be_->pool().retain(c.page);
                index_.emplace(hj, c);
                if (h != CHAIN_ROOT) {
                    auto pit = index_.find(h);
                    if (pit != index_.end()) ++pit->second.children;
                }
                ++stats_.cached_pages;
            } else if (it->second.parent != h || std::memcmp(it->second.tokens, tok, sizeof(tok)) != 0) {
                break;  // a hash collision with other content: this chain is not indexed further
            } else {
                it->second.last_use = ++clock_;
            }
        }
        h = hj;
    }
    r.indexed_pages = full;
}

// Drops the least recently used page that nothing else reads and that no indexed page continues.
bool Batcher::evict_one() {
    auto best = index_.end();
    for (auto it = index_.begin(); it != index_.end(); ++it) {
        if (it->second.children != 0 || be_->pool().ref[it->second.page] != 1) continue;
        if (best == index_.end() || it->second.last_use < best->second.last_use) best = it;
    }
    if (best == index_.end()) return false;
    if (best->second.parent != CHAIN_ROOT) {
        auto pit = index_.find(best->second.parent);
        if (pit != index_.end()) --pit->second.children;
    }
    be_->pool().release(best->second.page);
    index_.erase(best);
    ++stats_.evicted_pages;
    --stats_.cached_pages;
    return true;
}

int Batcher::admit() {
    std::vector<int32_t> shared;
    while (!waiting_.empty() && !free_slots_.empty()) {
        Request& r = reqs_.at(waiting_.front());
        const int slot = free_slots_.back();
        const int n_shared = match_prefix(r.prompt, shared);
        if (n_shared > 0) {
            const int st = be_->adopt_prefix(slot, shared.data(), n_shared);
            if (st != SP_OK) return st;
        }
        const int need = PagePool::pages_for((int64_t)(r.prompt.size() + r.max_new)) - n_shared;
        // pages that running requests have been promised stay theirs
        while (be_->pool().available() - reserved_total_ < need && evict_one()) {}
        if (be_->pool().available() - reserved_total_ < need) {
            if (n_shared > 0) be_->release(slot);
            break;  // first come, first served: later (smaller) requests do not overtake
        }
        free_slots_.pop_back();
        waiting_.pop_front();
        r.slot = slot;
        r.state = PREFILL;
        r.fed = (size_t)n_shared * POOL_PAGE_TOKENS;
        r.indexed_pages = n_shared;
        r.reserved = need;
        reserved_total_ += need;
        stats_.shared_tokens += r.fed;
        running_.push_back(r.id);
    }
    return SP_OK;
}

int Batcher::finish(Request& r) {
    index_sequence(r);
    int st = SP_OK;
    if (r.slot >= 0) {
        st = be_->release(r.slot);
        free_slots_.push_back(r.slot);
        r.slot = -1;
    }
    reserved_total_ -= r.reserved;
    r.reserved = 0;
    r.state = DONE;
    running_.erase(std::remove(running_.begin(), running_.end(), r.id), running_.end());
    ++stats_.finished;
    return st;
}

int Batcher::step(int* n_running, int* n_waiting) {
    int st = admit();
    if (st != SP_OK) return st;
    auto settle = [&](Request& r) {  // pages taken from the pool since the last look are no longer a promise
        const int total = PagePool::pages_for((int64_t)(r.prompt.size() + r.max_new));
        const int left = std::max(0, total - be_->pool().held[r.slot]);
        reserved_total_ += left - r.reserved;
        r.reserved = left;
    };
    // chunked prefill, oldest request first
    int budget = chunk_;
    const std::vector<uint64_t> order = running_;
    for (uint64_t id : order) {
        if (budget <= 0) break;
        Request& r = reqs_.at(id);
        if (r.state != PREFILL) continue;
        const int n = (int)std::min<size_t>((size_t)budget, r.prompt.size() - r.fed);
        const bool last = r.fed + (size_t)n == r.prompt.size();
        uint32_t tok = 0;
        st = be_->prefill(r.slot, r.prompt.data() + r.fed, n, last ? &tok : nullptr);
        if (st != SP_OK) return st;
        r.fed += (size_t)n;
        budget -= n;
        stats_.prefill_tokens += (uint64_t)n;
        settle(r);
        if (last) {
            r.out.push_back(tok);
            index_sequence(r);  // requests that arrive while this one still decodes already share its prompt
            if (is_eos(r, tok) || r.out.size() >= r.max_new) {
                if ((st = finish(r)) != SP_OK) return st;
            } else {
                r.state = DECODE;
            }
        }
    }
    // one decode step of every decoding sequence
    std::vector<uint64_t> dec;
    for (uint64_t id : running_)
        if (reqs_.at(id).state == DECODE) dec.push_back(id);
    const int rows = std::max(1, be_->max_step_rows());
    std::vector<uint32_t> ids, picks;
    std::vector<int32_t> slots;
    for (size_t g0 = 0; g0 < dec.size(); g0 += (size_t)rows) {
        const int b = (int)std::min<size_t>((size_t)rows, dec.size() - g0);
        ids.resize(b);
        slots.resize(b);
        picks.resize(b);
        for (int i = 0; i < b; ++i) {
            const Request& r = reqs_.at(dec[g0 + i]);
            ids[i] = r.out.back();
            slots[i] = r.slot;
        }
        st = be_->decode(ids.data(), slots.data(), b, picks.data());
        if (st != SP_OK) return st;
        stats_.decode_tokens += (uint64_t)b;
        stats_.decode_rows += (uint64_t)b;
        for (int i = 0; i < b; ++i) {
            Request& r = reqs_.at(dec[g0 + i]);
            r.out.push_back(picks[i]);
            settle(r);
            if (is_eos(r, picks[i]) || r.out.size() >= r.max_new)
                if ((st = finish(r)) != SP_OK) return st;
        }
    }
    ++stats_.steps;
    if (n_running) *n_running = (int)running_.size();
    if (n_waiting) *n_waiting = (int)waiting_.size();
    return SP_OK;
}

int Batcher::poll(uint64_t id, uint32_t* out, size_t cap, size_t* n, int* finished) const {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) { set_error("batcher: unknown request id"); return SP_ERR_ARG; }
    const Request& r = it->second;
    if (n) *n = r.out.size();
    if (finished) *finished = r.state == DONE ? 1 : 0;
    if (out) std::memcpy(out, r.out.data(), std::min(cap, r.out.size()) * sizeof(uint32_t));
    return SP_OK;
}

int Batcher::cancel(uint64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) { set_error("batcher: unknown request id"); return SP_ERR_ARG; }
    Request& r = it->second;
    if (r.state == DONE) return SP_OK;
    if (r.state == WAITING) {
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
        r.state = DONE;
        ++stats_.finished;
        return SP_OK;
    }
    return finish(r);
}

int Batcher::forget(uint64_t id) {
    auto it = reqs_.find(id);
    if (it == reqs_.end()) { set_error("batcher: unknown request id"); return SP_ERR_ARG; }
    if (it->second.state != DONE) { set_error("batcher: the request is still queued or running"); return SP_ERR_STATE; }
    reqs_.erase(it);
    return SP_OK;
}

// ── the CUDA engine behind the scheduler ──
namespace {
class EngineBackend : public SeqBackend {
  public:
    explicit EngineBackend(Engine* e) : e_(e) {}
    int max_slots() const override { return e_->d.max_batch; }
    int max_ctx() const override { return e_->d.max_ctx; }
    int max_step_rows() const override { return std::min(32, e_->d.max_tokens); }
    PagePool& pool() override { return e_->pages; }
    int seq_len(int slot) const override { return e_->seq_len[slot]; }
    int prefill(int slot, const uint32_t* ids, int n, uint32_t* argmax) override {
        slots_.assign((size_t)n, slot);
        return e_->forward(ids, slots_.data(), n, false, nullptr, argmax);
    }
    int decode(const uint32_t* ids, const int32_t* slots, int b, uint32_t* argmax) override {
        return e_->forward(ids, slots, b, true, nullptr, argmax);
    }
    int release(int slot) override { size_t kept; return e_->truncate(slot, 0, &kept); }
    int adopt_prefix(int slot, const int32_t* pages, int n) override { return e_->adopt_prefix(slot, pages, n); }

  private:
    Engine* e_;
    std::vector<int32_t> slots_;
};

// Host stand-in (tests of the scheduling logic): "KV content" of a page = the token ids written to it; the next token is
// a hash of the sequence as read back THROUGH the slot's page table, so a wrongly shared or prematurely recycled page
// changes the output.
class MockBackend : public SeqBackend {
  public:
    MockBackend(int vocab, int max_slots, int max_ctx, int n_pages) : vocab_(vocab), slots_(max_slots), ctx_(max_ctx) {
        pool_.init(max_slots, PagePool::pages_for(max_ctx), n_pages);
        content_.assign((size_t)n_pages * POOL_PAGE_TOKENS, 0xFFFFFFFFu);
        len_.assign(max_slots, 0);
    }
    int max_slots() const override { return slots_; }
    int max_ctx() const override { return ctx_; }
    int max_step_rows() const override { return 8; }
    PagePool& pool() override { return pool_; }
    int seq_len(int slot) const override { return len_[slot]; }
    int prefill(int slot, const uint32_t* ids, int n, uint32_t* argmax) override {
        for (int i = 0; i < n; ++i) {
            const int st = append(slot, ids[i]);
            if (st != SP_OK) return st;
        }
        if (argmax) *argmax = next(slot);
        return SP_OK;
    }
    int decode(const uint32_t* ids, const int32_t* slots, int b, uint32_t* argmax) override {
        for (int i = 0; i < b; ++i) {
            const int st = append(slots[i], ids[i]);
            if (st != SP_OK) return st;
            argmax[i] = next(slots[i]);
        }
        return SP_OK;
    }
    int release(int slot) override {
        pool_.shrink(slot, 0);
        len_[slot] = 0;
        return SP_OK;
    }
    int adopt_prefix(int slot, const int32_t* pages, int n) override {
        if (len_[slot] != 0 || !pool_.adopt(slot, pages, n)) { set_error("adopt_prefix: the slot is not empty or a page is not live"); return SP_ERR_STATE; }
        len_[slot] = n * POOL_PAGE_TOKENS;
        return SP_OK;
    }

  private:
    int append(int slot, uint32_t id) {
        if (len_[slot] >= ctx_) { set_error("KV cache full"); return SP_ERR_KV_FULL; }
        int from = 0, to = 0;
        const int r = pool_.privatise_tail(slot, len_[slot], &from, &to);
        if (r < 0 || !pool_.grow(slot, len_[slot] + 1)) { set_error("KV page pool exhausted"); return SP_ERR_KV_FULL; }
        if (r > 0) std::memcpy(&content_[(size_t)to * POOL_PAGE_TOKENS], &content_[(size_t)from * POOL_PAGE_TOKENS], POOL_PAGE_TOKENS * 4);
        const int pg = pool_.page_of(slot, len_[slot] / POOL_PAGE_TOKENS);
        if (pool_.ref[pg] != 1) { set_error("mock: write into a shared page"); return SP_ERR_STATE; }
        content_[(size_t)pg * POOL_PAGE_TOKENS + len_[slot] % POOL_PAGE_TOKENS] = id;
        ++len_[slot];
        return SP_OK;
    }
    uint32_t next(int slot) const {
        uint64_t h = 0xCBF29CE484222325ull;  // FNV-1a over the token ids
        for (int i = 0; i < len_[slot]; ++i) {
            const uint32_t t = content_[(size_t)pool_.page_of(slot, i / POOL_PAGE_TOKENS) * POOL_PAGE_TOKENS + i % POOL_PAGE_TOKENS];
            for (int b = 0; b < 4; ++b) {
                h ^= (t >> (8 * b)) & 0xFFu;
                h *= 0x100000001B3ull;
            }
        }
        return (uint32_t)(h % (uint64_t)vocab_);
    }
    int vocab_, slots_, ctx_;
    PagePool pool_;
    std::vector<uint32_t> content_;
    std::vector<int> len_;
};
}  // namespace

SeqBackend* make_mock_backend(int vocab, int max_slots, int max_ctx, int n_pages) { return new MockBackend(vocab, max_slots, max_ctx, n_pages); }
SeqBackend* make_engine_backend(Engine* e) { return new EngineBackend(e); }

}  // namespace sp
