// Host-side bookkeeping of the paged KV cache: which pool page holds tokens [16 j, 16 j + 16) of which sequence slot.
//
// Pages carry a reference count, so several slots (and the prefix cache of the batching scheduler) may name the same
// page: a prompt prefix that was computed once is read by every sequence that starts with it. A page that more than one
// owner names is never written: sequences only append, and appending into a partly filled page that is shared first
// moves the slot onto a private copy (copy-on-write; the caller copies the device bytes).
//
// The reference has one contiguous cache per engine and re-uses a prefix only within one conversation
// (truncate_cache, crates/sapient-models/src/forward/llama.rs:307-313; Pipeline's prefix match,
// crates/sapient-generate/src/pipeline.rs:818-830); batching and sharing across requests are on its roadmap
// (docs/ROADMAP.md:312).
#pragma once
#include <stdint.h>

#include <vector>

namespace sp {

constexpr int POOL_PAGE_TOKENS = 16;  // = KV_PAGE of the kernels

class PagePool {
  public:
    void init(int n_slots, int max_pages_per_slot, int n_pages) {
        n_slots_ = n_slots;
        max_pages_ = max_pages_per_slot;
        table.assign((size_t)n_slots * max_pages_per_slot, 0);
        held.assign(n_slots, 0);
        ref.assign(n_pages, 0);
        free_list.clear();
        for (int p = n_pages - 1; p >= 0; --p) free_list.push_back(p);
        dirty = true;
    }
    int available() const { return (int)free_list.size(); }
    int n_pages() const { return (int)ref.size(); }
    int max_pages() const { return max_pages_; }
    int page_of(int slot, int idx) const { return table[(size_t)slot * max_pages_ + idx]; }
    static int pages_for(int64_t tokens) { return (int)((tokens + POOL_PAGE_TOKENS - 1) / POOL_PAGE_TOKENS); }
    // Pages the slot still lacks to hold new_len tokens.
    int missing(int slot, int new_len) const { const int need = pages_for(new_len) - held[slot]; return need > 0 ? need : 0; }
    // Gives the slot fresh pages up to new_len tokens; false (nothing changed beyond what was already added) when the
    // pool runs out.
    bool grow(int slot, int new_len) {
        const int need = pages_for(new_len);
        if (need > max_pages_) return false;
        while (held[slot] < need) {
            if (free_list.empty()) return false;
            const int pg = free_list.back();
            free_list.pop_back();
            ref[pg] = 1;
            table[(size_t)slot * max_pages_ + held[slot]++] = pg;
            dirty = true;
        }
        return true;
    }
    // Keeps the first keep_pages pages of the slot; the rest lose this owner.
    void shrink(int slot, int keep_pages) {
        while (held[slot] > keep_pages) release(table[(size_t)slot * max_pages_ + --held[slot]]);
    }
    void retain(int pg) { ++ref[pg]; }
    void release(int pg) {
        if (--ref[pg] == 0) free_list.push_back(pg);
    }
    // An EMPTY slot starts as a reader of n pages that already hold its first 16 n tokens.
    bool adopt(int slot, const int32_t* pages, int n) {
        if (held[slot] != 0 || n > max_pages_) return false;
        for (int i = 0; i < n; ++i)
            if (pages[i] < 0 || pages[i] >= (int)ref.size() || ref[pages[i]] <= 0) return false;
        for (int i = 0; i < n; ++i) {
            retain(pages[i]);
            table[(size_t)slot * max_pages_ + i] = pages[i];
        }
        held[slot] = n;
        dirty = dirty || n > 0;
        return true;
    }
    // Before tokens are appended to a slot that holds `len` tokens: when the partly filled last page has other owners,
    // the slot moves to a fresh page. Returns 1 with (*from, *to) = the pages whose device bytes the caller copies,
    // 0 when nothing had to be done, -1 when the pool has no page left.
    int privatise_tail(int slot, int len, int* from, int* to) {
        if (len % POOL_PAGE_TOKENS == 0) return 0;
        const int idx = len / POOL_PAGE_TOKENS;
        if (idx >= held[slot]) return 0;
        const int pg = table[(size_t)slot * max_pages_ + idx];
        if (ref[pg] <= 1) return 0;
        if (free_list.empty()) return -1;
        const int fresh = free_list.back();
        free_list.pop_back();
        ref[fresh] = 1;
        --ref[pg];
        table[(size_t)slot * max_pages_ + idx] = fresh;
        dirty = true;
        *from = pg;
        *to = fresh;
        return 1;
    }

    std::vector<int32_t> table;  // [n_slots][max_pages]: the host copy of the device page table
    std::vector<int> held;       // pages each slot names
    std::vector<int> ref;        // owners per page (slots + external holders)
    std::vector<int> free_list;
    bool dirty = true;           // the device copy is out of date

  private:
    int n_slots_ = 0, max_pages_ = 0;
};

}  // namespace sp
