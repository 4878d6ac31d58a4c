// Paged cache bookkeeping on the host: page pools, per-request block tables, state slots.
//
// "The engine decides the block, the backend stores the numbers"
// (crates/engine/src/backend/mod.rs:10-12): this class owns which page belongs to whom; the
// device tensors that hold keys and values are allocated elsewhere and indexed by the page
// numbers handed out here. The reference has no allocator yet (its driver counts pages
// 0, 1, 2, ... per call, crates/engine/src/generate.rs:72-78); the invariants it asks of one
// (CLAUDE.md:71: every page free or referenced, nothing freed while in use) are checked by
// `check_invariants`.
//
// Layers are put in groups by what they need of the cache. A group has its own pool of pages
// and every request has one block table per group:
//   Full   - every key is kept while the request lives;
//   Window - only the last `window` keys are read, so a page is given back as soon as every
//            position in it has fallen out of the window of the next query.
// Beside the pages, each admitted request holds one state slot (an index below
// `num_state_slots`) for per-request state of fixed size.
#pragma once
#include <algorithm>
#include <climits>
#include <cstdint>
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

namespace vob {

enum GroupKind : int { kFull = 0, kWindow = 1 };

// What a group keeps of a request. The two questions every other piece of the runtime asks of a
// kind are answered HERE and nowhere else (the cache manager's `commit`, the scheduler's capacity
// check and `max_pages_held` only call them), so another kind is another case in these two
// functions.
struct GroupSpec {
    int kind = kFull;
    int window = 0;      // keys visible to a query, itself included (Window groups)
    int num_pages = 0;

    // First position whose key a query at position `pos` still reads.
    int64_t first_visible(int64_t pos) const {
        if (kind == kWindow) return std::max<int64_t>(0, pos + 1 - window);
        return 0;
    }
    // Most tokens whose pages a request of `total` tokens holds at any one time: a window group
    // holds the window plus the page being filled, a full group everything.
    int64_t max_live_tokens(int64_t total, int page_size) const {
        if (kind == kWindow) return std::min<int64_t>(total, (int64_t)window + page_size);
        return total;
    }
};

struct CacheError : std::runtime_error {
    using std::runtime_error::runtime_error;
};

class PagePool {
public:
    explicit PagePool(int num_pages) : refs_(num_pages, 0) {
        free_.reserve(num_pages);
        for (int p = num_pages - 1; p >= 0; --p) free_.push_back(p);   // page 0 is handed out first
    }
    int num_pages() const { return (int)refs_.size(); }
    int num_free() const { return (int)free_.size(); }
    // Last freed, first reused: a page that was just given back goes to the next taker, which
    // is what makes stale contents a tested case rather than a rare one.
    int take() {
        if (free_.empty()) return -1;
        int p = free_.back();
        free_.pop_back();
        refs_[p] = 1;
        return p;
    }
    void give_back(int p) {
        if (p < 0 || p >= (int)refs_.size()) throw CacheError("page " + std::to_string(p) + " is outside the pool");
        if (refs_[p] != 1) throw CacheError("page " + std::to_string(p) + " freed twice");
        refs_[p] = 0;
        free_.push_back(p);
    }
    int refcount(int p) const { return refs_[p]; }
    const std::vector<int32_t>& free_list() const { return free_; }

private:
    std::vector<int32_t> free_;
    std::vector<uint8_t> refs_;
};

struct RequestPages {
    int slot = -1;
    int64_t len = 0;                                  // tokens whose keys are in the cache
    int64_t reserved = 0;                             // tokens that pages are held for (>= len)
    std::vector<std::vector<int32_t>> tables;         // [group][logical page] -> page, -1 = not held
};

class CacheManager {
public:
    CacheManager(int page_size, std::vector<GroupSpec> groups, int num_state_slots)
        : page_size_(page_size), groups_(std::move(groups)) {
        if (page_size <= 0) throw CacheError("page_size must be positive");
        if (num_state_slots <= 0) throw CacheError("num_state_slots must be positive");
        for (const auto& g : groups_) {
            if (g.num_pages <= 0) throw CacheError("a cache group needs at least one page");
            if (g.kind == kWindow && g.window <= 0) throw CacheError("a window group needs a positive window");
            if (g.kind != kFull && g.kind != kWindow) throw CacheError("unknown cache group kind");
            pools_.emplace_back(g.num_pages);
        }
        for (int s = num_state_slots - 1; s >= 0; --s) free_slots_.push_back(s);
        num_slots_ = num_state_slots;
    }

    int page_size() const { return page_size_; }
    int num_groups() const { return (int)groups_.size(); }
    const GroupSpec& group(int g) const { return groups_.at(g); }
    int num_free_pages(int g) const { return pools_.at(g).num_free(); }
    int num_pages(int g) const { return pools_.at(g).num_pages(); }
    int num_free_slots() const { return (int)free_slots_.size(); }
    int num_state_slots() const { return num_slots_; }
    bool has(int64_t id) const { return reqs_.count(id) != 0; }
    size_t num_requests() const { return reqs_.size(); }

    // Take a state slot for a new request. Returns the slot, or -1 when none is free.
    int admit(int64_t id) {
        if (reqs_.count(id)) throw CacheError("request " + std::to_string(id) + " is already admitted");
        if (free_slots_.empty()) return -1;
        RequestPages r;
        r.slot = free_slots_.back();
        free_slots_.pop_back();
        r.tables.resize(groups_.size());
        reqs_[id] = std::move(r);
        return reqs_[id].slot;
    }

    const RequestPages& get(int64_t id) const {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) throw CacheError("request " + std::to_string(id) + " is not admitted");
        return it->second;
    }

    // First position whose key a query at position `pos` still reads in group g.
    int64_t first_visible(int g, int64_t pos) const { return groups_.at(g).first_visible(pos); }

    // Pages of group g that a request of `total` tokens holds at most at any one time (what a
    // pool must have for the request to fit at all).
    int64_t max_pages_held(int g, int64_t total) const {
        int64_t live = groups_.at(g).max_live_tokens(total, page_size_);
        return (live + page_size_ - 1) / page_size_;
    }

    // Pages that group g must add so that the request can take n_new more tokens.
    int pages_to_add(int64_t id, int g, int64_t n_new) const {
        const auto& r = get(id);
        int64_t end = r.len + n_new;
        int64_t need_pages = (end + page_size_ - 1) / page_size_;
        int have = 0;
        const auto& t = r.tables[g];
        // Pages below the table's length are either held or were given back for good.
        have = (int)t.size();
        return (int)std::max<int64_t>(0, need_pages - have);
    }

    // How many more tokens the request could take right now: room left in the pages it holds plus
    // what the free pages of the tightest group add.
    int64_t tokens_that_fit(int64_t id) const {
        const auto& r = get(id);
        int64_t best = INT64_MAX;
        for (size_t g = 0; g < groups_.size(); ++g) {
            int64_t room = (int64_t)r.tables[g].size() * page_size_ - r.len + (int64_t)pools_[g].num_free() * page_size_;
            best = std::min(best, room);
        }
        return best == INT64_MAX ? (int64_t)1 << 40 : best;    // no paged group: nothing limits it
    }

    // Hold pages for tokens [len, len + n_new) in every group; all groups or none.
    bool reserve(int64_t id, int64_t n_new) {
        if (n_new <= 0) throw CacheError("reserve: n_new must be positive");
        auto it = reqs_.find(id);
        if (it == reqs_.end()) throw CacheError("request " + std::to_string(id) + " is not admitted");
        for (size_t g = 0; g < groups_.size(); ++g)
            if (pages_to_add(id, (int)g, n_new) > pools_[g].num_free()) return false;
        RequestPages& r = it->second;
        for (size_t g = 0; g < groups_.size(); ++g) {
            int add = pages_to_add(id, (int)g, n_new);
            for (int i = 0; i < add; ++i) r.tables[g].push_back(pools_[g].take());
        }
        r.reserved = std::max(r.reserved, r.len + n_new);
        return true;
    }

    // The step that wrote n_new tokens is done: they count, and window groups give back every
    // page that the next query (at position len) can no longer see.
    std::vector<std::pair<int, int>> commit(int64_t id, int64_t n_new) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) throw CacheError("request " + std::to_string(id) + " is not admitted");
        RequestPages& r = it->second;
        if (n_new < 0 || r.len + n_new > r.reserved)
            throw CacheError("commit: " + std::to_string(n_new) + " tokens were not reserved");
        r.len += n_new;
        std::vector<std::pair<int, int>> released;   // (group, page)
        for (size_t g = 0; g < groups_.size(); ++g) {
            int64_t first = first_visible((int)g, r.len);        // next query sits at position len
            int64_t dead_pages = first / page_size_;             // pages wholly below `first` (none in a full group)
            auto& t = r.tables[g];
            for (int64_t i = 0; i < dead_pages && i < (int64_t)t.size(); ++i) {
                if (t[i] >= 0) {
                    pools_[g].give_back(t[i]);
                    released.emplace_back((int)g, t[i]);
                    t[i] = -1;
                }
            }
        }
        return released;
    }

    // The request ends (finished, aborted or preempted): everything it holds goes back.
    void release(int64_t id) {
        auto it = reqs_.find(id);
        if (it == reqs_.end()) throw CacheError("request " + std::to_string(id) + " is not admitted");
        RequestPages& r = it->second;
        for (size_t g = 0; g < groups_.size(); ++g)
            for (auto it2 = r.tables[g].rbegin(); it2 != r.tables[g].rend(); ++it2)
                if (*it2 >= 0) pools_[g].give_back(*it2);
        free_slots_.push_back(r.slot);
        reqs_.erase(it);
    }

    // Physical slot (page * page_size + offset) of position pos in group g; throws if the table
    // does not cover it (crates/engine/src/backend/paged.rs:48-52,57-80).
    int64_t slot_of(int64_t id, int g, int64_t pos) const {
        const auto& t = get(id).tables.at(g);
        int64_t lp = pos / page_size_;
        if (lp >= (int64_t)t.size() || t[lp] < 0)
            throw CacheError("block table of request " + std::to_string(id) + " does not cover position " +
                             std::to_string(pos) + ": " + std::to_string(pos + 1) + " tokens need " +
                             std::to_string(lp + 1) + " pages, table has " + std::to_string(t.size()));
        return (int64_t)t[lp] * page_size_ + pos % page_size_;
    }

    // Empty string if every page is either free or held by exactly one table entry, the counts
    // add up, and no slot is held twice; otherwise what is wrong.
    std::string check_invariants() const {
        for (size_t g = 0; g < groups_.size(); ++g) {
            std::vector<int> seen(pools_[g].num_pages(), 0);
            for (int p : pools_[g].free_list()) {
                if (p < 0 || p >= pools_[g].num_pages()) return "free list holds a page outside the pool";
                if (++seen[p] > 1) return "page " + std::to_string(p) + " is on the free list twice";
                if (pools_[g].refcount(p) != 0) return "free page " + std::to_string(p) + " has a reference";
            }
            size_t held = 0;
            for (const auto& kv : reqs_) {
                for (int p : kv.second.tables[g]) {
                    if (p < 0) continue;
                    if (p >= pools_[g].num_pages()) return "a table holds a page outside the pool";
                    if (++seen[p] > 1) return "page " + std::to_string(p) + " of group " + std::to_string(g) + " is held twice";
                    if (pools_[g].refcount(p) != 1) return "held page " + std::to_string(p) + " has no reference";
                    ++held;
                }
            }
            if (held + pools_[g].free_list().size() != (size_t)pools_[g].num_pages())
                return "group " + std::to_string(g) + ": " + std::to_string(held) + " held + " +
                       std::to_string(pools_[g].free_list().size()) + " free != " + std::to_string(pools_[g].num_pages());
        }
        std::vector<int> slot_seen(num_slots_, 0);
        for (int s : free_slots_) if (++slot_seen.at(s) > 1) return "state slot free twice";
        for (const auto& kv : reqs_) if (++slot_seen.at(kv.second.slot) > 1) return "state slot held twice";
        for (int c : slot_seen) if (c != 1) return "a state slot is lost";
        return "";
    }

private:
    int page_size_;
    int num_slots_ = 0;
    std::vector<GroupSpec> groups_;
    std::vector<PagePool> pools_;
    std::vector<int> free_slots_;
    std::map<int64_t, RequestPages> reqs_;
};

}  // namespace vob
