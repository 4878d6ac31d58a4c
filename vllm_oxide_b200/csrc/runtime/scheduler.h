// Continuous batching with chunked prefill: which requests run in the next step, with how many
// tokens each, and what happens when pages run out.
//
// The reference has no scheduler yet; it records what one must do (CLAUDE.md:68-72: one forward
// per step, one new token per running sequence per decode step, no allocation in the hot loop,
// output that does not depend on the batch; docs/grill-log.md:88: taking a page at a page's
// edge and preempting when the pool is empty are separate duties). The policy here:
//   * a step's budget is `max_batch_tokens` new tokens and `max_seqs` requests;
//   * running requests that need exactly one token (decoding) are served first, then running
//     requests still working through their prompt, then waiting requests in arrival order;
//   * a prompt is cut into portions of at most `prefill_chunk` tokens and at most what is left
//     of the budget, down to a single token;
//   * a request is admitted only if a state slot is free and its first portion gets pages;
//   * when a running request cannot get a page, the most recently admitted running request is
//     preempted: its pages and slot are given back and it returns to the FRONT of the waiting
//     queue, to be recomputed later from its prompt plus the tokens it had generated;
//   * a request that is alone and still cannot get a page is finished with reason "capacity".
// A request ends when it samples one of its stop tokens (the token is kept, as
// crates/engine/src/generate.rs:23,105-108), after max_new_tokens, or at max_model_len.
#pragma once
#include <algorithm>
#include <deque>
#include "step_batch.h"

namespace vob {

struct SamplingParams {
    int max_new_tokens = 16;
    float temperature = 0.f;
    uint64_t seed = 0;
    std::vector<int32_t> stop_token_ids;
};

struct Request {
    int64_t id = 0;
    std::vector<int32_t> tokens;     // prompt, then generated tokens
    int prompt_len = 0;
    int computed = 0;                // tokens whose keys are in the cache
    int generated = 0;
    int preemptions = 0;
    SamplingParams params;
};

struct PlannedEntry {
    int64_t id;
    int start;        // first token of the portion (index into the request's tokens)
    int count;        // tokens in the portion
    bool sample;      // the portion reaches the request's last token: a new token is picked
};

struct StepPlan {
    std::vector<PlannedEntry> entries;
    // every entry is one token that reaches its request's end: a pure decode step
    bool decode_only() const {
        if (entries.empty()) return false;
        for (const auto& e : entries) if (e.count != 1 || !e.sample) return false;
        return true;
    }
    std::vector<int64_t> sampling_ids() const {
        std::vector<int64_t> v;
        for (const auto& e : entries) if (e.sample) v.push_back(e.id);
        return v;
    }
    std::vector<int64_t> preempted;      // requests preempted while planning this step
    std::vector<int64_t> admitted;       // requests that entered the running set
    std::vector<std::pair<int64_t, std::string>> failed;   // finished without running: (id, reason)
};

struct Finished {
    int64_t id;
    std::string reason;     // "stop", "length", "capacity", "abort"
    std::vector<int32_t> output;   // generated tokens
};

class Scheduler {
public:
    Scheduler(CacheManager* cache, int max_batch_tokens, int max_seqs, int max_model_len, int prefill_chunk)
        : cache_(cache), max_batch_tokens_(max_batch_tokens), max_seqs_(max_seqs),
          max_model_len_(max_model_len), prefill_chunk_(prefill_chunk > 0 ? prefill_chunk : max_batch_tokens) {
        if (max_batch_tokens <= 0 || max_seqs <= 0 || max_model_len <= 0) throw CacheError("scheduler limits must be positive");
    }

    // The reference's capacity rule (crates/engine/src/generate.rs:55-71): the last token is never
    // fed back, so prompt + max_new - 1 positions must fit the model length and the pool.
    void add_request(int64_t id, const std::vector<int32_t>& prompt, const SamplingParams& p) {
        if (prompt.empty() || p.max_new_tokens <= 0) throw CacheError("generate: empty prompt or max_new = 0");
        if (requests_.count(id)) throw CacheError("request " + std::to_string(id) + " exists already");
        int64_t total = (int64_t)prompt.size() + p.max_new_tokens - 1;
        if (total > max_model_len_)
            throw CacheError("capacity: sequence length: need " + std::to_string(total) + ", limit " + std::to_string(max_model_len_));
        for (int g = 0; g < cache_->num_groups(); ++g) {
            int64_t pages = cache_->max_pages_held(g, total);      // the group's own rule (all tokens, a window, ...)
            if (pages > cache_->num_pages(g))
                throw CacheError("capacity: sequence length: need " + std::to_string(pages) + " pages, the pool has " +
                                 std::to_string(cache_->num_pages(g)));
        }
        Request r;
        r.id = id; r.tokens = prompt; r.prompt_len = (int)prompt.size(); r.params = p;
        requests_[id] = std::move(r);
        waiting_.push_back(id);
    }

    // Admission watermark: while other requests run, a waiting request is admitted only if so many
    // pages of every group stay free behind its first portion (room for the running requests to
    // grow, so that the newcomer is not preempted again at once). 0: admit whenever a token fits.
    void set_admission_watermark(int pages) {
        if (pages < 0) throw CacheError("scheduler: the admission watermark cannot be negative");
        watermark_pages_ = pages;
    }
    int admission_watermark() const { return watermark_pages_; }

    bool has_unfinished() const { return !waiting_.empty() || !running_.empty(); }
    size_t num_waiting() const { return waiting_.size(); }
    size_t num_running() const { return running_.size(); }
    const Request& request(int64_t id) const { return requests_.at(id); }
    const std::vector<int64_t>& running() const { return running_; }
    std::vector<int64_t> waiting() const { return std::vector<int64_t>(waiting_.begin(), waiting_.end()); }

    StepPlan schedule() {
        StepPlan plan;
        int budget = max_batch_tokens_;
        // pass 0: running requests that decode (one token left); pass 1: running requests in prefill
        for (int pass = 0; pass < 2; ++pass) {
            const std::vector<int64_t> snapshot = running_;
            for (int64_t id : snapshot) {
                if (budget <= 0) break;
                if (std::find(running_.begin(), running_.end(), id) == running_.end()) continue;   // preempted meanwhile
                Request& r = requests_.at(id);
                int remaining = (int)r.tokens.size() - r.computed;
                if ((pass == 0) != (remaining == 1)) continue;
                if (planned(plan, id)) continue;
                int want = std::min({remaining, prefill_chunk_, budget});
                while (true) {
                    int n = (int)std::min<int64_t>(want, cache_->tokens_that_fit(id));
                    if (n >= 1) {
                        cache_->reserve(id, n);
                        plan.entries.push_back({id, r.computed, n, r.computed + n == (int)r.tokens.size()});
                        budget -= n;
                        break;
                    }
                    // not one more token fits: preempt the most recently admitted running request
                    int64_t victim = running_.back();
                    if (victim == id) {
                        if (running_.size() == 1) finish_now(id, "capacity", plan);   // alone and stuck for good
                        else budget += preempt(id, plan);
                        break;
                    }
                    budget += preempt(victim, plan);
                    want = std::min({remaining, prefill_chunk_, budget});
                }
            }
        }
        // admission, first come first served; a preempted request waits at the front, and no one
        // is admitted in a step that had to preempt
        while (budget > 0 && !waiting_.empty() && (int)running_.size() < max_seqs_ && plan.preempted.empty()) {
            int64_t id = waiting_.front();
            Request& r = requests_.at(id);
            int slot = cache_->admit(id);
            if (slot < 0) break;
            int remaining = (int)r.tokens.size() - r.computed;
            int n = (int)std::min<int64_t>(std::min({remaining, prefill_chunk_, budget}), cache_->tokens_that_fit(id));
            if (n < 1) {
                cache_->release(id);
                if (!running_.empty()) break;          // wait until someone finishes
                waiting_.pop_front();                  // nothing runs and still no page: never fits
                done_.push_back(Finished{id, "capacity", generated_of(r)});
                plan.failed.emplace_back(id, "capacity");
                requests_.erase(id);
                continue;
            }
            if (watermark_pages_ > 0 && !running_.empty()) {
                bool room = true;
                for (int g = 0; g < cache_->num_groups(); ++g)
                    if (cache_->num_free_pages(g) - cache_->pages_to_add(id, g, n) < watermark_pages_) room = false;
                if (!room) {
                    cache_->release(id);
                    break;                             // wait until the running requests have given pages back
                }
            }
            cache_->reserve(id, n);
            waiting_.pop_front();
            running_.push_back(id);
            plan.admitted.push_back(id);
            plan.entries.push_back({id, r.computed, n, r.computed + n == (int)r.tokens.size()});
            budget -= n;
        }
        return plan;
    }

    // Build the device arrays of a plan.
    StepArrays arrays(const StepPlan& plan, int rows_cap, int seqs_cap, int logits_cap, int max_pages, int vocab) const {
        std::vector<StepEntry> es;
        for (const auto& pe : plan.entries) {
            const Request& r = requests_.at(pe.id);
            StepEntry e;
            e.id = pe.id;
            e.tokens.assign(r.tokens.begin() + pe.start, r.tokens.begin() + pe.start + pe.count);
            if (pe.sample) e.want.push_back(pe.count - 1);
            e.temperature = r.params.temperature;
            e.seed = r.params.seed;
            e.sample_step = r.generated;
            es.push_back(std::move(e));
        }
        return build_step(*cache_, es, rows_cap, seqs_cap, logits_cap, max_pages, vocab);
    }

    // The step ran: `sampled` holds one token per entry with sample == true, in plan order.
    std::vector<Finished> update(const StepPlan& plan, const std::vector<int32_t>& sampled) {
        std::vector<Finished> out;
        out.swap(done_);
        size_t si = 0;
        for (const auto& pe : plan.entries) {
            auto it = requests_.find(pe.id);
            if (it == requests_.end()) { if (pe.sample) ++si; continue; }
            Request& r = it->second;
            cache_->commit(pe.id, pe.count);
            r.computed += pe.count;
            if (!pe.sample) continue;
            if (si >= sampled.size()) throw CacheError("update: fewer sampled tokens than sampling entries");
            int32_t tok = sampled[si++];
            r.tokens.push_back(tok);
            r.generated += 1;
            const auto& stops = r.params.stop_token_ids;
            std::string reason;
            if (std::find(stops.begin(), stops.end(), tok) != stops.end()) reason = "stop";
            else if (r.generated >= r.params.max_new_tokens) reason = "length";
            else if ((int)r.tokens.size() > max_model_len_) reason = "length";
            if (!reason.empty()) {
                Finished f{pe.id, reason, generated_of(r)};
                cache_->release(pe.id);
                running_.erase(std::remove(running_.begin(), running_.end(), pe.id), running_.end());
                requests_.erase(it);
                out.push_back(std::move(f));
            }
        }
        return out;
    }

    // ------------------------------------------------------------------ running ahead of the host's reads
    // A decode step's picked tokens reach the host one step late when the engine launches step
    // n + 1 (which takes its input tokens from step n's picks on the device) before it reads
    // step n. For that the scheduler must plan step n + 1 without knowing step n's tokens:
    //   steady_decode()   the next step is sure to be a pure decode step of exactly the running
    //                     requests in their present order, whatever the steps in flight pick (a
    //                     stop token aside, which `resolve` handles): nobody waits, everybody
    //                     decodes, nobody reaches max_new_tokens or max_model_len with the next
    //                     token, every group has a free page for every running request;
    //   advance(plan)     the step was launched: its bookkeeping with a placeholder for each
    //                     token that is not known yet;
    //   resolve(plan, sampled, ahead)   the step's tokens are known; `ahead` steps (0 or 1) were
    //                     launched after it. A request that picked a stop token ends there:
    //                     what it was given in the steps launched since is dropped.
    bool steady_decode() const {
        if (!waiting_.empty() || running_.empty()) return false;
        for (int64_t id : running_) {
            const Request& r = requests_.at(id);
            if ((int)r.tokens.size() - r.computed != 1) return false;
            if (r.generated + 1 >= r.params.max_new_tokens) return false;
            if ((int)r.tokens.size() + 1 > max_model_len_) return false;
        }
        for (int g = 0; g < cache_->num_groups(); ++g)
            if (cache_->num_free_pages(g) < (int64_t)running_.size()) return false;
        return true;
    }

    void advance(const StepPlan& plan) {
        for (const auto& pe : plan.entries) {
            Request& r = requests_.at(pe.id);
            if (pe.count != 1 || !pe.sample) throw CacheError("advance: not a decode step");
            cache_->commit(pe.id, pe.count);
            r.computed += pe.count;
            r.tokens.push_back(0);           // placeholder until resolve()
            r.generated += 1;
        }
    }

    std::vector<Finished> resolve(const StepPlan& plan, const std::vector<int32_t>& sampled, int ahead) {
        std::vector<Finished> out;
        if (sampled.size() < plan.entries.size()) throw CacheError("resolve: fewer sampled tokens than entries");
        size_t si = 0;
        for (const auto& pe : plan.entries) {
            int32_t tok = sampled[si++];
            auto it = requests_.find(pe.id);
            if (it == requests_.end()) continue;                     // ended by an earlier resolve, or aborted
            Request& r = it->second;
            if ((int)r.tokens.size() < r.prompt_len + 1 + ahead) throw CacheError("resolve: no placeholder to fill");
            r.tokens[r.tokens.size() - 1 - ahead] = tok;
            const auto& stops = r.params.stop_token_ids;
            if (std::find(stops.begin(), stops.end(), tok) == stops.end()) continue;
            r.tokens.resize(r.tokens.size() - ahead);
            r.generated -= ahead;
            Finished f{pe.id, "stop", generated_of(r)};
            cache_->release(pe.id);
            running_.erase(std::remove(running_.begin(), running_.end(), pe.id), running_.end());
            requests_.erase(it);
            out.push_back(std::move(f));
        }
        return out;
    }

    // Requests finished without a step (capacity failures found while planning).
    std::vector<Finished> take_done() {
        std::vector<Finished> out;
        out.swap(done_);
        return out;
    }

    bool abort(int64_t id) {
        auto it = requests_.find(id);
        if (it == requests_.end()) return false;
        if (cache_->has(id)) cache_->release(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        waiting_.erase(std::remove(waiting_.begin(), waiting_.end(), id), waiting_.end());
        done_.push_back(Finished{id, "abort", generated_of(it->second)});
        requests_.erase(it);
        return true;
    }

private:
    static bool planned(const StepPlan& plan, int64_t id) {
        for (const auto& e : plan.entries) if (e.id == id) return true;
        return false;
    }
    static std::vector<int32_t> generated_of(const Request& r) {
        return std::vector<int32_t>(r.tokens.begin() + r.prompt_len, r.tokens.end());
    }
    void unplan(StepPlan& plan, int64_t id) {
        plan.entries.erase(std::remove_if(plan.entries.begin(), plan.entries.end(),
                                          [&](const PlannedEntry& e) { return e.id == id; }), plan.entries.end());
    }
    // Returns the tokens of this step's budget that the victim had been given.
    int preempt(int64_t id, StepPlan& plan) {
        Request& r = requests_.at(id);
        int freed = 0;
        for (const auto& e : plan.entries) if (e.id == id) freed += e.count;
        unplan(plan, id);
        cache_->release(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        r.computed = 0;                // recompute: prompt plus what was generated
        r.preemptions += 1;
        waiting_.push_front(id);
        plan.preempted.push_back(id);
        plan.admitted.erase(std::remove(plan.admitted.begin(), plan.admitted.end(), id), plan.admitted.end());
        return freed;
    }
    void finish_now(int64_t id, const std::string& reason, StepPlan& plan) {
        Request& r = requests_.at(id);
        unplan(plan, id);
        done_.push_back(Finished{id, reason, generated_of(r)});
        plan.failed.emplace_back(id, reason);
        cache_->release(id);
        running_.erase(std::remove(running_.begin(), running_.end(), id), running_.end());
        requests_.erase(id);
    }

    CacheManager* cache_;
    int max_batch_tokens_, max_seqs_, max_model_len_, prefill_chunk_;
    int watermark_pages_ = 0;
    std::map<int64_t, Request> requests_;
    std::deque<int64_t> waiting_;
    std::vector<int64_t> running_;
    std::vector<Finished> done_;
};

}  // namespace vob
