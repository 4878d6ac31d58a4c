// The arrays one step hands to the device, built on the host from (request, next tokens) pairs.
//
// They are the reference's per-step metadata (crates/engine/src/backend/paged.rs:97-143:
// positions, slot_mapping, row_seq, seq_row_starts, context_lens, block_tables), for a batch in
// which a portion of a prompt and a single decoded token are the same thing: `num_new` tokens
// after `context_len` cached ones. Everything is int32 and lives in ONE packed buffer, so a step
// costs one host-to-device copy; the section offsets depend only on the capacities
// (rows, requests, logit rows) the buffer was laid out for, which keeps device addresses fixed
// for steps of the same capacity class.
#pragma once
#include <cstring>
#include "cache_manager.h"

namespace vob {

struct StepEntry {
    int64_t id = 0;
    std::vector<int32_t> tokens;      // this step's new tokens of the request
    std::vector<int32_t> want;        // indices into `tokens` whose logits are wanted
    float temperature = 0.f;          // per wanted row: how a token is picked from it
    uint64_t seed = 0;
    int32_t sample_step = 0;          // index of the generated token this pick makes
};

struct StepLayout {
    int rows_cap = 0, seqs_cap = 0, logits_cap = 0, groups = 0, max_pages = 0;
    // offsets in int32 units
    int tokens = 0, positions = 0, row_seq = 0, seq_starts = 0, context_lens = 0, seq_lens = 0,
        state_slots = 0, logit_rows = 0, temperature = 0, seeds = 0, sample_steps = 0;
    std::vector<int> slot_mapping, block_tables;   // per group
    int total = 0;

    static int align4(int x) { return (x + 3) & ~3; }

    static StepLayout make(int rows_cap, int seqs_cap, int logits_cap, int groups, int max_pages) {
        StepLayout L;
        L.rows_cap = rows_cap; L.seqs_cap = seqs_cap; L.logits_cap = logits_cap;
        L.groups = groups; L.max_pages = max_pages;
        int o = 0;
        auto take = [&](int n) { int at = o; o = align4(o + n); return at; };
        L.tokens = take(rows_cap);
        L.positions = take(rows_cap);
        L.row_seq = take(rows_cap);
        L.seq_starts = take(seqs_cap + 1);
        L.context_lens = take(seqs_cap);
        L.seq_lens = take(seqs_cap);
        L.state_slots = take(seqs_cap);
        L.logit_rows = take(logits_cap);
        L.temperature = take(logits_cap);
        L.seeds = take(2 * logits_cap);
        L.sample_steps = take(logits_cap);
        for (int g = 0; g < groups; ++g) {
            L.slot_mapping.push_back(take(rows_cap));
            L.block_tables.push_back(take(seqs_cap * max_pages));
        }
        L.total = o;
        return L;
    }
};

struct StepArrays {
    StepLayout layout;
    std::vector<int32_t> data;      // layout.total ints
    int rows = 0, seqs = 0, logit_count = 0;
    int max_new = 0;                // longest portion in the batch
    int lead_single = 0;            // leading requests that bring exactly one token (rows 0 .. lead_single - 1)
    int64_t max_seq_len = 0;        // longest context after this step
    bool any_sampling = false;      // some row has temperature > 0
    std::vector<int64_t> ids;       // request of each sequence, in batch order
    std::vector<int32_t> new_counts;
    int used = 0;                   // ints from the start of `data` that this batch actually fills
};

// Lay the entries out. Every request must be admitted and must already hold pages for its new
// tokens (CacheManager::reserve). Rows beyond the real ones are padding: token 0, position -1
// (attention skips the row), request 0, no cache write.
inline StepArrays build_step(const CacheManager& cache, const std::vector<StepEntry>& entries,
                             int rows_cap, int seqs_cap, int logits_cap, int max_pages, int vocab_size) {
    StepArrays A;
    int T = 0, R = 0;
    for (const auto& e : entries) {
        if (e.tokens.empty()) throw CacheError("step: request " + std::to_string(e.id) + " brings no tokens");
        T += (int)e.tokens.size();
        R += (int)e.want.size();
    }
    int S = (int)entries.size();
    if (S == 0) throw CacheError("step: empty batch");
    if (T > rows_cap) throw CacheError("step: " + std::to_string(T) + " tokens exceed the limit of " + std::to_string(rows_cap));
    if (S > seqs_cap) throw CacheError("step: " + std::to_string(S) + " requests exceed the limit of " + std::to_string(seqs_cap));
    if (R > logits_cap) throw CacheError("step: " + std::to_string(R) + " logit rows exceed the limit of " + std::to_string(logits_cap));
    int G = cache.num_groups();
    A.layout = StepLayout::make(rows_cap, seqs_cap, logits_cap, G, max_pages);
    const StepLayout& L = A.layout;
    A.data.assign(L.total, 0);
    int32_t* d = A.data.data();
    for (int g = 0; g < G; ++g)
        for (int t = 0; t < rows_cap; ++t) d[L.slot_mapping[g] + t] = -1;
    for (int t = 0; t < rows_cap; ++t) d[L.positions + t] = -1;      // padding rows attend to nothing
    const int ps = cache.page_size();
    int row = 0, lr = 0;
    for (int s = 0; s < S; ++s) {
        const StepEntry& e = entries[s];
        for (int s2 = 0; s2 < s; ++s2)
            if (entries[s2].id == e.id) throw CacheError("step: request " + std::to_string(e.id) + " appears twice");
        const RequestPages& rp = cache.get(e.id);
        int n = (int)e.tokens.size();
        int64_t ctx = rp.len;
        if (ctx + n > rp.reserved)
            throw CacheError("step: request " + std::to_string(e.id) + " holds pages for " + std::to_string(rp.reserved) +
                             " tokens, the step needs " + std::to_string(ctx + n));
        if ((ctx + n + ps - 1) / ps > max_pages)
            throw CacheError("step: request " + std::to_string(e.id) + " needs more pages than a block table holds");
        d[L.seq_starts + s] = row;
        d[L.context_lens + s] = (int32_t)ctx;
        d[L.seq_lens + s] = (int32_t)(ctx + n);
        d[L.state_slots + s] = rp.slot;
        for (int g = 0; g < G; ++g) {
            const auto& tab = rp.tables[g];
            int32_t* bt = d + L.block_tables[g] + (size_t)s * max_pages;
            for (size_t i = 0; i < tab.size() && (int)i < max_pages; ++i) bt[i] = tab[i];
            for (int i = (int)tab.size(); i < max_pages; ++i) bt[i] = -1;
        }
        for (int i = 0; i < n; ++i) {
            int32_t tok = e.tokens[i];
            if (tok < 0 || tok >= vocab_size)
                throw CacheError("step: token " + std::to_string(tok) + " of request " + std::to_string(e.id) +
                                 " is outside the vocabulary of " + std::to_string(vocab_size));
            d[L.tokens + row] = tok;
            d[L.positions + row] = (int32_t)(ctx + i);
            d[L.row_seq + row] = s;
            for (int g = 0; g < G; ++g) d[L.slot_mapping[g] + row] = (int32_t)cache.slot_of(e.id, g, ctx + i);
            ++row;
        }
        for (int w : e.want) {
            if (w < 0 || w >= n) throw CacheError("step: wanted place " + std::to_string(w) + " is outside the " +
                                                  std::to_string(n) + " tokens of request " + std::to_string(e.id));
            d[L.logit_rows + lr] = d[L.seq_starts + s] + w;
            float temp = e.temperature;
            std::memcpy(&d[L.temperature + lr], &temp, 4);
            d[L.seeds + 2 * lr] = (int32_t)(uint32_t)(e.seed & 0xffffffffu);
            d[L.seeds + 2 * lr + 1] = (int32_t)(uint32_t)(e.seed >> 32);
            d[L.sample_steps + lr] = e.sample_step;
            if (temp > 0.f) A.any_sampling = true;
            ++lr;
        }
        A.max_new = std::max(A.max_new, n);
        if (n == 1 && A.lead_single == (int)A.ids.size()) ++A.lead_single;
        A.max_seq_len = std::max<int64_t>(A.max_seq_len, ctx + n);
        A.ids.push_back(e.id);
        A.new_counts.push_back(n);
    }
    d[L.seq_starts + S] = row;
    for (int s = S + 1; s <= seqs_cap; ++s) d[L.seq_starts + s] = row;
    // Padding rows carry position -1 and read no block table, so with one group (whose block
    // tables are the last section) only the first S rows of it need to reach the device.
    A.used = G == 1 ? L.block_tables[0] + S * max_pages : L.total;
    A.rows = T; A.seqs = S; A.logit_count = R;
    return A;
}

}  // namespace vob
