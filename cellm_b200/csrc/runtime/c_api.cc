// C entry points of the host runtime (cache manager and scheduler), called
// from Python through ctypes. Every function returns a status (0 or a count
// on success, negative on error); the message of the last error of the calling
// thread is read with cellm_last_error().
#include <algorithm>
#include <cstring>
#include <string>

#include "cache_manager.h"
#include "scheduler.h"

#define API extern "C" __attribute__((visibility("default")))

namespace {
thread_local std::string g_error;

// the step a scheduler planned last
const cellm::StepPlan& plan_of(void* s) { return static_cast<cellm::Scheduler*>(s)->last_plan(); }

template <typename F>
int guarded(F&& f) {
    try {
        return f();
    } catch (const std::exception& e) {
        g_error = e.what();
        return -1;
    } catch (...) {
        g_error = "unknown error";
        return -1;
    }
}
}  // namespace

API const char* cellm_last_error() { return g_error.c_str(); }

// ------------------------------------------------------------------ cache
API void* cellm_cache_create(int page_size, int n_groups, const int* pages, const int* windows, int num_slots) {
    try {
        std::vector<cellm::GroupSpec> groups;
        for (int g = 0; g < n_groups; ++g) groups.push_back({pages[g], windows[g]});
        return new cellm::CacheManager(page_size, std::move(groups), num_slots);
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}
API void cellm_cache_destroy(void* c) { delete static_cast<cellm::CacheManager*>(c); }
API int cellm_cache_add(void* c, long long id) {
    return guarded([&] {
        const int slot = static_cast<cellm::CacheManager*>(c)->add_request(id);
        if (slot < 0) { g_error = "cache: no free state slot"; return -2; }
        return slot;
    });
}
API int cellm_cache_reserve(void* c, long long id, int new_total) {
    return guarded([&] { return static_cast<cellm::CacheManager*>(c)->reserve(id, new_total) ? 1 : 0; });
}
API int cellm_cache_can_reserve(void* c, long long id, int new_total) {
    return guarded([&] { return static_cast<cellm::CacheManager*>(c)->can_reserve(id, new_total) ? 1 : 0; });
}
API int cellm_cache_commit(void* c, long long id, int new_total) {
    return guarded([&] { static_cast<cellm::CacheManager*>(c)->commit(id, new_total); return 0; });
}
API int cellm_cache_release(void* c, long long id) {
    return guarded([&] { static_cast<cellm::CacheManager*>(c)->release(id); return 0; });
}
API int cellm_cache_has(void* c, long long id) { return static_cast<cellm::CacheManager*>(c)->has(id) ? 1 : 0; }
API int cellm_cache_tokens(void* c, long long id) {
    return guarded([&] { return static_cast<cellm::CacheManager*>(c)->request(id).tokens; });
}
API int cellm_cache_slot(void* c, long long id) {
    return guarded([&] { return static_cast<cellm::CacheManager*>(c)->request(id).slot; });
}
// Copies the request's block table of group g into out (capacity cap); returns its length.
API int cellm_cache_block_table(void* c, long long id, int g, int* out, int cap) {
    return guarded([&] {
        const auto& b = static_cast<cellm::CacheManager*>(c)->request(id).blocks.at((size_t)g);
        if ((int)b.size() > cap) { g_error = "cache: block table longer than the buffer"; return -3; }
        if (!b.empty()) std::memcpy(out, b.data(), b.size() * sizeof(int));
        return (int)b.size();
    });
}
API int cellm_cache_free_pages(void* c, int g) {
    return guarded([&] { return static_cast<cellm::CacheManager*>(c)->free_pages(g); });
}
API int cellm_cache_free_slots(void* c) { return static_cast<cellm::CacheManager*>(c)->free_slots(); }
API int cellm_cache_live(void* c) { return static_cast<cellm::CacheManager*>(c)->live_requests(); }
API int cellm_cache_pages_for(void* c, int g, int tokens, int portion) {
    return guarded([&] { return static_cast<cellm::CacheManager*>(c)->pages_for(g, tokens, portion); });
}

// -------------------------------------------------------------- allocator
API void* cellm_alloc_create(int total) {
    try { return new cellm::BlockAllocator(total); } catch (const std::exception& e) { g_error = e.what(); return nullptr; }
}
API void cellm_alloc_destroy(void* a) { delete static_cast<cellm::BlockAllocator*>(a); }
API int cellm_alloc_alloc(void* a) { return static_cast<cellm::BlockAllocator*>(a)->alloc(); }
API int cellm_alloc_alloc_n(void* a, int n, int* out) {
    return guarded([&] {
        std::vector<int32_t> v;
        if (!static_cast<cellm::BlockAllocator*>(a)->alloc_n(n, v)) return 0;
        if (n > 0) std::memcpy(out, v.data(), (size_t)n * sizeof(int));
        return 1;
    });
}
API int cellm_alloc_free(void* a, int id) {
    return guarded([&] { static_cast<cellm::BlockAllocator*>(a)->free(id); return 0; });
}
API int cellm_alloc_free_count(void* a) { return static_cast<cellm::BlockAllocator*>(a)->free_count(); }
API int cellm_alloc_is_free(void* a, int id) {
    return guarded([&] { return static_cast<cellm::BlockAllocator*>(a)->is_free(id) ? 1 : 0; });
}

// -------------------------------------------------------------- scheduler
API void* cellm_sched_create(void* cache, int max_batch_tokens, int prefill_chunk, int max_positions) {
    try {
        cellm::SchedulerConfig cfg;
        cfg.max_batch_tokens = max_batch_tokens;
        cfg.prefill_chunk = prefill_chunk;
        cfg.max_positions = max_positions;
        return new cellm::Scheduler(cfg, static_cast<cellm::CacheManager*>(cache));
    } catch (const std::exception& e) {
        g_error = e.what();
        return nullptr;
    }
}
API void cellm_sched_destroy(void* s) { delete static_cast<cellm::Scheduler*>(s); }
API int cellm_sched_add(void* s, long long id, const int* tokens, int n, int max_new) {
    return guarded([&] { static_cast<cellm::Scheduler*>(s)->add_request(id, tokens, n, max_new); return 0; });
}
// Plans the next step; returns the number of entries. The scheduler keeps the plan, and its
// parts are then read with the *_plan_* calls on the same scheduler.
API int cellm_sched_schedule(void* s) {
    return guarded([&] { return (int)static_cast<cellm::Scheduler*>(s)->schedule().entries.size(); });
}
API int cellm_sched_plan_entries(void* s, long long* ids, int* starts, int* counts, int* wants, int cap) {
    const int n = (int)plan_of(s).entries.size();
    if (n > cap) return -3;
    for (int i = 0; i < n; ++i) {
        ids[i] = plan_of(s).entries[(size_t)i].id;
        starts[i] = plan_of(s).entries[(size_t)i].start;
        counts[i] = plan_of(s).entries[(size_t)i].count;
        wants[i] = plan_of(s).entries[(size_t)i].wants_logits;
    }
    return n;
}
API int cellm_sched_plan_preempted(void* s, long long* ids, int cap) {
    const int n = (int)plan_of(s).preempted.size();
    if (n > cap) return -3;
    for (int i = 0; i < n; ++i) ids[i] = plan_of(s).preempted[(size_t)i];
    return n;
}
API int cellm_sched_plan_admitted(void* s, long long* ids, int* slots, int cap) {
    const int n = (int)plan_of(s).admitted.size();
    if (n > cap) return -3;
    for (int i = 0; i < n; ++i) { ids[i] = plan_of(s).admitted[(size_t)i].first; slots[i] = plan_of(s).admitted[(size_t)i].second; }
    return n;
}
// Shape of the planned step: out[0..4] = entries, tokens, wanted rows, most tokens a
// request will hold after the step, 1 if every entry is one token whose logits are wanted.
API int cellm_sched_plan_shape(void* s, int* out) {
    int T = 0, R = 0, max_total = 0, all_decode = 1;
    for (const auto& e : plan_of(s).entries) {
        T += e.count;
        R += e.wants_logits ? 1 : 0;
        max_total = std::max(max_total, e.start + e.count);
        if (e.count != 1 || !e.wants_logits) all_decode = 0;
    }
    out[0] = (int)plan_of(s).entries.size(); out[1] = T; out[2] = R; out[3] = max_total; out[4] = all_decode;
    return 0;
}
// Writes the planned step's index arrays into buf, in the order the step function
// reads them: token ids [T], positions [T], entry of each token [T], cumulative
// lengths [B+1], tokens already cached [B], state slots [B], wanted rows [R], then one
// block table [B][width] per paged group (-1 where there is no page). Returns the
// number of ints written.
API int cellm_sched_plan_fill(void* s, int* buf, int cap, int width, int n_groups) {
    return guarded([&] {
        auto* sc = static_cast<cellm::Scheduler*>(s);
        const int B = (int)plan_of(s).entries.size();
        int T = 0, R = 0;
        for (const auto& e : plan_of(s).entries) { T += e.count; R += e.wants_logits ? 1 : 0; }
        const long long need = 3LL * T + (B + 1) + 2LL * B + R + (long long)n_groups * B * width;
        if (need > cap) { g_error = "scheduler: index buffer too small"; return -3; }
        int* ids = buf; int* pos = ids + T; int* seq = pos + T; int* cu = seq + T; int* ctx = cu + B + 1;
        int* slot = ctx + B; int* rows = slot + B; int* tabs = rows + R;
        int t = 0, r = 0;
        cu[0] = 0;
        for (int b = 0; b < B; ++b) {
            const auto& e = plan_of(s).entries[(size_t)b];
            const auto& rq = sc->request(e.id);
            const auto& rc = sc->cache().request(e.id);
            for (int i = 0; i < e.count; ++i, ++t) {
                ids[t] = rq.tokens[(size_t)(e.start + i)];
                pos[t] = e.start + i;
                seq[t] = b;
            }
            cu[b + 1] = t;
            ctx[b] = e.start;
            slot[b] = rc.slot;
            if (e.wants_logits) rows[r++] = t - 1;
            for (int g = 0; g < n_groups; ++g) {
                int* row = tabs + ((size_t)g * B + b) * width;
                const auto& blocks = rc.blocks.at((size_t)g);
                if ((int)blocks.size() > width) { g_error = "scheduler: block table wider than the buffer"; return -3; }
                for (int i = 0; i < width; ++i) row[i] = i < (int)blocks.size() ? blocks[(size_t)i] : -1;
            }
        }
        return (int)need;
    });
}
// Appends one sampled token per wanted row of the planned step, in the order of the
// entries; stops[i] != 0 ends request i. finished[i] becomes 1 where a request ended.
API int cellm_sched_append_rows(void* s, const int* tokens, const int* stops, int* finished, int n) {
    return guarded([&] {
        auto* sc = static_cast<cellm::Scheduler*>(s);
        int r = 0;
        for (const auto& e : plan_of(s).entries) {
            if (!e.wants_logits) continue;
            if (r >= n) { g_error = "scheduler: fewer tokens than wanted rows"; return -3; }
            // -2: the row's request ended meanwhile (a token of an earlier step, read after this step was planned,
            // ended it): nothing is appended
            if (tokens[r] == -2) { finished[r] = 1; ++r; continue; }
            finished[r] = sc->append_token(e.id, tokens[r], stops[r] != 0) ? 1 : 0;
            ++r;
        }
        return r;
    });
}
// The values of tokens that were appended as pending: request ids, their places in the requests' tokens, the
// values and whether each ends its request; finished[i] = 1 where the request is finished (or gone) afterwards.
API int cellm_sched_resolve_rows(void* s, const long long* ids, const int* index, const int* tokens, const int* stops,
                                 int* finished, int n) {
    return guarded([&] {
        auto* sc = static_cast<cellm::Scheduler*>(s);
        for (int i = 0; i < n; ++i) finished[i] = sc->resolve_token(ids[i], index[i], tokens[i], stops[i] != 0) ? 1 : 0;
        return n;
    });
}
API int cellm_sched_step_done(void* s) {
    return guarded([&] { static_cast<cellm::Scheduler*>(s)->step_done(plan_of(s)); return 0; });
}
API int cellm_sched_append(void* s, long long id, int token, int stop) {
    return guarded([&] { return static_cast<cellm::Scheduler*>(s)->append_token(id, token, stop != 0) ? 1 : 0; });
}
API int cellm_sched_cancel(void* s, long long id) {
    return guarded([&] { static_cast<cellm::Scheduler*>(s)->cancel(id); return 0; });
}
API int cellm_sched_forget(void* s, long long id) {
    return guarded([&] { static_cast<cellm::Scheduler*>(s)->forget(id); return 0; });
}
API int cellm_sched_has(void* s, long long id) { return static_cast<cellm::Scheduler*>(s)->has(id) ? 1 : 0; }
// info[0..5] = state, prompt_len, number of tokens, computed, generated, preemptions
API int cellm_sched_info(void* s, long long id, int* info) {
    return guarded([&] {
        const auto& r = static_cast<cellm::Scheduler*>(s)->request(id);
        info[0] = (int)r.state; info[1] = r.prompt_len; info[2] = (int)r.tokens.size();
        info[3] = r.computed; info[4] = r.generated; info[5] = r.preemptions;
        return 0;
    });
}
API int cellm_sched_tokens(void* s, long long id, int from, int* out, int cap) {
    return guarded([&] {
        const auto& r = static_cast<cellm::Scheduler*>(s)->request(id);
        const int n = (int)r.tokens.size() - from;
        if (from < 0 || n < 0) { g_error = "scheduler: token range out of bounds"; return -3; }
        if (n > cap) { g_error = "scheduler: token buffer too small"; return -3; }
        if (n > 0) std::memcpy(out, r.tokens.data() + from, (size_t)n * sizeof(int));
        return n;
    });
}
API const char* cellm_sched_finish_reason(void* s, long long id) {
    try { return static_cast<cellm::Scheduler*>(s)->request(id).finish_reason.c_str(); } catch (...) { return ""; }
}
// stats[0..5] = waiting, running, steps, tokens scheduled, preemptions, idle
API void cellm_sched_stats(void* s, long long* stats) {
    auto* sc = static_cast<cellm::Scheduler*>(s);
    stats[0] = sc->num_waiting(); stats[1] = sc->num_running(); stats[2] = (long long)sc->steps();
    stats[3] = (long long)sc->tokens_scheduled(); stats[4] = (long long)sc->preemptions(); stats[5] = sc->idle() ? 1 : 0;
}

// ------------------------------------------------------------------ executor
#include "executor.h"

// Sizes of the executor's structs, for the caller to check its own layout against: 0 ExecLinear, 1 ExecOp,
// 2 ExecProgram, 3 ExecItem, 4 ExecStep, 5 ExecRegs, 6 EmbedParams, 7 RmsNormParams, 8 ShortConvParams,
// 9 AttentionParams, 10 SwiGLUParams, 11 HeadParams, 12 PythonParams, 13 ExecOps, 14 LinearParams.
API long long cellm_exec_sizeof(int which) {
    switch (which) {
        case 0: return sizeof(cellm::ExecLinear);
        case 1: return sizeof(cellm::ExecOp);
        case 2: return sizeof(cellm::ExecProgram);
        case 3: return sizeof(cellm::ExecItem);
        case 4: return sizeof(cellm::ExecStep);
        case 5: return sizeof(cellm::ExecRegs);
        case 6: return sizeof(cellm::EmbedParams);
        case 7: return sizeof(cellm::RmsNormParams);
        case 8: return sizeof(cellm::ShortConvParams);
        case 9: return sizeof(cellm::AttentionParams);
        case 10: return sizeof(cellm::SwiGLUParams);
        case 11: return sizeof(cellm::HeadParams);
        case 12: return sizeof(cellm::PythonParams);
        case 13: return sizeof(cellm::ExecOps);
        case 14: return sizeof(cellm::LinearParams);
        default: return -1;
    }
}
// What a step needs (see exec_need): out[0] arena bytes, out[1] and out[2] workspace floats. Launches nothing.
API int cellm_exec_need(const void* program, void* step, long long* out) {
    return guarded([&] {
        cellm::exec_need(*static_cast<const cellm::ExecProgram*>(program), *static_cast<cellm::ExecStep*>(step), out);
        return 0;
    });
}
// Runs one step's forward pass; 0, or -1 with the reason in cellm_last_error().
API int cellm_exec_forward(const void* program, void* step) {
    return guarded([&] {
        return cellm::exec_forward(*static_cast<const cellm::ExecProgram*>(program), *static_cast<cellm::ExecStep*>(step));
    });
}
// One mixer or feed-forward record by itself (see exec_part); with dry != 0 it only fills need[0..2].
API int cellm_exec_part(const void* program, void* step, const void* op, const void* y_in, void* out, int dry, long long* need) {
    return guarded([&] {
        return cellm::exec_part(*static_cast<const cellm::ExecProgram*>(program), *static_cast<cellm::ExecStep*>(step),
                                *static_cast<const cellm::ExecOp*>(op), y_in, out, dry != 0, need);
    });
}
API int cellm_exec_plan_tiles(long long M, long long N, long long K, long long sms, long long* out) {
    cellm::plan_tiles(M, N, K, sms, &out[0], &out[1]);
    return 0;
}
