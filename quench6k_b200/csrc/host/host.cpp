// The host side of the engine in C++: the paged cache manager, the continuous-batching scheduler,
// the packing of a step's description and the choice of a token from a candidate pool, behind a
// C interface that Python calls through ctypes.
//
// The reference's host is Rust (crates/engine/src/flint.rs: contiguous per-sequence caches, one
// request at a time; crates/engine/src/session.rs and crates/cli/src/serve.rs: admission by memory
// plan, finish reasons Stop / Length / Cancelled).  The rules implemented here are this engine's own
// and are stated at each class; quench6k_b200/cache/manager.py and engine/scheduler.py hold a Python
// twin with the same rules, and the tests run both.
//
// Every exported function returns 0 or an error kind after storing a message:
//   1 runtime error, 2 out of pages, 3 out of slots, 4 unknown or duplicate request, 5 bad value.
#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <memory>
#include <string>
#include <unordered_map>
#include <vector>

#include <fcntl.h>
#include <sys/stat.h>
#include <unistd.h>
#include <cmath>
#include <thread>

#include "../fill_normal.h"


#define API extern "C" __attribute__((visibility("default")))

namespace {

enum { OK = 0, E_RUNTIME = 1, E_PAGES = 2, E_SLOTS = 3, E_KEY = 4, E_VALUE = 5 };

thread_local char g_msg[512] = "";

int fail(int kind, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_msg, sizeof g_msg, fmt, ap);
    va_end(ap);
    return kind;
}

// ---------------------------------------------------------------------------------------------
// Pages of one cache group: ids 0..n-1, a LIFO free list (a page that was just given back is the
// next one handed out; a request that takes several pages at once gets ascending numbers whenever
// they were returned in descending order), every page free or owned by exactly one request.
struct PagePool {
    int n = 0;
    std::vector<int> free_;
    std::vector<int64_t> owner;          // -1: free
    explicit PagePool(int count) : n(count), owner(count, -1) {
        free_.reserve(count);
        for (int p = count - 1; p >= 0; --p) free_.push_back(p);
    }
    int num_free() const { return (int)free_.size(); }
    int take(int64_t who) {
        const int page = free_.back();
        free_.pop_back();
        owner[page] = who;
        return page;
    }
    int give_back(int page, int64_t who) {
        if (page < 0 || page >= n) return fail(E_VALUE, "page %d outside the pool", page);
        if (owner[page] < 0) return fail(E_RUNTIME, "page %d freed twice", page);
        if (owner[page] != who) return fail(E_RUNTIME, "page %d belongs to request %lld, not %lld", page, (long long)owner[page], (long long)who);
        owner[page] = -1;
        free_.push_back(page);
        return OK;
    }
};

struct BlockTable {
    std::vector<int32_t> pages;          // by logical block; -1 where the page was given back
    int first_held = 0;                  // blocks [0, first_held) were given back
};

struct CacheRequest {
    int slot = -1;
    int64_t length = 0;                  // tokens whose keys are in the cache
    int reserved = 0;                    // tokens of the step in flight
    std::vector<BlockTable> tables;      // per group
};

struct Group {
    int sliding = 0;                     // 0: a request holds pages for every position; 1: only for the last `window`
    int window = 0;
};

// Keys and values in pages with a block table per request and group; a sliding group gives pages
// back as soon as no later query can see them; one state slot per request.
struct CacheManager {
    int page_size;
    std::vector<Group> groups;
    std::vector<PagePool> pools;
    int num_slots;
    std::vector<int> free_slots;
    std::unordered_map<int64_t, CacheRequest> requests;

    CacheRequest* find(int64_t id) {
        auto it = requests.find(id);
        return it == requests.end() ? nullptr : &it->second;
    }
    int first_needed_block(int g, int64_t start) const {
        if (!groups[g].sliding) return 0;
        const int64_t lo = start - groups[g].window + 1;
        return (int)((lo < 0 ? 0 : lo) / page_size);
    }
    int add(int64_t id, int* slot) {
        if (requests.count(id)) return fail(E_KEY, "request %lld is already live", (long long)id);
        if (free_slots.empty()) return fail(E_SLOTS, "all %d request slots are in use", num_slots);
        CacheRequest r;
        r.slot = free_slots.back();
        free_slots.pop_back();
        r.tables.resize(groups.size());
        *slot = r.slot;
        requests.emplace(id, std::move(r));
        return OK;
    }
    int remove(int64_t id) {
        CacheRequest* r = find(id);
        if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
        for (size_t g = 0; g < groups.size(); ++g) {
            BlockTable& t = r->tables[g];
            for (int b = (int)t.pages.size() - 1; b >= t.first_held; --b)
                if (int rc = pools[g].give_back(t.pages[b], id)) return rc;
        }
        free_slots.push_back(r->slot);
        requests.erase(id);
        return OK;
    }
    // Pages each pool must supply so that the request can run n_new more tokens: a table holds a
    // page for every block from the first one the next step reads up to its end, so the need is the
    // blocks past the table's end.
    int pages_needed(int64_t id, int n_new, int* out) {
        CacheRequest* r = find(id);
        if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
        const int64_t end = r->length + n_new;
        const int last = end > 0 ? (int)((end - 1) / page_size) : -1;
        for (size_t g = 0; g < groups.size(); ++g) {
            if (first_needed_block((int)g, r->length) < r->tables[g].first_held)
                return fail(E_RUNTIME, "a block the next step of request %lld reads was given back", (long long)id);
            const int have = (int)r->tables[g].pages.size();
            out[g] = last + 1 > have ? last + 1 - have : 0;
        }
        return OK;
    }
    int can_reserve(const int64_t* ids, const int* ns, int m, int* yes) {
        std::vector<int> total(groups.size(), 0), need(groups.size());
        for (int i = 0; i < m; ++i) {
            if (int rc = pages_needed(ids[i], ns[i], need.data())) return rc;
            for (size_t g = 0; g < groups.size(); ++g) total[g] += need[g];
        }
        *yes = 1;
        for (size_t g = 0; g < groups.size(); ++g)
            if (total[g] > pools[g].num_free()) *yes = 0;
        return OK;
    }
    // All groups or none: on failure nothing has changed.
    int reserve(int64_t id, int n_new) {
        CacheRequest* r = find(id);
        if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
        if (r->reserved) return fail(E_RUNTIME, "request %lld already has a step in flight", (long long)id);
        std::vector<int> need(groups.size());
        if (int rc = pages_needed(id, n_new, need.data())) return rc;
        for (size_t g = 0; g < groups.size(); ++g)
            if (need[g] > pools[g].num_free())
                return fail(E_PAGES, "group %d (%s) needs %d pages for request %lld, %d are free", (int)g,
                            groups[g].sliding ? "sliding" : "full", need[g], (long long)id, pools[g].num_free());
        for (size_t g = 0; g < groups.size(); ++g)
            for (int i = 0; i < need[g]; ++i) r->tables[g].pages.push_back(pools[g].take(id));
        r->reserved = n_new;
        return OK;
    }
    int commit(int64_t id) {
        CacheRequest* r = find(id);
        if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
        r->length += r->reserved;
        r->reserved = 0;
        for (size_t g = 0; g < groups.size(); ++g) {
            if (!groups[g].sliding) continue;
            // the next query sits at position `length` and sees keys > length - window
            const int64_t lo = r->length - groups[g].window + 1;
            BlockTable& t = r->tables[g];
            int dead = (int)((lo < 0 ? 0 : lo) / page_size);
            if (dead > (int)t.pages.size()) dead = (int)t.pages.size();
            for (int b = t.first_held; b < dead; ++b) {
                if (int rc = pools[g].give_back(t.pages[b], id)) return rc;
                t.pages[b] = -1;
            }
            if (dead > t.first_held) t.first_held = dead;
        }
        return OK;
    }
    int cancel(int64_t id) {
        CacheRequest* r = find(id);
        if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
        r->reserved = 0;
        return OK;
    }
    // No page lost, held twice, or both free and held; no slot lost or held twice.
    int check() {
        for (size_t g = 0; g < groups.size(); ++g) {
            PagePool& pool = pools[g];
            std::vector<int> seen(pool.n, 0);
            int held = 0;
            for (auto& kv : requests) {
                const BlockTable& t = kv.second.tables[g];
                for (int b = 0; b < (int)t.pages.size(); ++b) {
                    const int page = t.pages[b];
                    if ((page < 0) != (b < t.first_held))
                        return fail(E_RUNTIME, "group %d: request %lld block %d page %d first_held %d", (int)g, (long long)kv.first, b, page, t.first_held);
                    if (page < 0) continue;
                    if (page >= pool.n || seen[page]++) return fail(E_RUNTIME, "group %d: page %d held twice", (int)g, page);
                    if (pool.owner[page] != kv.first) return fail(E_RUNTIME, "group %d: page %d owner %lld != %lld", (int)g, page, (long long)pool.owner[page], (long long)kv.first);
                    ++held;
                }
            }
            for (int page : pool.free_) {
                if (seen[page] == 1) return fail(E_RUNTIME, "group %d: page %d is both free and held", (int)g, page);
                if (seen[page] == 2) return fail(E_RUNTIME, "group %d: page %d is twice in the free list", (int)g, page);
                seen[page] = 2;
            }
            if ((int)pool.free_.size() + held != pool.n) return fail(E_RUNTIME, "group %d: %d pages lost", (int)g, pool.n - (int)pool.free_.size() - held);
        }
        std::vector<int> slot_seen(num_slots, 0);
        for (auto& kv : requests)
            if (slot_seen[kv.second.slot]++) return fail(E_RUNTIME, "state slot %d is held twice", kv.second.slot);
        if ((int)requests.size() + (int)free_slots.size() != num_slots) return fail(E_RUNTIME, "a state slot is lost");
        return OK;
    }
};

// ---------------------------------------------------------------------------------------------
enum { FINISH_NONE = 0, FINISH_STOP = 1, FINISH_LENGTH = 2, FINISH_CANCELLED = 3 };

struct SchedRequest {
    int64_t id = 0;
    std::vector<int32_t> prompt, output, stops;
    int max_tokens = 0;
    int64_t num_computed = 0;
    int preemptions = 0;
    int finish = FINISH_NONE;
    int64_t num_tokens() const { return (int64_t)prompt.size() + (int64_t)output.size(); }
    int32_t token(int64_t i) const { return i < (int64_t)prompt.size() ? prompt[i] : output[i - prompt.size()]; }
};

struct Entry {
    int64_t id;
    int64_t start;
    int count;
    int samples;
};

// Continuous batching under a token budget: every running request whose prompt is in the cache
// decodes one token; what is left goes to prompt portions, first of running requests that are
// still prefilling (admission order), then of waiting requests, admitted first come first served
// while a slot, budget and pages for the portion are there (a portion shrinks to what the pools
// hold).  When pages run out for the decode tokens the most recently admitted running request is
// preempted (pages and slot back, to the front of the queue, recomputed from its tokens); a
// request running alone that cannot get a page ends with reason "length".
struct Scheduler {
    CacheManager* cm;
    int max_batch_tokens, max_running;
    std::deque<int64_t> waiting;
    std::vector<int64_t> running;                 // admission order
    std::unordered_map<int64_t, SchedRequest> by_id;
    std::vector<Entry> last;                      // the entries of the step in flight

    // Most tokens one request can ever hold: the smallest pool of a group that keeps every key bounds it.  A sliding
    // group holds a window's worth of pages whatever the length, so its (smaller) pool bounds nothing.
    int64_t capacity_tokens() const {
        int64_t least = (int64_t)1 << 60;
        for (size_t g = 0; g < cm->pools.size(); ++g)
            if (!cm->groups[g].sliding) least = std::min<int64_t>(least, (int64_t)cm->pools[g].n * cm->page_size);
        return least;
    }
    // A sliding group must hold its window and one more token wherever they lie on the pages, or no request could ever advance.
    int check_pools() const {
        for (size_t g = 0; g < cm->pools.size(); ++g) {
            if (!cm->groups[g].sliding) continue;
            const int need = (cm->groups[g].window + cm->page_size - 1) / cm->page_size + 1;
            if (cm->pools[g].n < need)
                return fail(E_VALUE, "cache group %d: %d pages cannot hold a window of %d keys and the next token (%d pages of %d)", (int)g,
                            cm->pools[g].n, cm->groups[g].window, need, cm->page_size);
        }
        return OK;
    }
    int release(int64_t id) { return cm->remove(id); }
    int finish(SchedRequest& r, int reason) {
        r.finish = reason;
        auto it = std::find(running.begin(), running.end(), r.id);
        if (it != running.end()) {
            running.erase(it);
            if (int rc = release(r.id)) return rc;
        } else {
            auto w = std::find(waiting.begin(), waiting.end(), r.id);
            if (w != waiting.end()) waiting.erase(w);
        }
        return OK;
    }
    int preempt(SchedRequest& r) {
        running.erase(std::find(running.begin(), running.end(), r.id));
        if (int rc = release(r.id)) return rc;
        r.num_computed = 0;
        r.preemptions += 1;
        waiting.push_front(r.id);
        return OK;
    }
    bool fits(std::vector<int64_t>& ids, std::vector<int>& ns, int64_t id, int n) {
        ids.push_back(id), ns.push_back(n);
        int yes = 0;
        cm->can_reserve(ids.data(), ns.data(), (int)ids.size(), &yes);
        ids.pop_back(), ns.pop_back();
        return yes != 0;
    }
    // Largest n <= want such that the pools hold the chosen entries plus n tokens of id.
    int fit(std::vector<int64_t>& ids, std::vector<int>& ns, int64_t id, int want) {
        if (want <= 0) return 0;
        if (fits(ids, ns, id, want)) return want;
        int lo = 0, hi = want;
        while (lo < hi) {
            const int mid = (lo + hi + 1) / 2;
            if (fits(ids, ns, id, mid)) lo = mid;
            else hi = mid - 1;
        }
        return lo;
    }
    int schedule(std::vector<Entry>& entries, std::vector<int64_t>& preempted, std::vector<int64_t>& finished,
                 std::vector<int64_t>& admitted, std::vector<int>& admitted_slots) {
        int budget = max_batch_tokens;
        std::vector<int64_t> ids;
        std::vector<int> ns;
        std::vector<SchedRequest*> decoding;
        while (true) {
            decoding.clear(), ids.clear(), ns.clear();
            for (int64_t id : running) {
                SchedRequest& r = by_id[id];
                if (r.num_computed == r.num_tokens() - 1 && !r.output.empty() && (int)decoding.size() < budget) decoding.push_back(&r);
            }
            for (auto* r : decoding) ids.push_back(r->id), ns.push_back(1);
            int yes = 0;
            if (int rc = cm->can_reserve(ids.data(), ns.data(), (int)ids.size(), &yes)) return rc;
            if (yes) break;
            if (running.size() == 1) {
                SchedRequest& lone = by_id[running[0]];
                if (int rc = finish(lone, FINISH_LENGTH)) return rc;
                finished.push_back(lone.id);
                continue;
            }
            SchedRequest& victim = by_id[running.back()];
            if (int rc = preempt(victim)) return rc;
            preempted.push_back(victim.id);
        }
        for (auto* r : decoding) entries.push_back({r->id, r->num_computed, 1, 1});
        budget -= (int)decoding.size();
        std::vector<int64_t> in_step(ids);
        // prompt portions of running requests still prefilling
        for (int64_t id : running) {
            if (budget <= 0) break;
            if (std::find(in_step.begin(), in_step.end(), id) != in_step.end()) continue;
            SchedRequest& r = by_id[id];
            const int64_t left = r.num_tokens() - r.num_computed;
            const int n = fit(ids, ns, id, (int)std::min<int64_t>(left, budget));
            if (n <= 0) continue;
            entries.push_back({id, r.num_computed, n, n == left});
            ids.push_back(id), ns.push_back(n), in_step.push_back(id);
            budget -= n;
        }
        // admit waiting requests, first come first served
        while (!waiting.empty() && budget > 0 && (int)running.size() < max_running && !cm->free_slots.empty()) {
            SchedRequest& r = by_id[waiting.front()];
            int slot = -1;
            if (int rc = cm->add(r.id, &slot)) return rc;
            const int64_t left = r.num_tokens();
            const int n = fit(ids, ns, r.id, (int)std::min<int64_t>(left, budget));
            if (n <= 0) {
                if (int rc = cm->remove(r.id)) return rc;
                break;                   // the head of the queue waits; nobody overtakes it
            }
            waiting.pop_front();
            running.push_back(r.id);
            admitted.push_back(r.id), admitted_slots.push_back(slot);
            entries.push_back({r.id, 0, n, n == left});
            ids.push_back(r.id), ns.push_back(n);
            budget -= n;
        }
        if (entries.empty() && finished.empty() && !running.empty()) {
            // every running request is mid-prefill and no page is free: make room from the back
            if (running.size() > 1) {
                SchedRequest& victim = by_id[running.back()];
                if (int rc = preempt(victim)) return rc;
                preempted.push_back(victim.id);
                return schedule(entries, preempted, finished, admitted, admitted_slots);
            }
            SchedRequest& lone = by_id[running[0]];
            if (int rc = finish(lone, FINISH_LENGTH)) return rc;
            finished.push_back(lone.id);
        }
        return OK;
    }
    // One sampled token per entry with samples = 1, in order.
    int update(const int32_t* sampled, int n_sampled, std::vector<int64_t>& done, std::vector<int>& reasons) {
        int at = 0;
        const int64_t cap = capacity_tokens();
        for (const Entry& e : last) {
            auto it = by_id.find(e.id);
            if (it == by_id.end() || it->second.finish != FINISH_NONE) {      // aborted while the step ran
                if (e.samples) ++at;
                continue;
            }
            SchedRequest& r = it->second;
            r.num_computed += e.count;
            if (!e.samples) continue;
            if (at >= n_sampled) return fail(E_VALUE, "update got %d sampled tokens, the step has more sampling entries", n_sampled);
            const int32_t tok = sampled[at++];
            r.output.push_back(tok);
            int reason = FINISH_NONE;
            if (std::find(r.stops.begin(), r.stops.end(), tok) != r.stops.end()) reason = FINISH_STOP;
            else if ((int)r.output.size() >= r.max_tokens) reason = FINISH_LENGTH;
            else if (r.num_tokens() + 1 > cap) reason = FINISH_LENGTH;
            if (reason != FINISH_NONE) {
                if (int rc = finish(r, reason)) return rc;
                done.push_back(r.id), reasons.push_back(reason);
            }
        }
        last.clear();
        return OK;
    }
};

template <typename T>
int copy_out(const std::vector<T>& v, T* out, int cap, int* n, const char* what) {
    if ((int)v.size() > cap) return fail(E_VALUE, "%s: %d results exceed the caller's room for %d", what, (int)v.size(), cap);
    std::copy(v.begin(), v.end(), out);
    *n = (int)v.size();
    return OK;
}

}  // namespace

API const char* q6k_host_last_error() { return g_msg; }
API int q6k_host_abi_version() { return 5; }

// ------------------------------------------------------------------------------- cache manager
API void* q6k_cm_create(int n_groups, const int* sliding, const int* windows, int page_size, const int* num_pages, int max_requests) {
    if (page_size <= 0 || n_groups < 0 || max_requests <= 0) {
        fail(E_VALUE, "cache manager: bad sizes (page_size %d, groups %d, requests %d)", page_size, n_groups, max_requests);
        return nullptr;
    }
    auto* cm = new CacheManager();
    cm->page_size = page_size;
    for (int g = 0; g < n_groups; ++g) {
        if (sliding[g] && windows[g] <= 0) {
            fail(E_VALUE, "a sliding group needs a positive window");
            delete cm;
            return nullptr;
        }
        cm->groups.push_back({sliding[g], windows[g]});
        cm->pools.emplace_back(num_pages[g]);
    }
    cm->num_slots = max_requests;
    for (int s = max_requests - 1; s >= 0; --s) cm->free_slots.push_back(s);
    return cm;
}
API void q6k_cm_destroy(void* h) { delete (CacheManager*)h; }
API int q6k_cm_add(void* h, int64_t id, int* slot) { return ((CacheManager*)h)->add(id, slot); }
API int q6k_cm_remove(void* h, int64_t id) { return ((CacheManager*)h)->remove(id); }
API int q6k_cm_info(void* h, int64_t id, int64_t* length, int* slot) {
    CacheRequest* r = ((CacheManager*)h)->find(id);
    if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
    *length = r->length, *slot = r->slot;
    return OK;
}
API int q6k_cm_pages_needed(void* h, int64_t id, int n_new, int* out) { return ((CacheManager*)h)->pages_needed(id, n_new, out); }
API int q6k_cm_can_reserve(void* h, const int64_t* ids, const int* ns, int m, int* yes) { return ((CacheManager*)h)->can_reserve(ids, ns, m, yes); }
API int q6k_cm_reserve(void* h, int64_t id, int n) { return ((CacheManager*)h)->reserve(id, n); }
API int q6k_cm_commit(void* h, int64_t id) { return ((CacheManager*)h)->commit(id); }
API int q6k_cm_cancel(void* h, int64_t id) { return ((CacheManager*)h)->cancel(id); }
API int q6k_cm_check(void* h) { return ((CacheManager*)h)->check(); }
API int q6k_cm_num_free(void* h, int group) { return ((CacheManager*)h)->pools[group].num_free(); }
API int q6k_cm_slots_free(void* h) { return (int)((CacheManager*)h)->free_slots.size(); }
API int q6k_cm_num_live(void* h) { return (int)((CacheManager*)h)->requests.size(); }
// A view of a request's block table in one group: valid until the request's next reserve or removal.
API int q6k_cm_table(void* h, int64_t id, int group, const int32_t** pages, int* len) {
    CacheRequest* r = ((CacheManager*)h)->find(id);
    if (!r) return fail(E_KEY, "request %lld is not live", (long long)id);
    *pages = r->tables[group].pages.data();
    *len = (int)r->tables[group].pages.size();
    return OK;
}

// The step's description as one int32 block (what the step function uploads in one copy):
// [tokens T | positions T | request of token T | q_start R+1 | pos_start R | slot R | logit rows W |
//  block table of group 0: R x widths[0] | group 1 ...], -1 where a table has no page.
// tokens: the entries' tokens back to back; want: for each entry want_counts[r] indices into its
// tokens.  meta: [total ints, T, wanted rows, max context, max q_len].  feed_limit > 0 admits token
// ids -1 .. -feed_limit: "the i-th token the step before has sampled", resolved on the device.
// pad > 0 appends that many filler entries after the R real ones (so that batches of nearby sizes share one recorded
// shape): one token 0 at position 0 each, its logits wanted, state slot pad_slot, one page pad_pages[g] per group
// (a page and a slot outside the manager's pools, which the caller sets aside; what the fillers compute is dropped).
API int q6k_cm_fill_step(void* h, int R, const int64_t* ids, const int* q_lens, const int32_t* tokens, const int* want,
                         const int* want_counts, const int* widths, int vocab, int feed_limit, int pad, const int* pad_pages,
                         int pad_slot, int32_t* out, int64_t capacity, int64_t* meta) {
    CacheManager* cm = (CacheManager*)h;
    if (pad < 0 || (pad > 0 && !pad_pages)) return fail(E_VALUE, "bad number of filler entries %d", pad);
    int64_t T = pad, W = pad;
    for (int r = 0; r < R; ++r) T += q_lens[r], W += want_counts[r];
    const int real = R;
    R += pad;
    int64_t total = 3 * T + (R + 1) + 2 * R + W;
    for (size_t g = 0; g < cm->groups.size(); ++g) total += (int64_t)R * widths[g];
    if (total > capacity) return fail(E_VALUE, "the step needs %lld ints, the block holds %lld", (long long)total, (long long)capacity);
    int32_t *tok = out, *pos = tok + T, *rot = pos + T, *qs = rot + T, *ps = qs + R + 1, *sl = ps + R, *lr = sl + R, *tab = lr + W;
    int64_t t = 0, w = 0, max_ctx = 0, max_q = 0, wi = 0;
    qs[0] = 0;
    for (int r = 0; r < real; ++r) {
        CacheRequest* cr = cm->find(ids[r]);
        if (!cr) return fail(E_KEY, "request %lld is not live", (long long)ids[r]);
        const int n = q_lens[r];
        for (int i = 0; i < n; ++i) {
            const int32_t v = tokens[t + i];
            if (v < -feed_limit || v >= vocab) return fail(E_VALUE, "request %lld: token id %d outside 0..%d", (long long)ids[r], v, vocab - 1);
            tok[t + i] = v, pos[t + i] = (int32_t)(cr->length + i), rot[t + i] = r;
        }
        for (int i = 0; i < want_counts[r]; ++i) {
            const int at = want[wi++];
            if (at < 0 || at >= n) return fail(E_VALUE, "request %lld: wanted place %d outside its %d tokens", (long long)ids[r], at, n);
            lr[w++] = (int32_t)(t + at);
        }
        t += n;
        qs[r + 1] = (int32_t)t, ps[r] = (int32_t)cr->length, sl[r] = cr->slot;
        max_ctx = std::max<int64_t>(max_ctx, cr->length + n), max_q = std::max<int64_t>(max_q, n);
    }
    for (int r = real; r < R; ++r) {
        tok[t] = 0, pos[t] = 0, rot[t] = r, lr[w++] = (int32_t)t;
        ++t;
        qs[r + 1] = (int32_t)t, ps[r] = 0, sl[r] = pad_slot;
        max_ctx = std::max<int64_t>(max_ctx, 1), max_q = std::max<int64_t>(max_q, 1);
    }
    for (size_t g = 0; g < cm->groups.size(); ++g) {
        const int wd = widths[g];
        if (wd < 1) return fail(E_VALUE, "the table of group %d is %d wide", (int)g, wd);
        for (int r = 0; r < real; ++r) {
            const std::vector<int32_t>& pages = cm->find(ids[r])->tables[g].pages;
            if ((int)pages.size() > wd) return fail(E_VALUE, "request %lld holds %d blocks in group %d, the table is %d wide", (long long)ids[r], (int)pages.size(), (int)g, wd);
            std::copy(pages.begin(), pages.end(), tab);
            std::fill(tab + pages.size(), tab + wd, -1);
            tab += wd;
        }
        for (int r = real; r < R; ++r) {
            tab[0] = pad_pages[g];
            std::fill(tab + 1, tab + wd, -1);
            tab += wd;
        }
    }
    meta[0] = total, meta[1] = T, meta[2] = W, meta[3] = max_ctx, meta[4] = max_q;
    return OK;
}

// ------------------------------------------------------------------------------- scheduler
API void* q6k_sched_create(void* cm, int max_batch_tokens, int max_running) {
    if (max_batch_tokens < 1) {
        fail(E_VALUE, "max_batch_tokens must be at least 1");
        return nullptr;
    }
    auto* s = new Scheduler();
    s->cm = (CacheManager*)cm, s->max_batch_tokens = max_batch_tokens, s->max_running = max_running;
    if (s->check_pools()) {
        delete s;
        return nullptr;
    }
    return s;
}
API void q6k_sched_destroy(void* h) { delete (Scheduler*)h; }
API int q6k_sched_add(void* h, int64_t id, const int32_t* prompt, int n, int max_tokens, const int32_t* stops, int n_stops) {
    Scheduler* s = (Scheduler*)h;
    if (s->by_id.count(id)) return fail(E_KEY, "request %lld already exists", (long long)id);
    if (n < 1) return fail(E_VALUE, "a request needs at least one prompt token");
    if (max_tokens < 1) return fail(E_VALUE, "max_tokens must be at least 1");
    if (n + 1 > s->capacity_tokens()) return fail(E_VALUE, "prompt of %d tokens exceeds the cache capacity of %lld tokens", n, (long long)s->capacity_tokens());
    SchedRequest r;
    r.id = id, r.prompt.assign(prompt, prompt + n), r.stops.assign(stops, stops + n_stops), r.max_tokens = max_tokens;
    s->by_id.emplace(id, std::move(r));
    s->waiting.push_back(id);
    return OK;
}
// A request whose prompt is taken to be in the cache already (the caller has reserved and committed
// its pages) with its first generated token given: it decodes from its next step on.
API int q6k_sched_adopt(void* h, int64_t id, const int32_t* prompt, int n, int32_t first_token, int max_tokens, const int32_t* stops, int n_stops) {
    Scheduler* s = (Scheduler*)h;
    if (s->by_id.count(id)) return fail(E_KEY, "request %lld already exists", (long long)id);
    SchedRequest r;
    r.id = id, r.prompt.assign(prompt, prompt + n), r.stops.assign(stops, stops + n_stops), r.max_tokens = max_tokens;
    r.output.push_back(first_token);
    r.num_computed = n;
    s->by_id.emplace(id, std::move(r));
    s->running.push_back(id);
    return OK;
}
API int q6k_sched_abort(void* h, int64_t id, int* was_live) {
    Scheduler* s = (Scheduler*)h;
    auto it = s->by_id.find(id);
    *was_live = 0;
    if (it == s->by_id.end() || it->second.finish != FINISH_NONE) return OK;
    *was_live = 1;
    if (int rc = s->finish(it->second, FINISH_CANCELLED)) return rc;
    s->by_id.erase(it);
    return OK;
}
API int q6k_sched_counts(void* h, int* waiting, int* running) {
    Scheduler* s = (Scheduler*)h;
    *waiting = (int)s->waiting.size(), *running = (int)s->running.size();
    return OK;
}
API int q6k_sched_queue(void* h, int which, int64_t* out, int cap, int* n) {
    Scheduler* s = (Scheduler*)h;
    std::vector<int64_t> v;
    if (which == 0) v.assign(s->waiting.begin(), s->waiting.end());
    else v = s->running;
    return copy_out(v, out, cap, n, "queue");
}
API int q6k_sched_request(void* h, int64_t id, int64_t* num_computed, int* n_output, int* preemptions, int* finish) {
    Scheduler* s = (Scheduler*)h;
    auto it = s->by_id.find(id);
    if (it == s->by_id.end()) return fail(E_KEY, "request %lld is unknown", (long long)id);
    *num_computed = it->second.num_computed, *n_output = (int)it->second.output.size();
    *preemptions = it->second.preemptions, *finish = it->second.finish;
    return OK;
}
// Builds one step.  entries: per entry (id, start, count, samples).  A request that ends here
// (cache exhausted) or is preempted is reported; admitted requests come with their state slots so
// that the caller can clear per-request state before the step runs.
API int q6k_sched_schedule(void* h, int cap, int64_t* ids, int64_t* starts, int* counts, int* samples, int* n_entries,
                           int64_t* preempted, int* n_preempted, int64_t* finished, int* n_finished, int64_t* admitted,
                           int* admitted_slots, int* n_admitted) {
    Scheduler* s = (Scheduler*)h;
    std::vector<Entry> entries;
    std::vector<int64_t> pre, fin, adm;
    std::vector<int> adm_slots;
    if (int rc = s->schedule(entries, pre, fin, adm, adm_slots)) return rc;
    if ((int)entries.size() > cap) return fail(E_VALUE, "schedule: %d entries exceed the caller's room for %d", (int)entries.size(), cap);
    for (size_t i = 0; i < entries.size(); ++i) ids[i] = entries[i].id, starts[i] = entries[i].start, counts[i] = entries[i].count, samples[i] = entries[i].samples;
    *n_entries = (int)entries.size();
    if (int rc = copy_out(pre, preempted, cap, n_preempted, "preempted")) return rc;
    if (int rc = copy_out(fin, finished, cap, n_finished, "finished")) return rc;
    if (int rc = copy_out(adm, admitted, cap, n_admitted, "admitted")) return rc;
    std::copy(adm_slots.begin(), adm_slots.end(), admitted_slots);
    for (int64_t id : fin) s->by_id.erase(id);
    s->last = entries;
    return OK;
}
// Copies tokens[start, start + count) of a request (prompt then output) into out.
API int q6k_sched_tokens(void* h, int64_t id, int64_t start, int count, int32_t* out) {
    Scheduler* s = (Scheduler*)h;
    auto it = s->by_id.find(id);
    if (it == s->by_id.end()) return fail(E_KEY, "request %lld is unknown", (long long)id);
    if (start < 0 || start + count > it->second.num_tokens()) return fail(E_VALUE, "request %lld has no tokens %lld..%lld", (long long)id, (long long)start, (long long)(start + count));
    for (int i = 0; i < count; ++i) out[i] = it->second.token(start + i);
    return OK;
}
// A token that was entered as a placeholder (the step that samples it was still running) gets its value.
API int q6k_sched_set_output_token(void* h, int64_t id, int index, int32_t tok) {
    Scheduler* s = (Scheduler*)h;
    auto it = s->by_id.find(id);
    if (it == s->by_id.end()) return fail(E_KEY, "request %lld is unknown", (long long)id);
    if (index < 0 || index >= (int)it->second.output.size()) return fail(E_VALUE, "request %lld has no output token %d", (long long)id, index);
    it->second.output[index] = tok;
    return OK;
}
// The request turns out to have ended with its n_keep-th output token (a stop token that was still
// a placeholder when later steps were planned): what came after is dropped, it ends with "stop".
API int q6k_sched_stop(void* h, int64_t id, int n_keep) {
    Scheduler* s = (Scheduler*)h;
    auto it = s->by_id.find(id);
    if (it == s->by_id.end()) return fail(E_KEY, "request %lld is unknown", (long long)id);
    SchedRequest& r = it->second;
    if (n_keep < 1 || n_keep > (int)r.output.size()) return fail(E_VALUE, "request %lld has %d output tokens, cannot keep %d", (long long)id, (int)r.output.size(), n_keep);
    r.output.resize(n_keep);
    if (int rc = s->finish(r, FINISH_STOP)) return rc;
    s->by_id.erase(it);
    return OK;
}
API int q6k_sched_update(void* h, const int32_t* sampled, int n_sampled, int cap, int64_t* done, int* reasons, int* n_done) {
    Scheduler* s = (Scheduler*)h;
    std::vector<int64_t> d;
    std::vector<int> why;
    if (int rc = s->update(sampled, n_sampled, d, why)) return rc;
    if (int rc = copy_out(d, done, cap, n_done, "finished")) return rc;
    std::copy(why.begin(), why.end(), reasons);
    for (int64_t id : d) s->by_id.erase(id);
    return OK;
}

// ------------------------------------------------------------------------------------ sampling
// One token per row from its candidate pool (ids and logits in any order), the way the reference's
// host does it (crates/cli/src/flint.rs:359-431): presence and repetition penalties on candidates
// the request has generated before; order by (logit descending, id ascending); greedy rows
// (temperature <= 0 or top_k == 1) take the first; the others compute p_i = exp((l_i - l_0) /
// temperature) in double precision from a 32-bit quotient, drop p_i < min_p, keep the shortest
// prefix whose normalised mass reaches top_p, and invert the CDF with u[row] * total.
// sizes[row] candidates of row `row` start at ids/vals + row * stride; sizes[row] <= 0 skips the
// row; generated[gen_start[row] .. gen_start[row + 1]) are the row's earlier output tokens.
API int q6k_sample_rows(int rows, int stride, const int32_t* ids, const float* vals, const int32_t* sizes, const float* temperature,
                        const int32_t* top_k, const float* top_p, const float* min_p, const float* presence, const float* repetition,
                        const int32_t* generated, const int64_t* gen_start, const double* u, int32_t* out) {
    std::vector<float> v;
    std::vector<int> order;
    std::vector<double> probs;
    for (int row = 0; row < rows; ++row) {
        const int n = sizes[row];
        if (n <= 0) continue;
        if (n > stride) return fail(E_VALUE, "row %d: %d candidates in a pool of %d", row, n, stride);
        const int32_t* id = ids + (size_t)row * stride;
        v.assign(vals + (size_t)row * stride, vals + (size_t)row * stride + n);
        if (presence[row] != 0.0f || repetition[row] != 1.0f) {
            const int32_t* g0 = generated + gen_start[row];
            const int32_t* g1 = generated + gen_start[row + 1];
            for (int i = 0; i < n; ++i)
                if (std::find(g0, g1, id[i]) != g1) {
                    float x = v[i] - presence[row];
                    v[i] = x > 0.0f ? x / repetition[row] : x * repetition[row];
                }
        }
        order.resize(n);
        for (int i = 0; i < n; ++i) order[i] = i;
        std::sort(order.begin(), order.end(), [&](int a, int b) { return v[a] != v[b] ? v[a] > v[b] : id[a] < id[b]; });
        if (temperature[row] <= 0.0f || top_k[row] == 1) {
            out[row] = id[order[0]];
            continue;
        }
        const int keep = top_k[row] == 0 ? n : std::min(top_k[row], n);
        const float top = v[order[0]];
        probs.resize(keep);
        for (int i = 0; i < keep; ++i) probs[i] = std::exp((double)((v[order[i]] - top) / temperature[row]));
        if (min_p[row] > 0.0f)
            for (double& q : probs)
                if (q < (double)min_p[row]) q = 0.0;
        double total = 0.0;
        for (double q : probs) total += q;
        int cut = keep;
        if (top_p[row] < 1.0f) {
            double acc = 0.0;
            for (int i = 0; i < keep; ++i) {
                acc += probs[i] / total;
                if (acc >= (double)top_p[row]) {
                    cut = i + 1;
                    break;
                }
            }
        }
        total = 0.0;
        for (int i = 0; i < cut; ++i) total += probs[i];
        double r = u[row] * total;
        int pick = cut - 1;
        for (int i = 0; i < cut; ++i) {
            r -= probs[i];
            if (r <= 0.0) {
                pick = i;
                break;
            }
        }
        out[row] = id[order[pick]];
    }
    return OK;
}

// --------------------------------------------------------------------------------- safetensors
// The index of one safetensors file: 8-byte little-endian header length, a JSON header
// {name: {"dtype": str, "shape": [ints], "data_offsets": [begin, end]}, "__metadata__": {...}}, then
// the raw data (the reference's reader: crates/engine/src/checkpoint.rs:174-246).  Byte ranges are
// checked against the shapes and the file; data is read with pread straight into the caller's memory.
// quench6k_b200/weights/safetensors_io.py holds a Python twin with the same messages.
namespace {

struct StEntry {
    std::string name, dtype;
    std::vector<int64_t> shape;
    int64_t begin = 0, end = 0;          // absolute byte offsets in the file
};

struct StFile {
    int fd = -1;
    int64_t size = 0;
    std::vector<StEntry> entries;
    ~StFile() {
        if (fd >= 0) close(fd);
    }
};

int dtype_width(const std::string& d) {
    if (d == "BF16" || d == "F16" || d == "I16") return 2;
    if (d == "F32" || d == "I32") return 4;
    if (d == "F64" || d == "I64") return 8;
    if (d == "I8" || d == "U8" || d == "BOOL") return 1;
    return 0;
}

// A JSON reader for what a safetensors header holds; `err` gets a reason when something else comes.
struct JsonIn {
    const char* p;
    const char* end;
    std::string err;
    void ws() {
        while (p < end && (*p == ' ' || *p == '\t' || *p == '\n' || *p == '\r')) ++p;
    }
    bool fail_at(const char* what) {
        if (err.empty()) err = std::string(what) + " at byte " + std::to_string((long long)(p - (end - len)));
        return false;
    }
    int64_t len = 0;
    bool eat(char c) {
        ws();
        if (p < end && *p == c) {
            ++p;
            return true;
        }
        return false;
    }
    bool string(std::string& out) {
        ws();
        if (p >= end || *p != '"') return fail_at("expected a string");
        ++p;
        out.clear();
        while (p < end && *p != '"') {
            unsigned char c = (unsigned char)*p++;
            if (c < 0x20) return fail_at("control character in a string");
            if (c != '\\') {
                out.push_back((char)c);
                continue;
            }
            if (p >= end) return fail_at("unfinished escape");
            const char e = *p++;
            switch (e) {
                case '"': out.push_back('"'); break;
                case '\\': out.push_back('\\'); break;
                case '/': out.push_back('/'); break;
                case 'b': out.push_back('\b'); break;
                case 'f': out.push_back('\f'); break;
                case 'n': out.push_back('\n'); break;
                case 'r': out.push_back('\r'); break;
                case 't': out.push_back('\t'); break;
                case 'u': {
                    if (end - p < 4) return fail_at("unfinished \\u escape");
                    unsigned v = 0;
                    for (int i = 0; i < 4; ++i) {
                        const char h = *p++;
                        v <<= 4;
                        if (h >= '0' && h <= '9') v |= (unsigned)(h - '0');
                        else if (h >= 'a' && h <= 'f') v |= (unsigned)(h - 'a' + 10);
                        else if (h >= 'A' && h <= 'F') v |= (unsigned)(h - 'A' + 10);
                        else return fail_at("bad \\u escape");
                    }
                    // UTF-8 of the code unit (surrogate pairs are kept as two units: names compare bytewise anyway)
                    if (v < 0x80) out.push_back((char)v);
                    else if (v < 0x800) out.push_back((char)(0xC0 | (v >> 6))), out.push_back((char)(0x80 | (v & 0x3F)));
                    else out.push_back((char)(0xE0 | (v >> 12))), out.push_back((char)(0x80 | ((v >> 6) & 0x3F))), out.push_back((char)(0x80 | (v & 0x3F)));
                    break;
                }
                default: return fail_at("unknown escape");
            }
        }
        if (p >= end) return fail_at("unfinished string");
        ++p;
        return true;
    }
    bool integer(int64_t& out) {
        ws();
        const char* s = p;
        bool neg = false;
        if (p < end && *p == '-') neg = true, ++p;
        if (p >= end || *p < '0' || *p > '9') {
            p = s;
            return fail_at("expected an integer");
        }
        int64_t v = 0;
        while (p < end && *p >= '0' && *p <= '9') {
            if (v > (INT64_MAX - 9) / 10) return fail_at("integer too large");
            v = v * 10 + (*p++ - '0');
        }
        if (p < end && (*p == '.' || *p == 'e' || *p == 'E')) return fail_at("expected an integer");
        out = neg ? -v : v;
        return true;
    }
    bool int_array(std::vector<int64_t>& out) {
        out.clear();
        if (!eat('[')) return fail_at("expected an array");
        if (eat(']')) return true;
        do {
            int64_t v;
            if (!integer(v)) return false;
            out.push_back(v);
        } while (eat(','));
        return eat(']') || fail_at("expected , or ]");
    }
    bool skip_value(int depth = 0) {                 // any JSON value (the metadata, keys this reader does not know)
        if (depth > 64) return fail_at("nested too deeply");
        ws();
        if (p >= end) return fail_at("unexpected end");
        if (*p == '"') {
            std::string s;
            return string(s);
        }
        if (*p == '{' || *p == '[') {
            const char open = *p++, shut = open == '{' ? '}' : ']';
            if (eat(shut)) return true;
            do {
                if (open == '{') {
                    std::string k;
                    if (!string(k)) return false;
                    if (!eat(':')) return fail_at("expected :");
                }
                if (!skip_value(depth + 1)) return false;
            } while (eat(','));
            return eat(shut) || fail_at("expected , or a closing bracket");
        }
        const char* s = p;
        while (p < end && (*p == '-' || *p == '+' || *p == '.' || (*p >= '0' && *p <= '9') || (*p >= 'a' && *p <= 'z') || (*p >= 'A' && *p <= 'Z'))) ++p;
        return p > s || fail_at("unexpected character");
    }
};

}  // namespace

// Opens a file and indexes its tensors; *handle is set on success.
API int q6k_st_open(const char* path, void** handle) {
    *handle = nullptr;
    auto f = std::make_unique<StFile>();
    f->fd = open(path, O_RDONLY | O_CLOEXEC);
    if (f->fd < 0) return fail(E_VALUE, "%s: cannot be opened", path);
    struct stat sb;
    if (fstat(f->fd, &sb) != 0) return fail(E_VALUE, "%s: cannot be examined", path);
    f->size = (int64_t)sb.st_size;
    unsigned char head[8];
    if (f->size < 8 || pread(f->fd, head, 8, 0) != 8) return fail(E_VALUE, "%s: shorter than a safetensors header", path);
    uint64_t n = 0;
    for (int i = 7; i >= 0; --i) n = (n << 8) | head[i];
    if (n > (uint64_t)(f->size - 8)) return fail(E_VALUE, "%s: header length %llu exceeds the file (%lld bytes)", path, (unsigned long long)n, (long long)f->size);
    std::string text((size_t)n, '\0');
    for (uint64_t got = 0; got < n;) {
        const ssize_t r = pread(f->fd, &text[(size_t)got], (size_t)(n - got), (off_t)(8 + got));
        if (r <= 0) return fail(E_VALUE, "%s: the header cannot be read", path);
        got += (uint64_t)r;
    }
    const int64_t base = 8 + (int64_t)n;
    JsonIn in{text.data(), text.data() + text.size(), std::string()};
    in.len = (int64_t)text.size();
    auto bad_json = [&]() { return fail(E_VALUE, "%s: header is not JSON (%s)", path, in.err.empty() ? "unexpected content" : in.err.c_str()); };
    if (!in.eat('{')) {
        in.fail_at("expected {");
        return bad_json();
    }
    if (!in.eat('}')) {
        do {
            std::string name;
            if (!in.string(name) || !in.eat(':')) {
                in.fail_at("expected a name and :");
                return bad_json();
            }
            if (name == "__metadata__") {
                if (!in.skip_value()) return bad_json();
                continue;
            }
            StEntry e;
            e.name = name;
            std::vector<int64_t> offs;
            bool has_dtype = false, has_shape = false;
            if (!in.eat('{')) {
                in.fail_at("expected {");
                return bad_json();
            }
            if (!in.eat('}')) {
                do {
                    std::string key;
                    if (!in.string(key) || !in.eat(':')) {
                        in.fail_at("expected a key and :");
                        return bad_json();
                    }
                    bool ok;
                    if (key == "dtype") ok = in.string(e.dtype), has_dtype = true;
                    else if (key == "shape") ok = in.int_array(e.shape), has_shape = true;
                    else if (key == "data_offsets") ok = in.int_array(offs);
                    else ok = in.skip_value();
                    if (!ok) return bad_json();
                } while (in.eat(','));
                if (!in.eat('}')) {
                    in.fail_at("expected , or }");
                    return bad_json();
                }
            }
            if (!has_dtype || !has_shape || offs.size() != 2)
                return fail(E_VALUE, "%s: tensor %s lacks dtype, shape or data_offsets", path, name.c_str());
            const int width = dtype_width(e.dtype);
            if (width == 0) return fail(E_VALUE, "%s: tensor %s has unsupported dtype %s", path, name.c_str(), e.dtype.c_str());
            int64_t count = 1;
            bool fits = true;
            for (int64_t d : e.shape) {
                if (d < 0 || (d > 0 && count > INT64_MAX / 16 / d)) fits = false;
                else count *= d;
            }
            const int64_t b = offs[0], en = offs[1];
            if (!fits || en - b != count * width || b < 0 || base + en > f->size) {
                std::string shp = "(";
                for (size_t i = 0; i < e.shape.size(); ++i) shp += (i ? ", " : "") + std::to_string((long long)e.shape[i]);
                shp += e.shape.size() == 1 ? ",)" : ")";
                return fail(E_VALUE, "%s: tensor %s has byte range %lld..%lld for shape %s %s in a file of %lld bytes", path, name.c_str(), (long long)b,
                            (long long)en, shp.c_str(), e.dtype.c_str(), (long long)f->size);
            }
            for (const StEntry& o : f->entries)
                if (o.name == name) return fail(E_VALUE, "%s: tensor %s is listed twice", path, name.c_str());
            e.begin = base + b, e.end = base + en;
            f->entries.push_back(std::move(e));
        } while (in.eat(','));
        if (!in.eat('}')) {
            in.fail_at("expected , or }");
            return bad_json();
        }
    }
    in.ws();
    if (in.p != in.end) {
        in.fail_at("content after the header's object");
        return bad_json();
    }
    *handle = f.release();
    return OK;
}
API void q6k_st_close(void* h) { delete (StFile*)h; }
API int q6k_st_count(void* h) { return (int)((StFile*)h)->entries.size(); }
// Entry i: its name (name_cap bytes with the final 0), dtype (at most 7 characters and the 0), up to 8 dimensions,
// and its absolute byte range.
API int q6k_st_entry(void* h, int i, char* name, int name_cap, char* dtype, int64_t* shape, int* ndim, int64_t* begin, int64_t* end) {
    StFile* f = (StFile*)h;
    if (i < 0 || i >= (int)f->entries.size()) return fail(E_VALUE, "tensor index %d outside 0..%d", i, (int)f->entries.size() - 1);
    const StEntry& e = f->entries[i];
    if ((int)e.name.size() + 1 > name_cap) return fail(E_VALUE, "tensor name of %d bytes exceeds the buffer", (int)e.name.size());
    if (e.shape.size() > 8) return fail(E_VALUE, "tensor %s has %d dimensions (at most 8)", e.name.c_str(), (int)e.shape.size());
    std::memcpy(name, e.name.c_str(), e.name.size() + 1);
    std::snprintf(dtype, 8, "%s", e.dtype.c_str());
    for (size_t d = 0; d < e.shape.size(); ++d) shape[d] = e.shape[d];
    *ndim = (int)e.shape.size(), *begin = e.begin, *end = e.end;
    return OK;
}
// nbytes of entry i from byte `offset` of its data into dst (a piece of a tensor: the loader streams large tensors through
// two pinned staging buffers).
API int q6k_st_read_range(void* h, int i, int64_t offset, void* dst, int64_t nbytes) {
    StFile* f = (StFile*)h;
    if (i < 0 || i >= (int)f->entries.size()) return fail(E_VALUE, "tensor index %d outside 0..%d", i, (int)f->entries.size() - 1);
    const StEntry& e = f->entries[i];
    if (offset < 0 || nbytes < 0 || offset + nbytes > e.end - e.begin)
        return fail(E_VALUE, "tensor %s holds %lld bytes, bytes %lld..%lld were asked for", e.name.c_str(), (long long)(e.end - e.begin), (long long)offset,
                    (long long)(offset + nbytes));
    for (int64_t got = 0; got < nbytes;) {
        const ssize_t r = pread(f->fd, (char*)dst + got, (size_t)std::min<int64_t>(nbytes - got, (int64_t)1 << 30), (off_t)(e.begin + offset + got));
        if (r <= 0) return fail(E_VALUE, "tensor %s: the file ends early", e.name.c_str());
        got += r;
    }
    return OK;
}
// The bytes of entry i into dst (nbytes must be the entry's size).
API int q6k_st_read(void* h, int i, void* dst, int64_t nbytes) {
    StFile* f = (StFile*)h;
    if (i < 0 || i >= (int)f->entries.size()) return fail(E_VALUE, "tensor index %d outside 0..%d", i, (int)f->entries.size() - 1);
    const StEntry& e = f->entries[i];
    if (nbytes != e.end - e.begin) return fail(E_VALUE, "tensor %s holds %lld bytes, %lld were asked for", e.name.c_str(), (long long)(e.end - e.begin), (long long)nbytes);
    for (int64_t got = 0; got < nbytes;) {
        const ssize_t r = pread(f->fd, (char*)dst + got, (size_t)std::min<int64_t>(nbytes - got, (int64_t)1 << 30), (off_t)(e.begin + got));
        if (r <= 0) return fail(E_VALUE, "tensor %s: the file ends early", e.name.c_str());
        got += r;
    }
    return OK;
}


// ------------------------------------------------------------------------------- random weights
namespace q6k_fill {
double sqrt_exact(double a) { return std::sqrt(a); }       // IEEE 754: correctly rounded
}

namespace {
inline uint16_t bf16_bits(float v) {                        // round to nearest, ties to even (NaN stays NaN)
    uint32_t u;
    std::memcpy(&u, &v, sizeof u);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    return (uint16_t)((u + 0x7fffu + ((u >> 16) & 1u)) >> 16);
}
}  // namespace

// out[i] = dtype(normal(key, start + i) * std + mean), i < n, on the host with `threads` threads; dtype 0: float32,
// 1: bfloat16.  The device twin is q6k_fill_normal (csrc/fill.cu); both include fill_normal.h.
API int q6k_fill_normal_host(void* out, int dtype, int64_t n, int64_t start, uint64_t key, float std, float mean, int threads) {
    if (n < 0 || start < 0 || (dtype != 0 && dtype != 1)) return fail(E_VALUE, "fill_normal: bad range or dtype (start %lld, n %lld, dtype %d)", (long long)start, (long long)n, dtype);
    auto work = [=](int64_t lo, int64_t hi) {
        for (int64_t i = lo; i < hi; ++i) {
            const float v = q6k_fill::element(key, (uint64_t)(start + i), std, mean);
            if (dtype == 0) ((float*)out)[i] = v;
            else ((uint16_t*)out)[i] = bf16_bits(v);
        }
    };
    const int t = (int)std::max<int64_t>(1, std::min<int64_t>(threads, n / 65536));
    if (t == 1) {
        work(0, n);
        return OK;
    }
    std::vector<std::thread> pool;
    const int64_t per = (n + t - 1) / t;
    for (int k = 0; k < t; ++k) pool.emplace_back(work, std::min<int64_t>(n, k * per), std::min<int64_t>(n, (k + 1) * per));
    for (auto& th : pool) th.join();
    return OK;
}
