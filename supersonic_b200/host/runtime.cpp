// The native core of the host side: who holds which slot and which page of the cache, how a
// step's tokens are laid out for the device, and the decisions of the generation loop that are
// pure arithmetic (which requests fit the next batch, how a long step is cut, when a sequence
// ends).  No CUDA and no Python in here: the Python classes above it (cache/, engine/) keep the
// tensors and call in through a C interface, and the tests that need no GPU run against this code.
//
// The reference keeps the same things in its Rust runner: per-sequence buffers that grow in
// 256-token chunks with a `kv_filled` count (crates/qwen35/src/state.rs:17-80, 225-311), one
// sequence stepped at a time (crates/runner/src/decode_engine.rs:10017-10061), a prompt carried
// through the cache chunk by chunk (crates/runner/src/prefill_engine.rs:1081-1094) and the stop
// rules of its generation loop (crates/runner/src/llama31_engine.rs:1075-1551).  Here the cache is
// paged (64 tokens a page), slots are pooled, and a step is a ragged batch.
//
// Every misuse (double free, an unknown id, running out) is an error code with a message, never
// corrupted state: SSB_HOST_FULL (no free slot, or too few free pages), SSB_HOST_MISUSE (a call
// that breaks the bookkeeping's rules), SSB_HOST_BAD_ARG (a malformed step).
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <map>
#include <string>
#include <vector>

#define SSB_HOST_API extern "C" __attribute__((visibility("default")))

namespace {

constexpr int PAGE_SHIFT = 6;
constexpr int PAGE_TOKENS = 1 << PAGE_SHIFT;
enum { SSB_HOST_OK = 0, SSB_HOST_FULL = -1, SSB_HOST_MISUSE = -2, SSB_HOST_BAD_ARG = -3 };

inline int pages_for(long long n_tokens) { return (int)((n_tokens + PAGE_TOKENS - 1) >> PAGE_SHIFT); }

template <typename... A>
std::string format(const char* fmt, A... a) {
    char buf[512];
    std::snprintf(buf, sizeof buf, fmt, a...);
    return std::string(buf);
}

// Ids 0..n-1, handed out lowest-first and taken back; freed ids are used again.
class FreeList {
public:
    FreeList(int n, std::string what) : n_(n), what_(std::move(what)), held_(n, 0) {
        free_.reserve(n);
        for (int i = 0; i < n; ++i) free_.push_back(i);
        std::make_heap(free_.begin(), free_.end(), std::greater<int>());
    }
    int capacity() const { return n_; }
    int n_free() const { return (int)free_.size(); }
    int n_held() const { return n_ - (int)free_.size(); }
    bool is_held(int i) const { return i >= 0 && i < n_ && held_[i]; }
    int take(std::string& err) {
        if (free_.empty()) { err = format("no free %s (all %d are held)", what_.c_str(), n_); return SSB_HOST_FULL; }
        std::pop_heap(free_.begin(), free_.end(), std::greater<int>());
        const int i = free_.back();
        free_.pop_back();
        held_[i] = 1;
        return i;
    }
    int give_back(int i, std::string& err) {
        if (i < 0 || i >= n_) { err = format("%s %d does not exist (there are %d)", what_.c_str(), i, n_); return SSB_HOST_MISUSE; }
        if (!held_[i]) { err = format("%s %d is given back but is not held", what_.c_str(), i); return SSB_HOST_MISUSE; }
        held_[i] = 0;
        free_.push_back(i);
        std::push_heap(free_.begin(), free_.end(), std::greater<int>());
        return SSB_HOST_OK;
    }
    // Invariant: every id is either free exactly once or held, never both.
    int check(std::string& err) const {
        std::vector<char> seen(n_, 0);
        for (int i : free_) {
            if (i < 0 || i >= n_ || seen[i]) { err = format("a %s is in the free list twice", what_.c_str()); return SSB_HOST_MISUSE; }
            seen[i] = 1;
        }
        for (int i = 0; i < n_; ++i)
            if ((bool)held_[i] == (bool)seen[i]) {
                err = format("%s %d is %s", what_.c_str(), i, held_[i] ? "both held and free" : "lost");
                return SSB_HOST_MISUSE;
            }
        return SSB_HOST_OK;
    }
    const std::string& what() const { return what_; }

private:
    int n_;
    std::string what_;
    std::vector<int> free_;      // a min-heap: the lowest free id is handed out first
    std::vector<char> held_;
};

// The pages of the cache entries that share one need (kv heads, head size, window): a pool of page
// ids, and per slot which page of its sequence lives in which of them.  The page table rows are
// written into memory the caller owns (pinned host memory that is copied to the device).
struct Group {
    int window;                                   // 0: every earlier key stays
    FreeList pool;
    std::vector<std::map<int, int>> held;         // per slot: page index within the sequence -> page id
    int32_t* table = nullptr;                     // [max_slots, pages_per_seq]
    int dirty_lo, dirty_hi;
    Group(int window_, int n_pages, int max_slots)
        : window(window_), pool(n_pages, "page"), held(max_slots), dirty_lo(max_slots), dirty_hi(-1) {}

    // First page a query at a position >= length can still read.
    int first_needed_page(long long length) const {
        if (window <= 0) return 0;
        const long long lo = length - window + 1;
        return lo > 0 ? (int)(lo >> PAGE_SHIFT) : 0;
    }
    // Pages that new_length tokens need and the slot does not hold yet.  A sequence that already has
    // tokens holds every page up to its last one (older ones may have been given back by a window):
    // only the last held page and those after it need a look.
    void missing_pages(int slot, long long length, long long new_length, std::vector<int>& out) const {
        out.clear();
        int first = first_needed_page(length);
        if (length > 0) first = std::max(first, pages_for(length) - 1);
        const auto& h = held[slot];
        for (int p = first; p < pages_for(new_length); ++p)
            if (!h.count(p)) out.push_back(p);
    }
};

struct CacheBook {
    int n_pages, pages_per_seq, max_slots;
    long long max_seq_tokens;
    FreeList slots;
    std::vector<long long> length;
    std::vector<Group> groups;
    std::string error;
    std::vector<int> scratch;

    CacheBook(int n_groups, const int* windows, int n_pages_, int pages_per_seq_, int max_slots_, long long max_seq)
        : n_pages(n_pages_), pages_per_seq(pages_per_seq_), max_slots(max_slots_), max_seq_tokens(max_seq),
          slots(max_slots_, "slot"), length(max_slots_, 0) {
        groups.reserve(n_groups);
        for (int g = 0; g < n_groups; ++g) groups.emplace_back(windows[g], n_pages_, max_slots_);
    }

    int need_held(int slot) {
        if (!slots.is_held(slot)) { error = format("slot %d is not held", slot); return SSB_HOST_MISUSE; }
        return SSB_HOST_OK;
    }

    // Room for n_new more tokens of the slot in every group, or in none.
    int reserve(int slot, long long n_new) {
        if (int rc = need_held(slot)) return rc;
        const long long len = length[slot], new_len = len + n_new;
        if (n_new < 0) { error = format("slot %d: %lld tokens asked for", slot, n_new); return SSB_HOST_BAD_ARG; }
        if (new_len > max_seq_tokens) {
            error = format("slot %d: %lld tokens exceed the %lld one sequence may hold", slot, new_len, max_seq_tokens);
            return SSB_HOST_FULL;
        }
        for (auto& g : groups) {
            g.missing_pages(slot, len, new_len, scratch);
            if ((int)scratch.size() > g.pool.n_free()) {
                error = format("slot %d needs %d more pages of %d tokens, %d of %d are free", slot, (int)scratch.size(),
                               PAGE_TOKENS, g.pool.n_free(), g.pool.capacity());
                return SSB_HOST_FULL;
            }
            if (!scratch.empty() && pages_for(new_len) > pages_per_seq) {
                error = format("%lld tokens exceed the %d a sequence may hold", new_len, pages_per_seq * PAGE_TOKENS);
                return SSB_HOST_FULL;
            }
        }
        for (auto& g : groups) {
            g.missing_pages(slot, len, new_len, scratch);
            if (scratch.empty()) continue;
            if (!g.table) { error = "a group's page table is not bound"; return SSB_HOST_MISUSE; }
            for (int p : scratch) {
                const int id = g.pool.take(error);
                if (id < 0) return id;            // cannot happen: the room was counted above
                g.held[slot][p] = id;
                g.table[(size_t)slot * pages_per_seq + p] = id;
            }
            g.dirty_lo = std::min(g.dirty_lo, slot);
            g.dirty_hi = std::max(g.dirty_hi, slot);
        }
        return SSB_HOST_OK;
    }

    // n_new tokens were appended; groups with a window give back what no later query reads.
    int advance(int slot, long long n_new) {
        if (int rc = need_held(slot)) return rc;
        length[slot] += n_new;
        for (auto& g : groups) {
            if (g.window <= 0) continue;
            const int first = g.first_needed_page(length[slot]);
            auto& h = g.held[slot];
            while (!h.empty() && h.begin()->first < first) {
                if (int rc = g.pool.give_back(h.begin()->second, error)) return rc;
                h.erase(h.begin());
            }
        }
        return SSB_HOST_OK;
    }

    int release(int slot) {
        if (!slots.is_held(slot)) { error = format("slot %d is released but is not held", slot); return SSB_HOST_MISUSE; }
        for (auto& g : groups) {
            for (auto& kv : g.held[slot])
                if (int rc = g.pool.give_back(kv.second, error)) return rc;
            g.held[slot].clear();
        }
        length[slot] = 0;
        return slots.give_back(slot, error);
    }

    // Invariants: no slot or page lost or held twice; held pages match the tables.
    int check() {
        if (int rc = slots.check(error)) return rc;
        for (auto& g : groups) {
            if (int rc = g.pool.check(error)) return rc;
            std::vector<char> seen(n_pages, 0);
            int n_seen = 0;
            for (int s = 0; s < max_slots; ++s) {
                if (!g.held[s].empty() && !slots.is_held(s)) { error = format("free slot %d still holds pages", s); return SSB_HOST_MISUSE; }
                for (auto& kv : g.held[s]) {
                    if (kv.second < 0 || kv.second >= n_pages || seen[kv.second]) { error = format("page %d is held twice", kv.second); return SSB_HOST_MISUSE; }
                    seen[kv.second] = 1;
                    ++n_seen;
                    if (!g.table || g.table[(size_t)s * pages_per_seq + kv.first] != kv.second) {
                        error = format("page table of slot %d disagrees at %d", s, kv.first);
                        return SSB_HOST_MISUSE;
                    }
                }
            }
            if (n_seen != g.pool.n_held()) { error = format("%d pages are marked held but %d are in use", g.pool.n_held(), n_seen); return SSB_HOST_MISUSE; }
        }
        return SSB_HOST_OK;
    }
};

struct ListHandle {
    FreeList list;
    std::string error;
    ListHandle(int n, const char* what) : list(n, what) {}
};

thread_local std::string g_error;             // of calls that have no object to keep it in

}  // namespace

// ---- a pool of ids on its own (what the cache is made of; tests use it directly) -----------------
SSB_HOST_API void* ssb_free_list_new(int n, const char* what) { return n > 0 ? new ListHandle(n, what ? what : "id") : nullptr; }
SSB_HOST_API void ssb_free_list_delete(void* h) { delete (ListHandle*)h; }
SSB_HOST_API const char* ssb_free_list_error(void* h) { return ((ListHandle*)h)->error.c_str(); }
SSB_HOST_API int ssb_free_list_take(void* h) { auto* l = (ListHandle*)h; return l->list.take(l->error); }
SSB_HOST_API int ssb_free_list_give_back(void* h, int i) { auto* l = (ListHandle*)h; return l->list.give_back(i, l->error); }
SSB_HOST_API int ssb_free_list_n_free(void* h) { return ((ListHandle*)h)->list.n_free(); }
SSB_HOST_API int ssb_free_list_is_held(void* h, int i) { return ((ListHandle*)h)->list.is_held(i) ? 1 : 0; }
SSB_HOST_API int ssb_free_list_check(void* h) { auto* l = (ListHandle*)h; return l->list.check(l->error); }

// ---- the cache's bookkeeping ----------------------------------------------------------------------
// windows[g]: the window of group g in tokens, 0 for none.
SSB_HOST_API void* ssb_cache_book_new(int n_groups, const int* windows, int n_pages, int pages_per_seq, int max_slots,
                                      long long max_seq_tokens) {
    if (n_groups < 0 || n_pages <= 0 || pages_per_seq <= 0 || max_slots <= 0 || max_seq_tokens <= 0) return nullptr;
    return new CacheBook(n_groups, windows, n_pages, pages_per_seq, max_slots, max_seq_tokens);
}
SSB_HOST_API void ssb_cache_book_delete(void* b) { delete (CacheBook*)b; }
SSB_HOST_API const char* ssb_cache_book_error(void* b) { return ((CacheBook*)b)->error.c_str(); }
// table: int32 [max_slots, pages_per_seq] that outlives the book; rows of held pages are kept up to date in it.
SSB_HOST_API int ssb_cache_book_bind_table(void* b, int group, int32_t* table) {
    auto* c = (CacheBook*)b;
    if (group < 0 || group >= (int)c->groups.size() || !table) { c->error = "no such group, or no table"; return SSB_HOST_BAD_ARG; }
    c->groups[group].table = table;
    return SSB_HOST_OK;
}
SSB_HOST_API int ssb_cache_book_acquire(void* b) {
    auto* c = (CacheBook*)b;
    const int s = c->slots.take(c->error);
    if (s >= 0) c->length[s] = 0;
    return s;
}
SSB_HOST_API int ssb_cache_book_release(void* b, int slot) { return ((CacheBook*)b)->release(slot); }
SSB_HOST_API int ssb_cache_book_is_held(void* b, int slot) { return ((CacheBook*)b)->slots.is_held(slot) ? 1 : 0; }
SSB_HOST_API long long ssb_cache_book_length(void* b, int slot) {
    auto* c = (CacheBook*)b;
    if (int rc = c->need_held(slot)) return rc;
    return c->length[slot];
}
SSB_HOST_API int ssb_cache_book_reserve(void* b, int slot, long long n_new) { return ((CacheBook*)b)->reserve(slot, n_new); }
SSB_HOST_API int ssb_cache_book_advance(void* b, int slot, long long n_new) { return ((CacheBook*)b)->advance(slot, n_new); }
// The same for several slots at once (a decode step): stops at the first that fails.
SSB_HOST_API int ssb_cache_book_reserve_each(void* b, int n, const int* slots, long long n_new) {
    for (int i = 0; i < n; ++i)
        if (int rc = ((CacheBook*)b)->reserve(slots[i], n_new)) return rc;
    return SSB_HOST_OK;
}
SSB_HOST_API int ssb_cache_book_advance_each(void* b, int n, const int* slots, long long n_new) {
    for (int i = 0; i < n; ++i)
        if (int rc = ((CacheBook*)b)->advance(slots[i], n_new)) return rc;
    return SSB_HOST_OK;
}
SSB_HOST_API int ssb_cache_book_lengths(void* b, int n, const int* slots, long long* out) {
    auto* c = (CacheBook*)b;
    for (int i = 0; i < n; ++i) {
        if (int rc = c->need_held(slots[i])) return rc;
        out[i] = c->length[slots[i]];
    }
    return SSB_HOST_OK;
}
// Rows of the group's table that changed since the last call: [*lo, *hi), empty if lo >= hi.
SSB_HOST_API int ssb_cache_book_take_dirty(void* b, int group, int* lo, int* hi) {
    auto* c = (CacheBook*)b;
    if (group < 0 || group >= (int)c->groups.size()) { c->error = "no such group"; return SSB_HOST_BAD_ARG; }
    auto& g = c->groups[group];
    *lo = g.dirty_lo;
    *hi = g.dirty_hi + 1;
    g.dirty_lo = c->max_slots;
    g.dirty_hi = -1;
    return SSB_HOST_OK;
}
SSB_HOST_API int ssb_cache_book_free_slots(void* b) { return ((CacheBook*)b)->slots.n_free(); }
SSB_HOST_API int ssb_cache_book_free_pages(void* b, int group) { return ((CacheBook*)b)->groups[group].pool.n_free(); }
SSB_HOST_API int ssb_cache_book_held_pages(void* b, int group) { return ((CacheBook*)b)->groups[group].pool.n_held(); }
// The pages a slot holds in a group: pairs (page index, page id) into out (room for cap pairs); returns their number.
SSB_HOST_API int ssb_cache_book_pages_of(void* b, int group, int slot, int* out, int cap) {
    auto* c = (CacheBook*)b;
    if (group < 0 || group >= (int)c->groups.size() || slot < 0 || slot >= c->max_slots) return SSB_HOST_BAD_ARG;
    int n = 0;
    for (auto& kv : c->groups[group].held[slot]) {
        if (n < cap) { out[2 * n] = kv.first; out[2 * n + 1] = kv.second; }
        ++n;
    }
    return n;
}
SSB_HOST_API int ssb_cache_book_check(void* b) { return ((CacheBook*)b)->check(); }

// ---- a step's layout ----------------------------------------------------------------------------
// Pages spanned by `longest` tokens, rounded down to a power of two: kernels size their grids from it
// (a sequence in the bucket spans fewer than twice as many pages), and a captured decode step stays
// valid while the bucket does.
SSB_HOST_API int ssb_decode_pages_bucket(long long longest) {
    int pages = std::max(1, pages_for(longest));
    int b = 1;
    while (2 * b <= pages) b *= 2;
    return b;
}

SSB_HOST_API const char* ssb_host_error() { return g_error.c_str(); }

// Lay the entries of a step out back to back.  Entry i: slot slots[i], starts[i] tokens already in the
// cache, counts[i] new tokens (tokens: all entries' ids one after another), want_counts[i] wanted places
// among them (want: all entries' places one after another).  flat (int32, room for 3 T + 3 B + 1 + W):
// token ids, positions, slot per token; slot and start per sequence; the B + 1 offsets of the sequences;
// the wanted rows.  sizes: T, B, W, longest run of new tokens, longest sequence after the step,
// 1 if every entry brings exactly one token.  vocab_size <= 0: ids are not checked.
SSB_HOST_API int ssb_pack_step(int n_entries, const int* slots, const long long* starts, const long long* counts,
                               const long long* tokens, const long long* want_counts, const long long* want,
                               long long vocab_size, int32_t* flat, long long flat_len, long long* sizes) {
    if (n_entries <= 0) { g_error = "a step needs at least one entry"; return SSB_HOST_BAD_ARG; }
    long long T = 0, W = 0, max_new = 0, max_total = 0;
    bool decode = true;
    for (int i = 0; i < n_entries; ++i) {
        if (counts[i] <= 0) { g_error = format("slot %d: an entry must bring at least one token", slots[i]); return SSB_HOST_BAD_ARG; }
        T += counts[i];
        W += want_counts[i];
        max_new = std::max(max_new, counts[i]);
        max_total = std::max(max_total, starts[i] + counts[i]);
        decode = decode && counts[i] == 1;
    }
    const int B = n_entries;
    if (flat_len < 3 * T + 3LL * B + 1 + W || max_total > 0x7fffffffLL) { g_error = "the step does not fit its buffer"; return SSB_HOST_BAD_ARG; }
    {
        std::vector<int> sorted(slots, slots + B);
        std::sort(sorted.begin(), sorted.end());
        if (std::adjacent_find(sorted.begin(), sorted.end()) != sorted.end()) { g_error = "a slot appears twice in one step"; return SSB_HOST_BAD_ARG; }
    }
    int32_t* tok = flat;
    int32_t* pos = flat + T;
    int32_t* slot_of = flat + 2 * T;
    int32_t* seq_slot = flat + 3 * T;
    int32_t* seq_start = seq_slot + B;
    int32_t* cu = seq_start + B;
    int32_t* rows = cu + B + 1;
    long long base = 0, w_at = 0, w_out = 0;
    std::string bad;
    int n_bad = 0;
    for (int i = 0; i < B; ++i) {
        const long long n = counts[i];
        for (long long j = 0; j < want_counts[i]; ++j) {
            const long long w = want[w_at + j];
            if (w < 0 || w >= n) { g_error = format("slot %d: wanted place %lld is outside its %lld tokens", slots[i], w, n); return SSB_HOST_BAD_ARG; }
            rows[w_out++] = (int32_t)(base + w);
        }
        w_at += want_counts[i];
        for (long long j = 0; j < n; ++j) {
            const long long t = tokens[base + j];
            if (vocab_size > 0 && (t < 0 || t >= vocab_size) && n_bad < 8) { bad += (n_bad ? ", " : "") + std::to_string(t); ++n_bad; }
            tok[base + j] = (int32_t)t;
            pos[base + j] = (int32_t)(starts[i] + j);
            slot_of[base + j] = slots[i];
        }
        seq_slot[i] = slots[i];
        seq_start[i] = (int32_t)starts[i];
        cu[i] = (int32_t)base;
        base += n;
    }
    cu[B] = (int32_t)base;
    if (n_bad) { g_error = format("token ids [%s] are outside the vocabulary of %lld", bad.c_str(), vocab_size); return SSB_HOST_BAD_ARG; }
    sizes[0] = T; sizes[1] = B; sizes[2] = W; sizes[3] = max_new; sizes[4] = max_total; sizes[5] = decode ? 1 : 0;
    return SSB_HOST_OK;
}

// Cut a step of counts[i] tokens per entry into sub-steps of at most `budget` tokens.  Entries keep
// their order, an entry that does not fit what is left of a chunk goes on in the next one, and no entry
// appears twice in a chunk.  out: triples (chunk, entry, first, end) as 4 values each, room for cap of
// them; returns the number of pieces (more than cap: call again with more room).
SSB_HOST_API long long ssb_plan_chunks(int n_entries, const long long* counts, long long budget, long long* out, long long cap) {
    if (budget < 1) { g_error = format("a step's token budget must be at least 1, not %lld", budget); return SSB_HOST_BAD_ARG; }
    long long pieces = 0, chunk = 0, room = budget;
    bool chunk_used = false;
    for (int i = 0; i < n_entries; ++i) {
        long long first = 0;
        while (first < counts[i]) {
            if (room == 0) { if (chunk_used) ++chunk; room = budget; chunk_used = false; }
            const long long take = std::min(room, counts[i] - first);
            if (pieces < cap) { out[4 * pieces] = chunk; out[4 * pieces + 1] = i; out[4 * pieces + 2] = first; out[4 * pieces + 3] = first + take; }
            ++pieces;
            chunk_used = true;
            first += take;
            room -= take;
        }
    }
    return pieces;
}

// ---- the generation loop's arithmetic -----------------------------------------------------------
// The next batch: requests in arrival order while their prompts plus budgets fit the free pages and
// slots (each sequence's need rounded up to whole pages).  Returns how many of the waiting requests
// (their prompt lengths in prompt_lens, in order) start now.  batch_size <= 0: no limit of its own.
SSB_HOST_API int ssb_plan_batch(int n_waiting, const long long* prompt_lens, long long max_new_tokens, long long free_tokens,
                                int free_slots, int page_tokens, int batch_size) {
    int chosen = 0;
    long long room = free_tokens;
    for (int i = 0; i < n_waiting; ++i) {
        if (chosen >= free_slots || (batch_size > 0 && chosen >= batch_size)) break;
        const long long tokens = prompt_lens[i] + std::max(max_new_tokens, 1LL);
        const long long need = (tokens + page_tokens - 1) / page_tokens * page_tokens;
        if (need > room) break;
        ++chosen;
        room -= need;
    }
    return chosen;
}

// Why a sequence ends after producing `token` as its n_generated-th: 1 a stop token, 2 its budget, 0 it goes on.
SSB_HOST_API int ssb_finished(long long token, long long n_generated, long long max_new_tokens, const long long* stop_ids, int n_stop) {
    for (int i = 0; i < n_stop; ++i)
        if (stop_ids[i] == token) return 1;
    return n_generated >= max_new_tokens ? 2 : 0;
}

// A decode batch after a step: tokens[i] is what row i sampled, generated[i] how many tokens row i had
// before it.  Writes why[i] (as ssb_finished) and returns how many rows go on.
SSB_HOST_API int ssb_finished_rows(int n, const long long* tokens, const long long* generated, long long max_new_tokens,
                                   const long long* stop_ids, int n_stop, int* why) {
    int alive = 0;
    for (int i = 0; i < n; ++i) {
        why[i] = ssb_finished(tokens[i], generated[i] + 1, max_new_tokens, stop_ids, n_stop);
        alive += why[i] == 0;
    }
    return alive;
}
