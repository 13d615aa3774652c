// The engine's host runtime: page and slot pools, per-request block tables, the step packer
// and the continuous-batching scheduler.  Plain C++17, no CUDA: it is compiled with the host
// compiler and loaded with ctypes like the kernel libraries.  Everything is single-threaded
// by contract (one engine loop owns a cache and its scheduler).
//
// Behaviour follows the reference's block pool (crates/vapi-cache/src/pool.rs:80-247),
// sequence (crates/vapi-engine/src/sequence.rs) and scheduler
// (crates/vapi-engine/src/scheduler.rs) without prefix cache and forks; the differences are
// that every paged group of layers has a pool and block tables of its own, that a windowed
// group gives pages back while the request runs, and that a request also holds a state slot.
#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <deque>
#include <string>
#include <unordered_map>
#include <vector>

#define API extern "C" __attribute__((visibility("default")))

namespace {

thread_local std::string g_error;

int fail(int code, const std::string& msg) {
    g_error = msg;
    return code;
}

// ---- pools ---------------------------------------------------------------------------------
// A free list and a held flag per id.  Freed ids go to the front of the list and are handed
// out again first, so a small pool reuses its pages quickly.  The watermark is a reserve that
// admission may not touch (can_allocate) while running requests still may (allocate).
struct Pool {
    int n = 0, watermark = 0;
    std::deque<int> free_list;
    std::vector<uint8_t> held;

    void init(int count, int wm) {
        n = count;
        watermark = std::max(0, std::min(wm, count - 1));
        free_list.clear();
        for (int i = 0; i < n; ++i) free_list.push_back(i);
        held.assign(n, 0);
    }
    int num_free() const { return (int)free_list.size(); }
    bool can_allocate(int k) const { return num_free() >= k + watermark; }
    int allocate() {
        if (free_list.empty()) return -1;
        int p = free_list.front();
        free_list.pop_front();
        held[p] = 1;
        return p;
    }
    // 0 ok, -1 outside the pool, -2 not held
    int release(int p) {
        if (p < 0 || p >= n) return -1;
        if (!held[p]) return -2;
        held[p] = 0;
        free_list.push_front(p);
        return 0;
    }
    bool check(std::string* why) const {
        std::vector<uint8_t> seen(n, 0);
        for (int p : free_list) {
            if (p < 0 || p >= n) { *why = "an id outside the pool is on the free list"; return false; }
            if (seen[p]) { *why = "an id is on the free list twice"; return false; }
            if (held[p]) { *why = "an id is free and held"; return false; }
            seen[p] = 1;
        }
        int h = 0;
        for (int i = 0; i < n; ++i) h += held[i];
        if (h + (int)free_list.size() != n) { *why = "an id is lost"; return false; }
        return true;
    }
};

// ---- the cache's books ------------------------------------------------------------------------
struct Group {
    Pool pool;
    int window = 0;                 // 0: every key is kept
    std::vector<int> set_aside;     // pages taken out of circulation for padding rows
};

struct Request {
    bool live = false;
    int slot = -1;
    int num_tokens = 0;                         // positions computed so far
    std::vector<std::vector<int>> tables;       // per group: page per logical page, -1 once released
    std::vector<int> first_live;                // per group: first logical page still held
};

struct Cache {
    int page_size = 0;
    std::vector<Group> groups;
    Pool slots;
    std::vector<Request> reqs;
    std::vector<int> free_handles;

    int pages_for(int tokens) const { return (tokens + page_size - 1) / page_size; }
    Request* get(int h) {
        if (h < 0 || h >= (int)reqs.size() || !reqs[h].live) return nullptr;
        return &reqs[h];
    }
    int open() {
        int slot = slots.allocate();
        if (slot < 0) return fail(-1, "no free state slot");
        int h;
        if (!free_handles.empty()) { h = free_handles.back(); free_handles.pop_back(); }
        else { h = (int)reqs.size(); reqs.emplace_back(); }
        Request& r = reqs[h];
        r.live = true;
        r.slot = slot;
        r.num_tokens = 0;
        r.tables.assign(groups.size(), {});
        r.first_live.assign(groups.size(), 0);
        return h;
    }
    bool can_admit(int total) const {
        if (slots.num_free() == 0) return false;
        int need = pages_for(total);
        for (const Group& g : groups)
            if (!g.pool.can_allocate(need)) return false;
        return true;
    }
    // Pages so that positions < total are covered in every group; all or nothing.
    int reserve(int h, int total, bool guarded) {
        Request* r = get(h);
        if (!r) return fail(-2, "the request is not live");
        int want = pages_for(total);
        for (size_t gi = 0; gi < groups.size(); ++gi) {
            int need = std::max(0, want - (int)r->tables[gi].size());
            const Pool& p = groups[gi].pool;
            if ((guarded && !p.can_allocate(need)) || p.num_free() < need) return 0;
        }
        for (size_t gi = 0; gi < groups.size(); ++gi) {
            int need = std::max(0, want - (int)r->tables[gi].size());
            for (int k = 0; k < need; ++k) r->tables[gi].push_back(groups[gi].pool.allocate());
        }
        return 1;
    }
    // The request has computed positions < total.  A windowed group gives back every page all
    // of whose positions are out of reach of any later query: the next query sits at a
    // position >= total and sees keys > total - window.
    int commit(int h, int total) {
        Request* r = get(h);
        if (!r) return fail(-2, "the request is not live");
        r->num_tokens = total;
        for (size_t gi = 0; gi < groups.size(); ++gi) {
            int w = groups[gi].window;
            if (w <= 0) continue;
            int dead_upto = total - w;
            std::vector<int>& tb = r->tables[gi];
            while (true) {
                int pi = r->first_live[gi];
                if (pi >= (int)tb.size() || (pi + 1) * page_size - 1 > dead_upto) break;
                groups[gi].pool.release(tb[pi]);
                tb[pi] = -1;
                r->first_live[gi] = pi + 1;
            }
        }
        return 0;
    }
    int close(int h) {
        Request* r = get(h);
        if (!r) return fail(-2, "the request is closed twice");
        for (size_t gi = 0; gi < groups.size(); ++gi) {
            for (int p : r->tables[gi])
                if (p >= 0) groups[gi].pool.release(p);
            r->tables[gi].clear();
        }
        slots.release(r->slot);
        r->live = false;
        free_handles.push_back(h);
        return 0;
    }
    bool check(std::string* why) const {
        for (size_t gi = 0; gi < groups.size(); ++gi) {
            const Group& g = groups[gi];
            if (!g.pool.check(why)) return false;
            std::vector<int> owners(g.pool.n, 0);
            for (const Request& r : reqs)
                if (r.live)
                    for (int p : r.tables[gi])
                        if (p >= 0) {
                            if (p >= g.pool.n) { *why = "a request holds a page outside the pool"; return false; }
                            owners[p]++;
                        }
            for (int p : g.set_aside) owners[p]++;
            for (int p = 0; p < g.pool.n; ++p) {
                if (owners[p] > 1) { *why = "a page is held by two requests"; return false; }
                if ((owners[p] == 1) != (g.pool.held[p] != 0)) {
                    *why = "pool and requests disagree about held pages";
                    return false;
                }
            }
        }
        if (!slots.check(why)) return false;
        std::vector<int> owners(slots.n, 0);
        int live = 0;
        for (const Request& r : reqs)
            if (r.live) {
                if (owners[r.slot]++) { *why = "a slot is held by two requests"; return false; }
                ++live;
            }
        if (slots.num_free() + live != slots.n) { *why = "a slot is lost"; return false; }
        return true;
    }
};

// ---- the packed step -----------------------------------------------------------------------
// Every index array of a step lives in one int32 buffer whose layout depends only on
// (token capacity, sequence capacity, table width, row capacity): a captured decode step of a
// given bucket always finds its inputs at the same offsets.  Arrays start on 16-byte
// boundaries.  Order: cu_q, seqlens_k, state_slots, table[g]..., tokens, positions, tok_seq,
// slots[g]..., rows, token_src, and the total as the last entry.  token_src[i] >= 0 says
// that token i is not known to the host yet: it is that row of the previous step's sampled
// output, and a kernel at the head of the step fetches it from there.
inline int round4(int x) { return (std::max(x, 1) + 3) / 4 * 4; }

void layout(int G, int n_cap, int s_cap, int width, int r_cap, int* out) {
    int off = 0, k = 0;
    auto put = [&](int count) { out[k++] = off; off += round4(count); };
    put(s_cap + 1);
    put(s_cap);
    put(s_cap);
    for (int g = 0; g < G; ++g) put(s_cap * width);
    put(n_cap);
    put(n_cap);
    put(n_cap);
    for (int g = 0; g < G; ++g) put(n_cap);
    put(r_cap);
    put(n_cap);
    out[k] = off;
}

struct PackArgs {
    int S;                      // live entries
    const int* handles;         // [S]
    const int* qlens;           // [S]
    const int* tokens;          // [sum qlens]
    const int* want_counts;     // [S]
    const int* wants;           // [sum want_counts] places within each entry's tokens
    const int* token_src;       // [sum qlens] or null: see the layout
    int n_cap, s_cap, width, r_cap;
    int padded;                 // 1: fill up to (n_cap, s_cap) with padding sequences
    const int* pad_pages;       // [G] when padded
    int scratch_slot;
};

// info: n, sequences, rows, max_q, max_k, rows_identity, total
int pack(Cache& c, const PackArgs& a, int* out, int* info) {
    const int G = (int)c.groups.size(), P = c.page_size;
    std::vector<int> lay(2 * G + 10);
    layout(G, a.n_cap, a.s_cap, a.width, a.r_cap, lay.data());
    const int o_cu = lay[0], o_k = lay[1], o_state = lay[2];
    const int* o_table = &lay[3];
    const int o_tok = lay[3 + G], o_pos = lay[4 + G], o_seq = lay[5 + G];
    const int* o_slots = &lay[6 + G];
    const int o_rows = lay[6 + 2 * G], o_src = lay[7 + 2 * G], total = lay[8 + 2 * G];
    std::memset(out, 0, sizeof(int) * (size_t)total);

    int n = 0, rows = 0, max_q = a.padded ? 1 : 0, max_k = a.padded ? 1 : 0;
    const int* tk = a.tokens;
    const int* wt = a.wants;
    const int* ts = a.token_src;
    for (int i = 0; i < a.n_cap; ++i) out[o_src + i] = -1;
    bool identity = true;
    if (a.S > a.s_cap) return fail(-3, "more sequences than the step's capacity");
    out[o_cu] = 0;
    for (int si = 0; si < a.S; ++si) {
        Request* r = c.get(a.handles[si]);
        if (!r) return fail(-2, "an entry's request is not live");
        const int q = a.qlens[si], st = r->num_tokens;
        if (q <= 0) return fail(-4, "an entry brings no tokens");
        if (n + q > a.n_cap) return fail(-3, "more tokens than the step's capacity");
        const int need = c.pages_for(st + q);
        if (need > a.width) return fail(-3, "a block table is wider than the step's capacity");
        for (int g = 0; g < G; ++g) {
            const std::vector<int>& tb = r->tables[g];
            if ((int)tb.size() < need) return fail(-5, "pages were not reserved for an entry's tokens");
            int* row = out + o_table[g] + si * a.width;
            const int cnt = std::min((int)tb.size(), a.width);
            for (int j = 0; j < cnt; ++j) row[j] = tb[j] < 0 ? 0 : tb[j];
            int* sl = out + o_slots[g] + n;
            for (int j = 0; j < q; ++j) {
                const int p = st + j, page = tb[p / P];
                if (page < 0) return fail(-5, "a token would be written to a page the window has released");
                sl[j] = page * P + p % P;
            }
        }
        for (int j = 0; j < q; ++j) {
            out[o_tok + n + j] = tk[j];
            if (ts) out[o_src + n + j] = ts[j];
            out[o_pos + n + j] = st + j;
            out[o_seq + n + j] = si;
        }
        for (int j = 0; j < a.want_counts[si]; ++j) {
            if (rows >= a.r_cap) return fail(-3, "more wanted rows than the step's capacity");
            if (wt[j] < 0 || wt[j] >= q) return fail(-4, "a wanted place is outside its entry's tokens");
            identity = identity && (n + wt[j] == rows);
            out[o_rows + rows++] = n + wt[j];
        }
        tk += q;
        if (ts) ts += q;
        wt += a.want_counts[si];
        out[o_k + si] = st + q;
        out[o_state + si] = r->slot;
        max_q = std::max(max_q, q);
        max_k = std::max(max_k, st + q);
        n += q;
        out[o_cu + si + 1] = n;
    }
    int S = a.S;
    if (a.padded) {
        // padding sequences of a fixed-shape step: one token each at position 0, written to a
        // page and a state slot that no request owns; nothing of theirs is read back
        for (int si = a.S; si < a.s_cap; ++si) {
            if (n >= a.n_cap || rows >= a.r_cap) return fail(-3, "padding exceeds the step's capacity");
            out[o_k + si] = 1;
            out[o_state + si] = a.scratch_slot;
            identity = identity && (rows == n);
            out[o_rows + rows++] = n;
            out[o_seq + n] = si;
            for (int g = 0; g < G; ++g) {
                out[o_slots[g] + n] = a.pad_pages[g] * P;
                out[o_table[g] + si * a.width] = a.pad_pages[g];
            }
            ++n;
            out[o_cu + si + 1] = n;
        }
        S = a.s_cap;
    }
    identity = identity && rows == n;
    info[0] = n; info[1] = S; info[2] = rows; info[3] = max_q; info[4] = max_k;
    info[5] = identity ? 1 : 0; info[6] = total;
    return 0;
}

// ---- sequences and the scheduler -----------------------------------------------------------
constexpr int UNKNOWN = -1;      // a token that a step in flight has yet to produce
enum Status { WAITING = 0, PREFILLING = 1, DECODING = 2, FINISHED = 3 };
enum Reason { R_NONE = -1, R_STOP = 0, R_LENGTH = 1, R_CANCELLED = 2, R_ERROR = 3 };

struct Seq {
    int id = 0;
    int status = WAITING;
    std::vector<int> tokens;
    int prompt_len = 0, num_computed = 0, prefill_target = 0;
    int handle = -1;                // the cache's request handle while it holds anything
    int preemptions = 0;
    int reason = R_NONE;
    int max_tokens = 0;
    bool ignore_eos = false;
    std::vector<int> stop_ids;
    // Running one step ahead: a token that a step in flight will produce stands in `tokens` as
    // UNKNOWN until the step's result has been read.  `pending` lists where those stand,
    // oldest first; `last_row` is the row of the newest one in its step's sampled output (the
    // next step's device-side input reads it from there); `parked` marks a request that has
    // reached a length limit and only waits for its last token.
    std::deque<int> pending;
    int last_row = -1;
    bool parked = false;

    int total_len() const { return (int)tokens.size(); }
    int num_generated() const { return (int)tokens.size() - prompt_len; }
    bool needs_prefill() const { return num_computed < prefill_target; }
};

struct Plan {
    std::vector<int> seq_ids, handles, starts, qlens, want_counts, wants, tokens;
    std::vector<int> token_src;     // per token: row of the previous step's sampled output it is, or -1
    std::vector<int> sampled, preempted, started;
    bool has_unknown = false, advanced = false;
    void clear() {
        seq_ids.clear(); handles.clear(); starts.clear(); qlens.clear(); want_counts.clear();
        wants.clear(); tokens.clear(); sampled.clear(); preempted.clear(); started.clear();
        token_src.clear();
        has_unknown = advanced = false;
    }
};

struct Sched {
    Cache* cache = nullptr;
    int max_seqs = 64, max_batched = 8192, chunk = 2048, max_context = 8192;
    std::vector<int> eos;
    std::unordered_map<int, Seq> seqs;
    std::deque<int> waiting;
    std::vector<int> running, finished;
    int next_id = 0;
    Plan plan;

    Seq* get(int sid) {
        auto it = seqs.find(sid);
        return it == seqs.end() ? nullptr : &it->second;
    }
    static void erase(std::vector<int>& v, int x) { v.erase(std::remove(v.begin(), v.end(), x), v.end()); }

    // Pages of the smallest group that requests can ever hold (pages set aside for the padding
    // rows of fixed-shape decode steps never come back).
    int min_pool_pages() const {
        int m = INT32_MAX;
        for (const Group& g : cache->groups) m = std::min(m, g.pool.n - (int)g.set_aside.size());
        return m;
    }
    int admit(const int* prompt, int n, int max_tokens, bool ignore_eos, const int* stop, int nstop) {
        if (n == 0) return fail(-1, "the prompt is empty");
        if (n >= max_context)
            return fail(-2, "the prompt has " + std::to_string(n) + " tokens; the context limit is " +
                                std::to_string(max_context));
        if (!cache->groups.empty() && cache->pages_for(n + 1) > min_pool_pages())
            return fail(-3, "the prompt has " + std::to_string(n) + " tokens; the whole cache holds fewer");
        int sid = next_id++;
        Seq& s = seqs[sid];
        s.id = sid;
        s.tokens.assign(prompt, prompt + n);
        s.prompt_len = s.prefill_target = n;
        s.max_tokens = max_tokens;
        s.ignore_eos = ignore_eos;
        s.stop_ids.assign(stop, stop + nstop);
        waiting.push_back(sid);
        return sid;
    }
    void push(Seq& s, int q) {
        const int start = s.num_computed;
        const bool completes = start + q >= s.total_len();
        plan.seq_ids.push_back(s.id);
        plan.handles.push_back(s.handle);
        plan.starts.push_back(start);
        plan.qlens.push_back(q);
        for (int t = start; t < start + q; ++t) {
            const int tok = s.tokens[t];
            plan.tokens.push_back(tok == UNKNOWN ? 0 : tok);
            plan.token_src.push_back(tok == UNKNOWN ? s.last_row : -1);
            plan.has_unknown = plan.has_unknown || tok == UNKNOWN;
        }
        plan.want_counts.push_back(completes ? 1 : 0);
        if (completes) {
            plan.wants.push_back(q - 1);
            plan.sampled.push_back(s.id);
        }
    }
    // Everything the request holds goes back; it keeps its tokens and returns to the front of
    // the queue to be computed again from position 0 (sequence.rs:167-176).
    void preempt(Seq& s) {
        if (s.handle >= 0) cache->close(s.handle);
        s.handle = -1;
        s.num_computed = 0;
        s.prefill_target = s.total_len();
        s.status = WAITING;
        s.preemptions++;
        erase(running, s.id);
        waiting.push_front(s.id);
        plan.preempted.push_back(s.id);
    }
    int prefill_chunk(Seq& s, int budget) {
        int q = std::min(std::min(s.prefill_target - s.num_computed, chunk), budget);
        if (q <= 0) return budget;
        if (cache->reserve(s.handle, s.num_computed + q, false) != 1) {
            preempt(s);
            return budget;
        }
        push(s, q);
        return budget - q;
    }
    bool can_ever_fit(const Seq& s) const {
        int need = cache->pages_for(s.prefill_target + 1);
        for (const Group& g : cache->groups)
            if (need + g.pool.watermark > g.pool.n - (int)g.set_aside.size()) return false;
        return true;
    }
    bool try_start(Seq& s) {
        if (!cache->can_admit(s.prefill_target + 1)) return false;
        int h = cache->open();
        if (h < 0) return false;
        if (cache->reserve(h, s.prefill_target + 1, true) != 1) {
            cache->close(h);
            return false;
        }
        s.handle = h;
        s.status = PREFILLING;
        return true;
    }
    void finish(int sid, int reason) {
        Seq* s = get(sid);
        if (!s || s->status == FINISHED) return;
        s->status = FINISHED;
        s->reason = reason;
        s->parked = false;
        while (!s->tokens.empty() && s->tokens.back() == UNKNOWN) s->tokens.pop_back();   // never learnt
        s->pending.clear();
        if (s->handle >= 0) cache->close(s->handle);
        s->handle = -1;
        erase(running, sid);
        waiting.erase(std::remove(waiting.begin(), waiting.end(), sid), waiting.end());
        finished.push_back(sid);
    }
    // One step: decode tokens of running requests first (one each), then the next portions
    // of prompts already started, then waiting requests in FIFO order while budget, request
    // slots and pages (watermark-checked) allow (scheduler.rs:329-431).
    int schedule() {
        plan.clear();
        int budget = max_batched;
        std::vector<int> order = running;
        for (int sid : order) {
            Seq* s = get(sid);
            if (!s || s->status == FINISHED) { erase(running, sid); continue; }
            if (s->needs_prefill() || budget == 0) continue;
            if (cache->reserve(s->handle, s->num_computed + 1, false) == 1) {
                push(*s, 1);
                --budget;
            } else {
                preempt(*s);
            }
        }
        order = running;
        for (int sid : order) {
            if (budget == 0) return (int)plan.seq_ids.size();
            Seq* s = get(sid);
            if (!s || !s->needs_prefill() || s->status == FINISHED) continue;
            budget = prefill_chunk(*s, budget);
        }
        while (budget > 0 && (int)running.size() < max_seqs && !waiting.empty()) {
            int sid = waiting.front();
            waiting.pop_front();
            Seq* s = get(sid);
            if (!s || s->status == FINISHED) continue;
            if (!can_ever_fit(*s)) {     // grown (by generation, then preemption) beyond the whole cache
                finish(sid, R_LENGTH);
                continue;
            }
            if (!try_start(*s)) {
                waiting.push_front(sid);
                break;
            }
            plan.started.push_back(sid);
            running.push_back(sid);
            budget = prefill_chunk(*s, budget);
        }
        return (int)plan.seq_ids.size();
    }
    // Whether the token at `idx` ends the request: EOS (unless ignored) or a stop id, and
    // only for a generated token (sequence.rs:179-202).
    bool stops_at(const Seq& s, int idx) const {
        if (idx < s.prompt_len) return false;
        const int tok = s.tokens[idx];
        const bool is_eos = !s.ignore_eos && std::find(eos.begin(), eos.end(), tok) != eos.end();
        return is_eos || std::find(s.stop_ids.begin(), s.stop_ids.end(), tok) != s.stop_ids.end();
    }
    bool at_length_limit(const Seq& s) const {
        return s.num_generated() >= s.max_tokens || s.total_len() >= max_context;
    }
    // The part of a commit that does not depend on what was sampled: every request of the
    // planned step has computed its tokens; a request that asked for logits gains a token whose
    // value is not known yet.  One that reaches a length limit with it is parked: it takes part
    // in no further step and is retired when the token's value arrives.
    int advance() {
        if (plan.advanced) return fail(-1, "the planned step has been advanced already");
        plan.advanced = true;
        for (size_t i = 0; i < plan.seq_ids.size(); ++i) {
            Seq* s = get(plan.seq_ids[i]);
            if (!s || s->status == FINISHED) continue;
            s->num_computed += plan.qlens[i];
            if (!s->needs_prefill() && s->status == PREFILLING) s->status = DECODING;
        }
        for (size_t i = 0; i < plan.sampled.size(); ++i) {
            Seq* s = get(plan.sampled[i]);
            if (!s || s->status == FINISHED) continue;
            s->pending.push_back((int)s->tokens.size());
            s->tokens.push_back(UNKNOWN);
            s->last_row = (int)i;
            s->prefill_target = std::max(s->prefill_target, s->num_computed);
            if (at_length_limit(*s)) {
                s->parked = true;
                erase(running, s->id);
            }
        }
        return 0;
    }
    // The values of tokens that an advanced step produced, for the requests `sids` in the
    // order of that step's wanted rows.  Retires what finished: EOS or a stop id -> STOP (what a
    // later step in flight has appended for the request in the meantime is dropped);
    // a length limit -> LENGTH.
    int resolve(const int* sids, const int* toks, int n, int* accepted) {
        for (int i = 0; i < n; ++i) {
            Seq* s = get(sids[i]);
            const bool takes = s && s->status != FINISHED && !s->pending.empty();
            if (accepted) accepted[i] = takes ? 1 : 0;      // 0: the request had ended before this token
            if (!takes) continue;
            const int idx = s->pending.front();
            s->pending.pop_front();
            s->tokens[idx] = toks[i];
            if (stops_at(*s, idx)) {
                s->tokens.resize(idx + 1);
                s->pending.clear();
                finish(s->id, R_STOP);
            } else if (s->parked && s->pending.empty()) {
                finish(s->id, R_LENGTH);
            }
        }
        return 0;
    }
    // Advance the planned step and give its sampled tokens at once.
    int commit(const int* sampled, int n) {
        if (n != (int)plan.sampled.size()) return fail(-1, "one sampled token per wanted row is needed");
        if (!plan.advanced && advance() != 0) return -1;
        std::vector<int> sids = plan.sampled;
        return resolve(sids.data(), sampled, n, nullptr);
    }
    // Whether the next step can be planned before the last one's tokens are known without any
    // risk of a preemption (whose recompute would need those tokens): every running request
    // can take one more page in every group.
    bool can_run_ahead() const {
        for (const Group& g : cache->groups)
            if (g.pool.num_free() < (int)running.size()) return false;
        return true;
    }
};

int copy_out(const std::vector<int>& v, int* out, int cap) {
    int n = std::min((int)v.size(), cap);
    if (n > 0 && out) std::memcpy(out, v.data(), sizeof(int) * (size_t)n);
    return (int)v.size();
}

}  // namespace

// =================================== the C interface ==========================================
API const char* vh_last_error() { return g_error.c_str(); }

// ---- stand-alone pools ---------------------------------------------------------------------
API void* vh_pool_new(int n, int watermark) {
    if (n <= 0) { g_error = "a pool needs at least one id"; return nullptr; }
    Pool* p = new Pool();
    p->init(n, watermark);
    return p;
}
API void vh_pool_delete(void* p) { delete (Pool*)p; }
API int vh_pool_size(void* p) { return ((Pool*)p)->n; }
API int vh_pool_watermark(void* p) { return ((Pool*)p)->watermark; }
API int vh_pool_num_free(void* p) { return ((Pool*)p)->num_free(); }
API int vh_pool_can_allocate(void* p, int k) { return ((Pool*)p)->can_allocate(k) ? 1 : 0; }
API int vh_pool_allocate(void* p) { return ((Pool*)p)->allocate(); }
API int vh_pool_release(void* p, int id) { return ((Pool*)p)->release(id); }
API int vh_pool_held(void* p, int* out, int cap) {
    Pool* q = (Pool*)p;
    int k = 0;
    for (int i = 0; i < q->n; ++i)
        if (q->held[i]) { if (k < cap) out[k] = i; ++k; }
    return k;
}
API int vh_pool_check(void* p) {
    std::string why;
    return ((Pool*)p)->check(&why) ? 0 : fail(-1, why);
}

// ---- the cache's books ------------------------------------------------------------------------
API void* vh_cache_new(int G, int page_size, const int* pages, const int* watermark, const int* window,
                       int num_slots) {
    if (page_size <= 0 || num_slots <= 0) { g_error = "page size and slot count must be positive"; return nullptr; }
    Cache* c = new Cache();
    c->page_size = page_size;
    c->groups.resize(G);
    for (int g = 0; g < G; ++g) {
        if (pages[g] <= 0) { delete c; g_error = "the cache needs at least one page per group"; return nullptr; }
        c->groups[g].pool.init(pages[g], watermark[g]);
        c->groups[g].window = window[g];
    }
    c->slots.init(num_slots, 0);
    return c;
}
API void vh_cache_delete(void* c) { delete (Cache*)c; }
API void* vh_cache_group_pool(void* c, int g) { return &((Cache*)c)->groups[g].pool; }   // borrowed
API void* vh_cache_slot_pool(void* c) { return &((Cache*)c)->slots; }                     // borrowed
API int vh_open(void* c) { return ((Cache*)c)->open(); }
API int vh_close(void* c, int h) { return ((Cache*)c)->close(h); }
API int vh_reserve(void* c, int h, int total, int guarded) { return ((Cache*)c)->reserve(h, total, guarded != 0); }
API int vh_commit(void* c, int h, int total) { return ((Cache*)c)->commit(h, total); }
API int vh_can_admit(void* c, int total) { return ((Cache*)c)->can_admit(total) ? 1 : 0; }
API int vh_is_live(void* c, int h) { return ((Cache*)c)->get(h) ? 1 : 0; }
API int vh_slot(void* c, int h) { Request* r = ((Cache*)c)->get(h); return r ? r->slot : -1; }
API int vh_num_tokens(void* c, int h) { Request* r = ((Cache*)c)->get(h); return r ? r->num_tokens : -1; }
API int vh_first_live(void* c, int h, int g) { Request* r = ((Cache*)c)->get(h); return r ? r->first_live[g] : -1; }
API int vh_table(void* c, int h, int g, int* out, int cap) {
    Request* r = ((Cache*)c)->get(h);
    if (!r) return 0;
    return copy_out(r->tables[g], out, cap);
}
API int vh_commit_many(void* c, int S, const int* handles, const int* qlens) {
    Cache* k = (Cache*)c;
    for (int i = 0; i < S; ++i) {
        Request* r = k->get(handles[i]);
        if (!r) return fail(-2, "the request is not live");
        k->commit(handles[i], r->num_tokens + qlens[i]);
    }
    return 0;
}
API int vh_set_aside(void* c, int* out) {
    Cache* k = (Cache*)c;
    for (Group& g : k->groups)
        if (g.pool.num_free() == 0) return 0;
    int i = 0;
    for (Group& g : k->groups) {
        int p = g.pool.allocate();
        g.set_aside.push_back(p);
        out[i++] = p;
    }
    return 1;
}
API int vh_cache_check(void* c) {
    std::string why;
    return ((Cache*)c)->check(&why) ? 0 : fail(-1, why);
}

// ---- the packed step -----------------------------------------------------------------------
API int vh_layout_len(int G) { return 2 * G + 9; }
API void vh_layout(int G, int n_cap, int s_cap, int width, int r_cap, int* out) {
    layout(G, n_cap, s_cap, width, r_cap, out);
}
API int vh_pack(void* c, int S, const int* handles, const int* qlens, const int* tokens, const int* want_counts,
                const int* wants, int n_cap, int s_cap, int width, int r_cap, int padded, const int* pad_pages,
                int scratch_slot, int* out, int* info) {
    PackArgs a{S, handles, qlens, tokens, want_counts, wants, nullptr, n_cap, s_cap, width, r_cap, padded,
               pad_pages, scratch_slot};
    return pack(*(Cache*)c, a, out, info);
}

// ---- the scheduler ---------------------------------------------------------------------------
API void* vs_new(void* cache, int max_seqs, int max_batched, int chunk, int max_context, const int* eos, int n_eos) {
    Sched* s = new Sched();
    s->cache = (Cache*)cache;
    s->max_seqs = max_seqs;
    s->max_batched = max_batched;
    s->chunk = chunk;
    s->max_context = max_context;
    s->eos.assign(eos, eos + n_eos);
    return s;
}
API void vs_delete(void* s) { delete (Sched*)s; }
API int vs_admit(void* s, const int* prompt, int n, int max_tokens, int ignore_eos, const int* stop, int nstop) {
    return ((Sched*)s)->admit(prompt, n, max_tokens, ignore_eos != 0, stop, nstop);
}
API int vs_schedule(void* s) { return ((Sched*)s)->schedule(); }
API int vs_commit(void* s, const int* sampled, int n) { return ((Sched*)s)->commit(sampled, n); }
API int vs_advance(void* s) { return ((Sched*)s)->advance(); }
API int vs_resolve(void* s, const int* sids, const int* toks, int n, int* accepted) {
    return ((Sched*)s)->resolve(sids, toks, n, accepted);
}
API int vs_can_run_ahead(void* s) { return ((Sched*)s)->can_run_ahead() ? 1 : 0; }
API void vs_finish(void* s, int sid, int reason) { ((Sched*)s)->finish(sid, reason); }
API int vs_fail_all(void* s, int* out, int cap) {
    Sched* k = (Sched*)s;
    std::vector<int> ids;
    for (auto& kv : k->seqs)
        if (kv.second.status != FINISHED) ids.push_back(kv.first);
    std::sort(ids.begin(), ids.end());
    for (int sid : ids) k->finish(sid, R_ERROR);
    return copy_out(ids, out, cap);
}
// which: 0 seq ids, 1 handles, 2 starts, 3 qlens, 4 want counts, 5 wants, 6 tokens, 7 sampled,
// 8 preempted, 9 started, 10 running, 11 waiting, 12 finished
API int vs_list(void* s, int which, int* out, int cap) {
    Sched* k = (Sched*)s;
    const Plan& p = k->plan;
    switch (which) {
        case 0: return copy_out(p.seq_ids, out, cap);
        case 1: return copy_out(p.handles, out, cap);
        case 2: return copy_out(p.starts, out, cap);
        case 3: return copy_out(p.qlens, out, cap);
        case 4: return copy_out(p.want_counts, out, cap);
        case 5: return copy_out(p.wants, out, cap);
        case 6: return copy_out(p.tokens, out, cap);
        case 7: return copy_out(p.sampled, out, cap);
        case 8: return copy_out(p.preempted, out, cap);
        case 9: return copy_out(p.started, out, cap);
        case 10: return copy_out(k->running, out, cap);
        case 11: { std::vector<int> w(k->waiting.begin(), k->waiting.end()); return copy_out(w, out, cap); }
        case 12: return copy_out(k->finished, out, cap);
        case 13: return copy_out(p.token_src, out, cap);
    }
    return fail(-1, "unknown list");
}
// sizes of the planned step: entries, tokens, wanted rows, preempted, started, pure decode (1/0),
// pages the longest entry's block table must cover, requests finished and not yet drained,
// whether a token of the step is still to be produced by the step before it
API void vs_plan_info(void* s, int* info) {
    Sched* k = (Sched*)s;
    const Plan& p = k->plan;
    int width = 1;
    for (size_t i = 0; i < p.qlens.size(); ++i) width = std::max(width, k->cache->pages_for(p.starts[i] + p.qlens[i]));
    info[6] = width;
    info[7] = (int)k->finished.size();
    info[8] = p.has_unknown ? 1 : 0;
    info[0] = (int)p.seq_ids.size();
    info[1] = (int)p.tokens.size();
    info[2] = (int)p.sampled.size();
    info[3] = (int)p.preempted.size();
    info[4] = (int)p.started.size();
    int pure = !p.seq_ids.empty();
    for (size_t i = 0; i < p.qlens.size(); ++i) pure = pure && p.qlens[i] == 1 && p.want_counts[i] == 1;
    info[5] = pure;
}
API int vs_pack_plan(void* s, int n_cap, int s_cap, int width, int r_cap, int padded, const int* pad_pages,
                     int scratch_slot, int* out, int* info) {
    Sched* k = (Sched*)s;
    const Plan& p = k->plan;
    PackArgs a{(int)p.seq_ids.size(), p.handles.data(), p.qlens.data(), p.tokens.data(), p.want_counts.data(),
               p.wants.data(), p.has_unknown ? p.token_src.data() : nullptr, n_cap, s_cap, width, r_cap, padded,
               pad_pages, scratch_slot};
    return pack(*k->cache, a, out, info);
}
// What the step function does after it ran the planned step: every entry's request has
// computed its tokens (windowed groups give pages back here).
API int vs_commit_cache(void* s) {
    Sched* k = (Sched*)s;
    const Plan& p = k->plan;
    for (size_t i = 0; i < p.handles.size(); ++i)
        if (k->cache->commit(p.handles[i], p.starts[i] + p.qlens[i]) != 0) return -2;
    return 0;
}
API void vs_clear_finished(void* s) { ((Sched*)s)->finished.clear(); }
API void vs_erase(void* s, int sid) { ((Sched*)s)->seqs.erase(sid); }
// field: 0 status, 1 prompt_len, 2 num_computed, 3 prefill_target, 4 handle, 5 preemptions, 6 reason,
// 7 total_len, 8 exists
API int vs_seq_get(void* s, int sid, int field) {
    Seq* q = ((Sched*)s)->get(sid);
    if (!q) return field == 8 ? 0 : -1;
    switch (field) {
        case 0: return q->status;
        case 1: return q->prompt_len;
        case 2: return q->num_computed;
        case 3: return q->prefill_target;
        case 4: return q->handle;
        case 5: return q->preemptions;
        case 6: return q->reason;
        case 7: return q->total_len();
        case 8: return 1;
    }
    return -1;
}
API int vs_seq_tokens(void* s, int sid, int from, int* out, int cap) {
    Seq* q = ((Sched*)s)->get(sid);
    if (!q) return 0;
    from = std::max(0, std::min(from, (int)q->tokens.size()));
    int n = std::min((int)q->tokens.size() - from, cap);
    if (n > 0 && out) std::memcpy(out, q->tokens.data() + from, sizeof(int) * (size_t)n);
    return (int)q->tokens.size() - from;
}
API int vs_counts(void* s, int which) {
    Sched* k = (Sched*)s;
    switch (which) {
        case 0: return (int)k->running.size();
        case 1: return (int)k->waiting.size();
        case 2: return (int)k->finished.size();
        case 3: return (int)k->seqs.size();
    }
    return -1;
}
