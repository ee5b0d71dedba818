// Continuous-batching decode scheduler over one model + one paged KV pool (one GPU).
//
// The reference generates one sequence at a time (GptAutoregressiveGenerator.generateGpuKv,
// src/main/java/com/veles/llm/jgpt/model/GptAutoregressiveGenerator.java:108-206) and allocates a fresh
// KvCacheGpu per call.  Here many requests share the pool; the per-sequence rules are the reference's
// (greedy argmax with lowest-index ties, stop when id 0 is sampled, zero tail), the batching policy is new
// and fully deterministic so that block tables, admissions and evictions can be compared bit for bit with a
// written specification:
//
//   step():
//     1. admission, FIFO: the head request needs ceil((prompt + max_new) / 16) blocks, reserved all at once
//        (so a running sequence can never run out of blocks).  If the pool is short, finished sequences are
//        evicted least-recently-used first (ties: lower sequence slot) until it fits; if it still does not
//        fit, admission stops for this step (no overtaking).  Likewise for sequence slots.
//     2. all requests admitted in this step are prefilled in one batched call (split when the rows exceed
//        the model workspace); the argmax of each last row is the request's first new token.
//     3. every request that was already running takes one batched decode step.
//     4. a request finishes when it has max_new tokens or sampled id 0; its blocks stay in the pool, marked
//        evictable, until admission needs them.
#include "common.cuh"

#include <algorithm>
#include <deque>

extern "C" {
int32_t jgpt_forward_prefill_batch(jgpt_model model, jgpt_kvpool pool, const int32_t *seq_ids_host,
                                   const int32_t *seq_starts_host, const int32_t *ids_host, const int32_t *rope_offsets_host,
                                   int32_t n, float *all_logits_host, float *last_logits_host, int32_t *next_tokens_host);
}

namespace jgpt {

enum : int { REQ_WAITING = 0, REQ_RUNNING = 1, REQ_FINISHED = 2 };
enum : int { EV_ADMIT = 1, EV_EVICT = 2, EV_FINISH = 3 };  // (type, a, b): admit(req, seq), evict(seq, req), finish(req, n_tokens)

struct Request {
    std::vector<int> prompt;
    std::vector<int> out;  // sampled tokens
    int max_new = 0, seq = -1, state = REQ_WAITING;
};

struct Sched {
    jgpt_model model = 0;
    jgpt_kvpool pool = 0;
    Pool *p = nullptr;
    int max_running = 0, max_rows = 0, max_seq = 0;
    std::vector<Request> reqs;
    std::deque<int> waiting;
    std::vector<int> running;          // request ids in admission order
    std::vector<int> seq_owner;        // sequence slot -> request id (or -1)
    std::vector<int> events;           // flat (type, a, b) triples
    long long steps = 0, tokens = 0;
};

Registry<Sched> &sched_registry() {
    static Registry<Sched> r;
    return r;
}

static void finish(Sched *s, int rid) {
    Request &r = s->reqs[(size_t)rid];
    r.state = REQ_FINISHED;
    jgpt_seq_mark_evictable(s->pool, r.seq, 1);
    s->events.insert(s->events.end(), {EV_FINISH, rid, (int)r.out.size()});
}

// Evicts finished sequences (LRU) until `need_blocks` blocks are free and, if need_slot, a sequence slot is free.
static int32_t make_room(Sched *s, int need_blocks, bool need_slot) {
    Pool *p = s->p;
    for (;;) {
        bool slot_ok = !need_slot;
        if (need_slot)
            for (int q = 0; q < p->max_seqs && !slot_ok; q++) slot_ok = !p->seqs[(size_t)q].used;
        if ((int)p->free_list.size() >= need_blocks && slot_ok) return JGPT_OK;
        // one victim at a time: the least recently used evictable sequence
        int victim = -1;
        for (int q = 0; q < p->max_seqs; q++) {
            const SeqState &st = p->seqs[(size_t)q];
            if (st.used && st.evictable && (victim < 0 || st.tick < p->seqs[(size_t)victim].tick)) victim = q;
        }
        if (victim < 0) return JGPT_ERR_POOL_EXHAUSTED;
        s->events.insert(s->events.end(), {EV_EVICT, victim, s->seq_owner[(size_t)victim]});
        s->seq_owner[(size_t)victim] = -1;
        int32_t rc = jgpt_seq_free(s->pool, victim);
        if (rc) return rc;
    }
}

}  // namespace jgpt

using namespace jgpt;

#define GET_SCHED(s, h)                                             \
    Sched *s = sched_registry().get(h);                             \
    JGPT_REQUIRE(s, JGPT_ERR_BAD_HANDLE, "bad scheduler handle")

extern "C" {

int32_t jgpt_sched_create(jgpt_model model, jgpt_kvpool pool, int32_t max_running, int32_t max_rows_per_call,
                          int32_t max_seq_len, uint64_t *out) {
    Pool *p = pool_registry().get(pool);
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");
    JGPT_REQUIRE(out && max_running >= 1 && max_rows_per_call >= 1 && max_seq_len >= 1, JGPT_ERR_INVALID_ARGUMENT, "bad limits");
    Sched *s = new Sched();
    s->model = model, s->pool = pool, s->p = p, s->max_running = std::min(max_running, max_rows_per_call);
    s->max_rows = max_rows_per_call, s->max_seq = max_seq_len;
    s->seq_owner.assign((size_t)p->max_seqs, -1);
    *out = sched_registry().add(s);
    return JGPT_OK;
}

int32_t jgpt_sched_destroy(uint64_t h) {
    GET_SCHED(s, h);
    sched_registry().remove(s);
    delete s;
    return JGPT_OK;
}

int32_t jgpt_sched_submit(uint64_t h, const int32_t *prompt_host, int32_t S, int32_t max_new, int32_t *req_id_out) {
    GET_SCHED(s, h);
    JGPT_REQUIRE(prompt_host && S >= 1 && max_new >= 1 && req_id_out, JGPT_ERR_INVALID_ARGUMENT, "bad request");
    // no sliding window while batching: the whole request must fit the context and the per-sequence table
    JGPT_REQUIRE(S + max_new - 1 <= s->max_seq && S + max_new <= s->p->max_blocks_per_seq * kBlockTokens + 1,
                 JGPT_ERR_INVALID_ARGUMENT, "prompt %d + %d new tokens exceed the context of %d", S, max_new, s->max_seq);
    JGPT_REQUIRE(S <= s->max_rows, JGPT_ERR_INVALID_ARGUMENT, "prompt of %d rows exceeds the per-call workspace of %d", S, s->max_rows);
    // a reservation larger than the whole pool could never be admitted and would block the queue for ever
    const int need_blocks = (S + max_new - 1 + kBlockTokens - 1) / kBlockTokens;
    JGPT_REQUIRE(need_blocks <= s->p->n_blocks, JGPT_ERR_INVALID_ARGUMENT,
                 "prompt %d + %d new tokens need %d blocks; the pool has %d", S, max_new, need_blocks, s->p->n_blocks);
    Request r;
    r.prompt.assign(prompt_host, prompt_host + S);
    r.max_new = max_new;
    s->reqs.push_back(std::move(r));
    *req_id_out = (int32_t)s->reqs.size() - 1;
    s->waiting.push_back(*req_id_out);
    return JGPT_OK;
}

// One scheduler step.  pairs_out receives (request id, token) for every token sampled in this step.
int32_t jgpt_sched_step(uint64_t h, int32_t *pairs_out, int32_t cap_pairs, int32_t *n_pairs_out, int32_t *n_running_out,
                        int32_t *n_waiting_out) {
    GET_SCHED(s, h);
    Pool *p = s->p;
    // a step samples at most one token per running request; check the buffer before any state changes
    JGPT_REQUIRE(!pairs_out || cap_pairs >= std::min(s->max_running, (int)(s->running.size() + s->waiting.size())),
                 JGPT_ERR_INVALID_ARGUMENT, "pairs buffer holds %d; a step can produce up to %d", cap_pairs,
                 std::min(s->max_running, (int)(s->running.size() + s->waiting.size())));
    std::vector<int> produced;  // flat pairs
    // the requests that were running before this step decode in phase 3
    const std::vector<int> decoding = s->running;

    // ---- 1. admission ----
    std::vector<int> admitted;
    while (!s->waiting.empty() && (int)s->running.size() < s->max_running) {
        const int rid = s->waiting.front();
        Request &r = s->reqs[(size_t)rid];
        const int S = (int)r.prompt.size();
        // blocks for every position the request can ever occupy: prompt + (max_new - 1) appended tokens
        const int need = (S + r.max_new - 1 + kBlockTokens - 1) / kBlockTokens;
        int32_t rc = make_room(s, need, true);
        if (rc == JGPT_ERR_POOL_EXHAUSTED) {
            // head of line waits for running requests to finish; nobody overtakes.  With nothing running there is
            // nothing to wait for (the blocks are held by sequences the scheduler does not own): report it instead
            // of returning OK for ever.
            if (s->running.empty())
                return fail(JGPT_ERR_POOL_EXHAUSTED, "request %d needs %d blocks: %d free, nothing running and nothing evictable", rid,
                            need, (int)p->free_list.size());
            break;
        }
        if (rc) return rc;
        int32_t seq = -1;
        rc = jgpt_seq_alloc(s->pool, &seq);
        if (rc) return rc;
        rc = jgpt_seq_reserve(s->pool, seq, S + r.max_new - 1);
        if (rc) return rc;
        r.seq = seq, r.state = REQ_RUNNING;
        s->seq_owner[(size_t)seq] = rid;
        s->waiting.pop_front();
        s->running.push_back(rid);
        admitted.push_back(rid);
        s->events.insert(s->events.end(), {EV_ADMIT, rid, seq});
    }

    // ---- 2. batched prefill of the newly admitted requests ----
    for (size_t a0 = 0; a0 < admitted.size();) {
        std::vector<int> seqs, starts{0}, ids, ro;
        size_t a1 = a0;
        while (a1 < admitted.size()) {
            const Request &r = s->reqs[(size_t)admitted[a1]];
            if (!seqs.empty() && (int)(ids.size() + r.prompt.size()) > s->max_rows) break;
            seqs.push_back(r.seq);
            ids.insert(ids.end(), r.prompt.begin(), r.prompt.end());
            starts.push_back((int)ids.size());
            ro.push_back(0);
            a1++;
        }
        std::vector<int> next(seqs.size());
        int32_t rc = jgpt_forward_prefill_batch(s->model, s->pool, seqs.data(), starts.data(), ids.data(), ro.data(), (int)seqs.size(),
                                                nullptr, nullptr, next.data());
        if (rc) return rc;
        for (size_t i = a0; i < a1; i++) {
            const int rid = admitted[i];
            s->reqs[(size_t)rid].out.push_back(next[i - a0]);
            produced.push_back(rid), produced.push_back(next[i - a0]);
        }
        a0 = a1;
    }

    // ---- 3. one decode step for the requests that were already running ----
    if (!decoding.empty()) {
        std::vector<int> seqs, toks, lens, rope;
        for (int rid : decoding) {
            const Request &r = s->reqs[(size_t)rid];
            seqs.push_back(r.seq), toks.push_back(r.out.back());
            lens.push_back(p->seqs[(size_t)r.seq].len), rope.push_back(p->seqs[(size_t)r.seq].len);
        }
        std::vector<int> next(seqs.size());
        int32_t rc = jgpt_forward_decode(s->model, s->pool, seqs.data(), toks.data(), lens.data(), rope.data(), (int)seqs.size(), nullptr,
                                         next.data());
        if (rc) return rc;
        for (size_t i = 0; i < decoding.size(); i++) {
            s->reqs[(size_t)decoding[i]].out.push_back(next[i]);
            produced.push_back(decoding[i]), produced.push_back(next[i]);
        }
    }

    // ---- 4. retire ----
    std::vector<int> still;
    for (int rid : s->running) {
        Request &r = s->reqs[(size_t)rid];
        if ((int)r.out.size() >= r.max_new || r.out.back() == 0) finish(s, rid);
        else still.push_back(rid);
    }
    s->running.swap(still);
    s->steps++, s->tokens += (long long)produced.size() / 2;

    const int np = (int)produced.size() / 2;
    if (n_pairs_out) *n_pairs_out = np;
    if (pairs_out) {
        JGPT_REQUIRE(cap_pairs >= np, JGPT_ERR_INVALID_ARGUMENT, "pairs buffer holds %d, step produced %d", cap_pairs, np);
        std::copy(produced.begin(), produced.end(), pairs_out);
    }
    if (n_running_out) *n_running_out = (int)s->running.size();
    if (n_waiting_out) *n_waiting_out = (int)s->waiting.size();
    return JGPT_OK;
}

// Tokens sampled so far for a request; state: 0 waiting, 1 running, 2 finished.
int32_t jgpt_sched_result(uint64_t h, int32_t req_id, int32_t *tokens_out, int32_t cap, int32_t *n_out, int32_t *state_out,
                          int32_t *seq_out) {
    GET_SCHED(s, h);
    JGPT_REQUIRE(req_id >= 0 && req_id < (int)s->reqs.size(), JGPT_ERR_OUT_OF_RANGE, "request %d unknown", req_id);
    const Request &r = s->reqs[(size_t)req_id];
    if (n_out) *n_out = (int)r.out.size();
    if (state_out) *state_out = r.state;
    if (seq_out) *seq_out = r.seq;
    if (tokens_out) {
        JGPT_REQUIRE(cap >= (int)r.out.size(), JGPT_ERR_INVALID_ARGUMENT, "buffer too small");
        std::copy(r.out.begin(), r.out.end(), tokens_out);
    }
    return JGPT_OK;
}

// Event log as flat (type, a, b) triples: 1 = admit(request, sequence slot), 2 = evict(sequence slot, request),
// 3 = finish(request, tokens sampled).
int32_t jgpt_sched_events(uint64_t h, int32_t *out, int32_t cap_ints, int32_t *n_ints_out) {
    GET_SCHED(s, h);
    if (n_ints_out) *n_ints_out = (int)s->events.size();
    if (out) {
        JGPT_REQUIRE(cap_ints >= (int)s->events.size(), JGPT_ERR_INVALID_ARGUMENT, "buffer too small");
        std::copy(s->events.begin(), s->events.end(), out);
    }
    return JGPT_OK;
}

}  // extern "C"
