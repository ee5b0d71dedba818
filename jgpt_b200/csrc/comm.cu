// Gather of the sampled token ids across the GPUs of one box (one process and one context per GPU).
//
// The decode path shards independent sequences over the GPUs and has no collective on its data path;
// the one thing every rank (and the host behind it) needs from the others is what they sampled in a
// step.  Each step a rank hands in a short list of int32 words -- (request id, token) pairs of its
// scheduler, or the token ids of a fixed batch -- and one ncclAllGather over NVLink brings every
// rank's list to every rank.  The reference has nothing to cite here: it drives device 0 only
// (src/main/cpp/jgpt_cuda_jni_ops_graph.inl:112,119).
//
// Design:
//   * NCCL is opened at run time (dlopen of libnccl.so.2) so a single-GPU host needs no NCCL at all.
//   * The communicator is non-blocking (ncclConfig_t::blocking = 0): every NCCL call returns at once and
//     completion is polled with ncclCommGetAsyncError against a host deadline, so a rank whose peers
//     are late gets JGPT_ERR_TIMEOUT back instead of a host thread stuck inside the library.
//   * Collectives run on a stream of their own, ordered after the context's stream by an event when
//     the words come from device memory.  A ring of `depth + 2` slots (page-locked host staging,
//     device send and receive buffers, one event each) lets the result of step t be read up to
//     `depth` steps later: the ranks never meet after every step, and one rank's prefill does not
//     stall the others' decode steps.
//   * Every rank contributes the same number of words (1 count + max_words payload, padded), so the
//     collective has one shape.  Results come back in submission order, rank by rank.
//   * No peer pointers are handed to any kernel and nothing here uses multicast loads; the transport
//     is whatever NCCL picks (set NCCL_NVLS_ENABLE=0 to keep it off NVLink multicast objects).
#include "common.cuh"

#include <dlfcn.h>
#include <nccl.h>

#include <chrono>
#include <deque>
#include <thread>

namespace jgpt {

namespace {

struct NcclApi {
    void *handle = nullptr;
    ncclResult_t (*GetUniqueId)(ncclUniqueId *) = nullptr;
    ncclResult_t (*CommInitRankConfig)(ncclComm_t *, int, ncclUniqueId, int, ncclConfig_t *) = nullptr;
    ncclResult_t (*CommGetAsyncError)(ncclComm_t, ncclResult_t *) = nullptr;
    ncclResult_t (*CommAbort)(ncclComm_t) = nullptr;
    ncclResult_t (*CommFinalize)(ncclComm_t) = nullptr;
    ncclResult_t (*CommDestroy)(ncclComm_t) = nullptr;
    ncclResult_t (*AllGather)(const void *, void *, size_t, ncclDataType_t, ncclComm_t, cudaStream_t) = nullptr;
    const char *(*GetErrorString)(ncclResult_t) = nullptr;
    ncclResult_t (*GetVersion)(int *) = nullptr;
    std::string error;
};

NcclApi &nccl_api() {
    static NcclApi api;
    static std::once_flag once;
    std::call_once(once, [] {
        const char *names[] = {getenv("JGPT_B200_NCCL_LIB"), "libnccl.so.2", "libnccl.so"};
        for (const char *n : names) {
            if (!n || !*n) continue;
            api.handle = dlopen(n, RTLD_NOW | RTLD_GLOBAL);
            if (api.handle) break;
        }
        if (!api.handle) {
            api.error = std::string("libnccl.so.2 not found (") + (dlerror() ? dlerror() : "dlopen failed") +
                        "); set JGPT_B200_NCCL_LIB to its path";
            return;
        }
#define JGPT_NCCL_SYM(field, name)                                                        \
    api.field = reinterpret_cast<decltype(api.field)>(dlsym(api.handle, name));           \
    if (!api.field && api.error.empty()) api.error = std::string("libnccl lacks ") + name
        JGPT_NCCL_SYM(GetUniqueId, "ncclGetUniqueId");
        JGPT_NCCL_SYM(CommInitRankConfig, "ncclCommInitRankConfig");
        JGPT_NCCL_SYM(CommGetAsyncError, "ncclCommGetAsyncError");
        JGPT_NCCL_SYM(CommAbort, "ncclCommAbort");
        JGPT_NCCL_SYM(CommFinalize, "ncclCommFinalize");
        JGPT_NCCL_SYM(CommDestroy, "ncclCommDestroy");
        JGPT_NCCL_SYM(AllGather, "ncclAllGather");
        JGPT_NCCL_SYM(GetErrorString, "ncclGetErrorString");
        JGPT_NCCL_SYM(GetVersion, "ncclGetVersion");
#undef JGPT_NCCL_SYM
    });
    return api;
}

using Clock = std::chrono::steady_clock;

struct Slot {
    int *send_host = nullptr, *recv_host = nullptr;  // page-locked
    int *send_dev = nullptr, *recv_dev = nullptr;
    cudaEvent_t done = nullptr;
};

struct Comm {
    Ctx *ctx = nullptr;
    ncclComm_t nccl = nullptr;  // null when world == 1 (nothing to communicate)
    int world = 1, rank = 0, max_words = 0, depth = 0, timeout_ms = 0;
    int words_per_rank = 0;  // 1 + max_words
    cudaStream_t stream = nullptr;
    cudaEvent_t ev_ready = nullptr;
    std::vector<Slot> slots;
    std::deque<int> in_flight, free_slots;
    bool broken = false;  // an NCCL call failed or timed out: only destroy is allowed
};

Registry<Comm> &comm_registry() {
    static Registry<Comm> r;
    return r;
}

// Polls the communicator until the call that returned `first` has left the "in progress" state or the deadline passes.
int32_t nccl_settle(Comm *c, ncclResult_t first, const char *what, int timeout_ms) {
    NcclApi &api = nccl_api();
    ncclResult_t state = first;
    const auto start = Clock::now();
    const auto deadline = start + std::chrono::milliseconds(timeout_ms);
    const auto spin_until = start + std::chrono::microseconds(200);
    while (state == ncclInProgress) {
        if (Clock::now() > deadline) {
            c->broken = true;
            return fail(JGPT_ERR_TIMEOUT, "%s: still in progress after %d ms (a peer rank is late or gone)", what, timeout_ms);
        }
        // A call on a healthy communicator settles within microseconds: ask without sleeping for the first
        // 200 us (a sleep costs about 0.1 ms of timer slack per step), then back off.
        if (Clock::now() > spin_until) std::this_thread::sleep_for(std::chrono::microseconds(50));
        const ncclResult_t q = api.CommGetAsyncError(c->nccl, &state);
        if (q != ncclSuccess) state = q;
    }
    if (state != ncclSuccess) {
        c->broken = true;
        return fail(JGPT_ERR_NCCL, "%s: %s", what, api.GetErrorString(state));
    }
    return JGPT_OK;
}

void free_comm(Comm *c) {
    make_current(c->ctx);
    if (c->nccl) {
        NcclApi &api = nccl_api();
        bool clean = !c->broken && c->in_flight.empty();
        if (clean) {
            // orderly shutdown: flush, then wait (bounded) for the finalize to settle before destroying
            ncclResult_t r = api.CommFinalize(c->nccl);
            ncclResult_t state = r;
            const auto deadline = Clock::now() + std::chrono::milliseconds(std::max(1000, c->timeout_ms));
            while (state == ncclInProgress && Clock::now() < deadline) {
                std::this_thread::sleep_for(std::chrono::microseconds(100));
                if (api.CommGetAsyncError(c->nccl, &state) != ncclSuccess) break;
            }
            clean = state == ncclSuccess;
            if (clean) api.CommDestroy(c->nccl);
        }
        if (!clean) api.CommAbort(c->nccl);  // ends collectives still waiting for a peer and frees the communicator
        c->nccl = nullptr;
    }
    if (c->stream) cudaStreamSynchronize(c->stream);
    for (Slot &s : c->slots) {
        if (s.send_host) cudaFreeHost(s.send_host);
        if (s.recv_host) cudaFreeHost(s.recv_host);
        if (s.send_dev) cudaFree(s.send_dev);
        if (s.recv_dev) cudaFree(s.recv_dev);
        if (s.done) cudaEventDestroy(s.done);
    }
    if (c->ev_ready) cudaEventDestroy(c->ev_ready);
    if (c->stream) cudaStreamDestroy(c->stream);
    delete c;
}

// Enqueues gather + download of the slot on the communication stream (the send buffer is already filled / being
// filled on that stream).
int32_t enqueue_gather(Comm *c, int slot_id) {
    Slot &s = c->slots[(size_t)slot_id];
    const size_t bytes = sizeof(int) * (size_t)c->words_per_rank;
    if (c->world > 1) {
        const ncclResult_t r = nccl_api().AllGather(s.send_dev, s.recv_dev, (size_t)c->words_per_rank, ncclInt32, c->nccl, c->stream);
        const int32_t rc = nccl_settle(c, r, "ncclAllGather(token ids)", c->timeout_ms);
        if (rc) return rc;
    } else {
        JGPT_CUDA_TRY(cudaMemcpyAsync(s.recv_dev, s.send_dev, bytes, cudaMemcpyDeviceToDevice, c->stream));
    }
    JGPT_CUDA_TRY(cudaMemcpyAsync(s.recv_host, s.recv_dev, bytes * (size_t)c->world, cudaMemcpyDeviceToHost, c->stream));
    JGPT_CUDA_TRY(cudaEventRecord(s.done, c->stream));
    c->in_flight.push_back(slot_id);
    return JGPT_OK;
}

}  // namespace

}  // namespace jgpt

using namespace jgpt;

#define GET_COMM(c, h)                                                   \
    Comm *c = comm_registry().get(h);                                    \
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad communicator handle");     \
    JGPT_CUDA_TRY(make_current(c->ctx))

extern "C" {

int32_t jgpt_comm_unique_id(void *id_out, int32_t cap_bytes) {
    JGPT_REQUIRE(id_out && cap_bytes >= (int32_t)sizeof(ncclUniqueId), JGPT_ERR_INVALID_ARGUMENT,
                 "the unique id needs a buffer of %d bytes", (int)sizeof(ncclUniqueId));
    NcclApi &api = nccl_api();
    JGPT_REQUIRE(api.error.empty(), JGPT_ERR_NCCL, "%s", api.error.c_str());
    ncclUniqueId id;
    const ncclResult_t r = api.GetUniqueId(&id);
    JGPT_REQUIRE(r == ncclSuccess, JGPT_ERR_NCCL, "ncclGetUniqueId: %s", api.GetErrorString(r));
    memcpy(id_out, &id, sizeof(id));
    return JGPT_OK;
}

int32_t jgpt_comm_create(jgpt_ctx ctxh, const void *unique_id, int32_t world, int32_t rank, int32_t max_words, int32_t depth,
                         int32_t timeout_ms, uint64_t *comm_out) {
    Ctx *ctx = ctx_registry().get(ctxh);
    JGPT_REQUIRE(ctx, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(comm_out && world >= 1 && rank >= 0 && rank < world && max_words >= 1 && max_words <= (1 << 20) && depth >= 0 &&
                     depth <= 64 && timeout_ms >= 1,
                 JGPT_ERR_INVALID_ARGUMENT, "bad communicator shape (world %d, rank %d, max_words %d, depth %d, timeout %d ms)", world,
                 rank, max_words, depth, timeout_ms);
    JGPT_REQUIRE(world == 1 || unique_id, JGPT_ERR_INVALID_ARGUMENT, "a communicator of %d ranks needs the unique id", world);
    JGPT_CUDA_TRY(make_current(ctx));
    Comm *c = new Comm();
    c->ctx = ctx, c->world = world, c->rank = rank, c->max_words = max_words, c->depth = depth, c->timeout_ms = timeout_ms;
    c->words_per_rank = 1 + max_words;
    auto bail = [&](int32_t rc) {
        const std::string keep = last_error_ref();
        c->broken = true;
        free_comm(c);
        last_error_ref() = keep;
        return rc;
    };
#define COMM_TRY(expr)                                                                                         \
    do {                                                                                                       \
        const cudaError_t e__ = (expr);                                                                        \
        if (e__ != cudaSuccess)                                                                                \
            return bail(fail(e__ == cudaErrorMemoryAllocation ? JGPT_ERR_OUT_OF_MEMORY : JGPT_ERR_CUDA, "%s: %s", #expr, \
                             cudaGetErrorString(e__)));                                                        \
    } while (0)
    COMM_TRY(cudaStreamCreateWithFlags(&c->stream, cudaStreamNonBlocking));
    COMM_TRY(cudaEventCreateWithFlags(&c->ev_ready, cudaEventDisableTiming));
    c->slots.resize((size_t)depth + 2);
    const size_t one = sizeof(int) * (size_t)c->words_per_rank;
    for (size_t i = 0; i < c->slots.size(); i++) {
        Slot &s = c->slots[i];
        COMM_TRY(cudaHostAlloc(&s.send_host, one, cudaHostAllocDefault));
        COMM_TRY(cudaHostAlloc(&s.recv_host, one * (size_t)world, cudaHostAllocDefault));
        COMM_TRY(cudaMalloc(&s.send_dev, one));
        COMM_TRY(cudaMalloc(&s.recv_dev, one * (size_t)world));
        COMM_TRY(cudaEventCreateWithFlags(&s.done, cudaEventDisableTiming));
        c->free_slots.push_back((int)i);
    }
#undef COMM_TRY
    if (world > 1) {
        NcclApi &api = nccl_api();
        if (!api.error.empty()) return bail(fail(JGPT_ERR_NCCL, "%s", api.error.c_str()));
        ncclUniqueId id;
        memcpy(&id, unique_id, sizeof(id));
        ncclConfig_t cfg = NCCL_CONFIG_INITIALIZER;
        cfg.blocking = 0;
        const ncclResult_t r = api.CommInitRankConfig(&c->nccl, world, id, rank, &cfg);
        if (r != ncclSuccess && r != ncclInProgress) return bail(fail(JGPT_ERR_NCCL, "ncclCommInitRankConfig: %s", api.GetErrorString(r)));
        int32_t rc = nccl_settle(c, r, "ncclCommInitRankConfig", std::max(timeout_ms, 60000));  // the rendezvous of all ranks
        if (rc) return bail(rc);
        // one collective now: NCCL sets up its connections at the first one, which every rank reaches here together,
        // so no later step pays for it or waits inside it for a peer
        Slot &s = c->slots[0];
        memset(s.send_host, 0, one);
        cudaError_t e = cudaMemcpyAsync(s.send_dev, s.send_host, one, cudaMemcpyHostToDevice, c->stream);
        if (e != cudaSuccess) return bail(fail(JGPT_ERR_CUDA, "warm-up upload: %s", cudaGetErrorString(e)));
        const ncclResult_t g = api.AllGather(s.send_dev, s.recv_dev, (size_t)c->words_per_rank, ncclInt32, c->nccl, c->stream);
        rc = nccl_settle(c, g, "ncclAllGather(warm-up)", std::max(timeout_ms, 60000));
        if (rc) return bail(rc);
        const auto deadline = Clock::now() + std::chrono::milliseconds(std::max(timeout_ms, 60000));
        while ((e = cudaStreamQuery(c->stream)) == cudaErrorNotReady) {
            if (Clock::now() > deadline) return bail(fail(JGPT_ERR_TIMEOUT, "warm-up all-gather did not finish: a peer rank is late or gone"));
            std::this_thread::sleep_for(std::chrono::microseconds(100));
        }
        if (e != cudaSuccess) return bail(fail(JGPT_ERR_CUDA, "warm-up all-gather: %s", cudaGetErrorString(e)));
    }
    *comm_out = comm_registry().add(c);
    return JGPT_OK;
}

int32_t jgpt_comm_destroy(uint64_t h) {
    Comm *c = comm_registry().get(h);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad communicator handle");
    comm_registry().remove(c);
    free_comm(c);
    return JGPT_OK;
}

static int32_t take_slot(Comm *c, int n_words, int *slot_out) {
    JGPT_REQUIRE(!c->broken, JGPT_ERR_ILLEGAL_STATE, "the communicator has failed; destroy it");
    JGPT_REQUIRE(n_words >= 0 && n_words <= c->max_words, JGPT_ERR_INVALID_ARGUMENT, "%d words exceed the gather buffer of %d", n_words,
                 c->max_words);
    JGPT_REQUIRE(!c->free_slots.empty(), JGPT_ERR_ILLEGAL_STATE, "%d steps are in flight; read one with jgpt_comm_pop first",
                 (int)c->in_flight.size());
    *slot_out = c->free_slots.front();
    c->free_slots.pop_front();
    return JGPT_OK;
}

int32_t jgpt_comm_submit(uint64_t h, const int32_t *words_host, int32_t n_words) {
    GET_COMM(c, h);
    JGPT_REQUIRE(words_host || n_words == 0, JGPT_ERR_INVALID_ARGUMENT, "null words");
    int slot_id = -1;
    int32_t rc = take_slot(c, n_words, &slot_id);
    if (rc) return rc;
    Slot &s = c->slots[(size_t)slot_id];
    s.send_host[0] = n_words;
    for (int i = 0; i < c->max_words; i++) s.send_host[1 + i] = i < n_words ? words_host[i] : -1;
    const cudaError_t e = cudaMemcpyAsync(s.send_dev, s.send_host, sizeof(int) * (size_t)c->words_per_rank, cudaMemcpyHostToDevice, c->stream);
    if (e != cudaSuccess) {
        c->free_slots.push_front(slot_id);
        return fail(JGPT_ERR_CUDA, "upload of the step's words: %s", cudaGetErrorString(e));
    }
    rc = enqueue_gather(c, slot_id);
    if (rc) c->free_slots.push_front(slot_id);
    return rc;
}

int32_t jgpt_comm_submit_device(uint64_t h, const int32_t *words_dev, int32_t n_words) {
    GET_COMM(c, h);
    JGPT_REQUIRE(words_dev || n_words == 0, JGPT_ERR_INVALID_ARGUMENT, "null words");
    int slot_id = -1;
    int32_t rc = take_slot(c, n_words, &slot_id);
    if (rc) return rc;
    Slot &s = c->slots[(size_t)slot_id];
    s.send_host[0] = n_words;
    for (int i = 0; i < c->max_words; i++) s.send_host[1 + i] = -1;
    auto undo = [&](int32_t code) {
        c->free_slots.push_front(slot_id);
        return code;
    };
    // the words are produced by work already enqueued on the context's stream: order the communication stream after it
    cudaError_t e = cudaEventRecord(c->ev_ready, c->ctx->stream);
    if (e == cudaSuccess) e = cudaStreamWaitEvent(c->stream, c->ev_ready, 0);
    if (e == cudaSuccess)
        e = cudaMemcpyAsync(s.send_dev, s.send_host, sizeof(int) * (size_t)c->words_per_rank, cudaMemcpyHostToDevice, c->stream);
    if (e == cudaSuccess && n_words > 0)
        e = cudaMemcpyAsync(s.send_dev + 1, words_dev, sizeof(int) * (size_t)n_words, cudaMemcpyDeviceToDevice, c->stream);
    if (e != cudaSuccess) return undo(fail(JGPT_ERR_CUDA, "staging of the step's device words: %s", cudaGetErrorString(e)));
    rc = enqueue_gather(c, slot_id);
    return rc ? undo(rc) : JGPT_OK;
}

int32_t jgpt_comm_in_flight(uint64_t h, int32_t *n_out, int32_t *must_pop_out) {
    GET_COMM(c, h);
    if (n_out) *n_out = (int32_t)c->in_flight.size();
    if (must_pop_out) *must_pop_out = (int)c->in_flight.size() > c->depth ? 1 : 0;
    return JGPT_OK;
}

int32_t jgpt_comm_pop(uint64_t h, int32_t *words_out, int32_t *counts_out, int32_t timeout_ms) {
    GET_COMM(c, h);
    JGPT_REQUIRE(!c->in_flight.empty(), JGPT_ERR_ILLEGAL_STATE, "no step is in flight");
    JGPT_REQUIRE(words_out && counts_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    const int slot_id = c->in_flight.front();
    Slot &s = c->slots[(size_t)slot_id];
    const auto deadline = Clock::now() + std::chrono::milliseconds(std::max(0, timeout_ms));
    for (;;) {
        const cudaError_t q = cudaEventQuery(s.done);
        if (q == cudaSuccess) break;
        if (q != cudaErrorNotReady) {
            c->broken = true;
            return fail(JGPT_ERR_CUDA, "token-id gather: %s", cudaGetErrorString(q));
        }
        if (c->nccl) {
            ncclResult_t state = ncclSuccess;
            const ncclResult_t g = nccl_api().CommGetAsyncError(c->nccl, &state);
            if (g != ncclSuccess || (state != ncclSuccess && state != ncclInProgress)) {
                c->broken = true;
                return fail(JGPT_ERR_NCCL, "token-id gather: %s", nccl_api().GetErrorString(g != ncclSuccess ? g : state));
            }
        }
        // the step stays in flight: the caller may wait again, or give up and destroy the communicator
        if (Clock::now() >= deadline)
            return fail(JGPT_ERR_TIMEOUT, "token-id gather of the oldest step not complete after %d ms (a peer rank is late or gone)", timeout_ms);
        std::this_thread::sleep_for(std::chrono::microseconds(20));
    }
    for (int r = 0; r < c->world; r++) {
        const int *row = s.recv_host + (size_t)r * c->words_per_rank;
        int cnt = row[0];
        if (cnt < 0 || cnt > c->max_words) {
            c->broken = true;
            return fail(JGPT_ERR_NCCL, "rank %d reported %d words; the gather buffer holds %d", r, cnt, c->max_words);
        }
        counts_out[r] = cnt;
        memcpy(words_out + (size_t)r * c->max_words, row + 1, sizeof(int) * (size_t)c->max_words);
    }
    c->in_flight.pop_front();
    c->free_slots.push_back(slot_id);
    return JGPT_OK;
}

}  // extern "C"
