// Shared internals of libjgpt_b200: handles, error reporting, context and pool objects.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <cstdarg>
#include <cstdint>
#include <cstdio>
#include <cstring>
#include <mutex>
#include <string>
#include <unordered_set>
#include <vector>

#include "../../include/jgpt_b200.h"

namespace jgpt {

// ------------------------------------------------------------------------------------------
// Errors.  Native reference code prints to stderr and returns with stale outputs
// (src/main/cpp/jgpt_cuda_error_macros.cuh:9-36); here every call returns a status and keeps a
// thread-local message.
// ------------------------------------------------------------------------------------------
std::string &last_error_ref();
int32_t fail(int32_t code, const char *fmt, ...);

#define JGPT_CUDA_TRY(expr)                                                                           \
    do {                                                                                              \
        cudaError_t _e = (expr);                                                                      \
        if (_e != cudaSuccess)                                                                        \
            return ::jgpt::fail(_e == cudaErrorMemoryAllocation ? JGPT_ERR_OUT_OF_MEMORY : JGPT_ERR_CUDA, \
                                "%s: %s (%s:%d)", #expr, cudaGetErrorString(_e), __FILE__, __LINE__); \
    } while (0)

#define JGPT_REQUIRE(cond, code, ...)                     \
    do {                                                  \
        if (!(cond)) return ::jgpt::fail(code, __VA_ARGS__); \
    } while (0)

// Bits of the device status word (Ctx::d_status).  Kernels never trap; they record and carry on.
enum : int {
    DEV_STATUS_BAD_BLOCK = 1,     // block-table entry outside [0, n_blocks)
    DEV_STATUS_BAD_POSITION = 2,  // slot / RoPE position outside the pool's range
    DEV_STATUS_BAD_SEQ = 4,       // sequence id outside [0, max_seqs)
    DEV_STATUS_WAIT_TIMEOUT = 8,  // a bounded mbarrier wait ran out
    DEV_STATUS_LEN_OVER_BOUND = 16  // lens[i] above the host-declared max_len
};

struct Ctx {
    int device = 0;
    cudaStream_t stream = nullptr;
    int *d_status = nullptr;  // device status word
    int *h_status = nullptr;  // pinned mirror
    int sm_count = 0;
};

struct SeqState {
    bool used = false;
    bool evictable = false;
    int len = 0;
    uint64_t tick = 0;
    std::vector<int> blocks;
};

constexpr int kBlockTokens = 16;

struct Pool {
    Ctx *ctx = nullptr;
    int layers = 0, heads = 0, dhead = 0, n_blocks = 0, max_seqs = 0, max_blocks_per_seq = 0, max_positions = 0;
    float rope_base = 10000.f;
    // device
    __half *kv = nullptr;      // [layers][n_blocks][heads][2][16][dhead]
    uint64_t kv_bytes = 0;
    int *d_table = nullptr;    // [max_seqs][max_blocks_per_seq], -1 = unmapped
    float2 *d_rope = nullptr;  // [max_positions][dhead/2] (cos, sin)
    float *d_partials = nullptr;  // split-K scratch
    uint64_t partials_floats = 0;
    int *d_tickets = nullptr;     // split-K arrival counters (self-resetting)
    int *d_item_counters = nullptr;  // [2] work-queue counters of the dynamic decode launch (self-resetting)
    uint64_t n_tickets = 0;
    int *d_gather_idx = nullptr;  // (sequence, length) pairs of a batched gather
    int gather_idx_cap = 0;
    int *d_evict_list = nullptr;  // freed block ids for the scrub kernel
    int evict_cap = 0;
    // copy streams + events of the pipelined host-buffer entry point (created on first use)
    cudaStream_t s_in = nullptr, s_out = nullptr;
    cudaEvent_t ev_in[4] = {}, ev_done[4] = {}, ev_start = nullptr;
    // which way the host-buffer entry point moves its bytes (measured over the pool's first calls)
    int host_mode = -1, host_tune_calls = 0, host_tune_n = -1, host_tune_layers = -1;
    double host_tune_best[3] = {1e30, 1e30, 1e30};
    void *d_prefill_desc = nullptr;  // per-sequence descriptors of a prefill call
    int prefill_desc_cap = 0;
    // staging for the host-buffer entry points (grow-only)
    float *d_stage_f = nullptr;
    uint64_t stage_f_floats = 0;
    int *d_stage_i = nullptr;
    uint64_t stage_i_ints = 0;
    float *h_stage_f = nullptr;  // pinned
    uint64_t h_stage_f_floats = 0;
    int *h_stage_i = nullptr;    // pinned
    uint64_t h_stage_i_ints = 0;
    // host allocator state (authoritative)
    std::vector<int> free_list;  // LIFO: back() is handed out next
    std::vector<SeqState> seqs;
    uint64_t clock = 0;
    // launch tuning (read once from the environment at creation)
    int chunk_blocks = 0;  // 0 = automatic
    int stages = 0;  // copy-ring stages, 0 = automatic
    int persistent = -1;  // < 0: automatic
    int head_group = 0;  // 0 = automatic
    int decode_mma = 0;  // 1: tensor-core consumer in the decode kernel (dhead 16)
    int prefill_fast = 0;  // d_head-16 prefill attention with single fp16 q / p operands (JGPT_B200_PREFILL_FAST)
    int cluster_merge = 1;  // split-K chunks of a sequence as a thread-block cluster, merged in shared memory (JGPT_B200_CLUSTER_MERGE=0: off)
    int stream_hint = 1;  // decode attention fetches K/V with an evict-first L2 policy (JGPT_B200_STREAM_HINT=0: off)
    int launch_overlap = 1;  // decode attention as a programmatic dependent launch: 0 off, 1 safe subset, 2 + early K/V fetch
    // Unique per pool object (low half) and bumped when a device buffer that kernels are handed is reallocated (high
    // half): captured CUDA graphs are keyed on it, so a pool re-created at the same address never replays an old graph.
    uint64_t generation = 0;
};

struct Model;

// Handle registry: a handle is the object's address, valid only while registered.
template <class T>
struct Registry {
    std::mutex mu;
    std::unordered_set<T *> live;
    uint64_t add(T *p) {
        std::lock_guard<std::mutex> g(mu);
        live.insert(p);
        return reinterpret_cast<uint64_t>(p);
    }
    T *get(uint64_t h) {
        std::lock_guard<std::mutex> g(mu);
        T *p = reinterpret_cast<T *>(h);
        return live.count(p) ? p : nullptr;
    }
    bool remove(T *p) {
        std::lock_guard<std::mutex> g(mu);
        return live.erase(p) != 0;
    }
};
Registry<Ctx> &ctx_registry();
Registry<Pool> &pool_registry();

// Makes the context's device current for the calling thread.
inline cudaError_t make_current(const Ctx *c) { return cudaSetDevice(c->device); }

int env_int(const char *name, int dflt);

// Device status word at the end of a self-synchronising entry point: enqueue the read with the step's other
// device-to-host copies, and after the stream sync turn a non-zero word into JGPT_ERR_DEVICE_CHECK (pool may be null).
cudaError_t status_enqueue_read(Ctx *c);
int32_t status_check_after_sync(Ctx *c, Pool *p, const char *what);

// Grow-only staging helpers (never called on the steady-state decode path once sized).
int32_t pool_ensure_staging(Pool *p, uint64_t n_floats, uint64_t n_ints);
int32_t pool_ensure_split_scratch(Pool *p, uint64_t partial_floats, uint64_t tickets);
// Returns the blocks reserved beyond n_tokens (and beyond the sequence's length) to the free list, last first.
int32_t pool_trim_reservation(Pool *p, int seq, int n_tokens);
// Push rows of the host block table to the device mirror.
int32_t pool_upload_table_row(Pool *p, int seq);

// One prompt of a prefill call: rows [row0, row0 + S) of the packed activations belong to sequence seq_id, row r
// sits at cache slot r - row0 and RoPE position rope_off + (r - row0).
struct PrefillSeq {
    int seq_id, row0, S, rope_off;
};
// What a projection epilogue needs to write K / V rows straight into the paged fp16 store (d_head 16).
struct PagedAppendArgs {
    __half *kv;
    const int *table;
    const float2 *rope;
    const PrefillSeq *seqs;
    int *status;
    int n_seqs, H, layer, n_blocks, mbs, max_positions;
};
// Validates the prompts of a prefill call against the pool and uploads their descriptors (p->d_prefill_desc).
int32_t prefill_upload_descriptors(Pool *p, const int *seq_ids_host, const int *seq_starts_host, const int *rope_offsets_host,
                                   int n_seqs, int *max_S_out, int *n_rows_out);

// Device addresses of one layer's tensors (fp32, row-major [in, out] as GPTModel keeps them).
struct LayerW {
    float *wq, *wk, *wv, *wo, *w1, *w2, *w3, *norm1, *norm2;
};

// A whole decode step (or several greedy steps) of up to fused_step_max_rows() rows as one cooperative launch
// (decode_fused.cu).  The caller fills the model / pool / scratch fields; fused_step_plan fills the splits.
constexpr int kFusedMaxLayers = 40;
constexpr int kFusedMaxKSplit = 4;   // k ranges a narrow projection (Wo, W2) is cut into at most
constexpr int kFusedMaxChunks = 8;   // attention chunks per (row, head) at most
struct FusedStepArgs {
    // model
    const float *tok, *pos, *norm_final, *lm_head;
    LayerW Lw[kFusedMaxLayers];  // by value: the kernel reads the addresses from its parameter space
    int vocab, max_seq, D, H, layers, F;
    float eps;
    // paged store
    __half *kv;
    const int *table;
    const float2 *rope;
    int n_blocks, mbs;
    // rows: idx = [5][n] token ids, position rows (unused here), sequence ids, RoPE positions, lengths after the append
    const int *idx;       // device copy, or nullptr: then idx_inline holds them (no upload before a per-token call)
    int idx_inline[20];
    int n, steps, stop_on_zero;
    // exchange buffers: (value, stamp) pairs, rows padded to the kernel's row count (4 at most)
    uint2 *ll_qkv;   // [rows][3 D]
    uint2 *ll_part;  // [rows][H][nch][18]
    uint2 *ll_po;    // [kFusedMaxKSplit][rows][D]
    uint2 *ll_pw2;   // [kFusedMaxKSplit][rows][D]
    uint2 *ll_act;   // [rows][F]
    uint2 *ll_cand;  // [grid][rows][2] best logit of each CTA's columns and its index
    unsigned stamp0;  // stamps of this launch: stamp0 + 1 ... stamp0 + steps * layers
    float *logits;   // [n][vocab]
    int *next;       // [steps][n] tokens picked
    int *steps_done;
    int *next_host, *steps_done_host;  // the same in mapped page-locked host memory (nullptr: not wanted)
    unsigned *sync_words;  // [1] abort word: holds stamp0 + 1 of a launch that gave up
    int *status;
    // plan
    int grid, nch, cb, ks_o, kl_o, ks_2, kl_2, amax, lm_stage;
    int test_withhold;  // tests only: one CTA withholds a result (JGPT_B200_FUSED_TEST_WITHHOLD=1)
    float scale_log2e;
};
int fused_step_max_rows();
void fused_step_plan(FusedStepArgs &A, int sm_count, int max_len);
int32_t launch_decode_fused(Ctx *ctx, FusedStepArgs &A);

// A decode step of a batch (decode_batch.cu): tile products on the tensor cores, a warp per attention unit, the same
// stamped hand-over between the phases.  Exchange arrays hold (value, stamp) pairs.
struct BatchStepArgs {
    const float *tok, *pos, *norm_final, *lm_head;
    LayerW Lw[kFusedMaxLayers];
    const float *w13[kFusedMaxLayers];  // W1/W3 interleaved in groups of 16 columns, [D][2 F]
    int vocab, max_seq, D, H, layers, F;
    float eps;
    __half *kv;
    const int *table;
    const float2 *rope;
    int n_blocks, mbs;
    const int *idx;  // [5][n] ids, position rows, sequence ids, RoPE positions, lengths after the append
    int n;
    uint2 *xa, *xb;    // [n][D] residual rows (ping-pong)
    uint2 *ssa, *ssb;  // [n][D / 32] partial row sums of squares
    uint2 *qkv;        // [n][3 D]
    uint2 *att;        // [n][D]
    uint2 *act;        // [n][F]
    uint2 *cand;       // [vocab tiles][n][2] best logit of a tile and its index
    uint2 *part;       // [n][H][nch_max][18] split-sequence partials (stamped pairs; a ticket elects the warp that merges)
    int *tickets;      // [n][H], zero between launches
    unsigned stamp0;   // stamps of this launch: stamp0 + 1 ... stamp0 + layers + 2
    unsigned *abort_word;
    int *status;
    float *logits;  // [n][vocab]
    int *next;      // [n]
    int cb, nch_max, kmax;
    float scale_log2e;
};
void batch_step_plan(BatchStepArgs &A, int sm_count, const int *lens_host);
int32_t launch_decode_batch(Ctx *ctx, BatchStepArgs &A);

// Kernel launchers (defined in the .cu files)
int32_t launch_kv_append(Pool *p, int layer, const float *k, const float *v, const int *seq_ids,
                         const int *slot_pos, const int *rope_pos, int n);
int32_t launch_kv_gather(Pool *p, int layer, int seq, int len, int max_seq_len, float *k_out, float *v_out);
int32_t launch_kv_scrub(Pool *p, const std::vector<int> &blocks);
int32_t launch_attn_decode(Pool *p, int layer0, int n_layers, const float *q, const float *k_new,
                           const float *v_new, const int *seq_ids, const int *rope_pos, const int *lens, int n,
                           int max_len, float *out, int overlap = -1);  // overlap < 0: the pool's setting
int32_t launch_attn_prefill(Pool *p, int layer, const float *q, const float *k, const float *v,
                            const int *seq_ids_host, const int *seq_starts_host, const int *rope_offsets_host,
                            int n_seqs, float *out, float *out_image = nullptr, bool skip_append = false, int fast_mode = -1);

#ifdef JGPT_B200_DECODE_TRACE
// Step timeline (trace builds only, never in the shipped library): per launch of the multi-launch decode step, the
// global-timer ns of {first CTA in, last CTA past its wait for the previous kernel, last CTA out}.
struct Timeline {
    unsigned long long *buf;  // device, 4 words per slot
    int slot;
};
Timeline timeline_next();  // the next slot of the step being enqueued (model.cu)
__device__ __forceinline__ unsigned long long timeline_now() {
    unsigned long long t;
    asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
    return t;
}
__device__ __forceinline__ void timeline_in(const Timeline &T) {
    if (T.buf && threadIdx.x == 0) {
        atomicMin(T.buf + 4 * T.slot, timeline_now());
        // which SM each of the launch's first 256 CTAs ran on (after the 256 slots of four words)
        const unsigned cta = blockIdx.x + gridDim.x * (blockIdx.y + gridDim.y * blockIdx.z);
        unsigned smid;
        asm volatile("mov.u32 %0, %%smid;" : "=r"(smid));
        if (cta < 256) T.buf[4 * 256 + 256 * T.slot + cta] = smid + 1;
    }
}
__device__ __forceinline__ void timeline_at(const Timeline &T, int which) {
    if (T.buf && threadIdx.x == 0) atomicMax(T.buf + 4 * T.slot + which, timeline_now());
}
#endif

}  // namespace jgpt
