// Paged fp16 K/V store: host block allocator (authoritative), device block-table mirror,
// and the append / gather / scrub kernels.
//
// HBM layout (fp16): kv[layer][physical block][head][K tile | V tile], tile = 16 tokens x dhead.
// For dhead 16 a (block, head) pair is 1 KiB and a (layer, block) slab over 24 heads is 24 KiB of
// contiguous memory: the decode kernel fetches such a slab with a single bulk copy.
#include "common.cuh"

#include <atomic>

#include <algorithm>
#include <cmath>

namespace jgpt {

// ------------------------------------------------------------------------------------------
// Kernels
// ------------------------------------------------------------------------------------------

// One thread moves CH = min(8, DH) consecutive elements of one (token, head) row of K and of V:
// fp32 in, RoPE on K (interleaved pairs, table lookup), fp16 round-to-nearest-even, one 16-byte
// store each.  RoPE arithmetic is mul, mul, sub / mul, mul, add with separate roundings
// (no FMA contraction) so the payload is reproducible on a CPU.
template <int DH>
__global__ void __launch_bounds__(256) kv_append_kernel(__half *__restrict__ kv, const int *__restrict__ table,
                                                        const float2 *__restrict__ rope, const float *__restrict__ k,
                                                        const float *__restrict__ v, const int *__restrict__ seq_ids,
                                                        const int *__restrict__ slot_pos, const int *__restrict__ rope_pos,
                                                        int n, int H, int layer, int n_blocks, int max_seqs, int mbs,
                                                        int max_positions, int *__restrict__ status) {
    constexpr int CH = DH < 8 ? DH : 8;  // elements per thread
    constexpr int CPR = DH / CH;         // chunks per row
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)n * H * CPR;
    if (gid >= total) return;
    const int c = (int)(gid % CPR);
    const int h = (int)((gid / CPR) % H);
    const int t = (int)(gid / ((long long)CPR * H));
    const int seq = seq_ids[t], sp = slot_pos[t], rp = rope_pos[t];
    if (seq < 0 || seq >= max_seqs) { atomicOr(status, DEV_STATUS_BAD_SEQ); return; }
    if (sp < 0 || sp >= mbs * kBlockTokens || rp < 0 || rp >= max_positions) {
        atomicOr(status, DEV_STATUS_BAD_POSITION);
        return;
    }
    const int phys = table[(size_t)seq * mbs + sp / kBlockTokens];
    if (phys < 0 || phys >= n_blocks) { atomicOr(status, DEV_STATUS_BAD_BLOCK); return; }
    const size_t src = ((size_t)t * H + h) * DH + c * CH;
    float kf[CH], vf[CH];
#pragma unroll
    for (int i = 0; i < CH; i += 4) {
        const float4 a = *reinterpret_cast<const float4 *>(k + src + i);
        const float4 b = *reinterpret_cast<const float4 *>(v + src + i);
        kf[i] = a.x, kf[i + 1] = a.y, kf[i + 2] = a.z, kf[i + 3] = a.w;
        vf[i] = b.x, vf[i + 1] = b.y, vf[i + 2] = b.z, vf[i + 3] = b.w;
    }
    const float2 *cs = rope + (size_t)rp * (DH / 2) + c * (CH / 2);
    __align__(16) __half kh[CH], vh[CH];
#pragma unroll
    for (int j = 0; j < CH / 2; j++) {
        const float2 r = cs[j];
        const float x1 = kf[2 * j], x2 = kf[2 * j + 1];
        kh[2 * j] = __float2half_rn(__fsub_rn(__fmul_rn(x1, r.x), __fmul_rn(x2, r.y)));
        kh[2 * j + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, r.y), __fmul_rn(x2, r.x)));
        vh[2 * j] = __float2half_rn(vf[2 * j]);
        vh[2 * j + 1] = __float2half_rn(vf[2 * j + 1]);
    }
    __half *dst = kv + (((size_t)layer * n_blocks + phys) * H + h) * (2 * kBlockTokens * DH) +
                  (size_t)(sp % kBlockTokens) * DH + c * CH;
    if constexpr (CH == 8) {
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(kh);
        *reinterpret_cast<uint4 *>(dst + kBlockTokens * DH) = *reinterpret_cast<const uint4 *>(vh);
    } else {
        *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(kh);
        *reinterpret_cast<uint2 *>(dst + kBlockTokens * DH) = *reinterpret_cast<const uint2 *>(vh);
    }
}

// Paged fp16 -> contiguous fp32 plane [H, max_seq_len, DH]; rows >= len are zero.
template <int DH>
__global__ void __launch_bounds__(256) kv_gather_kernel(const __half *__restrict__ kv, const int *__restrict__ table_row,
                                                        float *__restrict__ k_out, float *__restrict__ v_out, int H,
                                                        int layer, int n_blocks, int len, int max_seq_len,
                                                        int *__restrict__ status, const int *__restrict__ batch_idx, int mbs) {
    // Batched form (blockIdx.z = which sequence): batch_idx holds (sequence slot, length) pairs, table_row is the
    // whole table and the outputs are laid back to back, one [H, max_seq_len, DH] plane per sequence.
    if (batch_idx) {
        const int seq = batch_idx[2 * blockIdx.z];
        len = batch_idx[2 * blockIdx.z + 1];
        table_row += (size_t)seq * mbs;
        k_out += (size_t)blockIdx.z * H * max_seq_len * DH;
        v_out += (size_t)blockIdx.z * H * max_seq_len * DH;
    }
    constexpr int CH = DH < 8 ? DH : 8;
    constexpr int CPR = DH / CH;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)H * max_seq_len * CPR;
    if (gid >= total) return;
    const int c = (int)(gid % CPR);
    const int pos = (int)((gid / CPR) % max_seq_len);
    const int h = (int)(gid / ((long long)CPR * max_seq_len));
    float kf[CH], vf[CH];
#pragma unroll
    for (int i = 0; i < CH; i++) kf[i] = 0.f, vf[i] = 0.f;
    if (pos < len) {
        const int phys = table_row[pos / kBlockTokens];
        if (phys < 0 || phys >= n_blocks) {
            atomicOr(status, DEV_STATUS_BAD_BLOCK);
        } else {
            const __half *src = kv + (((size_t)layer * n_blocks + phys) * H + h) * (2 * kBlockTokens * DH) +
                                (size_t)(pos % kBlockTokens) * DH + c * CH;
            __align__(16) __half kh[CH], vh[CH];
            if constexpr (CH == 8) {
                *reinterpret_cast<uint4 *>(kh) = *reinterpret_cast<const uint4 *>(src);
                *reinterpret_cast<uint4 *>(vh) = *reinterpret_cast<const uint4 *>(src + kBlockTokens * DH);
            } else {
                *reinterpret_cast<uint2 *>(kh) = *reinterpret_cast<const uint2 *>(src);
                *reinterpret_cast<uint2 *>(vh) = *reinterpret_cast<const uint2 *>(src + kBlockTokens * DH);
            }
#pragma unroll
            for (int i = 0; i < CH; i++) kf[i] = __half2float(kh[i]), vf[i] = __half2float(vh[i]);
        }
    }
    const size_t dst = ((size_t)h * max_seq_len + pos) * DH + c * CH;
#pragma unroll
    for (int i = 0; i < CH; i += 4) {
        *reinterpret_cast<float4 *>(k_out + dst + i) = make_float4(kf[i], kf[i + 1], kf[i + 2], kf[i + 3]);
        *reinterpret_cast<float4 *>(v_out + dst + i) = make_float4(vf[i], vf[i + 1], vf[i + 2], vf[i + 3]);
    }
}

// Eviction scrub: zero-fill freed blocks in every layer (KvCache.clear() zero-fills its buffers,
// src/main/java/com/veles/llm/jgpt/model/KvCacheGpu.java:88-101).  grid = (freed blocks, layers).
__global__ void __launch_bounds__(256) kv_scrub_kernel(__half *__restrict__ kv, const int *__restrict__ blocks,
                                                       int n_blocks, size_t block_halfs, int *__restrict__ status) {
    const int phys = blocks[blockIdx.x];
    if (phys < 0 || phys >= n_blocks) {
        if (threadIdx.x == 0) atomicOr(status, DEV_STATUS_BAD_BLOCK);
        return;
    }
    uint4 *dst = reinterpret_cast<uint4 *>(kv + ((size_t)blockIdx.y * n_blocks + phys) * block_halfs);
    const size_t n16 = block_halfs * sizeof(__half) / 16;
    for (size_t i = threadIdx.x; i < n16; i += blockDim.x) dst[i] = make_uint4(0, 0, 0, 0);
}

// ------------------------------------------------------------------------------------------
// Launchers
// ------------------------------------------------------------------------------------------
#define JGPT_DISPATCH_DH(DHV, ...)                                                      \
    switch (DHV) {                                                                      \
        case 4: { constexpr int DH = 4; __VA_ARGS__; } break;                           \
        case 8: { constexpr int DH = 8; __VA_ARGS__; } break;                           \
        case 16: { constexpr int DH = 16; __VA_ARGS__; } break;                         \
        case 32: { constexpr int DH = 32; __VA_ARGS__; } break;                         \
        default: return fail(JGPT_ERR_UNSUPPORTED, "dhead %d not supported", DHV);      \
    }

int32_t launch_kv_append(Pool *p, int layer, const float *k, const float *v, const int *seq_ids, const int *slot_pos,
                         const int *rope_pos, int n) {
    const int cpr = p->dhead / (p->dhead < 8 ? p->dhead : 8);
    const long long total = (long long)n * p->heads * cpr;
    const int threads = 256;
    const unsigned grid = (unsigned)((total + threads - 1) / threads);
    JGPT_DISPATCH_DH(p->dhead, (kv_append_kernel<DH><<<grid, threads, 0, p->ctx->stream>>>(
                                   p->kv, p->d_table, p->d_rope, k, v, seq_ids, slot_pos, rope_pos, n, p->heads, layer,
                                   p->n_blocks, p->max_seqs, p->max_blocks_per_seq, p->max_positions, p->ctx->d_status)));
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

int32_t launch_kv_gather(Pool *p, int layer, int seq, int len, int max_seq_len, float *k_out, float *v_out) {
    const int cpr = p->dhead / (p->dhead < 8 ? p->dhead : 8);
    const long long total = (long long)p->heads * max_seq_len * cpr;
    const int threads = 256;
    const unsigned grid = (unsigned)((total + threads - 1) / threads);
    const int *row = p->d_table + (size_t)seq * p->max_blocks_per_seq;
    JGPT_DISPATCH_DH(p->dhead, (kv_gather_kernel<DH><<<grid, threads, 0, p->ctx->stream>>>(
                                   p->kv, row, k_out, v_out, p->heads, layer, p->n_blocks, len, max_seq_len,
                                   p->ctx->d_status, nullptr, 0)));
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// n sequences in ONE launch (a launch per sequence moves 4.7 MB at d_head 16 / context 1024 and is launch-bound).
static int32_t launch_kv_gather_batch(Pool *p, int layer, const std::vector<int> &seq_len_pairs, int max_seq_len, float *k_out,
                                      float *v_out) {
    const int n = (int)seq_len_pairs.size() / 2;
    if (n > p->gather_idx_cap) {
        if (p->d_gather_idx) JGPT_CUDA_TRY(cudaFree(p->d_gather_idx));
        p->d_gather_idx = nullptr;
        p->gather_idx_cap = std::max(n, 2 * p->gather_idx_cap);
        JGPT_CUDA_TRY(cudaMalloc(&p->d_gather_idx, sizeof(int) * 2 * (size_t)p->gather_idx_cap));
    }
    // pageable source: staged by the runtime before the call returns
    JGPT_CUDA_TRY(cudaMemcpyAsync(p->d_gather_idx, seq_len_pairs.data(), sizeof(int) * seq_len_pairs.size(), cudaMemcpyHostToDevice,
                                  p->ctx->stream));
    const int cpr = p->dhead / (p->dhead < 8 ? p->dhead : 8);
    const long long total = (long long)p->heads * max_seq_len * cpr;
    const dim3 grid((unsigned)((total + 255) / 256), 1, (unsigned)n);
    JGPT_DISPATCH_DH(p->dhead, (kv_gather_kernel<DH><<<grid, 256, 0, p->ctx->stream>>>(
                                   p->kv, p->d_table, k_out, v_out, p->heads, layer, p->n_blocks, 0, max_seq_len,
                                   p->ctx->d_status, p->d_gather_idx, p->max_blocks_per_seq)));
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

int32_t launch_kv_scrub(Pool *p, const std::vector<int> &blocks) {
    if (blocks.empty()) return JGPT_OK;
    if ((int)blocks.size() > p->evict_cap) {
        if (p->d_evict_list) JGPT_CUDA_TRY(cudaFree(p->d_evict_list));
        p->d_evict_list = nullptr;
        p->evict_cap = std::max<int>((int)blocks.size(), 2 * p->evict_cap);
        JGPT_CUDA_TRY(cudaMalloc(&p->d_evict_list, sizeof(int) * (size_t)p->evict_cap));
    }
    JGPT_CUDA_TRY(cudaMemcpyAsync(p->d_evict_list, blocks.data(), sizeof(int) * blocks.size(), cudaMemcpyHostToDevice,
                                  p->ctx->stream));
    const size_t block_halfs = (size_t)p->heads * 2 * kBlockTokens * p->dhead;
    dim3 grid((unsigned)blocks.size(), (unsigned)p->layers);
    kv_scrub_kernel<<<grid, 256, 0, p->ctx->stream>>>(p->kv, p->d_evict_list, p->n_blocks, block_halfs, p->ctx->d_status);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// ------------------------------------------------------------------------------------------
// Host-side helpers
// ------------------------------------------------------------------------------------------
int32_t pool_upload_table_row(Pool *p, int seq) {
    std::vector<int> row((size_t)p->max_blocks_per_seq, -1);
    const SeqState &s = p->seqs[(size_t)seq];
    for (size_t i = 0; i < s.blocks.size(); i++) row[i] = s.blocks[i];
    // Pageable source: the runtime stages it before returning, so `row` may die here.
    JGPT_CUDA_TRY(cudaMemcpyAsync(p->d_table + (size_t)seq * p->max_blocks_per_seq, row.data(), sizeof(int) * row.size(),
                                  cudaMemcpyHostToDevice, p->ctx->stream));
    return JGPT_OK;
}

static int32_t pool_upload_table_entries(Pool *p, int seq, int first, int count) {
    if (count <= 0) return JGPT_OK;
    const SeqState &s = p->seqs[(size_t)seq];
    JGPT_CUDA_TRY(cudaMemcpyAsync(p->d_table + (size_t)seq * p->max_blocks_per_seq + first, s.blocks.data() + first,
                                  sizeof(int) * (size_t)count, cudaMemcpyHostToDevice, p->ctx->stream));
    return JGPT_OK;
}

// Hands back the blocks a sequence holds beyond what n_tokens need, last block first: exactly the reverse of the
// pops jgpt_seq_reserve made, so reserving ahead and trimming leaves the allocator as if it had never reserved.
int32_t pool_trim_reservation(Pool *p, int seq, int n_tokens) {
    SeqState &s = p->seqs[(size_t)seq];
    const int keep = std::max((n_tokens + kBlockTokens - 1) / kBlockTokens, (s.len + kBlockTokens - 1) / kBlockTokens);
    const int have = (int)s.blocks.size();
    if (keep >= have) return JGPT_OK;
    while ((int)s.blocks.size() > keep) {
        p->free_list.push_back(s.blocks.back());
        s.blocks.pop_back();
    }
    JGPT_CUDA_TRY(cudaMemsetAsync(p->d_table + (size_t)seq * p->max_blocks_per_seq + keep, 0xFF, sizeof(int) * (size_t)(have - keep),
                                  p->ctx->stream));
    return JGPT_OK;
}

int32_t pool_ensure_staging(Pool *p, uint64_t n_floats, uint64_t n_ints) {
    if (n_floats > p->stage_f_floats) {
        JGPT_CUDA_TRY(cudaStreamSynchronize(p->ctx->stream));
        if (p->d_stage_f) JGPT_CUDA_TRY(cudaFree(p->d_stage_f));
        if (p->h_stage_f) JGPT_CUDA_TRY(cudaFreeHost(p->h_stage_f));
        p->d_stage_f = nullptr, p->h_stage_f = nullptr, p->stage_f_floats = 0;
        JGPT_CUDA_TRY(cudaMalloc(&p->d_stage_f, sizeof(float) * n_floats));
        JGPT_CUDA_TRY(cudaHostAlloc(&p->h_stage_f, sizeof(float) * n_floats, cudaHostAllocDefault));
        p->stage_f_floats = p->h_stage_f_floats = n_floats;
    }
    if (n_ints > p->stage_i_ints) {
        JGPT_CUDA_TRY(cudaStreamSynchronize(p->ctx->stream));
        if (p->d_stage_i) JGPT_CUDA_TRY(cudaFree(p->d_stage_i));
        if (p->h_stage_i) JGPT_CUDA_TRY(cudaFreeHost(p->h_stage_i));
        p->d_stage_i = nullptr, p->h_stage_i = nullptr, p->stage_i_ints = 0;
        JGPT_CUDA_TRY(cudaMalloc(&p->d_stage_i, sizeof(int) * n_ints));
        JGPT_CUDA_TRY(cudaHostAlloc(&p->h_stage_i, sizeof(int) * n_ints, cudaHostAllocDefault));
        p->stage_i_ints = p->h_stage_i_ints = n_ints;
    }
    return JGPT_OK;
}

int32_t pool_ensure_split_scratch(Pool *p, uint64_t partial_floats, uint64_t tickets) {
    if (partial_floats > p->partials_floats) {
        JGPT_CUDA_TRY(cudaStreamSynchronize(p->ctx->stream));
        if (p->d_partials) JGPT_CUDA_TRY(cudaFree(p->d_partials));
        p->d_partials = nullptr, p->partials_floats = 0;
        JGPT_CUDA_TRY(cudaMalloc(&p->d_partials, sizeof(float) * partial_floats));
        p->partials_floats = partial_floats;
        p->generation += (uint64_t)1 << 32;  // captured graphs hold the old address
    }
    if (tickets > p->n_tickets) {
        JGPT_CUDA_TRY(cudaStreamSynchronize(p->ctx->stream));
        if (p->d_tickets) JGPT_CUDA_TRY(cudaFree(p->d_tickets));
        p->d_tickets = nullptr, p->n_tickets = 0;
        JGPT_CUDA_TRY(cudaMalloc(&p->d_tickets, sizeof(int) * tickets));
        JGPT_CUDA_TRY(cudaMemsetAsync(p->d_tickets, 0, sizeof(int) * tickets, p->ctx->stream));
        p->n_tickets = tickets;
        p->generation += (uint64_t)1 << 32;
    }
    return JGPT_OK;
}

static void free_seq_blocks(Pool *p, SeqState &s, std::vector<int> *freed) {
    for (int b : s.blocks) {
        p->free_list.push_back(b);
        if (freed) freed->push_back(b);
    }
    s.blocks.clear();
    s.len = 0;
}

// Frees everything a pool owns (also a partly built one: null pointers are skipped by the runtime).
static void release_pool(Pool *p) {
    cudaFree(p->kv), cudaFree(p->d_table), cudaFree(p->d_rope), cudaFree(p->d_partials), cudaFree(p->d_tickets);
    cudaFree(p->d_evict_list), cudaFree(p->d_stage_f), cudaFree(p->d_stage_i);
    cudaFree(p->d_prefill_desc);
    cudaFree(p->d_item_counters);
    cudaFree(p->d_gather_idx);
    if (p->s_in) {
        cudaStreamDestroy(p->s_in), cudaStreamDestroy(p->s_out), cudaEventDestroy(p->ev_start);
        for (int g = 0; g < 4; g++) cudaEventDestroy(p->ev_in[g]), cudaEventDestroy(p->ev_done[g]);
    }
    cudaFreeHost(p->h_stage_f), cudaFreeHost(p->h_stage_i);
    delete p;
}

}  // namespace jgpt

using namespace jgpt;

#define GET_POOL(p, h)                                                      \
    Pool *p = pool_registry().get(h);                                       \
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");              \
    JGPT_CUDA_TRY(make_current(p->ctx))

#define CHECK_SEQ(p, seq)                                                                                  \
    JGPT_REQUIRE((seq) >= 0 && (seq) < (p)->max_seqs, JGPT_ERR_OUT_OF_RANGE, "seq %d outside [0,%d)", (seq), \
                 (p)->max_seqs);                                                                           \
    JGPT_REQUIRE((p)->seqs[(size_t)(seq)].used, JGPT_ERR_ILLEGAL_STATE, "seq %d is not allocated", (seq))

extern "C" {

int32_t jgpt_kvpool_create(jgpt_ctx ctxh, int32_t layers, int32_t heads, int32_t dhead, int32_t block_tokens,
                           int32_t n_blocks, int32_t max_seqs, int32_t max_blocks_per_seq, int32_t max_positions,
                           float rope_base, jgpt_kvpool *out) {
    Ctx *c = ctx_registry().get(ctxh);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(out, JGPT_ERR_INVALID_ARGUMENT, "out is null");
    // KvCacheGpu ctor: IllegalArgumentException on non-positive dimensions.
    JGPT_REQUIRE(layers > 0 && heads > 0 && dhead > 0 && n_blocks > 0 && max_seqs > 0 && max_blocks_per_seq > 0 &&
                     max_positions > 0,
                 JGPT_ERR_INVALID_ARGUMENT, "KV pool dimensions must be positive");
    JGPT_REQUIRE(block_tokens == kBlockTokens, JGPT_ERR_UNSUPPORTED, "block_tokens must be %d", kBlockTokens);
    JGPT_REQUIRE(dhead == 4 || dhead == 8 || dhead == 16 || dhead == 32, JGPT_ERR_UNSUPPORTED,
                 "dhead %d not supported (4, 8, 16, 32)", dhead);
    JGPT_REQUIRE(rope_base > 1.f, JGPT_ERR_INVALID_ARGUMENT, "rope_base must be > 1");
    JGPT_CUDA_TRY(make_current(c));
    Pool *p = new Pool();
    p->ctx = c;
    p->layers = layers, p->heads = heads, p->dhead = dhead, p->n_blocks = n_blocks, p->max_seqs = max_seqs;
    p->max_blocks_per_seq = max_blocks_per_seq, p->max_positions = max_positions, p->rope_base = rope_base;
    p->chunk_blocks = std::min(32, std::max(0, env_int("JGPT_B200_CHUNK_BLOCKS", 0)));  // 0 = automatic
    p->stages = env_int("JGPT_B200_STAGES", 0);  // 0 = automatic
    if (p->stages != 0) p->stages = std::min(8, std::max(2, p->stages));
    p->persistent = env_int("JGPT_B200_PERSISTENT", -1);
    p->head_group = env_int("JGPT_B200_HEAD_GROUP", 0);
    p->decode_mma = env_int("JGPT_B200_DECODE_MMA", 0);
    p->prefill_fast = env_int("JGPT_B200_PREFILL_FAST", 0);
    p->stream_hint = env_int("JGPT_B200_STREAM_HINT", 1);
    p->cluster_merge = env_int("JGPT_B200_CLUSTER_MERGE", 1);
    p->launch_overlap = std::min(2, std::max(0, env_int("JGPT_B200_LAUNCH_OVERLAP", 1)));
    p->kv_bytes = (uint64_t)layers * n_blocks * heads * 2 * kBlockTokens * dhead * sizeof(__half);
    cudaError_t e = cudaMalloc(&p->kv, p->kv_bytes);
    if (e != cudaSuccess) {
        cudaGetLastError();
        const uint64_t bytes = p->kv_bytes;
        delete p;
        return fail(JGPT_ERR_OUT_OF_MEMORY, "KV pool of %llu bytes does not fit: %s", (unsigned long long)bytes,
                    cudaGetErrorString(e));
    }
    // from here on a failure must give back what was already taken
    const int32_t rc_build = [&]() -> int32_t {
        JGPT_CUDA_TRY(cudaMemsetAsync(p->kv, 0, p->kv_bytes, c->stream));
        const size_t tn = (size_t)max_seqs * max_blocks_per_seq;
        JGPT_CUDA_TRY(cudaMalloc(&p->d_table, sizeof(int) * tn));
        JGPT_CUDA_TRY(cudaMemsetAsync(p->d_table, 0xFF, sizeof(int) * tn, c->stream));
        JGPT_CUDA_TRY(cudaMalloc(&p->d_item_counters, sizeof(int) * 2));
        JGPT_CUDA_TRY(cudaMemsetAsync(p->d_item_counters, 0, sizeof(int) * 2, c->stream));
        // RoPE table on the host with the reference's formula (rope_4d_kernel,
        // src/main/cpp/jgpt_cuda_extra_kernels_launches.inl:1151-1154): theta = (float)p / powf(base, 2j/dhead).
        {
            const int half = dhead / 2;
            std::vector<float2> tab((size_t)max_positions * half);
            for (int pos = 0; pos < max_positions; pos++)
                for (int j = 0; j < half; j++) {
                    const float theta = (float)pos / powf(rope_base, (2.f * (float)j) / (float)dhead);
                    tab[(size_t)pos * half + j] = make_float2(cosf(theta), sinf(theta));
                }
            JGPT_CUDA_TRY(cudaMalloc(&p->d_rope, sizeof(float2) * tab.size()));
            JGPT_CUDA_TRY(cudaMemcpyAsync(p->d_rope, tab.data(), sizeof(float2) * tab.size(), cudaMemcpyHostToDevice, c->stream));
            JGPT_CUDA_TRY(cudaStreamSynchronize(c->stream));
        }
        return JGPT_OK;
    }();
    if (rc_build) {
        const std::string keep = last_error_ref();
        release_pool(p);
        last_error_ref() = keep;
        return rc_build;
    }
    static std::atomic<uint64_t> next_generation{1};
    p->generation = next_generation.fetch_add(1);
    p->free_list.resize((size_t)n_blocks);
    for (int i = 0; i < n_blocks; i++) p->free_list[(size_t)i] = n_blocks - 1 - i;  // block 0 is handed out first
    p->seqs.resize((size_t)max_seqs);
    *out = pool_registry().add(p);
    return JGPT_OK;
}

int32_t jgpt_kvpool_destroy(jgpt_kvpool h) {
    GET_POOL(p, h);
    cudaStreamSynchronize(p->ctx->stream);
    pool_registry().remove(p);
    release_pool(p);
    return JGPT_OK;
}

int32_t jgpt_kvpool_free_blocks(jgpt_kvpool h, int32_t *n_free_out) {
    GET_POOL(p, h);
    JGPT_REQUIRE(n_free_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    *n_free_out = (int32_t)p->free_list.size();
    return JGPT_OK;
}

int32_t jgpt_kvpool_storage(jgpt_kvpool h, void **dev_out, uint64_t *bytes_out) {
    GET_POOL(p, h);
    if (dev_out) *dev_out = p->kv;
    if (bytes_out) *bytes_out = p->kv_bytes;
    return JGPT_OK;
}

int32_t jgpt_kvpool_set_tuning(jgpt_kvpool h, int32_t chunk_blocks, int32_t stages, int32_t head_group, int32_t persistent,
                               int32_t launch_overlap) {
    GET_POOL(p, h);
    JGPT_REQUIRE(chunk_blocks >= 0 && chunk_blocks <= 32, JGPT_ERR_INVALID_ARGUMENT, "chunk_blocks must be in [0, 32] (0 = automatic)");
    JGPT_REQUIRE(stages == 0 || (stages >= 2 && stages <= 8), JGPT_ERR_INVALID_ARGUMENT, "stages must be 0 (automatic) or in [2, 8]");
    JGPT_REQUIRE(head_group >= 0 && head_group <= p->heads && (head_group == 0 || p->heads % head_group == 0),
                 JGPT_ERR_INVALID_ARGUMENT, "head_group must be 0 (automatic) or a divisor of %d", p->heads);
    JGPT_REQUIRE(launch_overlap >= 0 && launch_overlap <= 2, JGPT_ERR_INVALID_ARGUMENT, "launch_overlap must be 0, 1 or 2");
    p->chunk_blocks = chunk_blocks, p->stages = stages, p->head_group = head_group, p->persistent = persistent;
    p->launch_overlap = launch_overlap;
    p->generation += (uint64_t)1 << 32;  // graphs captured with the old launch shapes must not be replayed
    return JGPT_OK;
}

int32_t jgpt_kvpool_table_device(jgpt_kvpool h, int32_t **dev_out, int32_t *row_stride_out) {
    GET_POOL(p, h);
    if (dev_out) *dev_out = p->d_table;
    if (row_stride_out) *row_stride_out = p->max_blocks_per_seq;
    return JGPT_OK;
}

int32_t jgpt_seq_alloc(jgpt_kvpool h, int32_t *seq_out) {
    GET_POOL(p, h);
    JGPT_REQUIRE(seq_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    for (int s = 0; s < p->max_seqs; s++)
        if (!p->seqs[(size_t)s].used) {
            SeqState &st = p->seqs[(size_t)s];
            st = SeqState();
            st.used = true;
            st.tick = ++p->clock;
            *seq_out = s;
            return JGPT_OK;
        }
    return fail(JGPT_ERR_POOL_EXHAUSTED, "all %d sequence slots are in use", p->max_seqs);
}

int32_t jgpt_seq_free(jgpt_kvpool h, int32_t seq) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    SeqState &s = p->seqs[(size_t)seq];
    free_seq_blocks(p, s, nullptr);
    s.used = false;
    return pool_upload_table_row(p, seq);
}

int32_t jgpt_seq_reserve(jgpt_kvpool h, int32_t seq, int32_t n_tokens) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    JGPT_REQUIRE(n_tokens >= 0, JGPT_ERR_INVALID_ARGUMENT, "n_tokens must be >= 0");
    SeqState &s = p->seqs[(size_t)seq];
    const int want = (n_tokens + kBlockTokens - 1) / kBlockTokens;
    const int have = (int)s.blocks.size();
    if (want <= have) return JGPT_OK;
    JGPT_REQUIRE(want <= p->max_blocks_per_seq, JGPT_ERR_INVALID_ARGUMENT, "%d tokens exceed the per-sequence limit of %d",
                 n_tokens, p->max_blocks_per_seq * kBlockTokens);
    if ((size_t)(want - have) > p->free_list.size())
        return fail(JGPT_ERR_POOL_EXHAUSTED, "need %d KV blocks, %zu free", want - have, p->free_list.size());
    for (int i = have; i < want; i++) {
        s.blocks.push_back(p->free_list.back());
        p->free_list.pop_back();
    }
    return pool_upload_table_entries(p, seq, have, want - have);
}

int32_t jgpt_seq_length(jgpt_kvpool h, int32_t seq, int32_t *len_out) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    JGPT_REQUIRE(len_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    *len_out = p->seqs[(size_t)seq].len;
    return JGPT_OK;
}

int32_t jgpt_seq_set_length(jgpt_kvpool h, int32_t seq, int32_t len) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    SeqState &s = p->seqs[(size_t)seq];
    JGPT_REQUIRE(len >= 0 && len <= (int)s.blocks.size() * kBlockTokens, JGPT_ERR_INVALID_ARGUMENT,
                 "length %d outside [0, %d]", len, (int)s.blocks.size() * kBlockTokens);
    s.len = len;
    s.tick = ++p->clock;
    return JGPT_OK;
}

int32_t jgpt_seq_clear(jgpt_kvpool h, int32_t seq, int32_t zero_fill) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    std::vector<int> freed;
    free_seq_blocks(p, p->seqs[(size_t)seq], &freed);
    int32_t rc = pool_upload_table_row(p, seq);
    if (rc) return rc;
    return zero_fill ? launch_kv_scrub(p, freed) : JGPT_OK;
}

// Block-granular rolling window: forget the oldest n_blocks KV blocks of a sequence.  The blocks go back to the free
// list in table order (the first dropped block is handed out last), the table shifts left, the length drops by
// n_blocks * 16.  O(blocks of the sequence) host work and one small table upload; no K/V byte moves (the reference
// clears its cache and re-prefills the whole window instead, GptAutoregressiveGenerator.java:51-88).
int32_t jgpt_seq_drop_front(jgpt_kvpool h, int32_t seq, int32_t n_blocks, int32_t zero_fill) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    SeqState &s = p->seqs[(size_t)seq];
    JGPT_REQUIRE(n_blocks >= 0 && n_blocks <= (int)s.blocks.size() && s.len >= n_blocks * kBlockTokens, JGPT_ERR_INVALID_ARGUMENT,
                 "cannot drop %d blocks from a sequence of %d tokens in %d blocks", n_blocks, s.len, (int)s.blocks.size());
    if (n_blocks == 0) return JGPT_OK;
    std::vector<int> freed(s.blocks.begin(), s.blocks.begin() + n_blocks);
    for (int b : freed) p->free_list.push_back(b);
    s.blocks.erase(s.blocks.begin(), s.blocks.begin() + n_blocks);
    s.len -= n_blocks * kBlockTokens;
    s.tick = ++p->clock;
    int32_t rc = pool_upload_table_row(p, seq);
    if (rc) return rc;
    return zero_fill ? launch_kv_scrub(p, freed) : JGPT_OK;
}

int32_t jgpt_seq_set_block_table(jgpt_kvpool h, int32_t seq, const int32_t *blocks_host, int32_t n) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    JGPT_REQUIRE(blocks_host && n >= 0 && n <= p->max_blocks_per_seq, JGPT_ERR_INVALID_ARGUMENT, "bad block list");
    std::vector<char> is_free((size_t)p->n_blocks, 0);
    for (int b : p->free_list) is_free[(size_t)b] = 1;
    for (int i = 0; i < n; i++) {
        const int b = blocks_host[i];
        JGPT_REQUIRE(b >= 0 && b < p->n_blocks, JGPT_ERR_OUT_OF_RANGE, "block %d outside the pool", b);
        JGPT_REQUIRE(is_free[(size_t)b] == 1, JGPT_ERR_ILLEGAL_STATE, "block %d is not free (or listed twice)", b);
        is_free[(size_t)b] = 2;
    }
    SeqState &s = p->seqs[(size_t)seq];
    free_seq_blocks(p, s, nullptr);
    std::vector<int> nf;
    nf.reserve(p->free_list.size());
    for (int b : p->free_list)
        if (is_free[(size_t)b] != 2) nf.push_back(b);
    p->free_list.swap(nf);
    s.blocks.assign(blocks_host, blocks_host + n);
    return pool_upload_table_row(p, seq);
}

int32_t jgpt_block_table_copy_out(jgpt_kvpool h, int32_t seq, int32_t *blocks_host, int32_t cap, int32_t *n_out) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    const SeqState &s = p->seqs[(size_t)seq];
    JGPT_REQUIRE(n_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    *n_out = (int32_t)s.blocks.size();
    JGPT_REQUIRE(cap >= *n_out && (blocks_host || *n_out == 0), JGPT_ERR_INVALID_ARGUMENT, "capacity %d < %d", cap, *n_out);
    for (size_t i = 0; i < s.blocks.size(); i++) blocks_host[i] = s.blocks[i];
    return JGPT_OK;
}

int32_t jgpt_block_table_copy_out_device(jgpt_kvpool h, int32_t seq, int32_t *blocks_host, int32_t cap, int32_t *n_out) {
    GET_POOL(p, h);
    JGPT_REQUIRE(seq >= 0 && seq < p->max_seqs, JGPT_ERR_OUT_OF_RANGE, "seq %d outside [0,%d)", seq, p->max_seqs);
    JGPT_REQUIRE(n_out && blocks_host && cap >= p->max_blocks_per_seq, JGPT_ERR_INVALID_ARGUMENT,
                 "need capacity >= max_blocks_per_seq (%d)", p->max_blocks_per_seq);
    JGPT_CUDA_TRY(cudaMemcpyAsync(blocks_host, p->d_table + (size_t)seq * p->max_blocks_per_seq,
                                  sizeof(int) * (size_t)p->max_blocks_per_seq, cudaMemcpyDeviceToHost, p->ctx->stream));
    JGPT_CUDA_TRY(cudaStreamSynchronize(p->ctx->stream));
    int n = 0;
    while (n < p->max_blocks_per_seq && blocks_host[n] >= 0) n++;
    *n_out = n;
    return JGPT_OK;
}

int32_t jgpt_seq_mark_evictable(jgpt_kvpool h, int32_t seq, int32_t evictable) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    p->seqs[(size_t)seq].evictable = evictable != 0;
    return JGPT_OK;
}

int32_t jgpt_kv_evict_lru(jgpt_kvpool h, int32_t need_free, int32_t zero_fill, int32_t *victims_host, int32_t cap,
                          int32_t *n_victims_out) {
    GET_POOL(p, h);
    JGPT_REQUIRE(n_victims_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    std::vector<std::pair<uint64_t, int>> order;
    for (int s = 0; s < p->max_seqs; s++)
        if (p->seqs[(size_t)s].used && p->seqs[(size_t)s].evictable) order.push_back({p->seqs[(size_t)s].tick, s});
    std::sort(order.begin(), order.end());
    std::vector<int> freed;
    int nv = 0;
    for (auto &o : order) {
        if ((int)p->free_list.size() >= need_free) break;
        JGPT_REQUIRE(nv < cap && victims_host, JGPT_ERR_INVALID_ARGUMENT, "victim buffer too small (%d)", cap);
        SeqState &s = p->seqs[(size_t)o.second];
        free_seq_blocks(p, s, &freed);
        s.used = false;
        victims_host[nv++] = o.second;
        int32_t rc = pool_upload_table_row(p, o.second);
        if (rc) return rc;
    }
    *n_victims_out = nv;
    if (zero_fill) {
        int32_t rc = launch_kv_scrub(p, freed);
        if (rc) return rc;
    }
    if ((int)p->free_list.size() < need_free)
        return fail(JGPT_ERR_POOL_EXHAUSTED, "evicted %d sequences, still only %zu of %d blocks free", nv,
                    p->free_list.size(), need_free);
    return JGPT_OK;
}

int32_t jgpt_kv_append(jgpt_kvpool h, int32_t layer, const float *k_dev, const float *v_dev, const int32_t *seq_ids_dev,
                       const int32_t *slot_pos_dev, const int32_t *rope_pos_dev, int32_t n) {
    GET_POOL(p, h);
    JGPT_REQUIRE(layer >= 0 && layer < p->layers, JGPT_ERR_OUT_OF_RANGE, "layer %d outside [0,%d)", layer, p->layers);
    if (n == 0) return JGPT_OK;
    JGPT_REQUIRE(n > 0 && k_dev && v_dev && seq_ids_dev && slot_pos_dev && rope_pos_dev, JGPT_ERR_INVALID_ARGUMENT,
                 "null pointer or negative count");
    return launch_kv_append(p, layer, k_dev, v_dev, seq_ids_dev, slot_pos_dev, rope_pos_dev, n);
}

int32_t jgpt_kv_gather(jgpt_kvpool h, int32_t layer, int32_t seq, int32_t len, int32_t max_seq_len, float *k_out_dev,
                       float *v_out_dev) {
    GET_POOL(p, h);
    CHECK_SEQ(p, seq);
    JGPT_REQUIRE(layer >= 0 && layer < p->layers, JGPT_ERR_OUT_OF_RANGE, "layer %d outside [0,%d)", layer, p->layers);
    JGPT_REQUIRE(max_seq_len > 0 && len >= 0 && len <= max_seq_len, JGPT_ERR_INVALID_ARGUMENT, "bad len/max_seq_len");
    JGPT_REQUIRE(len <= (int)p->seqs[(size_t)seq].blocks.size() * kBlockTokens, JGPT_ERR_INVALID_ARGUMENT,
                 "len %d beyond the reserved blocks", len);
    JGPT_REQUIRE(k_out_dev && v_out_dev, JGPT_ERR_INVALID_ARGUMENT, "null output");
    return launch_kv_gather(p, layer, seq, len, max_seq_len, k_out_dev, v_out_dev);
}

// getK / getV of many caches at once: sequence i's planes land at k_out_dev + i * heads * max_seq_len * dhead.
int32_t jgpt_kv_gather_batch(jgpt_kvpool h, int32_t layer, const int32_t *seq_ids_host, const int32_t *lens_host, int32_t n,
                             int32_t max_seq_len, float *k_out_dev, float *v_out_dev) {
    GET_POOL(p, h);
    JGPT_REQUIRE(layer >= 0 && layer < p->layers, JGPT_ERR_OUT_OF_RANGE, "layer %d outside [0,%d)", layer, p->layers);
    if (n == 0) return JGPT_OK;
    JGPT_REQUIRE(n > 0 && n <= 65535 && seq_ids_host && lens_host && k_out_dev && v_out_dev && max_seq_len > 0, JGPT_ERR_INVALID_ARGUMENT,
                 "null pointer or bad count");
    std::vector<int> pairs((size_t)2 * n);
    for (int i = 0; i < n; i++) {
        const int seq = seq_ids_host[i], len = lens_host[i];
        CHECK_SEQ(p, seq);
        JGPT_REQUIRE(len >= 0 && len <= max_seq_len && len <= (int)p->seqs[(size_t)seq].blocks.size() * kBlockTokens,
                     JGPT_ERR_INVALID_ARGUMENT, "len %d of sequence %d beyond max_seq_len or its reserved blocks", len, seq);
        pairs[(size_t)2 * i] = seq, pairs[(size_t)2 * i + 1] = len;
    }
    return launch_kv_gather_batch(p, layer, pairs, max_seq_len, k_out_dev, v_out_dev);
}

}  // extern "C"
