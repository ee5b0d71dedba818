// Single-query decode attention over the paged fp16 K/V store, optionally fused with the append
// of the step's new token.
//
// Work item = (layer, sequence, head group, chunk of `chunk_blocks` KV blocks).  A CTA owns a
// ring of shared-memory stages; one producer warp walks the block table and fetches, per KV
// block, the contiguous [head group][K tile | V tile] slab with ONE bulk async copy (TMA engine,
// cp.async.bulk + mbarrier complete_tx).  Consumer threads are (head, token-in-block) pairs: a
// thread scores its token against q (fp32 FMA), keeps a private online-softmax state
// (m, l, o[DH]) and, at the end of the chunk, the 16 lanes of a head merge their states with warp
// shuffles.  Chunks of one sequence are merged by the last CTA to arrive (atomic ticket, no
// waiting), through a small fp32 scratch buffer.
//
// The kernel is HBM-bound (about 1 FLOP per byte at dhead 16): what matters is bytes in flight
// per SM (stages x slab bytes x resident CTAs) and few, large, 16-byte-aligned transactions.
#include "common.cuh"
#include "ptx.cuh"

#include <algorithm>
#include <chrono>
#include <map>
#include <mutex>
#include <tuple>

namespace jgpt {

struct DecodeParams {
    __half *kv;
    const int *table;
    const float2 *rope;
    const float *q, *k_new, *v_new;
    float *out;
    const int *seq_ids, *rope_pos, *lens;
    float *partials;
    int *tickets;
    int *status;
    int n, H, HG, n_hg, layer0, n_layers, mbs, n_blocks, max_seqs, max_positions;
    int chunk_blocks, max_chunks, n_items, stages, max_len;
    float scale_log2e;
    // Launch overlap (programmatic dependent launch).  0: ordinary launch.  1: the launch may start while the previous
    // kernel on the stream drains; everything that reads memory waits for that kernel first (only the barrier set-up
    // runs ahead).  2: additionally the producer warp runs ahead -- lengths, block-table entries and the first K/V
    // slabs are fetched before the previous kernel has finished -- which is only legal when that kernel does not
    // write the K/V store of these layers, the block tables or the index arrays (the caller's promise).
    int overlap;
    int stream_hint;  // 1: K/V slabs are fetched with an evict-first L2 policy
    // 1: the launch is made of clusters of max_chunks CTAs, the chunks of one (layer, sequence, head group); their
    // partial softmax states are merged through distributed shared memory by the CTA of chunk 0 instead of through
    // global scratch and an arrival counter.  Every thread of the cluster passes two cluster barriers, whatever its path.
    int cluster;
    int dynamic;    // 1: CTAs claim work items from counters[0]; 0: item = blockIdx.x + k * gridDim.x
    int *counters;  // [0] next item, [1] CTAs that have finished (the last one resets both)
#ifdef JGPT_B200_DECODE_TRACE
    long long *trace;  // experiments only: 8 timestamps per CTA (never compiled into the shipped library)
    Timeline timeline;
#endif
};

constexpr int kMaxStages = 8;
constexpr int kItemRing = 4;

// Loads one token row of DH halfs from a shared-memory tile into fp32 registers.  For DH = 16
// (two 16-byte halves per row) the order of the two loads alternates with bit 2 of the token
// index so the 8 lanes of a quarter-warp hit 8 distinct 16-byte bank groups; a lane with that bit
// set therefore receives the row with its two halves exchanged (dims 8..15 first).  Callers keep q
// and the accumulator in the same exchanged order (see swap_halves) instead of selecting per load.
template <int DH>
__device__ __forceinline__ void load_row(const unsigned char *tile, int t, float (&r)[DH]) {
    if constexpr (DH == 16) {
        const int sw = (t >> 2) & 1;
        const uint4 lo = *reinterpret_cast<const uint4 *>(tile + t * 32 + sw * 16);
        const uint4 hi = *reinterpret_cast<const uint4 *>(tile + t * 32 + (sw ^ 1) * 16);
        const __half2 *pl = reinterpret_cast<const __half2 *>(&lo), *ph = reinterpret_cast<const __half2 *>(&hi);
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const float2 f = __half22float2(pl[i]), g = __half22float2(ph[i]);
            r[2 * i] = f.x, r[2 * i + 1] = f.y, r[8 + 2 * i] = g.x, r[8 + 2 * i + 1] = g.y;
        }
    } else if constexpr (DH >= 8) {
#pragma unroll
        for (int c = 0; c < DH / 8; c++) {
            const uint4 a = *reinterpret_cast<const uint4 *>(tile + t * (DH * 2) + c * 16);
            const __half2 *pa = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
            for (int i = 0; i < 4; i++) {
                const float2 f = __half22float2(pa[i]);
                r[c * 8 + 2 * i] = f.x, r[c * 8 + 2 * i + 1] = f.y;
            }
        }
    } else {
        const uint2 a = *reinterpret_cast<const uint2 *>(tile + t * (DH * 2));
        const __half2 *pa = reinterpret_cast<const __half2 *>(&a);
#pragma unroll
        for (int i = 0; i < 2; i++) {
            const float2 f = __half22float2(pa[i]);
            r[2 * i] = f.x, r[2 * i + 1] = f.y;
        }
    }
}

// Exchanges the two 8-element halves of a 16-element register row on lanes whose rows arrive exchanged.
template <int DH>
__device__ __forceinline__ void swap_halves(float (&r)[DH], int t) {
    if constexpr (DH == 16) {
        if ((t >> 2) & 1) {
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float x = r[j];
                r[j] = r[8 + j];
                r[8 + j] = x;
            }
        }
    }
}

// Sum v[0..DH) over the 16 lanes of a half-warp.  On return lane t holds, in v[i], the total of
// dimension (i*16 + t) for DH >= 16, or in v[0] the total of dimension (t % DH) for DH < 16.
template <int DH>
__device__ __forceinline__ void halfwarp_reduce_scatter(float (&v)[DH], int t) {
    if constexpr (DH >= 16) {
#pragma unroll
        for (int g = 0; g < DH / 16; g++) {
            float a8[8], a4[4], a2[2];
            const bool b8 = t & 8, b4 = t & 4, b2 = t & 2, b1 = t & 1;
#pragma unroll
            for (int j = 0; j < 8; j++) {
                const float keep = b8 ? v[g * 16 + 8 + j] : v[g * 16 + j];
                const float send = b8 ? v[g * 16 + j] : v[g * 16 + 8 + j];
                a8[j] = keep + __shfl_xor_sync(0xffffffffu, send, 8);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const float keep = b4 ? a8[4 + j] : a8[j];
                const float send = b4 ? a8[j] : a8[4 + j];
                a4[j] = keep + __shfl_xor_sync(0xffffffffu, send, 4);
            }
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const float keep = b2 ? a4[2 + j] : a4[j];
                const float send = b2 ? a4[j] : a4[2 + j];
                a2[j] = keep + __shfl_xor_sync(0xffffffffu, send, 2);
            }
            const float keep = b1 ? a2[1] : a2[0];
            const float send = b1 ? a2[0] : a2[1];
            v[g] = keep + __shfl_xor_sync(0xffffffffu, send, 1);
        }
    } else {
        float mine = 0.f;
#pragma unroll
        for (int d = 0; d < DH; d++) {
            float x = v[d];
#pragma unroll
            for (int off = 8; off >= 1; off >>= 1) x += __shfl_xor_sync(0xffffffffu, x, off);
            if (d == (t % DH)) mine = x;
        }
        v[0] = mine;
    }
}

// Head-group cap: slab <= 24 KiB and at most 30 heads (480 consumer threads + the producer warp).
template <int DH>
constexpr int max_head_group() { return (384 / DH) < 30 ? (384 / DH) : 30; }

template <int DH, bool FUSED, bool MMA>
__global__ void __launch_bounds__(max_head_group<DH>() * kBlockTokens + 32, 2) attn_decode_kernel(const DecodeParams P) {
    constexpr int BT = kBlockTokens;
    constexpr int TILE = BT * DH * 2;    // bytes of one K (or V) tile
    constexpr int HEAD_BYTES = 2 * TILE; // K tile | V tile
    constexpr int OPL = DH >= 16 ? DH / 16 : 1;  // output dims held per lane after the merge
    extern __shared__ __align__(128) unsigned char smem[];
    __shared__ uint64_t full_bar[kMaxStages], empty_bar[kMaxStages];
    __shared__ int s_last;
    __shared__ int s_abort_mem;
    constexpr int kMaxHG = (384 / DH) < 30 ? (384 / DH) : 30;  // == max_head_group<DH>()
    __shared__ float cl_part[kMaxHG * (DH + 2)];  // this CTA's partial (m, l, o[DH]) per head, cluster mode
    // Dynamic mode: the producer warp claims work items from a global counter and hands their ids to the
    // consumers through this small ring, so a resident CTA keeps its copy pipeline full across items and the
    // launch has no wave quantisation (items are a few KV blocks each, claimed as CTAs become free).
    __shared__ int item_ring[kItemRing];
    __shared__ uint64_t item_full[kItemRing], item_empty[kItemRing];
    volatile int *s_abort = &s_abort_mem;

    const int tid = threadIdx.x;
#ifdef JGPT_B200_DECODE_TRACE
    long long tr_gt0 = 0, tr_c0 = clock64(), tr_c1 = 0, tr_c2 = 0, tr_c3 = 0, tr_c4 = 0;
    timeline_in(P.timeline);
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(tr_gt0));
#endif
    const int n_cons = ((BT * P.HG + 31) / 32) * 32;  // consumer threads (padded to whole warps)
    const int n_cons_warps = n_cons / 32;
    const int stage_bytes = P.HG * HEAD_BYTES;
    const int NS = P.stages;

    if (tid == 0) {
        for (int s = 0; s < NS; s++) {
            mbar_init(&full_bar[s], 1);
            mbar_init(&empty_bar[s], (uint32_t)n_cons_warps);
        }
        for (int s = 0; s < kItemRing; s++) {
            mbar_init(&item_full[s], 1);
            mbar_init(&item_empty[s], (uint32_t)n_cons_warps);
        }
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

#ifdef JGPT_B200_DECODE_TRACE
    tr_c1 = clock64();
#endif
    const bool is_producer = tid >= n_cons;
    // q / k_new / v_new come from the previous kernel on the stream, and the split-K scratch and counters are shared
    // with it: the consumers always wait for it.  The producer touches neither; it waits unless the caller has
    // promised that what it reads (lengths, tables, cached K/V) is not written by that kernel.
    // With overlap 2 the scalar consumers wait later still: right before they read q (see below).
    const bool late_wait = P.overlap == 2 && !MMA;
    if (P.overlap && !(P.overlap == 2 && is_producer) && !(late_wait && !is_producer)) griddep_wait();
#ifdef JGPT_B200_DECODE_TRACE
    if (!late_wait) timeline_at(P.timeline, 1);
#endif
    bool waited = !late_wait || is_producer;
    uint32_t it = 0;  // KV blocks processed so far by this CTA (producer and consumers count alike)
    int stage = 0;    // it % NS, kept incrementally (no integer division in the block loop)
    uint32_t phase = 0;  // (it / NS) & 1
    int next_static = blockIdx.x;
    int rslot = 0, rcount = 0;  // item ring position (each side keeps its own)
    uint32_t rphase = 0;

    if (is_producer) {
        // ---------------- producer warp ----------------
        // Walks its work items, publishes each item id to the consumers and issues one bulk copy per KV block.
        // The next item is prepared while the current one is being copied (claim -> lengths -> block-table
        // entries are three dependent global-memory round trips): the steps are spread over the first copy
        // issues of the current item so their latency never leaves the copy ring empty.
        const int lane = tid & 31;
        const uint64_t l2_stream = l2_policy_evict_first();
        int raw = 0;                 // pending claim (lane 0 holds the atomic's result in dynamic mode)
        int nid = -1, n_i = 0, n_z = 0, n_hg = 0, n_c = 0, n_len = 0, n_seq = 0;  // next item, partly resolved
        int cur_nb = 0, cur_entry = 0, nxt_nb = 0, nxt_entry = 0;
        size_t cur_base = 0, nxt_base = 0;
        auto step_claim = [&]() {
            if (P.dynamic) {
                raw = -1;
                if (lane == 0) raw = atomicAdd(P.counters, 1);
            } else {
                raw = next_static;
                next_static += gridDim.x;
            }
        };
        auto step_resolve = [&]() {  // item id known: publish it, start loading its length and sequence id
            nid = P.dynamic ? __shfl_sync(0xffffffffu, raw, 0) : raw;
            if (nid >= P.n_items) nid = -1;
            if (P.dynamic) {
                if (lane == 0) {
                    if (rcount >= kItemRing && !*s_abort) mbar_wait_bounded(&item_empty[rslot], rphase ^ 1u, P.status, s_abort);
                    item_ring[rslot] = nid;
                    mbar_arrive(&item_full[rslot]);
                }
                rcount++;
                if (++rslot == kItemRing) rslot = 0, rphase ^= 1u;
            }
            if (nid >= 0) {
                int r = nid;
                n_c = r % P.max_chunks, r /= P.max_chunks;
                n_hg = r % P.n_hg, r /= P.n_hg;
                n_i = r % P.n, n_z = r / P.n;
                n_len = P.lens[n_i];
                n_seq = P.seq_ids[n_i];
            }
        };
        auto step_table = [&]() {  // length known: block range of the chunk, start loading its table entries
            nxt_nb = 0, nxt_entry = 0;
            if (nid < 0) return;
            const int len = min(n_len, P.max_len);
            const int nblk = len > 0 ? (len + BT - 1) / BT : 0;
            const int nsplit = (nblk + P.chunk_blocks - 1) / P.chunk_blocks;  // balanced chunks, see the consumers
            const int b0 = n_c < nsplit ? (int)((long long)n_c * nblk / nsplit) : nblk;
            const int b1 = n_c < nsplit ? (int)((long long)(n_c + 1) * nblk / nsplit) : nblk;
            if (b0 >= b1 || n_seq < 0 || n_seq >= P.max_seqs) return;  // empty chunk: the consumers skip it too
            nxt_nb = b1 - b0;
            if (lane < nxt_nb) nxt_entry = P.table[(size_t)n_seq * P.mbs + b0 + lane];
            nxt_base = (((size_t)(P.layer0 + n_z) * P.n_blocks) * P.H + (size_t)n_hg * P.HG) * (size_t)HEAD_BYTES;
        };
        step_claim(), step_resolve(), step_table();
        bool triggered = false;
        while (nid >= 0 && !*s_abort) {
            cur_nb = nxt_nb, cur_entry = nxt_entry, cur_base = nxt_base;
            step_claim();
            // static grids know at once whether another item follows; the work queue only after the claim resolves
            const int nid_after_this = P.dynamic ? 0 : (raw < P.n_items ? raw : -1);
            int pending = 2;  // step_resolve, step_table still to run for the next item
            for (int j = 0; j < cur_nb; j++, it++) {
                // Overlapped launches: once most of this CTA's copies are out -- and no further item is coming -- the next
                // launch on the stream may move in, so that ITS first slabs arrive as this launch's last ones are consumed.
                if (P.overlap && !triggered && nid_after_this < 0 && 5 * j >= 3 * cur_nb) {
                    griddep_launch_dependents();
                    triggered = true;
                }
                int phys = __shfl_sync(0xffffffffu, cur_entry, j);
                if (lane == 0) {
                    if (phys < 0 || phys >= P.n_blocks) {
                        atomicOr(P.status, DEV_STATUS_BAD_BLOCK);
                        phys = 0;
                    }
                    const int s = stage;
                    if (it >= (uint32_t)NS && !*s_abort) mbar_wait_bounded(&empty_bar[s], phase ^ 1u, P.status, s_abort);
                    if (!*s_abort) {
                        mbar_expect_tx(&full_bar[s], (uint32_t)stage_bytes);
                        const unsigned char *src = reinterpret_cast<const unsigned char *>(P.kv) + cur_base +
                                                   (size_t)phys * P.H * (size_t)HEAD_BYTES;
                        if (P.stream_hint) bulk_g2s_hint(smem + (size_t)s * stage_bytes, src, (uint32_t)stage_bytes, &full_bar[s], l2_stream);
                        else bulk_g2s(smem + (size_t)s * stage_bytes, src, (uint32_t)stage_bytes, &full_bar[s]);
                    }
                }
                if (++stage == NS) stage = 0, phase ^= 1u;
                if (pending == 2 && j >= 1) step_resolve(), pending = 1;
                else if (pending == 1 && j >= 3) step_table(), pending = 0;
            }
            if (pending == 2) step_resolve(), pending = 1;
            if (pending == 1) step_table();
        }
        // every copy of this CTA has been issued: at the latest now the next launch on the stream may move in
        if (P.overlap && !triggered) griddep_launch_dependents();
        if (P.cluster) cluster_sync(), cluster_sync();  // the two barriers of the consumers' merge
    } else
    for (;;) {
        // a bounded wait ran out: stop taking work (status word says why).  In cluster mode every warp must still walk
        // through its one item to the cluster barriers; with the abort flag up its waits return at once.
        if (*s_abort && !P.cluster) break;
        int item;
        if (!P.dynamic) {
            item = next_static;
            next_static += gridDim.x;
            if (item >= P.n_items) break;
        } else {
            if (!mbar_wait_bounded(&item_full[rslot], rphase, P.status, s_abort)) break;
            item = item_ring[rslot];
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&item_empty[rslot]);
            if (++rslot == kItemRing) rslot = 0, rphase ^= 1u;
            if (item < 0) break;
        }
        // item -> (z = layer slab, i = sequence row, hg = head group, c = chunk); chunk is fastest.
        int r = item;
        const int c = r % P.max_chunks;
        r /= P.max_chunks;
        const int hg = r % P.n_hg;
        r /= P.n_hg;
        const int i = r % P.n;
        const int z = r / P.n;
        int len = P.lens[i];
        if (len > P.max_len) {
            if (tid == 0) atomicOr(P.status, DEV_STATUS_LEN_OVER_BOUND);
            len = P.max_len;
        }
        const int nblk = len > 0 ? (len + BT - 1) / BT : 0;
        // The sequence's blocks are cut into nsplit chunks of equal size (+-1), none longer than chunk_blocks.
        const int nsplit = (nblk + P.chunk_blocks - 1) / P.chunk_blocks;
        const int b0 = c < nsplit ? (int)((long long)c * nblk / nsplit) : nblk;
        const int b1 = c < nsplit ? (int)((long long)(c + 1) * nblk / nsplit) : nblk;
        const int seq = P.seq_ids[i];
        const bool seq_ok = seq >= 0 && seq < P.max_seqs;
        if (!seq_ok && tid == 0) atomicOr(P.status, DEV_STATUS_BAD_SEQ);
        const size_t row = ((size_t)z * P.n + i) * (size_t)(P.H * DH);  // fp32 row of q / k / v / out
        const int head0 = hg * P.HG;
        const int rp_raw = P.rope_pos[i];
        if (!waited) {
            // Late wait (overlap 2): everything the previous kernel on the stream cannot have written -- lengths, ids,
            // RoPE position -- has been fetched above; q, k_new, v_new and every store come after the wait.
            griddep_wait();
            waited = true;
#ifdef JGPT_B200_DECODE_TRACE
            timeline_at(P.timeline, 1);
#endif
        }

        if (b0 >= b1 || !seq_ok) {
            // Empty chunk.  A sequence without any key (len <= 0) gets a zero output row.
            if ((nblk == 0 || !seq_ok) && c == 0)
                for (int e = tid; e < P.HG * DH; e += n_cons) P.out[row + (size_t)head0 * DH + e] = 0.f;
            if (P.cluster) cluster_sync(), cluster_sync();
            continue;
        }
        const int nb = b1 - b0;
        const size_t layer_base = (size_t)(P.layer0 + z) * P.n_blocks;

        if constexpr (MMA) {
            // ---------------- consumers, tensor-core form (dhead 16) ----------------
            // A warp owns two heads.  Per KV block and head: scores^T[16 tok x 8] = K[16 x 16] . Q^T[16 x 8] and
            // O^T[16 dh x 8] += V^T[16 x 16] . P^T[16 x 8] with mma.sync m16n8k16, K and V^T fragments straight
            // from the staged fp16 tile (ldmatrix: no fp16->fp32 conversion instructions at all).  Column 0 of
            // Q^T / P^T holds the fp16 high part of q / p, column 1 the low part, so sums over the two columns
            // keep fp32-level accuracy.  Scores and outputs live in the 8 lanes with (lane & 3) == 0.
            static_assert(!MMA || DH == 16, "the tensor-core consumer is written for dhead 16");
            const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, t4 = lane & 3;
            int rp = rp_raw;
            if (rp < 0 || rp >= P.max_positions) {
                if (tid == 0) atomicOr(P.status, DEV_STATUS_BAD_POSITION);
                rp = 0;
            }
            const float2 *cs = P.rope + (size_t)rp * (DH / 2);
            bool act[2];
            int hh_head[2];
            uint32_t qb[2][2];
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                const int hl = 2 * warp + hh;
                act[hh] = hl < P.HG;
                hh_head[hh] = head0 + (act[hh] ? hl : 0);
                const float *qp = P.q + row + (size_t)hh_head[hh] * DH;
                const float2 x0 = *reinterpret_cast<const float2 *>(qp + 2 * t4);      // dims 2t, 2t+1
                const float2 x1 = *reinterpret_cast<const float2 *>(qp + 2 * t4 + 8);  // dims 2t+8, 2t+9
                const float2 w0 = cs[t4], w1 = cs[t4 + 4];
                float v[4];
                v[0] = __fsub_rn(__fmul_rn(x0.x, w0.x), __fmul_rn(x0.y, w0.y)) * P.scale_log2e;
                v[1] = __fadd_rn(__fmul_rn(x0.x, w0.y), __fmul_rn(x0.y, w0.x)) * P.scale_log2e;
                v[2] = __fsub_rn(__fmul_rn(x1.x, w1.x), __fmul_rn(x1.y, w1.y)) * P.scale_log2e;
                v[3] = __fadd_rn(__fmul_rn(x1.x, w1.y), __fmul_rn(x1.y, w1.x)) * P.scale_log2e;
                __half part[4];
#pragma unroll
                for (int e = 0; e < 4; e++) {
                    const __half hi = __float2half_rn(v[e]);
                    const __half lo = __float2half_rn(v[e] - __half2float(hi));
                    part[e] = g == 0 ? hi : (g == 1 ? lo : __float2half_rn(0.f));
                }
                const __half2 p01 = __halves2half2(part[0], part[1]), p23 = __halves2half2(part[2], part[3]);
                qb[hh][0] = *reinterpret_cast<const uint32_t *>(&p01);
                qb[hh][1] = *reinterpret_cast<const uint32_t *>(&p23);
            }
            float m2[2] = {-INFINITY, -INFINITY}, ls[2] = {0.f, 0.f}, acc[2][4];
#pragma unroll
            for (int hh = 0; hh < 2; hh++)
#pragma unroll
                for (int e = 0; e < 4; e++) acc[hh][e] = 0.f;
            const int new_tok = len - 1;  // fused mode: the token being appended
            const bool has_new = FUSED && (new_tok / BT >= b0) && (new_tok / BT < b1);
            const int mi = lane >> 3, rr = lane & 7;
            const int k_off = ((mi & 1) * 8 + rr) * 32 + (mi >> 1) * 16;          // K tile as the A operand (rows = tokens)
            const int v_off = TILE + ((mi >> 1) * 8 + rr) * 32 + (mi & 1) * 16;   // V tile, transposed load (rows = dims)

            bool aborted = false;
            for (int j = 0; j < nb; j++, it++) {
                const int s = stage;
                const uint32_t ph = phase;
                if (++stage == NS) stage = 0, phase ^= 1u;
                if (!aborted && !mbar_wait_bounded(&full_bar[s], ph, P.status, s_abort)) aborted = true;
                if (aborted) continue;
                unsigned char *base = smem + (size_t)s * stage_bytes;
                if (FUSED && has_new && (b0 + j) == new_tok / BT) {
                    // Lanes 0 and 1 append the new token of the warp's two heads: RoPE'd K and raw V rounded to fp16,
                    // stored to the paged cache and into the staged tile (the bulk copy brought the slot's old content).
                    const bool my_act = lane == 0 ? act[0] : act[1];
                    if (lane < 2 && my_act) {
                        const int h = lane == 0 ? hh_head[0] : hh_head[1];
                        const float *kp = P.k_new + row + (size_t)h * DH, *vp = P.v_new + row + (size_t)h * DH;
                        __align__(16) __half kh[DH], vh[DH];
#pragma unroll
                        for (int jj = 0; jj < DH / 2; jj++) {
                            const float2 x = *reinterpret_cast<const float2 *>(kp + 2 * jj);
                            const float2 y = *reinterpret_cast<const float2 *>(vp + 2 * jj);
                            const float2 w = cs[jj];
                            kh[2 * jj] = __float2half_rn(__fsub_rn(__fmul_rn(x.x, w.x), __fmul_rn(x.y, w.y)));
                            kh[2 * jj + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x.x, w.y), __fmul_rn(x.y, w.x)));
                            vh[2 * jj] = __float2half_rn(y.x);
                            vh[2 * jj + 1] = __float2half_rn(y.y);
                        }
                        const int slot = new_tok % BT;
                        unsigned char *tile = base + (size_t)(2 * warp + lane) * HEAD_BYTES;
                        reinterpret_cast<uint4 *>(tile + slot * 32)[0] = reinterpret_cast<const uint4 *>(kh)[0];
                        reinterpret_cast<uint4 *>(tile + slot * 32)[1] = reinterpret_cast<const uint4 *>(kh)[1];
                        reinterpret_cast<uint4 *>(tile + TILE + slot * 32)[0] = reinterpret_cast<const uint4 *>(vh)[0];
                        reinterpret_cast<uint4 *>(tile + TILE + slot * 32)[1] = reinterpret_cast<const uint4 *>(vh)[1];
                        const int phys = P.table[(size_t)seq * P.mbs + new_tok / BT];
                        if (phys < 0 || phys >= P.n_blocks) {
                            atomicOr(P.status, DEV_STATUS_BAD_BLOCK);
                        } else {
                            __half *dst = P.kv + ((layer_base + phys) * P.H + h) * (size_t)(2 * BT * DH) + (size_t)slot * DH;
                            reinterpret_cast<uint4 *>(dst)[0] = reinterpret_cast<const uint4 *>(kh)[0];
                            reinterpret_cast<uint4 *>(dst)[1] = reinterpret_cast<const uint4 *>(kh)[1];
                            reinterpret_cast<uint4 *>(dst + BT * DH)[0] = reinterpret_cast<const uint4 *>(vh)[0];
                            reinterpret_cast<uint4 *>(dst + BT * DH)[1] = reinterpret_cast<const uint4 *>(vh)[1];
                        }
                        // these generic-proxy stores must be ordered before the next bulk copy into this stage
                        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    }
                    __syncwarp();
                }
                if ((b0 + j) == nblk - 1 && (len % BT) != 0) {
                    // Last block of the sequence: the V rows beyond the last token hold whatever the slot held before.
                    // Their probabilities are exactly 0, but 0 x Inf/NaN is NaN inside the MMA: clear them in the tile.
                    const int first_dead = len % BT;
                    for (int e = lane; e < 2 * (BT - first_dead) * 2; e += 32) {
                        const int hh = e & 1, half16 = (e >> 1) & 1, r = first_dead + (e >> 2);
                        if (hh == 0 ? act[0] : act[1])
                            *reinterpret_cast<uint4 *>(base + (size_t)(2 * warp + hh) * HEAD_BYTES + TILE + r * 32 + half16 * 16) =
                                make_uint4(0, 0, 0, 0);
                    }
                    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                    __syncwarp();
                }
                const int tok0 = (b0 + j) * BT + g;
#pragma unroll
                for (int hh = 0; hh < 2; hh++) {
                    if (!act[hh]) continue;  // warp-uniform
                    const unsigned char *tile = base + (size_t)(2 * warp + hh) * HEAD_BYTES;
                    uint32_t ka[4];
                    ldmatrix_x4(ka, tile + k_off);
                    float sc[4] = {0.f, 0.f, 0.f, 0.f};
                    mma_16816(sc, ka, qb[hh][0], qb[hh][1]);
                    float s0 = sc[0] + sc[1], s1 = sc[2] + sc[3];  // tokens g and g+8 (lanes with t4 == 0)
                    if (tok0 >= len) s0 = -INFINITY;
                    if (tok0 + 8 >= len) s1 = -INFINITY;
                    float bm = fmaxf(s0, s1);
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 4));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 8));
                    bm = fmaxf(bm, __shfl_xor_sync(0xffffffffu, bm, 16));
                    bm = __shfl_sync(0xffffffffu, bm, 0);  // the value of the t4 == 0 lanes, for every lane
                    const float mn = fmaxf(m2[hh], bm);    // finite: the block holds at least one attended token
                    const float corr = fast_exp2(m2[hh] - mn);
                    const float p0 = fast_exp2(s0 - mn), p1 = fast_exp2(s1 - mn);
                    ls[hh] = ls[hh] * corr + (p0 + p1);
                    m2[hh] = mn;
#pragma unroll
                    for (int e = 0; e < 4; e++) acc[hh][e] *= corr;
                    // P^T as the B operand: lanes with g == 0 carry the high parts of p[2t], p[2t+1], p[2t+8], p[2t+9],
                    // lanes with g == 1 the low parts, the other columns are zero.
                    const float x0 = __shfl_sync(0xffffffffu, p0, 8 * t4), x1 = __shfl_sync(0xffffffffu, p0, 8 * t4 + 4);
                    const float y0 = __shfl_sync(0xffffffffu, p1, 8 * t4), y1 = __shfl_sync(0xffffffffu, p1, 8 * t4 + 4);
                    const float pv[4] = {x0, x1, y0, y1};
                    __half part[4];
#pragma unroll
                    for (int e = 0; e < 4; e++) {
                        const __half hi = __float2half_rn(pv[e]);
                        const __half lo = __float2half_rn(pv[e] - __half2float(hi));
                        part[e] = g == 0 ? hi : (g == 1 ? lo : __float2half_rn(0.f));
                    }
                    const __half2 b01 = __halves2half2(part[0], part[1]), b23 = __halves2half2(part[2], part[3]);
                    uint32_t va[4];
                    ldmatrix_x4_trans(va, tile + v_off);
                    mma_16816(acc[hh], va, *reinterpret_cast<const uint32_t *>(&b01), *reinterpret_cast<const uint32_t *>(&b23));
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty_bar[s]);
            }

            // ---- per head: totals over the 8 score lanes, then write / publish ----
            constexpr int PSTRIDE = DH + 2;
            const size_t prow = (((size_t)z * P.n + i) * P.max_chunks) * (size_t)P.H;
            float og[2][2], lt[2];
#pragma unroll
            for (int hh = 0; hh < 2; hh++) {
                float l = ls[hh];
                l += __shfl_xor_sync(0xffffffffu, l, 4);
                l += __shfl_xor_sync(0xffffffffu, l, 8);
                l += __shfl_xor_sync(0xffffffffu, l, 16);
                lt[hh] = l;
                og[hh][0] = acc[hh][0] + acc[hh][1];  // dim g
                og[hh][1] = acc[hh][2] + acc[hh][3];  // dim g + 8
            }
            const bool lane_writes = t4 == 0 && !aborted;
            if (nsplit == 1) {
#pragma unroll
                for (int hh = 0; hh < 2; hh++)
                    if (lane_writes && act[hh]) {
                        const float inv = 1.f / fmaxf(lt[hh], 1e-12f);
                        float *op = P.out + row + (size_t)hh_head[hh] * DH;
                        op[g] = og[hh][0] * inv;
                        op[g + 8] = og[hh][1] * inv;
                    }
                continue;
            }
#pragma unroll
            for (int hh = 0; hh < 2; hh++)
                if (lane_writes && act[hh]) {
                    float *pp = P.partials + (prow + (size_t)c * P.H + hh_head[hh]) * PSTRIDE;
                    pp[2 + g] = og[hh][0];
                    pp[2 + g + 8] = og[hh][1];
                    if (g == 0) pp[0] = m2[hh], pp[1] = lt[hh];
                }
            __threadfence();
            named_bar_sync(1, n_cons);
            int *ticket = P.tickets + ((size_t)z * P.n + i) * P.n_hg + hg;
            if (tid == 0) {
                const int prev = atomicAdd(ticket, 1);
                s_last = (prev == nsplit - 1);
                if (prev == nsplit - 1) *ticket = 0;  // self-reset for the next launch
            }
            named_bar_sync(1, n_cons);
            if (s_last) {
                __threadfence();
#pragma unroll
                for (int hh = 0; hh < 2; hh++)
                    if (lane_writes && act[hh]) {
                        const int h = hh_head[hh];
                        float Mx = -INFINITY;
                        for (int cc = 0; cc < nsplit; cc++) Mx = fmaxf(Mx, __ldcg(P.partials + (prow + (size_t)cc * P.H + h) * PSTRIDE));
                        float L = 0.f, a0 = 0.f, a1 = 0.f;
                        for (int cc = 0; cc < nsplit; cc++) {
                            const float *pp = P.partials + (prow + (size_t)cc * P.H + h) * PSTRIDE;
                            const float w = exp2f(__ldcg(pp) - Mx);
                            L = fmaf(__ldcg(pp + 1), w, L);
                            a0 = fmaf(__ldcg(pp + 2 + g), w, a0);
                            a1 = fmaf(__ldcg(pp + 2 + g + 8), w, a1);
                        }
                        const float inv = 1.f / fmaxf(L, 1e-12f);
                        float *op = P.out + row + (size_t)h * DH;
                        op[g] = a0 * inv;
                        op[g + 8] = a1 * inv;
                    }
            }
            continue;
        }

        // ---------------- consumers, scalar form ----------------
        const int hl = tid / BT, t = tid % BT;
        const bool active = hl < P.HG;
        const int h = head0 + (active ? hl : 0);
        int rp = rp_raw;
        if (rp < 0 || rp >= P.max_positions) {
            if (tid == 0) atomicOr(P.status, DEV_STATUS_BAD_POSITION);
            rp = 0;
        }
        // q row: RoPE at rope_pos, then scaled by (1/sqrt(DH)) * log2(e) so that exp2f can be used.
        float q[DH];
        {
            const float *qp = P.q + row + (size_t)h * DH;
            const float2 *cs = P.rope + (size_t)rp * (DH / 2);
#pragma unroll
            for (int j = 0; j < DH / 2; j++) {
                const float2 x = *reinterpret_cast<const float2 *>(qp + 2 * j);
                const float2 w = cs[j];
                q[2 * j] = __fsub_rn(__fmul_rn(x.x, w.x), __fmul_rn(x.y, w.y)) * P.scale_log2e;
                q[2 * j + 1] = __fadd_rn(__fmul_rn(x.x, w.y), __fmul_rn(x.y, w.x)) * P.scale_log2e;
            }
        }
        // Fused append: the thread whose token is the new one computes the stored payload (RoPE'd K,
        // raw V, both rounded to fp16), writes it to the cache and scores it from registers.
        // Private online-softmax state of this (head, token lane).
        float m = -INFINITY, l = 0.f, o[DH];
#pragma unroll
        for (int d = 0; d < DH; d++) o[d] = 0.f;
        // Fused append: the new token sits at slot len-1.  The lane that owns that slot computes the
        // stored payload (RoPE'd K, raw V, both rounded to fp16), writes it to the cache and starts its
        // softmax state from it; the block loop below then covers the len-1 tokens already cached.
        const int len_cached = FUSED ? len - 1 : len;
        if constexpr (FUSED) {
            const int new_tok = len - 1;
            if (active && (new_tok / BT >= b0) && (new_tok / BT < b1) && (t == new_tok % BT)) {
                const float *kp = P.k_new + row + (size_t)h * DH, *vp = P.v_new + row + (size_t)h * DH;
                const float2 *cs = P.rope + (size_t)rp * (DH / 2);
                __align__(16) __half kh[DH], vh[DH];
                float sc = 0.f;
#pragma unroll
                for (int j = 0; j < DH / 2; j++) {
                    const float2 x = *reinterpret_cast<const float2 *>(kp + 2 * j);
                    const float2 y = *reinterpret_cast<const float2 *>(vp + 2 * j);
                    const float2 w = cs[j];
                    kh[2 * j] = __float2half_rn(__fsub_rn(__fmul_rn(x.x, w.x), __fmul_rn(x.y, w.y)));
                    kh[2 * j + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x.x, w.y), __fmul_rn(x.y, w.x)));
                    vh[2 * j] = __float2half_rn(y.x);
                    vh[2 * j + 1] = __float2half_rn(y.y);
                    sc = fmaf(q[2 * j], __half2float(kh[2 * j]), sc);
                    sc = fmaf(q[2 * j + 1], __half2float(kh[2 * j + 1]), sc);
                    o[2 * j] = __half2float(vh[2 * j]);
                    o[2 * j + 1] = __half2float(vh[2 * j + 1]);
                }
                m = sc, l = 1.f;
                const int phys = P.table[(size_t)seq * P.mbs + new_tok / BT];
                if (phys < 0 || phys >= P.n_blocks) {
                    atomicOr(P.status, DEV_STATUS_BAD_BLOCK);
                } else {
                    __half *dst = P.kv + ((layer_base + phys) * P.H + h) * (size_t)(2 * BT * DH) + (size_t)t * DH;
                    if constexpr (DH >= 8) {
#pragma unroll
                        for (int cc = 0; cc < DH / 8; cc++) {
                            reinterpret_cast<uint4 *>(dst)[cc] = reinterpret_cast<const uint4 *>(kh)[cc];
                            reinterpret_cast<uint4 *>(dst + BT * DH)[cc] = reinterpret_cast<const uint4 *>(vh)[cc];
                        }
                    } else {
                        *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(kh);
                        *reinterpret_cast<uint2 *>(dst + BT * DH) = *reinterpret_cast<const uint2 *>(vh);
                    }
                }
            }
        }

        swap_halves<DH>(q, t);  // match the order in which load_row delivers rows on this lane
        swap_halves<DH>(o, t);
        bool aborted = false;
        for (int j = 0; j < nb; j++, it++) {
            const int s = stage;
            const uint32_t ph = phase;
            if (++stage == NS) stage = 0, phase ^= 1u;
            if (!aborted && !mbar_wait_bounded(&full_bar[s], ph, P.status, s_abort)) aborted = true;
            if (aborted) continue;  // keep counting blocks, touch nothing
#ifdef JGPT_B200_DECODE_TRACE
            if (j == 0 && tr_c2 == 0) tr_c2 = clock64();
#endif
            const int tok = (b0 + j) * BT + t;
            if (active && tok < len_cached) {
                const unsigned char *ktile = smem + (size_t)s * stage_bytes + (size_t)hl * HEAD_BYTES;
                float kr[DH], vr[DH];
                load_row<DH>(ktile, t, kr);
                float sc = 0.f;
#pragma unroll
                for (int d = 0; d < DH; d++) sc = fmaf(q[d], kr[d], sc);
                if (sc > m) {  // new running maximum: rescale the private state
                    const float corr = fast_exp2(m - sc);  // m = -inf on the first token -> 0
                    l *= corr;
#pragma unroll
                    for (int d = 0; d < DH; d++) o[d] *= corr;
                    m = sc;
                }
                load_row<DH>(ktile + TILE, t, vr);
                const float pexp = fast_exp2(sc - m);
                l += pexp;
#pragma unroll
                for (int d = 0; d < DH; d++) o[d] = fmaf(pexp, vr[d], o[d]);
            }
            __syncwarp();
            if ((tid & 31) == 0) mbar_arrive(&empty_bar[s]);
        }
        // After a timed-out wait the thread keeps walking the barriers below (so nobody is left
        // waiting for it) but stores nothing; the item loop ends at its next iteration.

#ifdef JGPT_B200_DECODE_TRACE
        tr_c3 = clock64();
#endif
        // ---- merge the 16 token lanes of each head (warp shuffles) ----
        swap_halves<DH>(o, t);  // back to natural dimension order
        float M = m;
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
        const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
        l *= f;
#pragma unroll
        for (int d = 0; d < DH; d++) o[d] *= f;
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
        halfwarp_reduce_scatter<DH>(o, t);
        // lane t now holds dims {g*16 + t} (DH >= 16) or dim t % DH (DH < 16) in o[0..OPL)
        const bool writer = active && !aborted && (DH >= 16 || t < DH);

        if (nsplit == 1) {
            if (writer) {
                const float inv = 1.f / fmaxf(l, 1e-12f);
#pragma unroll
                for (int g = 0; g < OPL; g++) P.out[row + (size_t)h * DH + g * 16 + (DH >= 16 ? t : t % DH)] = o[g] * inv;
            }
            if (P.cluster) cluster_sync(), cluster_sync();
            continue;
        }
        if (P.cluster) {
            // ---- split-K inside a cluster: partials stay in shared memory, the CTA of chunk 0 merges them ----
            constexpr int PS = DH + 2;
            if (writer) {
                float *pp = cl_part + hl * PS;
#pragma unroll
                for (int g = 0; g < OPL; g++) pp[2 + g * 16 + (DH >= 16 ? t : t % DH)] = o[g];
                if (t == 0) pp[0] = M, pp[1] = l;
            } else if (active && aborted && t == 0) {
                cl_part[hl * PS] = -INFINITY, cl_part[hl * PS + 1] = 0.f;  // a chunk that gave up contributes nothing
            }
            cluster_sync();
            if (c == 0 && writer) {
                const float *pp = cl_part + hl * PS;
                float Mx = -INFINITY;
                for (int cc = 0; cc < nsplit; cc++) Mx = fmaxf(Mx, ld_cluster_f32(pp, (uint32_t)cc));
                float L = 0.f, acc[OPL];
#pragma unroll
                for (int g = 0; g < OPL; g++) acc[g] = 0.f;
                for (int cc = 0; cc < nsplit; cc++) {
                    const float mc = ld_cluster_f32(pp, (uint32_t)cc);
                    const float w = mc == -INFINITY ? 0.f : exp2f(mc - Mx);
                    L = fmaf(ld_cluster_f32(pp + 1, (uint32_t)cc), w, L);
#pragma unroll
                    for (int g = 0; g < OPL; g++)
                        acc[g] = fmaf(ld_cluster_f32(pp + 2 + g * 16 + (DH >= 16 ? t : t % DH), (uint32_t)cc), w, acc[g]);
                }
                const float inv = 1.f / fmaxf(L, 1e-12f);
#pragma unroll
                for (int g = 0; g < OPL; g++) P.out[row + (size_t)h * DH + g * 16 + (DH >= 16 ? t : t % DH)] = acc[g] * inv;
            }
            cluster_sync();  // nobody leaves (and frees its shared memory) before chunk 0 has read it
            continue;
        }

        // ---- split-K: publish the partial, last CTA of the sequence row merges ----
        constexpr int PSTRIDE = DH + 2;
        const size_t prow = (((size_t)z * P.n + i) * P.max_chunks) * (size_t)P.H;  // + c*H + head
        if (writer) {
            float *pp = P.partials + (prow + (size_t)c * P.H + h) * PSTRIDE;
#pragma unroll
            for (int g = 0; g < OPL; g++) pp[2 + g * 16 + (DH >= 16 ? t : t % DH)] = o[g];
            if (t == 0) pp[0] = M, pp[1] = l;
        }
#ifdef JGPT_B200_TRACE_NOMERGE
        if (P.n > 0) continue;  // timing experiment only: partials written, nobody merges
#endif
        __threadfence();
        named_bar_sync(1, n_cons);
        int *ticket = P.tickets + ((size_t)z * P.n + i) * P.n_hg + hg;
        if (tid == 0) {
            const int prev = atomicAdd(ticket, 1);
            s_last = (prev == nsplit - 1);
            if (prev == nsplit - 1) *ticket = 0;  // self-reset for the next launch
        }
        named_bar_sync(1, n_cons);
        if (s_last) {
            __threadfence();
            if (writer) {
                float Mx = -INFINITY;
                for (int cc = 0; cc < nsplit; cc++)
                    Mx = fmaxf(Mx, __ldcg(P.partials + (prow + (size_t)cc * P.H + h) * PSTRIDE));
                float L = 0.f, acc[OPL];
#pragma unroll
                for (int g = 0; g < OPL; g++) acc[g] = 0.f;
                for (int cc = 0; cc < nsplit; cc++) {
                    const float *pp = P.partials + (prow + (size_t)cc * P.H + h) * PSTRIDE;
                    const float w = exp2f(__ldcg(pp) - Mx);
                    L = fmaf(__ldcg(pp + 1), w, L);
#pragma unroll
                    for (int g = 0; g < OPL; g++) acc[g] = fmaf(__ldcg(pp + 2 + g * 16 + (DH >= 16 ? t : t % DH)), w, acc[g]);
                }
                const float inv = 1.f / fmaxf(L, 1e-12f);
#pragma unroll
                for (int g = 0; g < OPL; g++) P.out[row + (size_t)h * DH + g * 16 + (DH >= 16 ? t : t % DH)] = acc[g] * inv;
            }
        }
    }
    // Abort path only: before the CTA (and its shared memory) goes away, give the bulk copies that
    // were already issued a bounded chance to land.
    __syncthreads();
#ifdef JGPT_B200_DECODE_TRACE
    tr_c4 = clock64();
    timeline_at(P.timeline, 2);
    if (tid == 0 && P.trace) {
        long long gt1;
        unsigned smid;
        asm volatile("mov.u64 %0, %globaltimer;" : "=l"(gt1));
        asm volatile("mov.u32 %0, %smid;" : "=r"(smid));
        long long *tp = P.trace + (size_t)blockIdx.x * 8;
        tp[0] = tr_gt0, tp[1] = gt1, tp[2] = tr_c1 - tr_c0, tp[3] = tr_c2 - tr_c0, tp[4] = tr_c3 - tr_c0, tp[5] = tr_c4 - tr_c0, tp[6] = smid, tp[7] = 0;
    }
#endif
    if (*s_abort && tid == n_cons) {
        const uint32_t first = it > (uint32_t)NS ? it - NS : 0;
        for (uint32_t idx = first; idx < it; idx++)
            for (uint32_t spin = 0; spin < (1u << 16); spin++)
                if (mbar_try_wait(&full_bar[idx % NS], (idx / NS) & 1)) break;
    }
    // Dynamic mode: the last CTA to leave puts both counters back to zero for the next launch (by then every
    // CTA has drawn its sentinel, so nobody touches the item counter any more).
    if (P.dynamic && tid == 0) {
        __threadfence();
        if (atomicAdd(P.counters + 1, 1) == (int)gridDim.x - 1) {
            P.counters[0] = 0;
            P.counters[1] = 0;
            __threadfence();
        }
    }
}

// Raises a decode kernel's dynamic shared-memory limit to the largest request any launch makes, once per
// (kernel variant, device).  Guarded: contexts of different devices may launch from different host threads.
static cudaError_t decode_opt_in_smem(void (*kern)(const DecodeParams), int variant, int device) {
    static std::mutex mu;
    static bool done[16][64] = {};
    std::lock_guard<std::mutex> lock(mu);
    const bool tracked = variant >= 0 && variant < 16 && device >= 0 && device < 64;
    if (tracked && done[variant][device]) return cudaSuccess;
    const cudaError_t e = cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize, kMaxStages * 24 * 1024);
    if (e == cudaSuccess && tracked) done[variant][device] = true;
    return e;
}

// Largest divisor of H whose slab (HG * 64 * DH bytes) stays within 24 KiB and 480 consumer threads.
// A launch with few (layer, sequence) pairs - the model's per-layer decode step at small batch - takes the smallest
// group of at least 6 heads that still gives no more CTAs than fit at once (two per SM): more, lighter CTAs
// (measured on the decode step at batch 64: 0.638 ms with 24 heads per CTA, 0.613 ms with 6 or 8).
static int pick_head_group(int H, int DH, int forced, long long pairs = 0, long long slots = 0) {
    const int cap = std::min(30, std::max(1, 384 / DH));  // == max_head_group<DH>()
    if (forced > 0 && forced <= cap && H % forced == 0) return forced;
    int best = 1;
    for (int g = 1; g <= std::min(H, cap); g++)
        if (H % g == 0) best = g;
    if (pairs > 0 && slots > 0 && pairs * (H / best) < slots)
        for (int g = 6; g < best; g++)
            if (H % g == 0 && pairs * (H / g) <= slots) return g;
    return best;
}

template <int DH>
static int32_t launch_decode_t(Pool *p, const DecodeParams &P, bool fused, int threads, size_t smem, int grid) {
    // JGPT_B200_DECODE_MMA=1 selects the tensor-core consumer for dhead 16.  It is exact to the same tolerance but
    // measured 40 % slower on B200 (285 us against 203 us on the 12-layer batch-64 context-1024 step): per KV block
    // a warp runs two short dependent chains (ldmatrix, MMA, quad-strided shuffle reductions, exp2, hi/lo split of
    // p, MMA) on only 8 useful lanes, and the decode step is HBM-bound anyway.  The scalar consumer is the default.
    const bool want_mma = p->decode_mma != 0;  // read from the environment when the pool was created
    constexpr bool kCanMma = DH == 16;
    const bool mma = kCanMma && want_mma;
    void (*kern)(const DecodeParams) = fused ? attn_decode_kernel<DH, true, false> : attn_decode_kernel<DH, false, false>;
    if constexpr (kCanMma) {
        if (mma) kern = fused ? attn_decode_kernel<DH, true, true> : attn_decode_kernel<DH, false, true>;
    }
    // Opt in to > 48 KiB of dynamic shared memory once per kernel and device: the most a launch can ask for
    // (kMaxStages stages of a 24 KiB slab), so that no later, smaller request ever lowers the limit again.
    JGPT_CUDA_TRY(decode_opt_in_smem(kern, (fused ? 1 : 0) + (mma ? 2 : 0) + 4 * (DH == 4 ? 0 : DH == 8 ? 1 : DH == 16 ? 2 : 3),
                                     p->ctx->device));
    if (P.overlap || P.cluster) {
        cudaLaunchConfig_t cfg = {};
        cfg.gridDim = dim3((unsigned)grid), cfg.blockDim = dim3((unsigned)threads), cfg.dynamicSmemBytes = smem, cfg.stream = p->ctx->stream;
        cudaLaunchAttribute attr[2];
        int na = 0;
        if (P.overlap) {
            attr[na].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[na].val.programmaticStreamSerializationAllowed = 1;
            na++;
        }
        if (P.cluster) {
            attr[na].id = cudaLaunchAttributeClusterDimension;
            attr[na].val.clusterDim.x = (unsigned)P.max_chunks, attr[na].val.clusterDim.y = 1, attr[na].val.clusterDim.z = 1;
            na++;
        }
        cfg.attrs = attr, cfg.numAttrs = (unsigned)na;
        JGPT_CUDA_TRY(cudaLaunchKernelEx(&cfg, kern, P));
    } else {
        kern<<<grid, threads, smem, p->ctx->stream>>>(P);
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

#ifdef JGPT_B200_DECODE_TRACE
static long long *g_decode_trace = nullptr;
static int g_decode_trace_items = 0;
extern "C" __attribute__((visibility("default"))) int jgpt_debug_decode_trace(long long *host_out, int cap_items) {
    const int n = g_decode_trace_items < cap_items ? g_decode_trace_items : cap_items;
    cudaDeviceSynchronize();
    if (g_decode_trace && n > 0) cudaMemcpy(host_out, g_decode_trace, sizeof(long long) * 8 * 65536, cudaMemcpyDeviceToHost);
    return n;
}
#endif

// Clusters of `c` CTAs of the scalar dhead-16.. decode kernel (this block size and ring) that the device holds at once,
// as cudaOccupancyMaxActiveClusters reports it; cached per shape.  On B200 with 416 threads and a 72 KiB ring:
// 296 single CTAs, but 93 / 71 / 56 / 45 / 37 / 33 clusters of 3 / 4 / 5 / 6 / 7 / 8 (a cluster stays inside one GPC).
// 0 when the query fails (the caller then plans without clusters).
static int cluster_capacity(Pool *p, bool fused, int threads, size_t smem, int c) {
    static std::mutex mu;
    static std::map<std::tuple<int, int, int, size_t, int, int>, int> cache;
    const auto key = std::make_tuple(p->ctx->device, p->dhead, (int)fused, smem, threads, c);
    {
        std::lock_guard<std::mutex> lock(mu);
        auto it = cache.find(key);
        if (it != cache.end()) return it->second;
    }
    void (*kern)(const DecodeParams) = nullptr;
    int variant = -1;
    switch (p->dhead) {
        case 4: kern = fused ? attn_decode_kernel<4, true, false> : attn_decode_kernel<4, false, false>, variant = 0; break;
        case 8: kern = fused ? attn_decode_kernel<8, true, false> : attn_decode_kernel<8, false, false>, variant = 4; break;
        case 16: kern = fused ? attn_decode_kernel<16, true, false> : attn_decode_kernel<16, false, false>, variant = 8; break;
        case 32: kern = fused ? attn_decode_kernel<32, true, false> : attn_decode_kernel<32, false, false>, variant = 12; break;
        default: return 0;
    }
    int n = 0;
    if (decode_opt_in_smem(kern, variant + (fused ? 1 : 0), p->ctx->device) == cudaSuccess) {
        cudaLaunchConfig_t cfg = {};
        cudaLaunchAttribute attr[1];
        attr[0].id = cudaLaunchAttributeClusterDimension;
        attr[0].val.clusterDim.x = (unsigned)c, attr[0].val.clusterDim.y = 1, attr[0].val.clusterDim.z = 1;
        cfg.gridDim = dim3((unsigned)c * 64), cfg.blockDim = dim3((unsigned)threads), cfg.dynamicSmemBytes = smem;
        cfg.attrs = attr, cfg.numAttrs = 1;
        if (cudaOccupancyMaxActiveClusters(&n, kern, &cfg) != cudaSuccess) {
            (void)cudaGetLastError();
            n = 0;
        }
    }
    std::lock_guard<std::mutex> lock(mu);
    cache[key] = n;
    return n;
}

// Split-K chunk length of a launch with `base` (layer, sequence, head group) triples of up to max_blocks KV blocks.
// Two CTAs fit on an SM.  When the triples alone fill those slots the launch runs in several waves anyway and
// 32-block chunks keep the per-item set-up small.  Otherwise every sequence is cut into as many chunks as still
// fit in ONE wave (a few CTAs spilling into a second wave would double the launch time), at least 4 blocks each.
static int pick_chunk_blocks(const Pool *p, long long base, int max_blocks) {
    const long long slots = 2ll * p->ctx->sm_count;
    if (base >= slots) return 32;
    const long long nsplit = std::max(1ll, std::min(slots / base, (long long)(max_blocks + 3) / 4));
    const int cb = (int)((max_blocks + nsplit - 1) / nsplit);
    return std::min(32, std::max(4, cb));
}

int32_t launch_attn_decode(Pool *p, int layer0, int n_layers, const float *q, const float *k_new, const float *v_new,
                           const int *seq_ids, const int *rope_pos, const int *lens, int n, int max_len, float *out, int overlap) {
    DecodeParams P;
    memset(&P, 0, sizeof(P));
    const int DH = p->dhead;
    P.kv = p->kv, P.table = p->d_table, P.rope = p->d_rope;
    P.q = q, P.k_new = k_new, P.v_new = v_new, P.out = out;
    P.seq_ids = seq_ids, P.rope_pos = rope_pos, P.lens = lens;
    P.status = p->ctx->d_status;
    P.n = n, P.H = p->heads, P.layer0 = layer0, P.n_layers = n_layers, P.mbs = p->max_blocks_per_seq;
    P.n_blocks = p->n_blocks, P.max_seqs = p->max_seqs, P.max_positions = p->max_positions;
    const int ov = overlap >= 0 ? overlap : p->launch_overlap;
    // Head group and ring depth.  An overlapped single-layer launch (the per-layer decode loop) runs best with all
    // heads in one CTA (one 24 KiB slab per copy) and a three-stage ring, so that three CTAs fit on an SM and the next
    // launch's CTAs can move in beside the ones still draining: 20.7 us per layer at batch 64 / context 1024 against
    // 22.7 us for the ordinary launch (6-8 heads per CTA, four stages).
    const bool overlapped_single = ov >= 1 && n_layers == 1 && p->persistent <= 0;
    P.HG = overlapped_single ? pick_head_group(p->heads, DH, p->head_group)
                             : pick_head_group(p->heads, DH, p->head_group, (long long)n_layers * n, 2ll * p->ctx->sm_count);
    P.n_hg = p->heads / P.HG;
    const int max_blocks = std::min(p->max_blocks_per_seq, (max_len + kBlockTokens - 1) / kBlockTokens);
    // Work distribution.  Default (persistent <= 0): one CTA per work item, the hardware block scheduler hands
    // items to SMs as CTAs retire.  persistent = k > 0: k CTAs per SM claim items from a global counter (kept
    // for experiments: on B200 it measured 4-15 % slower than the plain grid at every chunk length).
    const int per_sm = p->persistent > 0 ? p->persistent : 2;
    const long long slots = (long long)per_sm * p->ctx->sm_count;
    const bool dynamic = p->persistent > 0;
    P.stages = p->stages > 0 ? p->stages : (overlapped_single ? 3 : 4);
    const int n_cons = ((kBlockTokens * P.HG + 31) / 32) * 32;
    const int threads = n_cons + 32;
    const size_t stage_bytes = (size_t)P.HG * 2 * kBlockTokens * DH * 2;
    const size_t smem = stage_bytes * P.stages;
    const bool may_cluster = p->cluster_merge && !dynamic && !p->decode_mma;
    if (p->chunk_blocks > 0) {
        P.chunk_blocks = p->chunk_blocks;
    } else if (overlapped_single && may_cluster) {
        // The per-layer launch of the model's decode step: the chunks of a sequence are one cluster, so the launch is one
        // wave only while the device holds `base` clusters of that size at once -- fewer CTAs than two per SM (see
        // cluster_capacity; clusters beyond it wait for a whole CTA time).  Most chunks of at least 4 blocks that stay
        // 1/16 under that number (a launch at the exact limit measured slower than the next smaller cluster).  JGPT-35M
        // step, ms per step before / after: 40 rows 0.591 / 0.509, 48 rows 0.614 / 0.512, 96 rows 0.775 / 0.672;
        // up to 29 rows ten chunks merged through global scratch became eight in a cluster (16 rows: 0.430 / 0.413).
        const long long base = (long long)n * P.n_hg;
        int c = 1;
        for (int t = std::min(8, (max_blocks + 3) / 4); t >= 2; t--)
            if (16 * base <= 15ll * cluster_capacity(p, k_new != nullptr, threads, smem, t)) {
                c = t;
                break;
            }
        const int c_min = (max_blocks + 31) / 32;  // a chunk holds at most 32 blocks
        if (c == 1 && (c_min > 1 || base > 2ll * p->ctx->sm_count)) {
            // No split fits one wave: take the one with the least rounds x (chunk length + ~6 blocks' worth of per-CTA
            // start-up and merge).  160 rows of 40 blocks: 3 chunks in 2 rounds (0.925 ms per step) against 2 chunks in
            // 2 rounds (0.985); 224 rows: 2 chunks in 2 rounds (1.217) against 3 chunks in 3 (1.264).
            long long best_cost = -1;
            for (int t = c_min; t <= std::min(8, (max_blocks + 3) / 4); t++) {
                const long long cap = t == 1 ? 2ll * p->ctx->sm_count : (long long)cluster_capacity(p, k_new != nullptr, threads, smem, t);
                if (cap <= 0) continue;
                // (clusters of three and more: a round counts as full at 15/16 of the capacity, like the one-wave rule above --
                // 186 rows are two rounds of 93 three-CTA clusters on paper and measured 0.98 ms against 0.92 ms with pairs)
                const long long full = t >= 3 ? 15 * cap : 16 * cap;
                const long long rounds = (16 * base + full - 1) / full, cost = rounds * ((max_blocks + t - 1) / t + 6);
                if (best_cost < 0 || cost < best_cost) best_cost = cost, c = t;
            }
        }
        c = std::max(c, c_min);
        P.chunk_blocks = std::min(32, std::max(4, (max_blocks + c - 1) / c));
    } else {
        P.chunk_blocks = pick_chunk_blocks(p, (long long)n_layers * n * P.n_hg, max_blocks);
    }
    P.max_len = max_blocks * kBlockTokens;
    P.max_chunks = std::max(1, (max_blocks + P.chunk_blocks - 1) / P.chunk_blocks);
    P.overlap = ov;
    P.stream_hint = p->stream_hint;
    P.scale_log2e = (1.0f / sqrtf((float)DH)) * 1.4426950408889634f;
    const long long items = (long long)n_layers * n * P.n_hg * P.max_chunks;
    JGPT_REQUIRE(items < (1ll << 31), JGPT_ERR_INVALID_ARGUMENT, "too many work items (%lld)", items);
    P.n_items = (int)items;
    // The chunks of one sequence as one thread-block cluster (up to the portable size of 8): merge in shared memory.
    // Not for the work queue (its CTAs take several items) nor for the tensor-core consumer (its own epilogue).
    // Only for launches of a wave or two: there the merge's global round trips are a visible part of the launch (per-layer
    // launch at batch 64 / context 1024: 24.1 -> 22.7 us).  A launch of many waves hides them behind other CTAs' copies,
    // and co-scheduling pairs of CTAs costs it more than it saves (12-layer launch: 198 us without, 202 us with).
    P.cluster = (may_cluster && P.max_chunks >= 2 && P.max_chunks <= 8 &&
                 items <= 4ll * p->ctx->sm_count) ? 1 : 0;
    if (P.max_chunks > 1 && !P.cluster) {
        int32_t rc = pool_ensure_split_scratch(p, (uint64_t)n_layers * n * P.max_chunks * p->heads * (DH + 2),
                                               (uint64_t)n_layers * n * P.n_hg);
        if (rc) return rc;
    }
    P.partials = p->d_partials, P.tickets = p->d_tickets;
#ifdef JGPT_B200_DECODE_TRACE
    {
        static long long *d_trace = nullptr;
        static int launch_no = 0;
        if (!d_trace) cudaMalloc(&d_trace, sizeof(long long) * 8 * 65536);
        // two halves used in turn: the last two launches can be compared (where did the second start / the first end)
        if (n_layers == 1) P.timeline = timeline_next();
        P.trace = P.n_items <= 32768 ? d_trace + (size_t)(launch_no & 1) * 8 * 32768 : nullptr;
        launch_no++;
        g_decode_trace = d_trace, g_decode_trace_items = P.n_items;
    }
#endif
    int grid = P.n_items;
    if (dynamic && (long long)P.n_items > slots) {
        grid = (int)slots;
        P.dynamic = 1;
        P.counters = p->d_item_counters;
    }
    if (P.dynamic && P.overlap > 1) P.overlap = 1;  // the work-queue counters are reset by the previous launch's last CTA
    const bool fused = k_new != nullptr;
    switch (DH) {
        case 4: return launch_decode_t<4>(p, P, fused, threads, smem, grid);
        case 8: return launch_decode_t<8>(p, P, fused, threads, smem, grid);
        case 16: return launch_decode_t<16>(p, P, fused, threads, smem, grid);
        case 32: return launch_decode_t<32>(p, P, fused, threads, smem, grid);
        default: return fail(JGPT_ERR_UNSUPPORTED, "dhead %d not supported", DH);
    }
}

}  // namespace jgpt

using namespace jgpt;

static int32_t decode_common(jgpt_kvpool h, int32_t layer0, int32_t n_layers, const float *q, const float *k, const float *v,
                             const int32_t *seq_ids, const int32_t *rope_pos, const int32_t *lens, int32_t n, int32_t max_len,
                             float *out, bool fused) {
    Pool *p = pool_registry().get(h);
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");
    JGPT_CUDA_TRY(make_current(p->ctx));
    JGPT_REQUIRE(n_layers >= 1 && layer0 >= 0 && layer0 + n_layers <= p->layers, JGPT_ERR_OUT_OF_RANGE,
                 "layers [%d, %d) outside [0,%d)", layer0, layer0 + n_layers, p->layers);
    if (n == 0) return JGPT_OK;
    JGPT_REQUIRE(n > 0 && q && seq_ids && rope_pos && lens && out && (!fused || (k && v)), JGPT_ERR_INVALID_ARGUMENT,
                 "null pointer or negative count");
    JGPT_REQUIRE(max_len >= 1, JGPT_ERR_INVALID_ARGUMENT, "max_len must be >= 1");
    return launch_attn_decode(p, layer0, n_layers, q, fused ? k : nullptr, fused ? v : nullptr, seq_ids, rope_pos, lens, n,
                              max_len, out);
}

extern "C" {

int32_t jgpt_attn_decode(jgpt_kvpool pool, int32_t layer0, int32_t n_layers, const float *q_dev, const int32_t *seq_ids_dev,
                         const int32_t *rope_pos_dev, const int32_t *lens_dev, int32_t n, int32_t max_len, float *out_dev) {
    return decode_common(pool, layer0, n_layers, q_dev, nullptr, nullptr, seq_ids_dev, rope_pos_dev, lens_dev, n, max_len,
                         out_dev, false);
}

int32_t jgpt_attn_decode_append(jgpt_kvpool pool, int32_t layer0, int32_t n_layers, const float *q_dev, const float *k_dev,
                                const float *v_dev, const int32_t *seq_ids_dev, const int32_t *rope_pos_dev,
                                const int32_t *lens_dev, int32_t n, int32_t max_len, float *out_dev) {
    return decode_common(pool, layer0, n_layers, q_dev, k_dev, v_dev, seq_ids_dev, rope_pos_dev, lens_dev, n, max_len,
                         out_dev, true);
}

int32_t jgpt_attn_decode_append_host(jgpt_kvpool pool, int32_t layer0, int32_t n_layers, const float *q_host,
                                     const float *k_host, const float *v_host, const int32_t *seq_ids_host,
                                     const int32_t *rope_pos_host, const int32_t *lens_host, int32_t n, float *out_host) {
    Pool *p = pool_registry().get(pool);
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");
    JGPT_CUDA_TRY(make_current(p->ctx));
    if (n == 0) return JGPT_OK;
    JGPT_REQUIRE(n > 0 && n_layers >= 1 && q_host && k_host && v_host && seq_ids_host && rope_pos_host && lens_host && out_host,
                 JGPT_ERR_INVALID_ARGUMENT, "null pointer or bad count");
    const size_t slab = (size_t)n_layers * n * p->heads * p->dhead;
    int32_t rc = pool_ensure_staging(p, 4 * slab, 3 * (size_t)n);
    if (rc) return rc;
    int max_len = 1;
    for (int i = 0; i < n; i++) {
        JGPT_REQUIRE(seq_ids_host[i] >= 0 && seq_ids_host[i] < p->max_seqs && p->seqs[(size_t)seq_ids_host[i]].used,
                     JGPT_ERR_OUT_OF_RANGE, "seq_ids[%d] = %d is not an allocated sequence", i, seq_ids_host[i]);
        JGPT_REQUIRE(lens_host[i] >= 1 && lens_host[i] <= (int)p->seqs[(size_t)seq_ids_host[i]].blocks.size() * kBlockTokens,
                     JGPT_ERR_ILLEGAL_STATE, "lens[%d] = %d is beyond the blocks reserved for sequence %d", i, lens_host[i],
                     seq_ids_host[i]);
        JGPT_REQUIRE(rope_pos_host[i] >= 0 && rope_pos_host[i] < p->max_positions, JGPT_ERR_INVALID_ARGUMENT,
                     "rope_pos[%d] = %d outside [0,%d)", i, rope_pos_host[i], p->max_positions);
        max_len = std::max(max_len, lens_host[i]);
    }
    cudaStream_t st = p->ctx->stream;
    float *dq = p->d_stage_f, *dk = dq + slab, *dv = dk + slab, *dout = dv + slab;
    int *dseq = p->d_stage_i, *drp = dseq + n, *dlen = drp + n;
    // Three ways to move the bytes.  STAGED: copies in and out around the kernel, pipelined over groups of layers
    // (works for any host memory).  ZEROCOPY (page-locked, device-mapped buffers): nothing is staged, the kernel
    // reads q / k / v and writes the result through the buffers' device addresses inside the one launch; fastest
    // when this process has the host fabric to itself (0.25 ms per 12-layer step against 0.30), slower when eight
    // processes do it at once (0.46 against 0.33: many small PCIe reads).  HYBRID: inputs by one copy each, the
    // result written in place.  Which one wins is a property of the machine at that moment, so the first calls
    // on a pool take turns (three samples each, same results whatever the way) and the fastest is kept;
    // JGPT_B200_HOST_ZEROCOPY = 0 / 1 / 2 pins STAGED / ZEROCOPY / HYBRID.
    enum { STAGED = 0, ZEROCOPY = 1, HYBRID = 2 };
    void *dp[4] = {};
    bool mapped = true;
    {
        const void *hp[4] = {q_host, k_host, v_host, out_host};
        for (int i = 0; i < 4 && mapped; i++) {
            cudaPointerAttributes a;
            if (cudaPointerGetAttributes(&a, hp[i]) != cudaSuccess) {
                cudaGetLastError();
                mapped = false;
            } else if (a.type != cudaMemoryTypeHost || !a.devicePointer) {
                mapped = false;
            } else {
                dp[i] = a.devicePointer;
            }
        }
    }
    int mode = STAGED;
    bool tuning = false;
    if (mapped) {
        const int pinned_mode = env_int("JGPT_B200_HOST_ZEROCOPY", -1);
        if (pinned_mode >= 0 && pinned_mode <= 2) {
            mode = pinned_mode;
        } else {
            if (p->host_tune_n != n || p->host_tune_layers != n_layers) {  // another shape: measure again
                p->host_tune_n = n, p->host_tune_layers = n_layers, p->host_tune_calls = 0, p->host_mode = -1;
                for (double &b : p->host_tune_best) b = 1e30;
            }
            // Which way wins is a property of the machine AT THAT MOMENT (other ranks load the same host fabric), so
            // the choice is kept under review: the first nine calls take turns (three samples each), and afterwards
            // two calls in every 128 go to the ways not in use; each way keeps a running average of what it cost.
            static const int order[3] = {ZEROCOPY, HYBRID, STAGED};
            const int c = p->host_tune_calls;
            if (c < 9) {
                mode = order[c % 3];
            } else {
                mode = p->host_mode;
                const int phase = (c - 9) % 128;
                if (phase == 126 || phase == 127) {
                    int others[2], k = 0;
                    for (int mth = 0; mth < 3; mth++)
                        if (mth != p->host_mode) others[k++] = mth;
                    mode = others[phase - 126];
                }
            }
            tuning = true;
        }
    }
    // The three index arrays travel as ONE copy out of the pool's page-locked staging area (three copies from
    // pageable memory cost ~15 us of driver staging per call; the previous call has synchronised, so the area is free).
    auto upload_indices = [&]() -> cudaError_t {
        memcpy(p->h_stage_i, seq_ids_host, sizeof(int) * (size_t)n);
        memcpy(p->h_stage_i + n, rope_pos_host, sizeof(int) * (size_t)n);
        memcpy(p->h_stage_i + 2 * (size_t)n, lens_host, sizeof(int) * (size_t)n);
        return cudaMemcpyAsync(dseq, p->h_stage_i, sizeof(int) * 3 * (size_t)n, cudaMemcpyHostToDevice, st);
    };
    const auto t_begin = std::chrono::steady_clock::now();
    auto finish = [&]() {
        if (!tuning) return;
        const double us = std::chrono::duration<double, std::micro>(std::chrono::steady_clock::now() - t_begin).count();
        double &avg = p->host_tune_best[mode];
        // first nine calls: the best of a way's three samples (the very first call of a way pays one-off set-up);
        // later: a running average that follows the machine's load
        if (p->host_tune_calls < 9) avg = std::min(avg, us);
        else avg = avg > 1e29 ? us : 0.75 * avg + 0.25 * us;
        p->host_tune_calls++;
        if (p->host_tune_calls >= 9) {
            int best = STAGED;
            for (int mth = 0; mth < 3; mth++)
                if (p->host_tune_best[mth] < p->host_tune_best[best]) best = mth;
            // change horses only for a clear gain: the samples are single wall-clock readings
            if (p->host_mode < 0 || p->host_tune_best[best] < 0.93 * p->host_tune_best[p->host_mode]) p->host_mode = best;
        }
    };
    if (mode == ZEROCOPY || mode == HYBRID) {
        JGPT_CUDA_TRY(upload_indices());
        const float *qi = static_cast<const float *>(dp[0]), *ki = static_cast<const float *>(dp[1]), *vi = static_cast<const float *>(dp[2]);
        if (mode == HYBRID) {
            JGPT_CUDA_TRY(cudaMemcpyAsync(dq, q_host, sizeof(float) * slab, cudaMemcpyHostToDevice, st));
            JGPT_CUDA_TRY(cudaMemcpyAsync(dk, k_host, sizeof(float) * slab, cudaMemcpyHostToDevice, st));
            JGPT_CUDA_TRY(cudaMemcpyAsync(dv, v_host, sizeof(float) * slab, cudaMemcpyHostToDevice, st));
            qi = dq, ki = dk, vi = dv;
        }
        rc = launch_attn_decode(p, layer0, n_layers, qi, ki, vi, dseq, drp, dlen, n, max_len, static_cast<float *>(dp[3]));
        if (rc) return rc;
        JGPT_CUDA_TRY(status_enqueue_read(p->ctx));
        JGPT_CUDA_TRY(cudaStreamSynchronize(st));
        finish();
        return status_check_after_sync(p->ctx, p, "jgpt_attn_decode_append_host");
    }
    JGPT_CUDA_TRY(upload_indices());
    // The layers of one call are independent, so the call is pipelined in groups of layers: while group g is
    // in the kernel, the inputs of group g+1 cross PCIe on the inbound copy engine and the outputs of group g-1
    // leave on the outbound one (three streams ordered by events).  One group = the plain path.
    constexpr int kMaxGroups = 4;  // events are allocated for up to four groups
    // Only the first group's inbound copy and the last group's outbound copy are exposed, but every launch costs
    // a fixed ~20 us.  Measured on the 12-layer step (us per step): one group 333, 4-4-4 301, 2-8-2 298,
    // 1-10-1 318, 1-5-5-1 325.  Default: a sixth of the layers first and last, the rest in between.
    // JGPT_B200_HOST_SPLIT = "a-b-c" (layers per group) overrides it, JGPT_B200_HOST_GROUPS = 1 selects the
    // unpipelined path.
    int sizes[kMaxGroups] = {n_layers, 0, 0, 0};
    int groups = 1;
    if (n_layers >= 3 && env_int("JGPT_B200_HOST_GROUPS", 3) > 1) {
        const int edge = std::max(1, n_layers / 6);
        groups = 3, sizes[0] = edge, sizes[1] = n_layers - 2 * edge, sizes[2] = edge;
    }
    if (const char *spec = getenv("JGPT_B200_HOST_SPLIT")) {
        int tmp[kMaxGroups] = {}, cnt = 0, sum = 0;
        for (const char *c = spec; *c && cnt < kMaxGroups;) {
            const int v = atoi(c);
            if (v <= 0) break;
            tmp[cnt++] = v, sum += v;
            while (*c && *c != '-') c++;
            if (*c == '-') c++;
        }
        if (cnt >= 1 && sum == n_layers) {
            groups = cnt;
            for (int g = 0; g < kMaxGroups; g++) sizes[g] = tmp[g];
        }
    }
    if (groups == 1) {
        JGPT_CUDA_TRY(cudaMemcpyAsync(dq, q_host, sizeof(float) * slab, cudaMemcpyHostToDevice, st));
        JGPT_CUDA_TRY(cudaMemcpyAsync(dk, k_host, sizeof(float) * slab, cudaMemcpyHostToDevice, st));
        JGPT_CUDA_TRY(cudaMemcpyAsync(dv, v_host, sizeof(float) * slab, cudaMemcpyHostToDevice, st));
        rc = launch_attn_decode(p, layer0, n_layers, dq, dk, dv, dseq, drp, dlen, n, max_len, dout);
        if (rc) return rc;
        JGPT_CUDA_TRY(cudaMemcpyAsync(out_host, dout, sizeof(float) * slab, cudaMemcpyDeviceToHost, st));
        JGPT_CUDA_TRY(status_enqueue_read(p->ctx));
        JGPT_CUDA_TRY(cudaStreamSynchronize(st));
        finish();
        return status_check_after_sync(p->ctx, p, "jgpt_attn_decode_append_host");
    }
    if (!p->s_in) {
        JGPT_CUDA_TRY(cudaStreamCreateWithFlags(&p->s_in, cudaStreamNonBlocking));
        JGPT_CUDA_TRY(cudaStreamCreateWithFlags(&p->s_out, cudaStreamNonBlocking));
        for (int g = 0; g < kMaxGroups; g++) {
            JGPT_CUDA_TRY(cudaEventCreateWithFlags(&p->ev_in[g], cudaEventDisableTiming));
            JGPT_CUDA_TRY(cudaEventCreateWithFlags(&p->ev_done[g], cudaEventDisableTiming));
        }
        JGPT_CUDA_TRY(cudaEventCreateWithFlags(&p->ev_start, cudaEventDisableTiming));
    }
    // the staging buffers may still be in use by earlier work on the main stream
    JGPT_CUDA_TRY(cudaEventRecord(p->ev_start, st));
    JGPT_CUDA_TRY(cudaStreamWaitEvent(p->s_in, p->ev_start, 0));
    const size_t per_layer = (size_t)n * p->heads * p->dhead;
    int l0 = 0;
    for (int g = 0; g < groups; g++) {
        const int nl = sizes[g];
        const size_t off = (size_t)l0 * per_layer, cnt = (size_t)nl * per_layer;
        JGPT_CUDA_TRY(cudaMemcpyAsync(dq + off, q_host + off, sizeof(float) * cnt, cudaMemcpyHostToDevice, p->s_in));
        JGPT_CUDA_TRY(cudaMemcpyAsync(dk + off, k_host + off, sizeof(float) * cnt, cudaMemcpyHostToDevice, p->s_in));
        JGPT_CUDA_TRY(cudaMemcpyAsync(dv + off, v_host + off, sizeof(float) * cnt, cudaMemcpyHostToDevice, p->s_in));
        JGPT_CUDA_TRY(cudaEventRecord(p->ev_in[g], p->s_in));
        JGPT_CUDA_TRY(cudaStreamWaitEvent(st, p->ev_in[g], 0));
        rc = launch_attn_decode(p, layer0 + l0, nl, dq + off, dk + off, dv + off, dseq, drp, dlen, n, max_len, dout + off);
        if (rc) return rc;
        JGPT_CUDA_TRY(cudaEventRecord(p->ev_done[g], st));
        JGPT_CUDA_TRY(cudaStreamWaitEvent(p->s_out, p->ev_done[g], 0));
        JGPT_CUDA_TRY(cudaMemcpyAsync(out_host + off, dout + off, sizeof(float) * cnt, cudaMemcpyDeviceToHost, p->s_out));
        l0 += nl;
    }
    JGPT_CUDA_TRY(status_enqueue_read(p->ctx));
    JGPT_CUDA_TRY(cudaStreamSynchronize(p->s_out));
    JGPT_CUDA_TRY(cudaStreamSynchronize(st));
    finish();
    return status_check_after_sync(p->ctx, p, "jgpt_attn_decode_append_host");
}

}  // extern "C"

// ------------------------------------------------------------------------------------------------
// Decode attention with its split-K scratch in a fixed, library-owned device array.
//
// jgpt_attn_decode sizes its split-K scratch (partial softmax states + arrival counters) with
// cudaMalloc the first time a launch needs more than it has.  Some hosts cannot tolerate that on the
// generation path: a process that has already handed the whole GPU to its own buffers (a trainer
// that samples text between optimizer steps with the device full, a server that sizes its KV pool to
// whatever memory is left) can see that late cudaMalloc fail, and any cudaMalloc/cudaFree stalls the
// device while it runs.  This variant never calls an allocator: its scratch is the array below.
//
// When the memory is taken: CUDA loads a module lazily, so the device memory of the array is
// reserved (and the kernel's code loaded) the first time this translation unit is used on a device --
// the set-up below -- not when the shared library is opened.  A call with n == 0 runs only that
// set-up, so a host can do it before it commits the rest of the GPU.  From then on every GPU that ran
// the set-up holds the array until the process exits.
//
// Limits, stated: kStaticPartialFloats fp32 partial words (4 MiB) and kStaticTickets counters
// (16 KiB) per device.  One layer per call.  Requests that need more are rejected.
// ------------------------------------------------------------------------------------------------
namespace jgpt {

constexpr size_t kStaticPartialFloats = size_t(1) << 20;  // 4 MiB of (m, l, o[dhead]) partials
constexpr size_t kStaticTickets = 4096;                   // arrival counters, one per (sequence row, head group)

// In host code this name is only a handle for cudaGetSymbolAddress, never an address to pass to a kernel.
static __device__ __align__(256) float g_decode_static_scratch[kStaticPartialFloats + kStaticTickets];

constexpr int kStaticMaxDevices = 64;
static float *g_static_scratch_addr[kStaticMaxDevices] = {};  // per device, resolved by the set-up
static std::mutex g_static_scratch_mu;                        // the table above and the opt-in below

// Once per device, with that device current: resolves the array's device address and loads the kernel
// (both trigger the lazy module load that reserves the array's memory).
static int32_t static_scratch_setup(const Pool *p, float **partials, int **tickets) {
    const Ctx *c = p->ctx;
    JGPT_REQUIRE(c->device >= 0 && c->device < kStaticMaxDevices, JGPT_ERR_UNSUPPORTED,
                 "device index %d is beyond the %d devices the static scratch table covers", c->device, kStaticMaxDevices);
    std::lock_guard<std::mutex> lock(g_static_scratch_mu);
    if (!g_static_scratch_addr[c->device]) {
        void *addr = nullptr;
        const cudaError_t e = cudaGetSymbolAddress(&addr, g_decode_static_scratch);
        if (e != cudaSuccess || !addr)
            return fail(e == cudaErrorMemoryAllocation ? JGPT_ERR_OUT_OF_MEMORY : JGPT_ERR_CUDA,
                        "cudaGetSymbolAddress(static decode scratch) on device %d: %s", c->device, cudaGetErrorString(e));
        cudaError_t a = cudaSuccess;
        switch (p->dhead) {
            case 4: a = decode_opt_in_smem(attn_decode_kernel<4, false, false>, 0, c->device); break;
            case 8: a = decode_opt_in_smem(attn_decode_kernel<8, false, false>, 4, c->device); break;
            case 16: a = decode_opt_in_smem(attn_decode_kernel<16, false, false>, 8, c->device); break;
            case 32: a = decode_opt_in_smem(attn_decode_kernel<32, false, false>, 12, c->device); break;
            default: break;
        }
        if (a != cudaSuccess) return fail(JGPT_ERR_CUDA, "static decode scratch set-up on device %d: %s", c->device, cudaGetErrorString(a));
        g_static_scratch_addr[c->device] = static_cast<float *>(addr);
    }
    *partials = g_static_scratch_addr[c->device];
    *tickets = reinterpret_cast<int *>(g_static_scratch_addr[c->device] + kStaticPartialFloats);
    return JGPT_OK;
}

static int32_t launch_attn_decode_static(Pool *p, int layer, const float *q, const int *seq_ids, const int *rope_pos,
                                         const int *lens, int n, int max_len, float *out) {
    DecodeParams P;
    memset(&P, 0, sizeof(P));
    const int DH = p->dhead;
    P.kv = p->kv, P.table = p->d_table, P.rope = p->d_rope;
    P.q = q, P.k_new = nullptr, P.v_new = nullptr, P.out = out;
    P.seq_ids = seq_ids, P.rope_pos = rope_pos, P.lens = lens;
    P.status = p->ctx->d_status;
    P.n = n, P.H = p->heads, P.layer0 = layer, P.n_layers = 1, P.mbs = p->max_blocks_per_seq;
    P.n_blocks = p->n_blocks, P.max_seqs = p->max_seqs, P.max_positions = p->max_positions;
    // same launch shape as jgpt_attn_decode gives a one-layer call (small batches get lighter CTAs)
    P.stream_hint = p->stream_hint;
    P.HG = pick_head_group(p->heads, DH, p->head_group, (long long)n, 2ll * p->ctx->sm_count);
    P.n_hg = p->heads / P.HG;
    const int max_blocks = std::min(p->max_blocks_per_seq, (max_len + kBlockTokens - 1) / kBlockTokens);
    P.chunk_blocks = p->chunk_blocks > 0 ? p->chunk_blocks : pick_chunk_blocks(p, (long long)n * P.n_hg, max_blocks);
    P.max_len = max_blocks * kBlockTokens;
    P.max_chunks = std::max(1, (max_blocks + P.chunk_blocks - 1) / P.chunk_blocks);
    P.stages = p->stages > 0 ? p->stages : 4;
    P.scale_log2e = (1.0f / sqrtf((float)DH)) * 1.4426950408889634f;
    const long long items = (long long)n * P.n_hg * P.max_chunks;
    JGPT_REQUIRE(items < (1ll << 31), JGPT_ERR_INVALID_ARGUMENT, "too many work items (%lld)", items);
    P.n_items = (int)items;
    int32_t rc = static_scratch_setup(p, &P.partials, &P.tickets);
    if (rc) return rc;
    if (P.max_chunks > 1) {
        // Only a split sequence touches the scratch; an unsplit launch needs none of it and has no size limit.
        const unsigned long long need_partials = (unsigned long long)n * P.max_chunks * p->heads * (DH + 2);
        const unsigned long long need_tickets = (unsigned long long)n * P.n_hg;
        JGPT_REQUIRE(need_partials <= kStaticPartialFloats && need_tickets <= kStaticTickets, JGPT_ERR_INVALID_ARGUMENT,
                     "request needs %llu partial words and %llu counters; the static scratch holds %llu and %llu "
                     "(lower n or max_len, or use jgpt_attn_decode)",
                     need_partials, need_tickets, (unsigned long long)kStaticPartialFloats,
                     (unsigned long long)kStaticTickets);
        // The array keeps whatever the previous call left.  Partials are always written before they are read;
        // the counters must start at zero (they reset themselves, but not if an earlier launch gave up half way).
        JGPT_CUDA_TRY(cudaMemsetAsync(P.tickets, 0, sizeof(int) * need_tickets, p->ctx->stream));
    }
    const int n_cons = ((kBlockTokens * P.HG + 31) / 32) * 32;
    const int threads = n_cons + 32;
    const size_t smem = (size_t)P.HG * 2 * kBlockTokens * DH * 2 * P.stages;
    void (*kern)(const DecodeParams) = nullptr;
    switch (DH) {
        case 4: kern = attn_decode_kernel<4, false, false>; break;
        case 8: kern = attn_decode_kernel<8, false, false>; break;
        case 16: kern = attn_decode_kernel<16, false, false>; break;
        case 32: kern = attn_decode_kernel<32, false, false>; break;
        default: return fail(JGPT_ERR_UNSUPPORTED, "dhead %d not supported", DH);
    }
    kern<<<P.n_items, threads, smem, p->ctx->stream>>>(P);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

}  // namespace jgpt

extern "C" int32_t jgpt_attn_decode_static_scratch(jgpt_kvpool pool, int32_t layer, const float *q_dev,
                                                   const int32_t *seq_ids_dev, const int32_t *rope_pos_dev,
                                                   const int32_t *lens_dev, int32_t n, int32_t max_len, float *out_dev) {
    Pool *p = pool_registry().get(pool);
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");
    JGPT_CUDA_TRY(make_current(p->ctx));
    JGPT_REQUIRE(layer >= 0 && layer < p->layers, JGPT_ERR_OUT_OF_RANGE, "layer %d outside [0,%d)", layer, p->layers);
    JGPT_REQUIRE(p->dhead == 4 || p->dhead == 8 || p->dhead == 16 || p->dhead == 32, JGPT_ERR_UNSUPPORTED,
                 "dhead %d not supported", p->dhead);
    if (n == 0) {  // set-up only: take the array's memory and load the kernel now, launch nothing
        float *partials;
        int *tickets;
        return static_scratch_setup(p, &partials, &tickets);
    }
    JGPT_REQUIRE(n > 0 && q_dev && seq_ids_dev && rope_pos_dev && lens_dev && out_dev, JGPT_ERR_INVALID_ARGUMENT,
                 "null pointer or negative count");
    JGPT_REQUIRE(max_len >= 1, JGPT_ERR_INVALID_ARGUMENT, "max_len must be >= 1");
    return launch_attn_decode_static(p, layer, q_dev, seq_ids_dev, rope_pos_dev, lens_dev, n, max_len, out_dev);
}
