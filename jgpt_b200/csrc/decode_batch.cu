// One decode step of a BATCH (5 rows and up) as one cooperative launch.
//
// The multi-launch step (model.cu: 63 kernels of 5-20 us replayed as a graph) spends most of its time in the hand-over
// between dependent kernels.  Here one grid of one CTA per SM walks the layer chain; results travel between the phases
// as (value, stamp) pairs (exchange.cuh), so there is no grid-wide barrier and a row tile moves on as soon as ITS
// inputs are complete - different row tiles can be in different phases.
//
//   per layer   A  RMSNorm + Q,K,V          tiles of 16 rows x 32 columns, split-TF32 mma.sync (fp32-level accuracy),
//               B  append + attention       one WARP per (row, head, chunk of the sequence): a lane pair owns a token,
//                                           lane t its K row, lane 16 + t its V row (one KV block of a head is 1 KiB
//                                           contiguous: a warp reads it with one 32-byte load per lane), private
//                                           online softmax, 16-lane shuffle merge; chunks of a (row, head) meet through
//                                           a ticket (last arriver merges, as in attn_decode.cu)
//               C  Wo + residual            tiles; epilogue leaves the row sums of squares of its 32 columns
//               D  RMSNorm + W1,W3 + SwiGLU tiles over the interleaved W1/W3 image
//               E  W2 + residual            tiles
//   then the LM head (tiles; every tile leaves its best logit per row) and the argmax over the tiles.
//
// A tile's weights stream through a cp.async ring that is started BEFORE the tile waits for its activations; the 16 x K
// slab of activations is read once (polling the stamps) into shared memory.  Arithmetic as the multi-launch step: the same
// tile shape, k order and reduction order as gemm_tc_small_kernel, so logits agree to rounding noise.
//
// Every wait is bounded (exchange.cuh); the launch is cooperative because CTAs wait for one another's data.
#include "common.cuh"
#include "exchange.cuh"
#include "ptx.cuh"

#include <algorithm>
#include <cmath>
#include <mutex>
#include <unordered_set>

namespace jgpt {
namespace {

constexpr int kThreads = 256;
constexpr int kWarps = 8;
constexpr int DH = 16, PS = DH + 2;
constexpr int BM = 16, BN = 32, BK = 64, STAGES = 4, WS = BN + 8;
constexpr int kSlabBatch = 12;  // 16-byte reads of the activation slab a thread keeps in flight
constexpr int kAttnGroup = 8;  // KV blocks (1 KiB each) a warp requests before it consumes them: 8 warps x 8 KiB in flight per SM

// Leaving early (a wait gave up): nothing may still be copying into this CTA's shared memory.
#define BATCH_BAIL()                                        \
    do {                                                    \
        asm volatile("cp.async.wait_all;" ::: "memory");    \
        return;                                             \
    } while (0)

#ifdef JGPT_B200_DECODE_TRACE
// Timing build only: per CTA, the global timer (ns) at the phase boundaries of the second layer and of the LM head.
constexpr int kBatchMarks = 24;
__device__ long long g_batch_trace[256 * kBatchMarks];
__device__ __forceinline__ long long global_ns() {
    long long t;
    asm volatile("mov.u64 %0, %globaltimer;" : "=l"(t));
    return t;
}
#define BATCH_MARK(cond, i)                                                                             \
    do {                                                                                                \
        if ((cond) && threadIdx.x == 0) g_batch_trace[blockIdx.x * kBatchMarks + (i)] = global_ns();    \
    } while (0)
#else
#define BATCH_MARK(cond, i) \
    do {                    \
    } while (0)
#endif

struct Shared {
    float *As;                       // [BM][lda]
    int lda;
    float (*Ws)[BK][WS];             // [STAGES]
    float (*red)[BM][BN + 1];        // [kWarps], aliases Ws once the k loop is over
    float *s_inv;                    // [BM]
    float *Sg;                       // [kmax] norm weights of the running tile
};

// ---- weights: one k tile (64 x 32) per cp.async group ----
__device__ __forceinline__ void w_tile_issue(const Shared &S, int buf, const float *W, int ldw, int n0, int k0, int K) {
    const int tid = threadIdx.x, w_k = tid >> 3, w_c = (tid & 7) * 4;
    const bool col_ok = n0 + w_c < ldw;
    const float *src = W + (size_t)(k0 + w_k) * ldw + (col_ok ? n0 + w_c : 0);
    const bool k1 = col_ok && k0 + w_k < K, k2 = col_ok && k0 + w_k + 32 < K;
    cp_async16(&S.Ws[buf][w_k][w_c], k1 ? src : W, k1);
    cp_async16(&S.Ws[buf][w_k + 32][w_c], k2 ? src + (size_t)32 * ldw : W, k2);
    asm volatile("cp.async.commit_group;" ::: "memory");
}
__device__ __forceinline__ void w_prefetch(const Shared &S, const float *W, int ldw, int n0, int K, const float *gamma = nullptr) {
    const int nk = (K + BK - 1) / BK;
    if (gamma)  // rides in the first group
        for (int c = threadIdx.x * 4; c < K; c += kThreads * 4) cp_async16(S.Sg + c, gamma + c, true);
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < nk) w_tile_issue(S, s, W, ldw, n0, s * BK, K);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
}

// ---- activations: rows m0 .. m0+16 of a stamped [M][K] array into As; rows >= M are zero ----
__device__ __forceinline__ void slab_load(const Shared &S, const uint2 *src, int K, int m0, int M, unsigned stamp, Poll &pl) {
    const int per_row = K / 2, items = BM * per_row;  // one item = two adjacent values
    for (int base = threadIdx.x; base < items; base += kThreads * kSlabBatch) {
        uint4 v[kSlabBatch];
        int cnt = 0;
#pragma unroll
        for (int j = 0; j < kSlabBatch; j++)
            if (base + j * kThreads < items) cnt = j + 1;
        ll_load<kSlabBatch>(v, cnt, stamp, pl, [&](int j) {
            const int it = base + j * kThreads, r = it / per_row, c2 = it % per_row;
            const int m = min(m0 + r, M - 1);  // rows beyond M re-read the last row (their products are never stored)
            return src + (size_t)m * K + 2 * c2;
        });
#pragma unroll
        for (int j = 0; j < kSlabBatch; j++)
            if (j < cnt) {
                const int it = base + j * kThreads, r = it / per_row, c2 = it % per_row;
                *reinterpret_cast<float2 *>(S.As + r * S.lda + 2 * c2) = make_float2(__uint_as_float(v[j].x), __uint_as_float(v[j].z));
            }
    }
}
// 1 / rms of the slab's rows from the partial sums of squares their producer left (added in ascending order)
__device__ __forceinline__ void inv_rms_load(const Shared &S, const uint2 *ss, int parts, int K, float eps, int m0, int M, unsigned stamp,
                                             Poll &pl) {
    if (threadIdx.x < BM) {
        const int m = min(m0 + (int)threadIdx.x, M - 1);
        float tot = 0.f;
        for (int p0 = 0; p0 < parts; p0 += 16) {
            uint4 v[8];
            const int cnt = min(8, (parts - p0 + 1) / 2);
            ll_load<8>(v, cnt, stamp, pl, [&](int j) { return ss + (size_t)m * parts + p0 + 2 * j; });
#pragma unroll
            for (int j = 0; j < 8; j++)
                if (j < cnt) {
                    tot += __uint_as_float(v[j].x);
                    if (p0 + 2 * j + 1 < parts) tot += __uint_as_float(v[j].z);
                }
        }
        const float rms = sqrtf(tot / (float)K + eps);
        S.s_inv[threadIdx.x] = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
    }
}

// ---- the k loop: As (resident slab) x W (ring) -> eight partial tiles in S.red ----
template <bool NORM>
__device__ __forceinline__ void tile_mma(const Shared &S, const float *W, int ldw, int n0, int K) {
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    float acc[4][4], cor[4][4];
#pragma unroll
    for (int j = 0; j < 4; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) acc[j][e] = 0.f, cor[j][e] = 0.f;
    const int nk = (K + BK - 1) / BK, ks = warp * 8;
    for (int kt = 0; kt < nk; kt++) {
        const int buf = kt % STAGES;
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();  // tile kt visible to all; everyone is done with the buffer refilled below
        if (kt + STAGES - 1 < nk) w_tile_issue(S, (kt + STAGES - 1) % STAGES, W, ldw, n0, (kt + STAGES - 1) * BK, K);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        const int k = kt * BK + ks + t;
        float a0 = k < K ? S.As[g * S.lda + k] : 0.f, a1 = k < K ? S.As[(g + 8) * S.lda + k] : 0.f;
        float a2 = k + 4 < K ? S.As[g * S.lda + k + 4] : 0.f, a3 = k + 4 < K ? S.As[(g + 8) * S.lda + k + 4] : 0.f;
        if (NORM) {
            const float g0 = k < K ? S.Sg[k] : 0.f, g1 = k + 4 < K ? S.Sg[k + 4] : 0.f;
            const float ia = S.s_inv[g], ib = S.s_inv[g + 8];
            a0 = a0 * ia * g0, a1 = a1 * ib * g0, a2 = a2 * ia * g1, a3 = a3 * ib * g1;
        }
        uint32_t ah[4], al[4];
        split_tf32(a0, ah[0], al[0]);
        split_tf32(a1, ah[1], al[1]);
        split_tf32(a2, ah[2], al[2]);
        split_tf32(a3, ah[3], al[3]);
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = j * 8 + g;
            uint32_t bh0, bl0, bh1, bl1;
            split_tf32(S.Ws[buf][ks + t][c], bh0, bl0);
            split_tf32(S.Ws[buf][ks + t + 4][c], bh1, bl1);
            mma_tf32(cor[j], al, bh0, bh1);
            mma_tf32(acc[j], ah, bh0, bh1);
            mma_tf32(cor[j], ah, bl0, bl1);
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the ring is dead: its memory takes the eight partial tiles
#pragma unroll
    for (int j = 0; j < 4; j++) {
        S.red[warp][g][j * 8 + 2 * t] = acc[j][0] + cor[j][0];
        S.red[warp][g][j * 8 + 2 * t + 1] = acc[j][1] + cor[j][1];
        S.red[warp][g + 8][j * 8 + 2 * t] = acc[j][2] + cor[j][2];
        S.red[warp][g + 8][j * 8 + 2 * t + 1] = acc[j][3] + cor[j][3];
    }
    __syncthreads();
}
__device__ __forceinline__ float red_sum(const Shared &S, int r, int c) {
    float v = S.red[0][r][c];
#pragma unroll
    for (int w = 1; w < kWarps; w++) v += S.red[w][r][c];
    return v;
}

// ---- one warp: (row, head, chunk) of the attention ----
__device__ __forceinline__ void attention_warp(const BatchStepArgs &A, int layer, int row, int h, int c, unsigned stamp, Poll &pl, bool tr = false) {
    const int lane = threadIdx.x & 31, t = lane & 15;
    const bool vlane = lane >= 16;
    const int n = A.n;
    const int seq = A.idx[2 * n + row], rp = A.idx[3 * n + row], len = A.idx[4 * n + row];
    const int nbk = (len + 15) >> 4, nch = (nbk + A.cb - 1) / A.cb;
    if (c >= nch) return;
    const int b0 = c * A.cb, b1 = min(nbk, b0 + A.cb);
    const bool owner = c == nch - 1;  // the chunk that holds slot len - 1
    BATCH_MARK(tr, 16);
    // block table entries of the chunk (cb <= 32) and the RoPE row: neither depends on this step's activations
    const int my_phys = (b0 + lane < b1) ? __ldcg(A.table + (size_t)seq * A.mbs + b0 + lane) : -1;
    float2 rope[DH / 2];
#pragma unroll
    for (int j = 0; j < DH / 2; j++) rope[j] = __ldg(A.rope + (size_t)rp * (DH / 2) + j);
    // q (lanes 0-7), and for the owner k (8-15) and v (16-23) of the new token: two values per lane
    float in0 = 0.f, in1 = 0.f;
    if (lane < (owner ? 24 : 8)) {
        uint4 v[1];
        const uint2 *src = A.qkv + (size_t)row * 3 * A.D + (size_t)(lane >> 3) * A.D + h * DH + 2 * (lane & 7);
        ll_load<1>(v, 1, stamp, pl, [&](int) { return src; });
        in0 = __uint_as_float(v[0].x), in1 = __uint_as_float(v[0].z);
    }
    BATCH_MARK(tr, 17);
    float q[DH];
#pragma unroll
    for (int j = 0; j < DH / 2; j++) {
        const float x0 = __shfl_sync(0xffffffffu, in0, j), x1 = __shfl_sync(0xffffffffu, in1, j);
        q[2 * j] = __fsub_rn(__fmul_rn(x0, rope[j].x), __fmul_rn(x1, rope[j].y)) * A.scale_log2e;
        q[2 * j + 1] = __fadd_rn(__fmul_rn(x0, rope[j].y), __fmul_rn(x1, rope[j].x)) * A.scale_log2e;
    }
    // this lane's row of the new token, as the store will hold it: lanes < 16 the RoPE'd k, lanes >= 16 the raw v
    __align__(16) __half newrow[DH];
    if (owner) {
#pragma unroll
        for (int j = 0; j < DH / 2; j++) {
            const float k0 = __shfl_sync(0xffffffffu, in0, 8 + j), k1 = __shfl_sync(0xffffffffu, in1, 8 + j);
            const float v0 = __shfl_sync(0xffffffffu, in0, 16 + j), v1 = __shfl_sync(0xffffffffu, in1, 16 + j);
            newrow[2 * j] = __float2half_rn(vlane ? v0 : __fsub_rn(__fmul_rn(k0, rope[j].x), __fmul_rn(k1, rope[j].y)));
            newrow[2 * j + 1] = __float2half_rn(vlane ? v1 : __fadd_rn(__fmul_rn(k0, rope[j].y), __fmul_rn(k1, rope[j].x)));
        }
    }
    float m = -INFINITY, l = 0.f, o[DH];
#pragma unroll
    for (int d = 0; d < DH; d++) o[d] = 0.f;
    const size_t layer_base = (size_t)layer * A.n_blocks;
    constexpr int U = kAttnGroup;  // KV blocks in flight per warp
    for (int bb = b0; bb < b1; bb += U) {
        __align__(16) __half rowv[U][DH];
        bool live[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const int blk = bb + u;
            const int phys = __shfl_sync(0xffffffffu, my_phys, (blk - b0) & 31);
            const int tok = blk * 16 + t;
            live[u] = blk < b1 && tok < len;
            if (blk < b1 && (phys < 0 || phys >= A.n_blocks)) {
                if (lane == 0) atomicOr(A.status, DEV_STATUS_BAD_BLOCK);
                live[u] = false;
            }
            if (live[u]) {
                __half *p = A.kv + ((layer_base + phys) * A.H + h) * (size_t)(2 * 16 * DH) + (size_t)lane * DH;
                if (tok == len - 1) {  // the appended token: stored, and used from registers
                    reinterpret_cast<uint4 *>(p)[0] = reinterpret_cast<const uint4 *>(newrow)[0];
                    reinterpret_cast<uint4 *>(p)[1] = reinterpret_cast<const uint4 *>(newrow)[1];
                    reinterpret_cast<uint4 *>(rowv[u])[0] = reinterpret_cast<const uint4 *>(newrow)[0];
                    reinterpret_cast<uint4 *>(rowv[u])[1] = reinterpret_cast<const uint4 *>(newrow)[1];
                } else {
                    reinterpret_cast<uint4 *>(rowv[u])[0] = __ldcg(reinterpret_cast<const uint4 *>(p));
                    reinterpret_cast<uint4 *>(rowv[u])[1] = __ldcg(reinterpret_cast<const uint4 *>(p) + 1);
                }
            }
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (bb + u >= b1) break;  // uniform over the warp
            float sc = 0.f;
            if (!vlane) {
#pragma unroll
                for (int d = 0; d < DH; d++) sc = fmaf(q[d], __half2float(rowv[u][d]), sc);
            }
            sc = __shfl_sync(0xffffffffu, sc, t);  // the K lane's score to its V lane
            if (live[u]) {  // live is the same for a K lane and its V lane
                if (sc > m) {
                    const float corr = fast_exp2(m - sc);
                    l *= corr;
                    if (vlane) {
#pragma unroll
                        for (int d = 0; d < DH; d++) o[d] *= corr;
                    }
                    m = sc;
                }
                const float pe = fast_exp2(sc - m);
                l += pe;
                if (vlane) {
#pragma unroll
                    for (int d = 0; d < DH; d++) o[d] = fmaf(pe, __half2float(rowv[u][d]), o[d]);
                }
            }
        }
    }
    // merge the 16 token lanes (both halves of the warp hold the same m and l)
    BATCH_MARK(tr, 18);
    float M = m;
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
    l *= f;
#pragma unroll
    for (int off = 8; off >= 1; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
#pragma unroll
    for (int d = 0; d < DH; d++) o[d] *= f;
#pragma unroll
    for (int width = DH / 2, off = 8; width >= 1; width >>= 1, off >>= 1) {  // lane 16 + j ends with dimension j
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < DH / 2; j++)
            if (j < width) {
                const float mine = upper ? o[j + width] : o[j], theirs = upper ? o[j] : o[j + width];
                o[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, off);
            }
    }
    uint2 *out = A.att + (size_t)row * A.D + h * DH;
    BATCH_MARK(tr, 19);
    if (nch == 1) {
        if (vlane) st_pair(out + t, o[0] / fmaxf(l, 1e-12f), stamp);
        return;
    }
    // The chunk's partial goes out as stamped pairs, so no fence is needed: a ticket (relaxed) only elects the warp that
    // merges; that warp reads every chunk's pairs until they carry the stamp.
    uint2 *pp = A.part + (((size_t)row * A.H + h) * A.nch_max + c) * PS;
    if (lane == 0) st_pair(pp, M, stamp), st_pair(pp + 1, l, stamp);
    if (vlane) st_pair(pp + 2 + t, o[0], stamp);
    int ticket = 0;
    if (lane == 0) ticket = atomicAdd(A.tickets + (size_t)row * A.H + h, 1);
    ticket = __shfl_sync(0xffffffffu, ticket, 0);
    BATCH_MARK(tr, 20);
    if (ticket != nch - 1) return;
    if (lane == 0) A.tickets[(size_t)row * A.H + h] = 0;  // for the next layer
    // lane L merges chunk L's 18 values (nch <= 32): one wait for all of them, then warp reductions
    const uint2 *p0 = A.part + (((size_t)row * A.H + h) * A.nch_max + min(lane, nch - 1)) * PS;
    uint4 v[PS / 2];
    ll_load<PS / 2>(v, PS / 2, stamp, pl, [&](int i) { return p0 + 2 * i; });
    const bool mine = lane < nch;
    const float mc = mine ? __uint_as_float(v[0].x) : -INFINITY;
    float Mx = mc;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) Mx = fmaxf(Mx, __shfl_xor_sync(0xffffffffu, Mx, off));
    const float w = (mine && mc != -INFINITY) ? exp2f(mc - Mx) : 0.f;
    float L = __uint_as_float(v[0].z) * w;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) L += __shfl_xor_sync(0xffffffffu, L, off);
    float od[DH];
#pragma unroll
    for (int i = 1; i < PS / 2; i++) od[2 * i - 2] = __uint_as_float(v[i].x) * w, od[2 * i - 1] = __uint_as_float(v[i].z) * w;
#pragma unroll
    for (int width = DH / 2, off = 16; width >= 1; width >>= 1, off >>= 1) {  // lane L ends with dimension L >> 1
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int i = 0; i < DH / 2; i++)
            if (i < width) {
                const float keep = upper ? od[i + width] : od[i], give = upper ? od[i] : od[i + width];
                od[i] = keep + __shfl_xor_sync(0xffffffffu, give, off);
            }
    }
    od[0] += __shfl_xor_sync(0xffffffffu, od[0], 1);
    if ((lane & 1) == 0) st_pair(out + (lane >> 1), od[0] / fmaxf(L, 1e-12f), stamp);
}

__global__ void __launch_bounds__(kThreads, 1) decode_batch_kernel(const BatchStepArgs A) {
    extern __shared__ __align__(16) float sm[];
    __shared__ float s_inv[BM];
    Shared S;
    S.lda = A.kmax + 4;
    S.As = sm;
    S.Ws = reinterpret_cast<float (*)[BK][WS]>(sm + BM * S.lda);
    S.red = reinterpret_cast<float (*)[BM][BN + 1]>(sm + BM * S.lda);
    S.Sg = sm + BM * S.lda + STAGES * BK * WS;
    S.s_inv = s_inv;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x, G = gridDim.x, n = A.n, D = A.D, F = A.F, V = A.vocab;
    const int mt_n = (n + BM - 1) / BM, parts = (D + 31) / 32;
    Poll pl{A.abort_word, A.stamp0 + 1u, A.status, 0};
    // epilogue mapping: thread = (row of the tile, two adjacent columns)
    const int er = tid >> 4, ec = (tid & 15) * 2;

    // ---- embedding + position rows, with their sums of squares (one partial, the others zero) ----
    const unsigned s_emb = A.stamp0 + 1u;
    for (int r = b; r < n; r += G) {
        const int id = A.idx[r], pr = A.idx[n + r];
        float ss = 0.f;
        for (int j = tid; j < D; j += kThreads) {
            const float v = __ldg(A.tok + (size_t)id * D + j) + __ldg(A.pos + (size_t)pr * D + j);
            st_pair(A.xa + (size_t)r * D + j, v, s_emb);
            ss = fmaf(v, v, ss);
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if (lane == 0) S.As[warp] = ss;
        __syncthreads();
        if (tid < parts) {
            float tot = 0.f;
            if (tid == 0)
                for (int w = 0; w < kWarps; w++) tot += S.As[w];
            st_pair(A.ssa + (size_t)r * parts + tid, tot, s_emb);
        }
        __syncthreads();
    }

    for (int l = 0; l < A.layers; l++) {
        const unsigned s_in = A.stamp0 + 1u + (unsigned)l, st = s_in + 1u;  // the layer's input x, what the layer writes
        const LayerW &Y = A.Lw[l];
        // ---- A: RMSNorm + Q,K,V  ->  qkv [n][3D]
        {
            const int nt_n = D / BN;  // column tiles per matrix
            for (int u = b; u < mt_n * 3 * nt_n; u += G) {
                const int mt = u / (3 * nt_n), zt = u % (3 * nt_n), z = zt / nt_n, n0 = (zt % nt_n) * BN, m0 = mt * BM;
                const float *W = z == 0 ? Y.wq : (z == 1 ? Y.wk : Y.wv);
                BATCH_MARK(l == 1 && u == b, 0);
                w_prefetch(S, W, D, n0, D, Y.norm1);
                slab_load(S, A.xa, D, m0, n, s_in, pl);
                inv_rms_load(S, A.ssa, parts, D, A.eps, m0, n, s_in, pl);
                if (__syncthreads_or(pl.failed)) BATCH_BAIL();
                BATCH_MARK(l == 1 && u == b, 1);
                tile_mma<true>(S, W, D, n0, D);
                const int m = m0 + er;
                if (m < n) {
                    uint2 *dst = A.qkv + (size_t)m * 3 * D + (size_t)z * D + n0 + ec;
                    st_pair(dst, red_sum(S, er, ec), st);
                    st_pair(dst + 1, red_sum(S, er, ec + 1), st);
                }
                __syncthreads();
                BATCH_MARK(l == 1 && u == b, 2);
            }
        }
        // ---- B: append + attention  ->  att [n][D]
        {
            const int units = n * A.nch_max * A.H;
            BATCH_MARK(l == 1, 3);
            for (int u = b * kWarps + warp; u < units; u += G * kWarps) {
                const int h = u % A.H, c = (u / A.H) % A.nch_max, row = u / (A.H * A.nch_max);
#ifdef JGPT_B200_DECODE_TRACE
                attention_warp(A, l, row, h, c, st, pl, l == 1 && u == b * kWarps && threadIdx.x == 0);
#else
                attention_warp(A, l, row, h, c, st, pl);
#endif
            }
            BATCH_MARK(l == 1, 4);
            if (__syncthreads_or(pl.failed)) BATCH_BAIL();
        }
        // ---- C: Wo + residual  ->  xb [n][D], ssb
        {
            const int nt_n = D / BN;
            for (int u = b; u < mt_n * nt_n; u += G) {
                const int mt = u / nt_n, n0 = (u % nt_n) * BN, m0 = mt * BM, m = m0 + er;
                BATCH_MARK(l == 1 && u == b, 6);
                w_prefetch(S, Y.wo, D, n0, D);
                uint4 rsd[1];
                ll_load<1>(rsd, 1, s_in, pl, [&](int) { return A.xa + (size_t)min(m, n - 1) * D + n0 + ec; });
                slab_load(S, A.att, D, m0, n, st, pl);
                if (__syncthreads_or(pl.failed)) BATCH_BAIL();
                BATCH_MARK(l == 1 && u == b, 7);
                tile_mma<false>(S, Y.wo, D, n0, D);
                const float v0 = red_sum(S, er, ec) + __uint_as_float(rsd[0].x), v1 = red_sum(S, er, ec + 1) + __uint_as_float(rsd[0].z);
                float sq = m < n ? v0 * v0 + v1 * v1 : 0.f;
#pragma unroll
                for (int off = 8; off >= 1; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
                if (m < n) {
                    uint2 *dst = A.xb + (size_t)m * D + n0 + ec;
                    st_pair(dst, v0, st), st_pair(dst + 1, v1, st);
                    if ((tid & 15) == 0) st_pair(A.ssb + (size_t)m * parts + n0 / BN, sq, st);
                }
                __syncthreads();
                BATCH_MARK(l == 1 && u == b, 8);
            }
        }
        // ---- D: RMSNorm + W1,W3 + SwiGLU (W1/W3 interleaved in groups of 16 columns)  ->  act [n][F]
        {
            const int nt_n = 2 * F / BN;
            for (int u = b; u < mt_n * nt_n; u += G) {
                const int mt = u / nt_n, nt = u % nt_n, n0 = nt * BN, m0 = mt * BM;
                BATCH_MARK(l == 1 && u == b, 9);
                w_prefetch(S, A.w13[l], 2 * F, n0, D, Y.norm2);
                slab_load(S, A.xb, D, m0, n, st, pl);
                inv_rms_load(S, A.ssb, parts, D, A.eps, m0, n, st, pl);
                if (__syncthreads_or(pl.failed)) BATCH_BAIL();
                BATCH_MARK(l == 1 && u == b, 10);
                tile_mma<true>(S, A.w13[l], 2 * F, n0, D);
                const int r = tid >> 4, c = tid & 15, m = m0 + r;
                if (m < n) {
                    const float hv = red_sum(S, r, c), gv = red_sum(S, r, 16 + c);
                    float sg;
                    if (gv >= 20.f) sg = 1.f;
                    else if (gv <= -20.f) sg = 0.f;
                    else sg = 1.f / (1.f + expf(-gv));
                    st_pair(A.act + (size_t)m * F + nt * 16 + c, hv * (gv * sg), st);
                }
                __syncthreads();
                BATCH_MARK(l == 1 && u == b, 11);
            }
        }
        // ---- E: W2 + residual  ->  xa [n][D], ssa (the next layer's input)
        {
            const int nt_n = D / BN;
            for (int u = b; u < mt_n * nt_n; u += G) {
                const int mt = u / nt_n, n0 = (u % nt_n) * BN, m0 = mt * BM, m = m0 + er;
                BATCH_MARK(l == 1 && u == b, 12);
                w_prefetch(S, Y.w2, D, n0, F);
                uint4 rsd[1];
                ll_load<1>(rsd, 1, st, pl, [&](int) { return A.xb + (size_t)min(m, n - 1) * D + n0 + ec; });
                slab_load(S, A.act, F, m0, n, st, pl);
                if (__syncthreads_or(pl.failed)) BATCH_BAIL();
                BATCH_MARK(l == 1 && u == b, 13);
                tile_mma<false>(S, Y.w2, D, n0, F);
                const float v0 = red_sum(S, er, ec) + __uint_as_float(rsd[0].x), v1 = red_sum(S, er, ec + 1) + __uint_as_float(rsd[0].z);
                float sq = m < n ? v0 * v0 + v1 * v1 : 0.f;
#pragma unroll
                for (int off = 8; off >= 1; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
                if (m < n) {
                    uint2 *dst = A.xa + (size_t)m * D + n0 + ec;
                    st_pair(dst, v0, st), st_pair(dst + 1, v1, st);
                    if ((tid & 15) == 0) st_pair(A.ssa + (size_t)m * parts + n0 / BN, sq, st);
                }
                __syncthreads();
                BATCH_MARK(l == 1 && u == b, 14);
            }
        }
    }

    // ---- final norm + LM head: logits, and per (column tile, row) the best logit with its index ----
    const unsigned s_last = A.stamp0 + 1u + (unsigned)A.layers, s_out = s_last + 1u;
    const int vt_n = (V + BN - 1) / BN;
    for (int u = b; u < mt_n * vt_n; u += G) {
        const int mt = u % mt_n, vt = u / mt_n, n0 = vt * BN, m0 = mt * BM, m = m0 + er;
        w_prefetch(S, A.lm_head, V, n0, D, A.norm_final);
        slab_load(S, A.xa, D, m0, n, s_last, pl);
        inv_rms_load(S, A.ssa, parts, D, A.eps, m0, n, s_last, pl);
        if (__syncthreads_or(pl.failed)) BATCH_BAIL();
        tile_mma<true>(S, A.lm_head, V, n0, D);
        float best = -INFINITY;
        int best_i = 0x7fffffff;
        if (m < n) {
#pragma unroll
            for (int j = 0; j < 2; j++) {
                const int col = n0 + ec + j;
                if (col < V) {
                    const float v = red_sum(S, er, ec + j);
                    A.logits[(size_t)m * V + col] = v;
                    if (v > best || (v == best && col < best_i)) best = v, best_i = col;
                }
            }
        }
#pragma unroll
        for (int off = 8; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
            if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
        }
        if (m < n && (tid & 15) == 0) {
            uint2 *dst = A.cand + ((size_t)vt * n + m) * 2;
            st_pair(dst, best, s_out), st_pair(dst + 1, __int_as_float(best_i), s_out);
        }
        __syncthreads();
    }
    // ---- argmax over the column tiles: one warp per row ----
    for (int r = b * kWarps + warp; r < n; r += G * kWarps) {
        float bv = -INFINITY;
        int bi = 0x7fffffff;
        for (int t0 = lane; t0 < vt_n; t0 += 32 * 8) {
            uint4 v[8];
            const int cnt = min(8, (vt_n - t0 + 31) / 32);
            ll_load<8>(v, cnt, s_out, pl, [&](int i) { return A.cand + ((size_t)(t0 + 32 * i) * n + r) * 2; });
#pragma unroll
            for (int i = 0; i < 8; i++) {
                const float cv = __uint_as_float(v[i].x);
                const int ci = (int)v[i].z;
                if (i < cnt && !pl.failed && (cv > bv || (cv == bv && ci < bi))) bv = cv, bi = ci;
            }
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, bv, off);
            const int oi = __shfl_xor_sync(0xffffffffu, bi, off);
            if (ov > bv || (ov == bv && oi < bi)) bv = ov, bi = oi;
        }
        if (bi == 0x7fffffff) bi = 0;
        if (lane == 0) A.next[r] = bi;
    }
}

size_t batch_smem_bytes(int kmax) {
    return sizeof(float) * ((size_t)BM * (kmax + 4) + (size_t)STAGES * BK * WS + kmax);
}

}  // namespace

#ifdef JGPT_B200_DECODE_TRACE
extern "C" __attribute__((visibility("default"))) int32_t jgpt_debug_batch_trace_read(long long *host, int32_t n_ctas) {
    JGPT_CUDA_TRY(cudaMemcpyFromSymbol(host, g_batch_trace, sizeof(long long) * (size_t)n_ctas * kBatchMarks));
    return JGPT_OK;
}
#endif

// Chunk length of the attention (KV blocks per warp unit): the candidate that fills the warps' rounds best.
void batch_step_plan(BatchStepArgs &A, int sm_count, const int *lens_host) {
    A.kmax = std::max(A.D, A.F);
    A.scale_log2e = (1.0f / sqrtf((float)DH)) * 1.4426950408889634f;
    const long warps = (long)sm_count * kWarps;
    int max_blocks = 1;
    for (int i = 0; i < A.n; i++) max_blocks = std::max(max_blocks, (lens_host[i] + 15) / 16);
    int best_cb = std::min(32, max_blocks);
    double best_cost = 1e30;
    for (int cb = 2; cb <= 32; cb++) {
        // cost model (us): rounds of the busiest warp x (one memory round trip per group of kAttnGroup blocks + ~1.3 per unit
        // for the table entry, q, the merge and the ticket)
        long units = 0;
        for (int i = 0; i < A.n; i++) units += (long)(((lens_host[i] + 15) / 16 + cb - 1) / cb) * A.H;
        const long rounds = (units + warps - 1) / warps;
        const double cost = (double)rounds * ((cb + kAttnGroup - 1) / kAttnGroup * 1.0 + 1.3);
        if (cost < best_cost) best_cost = cost, best_cb = cb;
    }
    A.cb = best_cb;
    A.nch_max = (max_blocks + A.cb - 1) / A.cb;
}

int32_t launch_decode_batch(Ctx *ctx, BatchStepArgs &A) {
    JGPT_REQUIRE(A.n >= 1 && A.D == A.H * DH && A.D % 64 == 0 && A.F % 16 == 0 && A.vocab % 4 == 0,
                 JGPT_ERR_INVALID_ARGUMENT, "batched fused decode step: unsupported geometry");
    const size_t smem = batch_smem_bytes(A.kmax);
    static std::mutex mu;
    static std::unordered_set<int> ready;
    {
        std::lock_guard<std::mutex> g(mu);
        if (!ready.count(ctx->device)) {
            int coop = 0, per_sm = 0;
            JGPT_CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
            JGPT_REQUIRE(coop, JGPT_ERR_UNSUPPORTED, "device %d has no cooperative launch", ctx->device);
            JGPT_CUDA_TRY(cudaFuncSetAttribute(decode_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
            JGPT_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_batch_kernel, kThreads, 160 * 1024));
            JGPT_REQUIRE(per_sm >= 1, JGPT_ERR_UNSUPPORTED, "the batched fused decode step does not fit an SM");
            ready.insert(ctx->device);
        }
    }
    JGPT_REQUIRE(smem <= 160 * 1024, JGPT_ERR_INVALID_ARGUMENT, "model too wide for the batched fused decode step");
    void *args[1] = {&A};
    const cudaError_t le = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(decode_batch_kernel), dim3((unsigned)ctx->sm_count), dim3(kThreads),
                                              args, smem, ctx->stream);
    if (le != cudaSuccess) {  // e.g. the grid cannot be resident at once on what this process may use of the device
        cudaGetLastError();
        return fail(JGPT_ERR_UNSUPPORTED, "cooperative launch refused: %s", cudaGetErrorString(le));
    }
    return JGPT_OK;
}

}  // namespace jgpt
