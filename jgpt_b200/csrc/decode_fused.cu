// One decode step of the whole model as ONE cooperative launch, for a handful of rows (interactive generation:
// GptAutoregressiveGenerator's loop, src/main/java/com/veles/llm/jgpt/model/GptAutoregressiveGenerator.java:108-206,
// decodes one row at a time).
//
// With 1-4 rows every kernel of the layer chain (norm + Q,K,V, attention, Wo, norm + W1/W3 + SwiGLU, W2) moves a few
// kilobytes per SM and lasts a few microseconds; a step of 63 dependent launches is then nothing but launch and
// drain latencies.  Here one grid of one CTA per SM walks the same chain.  What one phase hands to the next (a few
// kilobytes of activations) travels through global memory as (value, stamp) pairs written with one 8-byte store:
// a reader polls the words it needs until they carry the stamp of the step and layer it is working on, so there
// is no grid-wide barrier, no fence and no atomic on the path - one store and one load between two phases.  (A
// buffer is rewritten one layer later; by then every CTA has consumed it, because each phase needs the output of
// ALL CTAs of the phase before.)  Everything a phase reads that does not depend on the previous one - its slice
// of the weights - is already on its way while it polls.  The residual row lives in every CTA's shared memory
// (each CTA applies the same updates in the same order, so the copies stay bit-identical); the narrow projections
// (Wo, W2) are split over k and their partial rows are summed by the reader in a fixed order, so a step is
// deterministic and a row's result does not depend on the other rows of the batch.  Several steps can run in one
// launch (greedy generation: the argmax of one step is the input of the next), which also removes the host round
// trip between tokens.
//
// Arithmetic: plain fp32 FMA for the projections (a row-vector times a matrix has no tile for a tensor core), the
// attention as in attn_decode.cu: RoPE (adjacent pairs, apply_rope_4d_kernel) on q and on the appended k, K/V
// rounded to fp16 in the paged store, scores and softmax in fp32 in the log2 domain, split over the sequence.
//
// The CTAs wait for one another's data, so the launch is cooperative (all CTAs resident or the launch is refused),
// and every wait is bounded: a thread that runs out of polls records DEV_STATUS_WAIT_TIMEOUT, publishes the
// launch's tag in the abort word and its CTA leaves; the others see the tag and leave too.  Stamps grow from launch
// to launch, so whatever an abandoned launch left behind is never mistaken for data.
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
constexpr int kWarps = kThreads / 32;
constexpr int kSlices = kThreads / 2;  // k slices of a projection unit: thread = (k slice, which 4 of the unit's 8 columns)
constexpr int kTileK = 3 * kSlices;    // k rows one register tile of a unit covers
constexpr int DH = 16;                 // head size of this path
constexpr int PS = DH + 2;             // an attention partial: running maximum, sum, DH unnormalised outputs
constexpr int kCandBatch = 5;          // per-CTA candidates a lane polls at a time when the tokens are picked

#ifdef JGPT_B200_DECODE_TRACE
// Timing build only: per CTA, SM clock at the marks of one layer (the second layer of the launch's last step).
constexpr int kTraceMarks = 24;
__device__ long long g_fused_trace[256 * kTraceMarks];
__device__ long long g_fused_trace_ns[256 * kTraceMarks];  // the same marks on the global timer (comparable across SMs)
#define FUSED_MARK(i)                                                                            \
    do {                                                                                         \
        if (tracing && threadIdx.x == 0) {                                                       \
            long long gt_;                                                                       \
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));                              \
            g_fused_trace[blockIdx.x * kTraceMarks + (i)] = clock64();                           \
            g_fused_trace_ns[blockIdx.x * kTraceMarks + (i)] = gt_;                              \
        }                                                                                        \
    } while (0)
#else
#define FUSED_MARK(i) \
    do {              \
    } while (0)
#endif

// Register tile of a projection unit: for up to two matrices, the thread's 4 columns of 3 k rows.
struct WTile {
    float4 w[2][3];
};

template <int NW>
__device__ __forceinline__ void tile_load(WTile &t, const float *W0, const float *W1, int N, int col, int k0, int k1) {
    const int ks = threadIdx.x >> 1;
#pragma unroll
    for (int i = 0; i < 3; i++) {
        const int k = k0 + ks + kSlices * i;
        const bool in = k < k1;
        t.w[0][i] = in ? __ldg(reinterpret_cast<const float4 *>(W0 + (size_t)k * N + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
        if (NW == 2) t.w[1][i] = in ? __ldg(reinterpret_cast<const float4 *>(W1 + (size_t)k * N + col)) : make_float4(0.f, 0.f, 0.f, 0.f);
    }
}

// acc[z][r][0..4) = sum over this thread's k rows of a[r][k - kbase] * W_z[k][col..col+4), k in [k0, k1).
// `t` holds the first tile already when `loaded`.
template <int R, int NW>
__device__ __forceinline__ void unit_fma(WTile &t, bool loaded, const float *W0, const float *W1, int N, int col, int k0, int k1,
                                         const float *a, int lda, int kbase, float (&acc)[NW][R][4]) {
    const int ks = threadIdx.x >> 1;
#pragma unroll
    for (int z = 0; z < NW; z++)
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int j = 0; j < 4; j++) acc[z][r][j] = 0.f;
    for (int kc = k0; kc < k1; kc += kTileK) {
        if (!(loaded && kc == k0)) tile_load<NW>(t, W0, W1, N, col, kc, k1);
#pragma unroll
        for (int i = 0; i < 3; i++) {
            const int k = kc + ks + kSlices * i;
            if (k < k1) {
#pragma unroll
                for (int r = 0; r < R; r++) {
                    const float av = a[r * lda + (k - kbase)];
#pragma unroll
                    for (int z = 0; z < NW; z++) {
                        acc[z][r][0] = fmaf(av, t.w[z][i].x, acc[z][r][0]);
                        acc[z][r][1] = fmaf(av, t.w[z][i].y, acc[z][r][1]);
                        acc[z][r][2] = fmaf(av, t.w[z][i].z, acc[z][r][2]);
                        acc[z][r][3] = fmaf(av, t.w[z][i].w, acc[z][r][3]);
                    }
                }
            }
        }
    }
}

// Sums the k slices of a unit.  Afterwards lane (r * 8 + c) of warp 0 holds, for column c of the unit's 8 and row r,
// res[z].  Ends with a block barrier, so `red` may be reused at once.
template <int R, int NW>
__device__ __forceinline__ void unit_reduce(float (&acc)[NW][R][4], float *red, float (&res)[NW]) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
#pragma unroll
    for (int z = 0; z < NW; z++)
#pragma unroll
        for (int r = 0; r < R; r++)
#pragma unroll
            for (int j = 0; j < 4; j++) {
                float v = acc[z][r][j];
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                v += __shfl_xor_sync(0xffffffffu, v, 4);
                v += __shfl_xor_sync(0xffffffffu, v, 8);
                v += __shfl_xor_sync(0xffffffffu, v, 16);
                if (lane < 2) red[(((warp * 2 + lane) * NW + z) * R + r) * 4 + j] = v;
            }
    __syncthreads();
#pragma unroll
    for (int z = 0; z < NW; z++) res[z] = 0.f;
    if (warp == 0 && lane < R * 8) {
        const int r = lane >> 3, hf = (lane >> 2) & 1, j = lane & 3;
#pragma unroll
        for (int z = 0; z < NW; z++) {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) s += red[(((w * 2 + hf) * NW + z) * R + r) * 4 + j];
            res[z] = s;
        }
    }
    __syncthreads();
}

constexpr int kGammaRegs = 4;  // norm weights a thread keeps in registers: columns tid, tid + 256, ... (d_model <= 1024)
struct Gamma {
    float g[kGammaRegs];
};
// Issued before a wait, so that the weights are in registers when the rows arrive.
__device__ __forceinline__ void gamma_load(Gamma &gm, const float *gamma, int D) {
#pragma unroll
    for (int i = 0; i < kGammaRegs; i++) {
        const int j = threadIdx.x + kThreads * i;
        gm.g[i] = j < D ? __ldg(gamma + j) : 0.f;
    }
}

// x[r][:] += p[0][r][:] + p[1][r][:] + ... (ks partial rows, summed in that order; p == nullptr: nothing to add), then
// a[r][:] = x[r][:] * inv_rms(x[r]) * gamma, rows < n  (rms_norm_fwd_block_kernel,
// jgpt_cuda_extra_kernels_launches.inl:694-713).  Returns false when a wait gave up.
template <int R>
__device__ __forceinline__ bool residual_norm(float *x, const uint2 *p, int ks, int n, int D, unsigned stamp, Poll &pl, const Gamma &gm,
                                              float *a, float eps, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; r++) ss[r] = 0.f;
    const int half = D / 2;
    for (int e2 = threadIdx.x; e2 < n * half; e2 += kThreads) {
        float v0 = x[2 * e2], v1 = x[2 * e2 + 1];
        if (p) {
            uint4 v[kFusedMaxKSplit];
            ll_load<kFusedMaxKSplit>(v, ks, stamp, pl, [&](int j) { return p + (size_t)j * R * D + 2 * e2; });
            float s0 = __uint_as_float(v[0].x), s1 = __uint_as_float(v[0].z);
#pragma unroll
            for (int j = 1; j < kFusedMaxKSplit; j++)
                if (j < ks) s0 += __uint_as_float(v[j].x), s1 += __uint_as_float(v[j].z);
            v0 += s0, v1 += s1;
            x[2 * e2] = v0, x[2 * e2 + 1] = v1;
        }
        const int r = e2 / half;
#pragma unroll
        for (int rr = 0; rr < R; rr++)
            if (rr == r) ss[rr] = fmaf(v0, v0, fmaf(v1, v1, ss[rr]));
    }
#pragma unroll
    for (int r = 0; r < R; r++) {
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], off);
        if (lane == 0) red[warp * R + r] = ss[r];
    }
    if (__syncthreads_or(pl.failed)) return false;
#pragma unroll
    for (int r = 0; r < R; r++) {
        float sum = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) sum += red[w * R + r];
        const float rms = sqrtf(sum / (float)D + eps);
        const float inv = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
#pragma unroll
        for (int i = 0; i < kGammaRegs; i++) {
            const int j = threadIdx.x + kThreads * i;
            if (j < D) a[r * D + j] = x[r * D + j] * inv * gm.g[i];
        }
    }
    __syncthreads();
    return true;
}

// One (row, head, chunk) of the attention: RoPE on q, the new token appended by the chunk that owns its slot, a
// partial (maximum, sum, outputs) of this chunk's tokens left in `part`.  `sq` = 3 * DH floats of shared memory.
__device__ __forceinline__ bool attention_unit(const FusedStepArgs &A, int layer, int r, int h, int c, int step, unsigned stamp, Poll &pl,
                                               float *red, float *sq, const int *idx, bool trace_on = false) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = A.n;
    const int seq = idx[2 * n + r], rp = idx[3 * n + r] + step, len = idx[4 * n + r] + step;
    const int nbk = (len + 15) >> 4;
    const int b0 = c * A.cb, b1 = min(nbk, b0 + A.cb);  // a row shorter than the launch's longest leaves chunks empty
    const int t0 = b0 * 16, t1 = min(len, b1 * 16);
    const float2 *cs = A.rope + (size_t)rp * (DH / 2);
    const size_t layer_base = (size_t)layer * A.n_blocks;
    // Rows of the cache do not depend on this step (the appended one apart): the first token of every thread is on its
    // way before q has arrived.  A row appended in an earlier step of this launch was written by this same CTA (the
    // unit -> CTA map is fixed for a launch), so a block barrier orders it; L1 is bypassed all the same.
    __align__(16) __half kh[DH], vh[DH];
    auto row_ptr = [&](int tok, __half *&kp) -> bool {
        const int phys = __ldcg(A.table + (size_t)seq * A.mbs + (tok >> 4));
        if (phys < 0 || phys >= A.n_blocks) {
            atomicOr(A.status, DEV_STATUS_BAD_BLOCK);
            return false;
        }
        kp = A.kv + ((layer_base + phys) * A.H + h) * (size_t)(2 * 16 * DH) + (size_t)(tok & 15) * DH;
        return true;
    };
    auto row_load = [&](const __half *kp) {
        reinterpret_cast<uint4 *>(kh)[0] = __ldcg(reinterpret_cast<const uint4 *>(kp));
        reinterpret_cast<uint4 *>(kh)[1] = __ldcg(reinterpret_cast<const uint4 *>(kp) + 1);
        reinterpret_cast<uint4 *>(vh)[0] = __ldcg(reinterpret_cast<const uint4 *>(kp + 16 * DH));
        reinterpret_cast<uint4 *>(vh)[1] = __ldcg(reinterpret_cast<const uint4 *>(kp + 16 * DH) + 1);
    };
    __half *kp0 = nullptr;
    const int tok0 = t0 + tid;
    const bool ok0 = tok0 < t1 && row_ptr(tok0, kp0);
    if (ok0 && tok0 != len - 1) row_load(kp0);
    float2 rope[DH / 2];
#pragma unroll
    for (int j = 0; j < DH / 2; j++) rope[j] = __ldg(cs + j);
    // this head's q, k, v of the row: 3 x 8 pairs, polled by the LAST warp: it has no cache rows in flight unless the chunk
    // is longer than 224 tokens (a warp's wait for its poll may also wait for that warp's older loads from HBM)
    if (tid >= kThreads - 32 && tid < kThreads - 32 + 3 * DH / 2) {
        const int pt = tid - (kThreads - 32);
        uint4 v[1];
        const uint2 *src = A.ll_qkv + (size_t)r * 3 * A.D + (size_t)(pt / (DH / 2)) * A.D + h * DH + 2 * (pt % (DH / 2));
        ll_load<1>(v, 1, stamp, pl, [&](int) { return src; });
        sq[2 * pt] = __uint_as_float(v[0].x), sq[2 * pt + 1] = __uint_as_float(v[0].z);
    }
    if (__syncthreads_or(pl.failed)) return false;
#ifdef JGPT_B200_DECODE_TRACE
    if (threadIdx.x == 0 && trace_on) {
        long long gt_;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));
        g_fused_trace_ns[blockIdx.x * kTraceMarks + 14] = gt_;
    }
#endif
    float q[DH];
#pragma unroll
    for (int j = 0; j < DH / 2; j++) {
        const float2 w = rope[j];
        const float x0 = sq[2 * j], x1 = sq[2 * j + 1];
        q[2 * j] = __fsub_rn(__fmul_rn(x0, w.x), __fmul_rn(x1, w.y)) * A.scale_log2e;
        q[2 * j + 1] = __fadd_rn(__fmul_rn(x0, w.y), __fmul_rn(x1, w.x)) * A.scale_log2e;
    }
    float m = -INFINITY, l = 0.f, o[DH];
#pragma unroll
    for (int d = 0; d < DH; d++) o[d] = 0.f;
    for (int tok = tok0; tok < t1; tok += kThreads) {
        __half *kp = kp0;
        if (tok == tok0) {
            if (!ok0) continue;
        } else {
            if (!row_ptr(tok, kp)) continue;
            if (tok != len - 1) row_load(kp);
        }
        if (tok == len - 1) {  // the appended token: RoPE'd k and raw v, rounded to fp16, stored and scored from registers
#pragma unroll
            for (int j = 0; j < DH / 2; j++) {
                const float2 w = rope[j];
                const float k0 = sq[DH + 2 * j], k1 = sq[DH + 2 * j + 1];
                kh[2 * j] = __float2half_rn(__fsub_rn(__fmul_rn(k0, w.x), __fmul_rn(k1, w.y)));
                kh[2 * j + 1] = __float2half_rn(__fadd_rn(__fmul_rn(k0, w.y), __fmul_rn(k1, w.x)));
                vh[2 * j] = __float2half_rn(sq[2 * DH + 2 * j]);
                vh[2 * j + 1] = __float2half_rn(sq[2 * DH + 2 * j + 1]);
            }
            reinterpret_cast<uint4 *>(kp)[0] = reinterpret_cast<const uint4 *>(kh)[0];
            reinterpret_cast<uint4 *>(kp)[1] = reinterpret_cast<const uint4 *>(kh)[1];
            reinterpret_cast<uint4 *>(kp + 16 * DH)[0] = reinterpret_cast<const uint4 *>(vh)[0];
            reinterpret_cast<uint4 *>(kp + 16 * DH)[1] = reinterpret_cast<const uint4 *>(vh)[1];
        }
        float sc = 0.f;
#pragma unroll
        for (int d = 0; d < DH; d++) sc = fmaf(q[d], __half2float(kh[d]), sc);
        if (sc > m) {
            const float corr = fast_exp2(m - sc);
            l *= corr;
#pragma unroll
            for (int d = 0; d < DH; d++) o[d] *= corr;
            m = sc;
        }
        const float pe = fast_exp2(sc - m);
        l += pe;
#pragma unroll
        for (int d = 0; d < DH; d++) o[d] = fmaf(pe, __half2float(vh[d]), o[d]);
    }
#ifdef JGPT_B200_DECODE_TRACE
    if (threadIdx.x == 0 && trace_on) {
        long long gt_;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(gt_));
        g_fused_trace_ns[blockIdx.x * kTraceMarks + 15] = gt_;
    }
#endif
    // merge: lanes of a warp, then the warps
    float M = m;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
    l *= f;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
#pragma unroll
    for (int d = 0; d < DH; d++) o[d] *= f;
    // sum of the 32 lanes' o[0..16) with 16 shuffles: at every stage a lane keeps one half of what it still holds and
    // adds its partner's copy of that half; lane L ends with dimension L >> 1
#pragma unroll
    for (int width = DH / 2, off = 16; width >= 1; width >>= 1, off >>= 1) {
        const bool upper = (lane & off) != 0;
#pragma unroll
        for (int j = 0; j < DH / 2; j++)
            if (j < width) {
                const float mine = upper ? o[j + width] : o[j], theirs = upper ? o[j] : o[j + width];
                o[j] = mine + __shfl_xor_sync(0xffffffffu, theirs, off);
            }
    }
    o[0] += __shfl_xor_sync(0xffffffffu, o[0], 1);
    {
        float *w = red + warp * PS;
        if (lane == 0) w[0] = M, w[1] = l;
        if ((lane & 1) == 0) w[2 + (lane >> 1)] = o[0];
    }
    __syncthreads();
    if (tid < PS) {
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; w++) Mx = fmaxf(Mx, red[w * PS]);
        uint2 *dst = A.ll_part + (((size_t)r * A.H + h) * A.nch + c) * PS;
        if (tid == 0) {
            st_pair(dst, Mx, stamp);
        } else {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                const float mw = red[w * PS];
                s = fmaf(red[w * PS + tid], mw == -INFINITY ? 0.f : exp2f(mw - Mx), s);
            }
            st_pair(dst + tid, s, stamp);
        }
    }
    __syncthreads();
    return true;
}

// Merged attention output for model columns [k0, k1) (whole heads) of rows < n into a[r * lda + (k - k0)].
// A pair of adjacent dimensions of one row is merged by 4 / R threads.  The chunks form four classes (chunk mod 4, at
// most two chunks each); a thread owns R classes, fetches their (maximum, sum) and outputs in one wait, the threads
// of a pair exchange maxima and then the weighted sums per class through shared memory, and the classes are added in the
// order 0, 1, 2, 3 - the same association whatever R is, so a row's result does not depend on the size of the batch.
// All loops have compile-time bounds: the weights are independent exp2 evaluations, not a chain.
// `stage`: kThreads float4 (maxima) followed by 4 * (kThreads / (4 / R)) float4 (class sums).
static_assert(kFusedMaxChunks == 8, "the merge keeps two chunks per class");
template <int R>
__device__ __forceinline__ bool merge_attention(const FusedStepArgs &A, float *a, int lda, int k0, int k1, unsigned stamp, Poll &pl,
                                               float *stage) {
    constexpr int GROUPS = 4 / R, PT = kThreads / GROUPS;  // threads per pair, pairs per pass
    const int span2 = (k1 - k0) / 2, pairs = A.n * span2, nch = A.nch;
    const int g = threadIdx.x / PT, pe = threadIdx.x % PT;
    float4 *mx4 = reinterpret_cast<float4 *>(stage), *cls4 = mx4 + kThreads;  // cls4[class * PT + pair]
    for (int e0 = 0; e0 < pairs; e0 += PT) {
        const int e = e0 + pe;
        const bool live = e < pairs;
        int r = 0, k = k0;
        if (live) r = e / span2, k = k0 + 2 * (e % span2);
        const int h = k / DH, d = k % DH;
        const uint2 *pp = A.ll_part + (((size_t)r * A.H + h) * nch) * PS;
        // entry i: class g + GROUPS * (i / 4), its chunk (i / 2) % 2 (class, class + 4), (maximum, sum) or the two outputs
        uint4 v[4 * R];
        auto chunk_of = [&](int i) { return g + GROUPS * (i >> 2) + 4 * ((i >> 1) & 1); };
        ll_load<4 * R>(v, live ? 4 * R : 0, stamp, pl, [&](int i) {
            const int c = min(chunk_of(i), nch - 1);  // classes beyond the launch's chunks re-read the last chunk; never used
            return pp + c * PS + ((i & 1) ? 2 + d : 0);
        });
        float m_loc = -INFINITY;
#pragma unroll
        for (int i = 0; i < 4 * R; i += 2)
            if (chunk_of(i) < nch) m_loc = fmaxf(m_loc, __uint_as_float(v[i].x));
        mx4[threadIdx.x].x = m_loc;
        if (__syncthreads_or(pl.failed)) return false;
        float Mx = -INFINITY;
#pragma unroll
        for (int gg = 0; gg < GROUPS; gg++) Mx = fmaxf(Mx, mx4[gg * PT + pe].x);
#pragma unroll
        for (int vi = 0; vi < R; vi++) {  // this thread's classes
            float L = 0.f, acc0 = 0.f, acc1 = 0.f;
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int i = 4 * vi + 2 * half;
                if (chunk_of(i) < nch) {
                    const float mc = __uint_as_float(v[i].x);
                    const float w = mc == -INFINITY ? 0.f : exp2f(mc - Mx);
                    L = fmaf(__uint_as_float(v[i].z), w, L);
                    acc0 = fmaf(__uint_as_float(v[i + 1].x), w, acc0);
                    acc1 = fmaf(__uint_as_float(v[i + 1].z), w, acc1);
                }
            }
            cls4[(g + GROUPS * vi) * PT + pe] = make_float4(0.f, L, acc0, acc1);
        }
        __syncthreads();
        if (g == 0 && live) {
            float4 t = cls4[pe];
#pragma unroll
            for (int cl = 1; cl < 4; cl++) {
                const float4 o = cls4[cl * PT + pe];
                t.y += o.y, t.z += o.z, t.w += o.w;
            }
            const float inv = 1.f / fmaxf(t.y, 1e-12f);
            a[r * lda + (k - k0)] = t.z * inv, a[r * lda + (k - k0) + 1] = t.w * inv;
        }
        __syncthreads();
    }
    return true;
}

template <int R>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const FusedStepArgs A) {
    extern __shared__ __align__(16) float sm[];
    float *x = sm;                    // [R][D]  the residual rows
    float *a = x + R * A.D;           // [R][max(D, F)]  what the current projection multiplies
    float *red = a + R * A.amax;      // reductions
    float *sq = red + kWarps * 2 * 2 * R * 4 + kWarps * PS;  // q, k, v of one head
    float *stage = sq + 3 * DH;                              // [256][4] chunk partials on their way to be merged
    float *lm_w = stage + kThreads * 4 + 4 * kThreads * 4;  // [lm_stage][D][8] this CTA's first LM-head column blocks
    __shared__ int s_tok[R];
    __shared__ int s_idx[5 * 4];  // the rows' descriptors: out of the launch parameters (a per-token call) or device memory
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x, G = gridDim.x, n = A.n, D = A.D, F = A.F;
    const int half_col = (tid & 1) * 4;
    if (tid < 5 * A.n) s_idx[tid] = A.idx ? A.idx[tid] : A.idx_inline[tid];
    for (int e = tid; e < R * D; e += kThreads) x[e] = 0.f;
    for (int e = tid; e < R * A.amax; e += kThreads) a[e] = 0.f;
    __syncthreads();
    Poll pl{A.sync_words, A.stamp0 + 1u, A.status, 0};
    const int nA = 3 * D / 8, nO = D / 8, nD = F / 8, nL = A.vocab / 8;
    const int kso = A.ks_o, klo = A.kl_o, ks2 = A.ks_2, kl2 = A.kl_2;
    const bool out_lane = warp == 0 && lane < R * 8 && (lane >> 3) < n;  // lanes that hold a unit's results
    const int out_r = lane >> 3, out_c = lane & 7;

    WTile t;
    Gamma gam;
    bool have = false;
    auto load_A = [&](int l, int u) {  // unit u of the Q,K,V product: 8 columns of one of the three matrices
        const int z = u / nO, c0 = (u % nO) * 8;
        const float *W = z == 0 ? A.Lw[l].wq : (z == 1 ? A.Lw[l].wk : A.Lw[l].wv);
        tile_load<1>(t, W, nullptr, D, c0 + half_col, 0, D);
    };
    if (b < nA) load_A(0, b), have = true;

    int steps_done = 0;
    for (int step = 0; step < A.steps; step++) {
        // ---- embedding + learned position row (embedding_token_fwd_kernel + add_position_embedding_broadcast_kernel)
        for (int e = tid; e < n * D; e += kThreads) {
            const int r = e / D, j = e % D;
            const int id = step == 0 ? s_idx[r] : s_tok[r];
            const int pr = (s_idx[3 * n + r] + step) % A.max_seq;
            x[e] = __ldg(A.tok + (size_t)id * D + j) + __ldg(A.pos + (size_t)pr * D + j);
        }
        __syncthreads();

        gamma_load(gam, A.Lw[0].norm1, D);
        for (int l = 0; l < A.layers; l++) {
            const unsigned stamp = A.stamp0 + (unsigned)(step * A.layers + l) + 1u;  // of everything this layer writes
#ifdef JGPT_B200_DECODE_TRACE
            const bool tracing = step == A.steps - 1 && l == 1;
#endif
            FUSED_MARK(0);
            // ---- A: norm1 + Q,K,V
            if (!residual_norm<R>(x, l > 0 ? A.ll_pw2 : nullptr, ks2, n, D, stamp - 1u, pl, gam, a, A.eps, red)) goto leave;
            FUSED_MARK(2);
            for (int u = b; u < nA; u += G) {
                const int z = u / nO, c0 = (u % nO) * 8;
                const float *W = z == 0 ? A.Lw[l].wq : (z == 1 ? A.Lw[l].wk : A.Lw[l].wv);
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, have && u == b, W, nullptr, D, c0 + half_col, 0, D, a, D, 0, acc);
                FUSED_MARK(1);
                unit_reduce<R, 1>(acc, red, res);
                FUSED_MARK(7);
                // test hook (host-side fault injection): CTA 0 withholds its first layer's result, so the units that
                // need it run into their bounded wait and the launch reports WAIT_TIMEOUT
                if (out_lane && !(A.test_withhold && b == 0 && l == 0))
                    st_pair(A.ll_qkv + (size_t)out_r * 3 * D + z * D + c0 + out_c, res[0], stamp);
            }
            have = false;
            if (b < nO * kso) {  // Wo: unit = 8 columns x one k range; on its way while the attention runs
                const int c0 = (b % nO) * 8, k0 = (b / nO) * klo;
                tile_load<1>(t, A.Lw[l].wo, nullptr, D, c0 + half_col, k0, min(D, k0 + klo));
                have = true;
            }

            gamma_load(gam, A.Lw[l].norm2, D);
            if (l == A.layers - 1) {  // the LM head's weights for this CTA's first column blocks: into shared memory, well ahead
                for (int j = 0; j < A.lm_stage && b + j * G < nL; j++) {
                    const float *src = A.lm_head + (size_t)(b + j * G) * 8;
                    float *dst = lm_w + (size_t)j * D * 8;
                    for (int e = tid; e < D * 2; e += kThreads) cp_async16(dst + e * 4, src + (size_t)(e >> 1) * A.vocab + (e & 1) * 4, true);
                }
                asm volatile("cp.async.commit_group;" ::: "memory");
            }
            FUSED_MARK(3);
            // ---- B: append + attention partials
            for (int u = b; u < n * A.H * A.nch; u += G) {
                const int c = u % A.nch, h = (u / A.nch) % A.H, r = u / (A.nch * A.H);
#ifdef JGPT_B200_DECODE_TRACE
                if (!attention_unit(A, l, r, h, c, step, stamp, pl, red, sq, s_idx, tracing)) goto leave;
#else
                if (!attention_unit(A, l, r, h, c, step, stamp, pl, red, sq, s_idx)) goto leave;
#endif
            }

            FUSED_MARK(4);
            // ---- C: merged attention rows . Wo, partial rows per k range
            for (int u = b; u < nO * kso; u += G) {
                const int c0 = (u % nO) * 8, kj = u / nO, k0 = kj * klo, k1 = min(D, k0 + klo);
                                if (!merge_attention<R>(A, a, klo, k0, k1, stamp, pl, stage)) goto leave;
                FUSED_MARK(5);
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, have && u == b, A.Lw[l].wo, nullptr, D, c0 + half_col, k0, k1, a, klo, k0, acc);
                FUSED_MARK(12);
                unit_reduce<R, 1>(acc, red, res);
                FUSED_MARK(13);
                if (out_lane) st_pair(A.ll_po + ((size_t)kj * R + out_r) * D + c0 + out_c, res[0], stamp);
            }
            have = false;
            if (b < nD) {
                tile_load<2>(t, A.Lw[l].w1, A.Lw[l].w3, F, b * 8 + half_col, 0, D);
                have = true;
            }

            FUSED_MARK(6);
            // ---- D: x += attention projection; norm2 + W1, W3 + SwiGLU (sigmoid_kernel / mul_kernel, same file :799-832)
            if (!residual_norm<R>(x, A.ll_po, kso, n, D, stamp, pl, gam, a, A.eps, red)) goto leave;
            FUSED_MARK(8);
            for (int u = b; u < nD; u += G) {
                float acc[2][R][4], res[2];
                unit_fma<R, 2>(t, have && u == b, A.Lw[l].w1, A.Lw[l].w3, F, u * 8 + half_col, 0, D, a, D, 0, acc);
                unit_reduce<R, 2>(acc, red, res);
                if (out_lane) {
                    const float gv = res[1];
                    float sg;
                    if (gv >= 20.f) sg = 1.f;
                    else if (gv <= -20.f) sg = 0.f;
                    else sg = 1.f / (1.f + expf(-gv));
                    st_pair(A.ll_act + (size_t)out_r * F + u * 8 + out_c, res[0] * (gv * sg), stamp);
                }
            }
            have = false;
            if (b < nO * ks2) {
                const int c0 = (b % nO) * 8, k0 = (b / nO) * kl2;
                tile_load<1>(t, A.Lw[l].w2, nullptr, D, c0 + half_col, k0, min(F, k0 + kl2));
                have = true;
            }

            gamma_load(gam, l + 1 < A.layers ? A.Lw[l + 1].norm1 : A.norm_final, D);
            FUSED_MARK(9);
            // ---- E: activation . W2, partial rows per k range
            for (int u = b; u < nO * ks2; u += G) {
                const int c0 = (u % nO) * 8, kj = u / nO, k0 = kj * kl2, k1 = min(F, k0 + kl2), span2 = (k1 - k0) / 2;
                for (int e = tid; e < n * span2; e += kThreads) {
                    const int r = e / span2, k = 2 * (e % span2);
                    uint4 v[1];
                    const uint2 *src = A.ll_act + (size_t)r * F + k0 + k;
                    ll_load<1>(v, 1, stamp, pl, [&](int) { return src; });
                    a[r * kl2 + k] = __uint_as_float(v[0].x), a[r * kl2 + k + 1] = __uint_as_float(v[0].z);
                }
                if (__syncthreads_or(pl.failed)) goto leave;
                FUSED_MARK(10);
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, have && u == b, A.Lw[l].w2, nullptr, D, c0 + half_col, k0, k1, a, kl2, k0, acc);
                unit_reduce<R, 1>(acc, red, res);
                if (out_lane) st_pair(A.ll_pw2 + ((size_t)kj * R + out_r) * D + c0 + out_c, res[0], stamp);
            }
            have = false;
            FUSED_MARK(11);
            if (l + 1 < A.layers) {
                if (b < nA) load_A(l + 1, b), have = true;
            } else if (b < nL && A.lm_stage == 0) {
                tile_load<1>(t, A.lm_head, nullptr, A.vocab, b * 8 + half_col, 0, D);
                have = true;
            }
        }

        // ---- final norm + LM head; every CTA keeps the best (value, lowest index) of its columns per row
        {
            const unsigned stamp = A.stamp0 + (unsigned)((step + 1) * A.layers);  // the last layer's
#ifdef JGPT_B200_DECODE_TRACE
            const bool tracing = step == A.steps - 1;
#endif
            FUSED_MARK(16);
            if (!residual_norm<R>(x, A.ll_pw2, ks2, n, D, stamp, pl, gam, a, A.eps, red)) goto leave;
            FUSED_MARK(17);
            float best = -INFINITY;
            int best_i = 0x7fffffff;
            if (A.lm_stage > 0) {
                asm volatile("cp.async.wait_group 0;" ::: "memory");
                __syncthreads();
            }
            const int u_reg0 = b + A.lm_stage * G;  // first unit whose weights come through registers
            if (!have && u_reg0 < nL) tile_load<1>(t, A.lm_head, nullptr, A.vocab, u_reg0 * 8 + half_col, 0, D);
            int j = 0;
            for (int u = b; u < nL; u += G, j++) {
                float acc[1][R][4], res[1];
                WTile tn;  // beyond the staged blocks: the next unit's tile is on its way while this one is multiplied and reduced
                if (j < A.lm_stage) {  // weights in shared memory: [k][8 columns]
                    const float *wu = lm_w + (size_t)j * D * 8 + half_col;
#pragma unroll
                    for (int r = 0; r < R; r++)
#pragma unroll
                        for (int q4 = 0; q4 < 4; q4++) acc[0][r][q4] = 0.f;
                    for (int k = tid >> 1; k < D; k += kSlices) {
                        const float4 w = *reinterpret_cast<const float4 *>(wu + (size_t)k * 8);
#pragma unroll
                        for (int r = 0; r < R; r++) {
                            const float av = a[r * D + k];
                            acc[0][r][0] = fmaf(av, w.x, acc[0][r][0]), acc[0][r][1] = fmaf(av, w.y, acc[0][r][1]);
                            acc[0][r][2] = fmaf(av, w.z, acc[0][r][2]), acc[0][r][3] = fmaf(av, w.w, acc[0][r][3]);
                        }
                    }
                } else {
                    if (u + G < nL) tile_load<1>(tn, A.lm_head, nullptr, A.vocab, (u + G) * 8 + half_col, 0, D);
                    unit_fma<R, 1>(t, true, A.lm_head, nullptr, A.vocab, u * 8 + half_col, 0, D, a, D, 0, acc);
                }
                unit_reduce<R, 1>(acc, red, res);
                if (j >= A.lm_stage && u + G < nL) t = tn;
                if (out_lane) {
                    const int col = u * 8 + out_c;
                    A.logits[(size_t)out_r * A.vocab + col] = res[0];
                    if (res[0] > best || (res[0] == best && col < best_i)) best = res[0], best_i = col;
                }
            }
            have = false;
            if (warp == 0) {
#pragma unroll
                for (int off = 4; off >= 1; off >>= 1) {
                    const float ov = __shfl_xor_sync(0xffffffffu, best, off);
                    const int oi = __shfl_xor_sync(0xffffffffu, best_i, off);
                    if (ov > best || (ov == best && oi < best_i)) best = ov, best_i = oi;
                }
                if (lane < R * 8 && out_c == 0) {  // (value, stamp), (index, stamp)
                    uint2 *dst = A.ll_cand + ((size_t)b * R + out_r) * 2;
                    st_pair(dst, best, stamp);
                    st_pair(dst + 1, __int_as_float(best_i), stamp);
                }
            }
            FUSED_MARK(18);
            if (step + 1 < A.steps && b < nA) load_A(0, b), have = true;
            // every CTA picks the tokens itself (the same comparison order everywhere)
            if (warp < n) {
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int g0 = lane; g0 < G; g0 += 32 * kCandBatch) {  // this lane's CTAs, a batch of polls in flight at a time
                    uint4 v[kCandBatch];
                    const int cnt = min(kCandBatch, (G - g0 + 31) / 32);
                    ll_load<kCandBatch>(v, cnt, stamp, pl, [&](int i) { return A.ll_cand + ((size_t)(g0 + 32 * i) * R + warp) * 2; });
#pragma unroll
                    for (int i = 0; i < kCandBatch; i++) {
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
                if (bi == 0x7fffffff) bi = 0;  // nothing compared greater than -inf: index 0, as argmax_kernel answers
                if (lane == 0) {
                    s_tok[warp] = bi;
                    if (b == 0) {
                        A.next[(size_t)step * n + warp] = bi;
                        if (A.next_host) A.next_host[(size_t)step * n + warp] = bi;  // mapped host memory: no copy after the launch
                    }
                }
            }
            if (__syncthreads_or(pl.failed)) goto leave;
            FUSED_MARK(19);
            steps_done = step + 1;
            if (A.stop_on_zero && s_tok[0] == 0) break;
        }
    }
leave:
    asm volatile("cp.async.wait_all;" ::: "memory");  // nothing may still be copying into this CTA's shared memory
    if (b == 0 && tid == 0) {
        *A.steps_done = steps_done;
        if (A.steps_done_host) *A.steps_done_host = steps_done;
    }
}

template <int R>
static size_t fused_smem_bytes(const FusedStepArgs &A) {
    return sizeof(float) * ((size_t)R * A.D + (size_t)R * A.amax + (size_t)kWarps * 2 * 2 * R * 4 + kWarps * PS + 3 * DH + kThreads * 4 + 4 * kThreads * 4 + (size_t)A.lm_stage * A.D * 8);
}

template <int R>
static int32_t launch_rows(Ctx *ctx, FusedStepArgs &A) {
    const size_t smem = fused_smem_bytes<R>(A);
    static std::mutex mu;
    static std::unordered_set<int> ready;  // devices on which this instantiation has been opted in and sized
    static int grid_for[64] = {};
    {
        std::lock_guard<std::mutex> g(mu);
        if (!ready.count(ctx->device)) {
            int coop = 0, per_sm = 0;
            JGPT_CUDA_TRY(cudaDeviceGetAttribute(&coop, cudaDevAttrCooperativeLaunch, ctx->device));
            JGPT_REQUIRE(coop, JGPT_ERR_UNSUPPORTED, "device %d has no cooperative launch", ctx->device);
            JGPT_CUDA_TRY(cudaFuncSetAttribute(decode_step_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 160 * 1024));
            JGPT_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<R>, kThreads, 160 * 1024));
            JGPT_REQUIRE(per_sm >= 1, JGPT_ERR_UNSUPPORTED, "the fused decode step does not fit an SM");
            grid_for[ctx->device & 63] = ctx->sm_count;
            ready.insert(ctx->device);
        }
    }
    JGPT_REQUIRE(smem <= 160 * 1024, JGPT_ERR_INVALID_ARGUMENT, "model too wide for the fused decode step");
    const int G = grid_for[ctx->device & 63];
    JGPT_REQUIRE(G == A.grid, JGPT_ERR_ILLEGAL_STATE, "fused decode step sized for %d CTAs, device runs %d", A.grid, G);
    void *args[1] = {&A};
    const cudaError_t le = cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(decode_step_kernel<R>), dim3((unsigned)G), dim3(kThreads), args,
                                              smem, ctx->stream);
    if (le != cudaSuccess) {  // e.g. the grid cannot be resident at once on what this process may use of the device
        cudaGetLastError();
        return fail(JGPT_ERR_UNSUPPORTED, "cooperative launch refused: %s", cudaGetErrorString(le));
    }
    return JGPT_OK;
}

}  // namespace

#ifdef JGPT_B200_DECODE_TRACE
extern "C" __attribute__((visibility("default"))) int32_t jgpt_debug_fused_trace_read(long long *host, int32_t n_ctas) {
    JGPT_CUDA_TRY(cudaMemcpyFromSymbol(host, g_fused_trace, sizeof(long long) * (size_t)n_ctas * kTraceMarks));
    return JGPT_OK;
}
extern "C" __attribute__((visibility("default"))) int32_t jgpt_debug_fused_trace_read_ns(long long *host, int32_t n_ctas) {
    JGPT_CUDA_TRY(cudaMemcpyFromSymbol(host, g_fused_trace_ns, sizeof(long long) * (size_t)n_ctas * kTraceMarks));
    return JGPT_OK;
}
#endif

int fused_step_max_rows() { return 4; }

// Splits that depend on the grid: how many k ranges the narrow projections are cut into, the attention chunks.
void fused_step_plan(FusedStepArgs &A, int sm_count, int max_len) {
    A.grid = sm_count;
    const int nO = A.D / 8;
    auto plan = [&](int K, int &ks, int &kl) {
        ks = std::max(1, std::min(kFusedMaxKSplit, sm_count / std::max(1, nO)));
        kl = ((K + ks - 1) / ks + DH - 1) / DH * DH;  // whole heads for the attention rows
        ks = (K + kl - 1) / kl;
    };
    plan(A.D, A.ks_o, A.kl_o);
    plan(A.F, A.ks_2, A.kl_2);
    A.amax = std::max(A.D, A.F);
    // Attention chunks: a fixed number of KV blocks per chunk, chosen from the model and the device alone (one row of
    // max_seq tokens fills the grid once), so that a row's arithmetic does not depend on what else is in the batch.
    const int max_blocks = (A.max_seq + 15) / 16;
    A.cb = std::max(1, (max_blocks + std::max(1, sm_count / A.H) - 1) / std::max(1, sm_count / A.H));
    A.cb = std::max(A.cb, (max_blocks + kFusedMaxChunks - 1) / kFusedMaxChunks);
    const int nbk = std::min(max_blocks, (max_len + 15) / 16);
    A.nch = std::max(1, (nbk + A.cb - 1) / A.cb);
    A.scale_log2e = (1.0f / sqrtf((float)DH)) * 1.4426950408889634f;
    // LM head: as many of a CTA's column blocks as fit in 96 KB of shared memory are staged there during the last layer
    const int per_cta = (A.vocab / 8 + sm_count - 1) / sm_count;
    A.lm_stage = std::max(0, std::min(per_cta, (int)(96 * 1024 / (sizeof(float) * 8 * (size_t)A.D))));
}

int32_t launch_decode_fused(Ctx *ctx, FusedStepArgs &A) {
    // host-side fault injection for the tests: behave as a device that refuses the cooperative launch
    if (env_int("JGPT_B200_FUSED_REFUSE", 0)) return fail(JGPT_ERR_UNSUPPORTED, "cooperative launch refused (injected)");
    JGPT_REQUIRE(A.n >= 1 && A.n <= fused_step_max_rows() && A.steps >= 1, JGPT_ERR_INVALID_ARGUMENT, "fused decode step: %d rows, %d steps", A.n,
                 A.steps);
    JGPT_REQUIRE(A.D == A.H * DH && A.D % 8 == 0 && A.F % 8 == 0 && A.vocab % 8 == 0, JGPT_ERR_INVALID_ARGUMENT,
                 "fused decode step: unsupported geometry");
    if (A.n == 1) return launch_rows<1>(ctx, A);
    if (A.n == 2) return launch_rows<2>(ctx, A);
    return launch_rows<4>(ctx, A);
}

}  // namespace jgpt
