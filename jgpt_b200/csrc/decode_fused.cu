// One decode step of the whole model as ONE cooperative launch, for a handful of rows (interactive generation:
// GptAutoregressiveGenerator's loop, src/main/java/com/veles/llm/jgpt/model/GptAutoregressiveGenerator.java:108-206,
// decodes one row at a time).
//
// With 1-4 rows every kernel of the layer chain (norm + Q,K,V, attention, Wo, norm + W1/W3 + SwiGLU, W2) moves a few
// kilobytes per SM and lasts a few microseconds; a step of 63 dependent launches is then nothing but launch and
// drain latencies.  Here one grid of one CTA per SM walks the same chain, the CTAs meet at a counter in global
// memory between the phases (5 per layer), and everything a phase reads that does not depend on the previous one -
// its slice of the weights - is already on its way when the CTAs arrive at the counter.  The residual row lives in
// every CTA's shared memory (each CTA applies the same updates in the same order, so the copies stay bit-identical);
// the narrow projections (Wo, W2) are split over k and their partial rows are summed by the reader in a fixed
// order, so a step is deterministic.  Several steps can run in one launch (greedy generation: the argmax of one step
// is the input of the next), which also removes the host round trip between tokens.
//
// Arithmetic: plain fp32 FMA for the projections (a row-vector times a matrix has no tile for a tensor core), the
// attention as in attn_decode.cu: RoPE (adjacent pairs, apply_rope_4d_kernel) on q and on the appended k, K/V
// rounded to fp16 in the paged store, scores and softmax in fp32 in the log2 domain, split over the sequence.
//
// The CTAs wait for one another, so the launch is cooperative (all CTAs resident or the launch is refused), and
// every wait is bounded: a CTA that runs out of polls records DEV_STATUS_WAIT_TIMEOUT, raises the launch's abort
// word and leaves; the others see the word and leave too.
#include "common.cuh"
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
constexpr unsigned kPollLimit = 1u << 21;

__device__ __forceinline__ unsigned ld_acquire_u32(const unsigned *p) {
    unsigned v;
    asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(v) : "l"(p) : "memory");
    return v;
}

// All CTAs of the grid meet: the counter runs up by gridDim.x per meeting.  Returns false once the launch is aborted.
__device__ __forceinline__ bool grid_meet(const FusedStepArgs &A, unsigned &meetings, int *s_abort) {
    __syncthreads();
    if (threadIdx.x == 0) {
        const unsigned target = (++meetings) * gridDim.x;
        __threadfence();
        atomicAdd(A.sync_words, 1u);
        unsigned polls = 0;
        while (ld_acquire_u32(A.sync_words) < target) {
            if ((++polls & 255u) == 0u && ld_acquire_u32(A.sync_words + 2) != 0u) {
                *s_abort = 1;
                break;
            }
            if (polls > kPollLimit) {
                atomicOr(A.status, DEV_STATUS_WAIT_TIMEOUT);
                atomicExch(A.sync_words + 2, 1u);
                *s_abort = 1;
                break;
            }
        }
    } else {
        ++meetings;
    }
    __syncthreads();
    return *s_abort == 0;
}

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

// x[r][:] += p[0][r][:] + p[1][r][:] + ... (ks partial rows, summed in that order), rows < n.
template <int R>
__device__ __forceinline__ void add_partials(float *x, const float *p, int ks, int n, int D) {
    for (int e = threadIdx.x; e < n * D; e += kThreads) {
        float s = __ldcg(p + e);
        for (int j = 1; j < ks; j++) s += __ldcg(p + (size_t)j * R * D + e);
        x[e] += s;
    }
    __syncthreads();
}

// a[r][:] = x[r][:] * inv_rms(x[r]) * gamma  (rms_norm_fwd_block_kernel, jgpt_cuda_extra_kernels_launches.inl:694-713)
template <int R>
__device__ __forceinline__ void rms_norm_rows(const float *x, const float *gamma, float *a, int D, float eps, float *red) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    float ss[R];
#pragma unroll
    for (int r = 0; r < R; r++) {
        ss[r] = 0.f;
        for (int j = threadIdx.x; j < D; j += kThreads) ss[r] = fmaf(x[r * D + j], x[r * D + j], ss[r]);
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ss[r] += __shfl_xor_sync(0xffffffffu, ss[r], off);
        if (lane == 0) red[warp * R + r] = ss[r];
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < R; r++) {
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < kWarps; w++) s += red[w * R + r];
        const float rms = sqrtf(s / (float)D + eps);
        const float inv = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
        for (int j = threadIdx.x; j < D; j += kThreads) a[r * D + j] = x[r * D + j] * inv * __ldg(gamma + j);
    }
    __syncthreads();
}

// One (row, head, chunk) of the attention: RoPE on q, the new token appended by the chunk that owns its slot, a
// partial (maximum, sum, outputs) of this chunk's tokens left in `part`.
__device__ __forceinline__ void attention_unit(const FusedStepArgs &A, int layer, int r, int h, int c, int step, float *red) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n = A.n;
    const int seq = A.idx[2 * n + r], rp = A.idx[3 * n + r] + step, len = A.idx[4 * n + r] + step;
    const int nbk = (len + 15) >> 4;
    const int b0 = c * A.cb, b1 = min(nbk, b0 + A.cb);  // a row shorter than the launch's longest leaves chunks empty
    const int t0 = b0 * 16, t1 = min(len, b1 * 16);
    const float *row = A.qkv + (size_t)r * 3 * A.D;
    const float2 *cs = A.rope + (size_t)rp * (DH / 2);
    float q[DH];
#pragma unroll
    for (int j = 0; j < DH / 4; j++) {
        const float4 v = __ldcg(reinterpret_cast<const float4 *>(row + h * DH) + j);
        const float2 w0 = __ldg(cs + 2 * j), w1 = __ldg(cs + 2 * j + 1);
        q[4 * j] = __fsub_rn(__fmul_rn(v.x, w0.x), __fmul_rn(v.y, w0.y)) * A.scale_log2e;
        q[4 * j + 1] = __fadd_rn(__fmul_rn(v.x, w0.y), __fmul_rn(v.y, w0.x)) * A.scale_log2e;
        q[4 * j + 2] = __fsub_rn(__fmul_rn(v.z, w1.x), __fmul_rn(v.w, w1.y)) * A.scale_log2e;
        q[4 * j + 3] = __fadd_rn(__fmul_rn(v.z, w1.y), __fmul_rn(v.w, w1.x)) * A.scale_log2e;
    }
    float m = -INFINITY, l = 0.f, o[DH];
#pragma unroll
    for (int d = 0; d < DH; d++) o[d] = 0.f;
    const size_t layer_base = (size_t)layer * A.n_blocks;
    for (int tok = t0 + tid; tok < t1; tok += kThreads) {
        const int phys = __ldcg(A.table + (size_t)seq * A.mbs + (tok >> 4));
        if (phys < 0 || phys >= A.n_blocks) {
            atomicOr(A.status, DEV_STATUS_BAD_BLOCK);
            continue;
        }
        __half *kp = A.kv + ((layer_base + phys) * A.H + h) * (size_t)(2 * 16 * DH) + (size_t)(tok & 15) * DH;
        __align__(16) __half kh[DH], vh[DH];
        if (tok == len - 1) {  // the appended token: RoPE'd k and raw v, rounded to fp16, stored and scored from registers
            const float *kn = row + A.D + h * DH, *vn = row + 2 * A.D + h * DH;
#pragma unroll
            for (int j = 0; j < DH / 2; j++) {
                const float2 xk = __ldcg(reinterpret_cast<const float2 *>(kn) + j);
                const float2 xv = __ldcg(reinterpret_cast<const float2 *>(vn) + j);
                const float2 w = __ldg(cs + j);
                kh[2 * j] = __float2half_rn(__fsub_rn(__fmul_rn(xk.x, w.x), __fmul_rn(xk.y, w.y)));
                kh[2 * j + 1] = __float2half_rn(__fadd_rn(__fmul_rn(xk.x, w.y), __fmul_rn(xk.y, w.x)));
                vh[2 * j] = __float2half_rn(xv.x);
                vh[2 * j + 1] = __float2half_rn(xv.y);
            }
            reinterpret_cast<uint4 *>(kp)[0] = reinterpret_cast<const uint4 *>(kh)[0];
            reinterpret_cast<uint4 *>(kp)[1] = reinterpret_cast<const uint4 *>(kh)[1];
            reinterpret_cast<uint4 *>(kp + 16 * DH)[0] = reinterpret_cast<const uint4 *>(vh)[0];
            reinterpret_cast<uint4 *>(kp + 16 * DH)[1] = reinterpret_cast<const uint4 *>(vh)[1];
        } else {  // L1 is bypassed: in a launch of several steps another CTA wrote the rows of the earlier steps
            reinterpret_cast<uint4 *>(kh)[0] = __ldcg(reinterpret_cast<const uint4 *>(kp));
            reinterpret_cast<uint4 *>(kh)[1] = __ldcg(reinterpret_cast<const uint4 *>(kp) + 1);
            reinterpret_cast<uint4 *>(vh)[0] = __ldcg(reinterpret_cast<const uint4 *>(kp + 16 * DH));
            reinterpret_cast<uint4 *>(vh)[1] = __ldcg(reinterpret_cast<const uint4 *>(kp + 16 * DH) + 1);
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
    // merge: lanes of a warp, then the warps
    float M = m;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) M = fmaxf(M, __shfl_xor_sync(0xffffffffu, M, off));
    const float f = (m == -INFINITY) ? 0.f : exp2f(m - M);
    l *= f;
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) l += __shfl_xor_sync(0xffffffffu, l, off);
#pragma unroll
    for (int d = 0; d < DH; d++) {
        float v = o[d] * f;
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) v += __shfl_xor_sync(0xffffffffu, v, off);
        o[d] = v;
    }
    if (lane == 0) {
        float *w = red + warp * PS;
        w[0] = M, w[1] = l;
#pragma unroll
        for (int d = 0; d < DH; d++) w[2 + d] = o[d];
    }
    __syncthreads();
    if (tid < PS) {
        float Mx = -INFINITY;
#pragma unroll
        for (int w = 0; w < kWarps; w++) Mx = fmaxf(Mx, red[w * PS]);
        float *dst = A.part + (((size_t)r * A.H + h) * A.nch + c) * PS;
        if (tid == 0) {
            dst[0] = Mx;
        } else {
            float s = 0.f;
#pragma unroll
            for (int w = 0; w < kWarps; w++) {
                const float mw = red[w * PS];
                s = fmaf(red[w * PS + tid], mw == -INFINITY ? 0.f : exp2f(mw - Mx), s);
            }
            dst[tid] = s;
        }
    }
    __syncthreads();
}

// Merged attention output for model columns [k0, k1) of rows < n into a[r * lda + (k - k0)].
__device__ __forceinline__ void merge_attention(const FusedStepArgs &A, float *a, int lda, int k0, int k1) {
    const int span = k1 - k0;
    for (int e = threadIdx.x; e < A.n * span; e += kThreads) {
        const int r = e / span, k = k0 + e % span, h = k / DH, d = k % DH;
        const float *pp = A.part + (((size_t)r * A.H + h) * A.nch) * PS;
        float Mx = -INFINITY;
        for (int c = 0; c < A.nch; c++) Mx = fmaxf(Mx, __ldcg(pp + c * PS));
        float L = 0.f, acc = 0.f;
        for (int c = 0; c < A.nch; c++) {
            const float mc = __ldcg(pp + c * PS);
            const float w = mc == -INFINITY ? 0.f : exp2f(mc - Mx);
            L = fmaf(__ldcg(pp + c * PS + 1), w, L);
            acc = fmaf(__ldcg(pp + c * PS + 2 + d), w, acc);
        }
        a[r * lda + (k - k0)] = acc / fmaxf(L, 1e-12f);
    }
    __syncthreads();
}

template <int R>
__global__ void __launch_bounds__(kThreads, 1) decode_step_kernel(const FusedStepArgs A) {
    extern __shared__ __align__(16) float sm[];
    float *x = sm;                    // [R][D]  the residual rows
    float *a = x + R * A.D;           // [R][max(D, F)]  what the current projection multiplies
    float *red = a + R * A.amax;      // reductions
    __shared__ int s_abort;
    __shared__ int s_tok[R];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int b = blockIdx.x, G = gridDim.x, n = A.n, D = A.D, F = A.F;
    const int half_col = (tid & 1) * 4;
    if (tid == 0) s_abort = 0;
    for (int e = tid; e < R * D; e += kThreads) x[e] = 0.f;
    for (int e = tid; e < R * A.amax; e += kThreads) a[e] = 0.f;
    __syncthreads();
    unsigned meetings = 0;
    const int nA = 3 * D / 8, nO = D / 8, nD = F / 8, nL = A.vocab / 8;
    const int kso = A.ks_o, klo = A.kl_o, ks2 = A.ks_2, kl2 = A.kl_2;

    WTile t;
    bool have = false;
    auto load_A = [&](int l, int u) {  // unit u of the Q,K,V product: 8 columns of one of the three matrices
        const int z = u / nO, c0 = (u % nO) * 8;
        const float *W = z == 0 ? A.L[l].wq : (z == 1 ? A.L[l].wk : A.L[l].wv);
        tile_load<1>(t, W, nullptr, D, c0 + half_col, 0, D);
    };
    if (b < nA) load_A(0, b), have = true;

    int steps_done = 0;
    for (int step = 0; step < A.steps; step++) {
        // ---- embedding + learned position row (embedding_token_fwd_kernel + add_position_embedding_broadcast_kernel)
        for (int e = tid; e < n * D; e += kThreads) {
            const int r = e / D, j = e % D;
            const int id = step == 0 ? A.idx[r] : s_tok[r];
            const int pr = (A.idx[3 * n + r] + step) % A.max_seq;
            x[e] = __ldg(A.tok + (size_t)id * D + j) + __ldg(A.pos + (size_t)pr * D + j);
        }
        __syncthreads();

        for (int l = 0; l < A.layers; l++) {
            // ---- A: norm1 + Q,K,V
            if (l > 0) add_partials<R>(x, A.pw2, ks2, n, D);
            rms_norm_rows<R>(x, A.L[l].norm1, a, D, A.eps, red);
            for (int u = b; u < nA; u += G) {
                const int z = u / nO, c0 = (u % nO) * 8;
                const float *W = z == 0 ? A.L[l].wq : (z == 1 ? A.L[l].wk : A.L[l].wv);
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, have && u == b, W, nullptr, D, c0 + half_col, 0, D, a, D, 0, acc);
                unit_reduce<R, 1>(acc, red, res);
                if (warp == 0 && lane < R * 8 && (lane >> 3) < n) A.qkv[(size_t)(lane >> 3) * 3 * D + z * D + c0 + (lane & 7)] = res[0];
            }
            have = false;
            if (!grid_meet(A, meetings, &s_abort)) goto leave;

            // ---- B: append + attention partials
            for (int u = b; u < n * A.H * A.nch; u += G) {
                const int c = u % A.nch, h = (u / A.nch) % A.H, r = u / (A.nch * A.H);
                attention_unit(A, l, r, h, c, step, red);
            }
            if (b < nO * kso) {  // Wo: unit = 8 columns x one k range
                const int c0 = (b % nO) * 8, k0 = (b / nO) * klo;
                tile_load<1>(t, A.L[l].wo, nullptr, D, c0 + half_col, k0, min(D, k0 + klo));
                have = true;
            }
            if (!grid_meet(A, meetings, &s_abort)) goto leave;

            // ---- C: merged attention rows . Wo, partial rows per k range
            for (int u = b; u < nO * kso; u += G) {
                const int c0 = (u % nO) * 8, kj = u / nO, k0 = kj * klo, k1 = min(D, k0 + klo);
                merge_attention(A, a, klo, k0, k1);
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, have && u == b, A.L[l].wo, nullptr, D, c0 + half_col, k0, k1, a, klo, k0, acc);
                unit_reduce<R, 1>(acc, red, res);
                if (warp == 0 && lane < R * 8 && (lane >> 3) < n) A.po[((size_t)kj * R + (lane >> 3)) * D + c0 + (lane & 7)] = res[0];
            }
            have = false;
            if (b < nD) {
                tile_load<2>(t, A.L[l].w1, A.L[l].w3, F, b * 8 + half_col, 0, D);
                have = true;
            }
            if (!grid_meet(A, meetings, &s_abort)) goto leave;

            // ---- D: x += attention projection; norm2 + W1, W3 + SwiGLU (sigmoid_kernel / mul_kernel, same file :799-832)
            add_partials<R>(x, A.po, kso, n, D);
            rms_norm_rows<R>(x, A.L[l].norm2, a, D, A.eps, red);
            for (int u = b; u < nD; u += G) {
                float acc[2][R][4], res[2];
                unit_fma<R, 2>(t, have && u == b, A.L[l].w1, A.L[l].w3, F, u * 8 + half_col, 0, D, a, D, 0, acc);
                unit_reduce<R, 2>(acc, red, res);
                if (warp == 0 && lane < R * 8 && (lane >> 3) < n) {
                    const float gv = res[1];
                    float s;
                    if (gv >= 20.f) s = 1.f;
                    else if (gv <= -20.f) s = 0.f;
                    else s = 1.f / (1.f + expf(-gv));
                    A.act[(size_t)(lane >> 3) * F + u * 8 + (lane & 7)] = res[0] * (gv * s);
                }
            }
            have = false;
            if (b < nO * ks2) {
                const int c0 = (b % nO) * 8, k0 = (b / nO) * kl2;
                tile_load<1>(t, A.L[l].w2, nullptr, D, c0 + half_col, k0, min(F, k0 + kl2));
                have = true;
            }
            if (!grid_meet(A, meetings, &s_abort)) goto leave;

            // ---- E: activation . W2, partial rows per k range
            for (int u = b; u < nO * ks2; u += G) {
                const int c0 = (u % nO) * 8, kj = u / nO, k0 = kj * kl2, k1 = min(F, k0 + kl2);
                for (int e = tid; e < n * (k1 - k0); e += kThreads) {
                    const int r = e / (k1 - k0), k = e % (k1 - k0);
                    a[r * kl2 + k] = __ldcg(A.act + (size_t)r * F + k0 + k);
                }
                __syncthreads();
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, have && u == b, A.L[l].w2, nullptr, D, c0 + half_col, k0, k1, a, kl2, k0, acc);
                unit_reduce<R, 1>(acc, red, res);
                if (warp == 0 && lane < R * 8 && (lane >> 3) < n) A.pw2[((size_t)kj * R + (lane >> 3)) * D + c0 + (lane & 7)] = res[0];
            }
            have = false;
            if (l + 1 < A.layers) {
                if (b < nA) load_A(l + 1, b), have = true;
            } else if (b < nL) {
                tile_load<1>(t, A.lm_head, nullptr, A.vocab, b * 8 + half_col, 0, D);
                have = true;
            }
            if (!grid_meet(A, meetings, &s_abort)) goto leave;
        }

        // ---- final norm + LM head; every CTA keeps the best (value, lowest index) of its columns per row
        {
            add_partials<R>(x, A.pw2, ks2, n, D);
            rms_norm_rows<R>(x, A.norm_final, a, D, A.eps, red);
            float best = -INFINITY;
            int best_i = 0x7fffffff;
            if (!have && b < nL) tile_load<1>(t, A.lm_head, nullptr, A.vocab, b * 8 + half_col, 0, D);
            for (int u = b; u < nL; u += G) {
                WTile tn;  // the next unit's tile is on its way while this one is multiplied and reduced
                if (u + G < nL) tile_load<1>(tn, A.lm_head, nullptr, A.vocab, (u + G) * 8 + half_col, 0, D);
                float acc[1][R][4], res[1];
                unit_fma<R, 1>(t, true, A.lm_head, nullptr, A.vocab, u * 8 + half_col, 0, D, a, D, 0, acc);
                unit_reduce<R, 1>(acc, red, res);
                if (u + G < nL) t = tn;
                if (warp == 0 && lane < R * 8 && (lane >> 3) < n) {
                    const int col = u * 8 + (lane & 7);
                    A.logits[(size_t)(lane >> 3) * A.vocab + col] = res[0];
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
                if (lane < R * 8 && (lane & 7) == 0) {
                    A.cand_v[(size_t)b * R + (lane >> 3)] = best;
                    A.cand_i[(size_t)b * R + (lane >> 3)] = best_i;
                }
            }
            if (step + 1 < A.steps && b < nA) load_A(0, b), have = true;
            if (!grid_meet(A, meetings, &s_abort)) goto leave;
            // every CTA picks the tokens itself (the same comparison order everywhere): no further meeting
            if (warp < n) {
                float bv = -INFINITY;
                int bi = 0x7fffffff;
                for (int g = lane; g < G; g += 32) {
                    const float v = __ldcg(A.cand_v + (size_t)g * R + warp);
                    const int i = __ldcg(A.cand_i + (size_t)g * R + warp);
                    if (v > bv || (v == bv && i < bi)) bv = v, bi = i;
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
                    if (b == 0) A.next[(size_t)step * n + warp] = bi;
                }
            }
            __syncthreads();
            steps_done = step + 1;
            if (A.stop_on_zero && s_tok[0] == 0) break;
        }
    }
leave:
    __syncthreads();
    if (tid == 0) {
        if (b == 0) *A.steps_done = steps_done;
        __threadfence();
        // the last CTA to leave puts the meeting words back for the next launch
        if (atomicAdd(A.sync_words + 1, 1u) == (unsigned)G - 1u) {
            A.sync_words[0] = 0u, A.sync_words[1] = 0u, A.sync_words[2] = 0u;
            __threadfence();
        }
    }
}

template <int R>
static size_t fused_smem_bytes(const FusedStepArgs &A) {
    return sizeof(float) * ((size_t)R * A.D + (size_t)R * A.amax + (size_t)kWarps * 2 * 2 * R * 4 + kWarps * PS);
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
            JGPT_REQUIRE(coop, JGPT_ERR_CUDA, "device %d has no cooperative launch", ctx->device);
            JGPT_CUDA_TRY(cudaFuncSetAttribute(decode_step_kernel<R>, cudaFuncAttributeMaxDynamicSharedMemorySize, 64 * 1024));
            JGPT_CUDA_TRY(cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel<R>, kThreads, 64 * 1024));
            JGPT_REQUIRE(per_sm >= 1, JGPT_ERR_CUDA, "the fused decode step does not fit an SM");
            grid_for[ctx->device & 63] = ctx->sm_count;
            ready.insert(ctx->device);
        }
    }
    JGPT_REQUIRE(smem <= 64 * 1024, JGPT_ERR_INVALID_ARGUMENT, "model too wide for the fused decode step");
    const int G = grid_for[ctx->device & 63];
    JGPT_REQUIRE(G == A.grid, JGPT_ERR_ILLEGAL_STATE, "fused decode step sized for %d CTAs, device runs %d", A.grid, G);
    void *args[1] = {&A};
    JGPT_CUDA_TRY(cudaLaunchCooperativeKernel(reinterpret_cast<const void *>(decode_step_kernel<R>), dim3((unsigned)G), dim3(kThreads), args,
                                              smem, ctx->stream));
    return JGPT_OK;
}

}  // namespace

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
}

int32_t launch_decode_fused(Ctx *ctx, FusedStepArgs &A) {
    JGPT_REQUIRE(A.n >= 1 && A.n <= fused_step_max_rows() && A.steps >= 1, JGPT_ERR_INVALID_ARGUMENT, "fused decode step: %d rows, %d steps", A.n,
                 A.steps);
    JGPT_REQUIRE(A.D == A.H * DH && A.D % 8 == 0 && A.F % 8 == 0 && A.vocab % 8 == 0, JGPT_ERR_INVALID_ARGUMENT,
                 "fused decode step: unsupported geometry");
    if (A.n == 1) return launch_rows<1>(ctx, A);
    if (A.n == 2) return launch_rows<2>(ctx, A);
    return launch_rows<4>(ctx, A);
}

}  // namespace jgpt
