// Model weights on the device and the forward step around the attention kernels: embedding + learned
// positions, RMSNorm, fp32 projections, SwiGLU, LM head, greedy argmax / sampling, and the generation loop.
//
// Projections keep fp32 operands.  Default: tensor cores with split-TF32 operands (fp32-level accuracy; the
// reference runs the same GEMMs through cuBLAS under plain TF32 math,
// src/main/cpp/jgpt_cuda_jni_init_matmul.inl:67, 794, 892) - gemm_tc_small_kernel up to 512 rows (every decode
// step; RMSNorm, SwiGLU and the residual fused, the step replayed as a CUDA graph), the tcgen05 kernel of
// gemm_umma.cu above that (prefill).  JGPT_B200_STRICT_GEMM=1 selects a scalar kernel that accumulates every
// output element over k in ascending order in one thread (mul, then add), which is bit-reproducible against a
// scalar CPU loop.
#include "common.cuh"
#include "ptx.cuh"
#include "gemm_umma.cuh"

#include <algorithm>
#include <cmath>
#include <cstdio>
#include <unordered_map>

namespace jgpt {

struct Model {
    Ctx *ctx = nullptr;
    int vocab = 0, max_seq = 0, d_model = 0, heads = 0, layers = 0, d_ff = 0, max_rows = 0;
    float eps = 1e-5f;
    float *tok = nullptr, *pos = nullptr, *norm_final = nullptr, *lm_head = nullptr;
    std::vector<LayerW> L;
    float *arena = nullptr;  // the layers' tensors, one allocation
    size_t arena_floats = 0;
    bool l2_window = false;  // the context's stream carries an L2 access-policy window over the arena
    // workspace for up to max_rows rows
    float *x = nullptr, *xn = nullptr, *q = nullptr, *k = nullptr, *v = nullptr, *att = nullptr, *h1 = nullptr, *g = nullptr;
    float *logits = nullptr;  // [logit_rows, vocab]
    int logit_rows = 0;
    int *d_idx = nullptr;     // [5][max_rows]: ids, pos rows, seq ids, rope pos, lens
    int *h_idx = nullptr;     // pinned mirror
    int *d_next = nullptr;    // [max_rows] argmax
    int *h_next = nullptr;    // pinned
    int *d_rowsel = nullptr;  // [max_rows] rows whose logits are wanted
    int strict = 0;           // 0: tensor-core 3xTF32 projections; 1: k-ordered scalar fp32 (mul + add, two roundings)
    // Prefill-sized products (M >= umma_min_rows) run on the tcgen05 kernel over pre-tiled operand images.
    int umma_min_rows = 513;  // JGPT_B200_UMMA_MIN_ROWS; 0: never
    std::unordered_map<const float *, float *> wimg;   // weight images by source pointer; dropped when weights change
    std::unordered_map<const float *, float *> wpair;  // W1/W3 pair images by W1's pointer
    float *aimg = nullptr, *aimg2 = nullptr;  // activation images (grow-only): [rows, d_model]-sized and [rows, d_ff]-sized
    uint64_t aimg_floats = 0, aimg2_floats = 0;
    // Decode-sized steps (rows <= 512): RMSNorm and SwiGLU live inside the projections.
    float *ss_a = nullptr, *ss_b = nullptr;           // [max_rows][ceil(d_model / 32)] partial row sums of squares of x
    std::unordered_map<const float *, float *> w13i;  // interleaved W1/W3 pairs by W1's pointer; dropped when weights change
    std::unordered_map<const float *, float *> wscaled;  // weights with row k scaled by the preceding norm's gamma[k] (decode-sized steps), by the weights' pointer
    // Decode steps replayed as CUDA graphs (JGPT_B200_DECODE_GRAPH=0 turns it off).  A step's launches depend on
    // the batch size, on the attention's length bucket and on the addresses of every buffer involved; all of that
    // is the key.  A key seen for the second time is captured, from then on replayed.
    struct DecodeGraph {
        const void *key[8] = {};
        int n = 0, len_bucket = 0, geom[5] = {};
        float temperature = 0.f;  // 0: greedy argmax
        int top_k = 0;
        cudaGraphExec_t exec = nullptr;
        bool failed = false;  // capture refused once (an allocation or a synchronisation inside): stay eager
        uint64_t last_use = 0;
    };
    // on-device sampling: per-row uniform draws (pinned + device) and the [rows, vocab] work area of sample_kernel
    float *h_u = nullptr, *d_u = nullptr, *d_samp = nullptr;
    int samp_rows = 0;
    std::vector<DecodeGraph> decode_graphs;
    uint64_t decode_graph_clock = 0;
    int decode_graph_enabled = 1;
    bool first_launch_early = false;  // set while a decode step is enqueued: its embedding kernel lets layer 0's Q,K,V product move in early
    int k_split = 1;  // Wo / W2 of a step with few rows as pairs of CTAs that split the k range (JGPT_B200_K_SPLIT=0: off)
    int w_resident = 1;  // projections of the decode step keep their CTA's weight slice in shared memory when the grid allows (JGPT_B200_W_RESIDENT=0: off)
    int step_overlap = -1;  // programmatic dependent launches inside the decode step (JGPT_B200_STEP_OVERLAP 0..3; -1 = the default, 3)
    int prefill_fast = 1;  // single-fp16 q / p operands in the d_head-16 prefill attention (JGPT_B200_PREFILL_EXACT=1: off)
    // Steps of up to four rows as one cooperative launch (decode_fused.cu; JGPT_B200_FUSED_STEP=0: off).  Sized on first use.
    int fused_step = 1;
    uint2 *f_pairs = nullptr;   // exchange buffers of (value, stamp) pairs: qkv, attention partials, projection partials, ...
    uint64_t f_pairs_n = 0;
    uint32_t f_stamp = 0;       // stamps handed out so far; a launch uses f_stamp + 1 ... f_stamp + steps * layers
    int *f_ints = nullptr;      // tokens of a multi-step launch, steps done, abort word
    int *h_fused = nullptr;     // pinned: [kFusedMaxSteps * 4] tokens + steps done
    int *hd_idx = nullptr, *hd_status = nullptr;  // device-side addresses of h_idx and of the context's status mirror (decode step without copies)
    int *hd_fused = nullptr, *hd_next = nullptr;  // device-side addresses of h_fused and h_next: the kernel writes its results there itself
    // The same for batches (decode_batch.cu; JGPT_B200_FUSED_BATCH=1: on): rows 5 .. fused_batch_rows
    int fused_batch = 0;
    int fused_batch_rows = 0;   // rows the buffers below are sized for
    uint2 *fb_pairs = nullptr;
    uint64_t fb_pairs_n = 0;
    uint2 *fb_part = nullptr;
    int *fb_tickets = nullptr;
};
constexpr int kFusedBatchMaxRows = 256;
constexpr int kFusedMaxSteps = 256;  // greedy steps one launch runs at most

static void drop_decode_graphs(Model *m) {
    for (auto &g : m->decode_graphs)
        if (g.exec) cudaGraphExecDestroy(g.exec);
    m->decode_graphs.clear();
}

static void drop_weight_images(Model *m) {
    drop_decode_graphs(m);  // they hold the addresses freed below
    for (auto &kv : m->wimg) cudaFree(kv.second);
    for (auto &kv : m->wpair) cudaFree(kv.second);
    for (auto &kv : m->w13i) cudaFree(kv.second);
    for (auto &kv : m->wscaled) cudaFree(kv.second);
    m->wimg.clear(), m->wpair.clear(), m->w13i.clear(), m->wscaled.clear();
}

Registry<Model> &model_registry() {
    static Registry<Model> r;
    return r;
}

// ------------------------------------------------------------------------------------------------
// Kernels
// ------------------------------------------------------------------------------------------------

// x[r,:] = tok[id[r],:] + pos[posrow[r],:]   (embedding_token_fwd_kernel + add_position_embedding_broadcast_kernel,
// src/main/cpp/jgpt_cuda_extra_kernels_launches.inl:937-955, 1020-1032)
// With idx_host (the decode step): the step's five per-row words (id, position row, sequence, RoPE position, length; stride
// R) are read from the caller's page-locked host block by the row's own CTA and left in idx_dev for the attention launches:
// 5 n words instead of a copy of the whole 5 R block ahead of the step.
__global__ void __launch_bounds__(128) embed_pos_kernel(const float *__restrict__ tok, const float *__restrict__ pos,
                                                        const int *__restrict__ ids, const int *__restrict__ posrow,
                                                        float *__restrict__ x, int D, float *__restrict__ ss_out,
                                                        const int *idx_host = nullptr, int *idx_dev = nullptr, int R = 0) {
    __shared__ float red[4];
    __shared__ int s_word[5];
    const int r = blockIdx.x;
    griddep_launch_dependents();  // a successor launched as a programmatic dependent may move in (it waits for this kernel itself)
    int id, prow;
    if (idx_host) {
        if (threadIdx.x < 5) {
            const int w = idx_host[(size_t)threadIdx.x * R + r];
            idx_dev[(size_t)threadIdx.x * R + r] = w;
            s_word[threadIdx.x] = w;
        }
        __syncthreads();
        id = s_word[0], prow = s_word[1];
    } else {
        id = ids[r], prow = posrow[r];
    }
    const float4 *t = reinterpret_cast<const float4 *>(tok + (size_t)id * D);
    const float4 *p = reinterpret_cast<const float4 *>(pos + (size_t)prow * D);
    float4 *o = reinterpret_cast<float4 *>(x + (size_t)r * D);
    float ss = 0.f;
    for (int j = threadIdx.x; j < D / 4; j += blockDim.x) {
        const float4 a = t[j], b = p[j];
        const float4 v = make_float4(a.x + b.x, a.y + b.y, a.z + b.z, a.w + b.w);
        o[j] = v;
        ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
    }
    // sum of squares of the row (one partial): what the first fused RMSNorm of the decode-sized path consumes
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    if (threadIdx.x == 0) ss_out[r] = red[0] + red[1] + red[2] + red[3];
}

// RMSNorm, one block per row (rms_norm_fwd_block_kernel, same file :694-713):
// rms = sqrtf(sum(x^2)/D + eps); inv = (rms > 0 && finite) ? 1/rms : 0; y = x * inv * gamma.
__global__ void __launch_bounds__(128) rmsnorm_kernel(const float *__restrict__ x, const float *__restrict__ gamma,
                                                      float *__restrict__ y, int D, float eps) {
    __shared__ float red[4];
    const float *xr = x + (size_t)blockIdx.x * D;
    float ss = 0.f;
    for (int j = threadIdx.x; j < D; j += blockDim.x) ss += xr[j] * xr[j];
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
    __syncthreads();
    ss = red[0] + red[1] + red[2] + red[3];
    const float rms = sqrtf(ss / (float)D + eps);
    const float inv = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
    float *yr = y + (size_t)blockIdx.x * D;
    for (int j = threadIdx.x; j < D; j += blockDim.x) yr[j] = xr[j] * inv * gamma[j];
}

// act = h1 * (g * sigmoid(g)), sigmoid clamped to 1 / 0 at |g| >= 20 (sigmoid_kernel :799-815, mul_kernel :832).
__global__ void __launch_bounds__(256) swiglu_kernel(float *__restrict__ h1, const float *__restrict__ g, long long n) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    const float gv = g[i];
    float s;
    if (gv >= 20.f) s = 1.f;
    else if (gv <= -20.f) s = 0.f;
    else s = 1.f / (1.f + expf(-gv));
    h1[i] = h1[i] * (gv * s);
}

// Up to three products sharing A in one launch: C_z[M,N] = A[M,K] . W_z[K,N] (+ R_z), z = blockIdx.z.
// Row-major fp32; every C element is accumulated over k = 0..K-1 in order by one thread.
struct GemmBatch {
    const float *W[3];
    float *C[3];
    const float *R[3];  // optional residual added after the accumulation
};

template <int BM, int BN, int TM, int TN, bool STRICT>
__global__ void __launch_bounds__((BM / TM) * (BN / TN)) gemm_kernel(const float *__restrict__ A, const GemmBatch B, int M, int K,
                                                                     int N, const int *__restrict__ rowsel) {
    constexpr int BK = 16;
    constexpr int NT = (BM / TM) * (BN / TN);
    __shared__ float As[BK][BM + 1];
    __shared__ __align__(16) float Ws[BK][BN];
    const float *__restrict__ W = B.W[blockIdx.z];
    float *C = B.C[blockIdx.z];        // C and R may be the same buffer (x += A.W): each element is read
    const float *R = B.R[blockIdx.z];  // and then written by the one thread that owns it
    const int tid = threadIdx.x;
    const int tx = tid % (BN / TN), ty = tid / (BN / TN);
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; i++)
#pragma unroll
        for (int j = 0; j < TN; j++) acc[i][j] = 0.f;

    for (int k0 = 0; k0 < K; k0 += BK) {
        for (int e = tid; e < BM * BK; e += NT) {
            const int r = e / BK, kk = e % BK;
            const int m = m0 + r;
            float val = 0.f;
            if (m < M && k0 + kk < K) {
                const int src_row = rowsel ? rowsel[m] : m;
                val = A[(size_t)src_row * K + k0 + kk];
            }
            As[kk][r] = val;
        }
        for (int e = tid; e < BK * BN; e += NT) {
            const int kk = e / BN, c = e % BN;
            Ws[kk][c] = (k0 + kk < K && n0 + c < N) ? W[(size_t)(k0 + kk) * N + n0 + c] : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; kk++) {
            float a[TM], w[TN];
#pragma unroll
            for (int i = 0; i < TM; i++) a[i] = As[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; j++) w[j] = Ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; i++)
#pragma unroll
                for (int j = 0; j < TN; j++) {
                    if (STRICT) acc[i][j] = __fadd_rn(acc[i][j], __fmul_rn(a[i], w[j]));
                    else acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < TM; i++) {
        const int m = m0 + ty * TM + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < TN; j++) {
            const int n = n0 + tx * TN + j;
            if (n >= N) continue;
            float val = acc[i][j];
            if (R) val = __fadd_rn(R[(size_t)m * N + n], val);
            C[(size_t)m * N + n] = val;
        }
    }
}

// ------------------------------------------------------------------------------------------------
// Tensor-core projections with fp32-level accuracy ("3xTF32"): each fp32 operand is split into a TF32
// high part and a TF32 low part, and C += Ah.Bh + Ah.Bl + Al.Bh with fp32 accumulation
// (mma.sync m16n8k8).  The dropped Al.Bl term and the truncation of the low parts are ~2^-21 relative,
// i.e. the result differs from a k-ordered fp32 loop by rounding noise only, where plain TF32 (what the
// reference runs its cuBLAS GEMMs with) is ~2^-11.  A tile: BM x 32 (row major, stride 36 floats),
// W tile: 32 x BN (stride BN + 8): both fragment loads are bank-conflict free.  Multi-stage cp.async ring.
// ------------------------------------------------------------------------------------------------
// 128 threads = 4 warps laid out WARPS_M x WARPS_N over the BM x BN tile; needs K % 4 == 0 and N % 4 == 0.
template <int BM, int BN, int STAGES>
constexpr size_t gemm_tc_smem_bytes() { return sizeof(float) * (size_t)STAGES * (BM * (32 + 4) + 32 * (BN + 8)); }

template <int BM, int BN, int WARPS_M, int WARPS_N, int STAGES>
__global__ void __launch_bounds__(128) gemm_tc_kernel(const float *__restrict__ A, const GemmBatch B, int M, int K, int N,
                                                      const int *__restrict__ rowsel) {
    constexpr int BK = 32, AS = BK + 4, WS = BN + 8;
    constexpr int WM = BM / WARPS_M, WN = BN / WARPS_N;  // warp tile
    constexpr int MT = WM / 16, NT = WN / 8;
    static_assert(WARPS_M * WARPS_N == 4 && WM % 16 == 0 && WN % 8 == 0 && STAGES >= 2, "bad tile configuration");
    // STAGES k-tiles in flight: at decode sizes the whole product is a handful of tiles, so the kernel's time
    // is one memory latency plus the MMAs instead of one latency per tile.
    extern __shared__ __align__(16) float gemm_smem[];
    float (*As)[BM][AS] = reinterpret_cast<float (*)[BM][AS]>(gemm_smem);
    float (*Ws)[BK][WS] = reinterpret_cast<float (*)[BK][WS]>(gemm_smem + (size_t)STAGES * BM * AS);
    const float *__restrict__ W = B.W[blockIdx.z];
    float *C = B.C[blockIdx.z];
    const float *R = B.R[blockIdx.z];
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int wm = warp / WARPS_N, wn = warp % WARPS_N;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;

    auto load_tiles = [&](int buf, int k0) {
        for (int e = tid; e < BM * (BK / 4); e += 128) {  // A: BM rows x 8 chunks of 4 floats
            const int r = e / (BK / 4), c4 = (e % (BK / 4)) * 4;
            const int m = m0 + r;
            const bool ok = m < M && k0 + c4 < K;
            const int src_row = ok ? (rowsel ? rowsel[m] : m) : 0;
            cp_async16(&As[buf][r][c4], A + (size_t)src_row * K + (ok ? k0 + c4 : 0), ok);
        }
        for (int e = tid; e < BK * (BN / 4); e += 128) {  // W: 32 rows x BN/4 chunks
            const int kk = e / (BN / 4), c4 = (e % (BN / 4)) * 4;
            const bool ok = k0 + kk < K && n0 + c4 < N;
            cp_async16(&Ws[buf][kk][c4], W + (ok ? (size_t)(k0 + kk) * N + n0 + c4 : 0), ok);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    // Two accumulators per output tile: the big term (Ah.Bh) and the two correction terms.  They are summed in
    // the epilogue; keeping them apart shortens the dependent MMA chain per k-tile from 12 to 8 / 4 instructions.
    float acc[MT][NT][4], cor[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f, cor[i][j][e] = 0.f;

    const int nk = (K + BK - 1) / BK;
    // Prologue: STAGES-1 tiles in flight.  Every iteration commits exactly one group (an empty one past the
    // end), so "all but the newest STAGES-2 groups are complete" always means "tile kt has landed".
#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < nk) load_tiles(s, s * BK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
    }
    for (int kt = 0; kt < nk; kt++) {
        const int buf = kt % STAGES;
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();  // tile kt visible to all; everyone is done with the buffer refilled below (read at kt-1)
        if (kt + STAGES - 1 < nk) load_tiles((kt + STAGES - 1) % STAGES, (kt + STAGES - 1) * BK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
#pragma unroll
        for (int ks = 0; ks < BK; ks += 8) {
            uint32_t ah[MT][4], al[MT][4];
#pragma unroll
            for (int i = 0; i < MT; i++) {
                const int r = wm * WM + i * 16 + g;
                split_tf32(As[buf][r][ks + t], ah[i][0], al[i][0]);
                split_tf32(As[buf][r + 8][ks + t], ah[i][1], al[i][1]);
                split_tf32(As[buf][r][ks + t + 4], ah[i][2], al[i][2]);
                split_tf32(As[buf][r + 8][ks + t + 4], ah[i][3], al[i][3]);
            }
#pragma unroll
            for (int j = 0; j < NT; j++) {
                const int c = wn * WN + j * 8 + g;
                uint32_t bh0, bl0, bh1, bl1;
                split_tf32(Ws[buf][ks + t][c], bh0, bl0);
                split_tf32(Ws[buf][ks + t + 4][c], bh1, bl1);
#pragma unroll
                for (int i = 0; i < MT; i++) {
                    mma_tf32(cor[i][j], al[i], bh0, bh1);
                    mma_tf32(acc[i][j], ah[i], bh0, bh1);
                    mma_tf32(cor[i][j], ah[i], bl0, bl1);
                }
            }
        }
    }
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < NT; j++) {
            const int n = n0 + wn * WN + j * 8 + 2 * t;
            if (n >= N) continue;
#pragma unroll
            for (int hrow = 0; hrow < 2; hrow++) {
                const int m = m0 + wm * WM + i * 16 + g + hrow * 8;
                if (m >= M) continue;
                float2 val = make_float2(acc[i][j][2 * hrow] + cor[i][j][2 * hrow], acc[i][j][2 * hrow + 1] + cor[i][j][2 * hrow + 1]);
                if (R) {
                    const float2 r2 = *reinterpret_cast<const float2 *>(R + (size_t)m * N + n);
                    val.x += r2.x, val.y += r2.y;
                }
                *reinterpret_cast<float2 *>(C + (size_t)m * N + n) = val;
            }
        }
}

// Decode-sized M (a few rows of 16): the product is a chain of dependent steps, so the kernel is built for a
// short chain, not for throughput.  CTA tile 16 x 32, eight warps: every warp covers the whole tile (four
// independent accumulator pairs) but only its own 8-wide slice of each 64-wide k tile, so a warp issues an
// eighth of the fragment loads, splits and MMAs of the k loop; the eight partial tiles are added in warp
// order through shared memory (deterministic) in front of the residual epilogue.
constexpr int kSmallBK = 64;
template <int STAGES, int MT = 1>
__host__ __device__ constexpr size_t gemm_small_smem_bytes() { return sizeof(float) * (size_t)STAGES * (16 * MT * (kSmallBK + 4) + kSmallBK * (32 + 8)); }

//
// Fusions of the decode step (template flags):
//   NORM  the product is that of the RMS-normalised rows, y = (x * inv * gamma) W, computed as inv * (x (gamma W)):
//         W is the caller's copy of the weights with row k scaled by gamma[k] (scaled_weight), and the row factor inv
//         -- from the row's sum of squares, which the PRODUCER of x has left as `parts_in` partial sums per row (added in
//         ascending order: deterministic) -- is applied to the finished sums.  Normalising every A fragment inside the k
//         loop instead cost 1.3 us per launch (5.4 against 4.1 us for the Q,K,V product at batch 64): the loop could not
//         start before inv was known and carried two multiplies per fragment.
//   EPI 1 the epilogue also writes the sum of squares of its 32 output columns of every row (one partial per
//         column tile) for the next NORM.
//   EPI 2 W is a W1/W3 pair interleaved in groups of 16 columns; the epilogue writes h1 * g * sigmoid(g)
//         (16 columns of [M, N / 2]), sigmoid clamped to 1 / 0 at |g| >= 20 like swiglu_kernel.
struct SmallFuse {
    const float *gamma, *ss_in;
    float *ss_out;
    int parts_in;
    float eps;
    // Programmatic dependent launch.  bit 0: this launch carries the attribute, i.e. it may have started before the
    // previous kernel on the stream finished: wait for that kernel before touching memory.  bit 1: let the NEXT
    // launch on the stream move in early (it waits for this kernel itself before it reads this kernel's output).
    int pdl = 0;
    // 1: the launch's shared memory holds this CTA's whole weight slice (every k tile its own stage, none reused):
    // all of it is requested at the top of the kernel -- one trip to memory instead of one per STAGES - 1 tiles.
    int w_resident = 0;
    // 2 (EPI 1 only): the launch is made of clusters of two CTAs along x that share one output tile; each runs half of the
    // k tiles, the second hands its sums to the first through shared memory, the first adds them to its own (k halves in
    // order), then the residual, and stores.  For the Wo / W2 products of a step with few rows: 48 CTAs on 148 SMs otherwise.
    int k_split = 1;
#ifdef JGPT_B200_DECODE_TRACE
    Timeline timeline;
#endif
};

// MT = 2: 32-row tiles (two MMA row blocks per warp share every weight fragment) for the larger decode batches.
template <int STAGES, bool NORM, int EPI, int MT = 1>
__global__ void __launch_bounds__(256) gemm_tc_small_kernel(const float *__restrict__ A, const GemmBatch B, int M, int K, int N,
                                                            const int *__restrict__ rowsel, const SmallFuse F) {
    constexpr int BM = 16 * MT, BN = 32, BK = kSmallBK, AS = BK + 4, WS = BN + 8;
    static_assert(STAGES >= 2 && sizeof(float) * 8 * BM * (BN + 1) <= gemm_small_smem_bytes<STAGES, MT>(), "reduction buffer must fit");
    extern __shared__ __align__(16) float gemm_smem[];
    float (*As)[BM][AS] = reinterpret_cast<float (*)[BM][AS]>(gemm_smem);
    float (*Ws)[BK][WS] = reinterpret_cast<float (*)[BK][WS]>(gemm_smem + (size_t)STAGES * BM * AS);
    const int z = blockIdx.z;  // selects below: indexing B would copy it to local memory
    const float *__restrict__ W = z == 0 ? B.W[0] : (z == 1 ? B.W[1] : B.W[2]);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int k_split = (EPI == 1 && F.k_split == 2) ? 2 : 1;
    const int k_part = k_split == 2 ? (int)(blockIdx.x & 1) : 0, col_tile = k_split == 2 ? (int)(blockIdx.x >> 1) : (int)blockIdx.x;
    const int m0 = blockIdx.y * BM, n0 = col_tile * BN;
#ifdef JGPT_B200_DECODE_TRACE
    timeline_in(F.timeline);
#endif
    // weight tiles do not depend on the previous kernel either: a launch that moved in early requests the first
    // STAGES - 1 of them before it waits (they join the first committed group below)
    const int w_k = tid >> 3, w_c = (tid & 7) * 4;  // second chunk: k + 32
    const bool w_col_ok = n0 + w_c < N;
    const float *w_src = W + (size_t)w_k * N + (w_col_ok ? n0 + w_c : 0);
    auto load_w = [&](int buf, int k0) {
        const bool k1 = w_col_ok && k0 + w_k < K, k2 = w_col_ok && k0 + w_k + 32 < K;
        cp_async16(&Ws[buf][w_k][w_c], k1 ? w_src + (size_t)k0 * N : W, k1);
        cp_async16(&Ws[buf][w_k + 32][w_c], k2 ? w_src + (size_t)(k0 + 32) * N : W, k2);
    };
    const int nk_all = (K + BK - 1) / BK;
    const int kt_first = k_part * nk_all / k_split, nk = (k_part + 1) * nk_all / k_split - kt_first;  // this CTA's k tiles
    const int kbase = kt_first * BK;
    const bool w_resident = F.w_resident != 0;
    const bool early_w = (F.pdl & 1) != 0 || w_resident;
    if (w_resident) {
        for (int kt = 0; kt < nk; kt++) load_w(kt, kbase + kt * BK);
    } else if (early_w) {
#pragma unroll
        for (int s = 0; s < STAGES - 1; s++)
            if (s < nk) load_w(s, kbase + s * BK);
    }
    if (F.pdl & 1) griddep_wait();
#ifdef JGPT_B200_DECODE_TRACE
    timeline_at(F.timeline, 1);
#endif
    if (F.pdl & 2) griddep_launch_dependents();  // the whole grid is resident: the next launch cannot get in its way

    // this thread's copy slots of A: MT 16-byte chunks (rows a_r, a_r + 16)
    const int a_r = tid >> 4, a_c = (tid & 15) * 4;
    bool a_row_ok[MT];
    const float *a_src[MT];
#pragma unroll
    for (int i = 0; i < MT; i++) {
        a_row_ok[i] = m0 + a_r + 16 * i < M;
        a_src[i] = A + (size_t)(a_row_ok[i] ? (rowsel ? rowsel[m0 + a_r + 16 * i] : m0 + a_r + 16 * i) : 0) * K + a_c;
    }
    auto load_a = [&](int buf, int k0) {
#pragma unroll
        for (int i = 0; i < MT; i++) {
            const bool ak = a_row_ok[i] && k0 + a_c < K;
            cp_async16(&As[buf][a_r + 16 * i][a_c], ak ? a_src[i] + k0 : A, ak);
        }
    };
    auto load_tiles = [&](int buf, int k0) {
        load_a(buf, k0);
        if (!w_resident) load_w(buf, k0);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[MT][4][4], cor[MT][4][4];
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++)
#pragma unroll
            for (int e = 0; e < 4; e++) acc[i][j][e] = 0.f, cor[i][j][e] = 0.f;

#pragma unroll
    for (int s = 0; s < STAGES - 1; s++) {
        if (s < nk) {
            load_a(s, kbase + s * BK);
            if (!early_w) load_w(s, kbase + s * BK);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    }
    // the residual elements this thread adds in the epilogue, requested now so that they do not cost a round trip then
    const float *Rz = z == 0 ? B.R[0] : (z == 1 ? B.R[1] : B.R[2]);
    float rpre[2 * MT];
#pragma unroll
    for (int i = 0; i < 2 * MT; i++) {
        const int e = tid + 256 * i, m = m0 + (e >> 5), n = n0 + (e & 31);
        rpre[i] = (EPI != 2 && Rz && k_part == 0 && m < M && n < N) ? Rz[(size_t)m * N + n] : 0.f;
    }
    __shared__ float s_inv[BM];
    __shared__ float s_xch[EPI == 1 ? BM * BN : 1];  // k_split: the partner CTA's sums land here (never part of the tile ring)
    if (NORM && tid < BM) {
        const int m = m0 + tid;
        float inv = 0.f;
        if (m < M) {
            const float *pp = F.ss_in + (size_t)(rowsel ? rowsel[m] : m) * F.parts_in;
            float tot = 0.f;
            if (F.parts_in <= 16) {  // all partials requested before the first is added (same order of additions)
                float pv[16];
#pragma unroll
                for (int i = 0; i < 16; i++) pv[i] = i < F.parts_in ? pp[i] : 0.f;
#pragma unroll
                for (int i = 0; i < 16; i++)
                    if (i < F.parts_in) tot += pv[i];
            } else {
                for (int i = 0; i < F.parts_in; i++) tot += pp[i];
            }
            const float rms = sqrtf(tot / (float)K + F.eps);
            inv = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
        }
        s_inv[tid] = inv;
    }
    const int ks = warp * 8;
    for (int kt = 0; kt < nk; kt++) {
        const int buf = kt % STAGES, wbuf = w_resident ? kt : buf;
        asm volatile("cp.async.wait_group %0;" ::"n"(STAGES - 2) : "memory");
        __syncthreads();  // tile kt (and s_inv) visible to all; everyone is done with the buffer refilled below (read at kt-1)
        if (kt + STAGES - 1 < nk) load_tiles((kt + STAGES - 1) % STAGES, kbase + (kt + STAGES - 1) * BK);
        else asm volatile("cp.async.commit_group;" ::: "memory");
        uint32_t ah[MT][4], al[MT][4];
#pragma unroll
        for (int i = 0; i < MT; i++) {
            const int r = 16 * i + g;
            float a0 = As[buf][r][ks + t], a1 = As[buf][r + 8][ks + t], a2 = As[buf][r][ks + t + 4], a3 = As[buf][r + 8][ks + t + 4];
            split_tf32(a0, ah[i][0], al[i][0]);
            split_tf32(a1, ah[i][1], al[i][1]);
            split_tf32(a2, ah[i][2], al[i][2]);
            split_tf32(a3, ah[i][3], al[i][3]);
        }
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int c = j * 8 + g;
            uint32_t bh0, bl0, bh1, bl1;
            split_tf32(Ws[wbuf][ks + t][c], bh0, bl0);
            split_tf32(Ws[wbuf][ks + t + 4][c], bh1, bl1);
#pragma unroll
            for (int i = 0; i < MT; i++) {
                mma_tf32(cor[i][j], al[i], bh0, bh1);
                mma_tf32(acc[i][j], ah[i], bh0, bh1);
                mma_tf32(cor[i][j], ah[i], bl0, bl1);
            }
        }
    }
    asm volatile("cp.async.wait_group 0;" ::: "memory");
    __syncthreads();  // the stage buffers are dead: reuse them for the eight partial tiles
#ifdef JGPT_B200_DECODE_TRACE
    timeline_at(F.timeline, 3);
#endif
    float (*red)[BM][BN + 1] = reinterpret_cast<float (*)[BM][BN + 1]>(gemm_smem);
#pragma unroll
    for (int i = 0; i < MT; i++)
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const int r = 16 * i + g;
            red[warp][r][j * 8 + 2 * t] = acc[i][j][0] + cor[i][j][0];
            red[warp][r][j * 8 + 2 * t + 1] = acc[i][j][1] + cor[i][j][1];
            red[warp][r + 8][j * 8 + 2 * t] = acc[i][j][2] + cor[i][j][2];
            red[warp][r + 8][j * 8 + 2 * t + 1] = acc[i][j][3] + cor[i][j][3];
        }
    __syncthreads();
    float *C = z == 0 ? B.C[0] : (z == 1 ? B.C[1] : B.C[2]);
    const float *R = z == 0 ? B.R[0] : (z == 1 ? B.R[1] : B.R[2]);
    for (int e = tid; EPI == 2 && e < BM * 16; e += 256) {
        const int r = e >> 4, c = e & 15, m = m0 + r, n = col_tile * 16 + c, Fo = N / 2;
        if (m < M && n < Fo) {
            float h = red[0][r][c], gv = red[0][r][16 + c];
#pragma unroll
            for (int w = 1; w < 8; w++) h += red[w][r][c], gv += red[w][r][16 + c];
            if (NORM) h *= s_inv[r], gv *= s_inv[r];
            float sg;
            if (gv >= 20.f) sg = 1.f;
            else if (gv <= -20.f) sg = 0.f;
            else sg = 1.f / (1.f + expf(-gv));
            C[(size_t)m * Fo + n] = h * (gv * sg);
        }
    }
    float vsum[2 * MT];
#pragma unroll
    for (int i = 0; EPI != 2 && i < 2 * MT; i++) {  // one warp = one row of the tile per iteration
        const int e = tid + 256 * i, r = e >> 5, c = e & 31;
        float v = red[0][r][c];
#pragma unroll
        for (int w = 1; w < 8; w++) v += red[w][r][c];
        vsum[i] = NORM ? v * s_inv[r] : v;
    }
    if (EPI == 1 && k_split == 2) {
        // the second CTA of the pair puts its sums into the first one's shared memory (behind the partial tiles) and is done
        float *xch = s_xch;
        if (k_part == 1) {
#pragma unroll
            for (int i = 0; i < 2 * MT; i++) st_cluster_f32(xch + tid + 256 * i, 0u, vsum[i]);
        }
        cluster_sync();
        if (k_part == 1) {
#ifdef JGPT_B200_DECODE_TRACE
            timeline_at(F.timeline, 2);
#endif
            return;
        }
#pragma unroll
        for (int i = 0; i < 2 * MT; i++) vsum[i] += xch[tid + 256 * i];
    }
#pragma unroll
    for (int i = 0; EPI != 2 && i < 2 * MT; i++) {
        const int e = tid + 256 * i, r = e >> 5, c = e & 31, m = m0 + r, n = n0 + c;
        const bool ok = m < M && n < N;
        float v = 0.f;
        if (ok) {
            v = vsum[i];
            if (R) v += rpre[i];
            C[(size_t)m * N + n] = v;
        }
        if (EPI == 1) {
            float sq = v * v;
#pragma unroll
            for (int off = 16; off >= 1; off >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, off);
            if (lane == 0 && m < M) F.ss_out[(size_t)m * (gridDim.x / k_split) + col_tile] = sq;
        }
    }
#ifdef JGPT_B200_DECODE_TRACE
    timeline_at(F.timeline, 2);
#endif
}

// W1, W3 [K, Fo] -> [K, 2 Fo] with groups of 16 columns alternating (what EPI 2 expects).
__global__ void __launch_bounds__(256) interleave_pair_kernel(const float *__restrict__ W1, const float *__restrict__ W3, int K, int Fo,
                                                              float *__restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= (long long)K * 2 * Fo) return;
    const int k = (int)(i / (2 * Fo)), c = (int)(i % (2 * Fo));
    const int tile = c >> 5, within = c & 31;
    const int col = tile * 16 + (within & 15);
    out[i] = within < 16 ? W1[(size_t)k * Fo + col] : W3[(size_t)k * Fo + col];
}

// Greedy argmax per row, ties -> lowest index (argmaxLogitsGreedy,
// src/main/java/com/veles/llm/jgpt/model/GptAutoregressiveGenerator.java:288-299).
// out_host (optional): the ids also go to the caller's page-locked host array, and the context's status word to its
// host mirror, so that the step needs no copies behind its last kernel.
__global__ void __launch_bounds__(256) argmax_kernel(const float *__restrict__ logits, int V, int *__restrict__ out,
                                                     int *out_host = nullptr, const int *status_dev = nullptr, int *status_host = nullptr,
                                                     int pdl = 0) {
    if (pdl) griddep_wait();  // launched as a programmatic dependent of the LM head
    __shared__ float bv[8];
    __shared__ int bi[8];
    const float *row = logits + (size_t)blockIdx.x * V;
    float best = -INFINITY;
    int idx = 0x7fffffff;
    // eight loads in flight per thread: one load per iteration made the row a chain of V / 256 L2 round trips
    for (int j0 = threadIdx.x; j0 < V; j0 += 8 * 256) {
        float v[8];
#pragma unroll
        for (int u = 0; u < 8; u++) v[u] = j0 + 256 * u < V ? row[j0 + 256 * u] : -INFINITY;
#pragma unroll
        for (int u = 0; u < 8; u++) {
            const int j = j0 + 256 * u;
            if (j < V && (v[u] > best || (v[u] == best && j < idx))) best = v[u], idx = j;
        }
    }
    if (idx == 0x7fffffff) idx = 0;  // all NaN / -inf: the reference starts from index 0
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) {
        const float ov = __shfl_xor_sync(0xffffffffu, best, off);
        const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
        if (ov > best || (ov == best && oi < idx)) best = ov, idx = oi;
    }
    if ((threadIdx.x & 31) == 0) bv[threadIdx.x >> 5] = best, bi[threadIdx.x >> 5] = idx;
    __syncthreads();
    if (threadIdx.x == 0) {
        for (int w = 1; w < 8; w++)
            if (bv[w] > best || (bv[w] == best && bi[w] < idx)) best = bv[w], idx = bi[w];
        out[blockIdx.x] = idx;
        if (out_host) out_host[blockIdx.x] = idx;
        if (status_host && blockIdx.x == 0) *status_host = *status_dev;
    }
}

// sampleNextToken on the device (src/main/java/com/veles/llm/jgpt/model/GptAutoregressiveGenerator.java:208-286), one
// CTA per row, every step of the reference in its own order so that the token is the one the host routine picks:
// logits / temperature; keep the top_k by (logit descending, index ascending), the rest -inf; maximum;
// e = (float)exp((double)(z - max)); sum and the running CDF accumulated in fp32 in INDEX order by one thread
// (a float sum is not associative: a parallel reduction would move CDF boundaries); first index with u <= cdf,
// else the last one.  The uniform draw u is supplied per row (the reference draws from an unseeded
// ThreadLocalRandom).
__global__ void __launch_bounds__(256) sample_kernel(const float *__restrict__ logits, float *__restrict__ work, int V, float temperature,
                                                     int top_k, const float *__restrict__ u01, int *__restrict__ out) {
    __shared__ float bv[8];
    __shared__ int bi[8];
    __shared__ float s_thr_v, s_mx;
    __shared__ int s_thr_i;
    const float *row = logits + (size_t)blockIdx.x * V;
    float *z = work + (size_t)blockIdx.x * V;
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    for (int i = tid; i < V; i += 256) z[i] = temperature != 1.0f ? row[i] / temperature : row[i];
    __syncthreads();
    // block-wide "best" by (value descending, index ascending) among elements strictly after (pv, pi) in that order
    auto next_best = [&](float pv, int pi, bool first) {
        float best = -INFINITY;
        int idx = 0x7fffffff;
        for (int i = tid; i < V; i += 256) {
            const float v = z[i];
            const bool eligible = first || v < pv || (v == pv && i > pi);
            if (eligible && (v > best || (v == best && i < idx) || idx == 0x7fffffff)) best = v, idx = i;
        }
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) {
            const float ov = __shfl_xor_sync(0xffffffffu, best, off);
            const int oi = __shfl_xor_sync(0xffffffffu, idx, off);
            if (oi != 0x7fffffff && (idx == 0x7fffffff || ov > best || (ov == best && oi < idx))) best = ov, idx = oi;
        }
        if (lane == 0) bv[warp] = best, bi[warp] = idx;
        __syncthreads();
        if (tid == 0) {
            for (int w = 1; w < 8; w++)
                if (bi[w] != 0x7fffffff && (idx == 0x7fffffff || bv[w] > best || (bv[w] == best && bi[w] < idx))) best = bv[w], idx = bi[w];
            s_thr_v = best, s_thr_i = idx;
        }
        __syncthreads();
    };
    if (top_k > 0 && top_k < V) {
        next_best(0.f, 0, true);
        for (int r = 1; r < top_k; r++) next_best(s_thr_v, s_thr_i, false);
        const float tv = s_thr_v;
        const int ti = s_thr_i;  // the top_k-th element: everything after it in the order is dropped
        for (int i = tid; i < V; i += 256) {
            const float v = z[i];
            if (v < tv || (v == tv && i > ti)) z[i] = -INFINITY;
        }
        __syncthreads();
    }
    float mx = -INFINITY;
    for (int i = tid; i < V; i += 256) mx = fmaxf(mx, z[i]);
#pragma unroll
    for (int off = 16; off >= 1; off >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, off));
    if (lane == 0) bv[warp] = mx;
    __syncthreads();
    if (tid == 0) {
        for (int w = 1; w < 8; w++) mx = fmaxf(mx, bv[w]);
        s_mx = mx;
    }
    __syncthreads();
    mx = s_mx;
    for (int i = tid; i < V; i += 256) z[i] = (float)exp((double)(z[i] - mx));
    __syncthreads();
    if (tid == 0) {
        float sum = 0.f;
        for (int i = 0; i < V; i++) sum += z[i];
        const float u = u01[blockIdx.x];
        float cum = 0.f;
        int tok = V - 1;
        for (int i = 0; i < V; i++) {
            cum += z[i] / sum;
            if (u <= cum) {
                tok = i;
                break;
            }
        }
        out[blockIdx.x] = tok;
    }
}

// ------------------------------------------------------------------------------------------------
// Host side
// ------------------------------------------------------------------------------------------------
// From this many rows the decode-sized kernel uses 32-row tiles (JGPT_B200_SMALL_WIDE_ROWS).  Measured per decode
// step, 16-row against 32-row tiles: batch 64 0.64 / 0.71 ms, batch 128 0.83 / 0.89 ms, batch 256 1.40 / 1.31 ms.
static int small_rows_for_wide_tiles() {
    static const int v = env_int("JGPT_B200_SMALL_WIDE_ROWS", 256);
    return v;
}

// A launch of at most one CTA per SM that moves in early (programmatic dependent launch) asks for this much shared
// memory, more than half an SM's, so that no two of its CTAs share an SM: placed while the previous kernel still holds
// most SMs, the 48 CTAs of a Wo / W2 product otherwise land three to an SM on the few SMs with room (measured: on 24 SMs)
// and take 7 us after their wait instead of 3.5 us.
constexpr int kSoloSmemBytes = 115 * 1024;
constexpr int kSmallMaxSmemBytes = 219 * 1024;  // dynamic shared memory limit asked for the projection kernels: 227 KiB per CTA less their static arrays
constexpr size_t kSmemPerSm = 228 * 1024;       // of which 1 KiB per resident CTA is the system's

// The larger tile configurations need more than 48 KiB of dynamic shared memory: once per device.
static cudaError_t opt_in_shared_memory(const Ctx *ctx) {
    static bool opted[64] = {};
    if (opted[ctx->device & 63]) return cudaSuccess;
    cudaError_t e = cudaFuncSetAttribute(gemm_tc_kernel<64, 64, 2, 2, 3>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                         (int)gemm_tc_smem_bytes<64, 64, 3>());
    const int sb = kSmallMaxSmemBytes, sb2 = kSmallMaxSmemBytes;  // ring, solo padding or the whole weight slice (small_launch)
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, false, 0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, false, 1, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, true, 0, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, true, 2, 1>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, false, 0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb2);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, false, 1, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb2);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, true, 0, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb2);
    if (e == cudaSuccess) e = cudaFuncSetAttribute(gemm_tc_small_kernel<4, true, 2, 2>, cudaFuncAttributeMaxDynamicSharedMemorySize, sb2);
    if (e == cudaSuccess) opted[ctx->device & 63] = true;
    return e;
}

// The mma.sync / scalar kernels (any M; what decode-sized products use).
static int32_t gemm_small(Ctx *ctx, int strict, const float *A, int M, int K, int N, int nb, const float *const *W,
                          float *const *C, const float *const *R, const int *rowsel) {
    GemmBatch B;
    for (int z = 0; z < 3; z++) B.W[z] = z < nb ? W[z] : nullptr, B.C[z] = z < nb ? C[z] : nullptr, B.R[z] = (z < nb && R) ? R[z] : nullptr;
    cudaStream_t st = ctx->stream;
    if (!strict && K % 4 == 0 && N % 4 == 0) {  // tensor cores, 3xTF32
        // Decode-sized M: 16x32 tiles, the k loop split over eight warps (latency); above that 64x64 tiles.
        JGPT_CUDA_TRY(opt_in_shared_memory(ctx));
        if (M <= 512) {  // measured: faster than 32x32 tiles of four warps up to here (batch 128: 1.34 -> 1.04 ms per decode step)
            if (M >= small_rows_for_wide_tiles()) {
                dim3 grid((N + 31) / 32, (M + 31) / 32, nb);
                gemm_tc_small_kernel<4, false, 0, 2><<<grid, 256, gemm_small_smem_bytes<4, 2>(), st>>>(A, B, M, K, N, rowsel, SmallFuse{});
            } else {
                dim3 grid((N + 31) / 32, (M + 15) / 16, nb);
                gemm_tc_small_kernel<4, false, 0, 1><<<grid, 256, gemm_small_smem_bytes<4, 1>(), st>>>(A, B, M, K, N, rowsel, SmallFuse{});
            }
        } else {
            dim3 grid((N + 63) / 64, (M + 63) / 64, nb);
            gemm_tc_kernel<64, 64, 2, 2, 3><<<grid, 128, gemm_tc_smem_bytes<64, 64, 3>(), st>>>(A, B, M, K, N, rowsel);
        }
        JGPT_CUDA_TRY(cudaGetLastError());
        return JGPT_OK;
    }
    if (M <= 16) {
        dim3 grid((N + 63) / 64, (M + 15) / 16, nb);
        if (strict) gemm_kernel<16, 64, 1, 4, true><<<grid, 256, 0, st>>>(A, B, M, K, N, rowsel);
        else gemm_kernel<16, 64, 1, 4, false><<<grid, 256, 0, st>>>(A, B, M, K, N, rowsel);
    } else if (M <= 128) {
        dim3 grid((N + 63) / 64, (M + 31) / 32, nb);
        if (strict) gemm_kernel<32, 64, 2, 4, true><<<grid, 256, 0, st>>>(A, B, M, K, N, rowsel);
        else gemm_kernel<32, 64, 2, 4, false><<<grid, 256, 0, st>>>(A, B, M, K, N, rowsel);
    } else {
        dim3 grid((N + 63) / 64, (M + 63) / 64, nb);
        if (strict) gemm_kernel<64, 64, 4, 4, true><<<grid, 256, 0, st>>>(A, B, M, K, N, rowsel);
        else gemm_kernel<64, 64, 4, 4, false><<<grid, 256, 0, st>>>(A, B, M, K, N, rowsel);
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// Prefill-sized products: pack A into its image, look up (or build once) the weight images, run the tcgen05
// kernel.  Everything is ordered on the context's stream.
static int32_t ensure_image(Model *m, float **buf, uint64_t *cap, uint64_t need) {
    if (need <= *cap) return JGPT_OK;
    JGPT_CUDA_TRY(cudaStreamSynchronize(m->ctx->stream));
    if (*buf) JGPT_CUDA_TRY(cudaFree(*buf));
    *buf = nullptr, *cap = 0;
    JGPT_CUDA_TRY(cudaMalloc(buf, sizeof(float) * need));
    *cap = need;
    return JGPT_OK;
}
static int32_t weight_image(Model *m, const float *W, int K, int N, const float **out) {
    auto it = m->wimg.find(W);
    if (it == m->wimg.end()) {
        float *img = nullptr;
        JGPT_CUDA_TRY(cudaMalloc(&img, sizeof(float) * umma::weight_image_floats(K, N)));
        it = m->wimg.emplace(W, img).first;
        int32_t rc = umma::pack_weight(W, K, N, img, m->ctx->stream);
        if (rc) return rc;
    }
    *out = it->second;
    return JGPT_OK;
}
static int32_t weight_pair_image(Model *m, const float *W1, const float *W3, int K, int F, const float **out) {
    auto it = m->wpair.find(W1);
    if (it == m->wpair.end()) {
        float *img = nullptr;
        JGPT_CUDA_TRY(cudaMalloc(&img, sizeof(float) * umma::image_floats(2 * F, K, 256)));
        it = m->wpair.emplace(W1, img).first;
        int32_t rc = umma::pack_weight_pair(W1, W3, K, F, img, m->ctx->stream);
        if (rc) return rc;
    }
    *out = it->second;
    return JGPT_OK;
}

static int32_t gemm_umma(Model *m, const float *A, int M, int K, int N, int nb, const float *const *W, float *const *C,
                         const float *const *R, const int *rowsel) {
    cudaStream_t st = m->ctx->stream;
    int32_t rc = ensure_image(m, &m->aimg, &m->aimg_floats, umma::activation_image_floats(M, K));
    if (rc) return rc;
    umma::Batch b{};
    for (int z = 0; z < nb; z++) {
        rc = weight_image(m, W[z], K, N, &b.Wimg[z]);
        if (rc) return rc;
        b.C[z] = C[z], b.R[z] = R ? R[z] : nullptr;
    }
    rc = umma::pack_activations(A, rowsel, M, K, m->aimg, st);
    if (rc) return rc;
    return umma::launch(m->aimg, b, nb, M, K, N, m->ctx->d_status, st);
}

static int32_t gemm(Model *m, const float *A, int M, int K, int N, int nb, const float *const *W, float *const *C,
                    const float *const *R, const int *rowsel = nullptr) {
    if (!m->strict && m->umma_min_rows > 0 && M >= m->umma_min_rows && umma::shape_ok(K, N))
        return gemm_umma(m, A, M, K, N, nb, W, C, R, rowsel);
    return gemm_small(m->ctx, m->strict, A, M, K, N, nb, W, C, R, rowsel);
}

static int num_tensors(const Model *m) { return 4 + 9 * m->layers; }

static float *tensor_ptr(Model *m, int idx, uint64_t *count) {
    const uint64_t D = m->d_model, F = m->d_ff, V = m->vocab;
    const int n = num_tensors(m);
    if (idx == 0) { *count = V * D; return m->tok; }
    if (idx == 1) { *count = (uint64_t)m->max_seq * D; return m->pos; }
    if (idx == n - 2) { *count = D; return m->norm_final; }
    if (idx == n - 1) { *count = D * V; return m->lm_head; }
    LayerW &y = m->L[(size_t)((idx - 2) / 9)];
    switch ((idx - 2) % 9) {
        case 0: *count = D * D; return y.wq;
        case 1: *count = D * D; return y.wk;
        case 2: *count = D * D; return y.wv;
        case 3: *count = D * D; return y.wo;
        case 4: *count = D * F; return y.w1;
        case 5: *count = F * D; return y.w2;
        case 6: *count = D * F; return y.w3;
        case 7: *count = D; return y.norm1;
        default: *count = D; return y.norm2;
    }
}

static int32_t ensure_logits(Model *m, int rows) {
    if (rows <= m->logit_rows) return JGPT_OK;
    JGPT_CUDA_TRY(cudaStreamSynchronize(m->ctx->stream));
    if (m->logits) JGPT_CUDA_TRY(cudaFree(m->logits));
    m->logits = nullptr, m->logit_rows = 0;
    JGPT_CUDA_TRY(cudaMalloc(&m->logits, sizeof(float) * (size_t)rows * m->vocab));
    m->logit_rows = rows;
    return JGPT_OK;
}

struct SampleSpec {
    float temperature = 0.f;  // <= 0: greedy argmax on the device
    int top_k = 0;
};
static int32_t ensure_sample_work(Model *m, int rows) {
    if (rows <= m->samp_rows) return JGPT_OK;
    JGPT_CUDA_TRY(cudaStreamSynchronize(m->ctx->stream));
    if (m->d_samp) JGPT_CUDA_TRY(cudaFree(m->d_samp));
    m->d_samp = nullptr, m->samp_rows = 0;
    JGPT_CUDA_TRY(cudaMalloc(&m->d_samp, sizeof(float) * (size_t)rows * m->vocab));
    m->samp_rows = rows;
    return JGPT_OK;
}

// One decoder block over `rows` rows already in m->x.  Attention is supplied by the caller.
// The same decoder blocks for prefill-sized `rows`: every projection on the tcgen05 kernel, activations handed
// from producer to consumer as operand images (RMSNorm writes one, the W1/W3 product's SwiGLU epilogue writes
// one; only the attention output is packed by a kernel of its own).
// attn(l, image, kv_in_cache): attention of layer l; writes the Wo operand image itself when image != nullptr, the
// row-major m->att otherwise; kv_in_cache: the K / V rows of the layer are already in the paged store.
// `paged` != nullptr (a prefill at d_head 16): the attention can write that image, and the Q,K,V product writes
// K / V straight into the paged store (paged->layer is set per layer here).
template <class AttnFn>
static int32_t run_layers_umma(Model *m, int rows, const PagedAppendArgs *paged, AttnFn &&attn) {
    const bool attn_writes_image = paged != nullptr;
    const int D = m->d_model, F = m->d_ff;
    cudaStream_t st = m->ctx->stream;
    int *status = m->ctx->d_status;
    const bool fused_ffn = umma::swiglu_shape_ok(D, F);
    int32_t rc = ensure_image(m, &m->aimg, &m->aimg_floats, umma::activation_image_floats(rows, D));
    if (rc) return rc;
    rc = ensure_image(m, &m->aimg2, &m->aimg2_floats, umma::activation_image_floats(rows, F));
    if (rc) return rc;
    for (int l = 0; l < m->layers; l++) {
        const LayerW &y = m->L[(size_t)l];
        umma::Batch qkv{}, wo{}, w13{}, w2{};
        if ((rc = weight_image(m, y.wq, D, D, &qkv.Wimg[0]))) return rc;
        if ((rc = weight_image(m, y.wk, D, D, &qkv.Wimg[1]))) return rc;
        if ((rc = weight_image(m, y.wv, D, D, &qkv.Wimg[2]))) return rc;
        if ((rc = weight_image(m, y.wo, D, D, &wo.Wimg[0]))) return rc;
        if ((rc = weight_image(m, y.w2, F, D, &w2.Wimg[0]))) return rc;
        qkv.C[0] = m->q, qkv.C[1] = m->k, qkv.C[2] = m->v;
        wo.C[0] = m->x, wo.R[0] = m->x;  // x1 = x + attn.Wo (each element read then written by the same thread)
        w2.C[0] = m->x, w2.R[0] = m->x;
        if ((rc = umma::rmsnorm_pack(m->x, y.norm1, rows, D, m->eps, m->aimg, st))) return rc;
        if (paged) {
            PagedAppendArgs pa = *paged;
            pa.layer = l;
            if ((rc = umma::launch_qkv_paged(m->aimg, qkv, rows, D, D, pa, status, st))) return rc;
        } else {
            if ((rc = umma::launch(m->aimg, qkv, 3, rows, D, D, status, st))) return rc;
        }
        if ((rc = attn(l, attn_writes_image ? m->aimg : nullptr, paged != nullptr))) return rc;
        if (!attn_writes_image && (rc = umma::pack_activations(m->att, nullptr, rows, D, m->aimg, st))) return rc;
        if ((rc = umma::launch(m->aimg, wo, 1, rows, D, D, status, st))) return rc;
        if ((rc = umma::rmsnorm_pack(m->x, y.norm2, rows, D, m->eps, m->aimg, st))) return rc;
        if (fused_ffn) {
            const float *pair = nullptr;
            if ((rc = weight_pair_image(m, y.w1, y.w3, D, F, &pair))) return rc;
            if ((rc = umma::launch_swiglu(m->aimg, pair, rows, D, F, m->aimg2, status, st))) return rc;
        } else {
            if ((rc = weight_image(m, y.w1, D, F, &w13.Wimg[0]))) return rc;
            if ((rc = weight_image(m, y.w3, D, F, &w13.Wimg[1]))) return rc;
            w13.C[0] = m->h1, w13.C[1] = m->g;
            if ((rc = umma::launch(m->aimg, w13, 2, rows, D, F, status, st))) return rc;
            const long long nf = (long long)rows * F;
            swiglu_kernel<<<(unsigned)((nf + 255) / 256), 256, 0, st>>>(m->h1, m->g, nf);
            if ((rc = umma::pack_activations(m->h1, nullptr, rows, F, m->aimg2, st))) return rc;
        }
        if ((rc = umma::launch(m->aimg2, w2, 1, rows, F, D, status, st))) return rc;
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

#ifdef JGPT_B200_DECODE_TRACE
static unsigned long long *g_timeline_buf = nullptr;
static int g_timeline_slot = 0;
constexpr int kTimelineSlots = 256;
Timeline timeline_next() {
    if (!g_timeline_buf && cudaMalloc(&g_timeline_buf, sizeof(unsigned long long) * (4 + 256) * kTimelineSlots) != cudaSuccess) return Timeline{};
    Timeline T{};
    T.buf = g_timeline_buf, T.slot = g_timeline_slot < kTimelineSlots ? g_timeline_slot++ : kTimelineSlots - 1;
    return T;
}
#endif

// Decode-sized steps: every projection on gemm_tc_small_kernel with RMSNorm folded into the consumer (the producer
// of x leaves partial row sums of squares) and SwiGLU into the W1/W3 product: 4 projection launches + attention per
// layer instead of 7 launches + attention.
static bool small_mode(const Model *m, int rows) {
    return !m->strict && rows <= 512 && m->d_model % 4 == 0 && m->d_ff % 16 == 0 && m->vocab % 4 == 0 &&
           !(m->umma_min_rows > 0 && rows >= m->umma_min_rows);
}
static int32_t pair_interleaved(Model *m, const float *W1, const float *W3, int K, int Fo, const float **out, bool *fresh = nullptr) {
    auto it = m->w13i.find(W1);
    if (fresh) *fresh = it == m->w13i.end();
    if (it == m->w13i.end()) {
        float *buf = nullptr;
        JGPT_CUDA_TRY(cudaMalloc(&buf, sizeof(float) * (size_t)K * 2 * Fo));
        it = m->w13i.emplace(W1, buf).first;
        const long long n = (long long)K * 2 * Fo;
        interleave_pair_kernel<<<(unsigned)((n + 255) / 256), 256, 0, m->ctx->stream>>>(W1, W3, K, Fo, buf);
        JGPT_CUDA_TRY(cudaGetLastError());
    }
    *out = it->second;
    return JGPT_OK;
}
// W [K, N] with row k multiplied by gamma[k]: the weights a NORM product reads (built once per weight set).
__global__ void scale_rows_kernel(const float *__restrict__ W, const float *__restrict__ gamma, long long n, int N, float *__restrict__ out) {
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) out[i] = gamma[i / N] * W[i];
}
static int32_t scaled_weight(Model *m, const float *W, const float *gamma, int K, int N, const float **out, bool *fresh) {
    auto it = m->wscaled.find(W);
    if (it == m->wscaled.end()) {
        float *buf = nullptr;
        JGPT_CUDA_TRY(cudaMalloc(&buf, sizeof(float) * (size_t)K * N));
        it = m->wscaled.emplace(W, buf).first;
        const long long n = (long long)K * N;
        scale_rows_kernel<<<(unsigned)((n + 255) / 256), 256, 0, m->ctx->stream>>>(W, gamma, n, N, buf);
        JGPT_CUDA_TRY(cudaGetLastError());
        *fresh = true;  // just written by a kernel on this stream: the launch that reads it must not run ahead of its wait
    }
    *out = it->second;
    return JGPT_OK;
}

template <bool NORM, int EPI>
static int32_t small_launch(Model *m, const float *A, int M, int K, int N, int nb, const float *const *W, float *const *C,
                            const float *const *R, const int *rowsel, const SmallFuse &fuse_in) {
    JGPT_CUDA_TRY(opt_in_shared_memory(m->ctx));
    GemmBatch B;
    for (int z = 0; z < 3; z++) B.W[z] = z < nb ? W[z] : nullptr, B.C[z] = z < nb ? C[z] : nullptr, B.R[z] = (z < nb && R) ? R[z] : nullptr;
    cudaLaunchConfig_t cfg = {};
    cudaLaunchAttribute attr[2];
    unsigned n_attr = 0;
    SmallFuse fuse = fuse_in;
    if (fuse.pdl & 1) {
        attr[n_attr].id = cudaLaunchAttributeProgrammaticStreamSerialization;
        attr[n_attr].val.programmaticStreamSerializationAllowed = 1;
        n_attr++;
    }
#ifdef JGPT_B200_DECODE_TRACE
    fuse.timeline = timeline_next();
#endif
    cfg.blockDim = dim3(256), cfg.stream = m->ctx->stream;
    // 32-row tiles also where the 16-row grid would no longer be resident at once (three CTAs per SM) while the 32-row
    // grid is: a few CTAs left for a second wave cost a whole tile time (W1,W3 from 145 rows on: 160 rows 1.01 ms per step)
    const long long resident = 3ll * m->ctx->sm_count, col_tiles = (long long)((N + 31) / 32) * nb;
    const bool spills = col_tiles * ((M + 15) / 16) > resident && col_tiles * ((M + 31) / 32) <= resident;
    // a product of many column tiles (the LM head: 250) runs in several rounds of resident CTAs whatever the tile: with
    // 32-row tiles it has half as many CTAs, each fetching its weight tile once for twice the rows
    const bool many_cols = col_tiles > m->ctx->sm_count && M > 16;
    // Wo / W2 moving in early: 32-row tiles where only they bring the launch down to one CTA per SM (the early CTAs of a
    // larger grid are packed three to an SM wherever there is room: 200 rows 1.145 -> 1.088 ms per step)
    const bool solo_if_wide = EPI == 1 && (fuse.pdl & 1) && col_tiles * ((M + 15) / 16) > m->ctx->sm_count &&
                              col_tiles * ((M + 31) / 32) <= m->ctx->sm_count;
    const bool wide = M >= small_rows_for_wide_tiles() || spills || many_cols || solo_if_wide;
    // Wo / W2 of a step with few rows: pairs of CTAs split the k range (SmallFuse::k_split) while the launch still has at
    // most one CTA per SM.
    if (EPI == 1 && m->k_split && !rowsel && (K + kSmallBK - 1) / kSmallBK >= 4 &&
        2 * col_tiles * ((M + (wide ? 31 : 15)) / (wide ? 32 : 16)) <= m->ctx->sm_count) {
        fuse.k_split = 2;
        attr[n_attr].id = cudaLaunchAttributeClusterDimension;
        attr[n_attr].val.clusterDim.x = 2, attr[n_attr].val.clusterDim.y = 1, attr[n_attr].val.clusterDim.z = 1;
        n_attr++;
    }
    cfg.attrs = attr, cfg.numAttrs = n_attr;
    const bool solo = (fuse.pdl & 1) && fuse.k_split * col_tiles * ((M + (wide ? 31 : 15)) / (wide ? 32 : 16)) <= m->ctx->sm_count;
    // The CTA's whole weight slice in shared memory (SmallFuse::w_resident) where the launch is still resident at once
    // with that much shared memory per CTA.  The step's weights do not stay in L2 from one step to the next, so a
    // ring of four k tiles pays a trip to HBM per three tiles (W2, K = 768: 0.43 us per tile); with the slice
    // requested at the top - before the wait for the previous kernel - it is one trip, hidden when the launch moved in early.
    const int bm = wide ? 32 : 16;
    const long long ctas = fuse.k_split * col_tiles * ((M + bm - 1) / bm);
    const size_t ring = wide ? gemm_small_smem_bytes<4, 2>() : gemm_small_smem_bytes<4, 1>();
    const size_t k_tiles = ((size_t)(K + kSmallBK - 1) / kSmallBK + fuse.k_split - 1) / fuse.k_split;  // of the CTA with the most
    const size_t slice = sizeof(float) * (4 * (size_t)bm * (kSmallBK + 4) + k_tiles * kSmallBK * (32 + 8));
    const long long by_regs = wide ? 2 : 3;  // 128 / 80 registers per thread
    const long long per_sm = std::min<long long>(by_regs, (long long)(kSmemPerSm / (slice + 1024)));
    if (m->w_resident && slice <= kSmallMaxSmemBytes && per_sm >= 1 && ctas <= per_sm * m->ctx->sm_count) fuse.w_resident = 1;
    cfg.dynamicSmemBytes = fuse.w_resident ? std::max(slice, ring) : ring;
    if (solo) cfg.dynamicSmemBytes = std::max<size_t>(cfg.dynamicSmemBytes, kSoloSmemBytes);
    if (wide) {
        cfg.gridDim = dim3(fuse.k_split * ((N + 31) / 32), (M + 31) / 32, nb);
        JGPT_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tc_small_kernel<4, NORM, EPI, 2>, A, B, M, K, N, rowsel, fuse));
    } else {
        cfg.gridDim = dim3(fuse.k_split * ((N + 31) / 32), (M + 15) / 16, nb);
        JGPT_CUDA_TRY(cudaLaunchKernelEx(&cfg, gemm_tc_small_kernel<4, NORM, EPI, 1>, A, B, M, K, N, rowsel, fuse));
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// How far the launches of a decode step overlap (levels: see run_layers_small).  Measured on the JGPT-35M shapes, ms
// per step at batch 8 / 64 / 256: level 0: 0.45 / 0.59 / 1.26; 1: 0.42 / 0.574 / 1.256; 2: 0.41 / 0.566 / 1.247;
// 3: 0.375 / 0.535 / 1.21.  Level 3 only pays since early-launched projections of at most one CTA per SM keep an SM
// to themselves (kSoloSmemBytes) and request their weight tiles before they wait; before that it lost from 24 rows on
// (batch 64: 0.62 ms) because the early CTAs of Wo and W2 were packed three to an SM.
static int step_overlap_level(const Model *m, int rows) {
    (void)rows;
    return m->step_overlap >= 0 ? m->step_overlap : 3;
}

template <class AttnFn>
static int32_t run_layers_small(Model *m, int rows, AttnFn &&attn) {
#ifdef JGPT_B200_DECODE_TRACE
    g_timeline_slot = 0;
#endif
    const int D = m->d_model, F = m->d_ff, parts = (D + 31) / 32;
    for (int l = 0; l < m->layers; l++) {
        const LayerW &y = m->L[(size_t)l];
        int32_t rc;
        // x's sums of squares: one partial per row from the embedding, `parts` from a residual projection
        // Launch overlap inside the step (m->step_overlap): 1 = the attention launch moves in under the Q,K,V product
        // (its copy warp fetches tables and K/V slabs meanwhile; that product writes q / k / v only); 2 = the Wo product
        // moves in under the attention's tail as well; 3 = every projection of the layer chain.
        const int ov = step_overlap_level(m, rows);
        SmallFuse n1{y.norm1, m->ss_a, nullptr, l == 0 ? 1 : parts, m->eps, (ov >= 1 ? 2 : 0) | ((ov >= 3 && (l > 0 || m->first_launch_early)) ? 1 : 0)};
        const float *Wqkv[3] = {nullptr, nullptr, nullptr};
        bool fresh_qkv = false;
        if ((rc = scaled_weight(m, y.wq, y.norm1, D, D, &Wqkv[0], &fresh_qkv))) return rc;
        if ((rc = scaled_weight(m, y.wk, y.norm1, D, D, &Wqkv[1], &fresh_qkv))) return rc;
        if ((rc = scaled_weight(m, y.wv, y.norm1, D, D, &Wqkv[2], &fresh_qkv))) return rc;
        if (fresh_qkv) n1.pdl &= ~1;
        float *Cqkv[3] = {m->q, m->k, m->v};
        if ((rc = small_launch<true, 0>(m, m->x, rows, D, D, 3, Wqkv, Cqkv, nullptr, nullptr, n1))) return rc;
        if ((rc = attn(l, nullptr, false))) return rc;
        const float *Wo[1] = {y.wo};
        float *Cx[1] = {m->x};
        const float *Rx[1] = {m->x};  // x1 = x + attn.Wo (each element read then written by the same thread)
        if ((rc = small_launch<false, 1>(m, m->att, rows, D, D, 1, Wo, Cx, Rx, nullptr,
                                         SmallFuse{nullptr, nullptr, m->ss_b, 0, 0.f, (ov >= 2 ? 1 : 0) | (ov >= 3 ? 2 : 0)}))) return rc;
        const float *pair = nullptr;
        bool fresh = false;  // just written by a kernel on this stream: that launch must not read weights ahead of its wait
        if ((rc = pair_interleaved(m, y.w1, y.w3, D, F, &pair, &fresh))) return rc;
        if ((rc = scaled_weight(m, pair, y.norm2, D, 2 * F, &pair, &fresh))) return rc;
        const float *Wp[1] = {pair};
        float *Ch[1] = {m->h1};
        if ((rc = small_launch<true, 2>(m, m->x, rows, D, 2 * F, 1, Wp, Ch, nullptr, nullptr,
                                        SmallFuse{y.norm2, m->ss_b, nullptr, parts, m->eps, ov >= 3 ? (fresh ? 2 : 3) : 0}))) return rc;
        const float *W2[1] = {y.w2};
        if ((rc = small_launch<false, 1>(m, m->h1, rows, F, D, 1, W2, Cx, Rx, nullptr,
                                         SmallFuse{nullptr, nullptr, m->ss_a, 0, 0.f, ov >= 3 ? 3 : 0}))) return rc;
    }
    return JGPT_OK;
}

template <class AttnFn>
static int32_t run_layers(Model *m, int rows, const PagedAppendArgs *paged, AttnFn &&attn) {
    const int D = m->d_model, F = m->d_ff;
    if (small_mode(m, rows)) return run_layers_small(m, rows, attn);
    if (!m->strict && m->umma_min_rows > 0 && rows >= m->umma_min_rows && umma::shape_ok(D, D) && umma::shape_ok(D, F) &&
        umma::shape_ok(F, D) && sizeof(float) * 8 * (size_t)(D + 4) <= 48 * 1024)
        return run_layers_umma(m, rows, paged, attn);
    cudaStream_t st = m->ctx->stream;
    for (int l = 0; l < m->layers; l++) {
        const LayerW &y = m->L[(size_t)l];
        rmsnorm_kernel<<<rows, 128, 0, st>>>(m->x, y.norm1, m->xn, D, m->eps);
        const float *Wqkv[3] = {y.wq, y.wk, y.wv};
        float *Cqkv[3] = {m->q, m->k, m->v};
        int32_t rc = gemm(m, m->xn, rows, D, D, 3, Wqkv, Cqkv, nullptr);
        if (rc) return rc;
        rc = attn(l, nullptr, false);
        if (rc) return rc;
        const float *Wo[1] = {y.wo};
        float *Co[1] = {m->x};
        const float *Ro[1] = {m->x};  // x1 = x + attn.Wo (each element read then written by the same thread)
        rc = gemm(m, m->att, rows, D, D, 1, Wo, Co, Ro);
        if (rc) return rc;
        rmsnorm_kernel<<<rows, 128, 0, st>>>(m->x, y.norm2, m->xn, D, m->eps);
        const float *W13[2] = {y.w1, y.w3};
        float *C13[2] = {m->h1, m->g};
        rc = gemm(m, m->xn, rows, D, F, 2, W13, C13, nullptr);
        if (rc) return rc;
        const long long nf = (long long)rows * F;
        swiglu_kernel<<<(unsigned)((nf + 255) / 256), 256, 0, st>>>(m->h1, m->g, nf);
        const float *W2[1] = {y.w2};
        rc = gemm(m, m->h1, rows, F, D, 1, W2, Co, Ro);
        if (rc) return rc;
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// Final norm + LM head over the rows listed in d_rowsel[0..n_sel) (or all rows), then argmax.
static int32_t lm_head(Model *m, int rows, int n_sel, const SampleSpec &spec = SampleSpec(), bool to_host = false, bool early = false) {
    const int D = m->d_model;
    cudaStream_t st = m->ctx->stream;
    const int out_rows = n_sel > 0 ? n_sel : rows;
    int32_t rc = ensure_logits(m, out_rows);
    if (rc) return rc;
    const float *W[1] = {m->lm_head};
    float *C[1] = {m->logits};
    const int *rowsel = n_sel > 0 ? m->d_rowsel : nullptr;
    if (small_mode(m, rows)) {  // the last W2 projection left the row sums of squares in ss_a
        bool fresh = false;
        if ((rc = scaled_weight(m, m->lm_head, m->norm_final, D, m->vocab, &W[0], &fresh))) return rc;
        rc = small_launch<true, 0>(m, m->x, out_rows, D, m->vocab, 1, W, C, nullptr, rowsel,
                                   SmallFuse{m->norm_final, m->ss_a, nullptr, (D + 31) / 32, m->eps, (early && !fresh) ? 3 : (early ? 2 : 0)});
    } else {
        rmsnorm_kernel<<<rows, 128, 0, st>>>(m->x, m->norm_final, m->xn, D, m->eps);
        rc = gemm(m, m->xn, out_rows, D, m->vocab, 1, W, C, nullptr, rowsel);
    }
    if (rc) return rc;
    if (spec.temperature > 0.f) {  // the draws are in m->d_u (uploaded by the caller)
        rc = ensure_sample_work(m, out_rows);
        if (rc) return rc;
        sample_kernel<<<out_rows, 256, 0, st>>>(m->logits, m->d_samp, m->vocab, spec.temperature, spec.top_k, m->d_u, m->d_next);
    } else {
        if (to_host && early && small_mode(m, rows)) {  // moves in under the LM head's last CTAs
            cudaLaunchConfig_t cfg = {};
            cudaLaunchAttribute attr[1];
            attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
            attr[0].val.programmaticStreamSerializationAllowed = 1;
            cfg.gridDim = dim3((unsigned)out_rows), cfg.blockDim = dim3(256), cfg.stream = st, cfg.attrs = attr, cfg.numAttrs = 1;
            const float *lg = m->logits;
            JGPT_CUDA_TRY(cudaLaunchKernelEx(&cfg, argmax_kernel, lg, m->vocab, m->d_next, m->hd_next, (const int *)m->ctx->d_status, m->hd_status, 1));
        } else if (to_host) argmax_kernel<<<out_rows, 256, 0, st>>>(m->logits, m->vocab, m->d_next, m->hd_next, m->ctx->d_status, m->hd_status);
        else argmax_kernel<<<out_rows, 256, 0, st>>>(m->logits, m->vocab, m->d_next);
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// ---- the fused step (decode_fused.cu) ----
static bool fused_ok(const Model *m, const Pool *p, int n) {
    const size_t smem = sizeof(float) * 4 * ((size_t)m->d_model + (size_t)std::max(m->d_model, m->d_ff)) + 28672 + 96 * 1024;
    return m->fused_step && !m->strict && n >= 1 && n <= fused_step_max_rows() && p->dhead == 16 && m->d_model == m->heads * 16 &&
           m->d_model % 8 == 0 && m->d_ff % 8 == 0 && m->vocab % 8 == 0 && smem <= 156 * 1024 && m->layers <= kFusedMaxLayers &&
           m->d_model <= 1024;
}
static size_t fused_pair_count(const Model *m) {
    const size_t D = m->d_model, F = m->d_ff, H = m->heads, G = m->ctx->sm_count, R = 4;
    return R * 3 * D + R * H * kFusedMaxChunks * 18 + 2 * (size_t)kFusedMaxKSplit * R * D + R * F + G * R * 2;
}
static int32_t ensure_fused(Model *m) {
    if (m->f_pairs) return JGPT_OK;
    const size_t R = 4, ni = (size_t)kFusedMaxSteps * R + 4 + 4;
    m->f_pairs_n = fused_pair_count(m);
    if (!m->f_ints) JGPT_CUDA_TRY(cudaMalloc(&m->f_ints, sizeof(int) * ni));
    JGPT_CUDA_TRY(cudaMemsetAsync(m->f_ints, 0, sizeof(int) * ni, m->ctx->stream));
    if (!m->h_fused) JGPT_CUDA_TRY(cudaHostAlloc(&m->h_fused, sizeof(int) * ((size_t)kFusedMaxSteps * R + 4), cudaHostAllocDefault));
    uint2 *pairs = nullptr;
    JGPT_CUDA_TRY(cudaMalloc(&pairs, sizeof(uint2) * m->f_pairs_n));
    JGPT_CUDA_TRY(cudaMemsetAsync(pairs, 0, sizeof(uint2) * m->f_pairs_n, m->ctx->stream));  // stamp 0: never data
    JGPT_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&m->hd_fused), m->h_fused, 0));
    JGPT_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&m->hd_next), m->h_next, 0));
    m->f_pairs = pairs;
    m->f_stamp = 0;
    return JGPT_OK;
}
static int *fused_tokens_dev(Model *m) { return m->f_ints; }
static int *fused_steps_done_dev(Model *m) { return m->f_ints + (size_t)kFusedMaxSteps * 4; }
// Enqueues `steps` decode steps of the n rows described in m->d_idx (already uploaded).  Tokens go to `next_dev`
// ([steps][n]); with stop_on_zero (n == 1) the launch ends after a sampled 0.
// idx_host: the rows' descriptors ([5][n], travel in the launch parameters: no upload).  next_host / done_host: mapped
// host addresses the kernel also writes the tokens and the step count to (nullptr: not wanted).
static int32_t fused_enqueue(Model *m, Pool *p, int n, int steps, int stop_on_zero, int max_len_after, int *next_dev, const int *idx_host,
                             int *next_host, int *done_host) {
    const size_t D = m->d_model, F = m->d_ff, H = m->heads, R = 4;
    const uint32_t need = (uint32_t)steps * (uint32_t)m->layers;
    if (m->f_stamp > 0xE0000000u - need) {  // stamps about to wrap: start over from clean buffers
        JGPT_CUDA_TRY(cudaMemsetAsync(m->f_pairs, 0, sizeof(uint2) * m->f_pairs_n, m->ctx->stream));
        JGPT_CUDA_TRY(cudaMemsetAsync(fused_steps_done_dev(m) + 4, 0, sizeof(int) * 4, m->ctx->stream));
        m->f_stamp = 0;
    }
    FusedStepArgs A = {};
    A.tok = m->tok, A.pos = m->pos, A.norm_final = m->norm_final, A.lm_head = m->lm_head;
    for (int l = 0; l < m->layers; l++) A.Lw[l] = m->L[(size_t)l];
    A.vocab = m->vocab, A.max_seq = m->max_seq, A.D = m->d_model, A.H = m->heads, A.layers = m->layers, A.F = m->d_ff, A.eps = m->eps;
    A.kv = p->kv, A.table = p->d_table, A.rope = p->d_rope, A.n_blocks = p->n_blocks, A.mbs = p->max_blocks_per_seq;
    A.idx = nullptr, A.n = n, A.steps = steps, A.stop_on_zero = stop_on_zero;
    for (int i = 0; i < 5 * n; i++) A.idx_inline[i] = idx_host[i];
    A.next_host = next_host, A.steps_done_host = done_host;
    uint2 *f = m->f_pairs;
    A.ll_qkv = f, f += R * 3 * D;
    A.ll_part = f, f += R * H * kFusedMaxChunks * 18;
    A.ll_po = f, f += (size_t)kFusedMaxKSplit * R * D;
    A.ll_pw2 = f, f += (size_t)kFusedMaxKSplit * R * D;
    A.ll_act = f, f += R * F;
    A.ll_cand = f;
    A.stamp0 = m->f_stamp;
    m->f_stamp += need;
    A.logits = m->logits;
    A.steps_done = fused_steps_done_dev(m);
    A.sync_words = reinterpret_cast<unsigned *>(fused_steps_done_dev(m) + 4);
    A.next = next_dev;
    A.status = m->ctx->d_status;
    fused_step_plan(A, m->ctx->sm_count, max_len_after);
    A.test_withhold = env_int("JGPT_B200_FUSED_TEST_WITHHOLD", 0);
    return launch_decode_fused(m->ctx, A);
}

// ---- the fused step of a batch (decode_batch.cu) ----
static bool fused_batch_ok(const Model *m, const Pool *p, int n) {
    return m->fused_batch && !m->strict && n > fused_step_max_rows() && n <= std::min(kFusedBatchMaxRows, m->max_rows) && p->dhead == 16 &&
           m->d_model == m->heads * 16 && m->d_model % 64 == 0 && m->d_ff % 16 == 0 && m->vocab % 4 == 0 && m->layers <= kFusedMaxLayers &&
           std::max(m->d_model, m->d_ff) <= 2048;
}
static int fused_batch_max_chunks(const Model *m) { return ((m->max_seq + 15) / 16 + 1) / 2; }  // chunks hold >= 2 blocks
static int32_t ensure_fused_batch(Model *m) {
    if (m->fb_pairs) return JGPT_OK;
    const size_t R = (size_t)std::min(kFusedBatchMaxRows, m->max_rows), D = m->d_model, F = m->d_ff, H = m->heads;
    const size_t parts = (D + 31) / 32, vt = ((size_t)m->vocab + 31) / 32;
    m->fb_pairs_n = R * (2 * D + 2 * parts + 3 * D + D + F) + vt * R * 2;
    if (!m->fb_part) {
        const size_t np = R * H * (size_t)fused_batch_max_chunks(m) * 18;
        JGPT_CUDA_TRY(cudaMalloc(&m->fb_part, sizeof(uint2) * np));
        JGPT_CUDA_TRY(cudaMemsetAsync(m->fb_part, 0, sizeof(uint2) * np, m->ctx->stream));  // stamp 0: never data
    }
    if (!m->fb_tickets) JGPT_CUDA_TRY(cudaMalloc(&m->fb_tickets, sizeof(int) * (R * H + 4)));
    JGPT_CUDA_TRY(cudaMemsetAsync(m->fb_tickets, 0, sizeof(int) * (R * H + 4), m->ctx->stream));
    uint2 *pairs = nullptr;
    JGPT_CUDA_TRY(cudaMalloc(&pairs, sizeof(uint2) * m->fb_pairs_n));
    JGPT_CUDA_TRY(cudaMemsetAsync(pairs, 0, sizeof(uint2) * m->fb_pairs_n, m->ctx->stream));  // stamp 0: never data
    m->fb_pairs = pairs, m->fused_batch_rows = (int)R;
    return JGPT_OK;
}
// Puts the waits' bookkeeping back after a step that reported a failed device check.
static void fused_batch_reset(Model *m) {
    if (m->fb_tickets) cudaMemsetAsync(m->fb_tickets, 0, sizeof(int) * ((size_t)m->fused_batch_rows * m->heads + 4), m->ctx->stream);
}
static int32_t fused_batch_enqueue(Model *m, Pool *p, int n, const int *lens_host) {
    const size_t R = (size_t)m->fused_batch_rows, D = m->d_model, F = m->d_ff;
    const size_t parts = (D + 31) / 32;
    const uint32_t need = (uint32_t)m->layers + 2u;
    if (m->f_stamp > 0xE0000000u - need) {  // stamps about to wrap: start over from clean buffers (both step forms share the counter)
        JGPT_CUDA_TRY(cudaMemsetAsync(m->fb_pairs, 0, sizeof(uint2) * m->fb_pairs_n, m->ctx->stream));
        JGPT_CUDA_TRY(cudaMemsetAsync(m->fb_part, 0, sizeof(uint2) * (size_t)m->fused_batch_rows * m->heads * fused_batch_max_chunks(m) * 18, m->ctx->stream));
        if (m->f_pairs) JGPT_CUDA_TRY(cudaMemsetAsync(m->f_pairs, 0, sizeof(uint2) * m->f_pairs_n, m->ctx->stream));
        m->f_stamp = 0;
    }
    BatchStepArgs A = {};
    A.tok = m->tok, A.pos = m->pos, A.norm_final = m->norm_final, A.lm_head = m->lm_head;
    for (int l = 0; l < m->layers; l++) {
        A.Lw[l] = m->L[(size_t)l];
        int32_t rc = pair_interleaved(m, m->L[(size_t)l].w1, m->L[(size_t)l].w3, m->d_model, m->d_ff, &A.w13[l]);
        if (rc) return rc;
    }
    A.vocab = m->vocab, A.max_seq = m->max_seq, A.D = m->d_model, A.H = m->heads, A.layers = m->layers, A.F = m->d_ff, A.eps = m->eps;
    A.kv = p->kv, A.table = p->d_table, A.rope = p->d_rope, A.n_blocks = p->n_blocks, A.mbs = p->max_blocks_per_seq;
    A.idx = m->d_idx, A.n = n;
    uint2 *f = m->fb_pairs;
    A.xa = f, f += R * D;
    A.xb = f, f += R * D;
    A.ssa = f, f += R * parts;
    A.ssb = f, f += R * parts;
    A.qkv = f, f += R * 3 * D;
    A.att = f, f += R * D;
    A.act = f, f += R * F;
    A.cand = f;
    A.part = m->fb_part, A.tickets = m->fb_tickets;
    A.stamp0 = m->f_stamp;
    m->f_stamp += need;
    A.abort_word = reinterpret_cast<unsigned *>(m->fb_tickets + R * m->heads);
    A.status = m->ctx->d_status;
    A.logits = m->logits, A.next = m->d_next;
    batch_step_plan(A, m->ctx->sm_count, lens_host);
    JGPT_REQUIRE(A.nch_max <= std::min(32, fused_batch_max_chunks(m)), JGPT_ERR_ILLEGAL_STATE, "attention chunks %d exceed the scratch (%d)", A.nch_max,
                 fused_batch_max_chunks(m));
    return launch_decode_batch(m->ctx, A);
}

}  // namespace jgpt

using namespace jgpt;

#ifdef JGPT_B200_DECODE_TRACE
// Trace builds only: the step timeline (4 words per launch slot: first CTA in, last wait passed, last CTA out, unused).
extern "C" __attribute__((visibility("default"))) int32_t jgpt_debug_timeline_reset() {
    if (!g_timeline_buf) return 0;
    cudaDeviceSynchronize();
    std::vector<unsigned long long> init((size_t)4 * kTimelineSlots, 0ull);
    for (int i = 0; i < kTimelineSlots; i++) init[(size_t)4 * i] = ~0ull;
    cudaMemcpy(g_timeline_buf, init.data(), sizeof(unsigned long long) * init.size(), cudaMemcpyHostToDevice);
    cudaMemset(g_timeline_buf + 4 * kTimelineSlots, 0, sizeof(unsigned long long) * 256 * kTimelineSlots);
    return g_timeline_slot;
}
extern "C" __attribute__((visibility("default"))) int32_t jgpt_debug_timeline_read(unsigned long long *host, int32_t slots) {
    if (!g_timeline_buf) return 0;
    cudaDeviceSynchronize();
    const int n = std::min(slots, kTimelineSlots);
    cudaMemcpy(host, g_timeline_buf, sizeof(unsigned long long) * 4 * (size_t)n, cudaMemcpyDeviceToHost);
    return g_timeline_slot;
}
extern "C" __attribute__((visibility("default"))) int32_t jgpt_debug_timeline_read_sms(unsigned long long *host, int32_t slots) {
    if (!g_timeline_buf) return 0;
    cudaDeviceSynchronize();
    const int n = std::min(slots, kTimelineSlots);
    cudaMemcpy(host, g_timeline_buf + 4 * kTimelineSlots, sizeof(unsigned long long) * 256 * (size_t)n, cudaMemcpyDeviceToHost);
    return g_timeline_slot;
}
#endif

#define GET_MODEL(m, h)                                         \
    Model *m = model_registry().get(h);                         \
    JGPT_REQUIRE(m, JGPT_ERR_BAD_HANDLE, "bad model handle");   \
    JGPT_CUDA_TRY(make_current(m->ctx))

static int32_t check_pool(const Model *m, const Pool *p) {
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");
    JGPT_REQUIRE(p->ctx == m->ctx, JGPT_ERR_INVALID_ARGUMENT, "model and KV pool live on different contexts");
    // GptKvForward: "KvCacheGpu layer count mismatch" -> IllegalArgumentException
    JGPT_REQUIRE(p->layers == m->layers && p->heads == m->heads && p->dhead == m->d_model / m->heads, JGPT_ERR_INVALID_ARGUMENT,
                 "KV pool geometry (layers %d, heads %d, dhead %d) does not match the model", p->layers, p->heads, p->dhead);
    return JGPT_OK;
}

extern "C" {

// C[M,N] = A[M,K] . B[K,N], row-major fp32 device buffers, ordered on the context's stream
// (TensorOpsGPU.matmulGpuDevice, src/main/java/com/veles/llm/jgpt/TensorOpsGPU.java:1393).  Products with at
// least JGPT_B200_UMMA_MIN_ROWS rows (default 513: above what the decode-sized kernel takes) and K % 16 == 0, N % 4 == 0 take the tcgen05 kernel; their
// operand images live in stream-ordered scratch for the duration of the call.
int32_t jgpt_matmul_device(jgpt_ctx ctxh, const float *a_dev, const float *b_dev, float *c_dev, int32_t M, int32_t K, int32_t N) {
    Ctx *c = ctx_registry().get(ctxh);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(a_dev && b_dev && c_dev, JGPT_ERR_INVALID_ARGUMENT, "null buffer");
    JGPT_REQUIRE(M > 0 && K > 0 && N > 0, JGPT_ERR_INVALID_ARGUMENT, "matmul dimensions must be positive (M=%d K=%d N=%d)", M, K, N);
    JGPT_CUDA_TRY(make_current(c));
    const float *W[1] = {b_dev};
    float *C[1] = {c_dev};
    // Two getenv calls per call (a test knob that tests flip between calls; ~100 ns).  The stateless primitive has to
    // re-tile its weight operand on every call because nothing says the caller has not changed it -- the forward-step
    // entry points keep tiled weights cached instead.
    const int min_rows = env_int("JGPT_B200_UMMA_MIN_ROWS", 513);
    const int strict = env_int("JGPT_B200_STRICT_GEMM", 0);
    if (strict || min_rows <= 0 || M < min_rows || !umma::shape_ok(K, N))
        return gemm_small(c, strict, a_dev, M, K, N, 1, W, C, nullptr, nullptr);
    cudaStream_t st = c->stream;
    float *aimg = nullptr, *wimg = nullptr;
    JGPT_CUDA_TRY(cudaMallocAsync(&aimg, sizeof(float) * umma::activation_image_floats(M, K), st));
    cudaError_t e = cudaMallocAsync(&wimg, sizeof(float) * umma::weight_image_floats(K, N), st);
    if (e != cudaSuccess) {
        cudaFreeAsync(aimg, st);
        return fail(JGPT_ERR_OUT_OF_MEMORY, "matmul scratch: %s", cudaGetErrorString(e));
    }
    umma::Batch b{};
    b.Wimg[0] = wimg, b.C[0] = c_dev, b.R[0] = nullptr;
    int32_t rc = umma::pack_weight(b_dev, K, N, wimg, st);
    if (!rc) rc = umma::pack_activations(a_dev, nullptr, M, K, aimg, st);
    if (!rc) rc = umma::launch(aimg, b, 1, M, K, N, c->d_status, st);
    cudaFreeAsync(aimg, st);
    cudaFreeAsync(wimg, st);
    return rc;
}

int32_t jgpt_model_create(jgpt_ctx ctxh, int32_t vocab, int32_t max_seq_len, int32_t d_model, int32_t heads, int32_t layers,
                          int32_t d_ff, float rms_eps, int32_t max_rows, jgpt_model *out) {
    Ctx *c = ctx_registry().get(ctxh);
    JGPT_REQUIRE(c, JGPT_ERR_BAD_HANDLE, "bad context handle");
    JGPT_REQUIRE(out, JGPT_ERR_INVALID_ARGUMENT, "out is null");
    JGPT_REQUIRE(vocab > 0 && max_seq_len > 0 && d_model > 0 && heads > 0 && layers > 0 && d_ff > 0 && max_rows > 0,
                 JGPT_ERR_INVALID_ARGUMENT, "model dimensions must be positive");
    JGPT_REQUIRE(d_model % heads == 0, JGPT_ERR_INVALID_ARGUMENT, "d_model must be divisible by num_heads");
    JGPT_REQUIRE(d_model % 4 == 0, JGPT_ERR_UNSUPPORTED, "d_model must be a multiple of 4");
    JGPT_CUDA_TRY(make_current(c));
    Model *m = new Model();
    m->ctx = c, m->vocab = vocab, m->max_seq = max_seq_len, m->d_model = d_model, m->heads = heads, m->layers = layers;
    m->d_ff = d_ff, m->eps = rms_eps, m->max_rows = max_rows;
    m->strict = env_int("JGPT_B200_STRICT_GEMM", 0);
    m->umma_min_rows = env_int("JGPT_B200_UMMA_MIN_ROWS", 513);
    m->decode_graph_enabled = env_int("JGPT_B200_DECODE_GRAPH", 1);
    m->prefill_fast = env_int("JGPT_B200_PREFILL_EXACT", 0) ? 0 : 1;
    m->w_resident = env_int("JGPT_B200_W_RESIDENT", 1);
    m->k_split = env_int("JGPT_B200_K_SPLIT", 1);
    m->step_overlap = std::min(3, std::max(-1, env_int("JGPT_B200_STEP_OVERLAP", -1)));  // -1 = the default level
    m->fused_step = env_int("JGPT_B200_FUSED_STEP", 1);
    m->fused_batch = env_int("JGPT_B200_FUSED_BATCH", 0);  // measured slower than the multi-launch step so far: opt-in
    const size_t D = d_model, F = d_ff, V = vocab, R = max_rows;
    auto A = [&](float **p, size_t n) { return cudaMalloc(p, sizeof(float) * n); };
    JGPT_CUDA_TRY(A(&m->tok, V * D));
    JGPT_CUDA_TRY(A(&m->pos, (size_t)max_seq_len * D));
    JGPT_CUDA_TRY(A(&m->norm_final, D));
    JGPT_CUDA_TRY(A(&m->lm_head, D * V));
    // The layers' tensors live in ONE allocation, so that a single L2 access-policy window can cover them: a decode step
    // reads every weight once, and with the window they stay in L2 from step to step (set below).
    m->L.resize((size_t)layers);
    {
        auto up = [](size_t n) { return (n + 63) / 64 * 64; };  // 256-byte steps
        const size_t per_layer = 4 * up(D * D) + 3 * up(D * F) + 2 * up(D);
        m->arena_floats = per_layer * (size_t)layers;
        JGPT_CUDA_TRY(A(&m->arena, m->arena_floats));
        float *w = m->arena;
        auto take = [&](size_t n) {
            float *r = w;
            w += up(n);
            return r;
        };
        for (auto &y : m->L) {
            y.wq = take(D * D), y.wk = take(D * D), y.wv = take(D * D), y.wo = take(D * D);
            y.w1 = take(D * F), y.w2 = take(F * D), y.w3 = take(D * F);
            y.norm1 = take(D), y.norm2 = take(D);
        }
    }
    // JGPT_B200_L2_PERSIST=1 (default 0): set part of L2 aside for the window (a limit of this process's context, not a
    // device setting) and mark the layer weights as persisting for everything launched on the context's stream.
    // Measured on the JGPT-35M shapes (71 MB of layer weights, 79 MB may be set aside): the one-launch step called once
    // per token 0.169 against 0.179 ms, 127 steps in one launch 133.9 against 135.7 us per token, the batch-64 step
    // unchanged, the batch-256 step 3 % slower - too little to take 71 MB of L2 from everything else by default.
    if (env_int("JGPT_B200_L2_PERSIST", 0)) {
        int max_persist = 0, max_window = 0;
        cudaDeviceGetAttribute(&max_persist, cudaDevAttrMaxPersistingL2CacheSize, c->device);
        cudaDeviceGetAttribute(&max_window, cudaDevAttrMaxAccessPolicyWindowSize, c->device);
        const size_t bytes = sizeof(float) * m->arena_floats;
        if (max_persist > 0 && max_window > 0) {
            const size_t set_aside = std::min(bytes, (size_t)max_persist), window = std::min(bytes, (size_t)max_window);
            size_t cur = 0;
            cudaDeviceGetLimit(&cur, cudaLimitPersistingL2CacheSize);
            if (cur < set_aside) cudaDeviceSetLimit(cudaLimitPersistingL2CacheSize, set_aside);
            cudaStreamAttrValue av = {};
            av.accessPolicyWindow.base_ptr = m->arena;
            av.accessPolicyWindow.num_bytes = window;
            av.accessPolicyWindow.hitRatio = (float)std::min(1.0, (double)set_aside / (double)window);
            av.accessPolicyWindow.hitProp = cudaAccessPropertyPersisting;
            av.accessPolicyWindow.missProp = cudaAccessPropertyNormal;
            if (cudaStreamSetAttribute(c->stream, cudaStreamAttributeAccessPolicyWindow, &av) == cudaSuccess) m->l2_window = true;
            cudaGetLastError();  // a refusal leaves the defaults in place
        }
    }
    JGPT_CUDA_TRY(A(&m->x, R * D));
    JGPT_CUDA_TRY(A(&m->xn, R * D));
    JGPT_CUDA_TRY(A(&m->q, R * D));
    JGPT_CUDA_TRY(A(&m->k, R * D));
    JGPT_CUDA_TRY(A(&m->v, R * D));
    JGPT_CUDA_TRY(A(&m->att, R * D));
    JGPT_CUDA_TRY(A(&m->h1, R * F));
    JGPT_CUDA_TRY(A(&m->g, R * F));
    JGPT_CUDA_TRY(cudaMalloc(&m->d_idx, sizeof(int) * 5 * R));
    JGPT_CUDA_TRY(cudaHostAlloc(&m->h_idx, sizeof(int) * 5 * R, cudaHostAllocDefault));
    JGPT_CUDA_TRY(cudaMalloc(&m->d_next, sizeof(int) * R));
    JGPT_CUDA_TRY(cudaHostAlloc(&m->h_next, sizeof(int) * R, cudaHostAllocDefault));
    JGPT_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&m->hd_idx), m->h_idx, 0));
    JGPT_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&m->hd_next), m->h_next, 0));
    JGPT_CUDA_TRY(cudaHostGetDevicePointer(reinterpret_cast<void **>(&m->hd_status), m->ctx->h_status, 0));
    JGPT_CUDA_TRY(cudaMalloc(&m->d_rowsel, sizeof(int) * R));
    JGPT_CUDA_TRY(cudaHostAlloc(&m->h_u, sizeof(float) * R, cudaHostAllocDefault));
    JGPT_CUDA_TRY(A(&m->d_u, R));
    JGPT_CUDA_TRY(A(&m->ss_a, R * ((D + 31) / 32)));
    JGPT_CUDA_TRY(A(&m->ss_b, R * ((D + 31) / 32)));
    *out = model_registry().add(m);
    return JGPT_OK;
}

int32_t jgpt_model_destroy(jgpt_model h) {
    GET_MODEL(m, h);
    cudaStreamSynchronize(m->ctx->stream);
    model_registry().remove(m);
    cudaFree(m->tok), cudaFree(m->pos), cudaFree(m->norm_final), cudaFree(m->lm_head);
    if (m->l2_window) {  // take the window off the stream and give the persisting lines back
        cudaStreamAttrValue av = {};
        av.accessPolicyWindow.num_bytes = 0;
        cudaStreamSetAttribute(m->ctx->stream, cudaStreamAttributeAccessPolicyWindow, &av);
        cudaCtxResetPersistingL2Cache();
        cudaGetLastError();
    }
    cudaFree(m->arena);
    cudaFree(m->x), cudaFree(m->xn), cudaFree(m->q), cudaFree(m->k), cudaFree(m->v), cudaFree(m->att), cudaFree(m->h1);
    cudaFree(m->g), cudaFree(m->logits), cudaFree(m->d_idx), cudaFree(m->d_next), cudaFree(m->d_rowsel);
    cudaFreeHost(m->h_idx), cudaFreeHost(m->h_next);
    drop_weight_images(m);  // and the decode graphs
    cudaFree(m->aimg), cudaFree(m->aimg2), cudaFree(m->ss_a), cudaFree(m->ss_b), cudaFree(m->d_u), cudaFree(m->d_samp);
    cudaFreeHost(m->h_u);
    cudaFree(m->f_pairs), cudaFree(m->f_ints), cudaFreeHost(m->h_fused);
    cudaFree(m->fb_pairs), cudaFree(m->fb_part), cudaFree(m->fb_tickets);
    delete m;
    return JGPT_OK;
}

int32_t jgpt_model_num_tensors(jgpt_model h, int32_t *n_out) {
    GET_MODEL(m, h);
    JGPT_REQUIRE(n_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    *n_out = num_tensors(m);
    return JGPT_OK;
}

int32_t jgpt_model_set_tensor(jgpt_model h, int32_t idx, const float *host, uint64_t n_floats) {
    GET_MODEL(m, h);
    JGPT_REQUIRE(idx >= 0 && idx < num_tensors(m), JGPT_ERR_OUT_OF_RANGE, "tensor %d outside [0,%d)", idx, num_tensors(m));
    uint64_t count = 0;
    float *dst = tensor_ptr(m, idx, &count);
    JGPT_REQUIRE(host && n_floats == count, JGPT_ERR_INVALID_ARGUMENT, "tensor %d holds %llu floats, got %llu", idx,
                 (unsigned long long)count, (unsigned long long)n_floats);
    JGPT_CUDA_TRY(cudaMemcpyAsync(dst, host, sizeof(float) * count, cudaMemcpyHostToDevice, m->ctx->stream));
    JGPT_CUDA_TRY(cudaStreamSynchronize(m->ctx->stream));
    drop_weight_images(m);  // rebuilt from the new values on the next prefill-sized product
    return JGPT_OK;
}

// veles.weights.v1 (reader: src/main/java/com/veles/llm/jgpt/model/GptModelWeightsLoader.java:58-81;
// writer: training/LlmTrainerCheckpointIo.java:129-140): Java writeUTF tag, int32 BE tensor count, per tensor
// int32 BE rank, dims, big-endian fp32 payload.
int32_t jgpt_model_load_weights(jgpt_model h, const char *path) {
    GET_MODEL(m, h);
    JGPT_REQUIRE(path, JGPT_ERR_INVALID_ARGUMENT, "null path");
    FILE *f = fopen(path, "rb");
    if (!f) return fail(JGPT_ERR_IO, "cannot open %s", path);
    auto rd32 = [&](uint32_t *v) {
        unsigned char b[4];
        if (fread(b, 1, 4, f) != 4) return false;
        *v = ((uint32_t)b[0] << 24) | ((uint32_t)b[1] << 16) | ((uint32_t)b[2] << 8) | b[3];
        return true;
    };
    unsigned char hdr[18];
    if (fread(hdr, 1, 18, f) != 18 || hdr[0] != 0 || hdr[1] != 16 || memcmp(hdr + 2, "veles.weights.v1", 16) != 0) {
        fclose(f);
        return fail(JGPT_ERR_IO, "%s is not a veles.weights.v1 file", path);
    }
    uint32_t n = 0;
    if (!rd32(&n) || (int)n != num_tensors(m)) {
        fclose(f);
        return fail(JGPT_ERR_INVALID_ARGUMENT, "%s holds %u tensors, the model has %d", path, n, num_tensors(m));
    }
    cudaStreamSynchronize(m->ctx->stream);
    drop_weight_images(m);
    std::vector<float> buf;
    for (int i = 0; i < (int)n; i++) {
        uint64_t count = 0;
        float *dst = tensor_ptr(m, i, &count);
        uint32_t rank = 0;
        uint64_t prod = 1;
        bool ok = rd32(&rank) && rank >= 1 && rank <= 4;
        for (uint32_t d = 0; ok && d < rank; d++) {
            uint32_t dim = 0;
            ok = rd32(&dim);
            prod *= dim;
        }
        if (!ok || prod != count) {
            fclose(f);
            return fail(JGPT_ERR_INVALID_ARGUMENT, "%s: tensor %d has %llu elements, expected %llu", path, i,
                        (unsigned long long)prod, (unsigned long long)count);
        }
        buf.resize(count);
        if (fread(buf.data(), 4, count, f) != count) {
            fclose(f);
            return fail(JGPT_ERR_IO, "%s: truncated in tensor %d", path, i);
        }
        for (uint64_t j = 0; j < count; j++) {
            uint32_t u;
            memcpy(&u, &buf[j], 4);
            u = __builtin_bswap32(u);
            memcpy(&buf[j], &u, 4);
        }
        cudaError_t e = cudaMemcpy(dst, buf.data(), sizeof(float) * count, cudaMemcpyHostToDevice);
        if (e != cudaSuccess) {
            fclose(f);
            return fail(JGPT_ERR_CUDA, "upload of tensor %d: %s", i, cudaGetErrorString(e));
        }
    }
    fclose(f);
    return JGPT_OK;
}

// Tensor idx back on the host (GPTModel.getParameters() order), and the whole set as a veles.weights.v1 file: the
// writer of src/main/java/com/veles/llm/jgpt/training/LlmTrainerCheckpointIo.java:129-140 (writeUTF tag, int32 BE
// count, per tensor int32 BE rank and dims, big-endian fp32 payload; matrices rank 2, norm gains rank 1).
int32_t jgpt_model_get_tensor(jgpt_model h, int32_t idx, float *host, uint64_t n_floats) {
    GET_MODEL(m, h);
    JGPT_REQUIRE(idx >= 0 && idx < num_tensors(m), JGPT_ERR_OUT_OF_RANGE, "tensor %d outside [0,%d)", idx, num_tensors(m));
    uint64_t count = 0;
    const float *src = tensor_ptr(m, idx, &count);
    JGPT_REQUIRE(host && n_floats == count, JGPT_ERR_INVALID_ARGUMENT, "tensor %d holds %llu floats, got %llu", idx,
                 (unsigned long long)count, (unsigned long long)n_floats);
    JGPT_CUDA_TRY(cudaMemcpyAsync(host, src, sizeof(float) * count, cudaMemcpyDeviceToHost, m->ctx->stream));
    JGPT_CUDA_TRY(cudaStreamSynchronize(m->ctx->stream));
    return JGPT_OK;
}

int32_t jgpt_model_save_weights(jgpt_model h, const char *path) {
    GET_MODEL(m, h);
    JGPT_REQUIRE(path, JGPT_ERR_INVALID_ARGUMENT, "null path");
    FILE *f = fopen(path, "wb");
    if (!f) return fail(JGPT_ERR_IO, "cannot create %s", path);
    auto wr32 = [&](uint32_t v) {
        const unsigned char b[4] = {(unsigned char)(v >> 24), (unsigned char)(v >> 16), (unsigned char)(v >> 8), (unsigned char)v};
        return fwrite(b, 1, 4, f) == 4;
    };
    const unsigned char len[2] = {0, 16};
    bool ok = fwrite(len, 1, 2, f) == 2 && fwrite("veles.weights.v1", 1, 16, f) == 16 && wr32((uint32_t)num_tensors(m));
    const uint32_t D = (uint32_t)m->d_model, F = (uint32_t)m->d_ff, V = (uint32_t)m->vocab;
    std::vector<float> buf;
    for (int i = 0; ok && i < num_tensors(m); i++) {
        uint64_t count = 0;
        const float *src = tensor_ptr(m, i, &count);
        uint32_t d0 = 0, d1 = 0;  // d1 == 0: rank 1
        const int n = num_tensors(m);
        if (i == 0) d0 = V, d1 = D;
        else if (i == 1) d0 = (uint32_t)m->max_seq, d1 = D;
        else if (i == n - 2) d0 = D;
        else if (i == n - 1) d0 = D, d1 = V;
        else switch ((i - 2) % 9) {
            case 0: case 1: case 2: case 3: d0 = D, d1 = D; break;
            case 4: case 6: d0 = D, d1 = F; break;
            case 5: d0 = F, d1 = D; break;
            default: d0 = D; break;
        }
        buf.resize(count);
        const cudaError_t e = cudaMemcpy(buf.data(), src, sizeof(float) * count, cudaMemcpyDeviceToHost);
        if (e != cudaSuccess) {
            fclose(f);
            return fail(JGPT_ERR_CUDA, "download of tensor %d: %s", i, cudaGetErrorString(e));
        }
        ok = wr32(d1 ? 2u : 1u) && wr32(d0) && (!d1 || wr32(d1));
        for (uint64_t j = 0; j < count; j++) {
            uint32_t u;
            memcpy(&u, &buf[j], 4);
            u = __builtin_bswap32(u);
            memcpy(&buf[j], &u, 4);
        }
        ok = ok && fwrite(buf.data(), 4, count, f) == count;
    }
    ok = (fclose(f) == 0) && ok;
    if (!ok) return fail(JGPT_ERR_IO, "short write to %s", path);
    return JGPT_OK;
}

// Batched prefill: n sequences, sequence i = rows [seq_starts[i], seq_starts[i+1]) of ids_host, RoPE /
// position rows rope_offsets[i] + r, cache slots 0..S_i-1.  last_logits_host [n, vocab] and
// next_tokens_host [n] (argmax of the last row) may be NULL.  Sets every sequence's length to S_i.
int32_t jgpt_forward_prefill_batch(jgpt_model h, jgpt_kvpool poolh, const int32_t *seq_ids_host, const int32_t *seq_starts_host,
                                   const int32_t *ids_host, const int32_t *rope_offsets_host, int32_t n, float *all_logits_host,
                                   float *last_logits_host, int32_t *next_tokens_host) {
    GET_MODEL(m, h);
    Pool *p = pool_registry().get(poolh);
    int32_t rc = check_pool(m, p);
    if (rc) return rc;
    JGPT_REQUIRE(n >= 1 && seq_ids_host && seq_starts_host && ids_host && rope_offsets_host, JGPT_ERR_INVALID_ARGUMENT,
                 "null pointer or empty batch");
    const int rows = seq_starts_host[n];
    JGPT_REQUIRE(seq_starts_host[0] == 0 && rows >= 1, JGPT_ERR_INVALID_ARGUMENT, "seq_starts must begin at 0");
    JGPT_REQUIRE(rows <= m->max_rows, JGPT_ERR_INVALID_ARGUMENT, "%d prompt rows exceed the model workspace (%d rows)", rows,
                 m->max_rows);
    JGPT_REQUIRE(!all_logits_host || n == 1, JGPT_ERR_INVALID_ARGUMENT, "all-row logits are available for one sequence at a time");
    int *ids = m->h_idx, *posrow = m->h_idx + rows;  // packed [2][rows]
    for (int i = 0; i < n; i++) {
        const int s = seq_ids_host[i], S = seq_starts_host[i + 1] - seq_starts_host[i], ro = rope_offsets_host[i];
        JGPT_REQUIRE(s >= 0 && s < p->max_seqs && p->seqs[(size_t)s].used, JGPT_ERR_OUT_OF_RANGE, "sequence %d is not allocated", s);
        // forwardPrefill: seq_len > max_seq_len -> IllegalArgumentException; position rows must stay inside the table
        JGPT_REQUIRE(S >= 1 && S <= m->max_seq, JGPT_ERR_INVALID_ARGUMENT, "seq_len %d > max_seq_len %d", S, m->max_seq);
        JGPT_REQUIRE(ro >= 0 && ro + S <= m->max_seq, JGPT_ERR_INVALID_ARGUMENT, "position rows [%d, %d) outside the table of %d", ro,
                     ro + S, m->max_seq);
        for (int r = 0; r < S; r++) {
            const int id = ids_host[seq_starts_host[i] + r];
            JGPT_REQUIRE(id >= 0 && id < m->vocab, JGPT_ERR_INVALID_ARGUMENT, "token id %d outside [0,%d)", id, m->vocab);
            ids[seq_starts_host[i] + r] = id;
            posrow[seq_starts_host[i] + r] = ro + r;
        }
    }
    for (int i = 0; i < n; i++) {
        rc = jgpt_seq_reserve(poolh, seq_ids_host[i], seq_starts_host[i + 1] - seq_starts_host[i]);
        if (rc) return rc;
    }
    cudaStream_t st = m->ctx->stream;
    JGPT_CUDA_TRY(cudaMemcpyAsync(m->d_idx, m->h_idx, sizeof(int) * 2 * (size_t)rows, cudaMemcpyHostToDevice, st));
    embed_pos_kernel<<<rows, 128, 0, st>>>(m->tok, m->pos, m->d_idx, m->d_idx + rows, m->x, m->d_model, m->ss_a);
    // d_head 16: one head is exactly one 16-wide k tile of the Wo operand image, which the attention kernel can
    // then write itself, and the Q,K,V product can append K / V to the paged store from its epilogue
    PagedAppendArgs pa{};
    const PagedAppendArgs *paged = nullptr;
    if (p->dhead == 16 && m->d_model == p->heads * 16) {
        int max_S = 0, n_rows = 0;
        rc = prefill_upload_descriptors(p, seq_ids_host, seq_starts_host, rope_offsets_host, n, &max_S, &n_rows);
        if (rc) return rc;
        pa.kv = p->kv, pa.table = p->d_table, pa.rope = p->d_rope;
        pa.seqs = reinterpret_cast<const PrefillSeq *>(p->d_prefill_desc), pa.status = p->ctx->d_status;
        pa.n_seqs = n, pa.H = p->heads, pa.layer = 0, pa.n_blocks = p->n_blocks, pa.mbs = p->max_blocks_per_seq;
        pa.max_positions = p->max_positions;
        paged = &pa;
    }
    rc = run_layers(m, rows, paged, [&](int l, float *image, bool kv_in_cache) {
        return launch_attn_prefill(p, l, m->q, m->k, m->v, seq_ids_host, seq_starts_host, rope_offsets_host, n, m->att, image,
                                   kv_in_cache, m->prefill_fast);
    });
    if (rc) return rc;
    int n_sel = 0;
    if (!all_logits_host) {
        std::vector<int> sel((size_t)n);
        for (int i = 0; i < n; i++) sel[(size_t)i] = seq_starts_host[i + 1] - 1;
        JGPT_CUDA_TRY(cudaMemcpyAsync(m->d_rowsel, sel.data(), sizeof(int) * (size_t)n, cudaMemcpyHostToDevice, st));
        n_sel = n;
    }
    rc = lm_head(m, rows, n_sel);
    if (rc) return rc;
    const int out_rows = n_sel ? n_sel : rows;
    if (all_logits_host)
        JGPT_CUDA_TRY(cudaMemcpyAsync(all_logits_host, m->logits, sizeof(float) * (size_t)rows * m->vocab, cudaMemcpyDeviceToHost, st));
    if (last_logits_host) {
        const float *src = all_logits_host ? m->logits + (size_t)(rows - 1) * m->vocab : m->logits;
        const int nrow = all_logits_host ? 1 : n;
        JGPT_CUDA_TRY(cudaMemcpyAsync(last_logits_host, src, sizeof(float) * (size_t)nrow * m->vocab, cudaMemcpyDeviceToHost, st));
    }
    JGPT_CUDA_TRY(cudaMemcpyAsync(m->h_next, m->d_next, sizeof(int) * (size_t)out_rows, cudaMemcpyDeviceToHost, st));
    JGPT_CUDA_TRY(status_enqueue_read(m->ctx));
    JGPT_CUDA_TRY(cudaStreamSynchronize(st));
    // a kernel of the step recorded a failed self-check: no tokens, no length change
    rc = status_check_after_sync(m->ctx, p, "jgpt_forward_prefill");
    if (rc) return rc;
    if (next_tokens_host)
        for (int i = 0; i < n; i++) next_tokens_host[i] = all_logits_host ? m->h_next[rows - 1] : m->h_next[i];
    for (int i = 0; i < n; i++) {  // cache.setLength(seqLen)
        rc = jgpt_seq_set_length(poolh, seq_ids_host[i], seq_starts_host[i + 1] - seq_starts_host[i]);
        if (rc) return rc;
    }
    return JGPT_OK;
}

int32_t jgpt_forward_prefill(jgpt_model h, jgpt_kvpool poolh, int32_t seq, const int32_t *ids_host, int32_t S, int32_t rope_offset,
                             float *logits_host, float *last_logits_host, int32_t *next_token_host) {
    const int32_t starts[2] = {0, S};
    JGPT_REQUIRE(S >= 1, JGPT_ERR_INVALID_ARGUMENT, "empty prompt");
    return jgpt_forward_prefill_batch(h, poolh, &seq, starts, ids_host, &rope_offset, 1, logits_host, last_logits_host,
                                      next_token_host);
}

static int32_t forward_decode_impl(jgpt_model h, jgpt_kvpool poolh, const int32_t *seq_ids_host, const int32_t *ids_host,
                                   const int32_t *cache_len_before_host, const int32_t *rope_pos_host, int32_t n, float *logits_host,
                                   int32_t *next_tokens_host, const SampleSpec &spec, const float *u01_host) {
    GET_MODEL(m, h);
    Pool *p = pool_registry().get(poolh);
    int32_t rc = check_pool(m, p);
    if (rc) return rc;
    JGPT_REQUIRE(n >= 1 && seq_ids_host && ids_host && cache_len_before_host && rope_pos_host, JGPT_ERR_INVALID_ARGUMENT,
                 "null pointer or empty batch");
    JGPT_REQUIRE(n <= m->max_rows, JGPT_ERR_INVALID_ARGUMENT, "%d rows exceed the model workspace (%d rows)", n, m->max_rows);
    const int R = n;  // packed [5][n]: ids, position rows, sequence ids, RoPE positions, lengths
    int *ids = m->h_idx, *posrow = ids + R, *sid = posrow + R, *rp = sid + R, *lens = rp + R;
    int max_len = 1;
    for (int i = 0; i < n; i++) {
        const int s = seq_ids_host[i];
        JGPT_REQUIRE(s >= 0 && s < p->max_seqs && p->seqs[(size_t)s].used, JGPT_ERR_OUT_OF_RANGE, "sequence %d is not allocated", s);
        for (int j = 0; j < i; j++)
            JGPT_REQUIRE(seq_ids_host[j] != s, JGPT_ERR_INVALID_ARGUMENT, "sequence %d appears twice in one decode step", s);
        // forwardDecode: cache.length() != cacheLenBefore -> IllegalStateException; full cache -> IllegalStateException
        JGPT_REQUIRE(p->seqs[(size_t)s].len == cache_len_before_host[i], JGPT_ERR_ILLEGAL_STATE, "KV cache length %d != cacheLenBefore %d",
                     p->seqs[(size_t)s].len, cache_len_before_host[i]);
        JGPT_REQUIRE(cache_len_before_host[i] < m->max_seq && cache_len_before_host[i] < p->max_blocks_per_seq * kBlockTokens,
                     JGPT_ERR_ILLEGAL_STATE, "KV cache of sequence %d is full (%d tokens)", s, cache_len_before_host[i]);
        JGPT_REQUIRE(ids_host[i] >= 0 && ids_host[i] < m->vocab, JGPT_ERR_INVALID_ARGUMENT, "token id %d outside [0,%d)", ids_host[i],
                     m->vocab);
        // A pool created with the reference's geometry (max_positions == max_seq_len) rejects positions beyond the
        // context, as PositionEmbedding does.  A pool with a longer RoPE table opts in to the rolling window: RoPE at
        // the absolute position, position-table row = position mod max_seq_len.
        JGPT_REQUIRE(rope_pos_host[i] >= 0 && rope_pos_host[i] < p->max_positions,
                     JGPT_ERR_INVALID_ARGUMENT, "position %d outside the table of %d rows", rope_pos_host[i],
                     std::min(m->max_seq, p->max_positions));
        ids[i] = ids_host[i], posrow[i] = rope_pos_host[i] % m->max_seq, sid[i] = s, rp[i] = rope_pos_host[i], lens[i] = cache_len_before_host[i] + 1;
        max_len = std::max(max_len, lens[i]);
    }
    for (int i = 0; i < n; i++) {
        rc = jgpt_seq_reserve(poolh, seq_ids_host[i], cache_len_before_host[i] + 1);
        if (rc) return rc;
    }
    cudaStream_t st = m->ctx->stream;
    // The attention sizes its split for an upper bound of the lengths; a bound in steps of 128 tokens keeps the
    // launch shapes of consecutive steps identical (the exact lengths travel in d_idx).
    const int cap = std::min(m->max_seq, p->max_blocks_per_seq * kBlockTokens);
    const int len_bucket = std::min(cap, (max_len + 127) / 128 * 128);
    const bool sampled = spec.temperature > 0.f;
    if (sampled) {
        JGPT_REQUIRE(u01_host, JGPT_ERR_INVALID_ARGUMENT, "sampling needs one uniform draw per row");
        for (int i = 0; i < n; i++) m->h_u[i] = u01_host[i];
        rc = ensure_sample_work(m, n);  // before any capture: it may allocate
        if (rc) return rc;
    }
    // Greedy decode-sized steps move their few words themselves: the embedding kernel fetches the rows' descriptors from
    // the page-locked block, the argmax kernel leaves ids and status word in the host mirrors (three copies less per step;
    // the descriptor copy alone moved 5 R words whatever the batch).  JGPT_B200_STEP_COPIES=1: the copies.
    static const int step_copies = env_int("JGPT_B200_STEP_COPIES", 0);
    const bool no_copies = !sampled && !step_copies && small_mode(m, n);
    auto enqueue = [&]() -> int32_t {
        if (!no_copies) JGPT_CUDA_TRY(cudaMemcpyAsync(m->d_idx, m->h_idx, sizeof(int) * 5 * (size_t)R, cudaMemcpyHostToDevice, st));
        if (sampled) JGPT_CUDA_TRY(cudaMemcpyAsync(m->d_u, m->h_u, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, st));
        const bool chain_early = small_mode(m, n) && step_overlap_level(m, n) >= 3;
        m->first_launch_early = chain_early;
        if (no_copies) embed_pos_kernel<<<n, 128, 0, st>>>(m->tok, m->pos, nullptr, nullptr, m->x, m->d_model, m->ss_a, m->hd_idx, m->d_idx, R);
        else embed_pos_kernel<<<n, 128, 0, st>>>(m->tok, m->pos, m->d_idx, m->d_idx + R, m->x, m->d_model, m->ss_a);
        int32_t r2 = run_layers(m, n, nullptr, [&](int l, float *, bool) {
            return launch_attn_decode(p, l, 1, m->q, m->k, m->v, m->d_idx + 2 * R, m->d_idx + 3 * R, m->d_idx + 4 * R, n, len_bucket, m->att,
                                      (small_mode(m, n) && step_overlap_level(m, n) >= 1) ? 2 : -1);
        });
        m->first_launch_early = false;
        if (r2) return r2;
        r2 = lm_head(m, n, 0, spec, no_copies, chain_early);
        if (r2) return r2;
        if (!no_copies) {
            JGPT_CUDA_TRY(cudaMemcpyAsync(m->h_next, m->d_next, sizeof(int) * (size_t)n, cudaMemcpyDeviceToHost, st));
            JGPT_CUDA_TRY(status_enqueue_read(m->ctx));  // part of the replayed graph too
        }
        return JGPT_OK;
    };
    Model::DecodeGraph *slot = nullptr;
    // One cooperative launch for the whole step where that form exists and is switched on.  A device that cannot keep the
    // grid resident (fewer SMs than the context was sized for: MPS with a thread percentage, a green context) refuses the
    // launch: the form is switched off for this model and the step below runs as separate launches.
    bool one_launch = false;
    const int form = fused_ok(m, p, n) ? 1 : (fused_batch_ok(m, p, n) ? 2 : 0);
    if (form) {
        if ((rc = form == 1 ? ensure_fused(m) : ensure_fused_batch(m))) return rc;
        if ((rc = ensure_logits(m, n))) return rc;
        // the small form takes the rows' descriptors in its launch parameters and writes greedy tokens to h_next itself
        if (form == 2) JGPT_CUDA_TRY(cudaMemcpyAsync(m->d_idx, m->h_idx, sizeof(int) * 5 * (size_t)R, cudaMemcpyHostToDevice, st));
        if (sampled) JGPT_CUDA_TRY(cudaMemcpyAsync(m->d_u, m->h_u, sizeof(float) * (size_t)n, cudaMemcpyHostToDevice, st));
        rc = form == 1 ? fused_enqueue(m, p, n, 1, 0, max_len, m->d_next, m->h_idx, sampled ? nullptr : m->hd_next, nullptr)
                       : fused_batch_enqueue(m, p, n, lens);
        if (rc == JGPT_ERR_UNSUPPORTED) {
            (form == 1 ? m->fused_step : m->fused_batch) = 0;
        } else if (rc) {
            return rc;
        } else {
            if (sampled) {
                sample_kernel<<<n, 256, 0, st>>>(m->logits, m->d_samp, m->vocab, spec.temperature, spec.top_k, m->d_u, m->d_next);
                JGPT_CUDA_TRY(cudaGetLastError());
            }
            if (form == 2 || sampled) JGPT_CUDA_TRY(cudaMemcpyAsync(m->h_next, m->d_next, sizeof(int) * (size_t)n, cudaMemcpyDeviceToHost, st));
            JGPT_CUDA_TRY(status_enqueue_read(m->ctx));
            one_launch = true;
        }
    }
    if (one_launch) {
    } else if (m->decode_graph_enabled && small_mode(m, n)) {
        // Key: the pool object and its generation (unique per pool, bumped whenever a device buffer the kernels are
        // handed is reallocated), every other buffer address baked into the captured launches, and the pool geometry.
        auto make_key = [&]() {
            Model::DecodeGraph k;
            const void *key[8] = {p, reinterpret_cast<const void *>(p->generation), p->kv, p->d_table, p->d_rope, m->logits, m->d_idx, m->d_samp};
            for (int i = 0; i < 8; i++) k.key[i] = key[i];
            k.temperature = sampled ? spec.temperature : 0.f, k.top_k = sampled ? spec.top_k : 0;
            k.n = n, k.len_bucket = len_bucket, k.geom[0] = p->n_blocks, k.geom[1] = p->max_blocks_per_seq, k.geom[2] = p->heads;
            k.geom[3] = p->max_seqs, k.geom[4] = p->max_positions;
            return k;
        };
        Model::DecodeGraph want = make_key();
        for (auto &g : m->decode_graphs)
            if (g.n == want.n && g.len_bucket == want.len_bucket && g.temperature == want.temperature && g.top_k == want.top_k &&
                memcmp(g.key, want.key, sizeof(want.key)) == 0 &&
                memcmp(g.geom, want.geom, sizeof(want.geom)) == 0)
                slot = &g;
        if (!slot) {  // first time: run eagerly (this also sizes every grow-only buffer the step needs)
            if (m->decode_graphs.size() >= 32) {
                size_t oldest = 0;
                for (size_t i = 1; i < m->decode_graphs.size(); i++)
                    if (m->decode_graphs[i].last_use < m->decode_graphs[oldest].last_use) oldest = i;
                if (m->decode_graphs[oldest].exec) cudaGraphExecDestroy(m->decode_graphs[oldest].exec);
                m->decode_graphs.erase(m->decode_graphs.begin() + (long)oldest);
            }
            rc = enqueue();
            want = make_key();  // after the eager run: it may have grown the pool's split scratch (new generation)
            want.last_use = ++m->decode_graph_clock;
            m->decode_graphs.push_back(want);
        } else {
            slot->last_use = ++m->decode_graph_clock;
            if (!slot->exec && !slot->failed) {  // second time: capture
                cudaGraph_t g = nullptr;
                int32_t crc = JGPT_OK;
                if (cudaStreamBeginCapture(st, cudaStreamCaptureModeThreadLocal) == cudaSuccess) {
                    crc = enqueue();
                    const cudaError_t e = cudaStreamEndCapture(st, &g);
                    if (crc == JGPT_OK && e == cudaSuccess && g && cudaGraphInstantiate(&slot->exec, g, 0) != cudaSuccess) slot->exec = nullptr;
                    if (g) cudaGraphDestroy(g);
                }
                if (!slot->exec) {
                    slot->failed = true;
                    cudaGetLastError();  // the refused capture leaves an error behind; the eager run below reports real ones
                }
            }
            if (slot->exec) {
                const cudaError_t e = cudaGraphLaunch(slot->exec, st);
                rc = e == cudaSuccess ? JGPT_OK : fail(JGPT_ERR_CUDA, "cudaGraphLaunch: %s", cudaGetErrorString(e));
            } else {
                rc = enqueue();
            }
        }
    } else {
        rc = enqueue();
    }
    if (rc) return rc;
    if (logits_host)
        JGPT_CUDA_TRY(cudaMemcpyAsync(logits_host, m->logits, sizeof(float) * (size_t)n * m->vocab, cudaMemcpyDeviceToHost, st));
    JGPT_CUDA_TRY(cudaStreamSynchronize(st));
    // a kernel of the step recorded a failed self-check: no tokens, no length change
    rc = status_check_after_sync(m->ctx, p, "jgpt_forward_decode");
    if (rc) {
        fused_batch_reset(m);
        return rc;
    }
    if (next_tokens_host)
        for (int i = 0; i < n; i++) next_tokens_host[i] = m->h_next[i];
    for (int i = 0; i < n; i++) {  // cache.setLength(cacheLenBefore + 1)
        rc = jgpt_seq_set_length(poolh, seq_ids_host[i], cache_len_before_host[i] + 1);
        if (rc) return rc;
    }
    return JGPT_OK;
}

int32_t jgpt_forward_decode(jgpt_model h, jgpt_kvpool poolh, const int32_t *seq_ids_host, const int32_t *ids_host,
                            const int32_t *cache_len_before_host, const int32_t *rope_pos_host, int32_t n, float *logits_host,
                            int32_t *next_tokens_host) {
    return forward_decode_impl(h, poolh, seq_ids_host, ids_host, cache_len_before_host, rope_pos_host, n, logits_host,
                               next_tokens_host, SampleSpec(), nullptr);
}

// forwardDecode + sampleNextToken(logits, temperature, topK) in one call, the sampler on the device: no logits
// cross PCIe.  u01_host[n]: the uniform draw of each row.  temperature <= 0: greedy (top_k does not change an argmax).
int32_t jgpt_forward_decode_sample(jgpt_model h, jgpt_kvpool poolh, const int32_t *seq_ids_host, const int32_t *ids_host,
                                   const int32_t *cache_len_before_host, const int32_t *rope_pos_host, int32_t n, float temperature,
                                   int32_t top_k, const float *u01_host, int32_t *next_tokens_host) {
    JGPT_REQUIRE(next_tokens_host, JGPT_ERR_INVALID_ARGUMENT, "null output");
    SampleSpec spec;
    spec.temperature = temperature, spec.top_k = top_k;
    return forward_decode_impl(h, poolh, seq_ids_host, ids_host, cache_len_before_host, rope_pos_host, n, nullptr, next_tokens_host,
                               spec, u01_host);
}

int32_t jgpt_model_next_tokens_device(jgpt_model h, const int32_t **dev_out) {
    GET_MODEL(m, h);
    JGPT_REQUIRE(dev_out, JGPT_ERR_INVALID_ARGUMENT, "null output");
    *dev_out = m->d_next;
    return JGPT_OK;
}

// sampleNextToken on host logits (src/main/java/com/veles/llm/jgpt/model/GptAutoregressiveGenerator.java:208-286):
// temperature divide, stable top-k by (logit desc, index asc), softmax, inverse CDF with the supplied uniform
// draw (the reference draws from an unseeded ThreadLocalRandom); greedy when temperature <= 0.
int32_t jgpt_sample_next_token(const float *logits_host, int32_t vocab, float temperature, int32_t top_k, float u01,
                               int32_t *token_out) {
    JGPT_REQUIRE(logits_host && vocab > 0 && token_out, JGPT_ERR_INVALID_ARGUMENT, "null pointer or empty vocabulary");
    std::vector<float> z(logits_host, logits_host + vocab);
    if (temperature != 1.0f && temperature > 0)
        for (auto &x : z) x /= temperature;
    if (top_k > 0 && top_k < vocab) {
        std::vector<int> order((size_t)vocab);
        for (int i = 0; i < vocab; i++) order[(size_t)i] = i;
        std::partial_sort(order.begin(), order.begin() + top_k, order.end(),
                          [&](int a, int b) { return z[(size_t)a] > z[(size_t)b] || (z[(size_t)a] == z[(size_t)b] && a < b); });
        std::vector<char> keep((size_t)vocab, 0);
        for (int i = 0; i < top_k; i++) keep[(size_t)order[(size_t)i]] = 1;
        for (int i = 0; i < vocab; i++)
            if (!keep[(size_t)i]) z[(size_t)i] = -INFINITY;
    }
    if (temperature <= 0.f) {
        int best = 0;
        for (int i = 1; i < vocab; i++)
            if (z[(size_t)i] > z[(size_t)best]) best = i;
        *token_out = best;
        return JGPT_OK;
    }
    float mx = -INFINITY, sum = 0.f, cum = 0.f;
    for (float x : z) mx = std::max(mx, x);
    for (auto &x : z) x = (float)std::exp((double)(x - mx)), sum += x;
    for (auto &x : z) x /= sum;
    *token_out = vocab - 1;
    for (int i = 0; i < vocab; i++) {
        cum += z[(size_t)i];
        if (u01 <= cum) {
            *token_out = i;
            break;
        }
    }
    return JGPT_OK;
}

// Up to T greedy steps of one sequence in one launch (each step's argmax is the next step's input; the launch ends
// after a sampled 0).  Returns false - nothing done - when the blocks for T tokens cannot be reserved at once or
// the step is not valid as a single step either (the caller then takes the single step, which reports the error
// at the moment the reference would).  On true: *rc is the status, tokens[0..*done) the sampled ids, the cache length
// advanced by *done, blocks reserved beyond that handed back.
static bool fused_greedy_steps(Model *m, Pool *p, jgpt_kvpool poolh, int32_t seq, int32_t first_id, int32_t len_before, int32_t rope, int T,
                               int32_t *tokens, int *done, int32_t *rc) {
    *done = 0, *rc = JGPT_OK;
    if (first_id < 0 || first_id >= m->vocab || rope < 0 || len_before >= m->max_seq || len_before + T > p->max_blocks_per_seq * kBlockTokens ||
        len_before + T > m->max_seq || rope + T > p->max_positions)
        return false;
    if (jgpt_seq_reserve(poolh, seq, len_before + T) != JGPT_OK) return false;
    cudaStream_t st = m->ctx->stream;
    auto run = [&]() -> int32_t {
        int32_t r2;
        if ((r2 = ensure_fused(m))) return r2;
        if ((r2 = ensure_logits(m, 1))) return r2;
        int *ids = m->h_idx;  // packed [5][1]
        ids[0] = first_id, ids[1] = rope % m->max_seq, ids[2] = seq, ids[3] = rope, ids[4] = len_before + 1;
        m->h_fused[(size_t)kFusedMaxSteps * 4] = 0;  // the kernel writes the tokens and the step count into h_fused itself
        if ((r2 = fused_enqueue(m, p, 1, T, 1, len_before + T, fused_tokens_dev(m), m->h_idx, m->hd_fused, m->hd_fused + (size_t)kFusedMaxSteps * 4)))
            return r2;
        JGPT_CUDA_TRY(status_enqueue_read(m->ctx));
        JGPT_CUDA_TRY(cudaStreamSynchronize(st));
        if ((r2 = status_check_after_sync(m->ctx, p, "jgpt_generate_greedy"))) return r2;
        const int nd = m->h_fused[(size_t)kFusedMaxSteps * 4];
        JGPT_REQUIRE(nd >= 1 && nd <= T, JGPT_ERR_DEVICE_CHECK, "fused decode steps reported %d of %d done", nd, T);
        for (int i = 0; i < nd; i++) tokens[i] = m->h_fused[i];
        *done = nd;
        return jgpt_seq_set_length(poolh, seq, len_before + nd);
    };
    *rc = run();
    const int32_t trc = pool_trim_reservation(p, seq, p->seqs[(size_t)seq].len);
    if (*rc == JGPT_ERR_UNSUPPORTED) {  // the device refused the cooperative launch: nothing ran; the one-step path takes over
        m->fused_step = 0, *rc = JGPT_OK;
        return false;
    }
    if (*rc == JGPT_OK) *rc = trc;
    return true;
}

// GPTModel.generateGpuKv with temperature <= 0 (GptAutoregressiveGenerator.java:108-206).
int32_t jgpt_generate_greedy(jgpt_model h, jgpt_kvpool poolh, const int32_t *prompt_host, int32_t S, int32_t max_new,
                             int32_t *out_host, int32_t *n_sampled_out) {
    GET_MODEL(m, h);
    Pool *p = pool_registry().get(poolh);
    int32_t rc = check_pool(m, p);
    if (rc) return rc;
    JGPT_REQUIRE(prompt_host && out_host && S >= 1 && max_new >= 0, JGPT_ERR_INVALID_ARGUMENT, "bad prompt or output buffer");
    for (int i = 0; i < S + max_new; i++) out_host[i] = i < S ? prompt_host[i] : 0;
    if (n_sampled_out) *n_sampled_out = 0;
    if (max_new == 0) return JGPT_OK;
    int32_t seq = -1;
    rc = jgpt_seq_alloc(poolh, &seq);  // new KvCacheGpu(...)
    if (rc) return rc;
    int n = 0;
    int32_t tok = 0;
    rc = jgpt_forward_prefill(h, poolh, seq, prompt_host, S, 0, nullptr, nullptr, &tok);
    if (rc == JGPT_OK) {
        out_host[S] = tok, n = 1;
        for (int j = 1; j < max_new && tok != 0; j++) {
            const int cur = S + j;
            if (cur > m->max_seq) {  // sliding window: clear, re-prefill out[cur-maxSeq : maxSeq) at ropeOffset = start
                const int start = cur - m->max_seq, len = m->max_seq - start;
                if (len <= 0) {
                    rc = fail(JGPT_ERR_ILLEGAL_STATE, "sliding window: startIdx=%d maxSeqLen=%d", start, m->max_seq);
                    break;
                }
                rc = jgpt_seq_clear(poolh, seq, 0);
                if (rc) break;
                rc = jgpt_forward_prefill(h, poolh, seq, out_host + start, len, start, nullptr, nullptr, &tok);
            } else {
                const int32_t prev = out_host[S + j - 1], len_before = p->seqs[(size_t)seq].len, rope = S + j - 1;
                // as many of the remaining steps as fit before the window starts to slide, in one launch
                const int T = std::min(std::min(max_new - j, m->max_seq - cur + 1), std::min(p->max_positions - rope, kFusedMaxSteps));
                int done = 0;
                if (T >= 2 && fused_ok(m, p, 1) && fused_greedy_steps(m, p, poolh, seq, prev, len_before, rope, T, out_host + cur, &done, &rc)) {
                    if (rc) break;
                    n += done, j += done - 1, tok = out_host[cur + done - 1];
                    continue;
                }
                rc = jgpt_forward_decode(h, poolh, &seq, &prev, &len_before, &rope, 1, nullptr, &tok);
            }
            if (rc) break;
            out_host[cur] = tok, n++;
        }
    }
    const std::string keep = last_error_ref();
    jgpt_seq_free(poolh, seq);  // cache.close()
    if (rc) last_error_ref() = keep;
    if (n_sampled_out) *n_sampled_out = n;
    return rc;
}

// Greedy generation with a block-granular rolling window in place of the reference's clear-and-re-prefill: when the
// sequence has filled its context the oldest KV block is dropped (jgpt_seq_drop_front) and decoding continues; RoPE
// at absolute positions, position-table row = position mod max_seq_len.  The pool's RoPE table (max_positions) bounds
// how far generation can run.  Same tokens as jgpt_generate_greedy until the context first fills.
int32_t jgpt_generate_greedy_rolling(jgpt_model h, jgpt_kvpool poolh, const int32_t *prompt_host, int32_t S, int32_t max_new,
                                     int32_t *out_host, int32_t *n_sampled_out) {
    GET_MODEL(m, h);
    Pool *p = pool_registry().get(poolh);
    int32_t rc = check_pool(m, p);
    if (rc) return rc;
    JGPT_REQUIRE(prompt_host && out_host && S >= 1 && max_new >= 0, JGPT_ERR_INVALID_ARGUMENT, "bad prompt or output buffer");
    const int cap = std::min(m->max_seq, p->max_blocks_per_seq * kBlockTokens);
    JGPT_REQUIRE(S <= cap, JGPT_ERR_INVALID_ARGUMENT, "seq_len %d > max_seq_len %d", S, cap);
    JGPT_REQUIRE(S + max_new - 1 <= p->max_positions, JGPT_ERR_INVALID_ARGUMENT,
                 "prompt %d + %d new tokens run past the pool's RoPE table of %d positions", S, max_new, p->max_positions);
    for (int i = 0; i < S + max_new; i++) out_host[i] = i < S ? prompt_host[i] : 0;
    if (n_sampled_out) *n_sampled_out = 0;
    if (max_new == 0) return JGPT_OK;
    int32_t seq = -1;
    rc = jgpt_seq_alloc(poolh, &seq);
    if (rc) return rc;
    int n = 0;
    int32_t tok = 0;
    rc = jgpt_forward_prefill(h, poolh, seq, prompt_host, S, 0, nullptr, nullptr, &tok);
    if (rc == JGPT_OK) {
        out_host[S] = tok, n = 1;
        for (int j = 1; j < max_new && tok != 0; j++) {
            if (p->seqs[(size_t)seq].len >= cap) {
                rc = jgpt_seq_drop_front(poolh, seq, 1, 0);
                if (rc) break;
            }
            const int32_t prev = out_host[S + j - 1], len_before = p->seqs[(size_t)seq].len, rope = S + j - 1;
            // the steps up to the next dropped block in one launch (at most a block's worth once the window rolls)
            const int T = std::min(std::min(max_new - j, cap - len_before), std::min(p->max_positions - rope, kFusedMaxSteps));
            int done = 0;
            if (T >= 2 && fused_ok(m, p, 1) && fused_greedy_steps(m, p, poolh, seq, prev, len_before, rope, T, out_host + S + j, &done, &rc)) {
                if (rc) break;
                n += done, j += done - 1, tok = out_host[S + j];
                continue;
            }
            rc = jgpt_forward_decode(h, poolh, &seq, &prev, &len_before, &rope, 1, nullptr, &tok);
            if (rc) break;
            out_host[S + j] = tok, n++;
        }
    }
    const std::string keep = last_error_ref();
    jgpt_seq_free(poolh, seq);
    if (rc) last_error_ref() = keep;
    if (n_sampled_out) *n_sampled_out = n;
    return rc;
}

}  // extern "C"
