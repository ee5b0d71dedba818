// fp32 projections for prefill-sized M on the Blackwell tensor cores: tcgen05.mma (kind::tf32) issued by one
// thread per CTA, operands staged in shared memory by bulk async copies (TMA engine, non-multicast), the
// 128 x BN fp32 accumulator double-buffered in tensor memory and read back with tcgen05.ld by epilogue warps
// that overlap the next tile's MMAs.
//
// Accuracy: every fp32 operand is split into a TF32 high part and a TF32 low part and
// C += Ah.Wh + Al.Wh + Ah.Wl with fp32 accumulation, the same "3xTF32" scheme as the mma.sync kernel the
// small-M path uses (the reference runs these GEMMs through cuBLAS under plain TF32 math,
// src/main/cpp/jgpt_cuda_jni_init_matmul.inl:67, 794, 892).  The tensor core truncates when it adds into the
// fp32 accumulator; with all three products in one accumulator (3K / 8 additions) the result sits about
// 8e-9 * K of the largest element away from a float64 product (plain TF32: ~1e-3).
//
// Operand images.  Both operands are stored K-major in the tensor core's canonical no-swizzle layout so that
// one stage of one operand is ONE contiguous bulk copy: for a tile of TR rows and 16 k,
//     byte offset(r, k) = (r / 8) * 512 + (k / 4) * 128 + (r % 8) * 16 + (k % 4) * 4
// i.e. 8-row x 16-byte core matrices, 128 bytes each; the four core matrices of a row group along k are
// adjacent (leading-dimension byte offset 128), row groups follow each other (stride byte offset 512).
// A tile holds the high-part image followed by the low-part image; tiles are ordered [row tile][k tile].
// Weights are static, so their images are built once (transposed: image rows are output columns).
// Activation images are written by whatever produces the activation: the RMSNorm packer, the SwiGLU epilogue
// of the W1/W3 product, or the plain packer (attention output).
//
// Roles in the 320-thread CTA: warp 0 lane 0 issues the bulk copies, warp 1 allocates tensor memory and its
// lane 0 issues the MMAs, warps 2-9 are the epilogue (TMEM lane quarter = warp % 4, two warps per quarter).  Stages are handed over
// with mbarriers: full[s] by the copies' complete_tx, empty[s] and "accumulator buffer ready" by
// tcgen05.commit, "accumulator buffer drained" by the epilogue warps.  Every wait is bounded; on expiry the status word gets DEV_STATUS_WAIT_TIMEOUT and the CTA
// winds down through the common exit (tensor memory is always released).
#include "gemm_umma.cuh"

#include "ptx.cuh"

namespace jgpt {
namespace umma {

constexpr int A_TILE_FLOATS = BM * BK * 2;
constexpr uint32_t A_TILE_BYTES = A_TILE_FLOATS * 4;
constexpr uint32_t TMEM_COLS = 512;  // two accumulator buffers of 256 columns
constexpr uint32_t LBO = 128, SBO = 512;
constexpr int EPI_WARPS = 8;  // two per TMEM lane quarter, each draining half of the tile's columns
constexpr int THREADS = 64 + 32 * EPI_WARPS;

// ------------------------------------------------------------------------------------------------
// Packing
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void split_hi_lo(float x, float &hi, float &lo) {
    uint32_t h, l;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(h) : "f"(x));
    hi = __uint_as_float(h);
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(l) : "f"(x - hi));
    lo = __uint_as_float(l);
}
__device__ __forceinline__ void split4(const float4 v, float4 &hi, float4 &lo) {
    split_hi_lo(v.x, hi.x, lo.x), split_hi_lo(v.y, hi.y, lo.y), split_hi_lo(v.z, hi.z, lo.z), split_hi_lo(v.w, hi.w, lo.w);
}
// Float offset of the 16-byte chunk (row rr of the tile, k chunk k4) inside one half (hi or lo) of a tile.
__device__ __forceinline__ int chunk_offset(int rr, int k4) { return (rr >> 3) * 128 + k4 * 32 + (rr & 7) * 4; }

// One CTA per (k tile, row tile).  TRANSPOSED: the source is [K, rows] (a weight matrix), element (r, k) is
// src[k * rows + r]; otherwise the source is [rows, K].  Rows past `rows` are zero.
template <int TR, bool TRANSPOSED>
__global__ void __launch_bounds__(256) pack_kernel(const float *__restrict__ src, const int *__restrict__ rowsel, int rows, int K,
                                                   float *__restrict__ image) {
    const int kt = blockIdx.x, rt = blockIdx.y, nkt = K / BK;
    float *tile = image + ((size_t)rt * nkt + kt) * (size_t)(TR * BK * 2);
    for (int e = threadIdx.x; e < TR * (BK / 4); e += 256) {
        const int rr = e % TR, k4 = e / TR;  // consecutive threads: consecutive rows = consecutive 16-byte chunks
        const int r = rt * TR + rr, k = kt * BK + k4 * 4;
        float4 v = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < rows) {
            if (TRANSPOSED) {
                v.x = src[(size_t)(k + 0) * rows + r], v.y = src[(size_t)(k + 1) * rows + r];
                v.z = src[(size_t)(k + 2) * rows + r], v.w = src[(size_t)(k + 3) * rows + r];
            } else {
                const int sr = rowsel ? rowsel[r] : r;
                v = *reinterpret_cast<const float4 *>(src + (size_t)sr * K + k);
            }
        }
        float4 hi, lo;
        split4(v, hi, lo);
        const int off = chunk_offset(rr, k4);
        *reinterpret_cast<float4 *>(tile + off) = hi;
        *reinterpret_cast<float4 *>(tile + TR * BK + off) = lo;
    }
}

// 256-row tiles of the W1 / W3 pair: rows 0..127 = columns [128 t, +128) of W1, rows 128..255 = the same of W3.
__global__ void __launch_bounds__(256) pack_pair_kernel(const float *__restrict__ W1, const float *__restrict__ W3, int K, int F,
                                                        float *__restrict__ image) {
    constexpr int TR = 256;
    const int kt = blockIdx.x, rt = blockIdx.y, nkt = K / BK;
    float *tile = image + ((size_t)rt * nkt + kt) * (size_t)(TR * BK * 2);
    for (int e = threadIdx.x; e < TR * (BK / 4); e += 256) {
        const int rr = e % TR, k4 = e / TR;
        const float *__restrict__ src = rr < 128 ? W1 : W3;
        const int col = rt * 128 + (rr & 127), k = kt * BK + k4 * 4;
        float4 v;
        v.x = src[(size_t)(k + 0) * F + col], v.y = src[(size_t)(k + 1) * F + col];
        v.z = src[(size_t)(k + 2) * F + col], v.w = src[(size_t)(k + 3) * F + col];
        float4 hi, lo;
        split4(v, hi, lo);
        const int off = chunk_offset(rr, k4);
        *reinterpret_cast<float4 *>(tile + off) = hi;
        *reinterpret_cast<float4 *>(tile + TR * BK + off) = lo;
    }
}

// RMSNorm of 8 rows (one row group of the image) per CTA with exactly the reduction order of the row-major
// RMSNorm kernel and its 128 threads per row (strided partial sums, warp shuffle, four partials added in order;
// rms_norm_fwd_block_kernel, src/main/cpp/jgpt_cuda_extra_kernels_launches.inl:694-713), so both produce the
// same bits.  The normalised rows go through shared memory so that the image is written in contiguous
// 512-byte runs.
//
// One warp per row: lane l plays the row-major kernel's threads l, l + 32, l + 64, l + 96 (one partial sum
// each, elements taken in the same ascending order), the four butterflies run over the same lanes as that
// kernel's four warps, and the four results are added left to right.
__global__ void __launch_bounds__(256) rmsnorm_pack_kernel(const float *__restrict__ x, const float *__restrict__ gamma, int M, int D,
                                                           float eps, float *__restrict__ image) {
    extern __shared__ __align__(16) float rp_rows[];  // [8][D + 4]
    const int tid = threadIdx.x, rr = tid >> 5, lane = tid & 31;
    const int row = blockIdx.x * 8 + rr;
    const int stride = D + 4;
    const float *xr = x + (size_t)(row < M ? row : 0) * D;
    float ss[4] = {0.f, 0.f, 0.f, 0.f};
    if (row < M) {
        for (int j0 = 0; j0 < D; j0 += 128) {
#pragma unroll
            for (int w = 0; w < 4; w++) {
                const int j = j0 + 32 * w + lane;
                if (j < D) ss[w] += xr[j] * xr[j];
            }
        }
    }
#pragma unroll
    for (int w = 0; w < 4; w++)
#pragma unroll
        for (int off = 16; off >= 1; off >>= 1) ss[w] += __shfl_xor_sync(0xffffffffu, ss[w], off);
    const float tot = ss[0] + ss[1] + ss[2] + ss[3];
    const float rms = sqrtf(tot / (float)D + eps);
    const float inv = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
    for (int j = lane; j < D; j += 32) rp_rows[rr * stride + j] = row < M ? xr[j] * inv * gamma[j] : 0.f;
    __syncthreads();
    const int nkt = D / BK, mt = (blockIdx.x * 8) / BM, rg = ((blockIdx.x * 8) % BM) >> 3;
    float *base = image + (size_t)mt * nkt * A_TILE_FLOATS + rg * 128;
    for (int e = tid; e < nkt * 32; e += 256) {
        const int kt = e >> 5, k4 = (e >> 3) & 3, r8 = e & 7;
        const float4 v = *reinterpret_cast<const float4 *>(&rp_rows[r8 * stride + kt * BK + k4 * 4]);
        float4 hi, lo;
        split4(v, hi, lo);
        float *dst = base + (size_t)kt * A_TILE_FLOATS + k4 * 32 + r8 * 4;
        *reinterpret_cast<float4 *>(dst) = hi;
        *reinterpret_cast<float4 *>(dst + BM * BK) = lo;
    }
}

int32_t pack_activations(const float *A, const int *rowsel, int M, int K, float *image, cudaStream_t st) {
    dim3 grid(K / BK, (M + BM - 1) / BM);
    pack_kernel<BM, false><<<grid, 256, 0, st>>>(A, rowsel, M, K, image);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}
int32_t rmsnorm_pack(const float *x, const float *gamma, int M, int D, float eps, float *image, cudaStream_t st) {
    const size_t smem = sizeof(float) * 8 * (size_t)(D + 4);
    JGPT_REQUIRE(D % BK == 0 && smem <= 48 * 1024, JGPT_ERR_UNSUPPORTED, "rmsnorm_pack: d_model %d", D);
    const int padded_rows = (M + BM - 1) / BM * BM;  // rows past M are written as zeros
    rmsnorm_pack_kernel<<<padded_rows / 8, 256, smem, st>>>(x, gamma, M, D, eps, image);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}
int32_t pack_weight(const float *W, int K, int N, float *image, cudaStream_t st) {
    const int bn = tile_cols(N);
    dim3 grid(K / BK, (N + bn - 1) / bn);
    if (bn == 256) pack_kernel<256, true><<<grid, 256, 0, st>>>(W, nullptr, N, K, image);
    else pack_kernel<192, true><<<grid, 256, 0, st>>>(W, nullptr, N, K, image);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}
int32_t pack_weight_pair(const float *W1, const float *W3, int K, int F, float *image, cudaStream_t st) {
    JGPT_REQUIRE(swiglu_shape_ok(K, F), JGPT_ERR_UNSUPPORTED, "pack_weight_pair: K=%d F=%d", K, F);
    dim3 grid(K / BK, F / 128);
    pack_pair_kernel<<<grid, 256, 0, st>>>(W1, W3, K, F, image);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

// ------------------------------------------------------------------------------------------------
// tcgen05 wrappers
// ------------------------------------------------------------------------------------------------
__device__ __forceinline__ void tmem_alloc(uint32_t *smem_dst, uint32_t cols) {
    asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(smem_dst)), "r"(cols) : "memory");
    asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
}
__device__ __forceinline__ void tmem_dealloc(uint32_t taddr, uint32_t cols) {
    asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(taddr), "r"(cols) : "memory");
}
__device__ __forceinline__ void tc_fence_before() { asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory"); }
__device__ __forceinline__ void tc_fence_after() { asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory"); }

// Shared-memory matrix descriptor, no swizzle: start address, leading / stride byte offsets in 16-byte units,
// descriptor version 1 (bits 46-47), base offset 0, layout type 0.
__device__ __forceinline__ uint64_t smem_desc(uint32_t saddr) {
    return (uint64_t)((saddr & 0x3FFFFu) >> 4) | ((uint64_t)(LBO >> 4) << 16) | ((uint64_t)(SBO >> 4) << 32) | (1ull << 46);
}
// Instruction descriptor: D fp32 (bits 4-5 = 1), A and B TF32 (bits 7-9, 10-12 = 2), both K-major, N / 8 at
// bit 17, M / 16 at bit 24.
template <int BN>
__host__ __device__ constexpr uint32_t instr_desc() {
    return (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);
}

__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(idesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld32_nowait(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
}
__device__ __forceinline__ void tmem_ld_wait() { asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory"); }

// 32 columns starting at `col` of this warp's 32 accumulator lanes.
__device__ __forceinline__ void load_acc32(uint32_t tmem_acc, int quarter, int col, float (&out)[32]) {
    uint32_t v[32];
    tmem_ld32_nowait(tmem_acc + ((uint32_t)(quarter * 32) << 16) + (uint32_t)col, v);
    tmem_ld_wait();
#pragma unroll
    for (int j = 0; j < 32; j++) out[j] = __uint_as_float(v[j]);
}

// ------------------------------------------------------------------------------------------------
// The GEMM: a persistent CTA per SM walks the output tiles (n fastest, so CTAs running side by side share the
// A tile through L2).  The accumulator is double-buffered in tensor memory (2 x 256 columns): while the
// epilogue warps drain tile j, the MMA thread is already accumulating tile j + 1, and the bulk copies run
// ahead of both through the stage ring.
//
// MODE 0: C row major.  MODE 2: C = R + product.  MODE 1 (BN = 256 over a W1/W3 pair image): columns [0,128) of the tile are h1,
// columns [128,256) are g for the same 128 outputs; the epilogue writes h1 * g * sigmoid(g) (sigmoid clamped
// to 1 / 0 at |g| >= 20: sigmoid_kernel, mul_kernel, src/main/cpp/jgpt_cuda_extra_kernels_launches.inl:799-832)
// as the activation image of the next product.
// ------------------------------------------------------------------------------------------------
template <int BN, int STAGES>
constexpr uint32_t smem_bytes() { return (uint32_t)STAGES * (A_TILE_BYTES + (uint32_t)BN * BK * 8u) + 128u; }

struct TileWalk {
    int n_tiles_n, nb, total;  // tiles along N, products in the batch, total tiles
};

template <int BN, int STAGES, int MODE>
__global__ void __launch_bounds__(THREADS, 1) gemm_umma_kernel(const float *__restrict__ Aimg, const Batch B, const TileWalk walk,
                                                               int M, int K, int N, int *__restrict__ status, const PagedAppendArgs pa) {
    constexpr int W_TILE_FLOATS = BN * BK * 2;
    constexpr uint32_t W_TILE_BYTES = W_TILE_FLOATS * 4, STAGE_BYTES = A_TILE_BYTES + W_TILE_BYTES;
    constexpr uint32_t IDESC = instr_desc<BN>();
    static_assert(BN % 64 == 0 && BN <= 256 && (MODE != 1 || BN == 256), "bad tile width");
    static_assert(MODE >= 0 && MODE <= 3, "MODE 3: products 1 and 2 of the batch are K and V rows for the paged store");
    extern __shared__ uint8_t umma_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_full[2], acc_empty[2];
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort_mem;
    volatile int *s_abort = &s_abort_mem;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkt = K / BK;
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(umma_smem_raw) + 127) & ~(uintptr_t)127);

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&full_bar[s], 1), mbar_init(&empty_bar[s], 1);
        for (int b = 0; b < 2; b++) mbar_init(&acc_full[b], 1), mbar_init(&acc_empty[b], EPI_WARPS);  // one arrival per epilogue warp
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) tmem_alloc(&s_tmem_base, TMEM_COLS);
    tc_fence_before();
    __syncthreads();
    tc_fence_after();
    const uint32_t tmem = s_tmem_base;

    if (warp == 0) {
        if (lane == 0) {
            uint32_t it = 0;  // k steps issued so far, over all tiles: stage = it % STAGES
            for (int t = blockIdx.x; t < walk.total && !*s_abort; t += gridDim.x) {
                const int n_idx = t % walk.n_tiles_n, z = (t / walk.n_tiles_n) % walk.nb, m_idx = t / (walk.n_tiles_n * walk.nb);
                const float *__restrict__ a_src = Aimg + (size_t)m_idx * nkt * A_TILE_FLOATS;
                const float *__restrict__ w_src =
                    (z == 0 ? B.Wimg[0] : (z == 1 ? B.Wimg[1] : B.Wimg[2])) + (size_t)n_idx * nkt * W_TILE_FLOATS;
                for (int kt = 0; kt < nkt; kt++, it++) {
                    const uint32_t s = it % STAGES, use = it / STAGES;
                    if (use > 0 && !mbar_wait_bounded(&empty_bar[s], (use - 1) & 1u, status, s_abort)) break;
                    uint8_t *dst = tiles + (size_t)s * STAGE_BYTES;
                    mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                    bulk_g2s(dst, a_src + (size_t)kt * A_TILE_FLOATS, A_TILE_BYTES, &full_bar[s]);
                    bulk_g2s(dst + A_TILE_BYTES, w_src + (size_t)kt * W_TILE_FLOATS, W_TILE_BYTES, &full_bar[s]);
                }
            }
            if (*s_abort) {
                // Copies already issued still target this CTA's shared memory: give each a bounded chance to land.
                for (uint32_t k = it > (uint32_t)STAGES ? it - STAGES : 0; k < it; k++) {
                    const uint32_t s = k % STAGES, ph = (k / STAGES) & 1u;
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full_bar[s], ph); i++) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            uint32_t it = 0, j = 0;  // k steps consumed; tiles started
            bool ok = true;
            for (int t = blockIdx.x; t < walk.total && ok; t += gridDim.x, j++) {
                const uint32_t buf = j & 1u, round = j >> 1;
                if (round > 0 && !mbar_wait_bounded(&acc_empty[buf], (round - 1) & 1u, status, s_abort)) break;
                tc_fence_after();
                const uint32_t acc = tmem + buf * 256u;
                for (int kt = 0; kt < nkt; kt++, it++) {
                    const uint32_t s = it % STAGES, use = it / STAGES;
                    if (!mbar_wait_bounded(&full_bar[s], use & 1u, status, s_abort)) {
                        ok = false;
                        break;
                    }
                    tc_fence_after();
                    const uint32_t a_hi = smem_u32(tiles + (size_t)s * STAGE_BYTES), a_lo = a_hi + A_TILE_BYTES / 2;
                    const uint32_t w_hi = a_hi + A_TILE_BYTES, w_lo = w_hi + W_TILE_BYTES / 2;
#pragma unroll
                    for (int ks = 0; ks < BK / 8; ks++) {
                        const uint32_t adv = ks * 2 * LBO;  // two 16-byte core-matrix columns per K = 8 step
                        const uint64_t ah = smem_desc(a_hi + adv), al = smem_desc(a_lo + adv);
                        const uint64_t wh = smem_desc(w_hi + adv), wl = smem_desc(w_lo + adv);
                        mma_tf32_ss(acc, ah, wh, IDESC, (kt | ks) != 0);
                        mma_tf32_ss(acc, al, wh, IDESC, 1);
                        mma_tf32_ss(acc, ah, wl, IDESC, 1);
                    }
                    mma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
                }
                if (ok) mma_commit(&acc_full[buf]);
            }
        }
    } else {
        const int quarter = warp & 3;  // a warp reads TMEM lanes [32 * (warp % 4), +32)
        const int half = (warp - 2) >> 2;  // which half of the tile's columns
        const int rloc = quarter * 32 + lane;
        uint32_t j = 0;
        for (int t = blockIdx.x; t < walk.total; t += gridDim.x, j++) {
            const uint32_t buf = j & 1u, round = j >> 1;
            const uint32_t acc = tmem + buf * 256u;
            const int n_idx = t % walk.n_tiles_n, z = (t / walk.n_tiles_n) % walk.nb, m_idx = t / (walk.n_tiles_n * walk.nb);
            const int m = m_idx * BM + rloc, n0 = n_idx * BN;
            constexpr int SLABS = BN / 2 / 32;  // 32-column slabs per warp
            float4 res[MODE == 2 ? SLABS : 1][8];
            if (MODE == 2) {
                // The residual rows of this tile are requested before the accumulator is ready: their latency hides
                // behind the MMAs.  (R may be C itself: every element is read, then written, by this one thread.)
                const float *R = z == 0 ? B.R[0] : (z == 1 ? B.R[1] : B.R[2]);
#pragma unroll
                for (int sl = 0; sl < SLABS; sl++)
#pragma unroll
                    for (int q = 0; q < 8; q++) {
                        const int n = n0 + half * (BN / 2) + sl * 32 + q * 4;
                        res[sl][q] = (m < M && n < N) ? *reinterpret_cast<const float4 *>(R + (size_t)m * N + n)
                                                      : make_float4(0.f, 0.f, 0.f, 0.f);
                    }
            }
            int ok = 0;
            if (lane == 0) ok = mbar_wait_bounded(&acc_full[buf], round & 1u, status, s_abort) ? 1 : 0;
            ok = __shfl_sync(0xffffffffu, ok, 0);
            if (!ok) break;
            tc_fence_after();
            if (MODE == 3 && z != 0) {
                // K (z == 1) or V (z == 2) rows of a prefill: row m is slot m - row0 of its sequence.  Same arithmetic
                // and store shape as kv_append_rows_kernel (RoPE from the table with separately rounded products, fp16
                // round-to-nearest-even, 16-byte stores; the last prompt row zero-fills the rest of its block).
                bool row_ok = m < M;
                int slot = 0, tail = 0;
                size_t blk = 0;
                float2 cs[8];
                if (row_ok) {
                    int lo = 0, hi = pa.n_seqs - 1;
                    while (lo < hi) {
                        const int mid = (lo + hi + 1) >> 1;
                        if (pa.seqs[mid].row0 <= m) lo = mid; else hi = mid - 1;
                    }
                    const PrefillSeq sd = pa.seqs[lo];
                    slot = m - sd.row0;
                    const int rp = sd.rope_off + slot;
                    if (slot < 0 || slot >= sd.S || rp < 0 || rp >= pa.max_positions) {
                        atomicOr(pa.status, DEV_STATUS_BAD_POSITION);
                        row_ok = false;
                    } else {
                        const int phys = pa.table[(size_t)sd.seq_id * pa.mbs + slot / kBlockTokens];
                        if (phys < 0 || phys >= pa.n_blocks) {
                            atomicOr(pa.status, DEV_STATUS_BAD_BLOCK);
                            row_ok = false;
                        } else {
                            blk = ((size_t)pa.layer * pa.n_blocks + phys) * pa.H;
                            tail = slot == sd.S - 1 ? kBlockTokens - 1 - slot % kBlockTokens : 0;
                            if (z == 1) {
#pragma unroll
                                for (int q = 0; q < 8; q++) cs[q] = pa.rope[(size_t)rp * 8 + q];
                            }
                        }
                    }
                }
#pragma unroll
                for (int sl = 0; sl < SLABS; sl++) {
                    const int c0 = half * (BN / 2) + sl * 32;
                    if (n0 + c0 >= N) break;  // uniform across the warp
                    float v[32];
                    load_acc32(acc, quarter, c0, v);
                    if (row_ok) {
#pragma unroll
                        for (int hh = 0; hh < 2; hh++) {
                            const int head = (n0 + c0) / 16 + hh;
                            if (head < pa.H) {
                                __align__(16) __half hv[16];
#pragma unroll
                                for (int q = 0; q < 8; q++) {
                                    const float x1 = v[hh * 16 + 2 * q], x2 = v[hh * 16 + 2 * q + 1];
                                    if (z == 1) {
                                        hv[2 * q] = __float2half_rn(__fsub_rn(__fmul_rn(x1, cs[q].x), __fmul_rn(x2, cs[q].y)));
                                        hv[2 * q + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, cs[q].y), __fmul_rn(x2, cs[q].x)));
                                    } else {
                                        hv[2 * q] = __float2half_rn(x1), hv[2 * q + 1] = __float2half_rn(x2);
                                    }
                                }
                                __half *dst = pa.kv + (blk + head) * (size_t)(2 * kBlockTokens * 16) + (size_t)(slot % kBlockTokens) * 16 +
                                              (z == 2 ? kBlockTokens * 16 : 0);
                                *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(hv);
                                *reinterpret_cast<uint4 *>(dst + 8) = *reinterpret_cast<const uint4 *>(hv + 8);
                                for (int t2 = 1; t2 <= tail; t2++) {
                                    *reinterpret_cast<uint4 *>(dst + t2 * 16) = make_uint4(0, 0, 0, 0);
                                    *reinterpret_cast<uint4 *>(dst + t2 * 16 + 8) = make_uint4(0, 0, 0, 0);
                                }
                            }
                        }
                    }
                }
            } else if (MODE != 1) {
                float *C = z == 0 ? B.C[0] : (z == 1 ? B.C[1] : B.C[2]);  // selects, not an indexed copy of B
#pragma unroll
                for (int sl = 0; sl < SLABS; sl++) {
                    const int c0 = half * (BN / 2) + sl * 32;
                    if (n0 + c0 >= N) break;  // uniform across the warp
                    float v[32];
                    load_acc32(acc, quarter, c0, v);
                    if (m < M) {
#pragma unroll
                        for (int q = 0; q < 8; q++) {
                            const int n = n0 + c0 + q * 4;
                            if (n < N) {
                                float4 o = make_float4(v[4 * q], v[4 * q + 1], v[4 * q + 2], v[4 * q + 3]);
                                if (MODE == 2) {
                                    const float4 r4 = res[sl][q];
                                    o.x += r4.x, o.y += r4.y, o.z += r4.z, o.w += r4.w;
                                }
                                *reinterpret_cast<float4 *>(C + (size_t)m * N + n) = o;
                            }
                        }
                    }
                }
            } else {
                // N is F here; the activation image has F / 16 k tiles per row tile.  Rows past M are zero in A,
                // so h1 = g = 0 and zeros are written: the image stays fully defined.
                const int out_nkt = N / BK;
                float *__restrict__ out = B.C[0] + (size_t)m_idx * out_nkt * A_TILE_FLOATS + chunk_offset(rloc, 0);
#pragma unroll 1
                for (int c0 = half * 64; c0 < half * 64 + 64; c0 += 32) {
                    float h[32], g[32];
                    load_acc32(acc, quarter, c0, h);
                    load_acc32(acc, quarter, 128 + c0, g);
#pragma unroll
                    for (int q = 0; q < 32; q++) {
                        const float gv = g[q];
                        float s;
                        if (gv >= 20.f) s = 1.f;
                        else if (gv <= -20.f) s = 0.f;
                        else s = 1.f / (1.f + expf(-gv));
                        h[q] = h[q] * (gv * s);
                    }
#pragma unroll
                    for (int q = 0; q < 32; q += 4) {
                        const int k = n_idx * 128 + c0 + q;  // column of the activation = k of the next product
                        float4 hi, lo;
                        split4(make_float4(h[q], h[q + 1], h[q + 2], h[q + 3]), hi, lo);
                        float *dst = out + (size_t)(k / BK) * A_TILE_FLOATS + ((k % BK) >> 2) * 32;
                        *reinterpret_cast<float4 *>(dst) = hi;
                        *reinterpret_cast<float4 *>(dst + BM * BK) = lo;
                    }
                }
            }
            // this warp has read everything it needs from the buffer: hand it back to the MMA thread
            tc_fence_before();
            __syncwarp();
            if (lane == 0) mbar_arrive(&acc_empty[buf]);
        }
    }
    __syncwarp();
    tc_fence_before();
    __syncthreads();
    if (warp == 1) {
        tc_fence_after();
        tmem_dealloc(tmem, TMEM_COLS);
    }
}

static int sm_count_of_current_device() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 1;
    int &c = cached[dev & 63];
    if (c == 0 && cudaDeviceGetAttribute(&c, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess) c = 1;
    return c > 0 ? c : 1;
}

template <int BN, int STAGES, int MODE>
static int32_t launch_t(const TileWalk &walk, const float *Aimg, const Batch &b, int M, int K, int N, int *d_status, cudaStream_t st,
                        const PagedAppendArgs &pa = PagedAppendArgs()) {
    constexpr uint32_t smem = smem_bytes<BN, STAGES>();
    JGPT_CUDA_TRY(cudaFuncSetAttribute(gemm_umma_kernel<BN, STAGES, MODE>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const int grid = walk.total < sm_count_of_current_device() ? walk.total : sm_count_of_current_device();
    gemm_umma_kernel<BN, STAGES, MODE><<<grid, THREADS, smem, st>>>(Aimg, b, walk, M, K, N, d_status, pa);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

int32_t launch(const float *Aimg, const Batch &b, int nb, int M, int K, int N, int *d_status, cudaStream_t st) {
    JGPT_REQUIRE(shape_ok(K, N) && M > 0 && nb >= 1 && nb <= 3, JGPT_ERR_INVALID_ARGUMENT, "gemm_umma: unsupported shape M=%d K=%d N=%d", M, K, N);
    const int bn = tile_cols(N);
    TileWalk walk{(N + bn - 1) / bn, nb, 0};
    walk.total = walk.n_tiles_n * nb * ((M + BM - 1) / BM);
    bool residual = b.R[0] != nullptr;
    for (int z = 0; z < nb; z++)
        JGPT_REQUIRE((b.R[z] != nullptr) == residual, JGPT_ERR_INVALID_ARGUMENT, "gemm_umma: residuals for all products of a batch or for none");
    if (bn == 256) return residual ? launch_t<256, 4, 2>(walk, Aimg, b, M, K, N, d_status, st) : launch_t<256, 4, 0>(walk, Aimg, b, M, K, N, d_status, st);
    return residual ? launch_t<192, 5, 2>(walk, Aimg, b, M, K, N, d_status, st) : launch_t<192, 5, 0>(walk, Aimg, b, M, K, N, d_status, st);
}

int32_t launch_qkv_paged(const float *Aimg, const Batch &b, int M, int K, int N, const PagedAppendArgs &pa, int *d_status,
                         cudaStream_t st) {
    JGPT_REQUIRE(shape_ok(K, N) && M > 0 && N == pa.H * 16, JGPT_ERR_INVALID_ARGUMENT,
                 "gemm_umma qkv: unsupported shape M=%d K=%d N=%d (heads %d, d_head 16)", M, K, N, pa.H);
    const int bn = tile_cols(N);
    TileWalk walk{(N + bn - 1) / bn, 3, 0};
    walk.total = walk.n_tiles_n * 3 * ((M + BM - 1) / BM);
    if (bn == 256) return launch_t<256, 4, 3>(walk, Aimg, b, M, K, N, d_status, st, pa);
    return launch_t<192, 5, 3>(walk, Aimg, b, M, K, N, d_status, st, pa);
}

int32_t launch_swiglu(const float *Aimg, const float *Wpair_img, int M, int K, int F, float *act_image, int *d_status,
                      cudaStream_t st) {
    JGPT_REQUIRE(swiglu_shape_ok(K, F) && M > 0, JGPT_ERR_INVALID_ARGUMENT, "gemm_umma swiglu: unsupported shape M=%d K=%d F=%d", M, K, F);
    Batch b{};
    b.Wimg[0] = Wpair_img, b.C[0] = act_image;
    TileWalk walk{F / 128, 1, 0};
    walk.total = walk.n_tiles_n * ((M + BM - 1) / BM);
    return launch_t<256, 4, 1>(walk, Aimg, b, M, K, F, d_status, st);
}

}  // namespace umma
}  // namespace jgpt
