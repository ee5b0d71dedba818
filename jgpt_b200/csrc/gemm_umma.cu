// fp32 projections for prefill-sized M on the Blackwell tensor cores: tcgen05.mma (kind::tf32) issued by one
// thread per CTA, operands staged in shared memory by bulk async copies (TMA engine, non-multicast), two
// 128 x 256 fp32 accumulators (main product, correction products) held in tensor memory and read back with
// tcgen05.ld for the epilogue.
//
// Accuracy: every fp32 operand is split into a TF32 high part and a TF32 low part and
// C += Ah.Wh + Al.Wh + Ah.Wl with fp32 accumulation, the same "3xTF32" scheme as the mma.sync kernel the
// small-M path uses (the reference runs these GEMMs through cuBLAS under plain TF32 math,
// src/main/cpp/jgpt_cuda_jni_init_matmul.inl:67, 794, 892).
//
// Operand images.  Both operands are stored K-major in the tensor core's canonical no-swizzle layout so that
// one stage of one operand is ONE contiguous bulk copy: for a tile of TR rows and 16 k,
//     byte offset(r, k) = (r / 8) * 512 + (k / 4) * 128 + (r % 8) * 16 + (k % 4) * 4
// i.e. 8-row x 16-byte core matrices, 128 bytes each; the four core matrices of a row group along k are
// adjacent (leading-dimension byte offset 128), row groups follow each other (stride byte offset 512).
// A tile holds the high-part image followed by the low-part image; tiles are ordered [row tile][k tile].
// Weights are static, so their images are built once (transposed: image rows are output columns);
// activations are packed by a small kernel in front of the GEMM.
//
// Roles in the 192-thread CTA: warp 0 lane 0 issues the bulk copies, warp 1 allocates tensor memory and its
// lane 0 issues the MMAs, warps 2-5 are the epilogue (TMEM lane quarter = warp % 4).  Stages are handed over
// with mbarriers: full[s] by the copies' complete_tx, empty[s] and the final "accumulator ready" by
// tcgen05.commit.  Every wait is bounded; on expiry the status word gets DEV_STATUS_WAIT_TIMEOUT and the CTA
// winds down through the common exit (tensor memory is always released).
#include "gemm_umma.cuh"

#include "ptx.cuh"

namespace jgpt {
namespace umma {

constexpr int STAGES = 4;
constexpr int A_TILE_FLOATS = BM * BK * 2, W_TILE_FLOATS = BN * BK * 2;
constexpr uint32_t A_TILE_BYTES = A_TILE_FLOATS * 4, W_TILE_BYTES = W_TILE_FLOATS * 4;
constexpr uint32_t STAGE_BYTES = A_TILE_BYTES + W_TILE_BYTES;  // 48 KiB
constexpr uint32_t SMEM_BYTES = STAGES * STAGE_BYTES + 128;    // + alignment slack
constexpr uint32_t TMEM_COLS = 2 * BN;                         // main + correction accumulators (all 512 columns)
constexpr uint32_t LBO = 128, SBO = 512;
constexpr int THREADS = 192;

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
        split_hi_lo(v.x, hi.x, lo.x), split_hi_lo(v.y, hi.y, lo.y), split_hi_lo(v.z, hi.z, lo.z), split_hi_lo(v.w, hi.w, lo.w);
        const int off = (rr >> 3) * 128 + k4 * 32 + (rr & 7) * 4;  // floats
        *reinterpret_cast<float4 *>(tile + off) = hi;
        *reinterpret_cast<float4 *>(tile + TR * BK + off) = lo;
    }
}

int32_t pack_activations(const float *A, const int *rowsel, int M, int K, float *image, cudaStream_t st) {
    dim3 grid(K / BK, (M + BM - 1) / BM);
    pack_kernel<BM, false><<<grid, 256, 0, st>>>(A, rowsel, M, K, image);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}
int32_t pack_weight(const float *W, int K, int N, float *image, cudaStream_t st) {
    dim3 grid(K / BK, (N + BN - 1) / BN);
    pack_kernel<BN, true><<<grid, 256, 0, st>>>(W, nullptr, N, K, image);
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
constexpr uint32_t kInstrDesc = (1u << 4) | (2u << 7) | (2u << 10) | ((uint32_t)(BN >> 3) << 17) | ((uint32_t)(BM >> 4) << 24);

__device__ __forceinline__ void mma_tf32_ss(uint32_t tmem_d, uint64_t adesc, uint64_t bdesc, uint32_t accumulate) {
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "setp.ne.b32 p, %4, 0;\n\t"
        "tcgen05.mma.cta_group::1.kind::tf32 [%0], %1, %2, %3, p;\n\t}"
        ::"r"(tmem_d), "l"(adesc), "l"(bdesc), "r"(kInstrDesc), "r"(accumulate)
        : "memory");
}
// The mbarrier gets one arrival when every MMA this thread issued so far has completed.
__device__ __forceinline__ void mma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar)) : "memory");
}
// 32 lanes x 32 consecutive fp32 columns: thread t of the warp receives lane (base lane + t).
__device__ __forceinline__ void tmem_ld32(uint32_t taddr, uint32_t (&v)[32]) {
    asm volatile(
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
        "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,%26,%27,%28,%29,%30,%31}, [%32];"
        : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]), "=r"(v[8]), "=r"(v[9]),
          "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]),
          "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]),
          "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
        : "r"(taddr)
        : "memory");
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
}

// ------------------------------------------------------------------------------------------------
// The GEMM
// ------------------------------------------------------------------------------------------------
__global__ void __launch_bounds__(THREADS, 1) gemm_umma_kernel(const float *__restrict__ Aimg, const Batch B, int M, int K, int N,
                                                               int *__restrict__ status) {
    extern __shared__ uint8_t umma_smem_raw[];
    __shared__ __align__(8) uint64_t full_bar[STAGES], empty_bar[STAGES], acc_bar;
    __shared__ uint32_t s_tmem_base;
    __shared__ int s_abort_mem;
    volatile int *s_abort = &s_abort_mem;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int nkt = K / BK;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    uint8_t *tiles = reinterpret_cast<uint8_t *>((reinterpret_cast<uintptr_t>(umma_smem_raw) + 127) & ~(uintptr_t)127);
    const float *__restrict__ a_src = Aimg + (size_t)blockIdx.y * nkt * A_TILE_FLOATS;
    const float *__restrict__ w_src = B.Wimg[blockIdx.z] + (size_t)blockIdx.x * nkt * W_TILE_FLOATS;

    if (tid == 0) {
        for (int s = 0; s < STAGES; s++) mbar_init(&full_bar[s], 1), mbar_init(&empty_bar[s], 1);
        mbar_init(&acc_bar, 1);
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
            int issued = 0;
            for (int kt = 0; kt < nkt && !*s_abort; kt++, issued++) {
                const int s = kt % STAGES, use = kt / STAGES;
                if (use > 0 && !mbar_wait_bounded(&empty_bar[s], (uint32_t)(use - 1) & 1u, status, s_abort)) break;
                uint8_t *dst = tiles + (size_t)s * STAGE_BYTES;
                mbar_expect_tx(&full_bar[s], STAGE_BYTES);
                bulk_g2s(dst, a_src + (size_t)kt * A_TILE_FLOATS, A_TILE_BYTES, &full_bar[s]);
                bulk_g2s(dst + A_TILE_BYTES, w_src + (size_t)kt * W_TILE_FLOATS, W_TILE_BYTES, &full_bar[s]);
            }
            if (*s_abort) {
                // Copies already issued still target this CTA's shared memory: give each a bounded chance to land.
                for (int kt = max(0, issued - STAGES); kt < issued; kt++) {
                    const int s = kt % STAGES;
                    const uint32_t ph = (uint32_t)(kt / STAGES) & 1u;
                    for (uint32_t i = 0; i < (1u << 16) && !mbar_try_wait(&full_bar[s], ph); i++) {
                    }
                }
            }
        }
    } else if (warp == 1) {
        if (lane == 0) {
            bool ok = true;
            for (int kt = 0; kt < nkt; kt++) {
                const int s = kt % STAGES, use = kt / STAGES;
                if (!mbar_wait_bounded(&full_bar[s], (uint32_t)use & 1u, status, s_abort)) {
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
                    // The tensor core truncates when it adds into the fp32 accumulator, a bias that grows with
                    // the number of additions.  The two small correction products go to an accumulator of their
                    // own (where that bias is 2^-11 smaller), so the main one sees K / 8 additions, not 3K / 8.
                    mma_tf32_ss(tmem, ah, wh, (kt | ks) != 0);
                    mma_tf32_ss(tmem + BN, al, wh, (kt | ks) != 0);
                    mma_tf32_ss(tmem + BN, ah, wl, 1);
                }
                mma_commit(&empty_bar[s]);  // the stage is free once these MMAs have read it
            }
            if (ok) mma_commit(&acc_bar);
        }
    } else {
        int ok = 0;
        if (lane == 0) ok = mbar_wait_bounded(&acc_bar, 0u, status, s_abort) ? 1 : 0;
        ok = __shfl_sync(0xffffffffu, ok, 0);
        if (ok) {
            tc_fence_after();
            const int quarter = warp & 3;  // a warp reads TMEM lanes [32 * (warp % 4), +32)
            const int m = m0 + quarter * 32 + lane;
            float *__restrict__ C = B.C[blockIdx.z];
            const float *__restrict__ R = B.R[blockIdx.z];
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                if (n0 + c0 >= N) break;  // uniform across the CTA
                uint32_t v[32], w[32];
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)c0, v);
                tmem_ld32(tmem + ((uint32_t)(quarter * 32) << 16) + (uint32_t)(BN + c0), w);
#pragma unroll
                for (int j = 0; j < 32; j++) v[j] = __float_as_uint(__uint_as_float(v[j]) + __uint_as_float(w[j]));
                if (m < M) {
#pragma unroll
                    for (int j = 0; j < 32; j += 4) {
                        const int n = n0 + c0 + j;
                        if (n < N) {
                            float4 o = make_float4(__uint_as_float(v[j]), __uint_as_float(v[j + 1]), __uint_as_float(v[j + 2]),
                                                   __uint_as_float(v[j + 3]));
                            if (R) {
                                const float4 r4 = *reinterpret_cast<const float4 *>(R + (size_t)m * N + n);
                                o.x += r4.x, o.y += r4.y, o.z += r4.z, o.w += r4.w;
                            }
                            *reinterpret_cast<float4 *>(C + (size_t)m * N + n) = o;
                        }
                    }
                }
            }
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

int32_t launch(const float *Aimg, const Batch &b, int nb, int M, int K, int N, int *d_status, cudaStream_t st) {
    JGPT_REQUIRE(shape_ok(K, N) && M > 0 && nb >= 1 && nb <= 3, JGPT_ERR_INVALID_ARGUMENT, "gemm_umma: unsupported shape M=%d K=%d N=%d", M, K, N);
    static bool opted[64] = {};
    int dev = 0;
    JGPT_CUDA_TRY(cudaGetDevice(&dev));
    if (!opted[dev & 63]) {
        JGPT_CUDA_TRY(cudaFuncSetAttribute(gemm_umma_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)SMEM_BYTES));
        opted[dev & 63] = true;
    }
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM, nb);
    gemm_umma_kernel<<<grid, THREADS, SMEM_BYTES, st>>>(Aimg, b, M, K, N, d_status);
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

}  // namespace umma
}  // namespace jgpt
