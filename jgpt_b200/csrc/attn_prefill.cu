// Causal prefill attention that fills the paged cache.
//
// Two launches per layer:
//   1. kv_append_rows_kernel: RoPE(k) and v of every prompt row -> fp16 -> paged blocks (HBM-bound).
//   2. attn_prefill_mma_kernel (dhead 16): FlashAttention-2 style forward.  A CTA owns 64 query rows of
//      one (sequence, head); each of its 4 warps owns 16 rows.  K/V blocks (16 keys, 1 KiB per block and
//      head, straight out of the paged store) are staged to shared memory by bulk async copies, 4 blocks
//      per stage, double buffered.  Per 16x16 score tile: QK^T is 2 m16n8k16 MMAs (the whole K
//      dimension, 16, is one k-step) issued twice (q is split into fp16 hi + lo parts so the scores keep
//      fp32-level accuracy), online softmax on the accumulator fragments in registers (exp2 on the SFU),
//      the probabilities become the A fragments of P.V (again hi + lo).  At dhead 16 the kernel is bound
//      by exp / FMA issue, not by the tensor pipe.
//      attn_prefill_simt_kernel covers the other head sizes (one thread per query row).
#include "common.cuh"
#include "ptx.cuh"

#include <algorithm>

namespace jgpt {

struct PrefillParams {
    __half *kv;
    const int *table;
    const float2 *rope;
    const float *q, *k, *v;
    float *out;
    float *out_image;  // != nullptr (d_head 16): write the output as the tcgen05 projection's operand image instead
    const PrefillSeq *seqs;
    int *status;
    int n_seqs, n_rows, H, layer, n_blocks, mbs, max_positions;
    float scale_log2e;
};

// Row r of the packed [n_rows, H*DH] activations -> its sequence descriptor (rows of a sequence are consecutive).
__device__ __forceinline__ int find_seq(const PrefillSeq *seqs, int n_seqs, int r) {
    int lo = 0, hi = n_seqs - 1;
    while (lo < hi) {
        const int mid = (lo + hi + 1) >> 1;
        if (seqs[mid].row0 <= r) lo = mid; else hi = mid - 1;
    }
    return lo;
}

// Append of whole prompts: same arithmetic and store shape as kv_append_kernel, indices derived from the
// sequence descriptors (slot = row within the prompt, RoPE position = rope_off + slot).
template <int DH>
__global__ void __launch_bounds__(256) kv_append_rows_kernel(const PrefillParams P) {
    constexpr int CH = DH < 8 ? DH : 8;
    constexpr int CPR = DH / CH;
    const long long gid = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    const long long total = (long long)P.n_rows * P.H * CPR;
    if (gid >= total) return;
    const int c = (int)(gid % CPR);
    const int h = (int)((gid / CPR) % P.H);
    const int r = (int)(gid / ((long long)CPR * P.H));
    const PrefillSeq sd = P.seqs[find_seq(P.seqs, P.n_seqs, r)];
    const int slot = r - sd.row0, rp = sd.rope_off + slot;
    if (slot < 0 || slot >= sd.S || rp < 0 || rp >= P.max_positions) { atomicOr(P.status, DEV_STATUS_BAD_POSITION); return; }
    const int phys = P.table[(size_t)sd.seq_id * P.mbs + slot / kBlockTokens];
    if (phys < 0 || phys >= P.n_blocks) { atomicOr(P.status, DEV_STATUS_BAD_BLOCK); return; }
    const size_t src = ((size_t)r * P.H + h) * DH + c * CH;
    float kf[CH], vf[CH];
#pragma unroll
    for (int i = 0; i < CH; i += 4) {
        const float4 a = *reinterpret_cast<const float4 *>(P.k + src + i);
        const float4 b = *reinterpret_cast<const float4 *>(P.v + src + i);
        kf[i] = a.x, kf[i + 1] = a.y, kf[i + 2] = a.z, kf[i + 3] = a.w;
        vf[i] = b.x, vf[i + 1] = b.y, vf[i + 2] = b.z, vf[i + 3] = b.w;
    }
    const float2 *cs = P.rope + (size_t)rp * (DH / 2) + c * (CH / 2);
    __align__(16) __half kh[CH], vh[CH];
#pragma unroll
    for (int j = 0; j < CH / 2; j++) {
        const float2 w = cs[j];
        const float x1 = kf[2 * j], x2 = kf[2 * j + 1];
        kh[2 * j] = __float2half_rn(__fsub_rn(__fmul_rn(x1, w.x), __fmul_rn(x2, w.y)));
        kh[2 * j + 1] = __float2half_rn(__fadd_rn(__fmul_rn(x1, w.y), __fmul_rn(x2, w.x)));
        vh[2 * j] = __float2half_rn(vf[2 * j]);
        vh[2 * j + 1] = __float2half_rn(vf[2 * j + 1]);
    }
    __half *dst = P.kv + (((size_t)P.layer * P.n_blocks + phys) * P.H + h) * (2 * kBlockTokens * DH) +
                  (size_t)(slot % kBlockTokens) * DH + c * CH;
    if constexpr (CH == 8) {
        *reinterpret_cast<uint4 *>(dst) = *reinterpret_cast<const uint4 *>(kh);
        *reinterpret_cast<uint4 *>(dst + kBlockTokens * DH) = *reinterpret_cast<const uint4 *>(vh);
    } else {
        *reinterpret_cast<uint2 *>(dst) = *reinterpret_cast<const uint2 *>(kh);
        *reinterpret_cast<uint2 *>(dst + kBlockTokens * DH) = *reinterpret_cast<const uint2 *>(vh);
    }
    // The last prompt row also zero-fills the rest of its block (slots S .. end of block): the tensor-core
    // attention kernel multiplies those V rows by probability 0, which must not meet stale Inf/NaN.
    if (slot == sd.S - 1) {
        for (int s2 = slot % kBlockTokens + 1; s2 < kBlockTokens; s2++) {
            __half *z = dst + (size_t)(s2 - slot % kBlockTokens) * DH;
            if constexpr (CH == 8) {
                *reinterpret_cast<uint4 *>(z) = make_uint4(0, 0, 0, 0);
                *reinterpret_cast<uint4 *>(z + kBlockTokens * DH) = make_uint4(0, 0, 0, 0);
            } else {
                *reinterpret_cast<uint2 *>(z) = make_uint2(0, 0);
                *reinterpret_cast<uint2 *>(z + kBlockTokens * DH) = make_uint2(0, 0);
            }
        }
    }
}

// ------------------------------------------------------------------------------------------------
// dhead 16: tensor-core kernel
// ------------------------------------------------------------------------------------------------
constexpr int kQTile = 64;     // query rows per CTA (4 warps x 16)
constexpr int kStageBlocks = 8;  // KV blocks per pipeline stage (128 keys, 8 KiB)

__device__ __forceinline__ uint32_t pack_half2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// fp32 pair -> (hi, lo) fp16 pairs with hi + lo == value up to 2^-22 relative.
__device__ __forceinline__ void split_half2(float a, float b, uint32_t &hi, uint32_t &lo) {
    const __half ha = __float2half_rn(a), hb = __float2half_rn(b);
    const __half2 h = __halves2half2(ha, hb);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = pack_half2(a - __half2float(ha), b - __half2float(hb));
}

// FAST: the probabilities enter the P.V product as single fp16 values instead of fp16 high + low pairs (half the
// MMAs of that product and none of the split arithmetic, which was the larger part of the instruction count), and two
// KV blocks share one online-softmax update.  q keeps its high + low split (done once per CTA), so the scores are as
// exact as before; the cached K / V are fp16 anyway.  The only new error is the rounding of p (2^-11 relative):
// attention outputs stay within ~4e-4 of the exact mode on N(0,1) inputs and the logits of the JGPT-35M shapes within
// 5e-4 of an fp32 CPU evaluation, against a budget of 2e-3.  The exact mode (2e-5) remains the default of the
// standalone entry point.
template <bool FAST>
__global__ void __launch_bounds__(128) attn_prefill_mma_kernel(const PrefillParams P) {
    constexpr int DH = 16, BT = kBlockTokens, TILE_BYTES = 2 * BT * DH * 2;  // 1 KiB: K tile | V tile
    __shared__ __align__(128) unsigned char tiles[2][kStageBlocks][TILE_BYTES];
    __shared__ uint64_t full_bar[2];
    __shared__ int s_abort_mem;
    extern __shared__ int s_table[];  // physical block ids of this sequence, [nblk]
    volatile int *s_abort = &s_abort_mem;

    const PrefillSeq sd = P.seqs[blockIdx.z];
    const int h = blockIdx.y;
    const int r0 = blockIdx.x * kQTile;
    if (r0 >= sd.S) return;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, g = lane >> 2, t = lane & 3;
    const int nblk = min((sd.S + BT - 1) / BT, (r0 + kQTile - 1) / BT + 1);  // causal: nothing beyond the tile's last row
    for (int b = tid; b < nblk; b += blockDim.x) {
        int phys = P.table[(size_t)sd.seq_id * P.mbs + b];
        if (phys < 0 || phys >= P.n_blocks) {
            atomicOr(P.status, DEV_STATUS_BAD_BLOCK);
            phys = 0;
        }
        s_table[b] = phys;
    }
    if (tid == 0) {
        mbar_init(&full_bar[0], 1);
        mbar_init(&full_bar[1], 1);
        *s_abort = 0;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const unsigned char *kv_head = reinterpret_cast<const unsigned char *>(P.kv) +
                                   ((size_t)P.layer * P.n_blocks * P.H + h) * (size_t)TILE_BYTES;
    const size_t block_stride = (size_t)P.H * TILE_BYTES;
    const int nchunks = (nblk + kStageBlocks - 1) / kStageBlocks;
    auto issue = [&](int c) {  // thread 0 only
        const int b0 = c * kStageBlocks, nb = min(kStageBlocks, nblk - b0);
        mbar_expect_tx(&full_bar[c & 1], (uint32_t)(nb * TILE_BYTES));
        for (int b = 0; b < nb; b++)
            bulk_g2s(&tiles[c & 1][b][0], kv_head + (size_t)s_table[b0 + b] * block_stride, TILE_BYTES, &full_bar[c & 1]);
    };
    if (tid == 0) issue(0);

    // ---- this warp's 16 query rows: RoPE, scale, split into fp16 hi/lo A fragments ----
    const int rowA = r0 + warp * 16 + g, rowB = rowA + 8;
    uint32_t a_hi[4], a_lo[4];
    {
        const size_t D = (size_t)P.H * DH;
        float2 x[4];  // (rowA, cols 2t..), (rowB, cols 2t..), (rowA, cols 8+2t..), (rowB, cols 8+2t..)
#pragma unroll
        for (int e = 0; e < 4; e++) {
            const int row = (e & 1) ? rowB : rowA;
            const int col = 2 * t + ((e >> 1) ? 8 : 0);
            float2 val = make_float2(0.f, 0.f);
            if (row < sd.S) {
                const float2 raw = *reinterpret_cast<const float2 *>(P.q + (size_t)(sd.row0 + row) * D + h * DH + col);
                const float2 w = P.rope[(size_t)(sd.rope_off + row) * (DH / 2) + col / 2];
                val.x = __fsub_rn(__fmul_rn(raw.x, w.x), __fmul_rn(raw.y, w.y)) * P.scale_log2e;
                val.y = __fadd_rn(__fmul_rn(raw.x, w.y), __fmul_rn(raw.y, w.x)) * P.scale_log2e;
            }
            x[e] = val;
        }
#pragma unroll
        for (int e = 0; e < 4; e++) {
            split_half2(x[e].x, x[e].y, a_hi[e], a_lo[e]);  // once per CTA: q keeps fp32-level accuracy in both modes
        }
    }

    float o[2][4];
#pragma unroll
    for (int j = 0; j < 2; j++)
#pragma unroll
        for (int e = 0; e < 4; e++) o[j][e] = 0.f;
    float mA = -INFINITY, mB = -INFINITY, lA = 0.f, lB = 0.f;
    const int diag = r0 / BT + warp;  // last KV block this warp's rows can see
    const int mi = lane >> 3, rr = lane & 7;
    const int k_off = ((mi >> 1) * 8 + rr) * 32 + (mi & 1) * 16;             // ldmatrix row address inside the K tile
    const int v_off = BT * DH * 2 + ((mi & 1) * 8 + rr) * 32 + (mi >> 1) * 16;  // ... inside the V tile (transposed load)

    bool aborted = false;
    for (int c = 0; c < nchunks; c++) {
        if (tid == 0 && c + 1 < nchunks && !*s_abort) issue(c + 1);  // the other buffer was released by the barrier below
        if (!aborted && !mbar_wait_bounded(&full_bar[c & 1], (uint32_t)(c >> 1) & 1u, P.status, s_abort)) aborted = true;
        if (!aborted) {
            const int nb = min(kStageBlocks, nblk - c * kStageBlocks);
            for (int b = 0; b < nb; b++) {
                const int kb = c * kStageBlocks + b;
                if (kb > diag) break;
                if constexpr (FAST) {
                    // Two KV blocks (32 keys) below the diagonal share one online-softmax update: one running maximum,
                    // one correction factor and one rescale of the output tile instead of two.
                    if (b + 1 < nb && kb + 1 < diag) {
                        const unsigned char *t0 = &tiles[c & 1][b][0], *t1 = &tiles[c & 1][b + 1][0];
                        uint32_t k0[4], k1[4];
                        ldmatrix_x4(k0, t0 + k_off);
                        ldmatrix_x4(k1, t1 + k_off);
                        float s4[4][4];
#pragma unroll
                        for (int j = 0; j < 4; j++)
#pragma unroll
                            for (int e = 0; e < 4; e++) s4[j][e] = 0.f;
                        mma_16816(s4[0], a_hi, k0[0], k0[1]);
                        mma_16816(s4[1], a_hi, k0[2], k0[3]);
                        mma_16816(s4[2], a_hi, k1[0], k1[1]);
                        mma_16816(s4[3], a_hi, k1[2], k1[3]);
                        mma_16816(s4[0], a_lo, k0[0], k0[1]);
                        mma_16816(s4[1], a_lo, k0[2], k0[3]);
                        mma_16816(s4[2], a_lo, k1[0], k1[1]);
                        mma_16816(s4[3], a_lo, k1[2], k1[3]);
                        float mxA = fmaxf(fmaxf(fmaxf(s4[0][0], s4[0][1]), fmaxf(s4[1][0], s4[1][1])),
                                          fmaxf(fmaxf(s4[2][0], s4[2][1]), fmaxf(s4[3][0], s4[3][1])));
                        float mxB = fmaxf(fmaxf(fmaxf(s4[0][2], s4[0][3]), fmaxf(s4[1][2], s4[1][3])),
                                          fmaxf(fmaxf(s4[2][2], s4[2][3]), fmaxf(s4[3][2], s4[3][3])));
                        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
                        mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
                        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
                        mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
                        const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);
                        const float cA = fast_exp2(mA - nA), cB = fast_exp2(mB - nB);
                        mA = nA, mB = nB;
                        float sumA = 0.f, sumB = 0.f;
#pragma unroll
                        for (int j = 0; j < 4; j++) {
                            s4[j][0] = fast_exp2(s4[j][0] - nA), s4[j][1] = fast_exp2(s4[j][1] - nA);
                            s4[j][2] = fast_exp2(s4[j][2] - nB), s4[j][3] = fast_exp2(s4[j][3] - nB);
                            sumA += s4[j][0] + s4[j][1], sumB += s4[j][2] + s4[j][3];
                        }
#pragma unroll
                        for (int j = 0; j < 2; j++) o[j][0] *= cA, o[j][1] *= cA, o[j][2] *= cB, o[j][3] *= cB;
                        lA = lA * cA + sumA, lB = lB * cB + sumB;
                        uint32_t v0[4], v1[4];
                        ldmatrix_x4_trans(v0, t0 + v_off);
                        ldmatrix_x4_trans(v1, t1 + v_off);
                        const uint32_t p0[4] = {pack_half2(s4[0][0], s4[0][1]), pack_half2(s4[0][2], s4[0][3]),
                                                pack_half2(s4[1][0], s4[1][1]), pack_half2(s4[1][2], s4[1][3])};
                        const uint32_t p1[4] = {pack_half2(s4[2][0], s4[2][1]), pack_half2(s4[2][2], s4[2][3]),
                                                pack_half2(s4[3][0], s4[3][1]), pack_half2(s4[3][2], s4[3][3])};
#pragma unroll
                        for (int j = 0; j < 2; j++) {
                            mma_16816(o[j], p0, v0[2 * j], v0[2 * j + 1]);
                            mma_16816(o[j], p1, v1[2 * j], v1[2 * j + 1]);
                        }
                        b++;  // two blocks done
                        continue;
                    }
                }
                const unsigned char *tile = &tiles[c & 1][b][0];
                uint32_t kf[4];
                ldmatrix_x4(kf, tile + k_off);
                float s[2][4];
#pragma unroll
                for (int j = 0; j < 2; j++) {
#pragma unroll
                    for (int e = 0; e < 4; e++) s[j][e] = 0.f;
                    mma_16816(s[j], a_hi, kf[2 * j], kf[2 * j + 1]);
                    mma_16816(s[j], a_lo, kf[2 * j], kf[2 * j + 1]);
                }
                if (kb == diag) {  // causal mask inside the diagonal block
#pragma unroll
                    for (int j = 0; j < 2; j++)
#pragma unroll
                        for (int e = 0; e < 4; e++) {
                            const int key = kb * BT + 8 * j + 2 * t + (e & 1);
                            const int row = (e & 2) ? rowB : rowA;
                            if (key > row) s[j][e] = -INFINITY;
                        }
                }
                float mxA = fmaxf(fmaxf(s[0][0], s[0][1]), fmaxf(s[1][0], s[1][1]));
                float mxB = fmaxf(fmaxf(s[0][2], s[0][3]), fmaxf(s[1][2], s[1][3]));
                mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 1));
                mxA = fmaxf(mxA, __shfl_xor_sync(0xffffffffu, mxA, 2));
                mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 1));
                mxB = fmaxf(mxB, __shfl_xor_sync(0xffffffffu, mxB, 2));
                const float nA = fmaxf(mA, mxA), nB = fmaxf(mB, mxB);  // finite: key 0 is visible to every row
                const float cA = fast_exp2(mA - nA), cB = fast_exp2(mB - nB);
                mA = nA, mB = nB;
                float sumA = 0.f, sumB = 0.f;
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    s[j][0] = fast_exp2(s[j][0] - nA), s[j][1] = fast_exp2(s[j][1] - nA);
                    s[j][2] = fast_exp2(s[j][2] - nB), s[j][3] = fast_exp2(s[j][3] - nB);
                    sumA += s[j][0] + s[j][1], sumB += s[j][2] + s[j][3];
                    o[j][0] *= cA, o[j][1] *= cA, o[j][2] *= cB, o[j][3] *= cB;
                }
                lA = lA * cA + sumA, lB = lB * cB + sumB;
                uint32_t p_hi[4], p_lo[4];
                if constexpr (FAST) {
                    p_hi[0] = pack_half2(s[0][0], s[0][1]), p_hi[1] = pack_half2(s[0][2], s[0][3]);
                    p_hi[2] = pack_half2(s[1][0], s[1][1]), p_hi[3] = pack_half2(s[1][2], s[1][3]);
                    p_lo[0] = p_lo[1] = p_lo[2] = p_lo[3] = 0u;
                } else {
                    split_half2(s[0][0], s[0][1], p_hi[0], p_lo[0]);  // row g,   keys 2t, 2t+1
                    split_half2(s[0][2], s[0][3], p_hi[1], p_lo[1]);  // row g+8, keys 2t, 2t+1
                    split_half2(s[1][0], s[1][1], p_hi[2], p_lo[2]);  // row g,   keys 8+2t, ..
                    split_half2(s[1][2], s[1][3], p_hi[3], p_lo[3]);  // row g+8, keys 8+2t, ..
                }
                uint32_t vf[4];
                ldmatrix_x4_trans(vf, tile + v_off);
#pragma unroll
                for (int j = 0; j < 2; j++) {
                    mma_16816(o[j], p_hi, vf[2 * j], vf[2 * j + 1]);
                    if constexpr (!FAST) mma_16816(o[j], p_lo, vf[2 * j], vf[2 * j + 1]);
                }
            }
        }
        __syncthreads();  // everyone is done with buffer c & 1 (it is refilled at the top of iteration c + 1)
    }
    if (aborted) return;

    lA += __shfl_xor_sync(0xffffffffu, lA, 1);
    lA += __shfl_xor_sync(0xffffffffu, lA, 2);
    lB += __shfl_xor_sync(0xffffffffu, lB, 1);
    lB += __shfl_xor_sync(0xffffffffu, lB, 2);
    const float iA = 1.f / fmaxf(lA, 1e-12f), iB = 1.f / fmaxf(lB, 1e-12f);
    const size_t D = (size_t)P.H * DH;
    if (P.out_image) {
        // Operand image of the next projection (see gemm_umma.cu): 128-row tiles x 16-wide k tiles, TF32 high parts
        // then low parts; head h is k tile h.  Lane (g, t) holds columns 8j + 2t, 8j + 2t + 1: half of the 16-byte
        // chunk 2j + t / 2, so a warp store covers eight rows x two chunks = two full 128-byte lines.
        auto put = [&](int row, int j, float a, float b) {
            const size_t grow = (size_t)sd.row0 + row;
            float *tile = P.out_image + ((grow >> 7) * (size_t)P.H + h) * (size_t)(128 * 16 * 2);
            const int rr = (int)(grow & 127), k4 = 2 * j + (t >> 1);
            float *dst = tile + (rr >> 3) * 128 + k4 * 32 + (rr & 7) * 4 + (t & 1) * 2;
            uint32_t ha, hb, la, lb;
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(ha) : "f"(a));
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(hb) : "f"(b));
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(la) : "f"(a - __uint_as_float(ha)));
            asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(lb) : "f"(b - __uint_as_float(hb)));
            *reinterpret_cast<float2 *>(dst) = make_float2(__uint_as_float(ha), __uint_as_float(hb));
            *reinterpret_cast<float2 *>(dst + 128 * 16) = make_float2(__uint_as_float(la), __uint_as_float(lb));
        };
#pragma unroll
        for (int j = 0; j < 2; j++) {
            if (rowA < sd.S) put(rowA, j, o[j][0] * iA, o[j][1] * iA);
            if (rowB < sd.S) put(rowB, j, o[j][2] * iB, o[j][3] * iB);
        }
        return;
    }
#pragma unroll
    for (int j = 0; j < 2; j++) {
        if (rowA < sd.S)
            *reinterpret_cast<float2 *>(P.out + (size_t)(sd.row0 + rowA) * D + h * DH + 8 * j + 2 * t) =
                make_float2(o[j][0] * iA, o[j][1] * iA);
        if (rowB < sd.S)
            *reinterpret_cast<float2 *>(P.out + (size_t)(sd.row0 + rowB) * D + h * DH + 8 * j + 2 * t) =
                make_float2(o[j][2] * iB, o[j][3] * iB);
    }
}

// ------------------------------------------------------------------------------------------------
// Other head sizes: one thread per (sequence, head, query row), keys read from the paged store.
// ------------------------------------------------------------------------------------------------
template <int DH>
__global__ void __launch_bounds__(128) attn_prefill_simt_kernel(const PrefillParams P) {
    const PrefillSeq sd = P.seqs[blockIdx.z];
    const int h = blockIdx.y;
    const int row = blockIdx.x * blockDim.x + threadIdx.x;
    if (row >= sd.S) return;
    const size_t D = (size_t)P.H * DH;
    float q[DH], o[DH];
    {
        const float *qp = P.q + (size_t)(sd.row0 + row) * D + h * DH;
        const float2 *cs = P.rope + (size_t)(sd.rope_off + row) * (DH / 2);
#pragma unroll
        for (int j = 0; j < DH / 2; j++) {
            const float2 w = cs[j];
            q[2 * j] = __fsub_rn(__fmul_rn(qp[2 * j], w.x), __fmul_rn(qp[2 * j + 1], w.y)) * P.scale_log2e;
            q[2 * j + 1] = __fadd_rn(__fmul_rn(qp[2 * j], w.y), __fmul_rn(qp[2 * j + 1], w.x)) * P.scale_log2e;
        }
    }
#pragma unroll
    for (int d = 0; d < DH; d++) o[d] = 0.f;
    float m = -INFINITY, l = 0.f;
    for (int key = 0; key <= row; key++) {
        int phys = P.table[(size_t)sd.seq_id * P.mbs + key / kBlockTokens];
        if (phys < 0 || phys >= P.n_blocks) {
            atomicOr(P.status, DEV_STATUS_BAD_BLOCK);
            phys = 0;
        }
        const __half *kp = P.kv + (((size_t)P.layer * P.n_blocks + phys) * P.H + h) * (2 * kBlockTokens * DH) +
                           (size_t)(key % kBlockTokens) * DH;
        const __half *vp = kp + kBlockTokens * DH;
        float sc = 0.f;
#pragma unroll
        for (int d = 0; d < DH; d++) sc = fmaf(q[d], __half2float(kp[d]), sc);
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
        for (int d = 0; d < DH; d++) o[d] = fmaf(pe, __half2float(vp[d]), o[d]);
    }
    const float inv = 1.f / fmaxf(l, 1e-12f);
    float *op = P.out + (size_t)(sd.row0 + row) * D + h * DH;
#pragma unroll
    for (int d = 0; d < DH; d++) op[d] = o[d] * inv;
}

// ------------------------------------------------------------------------------------------------
// Launcher
// ------------------------------------------------------------------------------------------------
int32_t prefill_upload_descriptors(Pool *p, const int *seq_ids_host, const int *seq_starts_host, const int *rope_offsets_host,
                                   int n_seqs, int *max_S_out, int *n_rows_out) {
    std::vector<PrefillSeq> desc((size_t)n_seqs);
    int max_S = 0;
    for (int i = 0; i < n_seqs; i++) {
        const int s = seq_ids_host[i], S = seq_starts_host[i + 1] - seq_starts_host[i], ro = rope_offsets_host[i];
        JGPT_REQUIRE(s >= 0 && s < p->max_seqs && p->seqs[(size_t)s].used, JGPT_ERR_OUT_OF_RANGE,
                     "seq_ids[%d] = %d is not an allocated sequence", i, s);
        JGPT_REQUIRE(S >= 1 && seq_starts_host[i] >= 0 && (i == 0 ? seq_starts_host[0] == 0 : true), JGPT_ERR_INVALID_ARGUMENT,
                     "sequence %d: seq_starts must begin at 0 and increase", i);
        JGPT_REQUIRE(S <= (int)p->seqs[(size_t)s].blocks.size() * kBlockTokens, JGPT_ERR_ILLEGAL_STATE,
                     "sequence %d: %d prompt tokens exceed the %zu reserved blocks", s, S, p->seqs[(size_t)s].blocks.size());
        JGPT_REQUIRE(ro >= 0 && ro + S <= p->max_positions, JGPT_ERR_INVALID_ARGUMENT,
                     "sequence %d: RoPE positions [%d, %d) outside [0,%d)", s, ro, ro + S, p->max_positions);
        desc[(size_t)i] = PrefillSeq{s, seq_starts_host[i], S, ro};
        max_S = std::max(max_S, S);
    }
    if (n_seqs > p->prefill_desc_cap) {
        JGPT_CUDA_TRY(cudaStreamSynchronize(p->ctx->stream));
        if (p->d_prefill_desc) JGPT_CUDA_TRY(cudaFree(p->d_prefill_desc));
        p->d_prefill_desc = nullptr;
        p->prefill_desc_cap = std::max(n_seqs, 2 * p->prefill_desc_cap);
        JGPT_CUDA_TRY(cudaMalloc(&p->d_prefill_desc, sizeof(PrefillSeq) * (size_t)p->prefill_desc_cap));
    }
    JGPT_CUDA_TRY(cudaMemcpyAsync(p->d_prefill_desc, desc.data(), sizeof(PrefillSeq) * desc.size(), cudaMemcpyHostToDevice,
                                  p->ctx->stream));  // pageable source: staged before the call returns
    *max_S_out = max_S, *n_rows_out = seq_starts_host[n_seqs];
    return JGPT_OK;
}

int32_t launch_attn_prefill(Pool *p, int layer, const float *q, const float *k, const float *v, const int *seq_ids_host,
                            const int *seq_starts_host, const int *rope_offsets_host, int n_seqs, float *out, float *out_image,
                            bool skip_append, int fast_mode) {
    JGPT_REQUIRE(!out_image || p->dhead == 16, JGPT_ERR_INVALID_ARGUMENT, "image output needs d_head 16");
    int max_S = 0, n_rows = 0;
    int32_t rc0 = prefill_upload_descriptors(p, seq_ids_host, seq_starts_host, rope_offsets_host, n_seqs, &max_S, &n_rows);
    if (rc0) return rc0;
    PrefillParams P;
    memset(&P, 0, sizeof(P));
    P.kv = p->kv, P.table = p->d_table, P.rope = p->d_rope, P.q = q, P.k = k, P.v = v, P.out = out, P.out_image = out_image;
    P.seqs = reinterpret_cast<const PrefillSeq *>(p->d_prefill_desc), P.status = p->ctx->d_status;
    P.n_seqs = n_seqs, P.n_rows = n_rows, P.H = p->heads, P.layer = layer, P.n_blocks = p->n_blocks;
    P.mbs = p->max_blocks_per_seq, P.max_positions = p->max_positions;
    P.scale_log2e = (1.0f / sqrtf((float)p->dhead)) * 1.4426950408889634f;
    const int DH = p->dhead;
    const int cpr = DH / (DH < 8 ? DH : 8);
    const long long total = (long long)n_rows * p->heads * cpr;
    const unsigned agrid = (unsigned)((total + 255) / 256);
    cudaStream_t st = p->ctx->stream;
    if (!skip_append) {  // skipped when the K / V projection's epilogue has already written the paged store
        switch (DH) {
            case 4: kv_append_rows_kernel<4><<<agrid, 256, 0, st>>>(P); break;
            case 8: kv_append_rows_kernel<8><<<agrid, 256, 0, st>>>(P); break;
            case 16: kv_append_rows_kernel<16><<<agrid, 256, 0, st>>>(P); break;
            case 32: kv_append_rows_kernel<32><<<agrid, 256, 0, st>>>(P); break;
            default: return fail(JGPT_ERR_UNSUPPORTED, "dhead %d not supported", DH);
        }
        JGPT_CUDA_TRY(cudaGetLastError());
    }
    if (DH == 16) {
        dim3 grid((unsigned)((max_S + kQTile - 1) / kQTile), (unsigned)p->heads, (unsigned)n_seqs);
        const size_t smem = sizeof(int) * (size_t)((max_S + kBlockTokens - 1) / kBlockTokens);
        const bool fast = fast_mode < 0 ? p->prefill_fast != 0 : fast_mode != 0;
        if (fast) attn_prefill_mma_kernel<true><<<grid, 128, smem, st>>>(P);
        else attn_prefill_mma_kernel<false><<<grid, 128, smem, st>>>(P);
    } else {
        dim3 grid((unsigned)((max_S + 127) / 128), (unsigned)p->heads, (unsigned)n_seqs);
        switch (DH) {
            case 4: attn_prefill_simt_kernel<4><<<grid, 128, 0, st>>>(P); break;
            case 8: attn_prefill_simt_kernel<8><<<grid, 128, 0, st>>>(P); break;
            default: attn_prefill_simt_kernel<32><<<grid, 128, 0, st>>>(P); break;
        }
    }
    JGPT_CUDA_TRY(cudaGetLastError());
    return JGPT_OK;
}

}  // namespace jgpt

using namespace jgpt;

extern "C" int32_t jgpt_attn_prefill(jgpt_kvpool pool, int32_t layer, const float *q_dev, const float *k_dev, const float *v_dev,
                                     const int32_t *seq_ids_host, const int32_t *seq_starts_host,
                                     const int32_t *rope_offsets_host, int32_t n_seqs, float *out_dev) {
    Pool *p = pool_registry().get(pool);
    JGPT_REQUIRE(p, JGPT_ERR_BAD_HANDLE, "bad kvpool handle");
    JGPT_CUDA_TRY(make_current(p->ctx));
    JGPT_REQUIRE(layer >= 0 && layer < p->layers, JGPT_ERR_OUT_OF_RANGE, "layer %d outside [0,%d)", layer, p->layers);
    if (n_seqs == 0) return JGPT_OK;
    JGPT_REQUIRE(n_seqs > 0 && q_dev && k_dev && v_dev && seq_ids_host && seq_starts_host && rope_offsets_host && out_dev,
                 JGPT_ERR_INVALID_ARGUMENT, "null pointer or negative count");
    return launch_attn_prefill(p, layer, q_dev, k_dev, v_dev, seq_ids_host, seq_starts_host, rope_offsets_host, n_seqs, out_dev);
}
