// Large-M fp32 projections on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
// Host-side interface of gemm_umma.cu; operands are pre-tiled "images" (see the layout note there).
#pragma once

#include "common.cuh"

namespace jgpt {
namespace umma {

constexpr int BM = 128;  // rows of C per CTA (one TMEM lane per row)
constexpr int BK = 16;   // k extent of one pipeline stage (two K=8 tensor-core steps)

// Columns of C per CTA (one fp32 TMEM column per column): the widest tile that leaves no padded columns.
inline int tile_cols(int N) { return N % 256 == 0 ? 256 : (N % 192 == 0 ? 192 : 256); }

// Floats of the tiled hi/lo image of a [rows, K] operand whose rows are grouped in tiles of `tile_rows`.
inline uint64_t image_floats(int rows, int K, int tile_rows) {
    const uint64_t tiles = (uint64_t)(rows + tile_rows - 1) / tile_rows;
    return tiles * (uint64_t)tile_rows * (uint64_t)K * 2u;
}
inline uint64_t activation_image_floats(int M, int K) { return image_floats(M, K, BM); }
inline uint64_t weight_image_floats(int K, int N) { return image_floats(N, K, tile_cols(N)); }

// A[M, K] row major (row r taken from rowsel[r] when rowsel != nullptr) -> activation image.
int32_t pack_activations(const float *A, const int *rowsel, int M, int K, float *image, cudaStream_t st);
// RMSNorm of x[M, D] with gamma, written straight into an activation image (same arithmetic as the row-major
// RMSNorm kernel of the forward step).
int32_t rmsnorm_pack(const float *x, const float *gamma, int M, int D, float eps, float *image, cudaStream_t st);
// W[K, N] row major -> image of W^T (rows = output columns) in tiles of tile_cols(N) rows.
int32_t pack_weight(const float *W, int K, int N, float *image, cudaStream_t st);
// W1, W3 [K, F] -> one image of 2F rows in 256-row tiles: tile t = columns [128 t, 128 t + 128) of W1
// followed by the same columns of W3 (needs F % 128 == 0).
int32_t pack_weight_pair(const float *W1, const float *W3, int K, int F, float *image, cudaStream_t st);

struct Batch {
    const float *Wimg[3];
    float *C[3];
    const float *R[3];  // optional residual, may alias C
};
// C_z[M, N] = A . W_z (+ R_z) for z < nb; needs K % 16 == 0 and N % 4 == 0.
int32_t launch(const float *Aimg, const Batch &b, int nb, int M, int K, int N, int *d_status, cudaStream_t st);
// act = (A . W1) * silu(A . W3), written as the activation image [M, F] of the next product.
int32_t launch_swiglu(const float *Aimg, const float *Wpair_img, int M, int K, int F, float *act_image, int *d_status,
                      cudaStream_t st);

// The Q, K, V products of a prefill (b.Wimg[0..2]; d_head 16, N = heads * 16): Q goes to b.C[0] row major, K gets its
// RoPE and both K and V are written as fp16 straight into the paged store - the arithmetic and the stores of the
// append kernel, without the fp32 round trip through memory.
int32_t launch_qkv_paged(const float *Aimg, const Batch &b, int M, int K, int N, const PagedAppendArgs &pa, int *d_status,
                         cudaStream_t st);

inline bool shape_ok(int K, int N) { return K >= BK && K % BK == 0 && N % 4 == 0; }
inline bool swiglu_shape_ok(int K, int F) { return K >= BK && K % BK == 0 && F % 128 == 0; }

}  // namespace umma
}  // namespace jgpt
