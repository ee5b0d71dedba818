// Large-M fp32 projections on the 5th-generation tensor cores (tcgen05.mma, accumulator in tensor memory).
// Host-side interface of gemm_umma.cu; operands are pre-tiled "images" (see the layout note there).
#pragma once

#include "common.cuh"

namespace jgpt {
namespace umma {

constexpr int BM = 128;   // rows of C per CTA (one TMEM lane per row)
constexpr int BN = 256;   // columns of C per CTA (one fp32 TMEM column per column)
constexpr int BK = 16;    // k extent of one pipeline stage (two K=8 tensor-core steps)

// Floats of the tiled hi/lo image of a [rows, K] operand whose rows are grouped in tiles of `tile_rows`.
inline uint64_t image_floats(int rows, int K, int tile_rows) {
    const uint64_t tiles = (uint64_t)(rows + tile_rows - 1) / tile_rows;
    return tiles * (uint64_t)tile_rows * (uint64_t)K * 2u;
}

// A[M, K] row major (row r taken from rowsel[r] when rowsel != nullptr) -> image with 128-row tiles.
int32_t pack_activations(const float *A, const int *rowsel, int M, int K, float *image, cudaStream_t st);
// W[K, N] row major -> image of W^T (rows = output columns) with 256-row tiles.
int32_t pack_weight(const float *W, int K, int N, float *image, cudaStream_t st);

struct Batch {
    const float *Wimg[3];
    float *C[3];
    const float *R[3];  // optional residual, may alias C
};
// C_z[M, N] = A . W_z (+ R_z) for z < nb; needs K % 16 == 0 and N % 4 == 0.
int32_t launch(const float *Aimg, const Batch &b, int nb, int M, int K, int N, int *d_status, cudaStream_t st);

inline bool shape_ok(int K, int N) { return K >= BK && K % BK == 0 && N % 4 == 0; }

}  // namespace umma
}  // namespace jgpt
