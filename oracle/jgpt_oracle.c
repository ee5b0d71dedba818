/*
 * CPU oracle for the JGPT KV-cache decode path.  TEST INFRASTRUCTURE ONLY.
 *
 * This file is a plain-C restatement (fp32, batch 1, contiguous KV cache) of what the
 * reference computes on its generation path.  It exists so that the CUDA library can be
 * checked against it; nothing in the shipped library links, loads or calls it.  Only the
 * test-suite, the smoke check and the CPU-baseline leg of the benchmark may use it.
 *
 * Parity status: the reference holds no golden vectors for this path (its tests compare
 * two of its own paths on unseeded random weights).  The oracle is pinned to the literal
 * known-answer cases of the reference's op tests (RMSNorm, matmul, softmax, sigmoid,
 * split/concat: src/test/java/com/veles/llm/jgpt/ops/TensorOpsTest.java:70-196) and to the
 * invariants of src/test/java/com/veles/llm/jgpt/model/KvCacheTest.java:14-70
 * (prefill == full forward, decode == row of forward).  Everything the reference does not
 * have at all (paged blocks, block tables, eviction) is "parity unpinned" by the reference
 * and is defined by equivalence to the contiguous layout restated here.
 *
 * Every function cites the reference file:line it follows.  Paths are relative to the
 * reference project root; KL = src/main/cpp/jgpt_cuda_extra_kernels_launches.inl,
 * J = src/main/java/com/veles/llm/jgpt.
 *
 * Build: see oracle/Makefile (-O2 -ffp-contract=off so that a*b-c*d is two roundings, the
 * same as the explicit __fmul_rn/__fsub_rn sequence in the CUDA append kernel).
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define OG_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------------------------
 * Elementary ops
 * ---------------------------------------------------------------------------------------- */

/* RMSNorm: KL:668-686 (thread-per-row) and KL:694-713 (block-per-row) compute the same thing:
 * rms = sqrtf(sum(x^2)/D + eps); inv = (rms>0 && finite) ? 1/rms : 0; y = x*inv*gamma. */
OG_API void og_rmsnorm(const float *x, const float *gamma, float *out, int rows, int D, float eps) {
    for (int r = 0; r < rows; r++) {
        const float *xr = x + (size_t)r * D;
        float *orow = out + (size_t)r * D;
        float ss = 0.f;
        for (int j = 0; j < D; j++) ss += xr[j] * xr[j];
        float rms = sqrtf(ss / (float)D + eps);
        float inv = (rms > 0.f && isfinite(rms)) ? (1.f / rms) : 0.f;
        for (int j = 0; j < D; j++) orow[j] = xr[j] * inv * gamma[j];
    }
}

/* Row-major C[M,N] = A[M,K] * B[K,N], fp32 accumulate in k order.
 * Reference: cuBLAS Sgemm call sites, src/main/cpp/jgpt_cuda_jni_init_matmul.inl:67 (matmulGPU);
 * J/ops/TensorOps.java:2807-2835.  The reference runs Sgemm under TF32 math mode; this is exact
 * fp32, i.e. the value the reference approximates. */
OG_API void og_matmul(const float *A, const float *B, float *C, int M, int K, int N) {
    if (M >= 4) {
#pragma omp parallel for schedule(static)
        for (int i = 0; i < M; i++) {
            float *c = C + (size_t)i * N;
            for (int j = 0; j < N; j++) c[j] = 0.f;
            for (int k = 0; k < K; k++) {
                const float a = A[(size_t)i * K + k];
                const float *b = B + (size_t)k * N;
                for (int j = 0; j < N; j++) c[j] += a * b[j];
            }
        }
    } else {
        for (int i = 0; i < M; i++) {
            float *c = C + (size_t)i * N;
            const int chunk = 256;
            const int nchunks = (N + chunk - 1) / chunk;
#pragma omp parallel for schedule(static) if (N * (long)K > 200000)
            for (int cj = 0; cj < nchunks; cj++) {
                const int j0 = cj * chunk, j1 = (j0 + chunk < N) ? j0 + chunk : N;
                for (int j = j0; j < j1; j++) c[j] = 0.f;
                for (int k = 0; k < K; k++) {
                    const float a = A[(size_t)i * K + k];
                    const float *b = B + (size_t)k * N;
                    for (int j = j0; j < j1; j++) c[j] += a * b[j];
                }
            }
        }
    }
}

/* Softmax over the last axis.  KL:13-34 (inner < 64: 1/sum) and KL:176-201 (inner >= 64:
 * 1/max(sum,1e-12)); dispatch threshold as in launch helper (thread-per-row for inner < 64). */
OG_API void og_softmax_last_dim(const float *src, float *dst, long rows, int inner) {
    for (long r = 0; r < rows; r++) {
        const float *s = src + r * inner;
        float *d = dst + r * inner;
        float m = -INFINITY;
        for (int j = 0; j < inner; j++) m = fmaxf(m, s[j]);
        float sum = 0.f;
        for (int j = 0; j < inner; j++) {
            float e = expf(s[j] - m);
            d[j] = e;
            sum += e;
        }
        float inv = (inner < 64) ? (1.f / sum) : (1.f / fmaxf(sum, 1e-12f));
        for (int j = 0; j < inner; j++) d[j] *= inv;
    }
}

/* Sigmoid with the reference's clamps: KL:799-815. */
static inline float og_sigmoid1(float x) {
    if (x >= 20.f) return 1.f;
    if (x <= -20.f) return 0.f;
    return 1.f / (1.f + expf(-x));
}
OG_API void og_sigmoid(const float *src, float *dst, int n) {
    for (int i = 0; i < n; i++) dst[i] = og_sigmoid1(src[i]);
}

/* [B,S,D] -> [B,H,S,Dh] and back: KL:1063-1083, KL:1101-1125. */
OG_API void og_split_heads(const float *src, float *dst, int B, int S, int D, int H) {
    const int Dh = D / H;
    for (int b = 0; b < B; b++)
        for (int h = 0; h < H; h++)
            for (int s = 0; s < S; s++)
                for (int j = 0; j < Dh; j++)
                    dst[(((size_t)b * H + h) * S + s) * Dh + j] = src[((size_t)b * S + s) * D + h * Dh + j];
}
OG_API void og_concat_heads(const float *src, float *dst, int B, int H, int S, int Dh) {
    const int D = H * Dh;
    for (int b = 0; b < B; b++)
        for (int h = 0; h < H; h++)
            for (int s = 0; s < S; s++)
                for (int j = 0; j < Dh; j++)
                    dst[((size_t)b * S + s) * D + h * Dh + j] = src[(((size_t)b * H + h) * S + s) * Dh + j];
}

/* Interleaved-pair RoPE on [B,H,S,Dh]: KL:1127-1159.  position = positions[i] (i < nPos) or
 * i + posBaseOffset.  theta = (float)p / powf(10000, 2j/Dh). */
OG_API void og_rope_cos_sin(int p, int j, int Dh, float *c, float *s) {
    float theta = (float)p / powf(10000.f, (2.f * (float)j) / (float)Dh);
    *c = cosf(theta);
    *s = sinf(theta);
}
OG_API void og_rope_4d(const float *src, float *dst, int B, int H, int S, int Dh, const int *positions, int nPos,
                       int posBaseOffset) {
    const int half = Dh / 2;
    for (int b = 0; b < B; b++)
        for (int h = 0; h < H; h++)
            for (int i = 0; i < S; i++) {
                const size_t base = (((size_t)b * H + h) * S + i) * Dh;
                const int p = (positions != NULL && i < nPos) ? positions[i] : (i + posBaseOffset);
                for (int j = 0; j < half; j++) {
                    float c, s;
                    og_rope_cos_sin(p, j, Dh, &c, &s);
                    const float x1 = src[base + 2 * j], x2 = src[base + 2 * j + 1];
                    dst[base + 2 * j] = x1 * c - x2 * s;
                    dst[base + 2 * j + 1] = x1 * s + x2 * c;
                }
            }
}

/* Round an fp32 value through IEEE binary16, round-to-nearest-even, as the reference's
 * float_to_half kernel (__float2half_rn, src/main/cpp/jgpt_cuda_kernels_launches_macros.inl:68). */
OG_API float og_round_fp16(float x) { return (float)(_Float16)x; }

/* ------------------------------------------------------------------------------------------
 * Contiguous KV cache: J/model/KvCache.java:13-105; index h*maxSeq*Dh + pos*Dh + j
 * (J/ops/TensorOps.java:2513-2557; kernel KL:1085-1099).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    int layers, heads, dhead, max_seq, length;
    int kv_fp16; /* test mode: round payload through binary16 on write (what a fp16 store holds) */
    float **k, **v;
} og_cache;

OG_API og_cache *og_cache_create(int layers, int heads, int dhead, int max_seq) {
    if (layers <= 0 || heads <= 0 || dhead <= 0 || max_seq <= 0) return NULL; /* KvCache.java ctor: IAE */
    og_cache *c = (og_cache *)calloc(1, sizeof(og_cache));
    c->layers = layers, c->heads = heads, c->dhead = dhead, c->max_seq = max_seq;
    c->k = (float **)calloc(layers, sizeof(float *));
    c->v = (float **)calloc(layers, sizeof(float *));
    for (int l = 0; l < layers; l++) {
        c->k[l] = (float *)calloc((size_t)heads * max_seq * dhead, sizeof(float));
        c->v[l] = (float *)calloc((size_t)heads * max_seq * dhead, sizeof(float));
    }
    return c;
}
OG_API void og_cache_free(og_cache *c) {
    if (!c) return;
    for (int l = 0; l < c->layers; l++) free(c->k[l]), free(c->v[l]);
    free(c->k), free(c->v), free(c);
}
OG_API void og_cache_clear(og_cache *c) { /* KvCache.clear(): zero-fill + length 0 */
    for (int l = 0; l < c->layers; l++) {
        memset(c->k[l], 0, sizeof(float) * (size_t)c->heads * c->max_seq * c->dhead);
        memset(c->v[l], 0, sizeof(float) * (size_t)c->heads * c->max_seq * c->dhead);
    }
    c->length = 0;
}
/* Block-granular rolling window (no reference counterpart; the reference clears the cache and re-prefills,
 * J/model/GptAutoregressiveGenerator.java:51-88): forget the oldest n_tokens cached tokens.  Rows [n, length) of every
 * head move to [0, length - n) with their payload untouched (keys keep the RoPE of their absolute positions), the
 * vacated tail is zeroed, the length drops by n.  -1 unless 0 <= n_tokens <= length. */
OG_API int og_cache_drop_front(og_cache *c, int n_tokens) {
    if (n_tokens < 0 || n_tokens > c->length) return -1;
    const size_t row = (size_t)c->dhead;
    for (int l = 0; l < c->layers; l++)
        for (int h = 0; h < c->heads; h++) {
            float *planes[2] = {c->k[l] + (size_t)h * c->max_seq * row, c->v[l] + (size_t)h * c->max_seq * row};
            for (int t = 0; t < 2; t++) {
                memmove(planes[t], planes[t] + (size_t)n_tokens * row, sizeof(float) * (size_t)(c->length - n_tokens) * row);
                memset(planes[t] + (size_t)(c->length - n_tokens) * row, 0, sizeof(float) * (size_t)n_tokens * row);
            }
        }
    c->length -= n_tokens;
    return 0;
}
OG_API int og_cache_length(const og_cache *c) { return c->length; }
OG_API int og_cache_set_length(og_cache *c, int len) { /* KvCache.setLength: IAE unless 0<=len<=maxSeq */
    if (len < 0 || len > c->max_seq) return -1;
    c->length = len;
    return 0;
}
OG_API void og_cache_set_kv_fp16(og_cache *c, int on) { c->kv_fp16 = on; }
OG_API float *og_cache_k(og_cache *c, int layer) { return (layer < 0 || layer >= c->layers) ? NULL : c->k[layer]; }
OG_API float *og_cache_v(og_cache *c, int layer) { return (layer < 0 || layer >= c->layers) ? NULL : c->v[layer]; }

/* Write S tokens of head-major [H,S,Dh] into the cache at positions pos0..pos0+S-1
 * (TensorOps.copyKvHeadsIntoCache :2513-2535 with pos0 = 0; copyKvOneTokenIntoCache :2537-2557
 * with S = 1, pos0 = cacheLenBefore). */
static void og_cache_write(const og_cache *c, float *dst, const float *heads4d, int S, int pos0) {
    const int H = c->heads, Dh = c->dhead, MS = c->max_seq;
    for (int h = 0; h < H; h++)
        for (int s = 0; s < S; s++)
            for (int j = 0; j < Dh; j++) {
                float v = heads4d[((size_t)h * S + s) * Dh + j];
                if (c->kv_fp16) v = og_round_fp16(v);
                dst[(size_t)h * MS * Dh + (size_t)(pos0 + s) * Dh + j] = v;
            }
}

/* ------------------------------------------------------------------------------------------
 * Attention
 * ---------------------------------------------------------------------------------------- */

/* Single-query attention for one head over `len` cached keys:
 * J/ops/TensorOps.java:1088-1140 (scores = q.K^T, * scale, softmaxLastDim, .V).
 * kc/vc point at the head's [maxSeq, Dh] plane (only the first len rows are read). */
OG_API void og_attn_query_one(const float *q, const float *kc, const float *vc, int len, int Dh, float scale,
                              float *out, float *scratch /* >= len floats */) {
    for (int j = 0; j < len; j++) {
        float s = 0.f;
        for (int d = 0; d < Dh; d++) s += q[d] * kc[(size_t)j * Dh + d];
        scratch[j] = s * scale;
    }
    og_softmax_last_dim(scratch, scratch, 1, len);
    for (int d = 0; d < Dh; d++) out[d] = 0.f;
    for (int j = 0; j < len; j++) {
        const float p = scratch[j];
        for (int d = 0; d < Dh; d++) out[d] += p * vc[(size_t)j * Dh + d];
    }
}

/* Causal prefill attention on head-major [H,S,Dh]: J/ops/TensorOps.java:990-1041 with the 0/-inf
 * mask of :956-973; native softmax(scale*s + mask) KL:239-276.  The loop nest is the one the
 * reference itself writes as CPU code in src/test/java/com/veles/llm/jgpt/ops/AttentionForwardGpuTest.java:44-81. */
OG_API void og_attn_prefill_causal(const float *Q, const float *K, const float *V, float *out, int H, int S, int Dh,
                                   float scale) {
#pragma omp parallel for schedule(dynamic, 1)
    for (int h = 0; h < H; h++) {
        float *z = (float *)malloc(sizeof(float) * S);
        for (int i = 0; i < S; i++) {
            const float *q = Q + ((size_t)h * S + i) * Dh;
            float m = -INFINITY;
            for (int j = 0; j < S; j++) {
                float s = 0.f;
                for (int d = 0; d < Dh; d++) s += q[d] * K[((size_t)h * S + j) * Dh + d];
                float v = s * scale + ((j > i) ? -INFINITY : 0.f);
                z[j] = v;
                m = fmaxf(m, v);
            }
            float sum = 0.f;
            for (int j = 0; j < S; j++) sum += expf(z[j] - m);
            const float inv = 1.f / fmaxf(sum, 1e-12f);
            float *o = out + ((size_t)h * S + i) * Dh;
            for (int d = 0; d < Dh; d++) o[d] = 0.f;
            for (int j = 0; j < S; j++) {
                const float p = expf(z[j] - m) * inv;
                for (int d = 0; d < Dh; d++) o[d] += p * V[((size_t)h * S + j) * Dh + d];
            }
        }
        free(z);
    }
}

/* ------------------------------------------------------------------------------------------
 * Model: parameter order J/model/GPTModel.java:1928-1938, J/model/DecoderBlock.java:42-52
 * (Wq,Wk,Wv,Wo,W1,W2,W3,norm1,norm2); all matrices used as y = x.W (row-major [in,out]).
 * ---------------------------------------------------------------------------------------- */
typedef struct {
    float *wq, *wk, *wv, *wo, *w1, *w2, *w3, *norm1, *norm2;
} og_layer;
typedef struct {
    int vocab, max_seq, d_model, heads, layers, d_ff;
    float eps;
    float *tok, *pos, *norm_final, *lm_head;
    og_layer *L;
} og_model;

OG_API og_model *og_model_create(int vocab, int max_seq, int d_model, int heads, int layers, int d_ff, float eps) {
    if (vocab <= 0 || max_seq <= 0 || d_model <= 0 || heads <= 0 || layers <= 0 || d_ff <= 0) return NULL;
    if (d_model % heads != 0) return NULL;
    og_model *m = (og_model *)calloc(1, sizeof(og_model));
    m->vocab = vocab, m->max_seq = max_seq, m->d_model = d_model, m->heads = heads, m->layers = layers;
    m->d_ff = d_ff, m->eps = eps;
    const size_t D = d_model, F = d_ff;
    m->tok = (float *)calloc((size_t)vocab * D, 4);
    m->pos = (float *)calloc((size_t)max_seq * D, 4);
    m->norm_final = (float *)calloc(D, 4);
    m->lm_head = (float *)calloc(D * vocab, 4);
    m->L = (og_layer *)calloc(layers, sizeof(og_layer));
    for (int l = 0; l < layers; l++) {
        og_layer *y = &m->L[l];
        y->wq = (float *)calloc(D * D, 4), y->wk = (float *)calloc(D * D, 4);
        y->wv = (float *)calloc(D * D, 4), y->wo = (float *)calloc(D * D, 4);
        y->w1 = (float *)calloc(D * F, 4), y->w2 = (float *)calloc(F * D, 4), y->w3 = (float *)calloc(D * F, 4);
        y->norm1 = (float *)calloc(D, 4), y->norm2 = (float *)calloc(D, 4);
    }
    return m;
}
OG_API void og_model_free(og_model *m) {
    if (!m) return;
    for (int l = 0; l < m->layers; l++) {
        og_layer *y = &m->L[l];
        free(y->wq), free(y->wk), free(y->wv), free(y->wo), free(y->w1), free(y->w2), free(y->w3);
        free(y->norm1), free(y->norm2);
    }
    free(m->L), free(m->tok), free(m->pos), free(m->norm_final), free(m->lm_head), free(m);
}

/* Number of parameter tensors and the i-th tensor (pointer, rank, dims) in file order. */
OG_API int og_model_num_tensors(const og_model *m) { return 4 + 9 * m->layers; }
OG_API float *og_model_tensor(og_model *m, int idx, int *rank, int *d0, int *d1) {
    const int D = m->d_model, F = m->d_ff, V = m->vocab, n = og_model_num_tensors(m);
    if (idx < 0 || idx >= n) return NULL;
    if (idx == 0) { *rank = 2, *d0 = V, *d1 = D; return m->tok; }
    if (idx == 1) { *rank = 2, *d0 = m->max_seq, *d1 = D; return m->pos; }
    if (idx == n - 2) { *rank = 1, *d0 = D, *d1 = 1; return m->norm_final; }
    if (idx == n - 1) { *rank = 2, *d0 = D, *d1 = V; return m->lm_head; }
    og_layer *y = &m->L[(idx - 2) / 9];
    switch ((idx - 2) % 9) {
        case 0: *rank = 2, *d0 = D, *d1 = D; return y->wq;
        case 1: *rank = 2, *d0 = D, *d1 = D; return y->wk;
        case 2: *rank = 2, *d0 = D, *d1 = D; return y->wv;
        case 3: *rank = 2, *d0 = D, *d1 = D; return y->wo;
        case 4: *rank = 2, *d0 = D, *d1 = F; return y->w1;
        case 5: *rank = 2, *d0 = F, *d1 = D; return y->w2;
        case 6: *rank = 2, *d0 = D, *d1 = F; return y->w3;
        case 7: *rank = 1, *d0 = D, *d1 = 1; return y->norm1;
        default: *rank = 1, *d0 = D, *d1 = 1; return y->norm2;
    }
}

/* veles.weights.v1: writer J/training/LlmTrainerCheckpointIo.java:129-140, reader
 * J/model/GptModelWeightsLoader.java:58-81.  u16 BE length + "veles.weights.v1" (Java writeUTF),
 * i32 BE tensor count, then per tensor i32 BE rank, rank x i32 BE dims, big-endian f32 payload. */
static void put_be32(FILE *f, uint32_t v) {
    unsigned char b[4] = {(unsigned char)(v >> 24), (unsigned char)(v >> 16), (unsigned char)(v >> 8), (unsigned char)v};
    fwrite(b, 1, 4, f);
}
static int get_be32(FILE *f, uint32_t *v) {
    unsigned char b[4];
    if (fread(b, 1, 4, f) != 4) return -1;
    *v = ((uint32_t)b[0] << 24) | ((uint32_t)b[1] << 16) | ((uint32_t)b[2] << 8) | b[3];
    return 0;
}
OG_API int og_model_save(og_model *m, const char *path) {
    FILE *f = fopen(path, "wb");
    if (!f) return -1;
    const char *tag = "veles.weights.v1";
    unsigned char l2[2] = {0, 16};
    fwrite(l2, 1, 2, f), fwrite(tag, 1, 16, f);
    const int n = og_model_num_tensors(m);
    put_be32(f, (uint32_t)n);
    for (int i = 0; i < n; i++) {
        int rank, d0, d1;
        float *p = og_model_tensor(m, i, &rank, &d0, &d1);
        put_be32(f, (uint32_t)rank), put_be32(f, (uint32_t)d0);
        if (rank == 2) put_be32(f, (uint32_t)d1);
        const size_t cnt = (size_t)d0 * (rank == 2 ? d1 : 1);
        for (size_t j = 0; j < cnt; j++) {
            uint32_t u;
            memcpy(&u, p + j, 4);
            put_be32(f, u);
        }
    }
    fclose(f);
    return 0;
}
OG_API int og_model_load(og_model *m, const char *path) {
    FILE *f = fopen(path, "rb");
    if (!f) return -1;
    unsigned char hdr[18];
    if (fread(hdr, 1, 18, f) != 18 || hdr[0] != 0 || hdr[1] != 16 || memcmp(hdr + 2, "veles.weights.v1", 16) != 0) {
        fclose(f);
        return -2;
    }
    uint32_t n;
    if (get_be32(f, &n) || (int)n != og_model_num_tensors(m)) { fclose(f); return -3; }
    for (int i = 0; i < (int)n; i++) {
        int rank, d0, d1;
        float *p = og_model_tensor(m, i, &rank, &d0, &d1);
        uint32_t r, a, b = 1;
        if (get_be32(f, &r) || (int)r != rank || get_be32(f, &a) || (int)a != d0) { fclose(f); return -4; }
        if (rank == 2 && (get_be32(f, &b) || (int)b != d1)) { fclose(f); return -4; }
        const size_t cnt = (size_t)d0 * (rank == 2 ? d1 : 1);
        for (size_t j = 0; j < cnt; j++) {
            uint32_t u;
            if (get_be32(f, &u)) { fclose(f); return -5; }
            memcpy(p + j, &u, 4);
        }
    }
    fclose(f);
    return 0;
}

/* Embedding + learned absolute position rows: J/model/GptKvForward.java:25-26, 102-103;
 * kernels KL:937-955 and KL:1020-1032.  Returns -1 on an id or a position row out of range
 * (the reference throws IllegalArgumentException: J/model/TokenEmbedding.java:158-203,
 * J/model/PositionEmbedding.java:64-105). */
static int og_embed(const og_model *m, const int *ids, int S, int pos_row_start, float *x) {
    const int D = m->d_model;
    if (pos_row_start < 0 || pos_row_start + S > m->max_seq) return -1;
    for (int s = 0; s < S; s++) {
        if (ids[s] < 0 || ids[s] >= m->vocab) return -1;
        const float *t = m->tok + (size_t)ids[s] * D, *p = m->pos + (size_t)(pos_row_start + s) * D;
        for (int j = 0; j < D; j++) x[(size_t)s * D + j] = t[j] + p[j];
    }
    return 0;
}

/* FFN half of the block: J/ops/TensorOps.java:405-465, fused variant :566-667.
 * x1 = x + a;  n2 = rmsnorm(x1);  h1 = n2.W1;  g = n2.W3;  act = h1 * (g*sigmoid(g));  x = x1 + act.W2. */
static void og_ffn_residual(const og_model *m, const og_layer *y, float *x /* [S,D] in/out = x1 */, int S) {
    const int D = m->d_model, F = m->d_ff;
    float *n2 = (float *)malloc(sizeof(float) * (size_t)S * D);
    float *h1 = (float *)malloc(sizeof(float) * (size_t)S * F);
    float *g = (float *)malloc(sizeof(float) * (size_t)S * F);
    float *f = (float *)malloc(sizeof(float) * (size_t)S * D);
    og_rmsnorm(x, y->norm2, n2, S, D, m->eps);
    og_matmul(n2, y->w1, h1, S, D, F);
    og_matmul(n2, y->w3, g, S, D, F);
    for (size_t i = 0; i < (size_t)S * F; i++) {
        const float sg = og_sigmoid1(g[i]);
        const float gate = g[i] * sg;
        h1[i] = h1[i] * gate;
    }
    og_matmul(h1, y->w2, f, S, F, D);
    for (size_t i = 0; i < (size_t)S * D; i++) x[i] = x[i] + f[i];
    free(n2), free(h1), free(g), free(f);
}

/* Attention half for S tokens (prefill, J/ops/TensorOps.java:2148-2234) or one token (decode,
 * :2239-2309).  cache may be NULL (full forward without a cache).  On return x holds x + attn.Wo. */
static void og_attn_residual(const og_model *m, const og_layer *y, float *x, int S, og_cache *cache, int layer,
                             int decode, int cache_len_before, int rope_offset_or_pos) {
    const int D = m->d_model, H = m->heads, Dh = D / H;
    const float scale = 1.0f / (float)sqrt((double)Dh);
    const size_t SD = (size_t)S * D;
    float *n1 = (float *)malloc(4 * SD), *q = (float *)malloc(4 * SD), *k = (float *)malloc(4 * SD);
    float *v = (float *)malloc(4 * SD), *qh = (float *)malloc(4 * SD), *kh = (float *)malloc(4 * SD);
    float *vh = (float *)malloc(4 * SD), *oh = (float *)malloc(4 * SD), *cat = (float *)malloc(4 * SD);
    float *a = (float *)malloc(4 * SD);
    og_rmsnorm(x, y->norm1, n1, S, D, m->eps);
    og_matmul(n1, y->wq, q, S, D, D);
    og_matmul(n1, y->wk, k, S, D, D);
    og_matmul(n1, y->wv, v, S, D, D);
    og_split_heads(q, qh, 1, S, D, H);
    og_split_heads(k, kh, 1, S, D, H);
    og_split_heads(v, vh, 1, S, D, H);
    if (decode) {
        int p = rope_offset_or_pos; /* explicit position array {ropePosition} */
        og_rope_4d(qh, qh, 1, H, 1, Dh, &p, 1, 0);
        og_rope_4d(kh, kh, 1, H, 1, Dh, &p, 1, 0);
        og_cache_write(cache, cache->k[layer], kh, 1, cache_len_before);
        og_cache_write(cache, cache->v[layer], vh, 1, cache_len_before);
        const int len = cache_len_before + 1;
        float *scr = (float *)malloc(4 * (size_t)len);
        for (int h = 0; h < H; h++)
            og_attn_query_one(qh + (size_t)h * Dh, cache->k[layer] + (size_t)h * cache->max_seq * Dh,
                              cache->v[layer] + (size_t)h * cache->max_seq * Dh, len, Dh, scale, oh + (size_t)h * Dh,
                              scr);
        free(scr);
    } else {
        og_rope_4d(qh, qh, 1, H, S, Dh, NULL, 0, rope_offset_or_pos);
        og_rope_4d(kh, kh, 1, H, S, Dh, NULL, 0, rope_offset_or_pos);
        if (cache) {
            og_cache_write(cache, cache->k[layer], kh, S, 0);
            og_cache_write(cache, cache->v[layer], vh, S, 0);
            if (cache->kv_fp16) { /* attend over what the store holds */
                for (size_t i = 0; i < SD; i++) kh[i] = og_round_fp16(kh[i]), vh[i] = og_round_fp16(vh[i]);
            }
        }
        og_attn_prefill_causal(qh, kh, vh, oh, H, S, Dh, scale);
    }
    og_concat_heads(oh, cat, 1, H, S, Dh);
    og_matmul(cat, y->wo, a, S, D, D);
    for (size_t i = 0; i < SD; i++) x[i] = x[i] + a[i];
    free(n1), free(q), free(k), free(v), free(qh), free(kh), free(vh), free(oh), free(cat), free(a);
}

/* forwardPrefill: J/model/GptKvForward.java:12-90.  logits [S,V].  Error codes mirror the
 * reference's exceptions: -1 IllegalArgument (S > maxSeq, layer mismatch, id/pos out of range). */
OG_API int og_forward_prefill(const og_model *m, const int *ids, int S, og_cache *cache, int rope_offset,
                              float *logits) {
    const int D = m->d_model;
    if (S <= 0 || S > m->max_seq) return -1;
    if (cache && (cache->layers != m->layers || S > cache->max_seq)) return -1;
    float *x = (float *)malloc(4 * (size_t)S * D), *xn = (float *)malloc(4 * (size_t)S * D);
    if (og_embed(m, ids, S, rope_offset, x)) { free(x), free(xn); return -1; }
    for (int l = 0; l < m->layers; l++) {
        og_attn_residual(m, &m->L[l], x, S, cache, l, 0, 0, rope_offset);
        og_ffn_residual(m, &m->L[l], x, S);
    }
    og_rmsnorm(x, m->norm_final, xn, S, D, m->eps);
    og_matmul(xn, m->lm_head, logits, S, D, m->vocab);
    if (cache) cache->length = S;
    free(x), free(xn);
    return 0;
}

/* Full forward without a cache (the eval path the reference's KvCacheTest compares against,
 * J/model/GPTModel.java:1121-1149): same math as prefill with ropeOffset 0 and no cache writes. */
OG_API int og_forward(const og_model *m, const int *ids, int S, float *logits) {
    return og_forward_prefill(m, ids, S, NULL, 0, logits);
}

/* forwardDecode: J/model/GptKvForward.java:92-170.  -1 = IllegalArgument, -2 = IllegalState
 * (cache.length() != cacheLenBefore, or cache full). logits [V]. */
static int og_forward_decode_rows(const og_model *m, int id, og_cache *cache, int cache_len_before, int rope_position,
                                  int pos_row, float *logits);
OG_API int og_forward_decode(const og_model *m, int id, og_cache *cache, int cache_len_before, int rope_position,
                             float *logits) {
    return og_forward_decode_rows(m, id, cache, cache_len_before, rope_position, rope_position, logits);
}
/* The rolling-window form of the same step: RoPE at the token's absolute position (which may lie beyond the context),
 * position-table row = position mod maxSeq, so that every token keeps the row it was embedded with for as long as it
 * stays in the window.  Identical to og_forward_decode while rope_position < maxSeq. */
OG_API int og_forward_decode_rolling(const og_model *m, int id, og_cache *cache, int cache_len_before, int rope_position,
                                     float *logits) {
    if (rope_position < 0) return -1;
    return og_forward_decode_rows(m, id, cache, cache_len_before, rope_position, rope_position % m->max_seq, logits);
}
static int og_forward_decode_rows(const og_model *m, int id, og_cache *cache, int cache_len_before, int rope_position,
                                  int pos_row, float *logits) {
    const int D = m->d_model;
    if (cache->length != cache_len_before) return -2;
    if (cache_len_before >= cache->max_seq) return -2;
    float *x = (float *)malloc(4 * (size_t)D), *xn = (float *)malloc(4 * (size_t)D);
    if (og_embed(m, &id, 1, pos_row, x)) { free(x), free(xn); return -1; }
    for (int l = 0; l < m->layers; l++) {
        og_attn_residual(m, &m->L[l], x, 1, cache, l, 1, cache_len_before, rope_position);
        og_ffn_residual(m, &m->L[l], x, 1);
    }
    og_rmsnorm(x, m->norm_final, xn, 1, D, m->eps);
    og_matmul(xn, m->lm_head, logits, 1, D, m->vocab);
    cache->length = cache_len_before + 1;
    free(x), free(xn);
    return 0;
}

/* Greedy argmax, ties -> lowest index: J/model/GptAutoregressiveGenerator.java:288-299. */
OG_API int og_argmax(const float *logits, int n) {
    int best = 0;
    float bv = logits[0];
    for (int i = 1; i < n; i++) {
        const float v = logits[i];
        if (v > bv || (v == bv && i < best)) bv = v, best = i;
    }
    return best;
}

/* sampleNextToken: J/model/GptAutoregressiveGenerator.java:208-286.  The uniform draw is an
 * argument (the reference uses an unseeded ThreadLocalRandom). */
OG_API int og_sample_next_token(const float *logits_in, int V, float temperature, int topK, float u01) {
    float *z = (float *)malloc(4 * (size_t)V);
    memcpy(z, logits_in, 4 * (size_t)V);
    if (temperature != 1.0f && temperature > 0) for (int i = 0; i < V; i++) z[i] /= temperature;
    if (topK > 0 && topK < V) {
        /* keep the topK by (logit desc, index asc) */
        unsigned char *keep = (unsigned char *)calloc(V, 1);
        for (int r = 0; r < topK; r++) {
            int best = -1;
            for (int i = 0; i < V; i++) {
                if (keep[i]) continue;
                if (best < 0 || z[i] > z[best]) best = i; /* first (lowest) index wins ties */
            }
            keep[best] = 1;
        }
        for (int i = 0; i < V; i++) if (!keep[i]) z[i] = -INFINITY;
        free(keep);
    }
    int tok;
    if (temperature <= 0.f) {
        tok = og_argmax(z, V);
    } else {
        float mx = -INFINITY, sum = 0.f, cum = 0.f;
        for (int i = 0; i < V; i++) mx = fmaxf(mx, z[i]);
        for (int i = 0; i < V; i++) { z[i] = (float)exp((double)(z[i] - mx)); sum += z[i]; }
        for (int i = 0; i < V; i++) z[i] /= sum;
        tok = V - 1;
        for (int i = 0; i < V; i++) { cum += z[i]; if (u01 <= cum) { tok = i; break; } }
    }
    free(z);
    return tok;
}

/* Greedy generation loop: J/model/GptAutoregressiveGenerator.java:20-106.  out has S+maxNew ints,
 * prompt copied, tail left 0 after an early stop on sampled id 0.  Sliding window re-prefill of
 * out[cur-maxSeq : maxSeq) with ropeOffset = cur-maxSeq (:51-88).  Returns the number of sampled
 * tokens, -1 IllegalArgument, -2 IllegalState (window empty).  If logits_trace is non-NULL it
 * receives the V logits each sampled token was drawn from (maxNew rows). */
OG_API int og_generate_greedy(const og_model *m, const int *prompt, int S, int max_new, int kv_fp16, int *out,
                              float *logits_trace) {
    const int V = m->vocab, Dh = m->d_model / m->heads;
    for (int i = 0; i < S + max_new; i++) out[i] = (i < S) ? prompt[i] : 0;
    if (max_new <= 0) return 0;
    og_cache *cache = og_cache_create(m->layers, m->heads, Dh, m->max_seq);
    cache->kv_fp16 = kv_fp16;
    float *logits = (float *)malloc(4 * (size_t)(S > m->max_seq ? S : m->max_seq) * V);
    int rc = og_forward_prefill(m, prompt, S, cache, 0, logits);
    if (rc) { og_cache_free(cache), free(logits); return rc; }
    int n = 0;
    const float *row = logits + (size_t)(S - 1) * V;
    int tok = og_argmax(row, V);
    if (logits_trace) memcpy(logits_trace + (size_t)n * V, row, 4 * (size_t)V);
    out[S] = tok, n = 1;
    if (tok != 0) {
        for (int j = 1; j < max_new; j++) {
            const int cur = S + j;
            if (cur > m->max_seq) {
                const int start = cur - m->max_seq, len = m->max_seq - start;
                if (len <= 0) { n = -2; break; }
                og_cache_clear(cache);
                rc = og_forward_prefill(m, out + start, len, cache, start, logits);
                if (rc) { n = rc; break; }
                row = logits + (size_t)(len - 1) * V;
            } else {
                rc = og_forward_decode(m, out[S + j - 1], cache, cache->length, S + j - 1, logits);
                if (rc) { n = rc; break; }
                row = logits;
            }
            tok = og_argmax(row, V);
            if (logits_trace) memcpy(logits_trace + (size_t)n * V, row, 4 * (size_t)V);
            out[cur] = tok, n++;
            if (tok == 0) break;
        }
    }
    og_cache_free(cache), free(logits);
    return n;
}

/* Greedy generation with the block-granular rolling window instead of the reference's clear-and-re-prefill: when the
 * cache is full the oldest `block` tokens are dropped and decoding simply continues (RoPE at absolute positions,
 * position row = position mod maxSeq).  Same outputs as og_generate_greedy until the context first fills. */
OG_API int og_generate_greedy_rolling(const og_model *m, const int *prompt, int S, int max_new, int kv_fp16, int block,
                                      int *out) {
    const int V = m->vocab, Dh = m->d_model / m->heads;
    for (int i = 0; i < S + max_new; i++) out[i] = (i < S) ? prompt[i] : 0;
    if (max_new <= 0) return 0;
    if (block <= 0 || S > m->max_seq) return -1;
    og_cache *cache = og_cache_create(m->layers, m->heads, Dh, m->max_seq);
    cache->kv_fp16 = kv_fp16;
    float *logits = (float *)malloc(4 * (size_t)m->max_seq * V);
    int rc = og_forward_prefill(m, prompt, S, cache, 0, logits);
    if (rc) { og_cache_free(cache), free(logits); return rc; }
    int n = 0, tok = og_argmax(logits + (size_t)(S - 1) * V, V);
    out[S] = tok, n = 1;
    for (int j = 1; j < max_new && tok != 0; j++) {
        if (cache->length >= cache->max_seq && og_cache_drop_front(cache, block)) { n = -2; break; }
        rc = og_forward_decode_rolling(m, out[S + j - 1], cache, cache->length, S + j - 1, logits);
        if (rc) { n = rc; break; }
        tok = og_argmax(logits, V);
        out[S + j] = tok, n++;
    }
    og_cache_free(cache), free(logits);
    return n;
}

/* ------------------------------------------------------------------------------------------
 * Batched append + single-query attention over contiguous per-sequence planes: the attention
 * half of the decode step (TensorOps.java:2239-2309 minus the projections) for n independent
 * sequences.  This is the CPU side of the append + decode-attention microbenchmark.
 *   q,k,v    [n, H*Dh] fp32 (token-major, head h owns columns h*Dh..), q and k before RoPE
 *   kc,vc    n planes of [H, maxSeq, Dh] laid back to back (kc + i*H*maxSeq*Dh)
 *   lens[i]  cacheLenBefore of sequence i;  rope_pos[i]  RoPE position of the new token
 *   out      [n, H*Dh]
 * kv_fp16 != 0 rounds the appended payload through binary16 first.
 * ---------------------------------------------------------------------------------------- */
OG_API void og_decode_attn_batch(const float *q, const float *k, const float *v, float *kc, float *vc,
                                 const int *lens, const int *rope_pos, int n, int H, int Dh, int max_seq,
                                 int kv_fp16, float *out) {
    const float scale = 1.0f / (float)sqrt((double)Dh);
    const size_t plane = (size_t)H * max_seq * Dh;
#pragma omp parallel for schedule(dynamic, 1) collapse(2)
    for (int i = 0; i < n; i++)
        for (int h = 0; h < H; h++) {
            const int len0 = lens[i], p = rope_pos[i];
            float qr[256], kr[256];
            for (int j = 0; j < Dh / 2; j++) {
                float c, s;
                og_rope_cos_sin(p, j, Dh, &c, &s);
                const float *qq = q + (size_t)i * H * Dh + (size_t)h * Dh, *kk = k + (size_t)i * H * Dh + (size_t)h * Dh;
                qr[2 * j] = qq[2 * j] * c - qq[2 * j + 1] * s, qr[2 * j + 1] = qq[2 * j] * s + qq[2 * j + 1] * c;
                kr[2 * j] = kk[2 * j] * c - kk[2 * j + 1] * s, kr[2 * j + 1] = kk[2 * j] * s + kk[2 * j + 1] * c;
            }
            float *kp = kc + i * plane + (size_t)h * max_seq * Dh, *vp = vc + i * plane + (size_t)h * max_seq * Dh;
            for (int d = 0; d < Dh; d++) {
                float kv = kr[d], vv = v[(size_t)i * H * Dh + (size_t)h * Dh + d];
                if (kv_fp16) kv = og_round_fp16(kv), vv = og_round_fp16(vv);
                kp[(size_t)len0 * Dh + d] = kv, vp[(size_t)len0 * Dh + d] = vv;
            }
            float *scr = (float *)malloc(4 * (size_t)(len0 + 1));
            og_attn_query_one(qr, kp, vp, len0 + 1, Dh, scale, out + (size_t)i * H * Dh + (size_t)h * Dh, scr);
            free(scr);
        }
}

OG_API int og_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
OG_API void og_set_num_threads(int n) {
#ifdef _OPENMP
    omp_set_num_threads(n);
#else
    (void)n;
#endif
}
