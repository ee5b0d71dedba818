/* Test-only harness around the REFERENCE's own CUDA kernels (never part of the shipped library).
 *
 * Purpose: the CPU oracle (oracle/jgpt_oracle.c) is a restatement of the reference's arithmetic; this
 * file lets a GPU test check that restatement against the reference's kernels themselves.  It is
 * compiled only where the reference checkout is present, by oracle/Makefile (target `ref`), with
 *     -I <reference>/src/main/cpp  -I oracle/ref_harness
 * so the `#include "jgpt_cuda_extra_kernels_launches.inl"` below pulls the reference's kernel file
 * from where it lies: no reference source is copied into this repository.  The product of the
 * build (oracle/_ref/libjgpt_ref_kernels.so) is git-ignored.
 *
 * What the harness supplies itself, because in the reference they live in translation units that need
 * a JDK: the stream accessors declared by jgpt_cuda_stream.cuh (here: one non-blocking stream, as the
 * reference creates) and the small `static` workspace helpers that jgpt_cuda_extra.cu defines before
 * including the kernel file (here: plain grow-only cudaMalloc buffers).  The JNI header is the
 * stand-in under oracle/ref_harness/jni.h; no JNI function is ever called.
 *
 * Every wrapper takes HOST pointers, copies in, runs the reference kernel or launch helper with the
 * launch shape the reference's JNI call sites use (threads = min(256, max threads per block),
 * blocks = ceil(total / threads)), copies out and synchronises.  Return value: 0 ok, non-zero CUDA
 * error code or -1 when a reference helper reported failure.
 */
#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <cublas_v2.h>
#include <jni.h>
#include <math.h>
#include <stdio.h>
#include <stdlib.h>
#include <cstdint>
#include <algorithm>
#include <climits>
#include <cstring>
#include <cstddef>
#include <mutex>

#include "jgpt_cuda_stream.cuh"
#include "jgpt_cuda_cublas_common.cuh"
#include "jgpt_cuda_extra_thread_resources.cuh"
#include "jgpt_cuda_graph_prewarm.h"
#include "jgpt_cuda_size_check.cuh"

// ---- what jgpt_cuda.cu provides in the reference build ---------------------------------------------
static cudaStream_t g_harness_stream = nullptr;
static std::mutex g_harness_mu;

extern "C" cudaStream_t jgpt_cuda_stream_handle(void) { return g_harness_stream; }
extern "C" void jgpt_cuda_ensure_stream(void) {
    std::lock_guard<std::mutex> lock(g_harness_mu);
    if (g_harness_stream == nullptr) cudaStreamCreateWithFlags(&g_harness_stream, cudaStreamNonBlocking);
}
extern "C" int jgpt_cuda_sync_stream_unless_capturing(const char* ctx) {
    cudaError_t e = cudaStreamSynchronize(g_harness_stream);
    if (e != cudaSuccess) {
        fprintf(stderr, "%s: %s\n", ctx ? ctx : "sync", cudaGetErrorString(e));
        return 0;
    }
    return 1;
}
extern "C" int jgpt_cuda_max_threads_per_block(void) {
    int v = 1024;
    cudaDeviceGetAttribute(&v, cudaDevAttrMaxThreadsPerBlock, 0);
    return v;
}
extern "C" int jgpt_cuda_get_optimal_block_size(void) { return std::min(256, jgpt_cuda_max_threads_per_block()); }

// ---- what jgpt_cuda_extra.cu defines before including the kernel file ---------------------------------
namespace jgpt_extra {
ExtraThreadResources& jgpt_extra_tls() {
    thread_local ExtraThreadResources tr;
    return tr;
}
}  // namespace jgpt_extra

static cublasHandle_t get_extra_cublas_handle() { return jgpt_cuda_detail::get_cublas_handle(); }

struct GrowBuf {
    void* p = nullptr;
    size_t n = 0;
    bool ensure(size_t bytes) {
        if (bytes <= n) return true;
        if (p) cudaFree(p);
        p = nullptr;
        n = 0;
        if (cudaMalloc(&p, bytes) != cudaSuccess) return false;
        n = bytes;
        return true;
    }
};
static GrowBuf g_ws_a, g_ws_b, g_ws_c;

static void ce_async_host_free() {}
static void ce_async_host_ensure() {}
static void ce_pinned_flt_targets_free() {}
static void ce_pinned_flt_targets_ensure(size_t) {}
static void ce_free_cached() {}
static bool ce_ensure_logits_grad_buffers(size_t) { return false; }
static bool softmax_pair_ensure(size_t bytes_per, float** d_src, float** d_dst) {
    if (!g_ws_a.ensure(bytes_per) || !g_ws_b.ensure(bytes_per)) return false;
    *d_src = (float*) g_ws_a.p;
    *d_dst = (float*) g_ws_b.p;
    return true;
}
static void softmax_pair_free_cached() {}
static bool adamw_pool_ensure(size_t) { return false; }
static void adamw_pool_free_cached() {}
static bool attn_bwd_host_ensure(size_t, size_t, size_t, float**, float**, float**, float**, float**, float**, float**,
                                 float**, float**, float**) {
    return false;
}
static void attn_bwd_host_free_cached() {}
static bool attn_bwd_aux_ensure(size_t, size_t, float**, float**) { return false; }
static void attn_bwd_aux_free_cached() {}
static bool attn_fwd_aux_ensure(size_t bytesQK, size_t bytesProb, size_t bytesMask, bool with_mask, float** d_scores,
                                float** d_probs, float** d_mask) {
    (void) bytesQK;
    if (!g_ws_a.ensure(bytesProb) || !g_ws_b.ensure(bytesProb)) return false;
    *d_scores = (float*) g_ws_a.p;
    *d_probs = (float*) g_ws_b.p;
    if (with_mask) {
        if (!g_ws_c.ensure(bytesMask)) return false;
        *d_mask = (float*) g_ws_c.p;
    } else if (d_mask) {
        *d_mask = nullptr;
    }
    return true;
}
static bool fa_ensure_D(size_t) { return false; }

#include "jgpt_cuda_extra_kernels_launches.inl"

// silence "defined but not used" for helpers only the JNI files of the reference call
static void* const g_unused_refs[] __attribute__((unused)) = {
        (void*) ce_async_host_free, (void*) ce_async_host_ensure, (void*) ce_pinned_flt_targets_free,
        (void*) ce_pinned_flt_targets_ensure, (void*) ce_free_cached, (void*) ce_ensure_logits_grad_buffers,
        (void*) softmax_pair_ensure, (void*) softmax_pair_free_cached, (void*) adamw_pool_ensure,
        (void*) adamw_pool_free_cached, (void*) attn_bwd_host_ensure, (void*) attn_bwd_host_free_cached,
        (void*) attn_bwd_aux_ensure, (void*) attn_bwd_aux_free_cached, (void*) attn_fwd_aux_ensure, (void*) fa_ensure_D};

// ---- the wrappers ---------------------------------------------------------------------------------------
#define REF_EXPORT extern "C" __attribute__((visibility("default")))
#define REF_TRY(call)                           \
    do {                                        \
        cudaError_t e__ = (call);               \
        if (e__ != cudaSuccess) return (int) e__; \
    } while (0)

namespace {
struct DevBuf {
    void* p = nullptr;
    ~DevBuf() {
        if (p) cudaFree(p);
    }
    cudaError_t alloc(size_t bytes) { return cudaMalloc(&p, bytes ? bytes : 4); }
    // Copies go on the harness stream, in front of / behind the kernels they feed: that stream is non-blocking, so a
    // plain cudaMemcpy from pageable memory (which may return before its DMA has landed) would not be ordered with it.
    cudaError_t up(const void* h, size_t bytes) {
        cudaError_t e = alloc(bytes);
        if (e != cudaSuccess || !bytes) return e;
        e = cudaMemcpyAsync(p, h, bytes, cudaMemcpyHostToDevice, jgpt_cuda_stream_handle());
        return e != cudaSuccess ? e : cudaStreamSynchronize(jgpt_cuda_stream_handle());
    }
    cudaError_t down(void* h, size_t bytes) const {
        if (!bytes) return cudaSuccess;
        cudaError_t e = cudaMemcpyAsync(h, p, bytes, cudaMemcpyDeviceToHost, jgpt_cuda_stream_handle());
        return e != cudaSuccess ? e : cudaStreamSynchronize(jgpt_cuda_stream_handle());
    }
    template <class T>
    T* as() const { return (T*) p; }
};
int blocks_for(long long total, int threads) { return (int) ((total + threads - 1) / threads); }
int finish() {
    REF_TRY(cudaGetLastError());
    REF_TRY(cudaStreamSynchronize(jgpt_cuda_stream_handle()));
    return 0;
}
}  // namespace

REF_EXPORT int ref_device_count(void) {
    int n = 0;
    return cudaGetDeviceCount(&n) == cudaSuccess ? n : 0;
}

/* rope_4d_kernel: src/dst [batch, heads, seq, dhead]; positions may be NULL (then i + pos_base). */
REF_EXPORT int ref_rope_4d(const float* src, float* dst, int batch, int heads, int seq, int dhead, const int* positions,
                           int pos_len, int pos_base) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) batch * heads * seq * dhead;
    DevBuf s, d, p;
    REF_TRY(s.up(src, n * 4));
    REF_TRY(d.alloc(n * 4));
    if (positions) REF_TRY(p.up(positions, (size_t) pos_len * 4));
    long long total = (long long) batch * heads * seq * (dhead / 2);
    int threads = jgpt_cuda_get_optimal_block_size();
    rope_4d_kernel<<<blocks_for(total, threads), threads, 0, kTensorCudaStream>>>(
            s.as<float>(), d.as<float>(), batch, heads, seq, dhead, positions ? p.as<int>() : nullptr, pos_len, pos_base);
    if (int r = finish()) return r;
    REF_TRY(d.down(dst, n * 4));
    return 0;
}

/* kv_heads4d_to_cache_kernel: src [heads, seq, dhead] -> cache [heads, max_seq, dhead] at rows [0, seq) of
 * (cache + pos_offset*dhead), the way copyKvHeads4dToCacheGPUDevice offsets the destination. */
REF_EXPORT int ref_kv_heads4d_to_cache(const float* src, float* cache, int heads, int seq, int max_seq, int dhead,
                                       int pos_offset) {
    jgpt_cuda_ensure_stream();
    size_t ns = (size_t) heads * seq * dhead, nc = (size_t) heads * max_seq * dhead;
    if (pos_offset < 0 || pos_offset + seq > max_seq) return -2;
    DevBuf s, c;
    REF_TRY(s.up(src, ns * 4));
    REF_TRY(c.up(cache, nc * 4));
    int threads = jgpt_cuda_get_optimal_block_size();
    kv_heads4d_to_cache_kernel<<<blocks_for((long long) ns, threads), threads, 0, kTensorCudaStream>>>(
            s.as<float>(), c.as<float>() + (size_t) pos_offset * dhead, heads, seq, max_seq, dhead);
    if (int r = finish()) return r;
    REF_TRY(c.down(cache, nc * 4));
    return 0;
}

/* launch_softmax_last_dim: thread-per-row below 64 columns, block-per-row from 64. */
REF_EXPORT int ref_softmax_last_dim(const float* src, float* dst, long long nrows, int inner, int use_fp16_branch) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) nrows * inner;
    DevBuf s, d;
    REF_TRY(s.up(src, n * 4));
    REF_TRY(d.alloc(n * 4));
    launch_softmax_last_dim(s.as<float>(), d.as<float>(), nrows, inner, use_fp16_branch != 0);
    if (int r = finish()) return r;
    REF_TRY(d.down(dst, n * 4));
    return 0;
}

/* launch_softmax_scaled_masked_block_chunked: rows = batch*seq of length seq, mask [seq, seq] or NULL. */
REF_EXPORT int ref_softmax_scaled_masked(const float* scores, float* probs, const float* mask, float scale,
                                         long long nrows, int inner) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) nrows * inner;
    DevBuf s, d, m;
    REF_TRY(s.up(scores, n * 4));
    REF_TRY(d.alloc(n * 4));
    if (mask) REF_TRY(m.up(mask, (size_t) inner * inner * 4));
    size_t smem = ((size_t) kSoftmaxSharedPrefixFloats + (size_t) inner) * sizeof(float);
    if (smem > 48u * 1024u) return -3;  // the reference raises no shared-memory limit for this kernel
    if (!launch_softmax_scaled_masked_block_chunked(s.as<float>(), d.as<float>(), mask ? m.as<float>() : nullptr, scale,
                                                    nrows, inner, kTensorCudaStream))
        return -1;
    if (int r = finish()) return r;
    REF_TRY(d.down(probs, n * 4));
    return 0;
}

/* launch_rms_norm_fwd */
REF_EXPORT int ref_rms_norm(const float* src, const float* gamma, float* dst, int outer, int last_dim, float eps) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) outer * last_dim;
    DevBuf s, g, d;
    REF_TRY(s.up(src, n * 4));
    REF_TRY(g.up(gamma, (size_t) last_dim * 4));
    REF_TRY(d.alloc(n * 4));
    launch_rms_norm_fwd(s.as<float>(), g.as<float>(), d.as<float>(), outer, last_dim, eps);
    if (int r = finish()) return r;
    REF_TRY(d.down(dst, n * 4));
    return 0;
}

REF_EXPORT int ref_sigmoid(const float* src, float* dst, int n) {
    jgpt_cuda_ensure_stream();
    DevBuf s, d;
    REF_TRY(s.up(src, (size_t) n * 4));
    REF_TRY(d.alloc((size_t) n * 4));
    int threads = jgpt_cuda_get_optimal_block_size();
    sigmoid_kernel<<<blocks_for(n, threads), threads, 0, kTensorCudaStream>>>(s.as<float>(), d.as<float>(), n);
    if (int r = finish()) return r;
    REF_TRY(d.down(dst, (size_t) n * 4));
    return 0;
}

REF_EXPORT int ref_mul(const float* a, const float* b, float* c, int n) {
    jgpt_cuda_ensure_stream();
    DevBuf da, db, dc;
    REF_TRY(da.up(a, (size_t) n * 4));
    REF_TRY(db.up(b, (size_t) n * 4));
    REF_TRY(dc.alloc((size_t) n * 4));
    int threads = jgpt_cuda_get_optimal_block_size();
    mul_kernel<<<blocks_for(n, threads), threads, 0, kTensorCudaStream>>>(da.as<float>(), db.as<float>(), dc.as<float>(), n);
    if (int r = finish()) return r;
    REF_TRY(dc.down(c, (size_t) n * 4));
    return 0;
}

/* embedding_token_fwd_kernel then add_position_embedding_broadcast_kernel: x = tok[id] + pos[pos_row_start + s]. */
REF_EXPORT int ref_embed_pos(const float* tokens_as_float, const float* tok_table, const float* pos_table, float* out,
                             int batch, int seq, int d_model, int vocab, int pos_rows, int pos_row_start) {
    jgpt_cuda_ensure_stream();
    if (pos_row_start < 0 || pos_row_start + seq > pos_rows) return -2;
    size_t n = (size_t) batch * seq * d_model;
    DevBuf t, w, p, o;
    REF_TRY(t.up(tokens_as_float, (size_t) batch * seq * 4));
    REF_TRY(w.up(tok_table, (size_t) vocab * d_model * 4));
    REF_TRY(p.up(pos_table, (size_t) pos_rows * d_model * 4));
    REF_TRY(o.alloc(n * 4));
    int threads = jgpt_cuda_get_optimal_block_size();
    embedding_token_fwd_kernel<<<blocks_for((long long) n, threads), threads, 0, kTensorCudaStream>>>(
            t.as<float>(), w.as<float>(), o.as<float>(), batch, seq, d_model, vocab);
    add_position_embedding_broadcast_kernel<<<blocks_for((long long) n, threads), threads, 0, kTensorCudaStream>>>(
            o.as<float>(), p.as<float>(), pos_row_start, batch, seq, d_model);
    if (int r = finish()) return r;
    REF_TRY(o.down(out, n * 4));
    return 0;
}

/* split_heads_kernel [batch, seq, d_model] -> [batch, heads, seq, dhead]; concat_heads_kernel is the inverse. */
REF_EXPORT int ref_split_heads(const float* src, float* dst, int batch, int seq, int d_model, int heads) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) batch * seq * d_model;
    DevBuf s, d;
    REF_TRY(s.up(src, n * 4));
    REF_TRY(d.alloc(n * 4));
    int threads = jgpt_cuda_get_optimal_block_size();
    split_heads_kernel<<<blocks_for((long long) n, threads), threads, 0, kTensorCudaStream>>>(s.as<float>(), d.as<float>(), batch,
                                                                                             seq, d_model, heads);
    if (int r = finish()) return r;
    REF_TRY(d.down(dst, n * 4));
    return 0;
}
REF_EXPORT int ref_concat_heads(const float* src, float* dst, int batch, int heads, int seq, int dhead) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) batch * seq * heads * dhead;
    DevBuf s, d;
    REF_TRY(s.up(src, n * 4));
    REF_TRY(d.alloc(n * 4));
    int threads = jgpt_cuda_get_optimal_block_size();
    concat_heads_kernel<<<blocks_for((long long) n, threads), threads, 0, kTensorCudaStream>>>(s.as<float>(), d.as<float>(), batch,
                                                                                              heads, seq, dhead);
    if (int r = finish()) return r;
    REF_TRY(d.down(dst, n * 4));
    return 0;
}

/* flash_attn_fwd_run: causal, Q/K/V/O [BH, S, 16] fp32, LSE [BH, S]. */
REF_EXPORT int ref_flash_attn_fwd(const float* q, const float* k, const float* v, float* o, float* lse, int BH, int S,
                                  float scale) {
    jgpt_cuda_ensure_stream();
    size_t n = (size_t) BH * S * kFaDh;
    DevBuf dq, dk, dv, dout, dl;
    REF_TRY(dq.up(q, n * 4));
    REF_TRY(dk.up(k, n * 4));
    REF_TRY(dv.up(v, n * 4));
    REF_TRY(dout.alloc(n * 4));
    REF_TRY(dl.alloc((size_t) BH * S * 4));
    if (!flash_attn_fwd_run(dq.as<float>(), dk.as<float>(), dv.as<float>(), dout.as<float>(), dl.as<float>(), BH, S, scale))
        return -1;
    if (int r = finish()) return r;
    REF_TRY(dout.down(o, n * 4));
    REF_TRY(dl.down(lse, (size_t) BH * S * 4));
    return 0;
}

/* attn_fwd_run_core: scores = Q.K^T (cuBLAS, TF32 math mode as the reference sets it), fused
 * scale + mask + softmax, out = P.V.  q,k [batch, seq, dk]; v, out [batch, seq, dv]; mask [seq, seq] or NULL. */
REF_EXPORT int ref_attn_fwd_core(const float* q, const float* k, const float* v, const float* mask, float* out, float* probs,
                                 int batch, int seq, int dk, int dv, float scale) {
    jgpt_cuda_ensure_stream();
    size_t nqk = (size_t) batch * seq * dk, nv = (size_t) batch * seq * dv, np = (size_t) batch * seq * seq;
    size_t smem = ((size_t) kSoftmaxSharedPrefixFloats + (size_t) seq) * sizeof(float);
    if (smem > 48u * 1024u) return -3;
    DevBuf dq, dk_, dv_, dm, dsc, dpr, dout;
    REF_TRY(dq.up(q, nqk * 4));
    REF_TRY(dk_.up(k, nqk * 4));
    REF_TRY(dv_.up(v, nv * 4));
    if (mask) REF_TRY(dm.up(mask, (size_t) seq * seq * 4));
    REF_TRY(dsc.alloc(np * 4));
    REF_TRY(dpr.alloc(np * 4));
    REF_TRY(dout.alloc(nv * 4));
    if (!attn_fwd_run_core(dq.as<float>(), dk_.as<float>(), dv_.as<float>(), dsc.as<float>(), dpr.as<float>(), dout.as<float>(),
                           mask ? dm.as<float>() : nullptr, batch, seq, dk, dv, scale, false))
        return -1;
    if (int r = finish()) return r;
    REF_TRY(dout.down(out, nv * 4));
    if (probs) REF_TRY(dpr.down(probs, np * 4));
    return 0;
}

/* batched_sgemm_row_major_extra: C[M,N] = A[M,K].B[K,N] per batch (cuBLAS, TF32 math mode). */
REF_EXPORT int ref_matmul_row_major(const float* a, const float* b, float* c, int batch, int M, int K, int N) {
    jgpt_cuda_ensure_stream();
    DevBuf da, db, dc;
    REF_TRY(da.up(a, (size_t) batch * M * K * 4));
    REF_TRY(db.up(b, (size_t) batch * K * N * 4));
    REF_TRY(dc.alloc((size_t) batch * M * N * 4));
    if (!batched_sgemm_row_major_extra(da.as<float>(), db.as<float>(), dc.as<float>(), batch, M, K, N, 1.0f, 0.0f)) return -1;
    if (int r = finish()) return r;
    REF_TRY(dc.down(c, (size_t) batch * M * N * 4));
    return 0;
}
