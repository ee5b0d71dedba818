/*
 * jgpt_b200 — C ABI of the B200-native KV-cache decode path for JGPT.
 *
 * Plain C: extern "C", POD arguments, opaque 64-bit handles, int32 status codes.  No PyTorch,
 * no JNI types.  A JNI shim or a Java FFM (java.lang.foreign) downcall binds these symbols
 * one to one.  Every entry point names the reference interface it replaces; paths are relative
 * to the reference project root, J = src/main/java/com/veles/llm/jgpt, C = src/main/cpp.
 *
 * Conventions
 *   - Every function returns a status (0 = JGPT_OK).  jgpt_last_error() returns the message of
 *     the last failing call on the calling thread.  The Java side maps JGPT_ERR_INVALID_ARGUMENT
 *     to IllegalArgumentException, JGPT_ERR_ILLEGAL_STATE to IllegalStateException,
 *     JGPT_ERR_OUT_OF_RANGE to IndexOutOfBoundsException, JGPT_ERR_OUT_OF_MEMORY to OutOfMemoryError,
 *     i.e. the classes the reference throws for the same misuse.
 *   - One CUDA stream per context.  Calls on one context are stream ordered and must come from
 *     one thread at a time (the reference is single threaded per model/cache as well:
 *     J/model/KvCache.java:11).  Functions that write HOST memory synchronise before returning;
 *     all others are asynchronous until jgpt_sync().
 *   - "dev" pointers are device addresses on the context's GPU; "host" pointers are ordinary
 *     host memory.  fp32 activations are row major, token major: [n_tokens, heads*dhead], head h
 *     owning columns [h*dhead, (h+1)*dhead) — the layout the projections x.W produce, so the
 *     reference's split_heads / concat_heads transposes disappear.
 *   - There is no CPU fallback: without a usable GPU jgpt_ctx_create fails.
 */
#ifndef JGPT_B200_H
#define JGPT_B200_H

#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define JGPT_API __attribute__((visibility("default")))

typedef uint64_t jgpt_ctx;    /* one GPU + one stream                    */
typedef uint64_t jgpt_kvpool; /* paged fp16 K/V store of one model       */
typedef uint64_t jgpt_model;  /* device-resident weights + step workspace */


enum {
    JGPT_OK = 0,
    JGPT_ERR_INVALID_ARGUMENT = 1, /* IllegalArgumentException   */
    JGPT_ERR_ILLEGAL_STATE = 2,    /* IllegalStateException      */
    JGPT_ERR_OUT_OF_RANGE = 3,     /* IndexOutOfBoundsException  */
    JGPT_ERR_OUT_OF_MEMORY = 4,    /* OutOfMemoryError (device)  */
    JGPT_ERR_POOL_EXHAUSTED = 5,   /* no free KV block / sequence slot */
    JGPT_ERR_BAD_HANDLE = 6,
    JGPT_ERR_CUDA = 7,
    JGPT_ERR_UNSUPPORTED = 8,      /* the reference returns null / throws ISE for unsupported shapes */
    JGPT_ERR_DEVICE_CHECK = 9,     /* a kernel reported a failed self-check or a timed-out wait */
    JGPT_ERR_IO = 10,
    JGPT_ERR_NCCL = 11,            /* the collective library reported an error (or is missing) */
    JGPT_ERR_TIMEOUT = 12          /* a bounded host-side wait ran out; nothing blocks for ever */
};

/* ---------------------------------------------------------------------------------------------
 * Runtime: context, stream, device buffers
 * ------------------------------------------------------------------------------------------- */

/* Replaces TensorOpsGPU.initGPU / isGpuAvailable / requireCuda (J/TensorOpsGPU.java:87-132,
 * 1197-1203; native C/jgpt_cuda_jni_ops_graph.inl:97-107) and the process-global stream of
 * C/jgpt_cuda_runtime.inl:234-250.  `device` selects the GPU (the reference hard-codes 0). */
JGPT_API int32_t jgpt_ctx_create(int32_t device, jgpt_ctx *out);
JGPT_API int32_t jgpt_ctx_destroy(jgpt_ctx ctx);
/* TensorOpsGPU.synchronizeStream (C/jgpt_cuda_jni_ops_graph.inl:123-176).  Also reads the
 * device status word and returns JGPT_ERR_DEVICE_CHECK if a kernel recorded a failure. */
JGPT_API int32_t jgpt_sync(jgpt_ctx ctx);
JGPT_API const char *jgpt_last_error(void);
/* cudaStream_t of the context, for callers that enqueue their own work or time with events. */
JGPT_API int32_t jgpt_ctx_stream(jgpt_ctx ctx, void **stream_out);
JGPT_API int32_t jgpt_device_count(int32_t *out);
/* PCI address of a device, lower case ("0000:1b:00.0"), for hosts that bind a rank's thread and page-locked
 * buffers to the GPU's NUMA node (/sys/bus/pci/devices/<id>/numa_node).  No reference counterpart (one GPU). */
JGPT_API int32_t jgpt_device_pci_bus_id(int32_t device, char *out, int32_t cap);
/* The JGPT_* environment settings that reach this path, parsed with the reference's rules
 * (J/TensorOpsGpuInit.java:30-101: JGPT_RMSNORM_EPS in (0, 1e-2], default 1e-5 with JGPT_FP16_MATMUL else
 * 1e-6; J/training/LLMConfig.java:190-199: JGPT_MAX_SEQ_LEN positive, 0 here = not set) plus this
 * library's own: JGPT_KV_BLOCK_TOKENS (16), JGPT_KV_POOL_BLOCKS (0 = not set), JGPT_KV_BACKEND
 * (unset or "b200" -> 1; anything else -> 0: the host keeps the reference's own KV path).
 * Needs no GPU.  Any output pointer may be NULL. */
JGPT_API int32_t jgpt_env_config(int32_t *kv_block_tokens_out, int32_t *kv_pool_blocks_out,
                                 int32_t *max_seq_len_out, float *rmsnorm_eps_out, int32_t *backend_b200_out);

/* GpuFloatBuffer.allocate / close / copyFrom / copyTo / clear (J/GpuFloatBuffer.java:46-130,
 * natives C/jgpt_cuda_jni_buffers.inl:185-487).  jgpt_d2h synchronises before returning. */
JGPT_API int32_t jgpt_dev_alloc(jgpt_ctx ctx, uint64_t bytes, void **dev_out);
JGPT_API int32_t jgpt_dev_free(jgpt_ctx ctx, void *dev);
JGPT_API int32_t jgpt_h2d(jgpt_ctx ctx, void *dev_dst, const void *host_src, uint64_t bytes);
JGPT_API int32_t jgpt_d2h(jgpt_ctx ctx, void *host_dst, const void *dev_src, uint64_t bytes);
JGPT_API int32_t jgpt_dev_memset(jgpt_ctx ctx, void *dev, int32_t byte_value, uint64_t bytes);
/* TensorOpsGPU.getGpuMemoryAllocated0 / getGpuMemoryReserved0 (C/jgpt_cuda_jni_ops_graph.inl:471-491):
 * free and total bytes of the context's device (cudaMemGetInfo); allocated = total - free. */
JGPT_API int32_t jgpt_mem_info(jgpt_ctx ctx, uint64_t *free_bytes_out, uint64_t *total_bytes_out);
/* cuda.CudaPinnedHost (C/jgpt_cuda_jni_ops_graph.inl:494-519). */
JGPT_API int32_t jgpt_host_alloc_pinned(uint64_t bytes, void **host_out);
JGPT_API int32_t jgpt_host_free_pinned(void *host);

/* Device-side timing on the context's stream (the reference has no equivalent; benchmarks use it). */
JGPT_API int32_t jgpt_event_create(uint64_t *event_out);
JGPT_API int32_t jgpt_event_destroy(uint64_t event);
JGPT_API int32_t jgpt_event_record(jgpt_ctx ctx, uint64_t event);
JGPT_API int32_t jgpt_event_elapsed_ms(uint64_t start, uint64_t stop, float *ms_out); /* syncs on stop */

/* CUDA graphs on the context's stream.  Replaces TensorOpsGPU.cudaStreamBeginCapture0 /
 * cudaStreamEndCaptureAndInstantiate0 / cudaGraphExecLaunch0 / cudaGraphExecDestroy0
 * (J/TensorOpsGPU.java:1023-1054, C/jgpt_cuda_jni_ops_graph.inl:185-460).  Everything enqueued on the
 * context between begin and end is recorded instead of run; calls that synchronise or allocate
 * (host-buffer entry points, first-use scratch growth) must not be made while capturing. */
JGPT_API int32_t jgpt_graph_begin_capture(jgpt_ctx ctx);
JGPT_API int32_t jgpt_graph_end_capture(jgpt_ctx ctx, uint64_t *graph_exec_out);
JGPT_API int32_t jgpt_graph_launch(jgpt_ctx ctx, uint64_t graph_exec);
JGPT_API int32_t jgpt_graph_destroy(uint64_t graph_exec);

/* ---------------------------------------------------------------------------------------------
 * Paged KV store.  Replaces KvCache / KvCacheGpu (J/model/KvCache.java:13-105,
 * J/model/KvCacheGpu.java:12-118): instead of one contiguous fp32 [heads, maxSeq, dhead] buffer
 * per layer and sequence, fp16 K/V live in fixed blocks of `block_tokens` tokens per layer and
 * head; a per-sequence block table maps logical block -> physical block.  A "sequence" is one
 * KvCacheGpu instance of the reference.
 *
 * HBM layout: kv[layer][physical block][head][K: block_tokens x dhead | V: block_tokens x dhead]
 * (fp16).  K is stored after RoPE, V raw (J/model/KvCache.java:8).
 * ------------------------------------------------------------------------------------------- */

/* KvCacheGpu(numLayers, numHeads, dHead, maxSeqLen) (J/model/KvCacheGpu.java:24-45): rejects
 * non-positive dimensions with JGPT_ERR_INVALID_ARGUMENT.  dhead in {4,8,16,32}; block_tokens
 * must be 16.  max_positions bounds the RoPE table (positions 0..max_positions-1). */
JGPT_API int32_t jgpt_kvpool_create(jgpt_ctx ctx, int32_t layers, int32_t heads, int32_t dhead,
                                    int32_t block_tokens, int32_t n_blocks, int32_t max_seqs,
                                    int32_t max_blocks_per_seq, int32_t max_positions, float rope_base,
                                    jgpt_kvpool *out);
JGPT_API int32_t jgpt_kvpool_destroy(jgpt_kvpool pool); /* KvCacheGpu.close() */
JGPT_API int32_t jgpt_kvpool_free_blocks(jgpt_kvpool pool, int32_t *n_free_out);
/* Device address and byte size of the K/V storage (tests poison / inspect it). */
JGPT_API int32_t jgpt_kvpool_storage(jgpt_kvpool pool, void **dev_out, uint64_t *bytes_out);
/* Launch tuning of the decode-attention kernel for this pool (the values JGPT_B200_CHUNK_BLOCKS / _STAGES /
 * _HEAD_GROUP / _PERSISTENT / _LAUNCH_OVERLAP give at creation): KV blocks per split-K chunk (0 = automatic,
 * <= 32), copy-ring stages (2..8), heads per CTA (0 = automatic, else a divisor of heads), persistent (<= 0: one
 * CTA per work item; k > 0: k CTAs per SM claiming items from a queue), and launch_overlap: 0 = ordinary launches;
 * 1 = programmatic dependent launch, the kernel starts while the previous kernel on the stream drains but reads
 * nothing before that kernel has finished; 2 = additionally the copy warp fetches lengths, block-table entries and
 * the first K/V slabs early -- ONLY for callers whose previous kernel on the stream does not write the K/V of the
 * launch's layers, the block tables or the index arrays (true for a per-layer decode loop: the predecessor is a
 * projection or another layer's attention).  Results do not depend on any of them. */
JGPT_API int32_t jgpt_kvpool_set_tuning(jgpt_kvpool pool, int32_t chunk_blocks, int32_t stages, int32_t head_group,
                                        int32_t persistent, int32_t launch_overlap);
/* Device mirror of the block tables, int32 [max_seqs][row_stride], -1 = unmapped (read-only for
 * callers' own kernels; tests corrupt an entry to exercise the kernels' self-checks). */
JGPT_API int32_t jgpt_kvpool_table_device(jgpt_kvpool pool, int32_t **dev_out, int32_t *row_stride_out);

/* Sequence lifecycle: `new KvCacheGpu(..)` / close(); length(), setLength(), clear()
 * (J/model/KvCacheGpu.java:60-101).  seq ids are small ints (lowest free slot first). */
JGPT_API int32_t jgpt_seq_alloc(jgpt_kvpool pool, int32_t *seq_out);
JGPT_API int32_t jgpt_seq_free(jgpt_kvpool pool, int32_t seq);
/* Make sure blocks exist for token positions [0, n_tokens): all or nothing,
 * JGPT_ERR_POOL_EXHAUSTED when the free list is too short, JGPT_ERR_INVALID_ARGUMENT when
 * n_tokens exceeds max_blocks_per_seq*block_tokens. */
JGPT_API int32_t jgpt_seq_reserve(jgpt_kvpool pool, int32_t seq, int32_t n_tokens);
JGPT_API int32_t jgpt_seq_length(jgpt_kvpool pool, int32_t seq, int32_t *len_out);
/* setLength: JGPT_ERR_INVALID_ARGUMENT unless 0 <= len <= reserved capacity. */
JGPT_API int32_t jgpt_seq_set_length(jgpt_kvpool pool, int32_t seq, int32_t len);
/* clear(): length 0, blocks returned to the pool and (zero_fill != 0) scrubbed by the eviction kernel. */
JGPT_API int32_t jgpt_seq_clear(jgpt_kvpool pool, int32_t seq, int32_t zero_fill);
/* Block-granular rolling window.  No counterpart in the reference, which clears the cache and re-prefills the
 * window when the context is full (J/model/GptAutoregressiveGenerator.java:51-88, O(window^2) per overflow).
 * Forgets the oldest n_blocks KV blocks of the sequence: they return to the free list, the block table shifts
 * left and the length drops by 16 * n_blocks; no K/V byte moves.  Cached keys keep the RoPE of their absolute
 * positions.  JGPT_ERR_INVALID_ARGUMENT unless the sequence holds at least that many full blocks. */
JGPT_API int32_t jgpt_seq_drop_front(jgpt_kvpool pool, int32_t seq, int32_t n_blocks, int32_t zero_fill);
/* Install an explicit block table (benchmark: seeded permutation of the pool).  The blocks must be free. */
JGPT_API int32_t jgpt_seq_set_block_table(jgpt_kvpool pool, int32_t seq, const int32_t *blocks_host, int32_t n);
/* Copy the sequence's block table out (bit-exact checks against the allocator specification). */
JGPT_API int32_t jgpt_block_table_copy_out(jgpt_kvpool pool, int32_t seq, int32_t *blocks_host, int32_t cap,
                                           int32_t *n_out);
/* Same, read back from the DEVICE mirror the kernels use. */
JGPT_API int32_t jgpt_block_table_copy_out_device(jgpt_kvpool pool, int32_t seq, int32_t *blocks_host,
                                                  int32_t cap, int32_t *n_out);
/* LRU eviction: frees whole sequences marked evictable (finished), least recently used first
 * (ties: lower seq id), until `need_free` blocks are free.  Victim ids are written to
 * victims_host.  zero_fill != 0 scrubs the freed blocks on the device (eviction kernel). */
JGPT_API int32_t jgpt_seq_mark_evictable(jgpt_kvpool pool, int32_t seq, int32_t evictable);
JGPT_API int32_t jgpt_kv_evict_lru(jgpt_kvpool pool, int32_t need_free, int32_t zero_fill, int32_t *victims_host,
                                   int32_t cap, int32_t *n_victims_out);

/* Append kernel.  Replaces rope_4d_kernel + kv_heads4d_to_cache_kernel
 * (C/jgpt_cuda_extra_kernels_launches.inl:1127-1159, 1085-1099; TensorOps.copyKvHeadsIntoCache /
 * copyKvOneTokenIntoCache, J/ops/TensorOps.java:2446-2557).  For token t in [0,n):
 *   K row = RoPE(k_dev[t], rope_pos[t]) -> fp16 -> block_table[seq_ids[t]][slot_pos[t]/16], slot slot_pos[t]%16
 *   V row = v_dev[t] -> fp16, same place.
 * k_dev, v_dev: fp32 [n, heads*dhead]; seq_ids, slot_pos, rope_pos: int32 [n], all device memory. */
JGPT_API int32_t jgpt_kv_append(jgpt_kvpool pool, int32_t layer, const float *k_dev, const float *v_dev,
                                const int32_t *seq_ids_dev, const int32_t *slot_pos_dev,
                                const int32_t *rope_pos_dev, int32_t n);

/* Gather kernel: paged fp16 -> the reference's contiguous fp32 plane [heads, max_seq_len, dhead]
 * (index h*maxSeq*dhead + pos*dhead + j, J/model/KvCacheGpu.java:7-8), rows >= len zero.
 * Backs KvCacheGpu.getK/getV (J/model/KvCacheGpu.java:47-58) and TensorOps.sliceKvHeadPrefixFromGpu
 * (J/ops/TensorOps.java:2333-2339). */
JGPT_API int32_t jgpt_kv_gather(jgpt_kvpool pool, int32_t layer, int32_t seq, int32_t len, int32_t max_seq_len,
                                float *k_out_dev, float *v_out_dev);
/* The same for n caches in one launch: sequence i's planes at k_out_dev + i * heads * max_seq_len * dhead
 * (a launch per cache moves only a few megabytes and is launch-bound). */
JGPT_API int32_t jgpt_kv_gather_batch(jgpt_kvpool pool, int32_t layer, const int32_t *seq_ids_host,
                                      const int32_t *lens_host, int32_t n, int32_t max_seq_len, float *k_out_dev,
                                      float *v_out_dev);

/* Decode attention.  Replaces the per-head chain of TensorOps.scaledDotProductAttentionQueryOne
 * (J/ops/TensorOps.java:1088-1140) inside multiHeadAttentionWithRoPEDecode (:2239-2309).
 * For i in [0,n): RoPE(q[i]) at rope_pos[i]; softmax(scale * q.K^T) over lens[i] cached keys of
 * sequence seq_ids[i]; out[i] = P.V in the concat-heads layout [n, heads*dhead].
 * q_dev/out_dev hold `n_layers` slabs of [n, heads*dhead] (slab l uses pool layer layer0+l);
 * n_layers = 1 inside the model step, > 1 only when the per-layer queries are independent
 * (the microbenchmark).  max_len is a host-known upper bound of lens[] (sizes the split grid). */
JGPT_API int32_t jgpt_attn_decode(jgpt_kvpool pool, int32_t layer0, int32_t n_layers, const float *q_dev,
                                  const int32_t *seq_ids_dev, const int32_t *rope_pos_dev,
                                  const int32_t *lens_dev, int32_t n, int32_t max_len, float *out_dev);

/* Fused append + decode attention: the whole attention core of one decode step
 * (J/ops/TensorOps.java:2279-2301).  The new token of sequence i is written at slot lens[i]-1
 * (lens = cacheLenBefore + 1) with RoPE at rope_pos[i], and attended together with the cached ones. */
JGPT_API int32_t jgpt_attn_decode_append(jgpt_kvpool pool, int32_t layer0, int32_t n_layers, const float *q_dev,
                                         const float *k_dev, const float *v_dev, const int32_t *seq_ids_dev,
                                         const int32_t *rope_pos_dev, const int32_t *lens_dev, int32_t n,
                                         int32_t max_len, float *out_dev);

/* Host-buffer form of the fused step (what a JNI caller holding float[] uses), synchronous.
 * q, k, v and out in page-locked memory (jgpt_host_alloc_pinned, the reference's CudaPinnedHost):
 * nothing is staged, the kernel reads the inputs and writes the result through the buffers' device
 * mappings inside the one launch.  Pageable buffers: copied in and out around the kernel, pipelined
 * over groups of layers on separate copy streams.  Same results either way. */
JGPT_API int32_t jgpt_attn_decode_append_host(jgpt_kvpool pool, int32_t layer0, int32_t n_layers,
                                              const float *q_host, const float *k_host, const float *v_host,
                                              const int32_t *seq_ids_host, const int32_t *rope_pos_host,
                                              const int32_t *lens_host, int32_t n, float *out_host);

/* Causal prefill attention that fills the cache.  Replaces attn_fwd_run_core + masked softmax
 * (C/jgpt_cuda_extra_kernels_launches.inl:1840-1870, 239-276) and the reference's own FA-2 forward
 * (:1916-2050), fused with RoPE and the append of :1085-1099.
 * n_seqs sequences, sequence i contributing S_i = seq_starts[i+1]-seq_starts[i] consecutive rows of
 * q/k/v [n_tokens, heads*dhead] (fp32, before RoPE); row r of sequence i sits at cache slot r and
 * RoPE position rope_offsets[i] + r.  seq_starts_host has n_seqs+1 entries (host). */
JGPT_API int32_t jgpt_attn_prefill(jgpt_kvpool pool, int32_t layer, const float *q_dev, const float *k_dev,
                                   const float *v_dev, const int32_t *seq_ids_host,
                                   const int32_t *seq_starts_host, const int32_t *rope_offsets_host,
                                   int32_t n_seqs, float *out_dev);

/* ---------------------------------------------------------------------------------------------
 * Model + forward step.  Replaces GPTModel weights upload (J/model/GPTModel.java:241-293),
 * loadWeights (:1944-1965) and GptKvForward.forwardPrefillGpu / forwardDecodeGpu
 * (J/model/GptKvForward.java:46-90, 131-170).
 * ------------------------------------------------------------------------------------------- */
/* C[M,N] = A[M,K] . B[K,N], row-major fp32 device buffers, ordered on the context's stream: the
 * projection primitive of the forward step (TensorOpsGPU.matmulGpuDevice, J/TensorOpsGPU.java:1393;
 * native GEMM src/main/cpp/jgpt_cuda_jni_init_matmul.inl:67).  fp32-level accuracy (split-TF32
 * operands on the tensor cores; tcgen05 + tensor memory for prefill-sized M). */
JGPT_API int32_t jgpt_matmul_device(jgpt_ctx ctx, const float *a_dev, const float *b_dev, float *c_dev,
                                    int32_t M, int32_t K, int32_t N);

JGPT_API int32_t jgpt_model_create(jgpt_ctx ctx, int32_t vocab, int32_t max_seq_len, int32_t d_model,
                                   int32_t heads, int32_t layers, int32_t d_ff, float rms_eps,
                                   int32_t max_rows, jgpt_model *out);
JGPT_API int32_t jgpt_model_destroy(jgpt_model model);
/* Tensor idx in GPTModel.getParameters() order (:1928-1938): tok, pos, per layer
 * Wq,Wk,Wv,Wo,W1,W2,W3,norm1,norm2, then normFinal, lmHead.  host fp32, n_floats must match. */
JGPT_API int32_t jgpt_model_num_tensors(jgpt_model model, int32_t *n_out);
JGPT_API int32_t jgpt_model_set_tensor(jgpt_model model, int32_t idx, const float *host, uint64_t n_floats);
/* veles.weights.v1 file (J/model/GptModelWeightsLoader.java:58-81). */
JGPT_API int32_t jgpt_model_load_weights(jgpt_model model, const char *path);
/* The reverse: one tensor back to the host, and the whole set written as veles.weights.v1 (the writer
 * of J/training/LlmTrainerCheckpointIo.java:129-140). */
JGPT_API int32_t jgpt_model_get_tensor(jgpt_model model, int32_t idx, float *host, uint64_t n_floats);
JGPT_API int32_t jgpt_model_save_weights(jgpt_model model, const char *path);

/* forwardPrefill(ids [1,S], cache, ropeOffset) -> logits [S, vocab] (host).  Error contract of
 * J/model/GptKvForward.java:47-60.  logits_host [S, vocab], last_logits_host [vocab] and next_token_host
 * (greedy argmax of the last row) may each be NULL.  Sets the sequence length to S.  max_rows of
 * jgpt_model_create bounds the rows (tokens) of one forward call. */
JGPT_API int32_t jgpt_forward_prefill(jgpt_model model, jgpt_kvpool pool, int32_t seq, const int32_t *ids_host,
                                      int32_t S, int32_t rope_offset, float *logits_host,
                                      float *last_logits_host, int32_t *next_token_host);
/* The same for n prompts packed back to back (the reference loops over sequences: its prefill is
 * batch-1 only, J/model/GptKvForward.java:14-16).  Sequence i owns rows [seq_starts[i], seq_starts[i+1])
 * of ids_host.  all_logits_host [rows, vocab] only for n == 1; last_logits_host [n, vocab] and
 * next_tokens_host [n] (greedy argmax of each last row) may be NULL. */
JGPT_API int32_t jgpt_forward_prefill_batch(jgpt_model model, jgpt_kvpool pool, const int32_t *seq_ids_host,
                                            const int32_t *seq_starts_host, const int32_t *ids_host,
                                            const int32_t *rope_offsets_host, int32_t n, float *all_logits_host,
                                            float *last_logits_host, int32_t *next_tokens_host);
/* Batched forwardDecode: for i in [0,n) token ids[i] of sequence seq_ids[i] with
 * cacheLenBefore[i] (must equal the stored length, else JGPT_ERR_ILLEGAL_STATE; full ->
 * JGPT_ERR_ILLEGAL_STATE) and ropePosition[i] (J/model/GptKvForward.java:131-141).
 * logits_host [n, vocab] may be NULL; next_tokens_host [n] (greedy argmax on the device, ties ->
 * lowest id, J/model/GptAutoregressiveGenerator.java:288-299) may be NULL.  Lengths become +1.
 * Up to 512 rows the step's launches are replayed as a CUDA graph from the second call with the
 * same batch size and 128-token length bucket on (the reference replays its decoder layers the same
 * way, cudaGraphExecLaunch0; JGPT_B200_DECODE_GRAPH=0 launches every kernel eagerly). */
JGPT_API int32_t jgpt_forward_decode(jgpt_model model, jgpt_kvpool pool, const int32_t *seq_ids_host,
                                     const int32_t *ids_host, const int32_t *cache_len_before_host,
                                     const int32_t *rope_pos_host, int32_t n, float *logits_host,
                                     int32_t *next_tokens_host);
/* forwardDecode followed by sampleNextToken(logits, temperature, topK)
 * (J/model/GptAutoregressiveGenerator.java:208-286) with the sampler on the device: temperature
 * divide, stable top-k by (logit desc, index asc), softmax, inverse CDF in index order — the steps
 * and the summation order of the host routine, so the same draw gives the same token and no
 * logits cross PCIe.  u01_host [n]: one uniform draw per row (the reference draws from an unseeded
 * ThreadLocalRandom).  temperature <= 0: greedy. */
JGPT_API int32_t jgpt_forward_decode_sample(jgpt_model model, jgpt_kvpool pool, const int32_t *seq_ids_host,
                                            const int32_t *ids_host, const int32_t *cache_len_before_host,
                                            const int32_t *rope_pos_host, int32_t n, float temperature,
                                            int32_t top_k, const float *u01_host, int32_t *next_tokens_host);
/* sampleNextToken on host logits (J/model/GptAutoregressiveGenerator.java:208-286): temperature, stable
 * top-k by (logit desc, index asc), softmax, inverse CDF with the caller's uniform draw u01 (the
 * reference draws from an unseeded ThreadLocalRandom); greedy with lowest-index ties when temperature <= 0. */
JGPT_API int32_t jgpt_sample_next_token(const float *logits_host, int32_t vocab, float temperature, int32_t top_k,
                                        float u01, int32_t *token_out);
/* GPTModel.generateGpuKv, greedy (temperature <= 0) (J/model/GptAutoregressiveGenerator.java:108-206):
 * out_host [S + max_new]; prompt kept, stop on sampled id 0 with a zero tail, sliding-window
 * re-prefill when the context overflows.  n_sampled_out = number of sampled tokens. */
JGPT_API int32_t jgpt_generate_greedy(jgpt_model model, jgpt_kvpool pool, const int32_t *prompt_host, int32_t S,
                                      int32_t max_new, int32_t *out_host, int32_t *n_sampled_out);
/* The same loop with the rolling window instead of the re-prefill: when the sequence has filled its context the
 * oldest block is dropped (jgpt_seq_drop_front) and decoding continues, RoPE at the absolute position and the
 * position-table row = position mod max_seq_len (each token keeps the row it was embedded with while it stays
 * in the window).  Needs a pool whose RoPE table (max_positions) covers S + max_new - 1 positions; jgpt_forward_decode
 * accepts positions beyond max_seq_len only on such a pool, otherwise it rejects them as the reference does.
 * Identical to jgpt_generate_greedy until the context first fills; not an exact-parity mode after that. */
JGPT_API int32_t jgpt_generate_greedy_rolling(jgpt_model model, jgpt_kvpool pool, const int32_t *prompt_host, int32_t S,
                                              int32_t max_new, int32_t *out_host, int32_t *n_sampled_out);


/* ---------------------------------------------------------------------------------------------
 * Continuous-batching scheduler (one model + one pool on one GPU).  The reference generates one
 * sequence per call with a fresh KvCacheGpu (J/model/GptAutoregressiveGenerator.java:108-206); the
 * per-sequence rules are kept (greedy argmax, lowest-index ties, stop on sampled id 0), the batching
 * policy is new and deterministic: FIFO admission that reserves ceil((prompt + max_new - 1)/16)
 * blocks up front, LRU eviction of finished sequences when the pool or the sequence slots run
 * short, one batched prefill for the requests admitted in a step, one batched decode step for the
 * requests already running.
 * ------------------------------------------------------------------------------------------- */
JGPT_API int32_t jgpt_sched_create(jgpt_model model, jgpt_kvpool pool, int32_t max_running,
                                   int32_t max_rows_per_call, int32_t max_seq_len, uint64_t *sched_out);
JGPT_API int32_t jgpt_sched_destroy(uint64_t sched);
/* Queue a request: prompt of S ids, up to max_new sampled tokens.  JGPT_ERR_INVALID_ARGUMENT when
 * S + max_new - 1 exceeds the context (there is no sliding window while batching). */
JGPT_API int32_t jgpt_sched_submit(uint64_t sched, const int32_t *prompt_host, int32_t S, int32_t max_new,
                                   int32_t *req_id_out);
/* One step.  pairs_out receives (request id, token) for each token sampled in this step. */
JGPT_API int32_t jgpt_sched_step(uint64_t sched, int32_t *pairs_out, int32_t cap_pairs, int32_t *n_pairs_out,
                                 int32_t *n_running_out, int32_t *n_waiting_out);
/* Tokens sampled so far for a request; state 0 waiting, 1 running, 2 finished; its sequence slot. */
JGPT_API int32_t jgpt_sched_result(uint64_t sched, int32_t req_id, int32_t *tokens_out, int32_t cap,
                                   int32_t *n_out, int32_t *state_out, int32_t *seq_out);
/* Event log, flat (type, a, b) triples: 1 admit(request, sequence slot), 2 evict(sequence slot,
 * request), 3 finish(request, tokens sampled). */
JGPT_API int32_t jgpt_sched_events(uint64_t sched, int32_t *out, int32_t cap_ints, int32_t *n_ints_out);

/* ---------------------------------------------------------------------------------------------
 * Multi-GPU: gather of the sampled token ids (one process + one context per GPU of one box).
 * Sequences are sharded over the GPUs and never interact; the only exchange is what each rank
 * sampled in a step.  The reference has no counterpart: it drives device 0 only
 * (C/jgpt_cuda_jni_ops_graph.inl:112,119).  NCCL (libnccl.so.2, or the path in JGPT_B200_NCCL_LIB)
 * is opened at run time, so single-GPU hosts do not need it.
 * ------------------------------------------------------------------------------------------- */

/* Rank 0 makes the 128-byte rendezvous id (ncclGetUniqueId) and gives it to the other ranks by
 * whatever channel the host has (a file, a socket, the launcher's store). */
JGPT_API int32_t jgpt_comm_unique_id(void *id_out, int32_t cap_bytes);
/* Joins `world` ranks.  Each step a rank contributes up to max_words int32 words; up to `depth`
 * steps may be in flight before a result has to be read (the ring holds depth + 2 slots).
 * timeout_ms bounds every wait on the other ranks inside later calls (the rendezvous itself is given
 * at least 60 s); a wait that runs out returns JGPT_ERR_TIMEOUT.  world = 1 needs no id and no NCCL.
 * Allocates its buffers here, nothing later. */
JGPT_API int32_t jgpt_comm_create(jgpt_ctx ctx, const void *unique_id, int32_t world, int32_t rank,
                                  int32_t max_words, int32_t depth, int32_t timeout_ms, uint64_t *comm_out);
/* Orderly when nothing is in flight; otherwise aborts the communicator (ncclCommAbort), which also
 * ends a collective that is still waiting for a rank that never came. */
JGPT_API int32_t jgpt_comm_destroy(uint64_t comm);
/* One step's words from host memory, e.g. the (request id, token) pairs of jgpt_sched_step.
 * Enqueues upload, ncclAllGather and download on the communicator's own stream and returns. */
JGPT_API int32_t jgpt_comm_submit(uint64_t comm, const int32_t *words_host, int32_t n_words);
/* The same from device memory, ordered after the work already enqueued on the context's stream:
 * e.g. the token ids the sampler of jgpt_forward_decode left on the device
 * (jgpt_model_next_tokens_device), without a round trip through the host. */
JGPT_API int32_t jgpt_comm_submit_device(uint64_t comm, const int32_t *words_dev, int32_t n_words);
/* Steps in flight; *must_pop_out = 1 when more than `depth` are, i.e. read one before submitting. */
JGPT_API int32_t jgpt_comm_in_flight(uint64_t comm, int32_t *n_out, int32_t *must_pop_out);
/* Result of the oldest step in flight: words_out [world][max_words] (unused tail = -1) and
 * counts_out [world], rank by rank, identical on every rank.  Waits at most timeout_ms; on
 * JGPT_ERR_TIMEOUT the step stays in flight and the call may be repeated. */
JGPT_API int32_t jgpt_comm_pop(uint64_t comm, int32_t *words_out, int32_t *counts_out, int32_t timeout_ms);
/* Device address of the token ids sampled by the model's last forward step ([rows] int32). */
JGPT_API int32_t jgpt_model_next_tokens_device(jgpt_model model, const int32_t **dev_out);

/* Decode attention that allocates nothing.  No counterpart in the reference.
 *
 * Same computation as jgpt_attn_decode for ONE layer, but the split-K scratch (partial softmax
 * states and arrival counters) lives in a fixed array inside the library instead of memory that
 * jgpt_attn_decode obtains with cudaMalloc when a launch first needs it.  It is meant for hosts
 * that must not allocate while generating: a process that has already given the whole GPU to its
 * own buffers (a late cudaMalloc may fail there, and every cudaMalloc/cudaFree stalls the device).
 * The call makes no cudaMalloc / cudaFree and uses no allocating library routine.
 *
 *   - Set-up and when the memory is taken.  The first call on a device resolves the array's device
 *     address (cudaGetSymbolAddress) and raises the kernel's shared-memory limit.  CUDA loads code
 *     lazily, so it is this first use -- not opening the library -- that reserves the array's
 *     4 MiB + 16 KiB on that GPU and loads the kernel; from then on the GPU holds them until the
 *     process exits and later calls take no device memory at all.  A call with n = 0 performs only
 *     the set-up (pointers may be NULL): make it once per device BEFORE the host commits the rest of
 *     the GPU and before any stream capture.
 *   - Limits apply only when a sequence is split into chunks (one chunk needs no scratch):
 *     n * chunks * heads * (dhead+2) <= 1,048,576 partial words and n * head_groups <= 4,096
 *     counters, where chunks <= ceil(ceil(max_len/16) / 4) (a chunk is never shorter than 4 blocks)
 *     and head_groups <= heads; a request within those caller-computable bounds always fits.
 *     Larger requests return JGPT_ERR_INVALID_ARGUMENT with a message that states the numbers.
 *   - All calls on a device share the one array and it keeps the previous call's contents: the call
 *     clears the counters it uses on the stream before launching.  Two calls that overlap on the
 *     GPU (different contexts or streams on the same device) race on it; keep them stream ordered. */
JGPT_API int32_t jgpt_attn_decode_static_scratch(jgpt_kvpool pool, int32_t layer, const float *q_dev,
                                                 const int32_t *seq_ids_dev, const int32_t *rope_pos_dev,
                                                 const int32_t *lens_dev, int32_t n, int32_t max_len,
                                                 float *out_dev);

#ifdef __cplusplus
}
#endif
#endif /* JGPT_B200_H */
