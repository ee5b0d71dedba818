// GENERATED from include/jgpt_b200.h: one downcall handle and one typed static method per C entry point.
// Not compiled where this repository is built (no JDK there); it targets the reference's own toolchain
// (Java 25, java.lang.foreign, launched with --enable-native-access=ALL-UNNAMED as scripts/jgpt-chat.sh does).
package com.veles.llm.jgpt.b200;

import static java.lang.foreign.ValueLayout.ADDRESS;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.FunctionDescriptor;
import java.lang.foreign.Linker;
import java.lang.foreign.MemorySegment;
import java.lang.foreign.SymbolLookup;
import java.lang.invoke.MethodHandle;

/** Raw bindings of libjgpt_b200.so.  Every method returns the C status code unchanged; see {@link B200Status}. */
public final class JgptB200 {
    private JgptB200() {}

    private static final Linker LINKER = Linker.nativeLinker();
    private static final SymbolLookup LIB = B200Library.lookup();

    private static MethodHandle bind(String name, FunctionDescriptor fd) {
        return LINKER.downcallHandle(
                LIB.find(name).orElseThrow(() -> new UnsatisfiedLinkError("libjgpt_b200.so lacks " + name)), fd);
    }

    private static RuntimeException rethrow(Throwable t) {
        if (t instanceof RuntimeException r) return r;
        if (t instanceof Error e) throw e;
        return new IllegalStateException(t);
    }

    private static final MethodHandle H_CTX_CREATE = bind("jgpt_ctx_create", FunctionDescriptor.of(JAVA_INT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_CTX_DESTROY = bind("jgpt_ctx_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_SYNC = bind("jgpt_sync", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_LAST_ERROR = bind("jgpt_last_error", FunctionDescriptor.of(ADDRESS));
    private static final MethodHandle H_CTX_STREAM = bind("jgpt_ctx_stream", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_DEVICE_COUNT = bind("jgpt_device_count", FunctionDescriptor.of(JAVA_INT, ADDRESS));
    private static final MethodHandle H_DEVICE_PCI_BUS_ID = bind("jgpt_device_pci_bus_id", FunctionDescriptor.of(JAVA_INT, JAVA_INT, ADDRESS, JAVA_INT));
    private static final MethodHandle H_ENV_CONFIG = bind("jgpt_env_config", FunctionDescriptor.of(JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS));
    private static final MethodHandle H_DEV_ALLOC = bind("jgpt_dev_alloc", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_DEV_FREE = bind("jgpt_dev_free", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_H2D = bind("jgpt_h2d", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, JAVA_LONG));
    private static final MethodHandle H_D2H = bind("jgpt_d2h", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, JAVA_LONG));
    private static final MethodHandle H_DEV_MEMSET = bind("jgpt_dev_memset", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_MEM_INFO = bind("jgpt_mem_info", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS));
    private static final MethodHandle H_HOST_ALLOC_PINNED = bind("jgpt_host_alloc_pinned", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_HOST_FREE_PINNED = bind("jgpt_host_free_pinned", FunctionDescriptor.of(JAVA_INT, ADDRESS));
    private static final MethodHandle H_EVENT_CREATE = bind("jgpt_event_create", FunctionDescriptor.of(JAVA_INT, ADDRESS));
    private static final MethodHandle H_EVENT_DESTROY = bind("jgpt_event_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_EVENT_RECORD = bind("jgpt_event_record", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG));
    private static final MethodHandle H_EVENT_ELAPSED_MS = bind("jgpt_event_elapsed_ms", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_GRAPH_BEGIN_CAPTURE = bind("jgpt_graph_begin_capture", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_GRAPH_END_CAPTURE = bind("jgpt_graph_end_capture", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_GRAPH_LAUNCH = bind("jgpt_graph_launch", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG));
    private static final MethodHandle H_GRAPH_DESTROY = bind("jgpt_graph_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_KVPOOL_CREATE = bind("jgpt_kvpool_create", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_FLOAT, ADDRESS));
    private static final MethodHandle H_KVPOOL_DESTROY = bind("jgpt_kvpool_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_KVPOOL_FREE_BLOCKS = bind("jgpt_kvpool_free_blocks", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_KVPOOL_STORAGE = bind("jgpt_kvpool_storage", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS));
    private static final MethodHandle H_KVPOOL_SET_TUNING = bind("jgpt_kvpool_set_tuning", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_KVPOOL_TABLE_DEVICE = bind("jgpt_kvpool_table_device", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS));
    private static final MethodHandle H_SEQ_ALLOC = bind("jgpt_seq_alloc", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_SEQ_FREE = bind("jgpt_seq_free", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT));
    private static final MethodHandle H_SEQ_RESERVE = bind("jgpt_seq_reserve", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_SEQ_LENGTH = bind("jgpt_seq_length", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS));
    private static final MethodHandle H_SEQ_SET_LENGTH = bind("jgpt_seq_set_length", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_SEQ_CLEAR = bind("jgpt_seq_clear", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_SEQ_DROP_FRONT = bind("jgpt_seq_drop_front", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_SEQ_SET_BLOCK_TABLE = bind("jgpt_seq_set_block_table", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_INT));
    private static final MethodHandle H_BLOCK_TABLE_COPY_OUT = bind("jgpt_block_table_copy_out", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS));
    private static final MethodHandle H_BLOCK_TABLE_COPY_OUT_DEVICE = bind("jgpt_block_table_copy_out_device", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS));
    private static final MethodHandle H_SEQ_MARK_EVICTABLE = bind("jgpt_seq_mark_evictable", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_KV_EVICT_LRU = bind("jgpt_kv_evict_lru", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS));
    private static final MethodHandle H_KV_APPEND = bind("jgpt_kv_append", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT));
    private static final MethodHandle H_KV_GATHER = bind("jgpt_kv_gather", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
    private static final MethodHandle H_KV_GATHER_BATCH = bind("jgpt_kv_gather_batch", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
    private static final MethodHandle H_ATTN_DECODE = bind("jgpt_attn_decode", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_ATTN_DECODE_APPEND = bind("jgpt_attn_decode_append", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_ATTN_DECODE_APPEND_HOST = bind("jgpt_attn_decode_append_host", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
    private static final MethodHandle H_ATTN_PREFILL = bind("jgpt_attn_prefill", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS));
    private static final MethodHandle H_MATMUL_DEVICE = bind("jgpt_matmul_device", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT));
    private static final MethodHandle H_MODEL_CREATE = bind("jgpt_model_create", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_FLOAT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_MODEL_DESTROY = bind("jgpt_model_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_MODEL_NUM_TENSORS = bind("jgpt_model_num_tensors", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_MODEL_SET_TENSOR = bind("jgpt_model_set_tensor", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_LONG));
    private static final MethodHandle H_MODEL_LOAD_WEIGHTS = bind("jgpt_model_load_weights", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_MODEL_GET_TENSOR = bind("jgpt_model_get_tensor", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_LONG));
    private static final MethodHandle H_MODEL_SAVE_WEIGHTS = bind("jgpt_model_save_weights", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_FORWARD_PREFILL = bind("jgpt_forward_prefill", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
    private static final MethodHandle H_FORWARD_PREFILL_BATCH = bind("jgpt_forward_prefill_batch", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
    private static final MethodHandle H_FORWARD_DECODE = bind("jgpt_forward_decode", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, ADDRESS, ADDRESS));
    private static final MethodHandle H_FORWARD_DECODE_SAMPLE = bind("jgpt_forward_decode_sample", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_FLOAT, JAVA_INT, ADDRESS, ADDRESS));
    private static final MethodHandle H_SAMPLE_NEXT_TOKEN = bind("jgpt_sample_next_token", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT, JAVA_FLOAT, JAVA_INT, JAVA_FLOAT, ADDRESS));
    private static final MethodHandle H_GENERATE_GREEDY = bind("jgpt_generate_greedy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
    private static final MethodHandle H_GENERATE_GREEDY_ROLLING = bind("jgpt_generate_greedy_rolling", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS, ADDRESS));
    private static final MethodHandle H_SCHED_CREATE = bind("jgpt_sched_create", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_LONG, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_SCHED_DESTROY = bind("jgpt_sched_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_SCHED_SUBMIT = bind("jgpt_sched_submit", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_SCHED_STEP = bind("jgpt_sched_step", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
    private static final MethodHandle H_SCHED_RESULT = bind("jgpt_sched_result", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, JAVA_INT, ADDRESS, ADDRESS, ADDRESS));
    private static final MethodHandle H_SCHED_EVENTS = bind("jgpt_sched_events", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, ADDRESS));
    private static final MethodHandle H_COMM_UNIQUE_ID = bind("jgpt_comm_unique_id", FunctionDescriptor.of(JAVA_INT, ADDRESS, JAVA_INT));
    private static final MethodHandle H_COMM_CREATE = bind("jgpt_comm_create", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, JAVA_INT, ADDRESS));
    private static final MethodHandle H_COMM_DESTROY = bind("jgpt_comm_destroy", FunctionDescriptor.of(JAVA_INT, JAVA_LONG));
    private static final MethodHandle H_COMM_SUBMIT = bind("jgpt_comm_submit", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT));
    private static final MethodHandle H_COMM_SUBMIT_DEVICE = bind("jgpt_comm_submit_device", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, JAVA_INT));
    private static final MethodHandle H_COMM_IN_FLIGHT = bind("jgpt_comm_in_flight", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS));
    private static final MethodHandle H_COMM_POP = bind("jgpt_comm_pop", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS, ADDRESS, JAVA_INT));
    private static final MethodHandle H_MODEL_NEXT_TOKENS_DEVICE = bind("jgpt_model_next_tokens_device", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, ADDRESS));
    private static final MethodHandle H_ATTN_DECODE_STATIC_SCRATCH = bind("jgpt_attn_decode_static_scratch", FunctionDescriptor.of(JAVA_INT, JAVA_LONG, JAVA_INT, ADDRESS, ADDRESS, ADDRESS, ADDRESS, JAVA_INT, JAVA_INT, ADDRESS));

    /** jgpt_ctx_create */
    public static int ctxCreate(int device, MemorySegment out) {
        try { return (int) H_CTX_CREATE.invokeExact(device, out); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_ctx_destroy */
    public static int ctxDestroy(long ctx) {
        try { return (int) H_CTX_DESTROY.invokeExact(ctx); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sync */
    public static int sync(long ctx) {
        try { return (int) H_SYNC.invokeExact(ctx); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_last_error */
    public static MemorySegment lastError() {
        try { return (MemorySegment) H_LAST_ERROR.invokeExact(); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_ctx_stream */
    public static int ctxStream(long ctx, MemorySegment stream_out) {
        try { return (int) H_CTX_STREAM.invokeExact(ctx, streamOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_device_count */
    public static int deviceCount(MemorySegment out) {
        try { return (int) H_DEVICE_COUNT.invokeExact(out); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_device_pci_bus_id */
    public static int devicePciBusId(int device, MemorySegment out, int cap) {
        try { return (int) H_DEVICE_PCI_BUS_ID.invokeExact(device, out, cap); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_env_config */
    public static int envConfig(MemorySegment kv_block_tokens_out, MemorySegment kv_pool_blocks_out, MemorySegment max_seq_len_out, MemorySegment rmsnorm_eps_out, MemorySegment backend_b200_out) {
        try { return (int) H_ENV_CONFIG.invokeExact(kvBlockTokensOut, kvPoolBlocksOut, maxSeqLenOut, rmsnormEpsOut, backendB200Out); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_dev_alloc */
    public static int devAlloc(long ctx, long bytes, MemorySegment dev_out) {
        try { return (int) H_DEV_ALLOC.invokeExact(ctx, bytes, devOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_dev_free */
    public static int devFree(long ctx, MemorySegment dev) {
        try { return (int) H_DEV_FREE.invokeExact(ctx, dev); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_h2d */
    public static int h2d(long ctx, MemorySegment dev_dst, MemorySegment host_src, long bytes) {
        try { return (int) H_H2D.invokeExact(ctx, devDst, hostSrc, bytes); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_d2h */
    public static int d2h(long ctx, MemorySegment host_dst, MemorySegment dev_src, long bytes) {
        try { return (int) H_D2H.invokeExact(ctx, hostDst, devSrc, bytes); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_dev_memset */
    public static int devMemset(long ctx, MemorySegment dev, int byte_value, long bytes) {
        try { return (int) H_DEV_MEMSET.invokeExact(ctx, dev, byteValue, bytes); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_mem_info */
    public static int memInfo(long ctx, MemorySegment free_bytes_out, MemorySegment total_bytes_out) {
        try { return (int) H_MEM_INFO.invokeExact(ctx, freeBytesOut, totalBytesOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_host_alloc_pinned */
    public static int hostAllocPinned(long bytes, MemorySegment host_out) {
        try { return (int) H_HOST_ALLOC_PINNED.invokeExact(bytes, hostOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_host_free_pinned */
    public static int hostFreePinned(MemorySegment host) {
        try { return (int) H_HOST_FREE_PINNED.invokeExact(host); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_event_create */
    public static int eventCreate(MemorySegment event_out) {
        try { return (int) H_EVENT_CREATE.invokeExact(eventOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_event_destroy */
    public static int eventDestroy(long event) {
        try { return (int) H_EVENT_DESTROY.invokeExact(event); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_event_record */
    public static int eventRecord(long ctx, long event) {
        try { return (int) H_EVENT_RECORD.invokeExact(ctx, event); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_event_elapsed_ms */
    public static int eventElapsedMs(long start, long stop, MemorySegment ms_out) {
        try { return (int) H_EVENT_ELAPSED_MS.invokeExact(start, stop, msOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_graph_begin_capture */
    public static int graphBeginCapture(long ctx) {
        try { return (int) H_GRAPH_BEGIN_CAPTURE.invokeExact(ctx); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_graph_end_capture */
    public static int graphEndCapture(long ctx, MemorySegment graph_exec_out) {
        try { return (int) H_GRAPH_END_CAPTURE.invokeExact(ctx, graphExecOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_graph_launch */
    public static int graphLaunch(long ctx, long graph_exec) {
        try { return (int) H_GRAPH_LAUNCH.invokeExact(ctx, graphExec); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_graph_destroy */
    public static int graphDestroy(long graph_exec) {
        try { return (int) H_GRAPH_DESTROY.invokeExact(graphExec); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kvpool_create */
    public static int kvpoolCreate(long ctx, int layers, int heads, int dhead, int block_tokens, int n_blocks, int max_seqs, int max_blocks_per_seq, int max_positions, float rope_base, MemorySegment out) {
        try { return (int) H_KVPOOL_CREATE.invokeExact(ctx, layers, heads, dhead, blockTokens, nBlocks, maxSeqs, maxBlocksPerSeq, maxPositions, ropeBase, out); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kvpool_destroy */
    public static int kvpoolDestroy(long pool) {
        try { return (int) H_KVPOOL_DESTROY.invokeExact(pool); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kvpool_free_blocks */
    public static int kvpoolFreeBlocks(long pool, MemorySegment n_free_out) {
        try { return (int) H_KVPOOL_FREE_BLOCKS.invokeExact(pool, nFreeOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kvpool_storage */
    public static int kvpoolStorage(long pool, MemorySegment dev_out, MemorySegment bytes_out) {
        try { return (int) H_KVPOOL_STORAGE.invokeExact(pool, devOut, bytesOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kvpool_set_tuning */
    public static int kvpoolSetTuning(long pool, int chunk_blocks, int stages, int head_group, int persistent, int launch_overlap) {
        try { return (int) H_KVPOOL_SET_TUNING.invokeExact(pool, chunkBlocks, stages, headGroup, persistent, launchOverlap); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kvpool_table_device */
    public static int kvpoolTableDevice(long pool, MemorySegment dev_out, MemorySegment row_stride_out) {
        try { return (int) H_KVPOOL_TABLE_DEVICE.invokeExact(pool, devOut, rowStrideOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_alloc */
    public static int seqAlloc(long pool, MemorySegment seq_out) {
        try { return (int) H_SEQ_ALLOC.invokeExact(pool, seqOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_free */
    public static int seqFree(long pool, int seq) {
        try { return (int) H_SEQ_FREE.invokeExact(pool, seq); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_reserve */
    public static int seqReserve(long pool, int seq, int n_tokens) {
        try { return (int) H_SEQ_RESERVE.invokeExact(pool, seq, nTokens); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_length */
    public static int seqLength(long pool, int seq, MemorySegment len_out) {
        try { return (int) H_SEQ_LENGTH.invokeExact(pool, seq, lenOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_set_length */
    public static int seqSetLength(long pool, int seq, int len) {
        try { return (int) H_SEQ_SET_LENGTH.invokeExact(pool, seq, len); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_clear */
    public static int seqClear(long pool, int seq, int zero_fill) {
        try { return (int) H_SEQ_CLEAR.invokeExact(pool, seq, zeroFill); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_drop_front */
    public static int seqDropFront(long pool, int seq, int n_blocks, int zero_fill) {
        try { return (int) H_SEQ_DROP_FRONT.invokeExact(pool, seq, nBlocks, zeroFill); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_set_block_table */
    public static int seqSetBlockTable(long pool, int seq, MemorySegment blocks_host, int n) {
        try { return (int) H_SEQ_SET_BLOCK_TABLE.invokeExact(pool, seq, blocksHost, n); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_block_table_copy_out */
    public static int blockTableCopyOut(long pool, int seq, MemorySegment blocks_host, int cap, MemorySegment n_out) {
        try { return (int) H_BLOCK_TABLE_COPY_OUT.invokeExact(pool, seq, blocksHost, cap, nOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_block_table_copy_out_device */
    public static int blockTableCopyOutDevice(long pool, int seq, MemorySegment blocks_host, int cap, MemorySegment n_out) {
        try { return (int) H_BLOCK_TABLE_COPY_OUT_DEVICE.invokeExact(pool, seq, blocksHost, cap, nOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_seq_mark_evictable */
    public static int seqMarkEvictable(long pool, int seq, int evictable) {
        try { return (int) H_SEQ_MARK_EVICTABLE.invokeExact(pool, seq, evictable); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kv_evict_lru */
    public static int kvEvictLru(long pool, int need_free, int zero_fill, MemorySegment victims_host, int cap, MemorySegment n_victims_out) {
        try { return (int) H_KV_EVICT_LRU.invokeExact(pool, needFree, zeroFill, victimsHost, cap, nVictimsOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kv_append */
    public static int kvAppend(long pool, int layer, MemorySegment k_dev, MemorySegment v_dev, MemorySegment seq_ids_dev, MemorySegment slot_pos_dev, MemorySegment rope_pos_dev, int n) {
        try { return (int) H_KV_APPEND.invokeExact(pool, layer, kDev, vDev, seqIdsDev, slotPosDev, ropePosDev, n); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kv_gather */
    public static int kvGather(long pool, int layer, int seq, int len, int max_seq_len, MemorySegment k_out_dev, MemorySegment v_out_dev) {
        try { return (int) H_KV_GATHER.invokeExact(pool, layer, seq, len, maxSeqLen, kOutDev, vOutDev); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_kv_gather_batch */
    public static int kvGatherBatch(long pool, int layer, MemorySegment seq_ids_host, MemorySegment lens_host, int n, int max_seq_len, MemorySegment k_out_dev, MemorySegment v_out_dev) {
        try { return (int) H_KV_GATHER_BATCH.invokeExact(pool, layer, seqIdsHost, lensHost, n, maxSeqLen, kOutDev, vOutDev); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_attn_decode */
    public static int attnDecode(long pool, int layer0, int n_layers, MemorySegment q_dev, MemorySegment seq_ids_dev, MemorySegment rope_pos_dev, MemorySegment lens_dev, int n, int max_len, MemorySegment out_dev) {
        try { return (int) H_ATTN_DECODE.invokeExact(pool, layer0, nLayers, qDev, seqIdsDev, ropePosDev, lensDev, n, maxLen, outDev); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_attn_decode_append */
    public static int attnDecodeAppend(long pool, int layer0, int n_layers, MemorySegment q_dev, MemorySegment k_dev, MemorySegment v_dev, MemorySegment seq_ids_dev, MemorySegment rope_pos_dev, MemorySegment lens_dev, int n, int max_len, MemorySegment out_dev) {
        try { return (int) H_ATTN_DECODE_APPEND.invokeExact(pool, layer0, nLayers, qDev, kDev, vDev, seqIdsDev, ropePosDev, lensDev, n, maxLen, outDev); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_attn_decode_append_host */
    public static int attnDecodeAppendHost(long pool, int layer0, int n_layers, MemorySegment q_host, MemorySegment k_host, MemorySegment v_host, MemorySegment seq_ids_host, MemorySegment rope_pos_host, MemorySegment lens_host, int n, MemorySegment out_host) {
        try { return (int) H_ATTN_DECODE_APPEND_HOST.invokeExact(pool, layer0, nLayers, qHost, kHost, vHost, seqIdsHost, ropePosHost, lensHost, n, outHost); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_attn_prefill */
    public static int attnPrefill(long pool, int layer, MemorySegment q_dev, MemorySegment k_dev, MemorySegment v_dev, MemorySegment seq_ids_host, MemorySegment seq_starts_host, MemorySegment rope_offsets_host, int n_seqs, MemorySegment out_dev) {
        try { return (int) H_ATTN_PREFILL.invokeExact(pool, layer, qDev, kDev, vDev, seqIdsHost, seqStartsHost, ropeOffsetsHost, nSeqs, outDev); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_matmul_device */
    public static int matmulDevice(long ctx, MemorySegment a_dev, MemorySegment b_dev, MemorySegment c_dev, int M, int K, int N) {
        try { return (int) H_MATMUL_DEVICE.invokeExact(ctx, aDev, bDev, cDev, M, K, N); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_create */
    public static int modelCreate(long ctx, int vocab, int max_seq_len, int d_model, int heads, int layers, int d_ff, float rms_eps, int max_rows, MemorySegment out) {
        try { return (int) H_MODEL_CREATE.invokeExact(ctx, vocab, maxSeqLen, dModel, heads, layers, dFf, rmsEps, maxRows, out); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_destroy */
    public static int modelDestroy(long model) {
        try { return (int) H_MODEL_DESTROY.invokeExact(model); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_num_tensors */
    public static int modelNumTensors(long model, MemorySegment n_out) {
        try { return (int) H_MODEL_NUM_TENSORS.invokeExact(model, nOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_set_tensor */
    public static int modelSetTensor(long model, int idx, MemorySegment host, long n_floats) {
        try { return (int) H_MODEL_SET_TENSOR.invokeExact(model, idx, host, nFloats); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_load_weights */
    public static int modelLoadWeights(long model, MemorySegment path) {
        try { return (int) H_MODEL_LOAD_WEIGHTS.invokeExact(model, path); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_get_tensor */
    public static int modelGetTensor(long model, int idx, MemorySegment host, long n_floats) {
        try { return (int) H_MODEL_GET_TENSOR.invokeExact(model, idx, host, nFloats); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_save_weights */
    public static int modelSaveWeights(long model, MemorySegment path) {
        try { return (int) H_MODEL_SAVE_WEIGHTS.invokeExact(model, path); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_forward_prefill */
    public static int forwardPrefill(long model, long pool, int seq, MemorySegment ids_host, int S, int rope_offset, MemorySegment logits_host, MemorySegment last_logits_host, MemorySegment next_token_host) {
        try { return (int) H_FORWARD_PREFILL.invokeExact(model, pool, seq, idsHost, S, ropeOffset, logitsHost, lastLogitsHost, nextTokenHost); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_forward_prefill_batch */
    public static int forwardPrefillBatch(long model, long pool, MemorySegment seq_ids_host, MemorySegment seq_starts_host, MemorySegment ids_host, MemorySegment rope_offsets_host, int n, MemorySegment all_logits_host, MemorySegment last_logits_host, MemorySegment next_tokens_host) {
        try { return (int) H_FORWARD_PREFILL_BATCH.invokeExact(model, pool, seqIdsHost, seqStartsHost, idsHost, ropeOffsetsHost, n, allLogitsHost, lastLogitsHost, nextTokensHost); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_forward_decode */
    public static int forwardDecode(long model, long pool, MemorySegment seq_ids_host, MemorySegment ids_host, MemorySegment cache_len_before_host, MemorySegment rope_pos_host, int n, MemorySegment logits_host, MemorySegment next_tokens_host) {
        try { return (int) H_FORWARD_DECODE.invokeExact(model, pool, seqIdsHost, idsHost, cacheLenBeforeHost, ropePosHost, n, logitsHost, nextTokensHost); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_forward_decode_sample */
    public static int forwardDecodeSample(long model, long pool, MemorySegment seq_ids_host, MemorySegment ids_host, MemorySegment cache_len_before_host, MemorySegment rope_pos_host, int n, float temperature, int top_k, MemorySegment u01_host, MemorySegment next_tokens_host) {
        try { return (int) H_FORWARD_DECODE_SAMPLE.invokeExact(model, pool, seqIdsHost, idsHost, cacheLenBeforeHost, ropePosHost, n, temperature, topK, u01Host, nextTokensHost); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sample_next_token */
    public static int sampleNextToken(MemorySegment logits_host, int vocab, float temperature, int top_k, float u01, MemorySegment token_out) {
        try { return (int) H_SAMPLE_NEXT_TOKEN.invokeExact(logitsHost, vocab, temperature, topK, u01, tokenOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_generate_greedy */
    public static int generateGreedy(long model, long pool, MemorySegment prompt_host, int S, int max_new, MemorySegment out_host, MemorySegment n_sampled_out) {
        try { return (int) H_GENERATE_GREEDY.invokeExact(model, pool, promptHost, S, maxNew, outHost, nSampledOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_generate_greedy_rolling */
    public static int generateGreedyRolling(long model, long pool, MemorySegment prompt_host, int S, int max_new, MemorySegment out_host, MemorySegment n_sampled_out) {
        try { return (int) H_GENERATE_GREEDY_ROLLING.invokeExact(model, pool, promptHost, S, maxNew, outHost, nSampledOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sched_create */
    public static int schedCreate(long model, long pool, int max_running, int max_rows_per_call, int max_seq_len, MemorySegment sched_out) {
        try { return (int) H_SCHED_CREATE.invokeExact(model, pool, maxRunning, maxRowsPerCall, maxSeqLen, schedOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sched_destroy */
    public static int schedDestroy(long sched) {
        try { return (int) H_SCHED_DESTROY.invokeExact(sched); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sched_submit */
    public static int schedSubmit(long sched, MemorySegment prompt_host, int S, int max_new, MemorySegment req_id_out) {
        try { return (int) H_SCHED_SUBMIT.invokeExact(sched, promptHost, S, maxNew, reqIdOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sched_step */
    public static int schedStep(long sched, MemorySegment pairs_out, int cap_pairs, MemorySegment n_pairs_out, MemorySegment n_running_out, MemorySegment n_waiting_out) {
        try { return (int) H_SCHED_STEP.invokeExact(sched, pairsOut, capPairs, nPairsOut, nRunningOut, nWaitingOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sched_result */
    public static int schedResult(long sched, int req_id, MemorySegment tokens_out, int cap, MemorySegment n_out, MemorySegment state_out, MemorySegment seq_out) {
        try { return (int) H_SCHED_RESULT.invokeExact(sched, reqId, tokensOut, cap, nOut, stateOut, seqOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_sched_events */
    public static int schedEvents(long sched, MemorySegment out, int cap_ints, MemorySegment n_ints_out) {
        try { return (int) H_SCHED_EVENTS.invokeExact(sched, out, capInts, nIntsOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_unique_id */
    public static int commUniqueId(MemorySegment id_out, int cap_bytes) {
        try { return (int) H_COMM_UNIQUE_ID.invokeExact(idOut, capBytes); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_create */
    public static int commCreate(long ctx, MemorySegment unique_id, int world, int rank, int max_words, int depth, int timeout_ms, MemorySegment comm_out) {
        try { return (int) H_COMM_CREATE.invokeExact(ctx, uniqueId, world, rank, maxWords, depth, timeoutMs, commOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_destroy */
    public static int commDestroy(long comm) {
        try { return (int) H_COMM_DESTROY.invokeExact(comm); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_submit */
    public static int commSubmit(long comm, MemorySegment words_host, int n_words) {
        try { return (int) H_COMM_SUBMIT.invokeExact(comm, wordsHost, nWords); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_submit_device */
    public static int commSubmitDevice(long comm, MemorySegment words_dev, int n_words) {
        try { return (int) H_COMM_SUBMIT_DEVICE.invokeExact(comm, wordsDev, nWords); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_in_flight */
    public static int commInFlight(long comm, MemorySegment n_out, MemorySegment must_pop_out) {
        try { return (int) H_COMM_IN_FLIGHT.invokeExact(comm, nOut, mustPopOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_comm_pop */
    public static int commPop(long comm, MemorySegment words_out, MemorySegment counts_out, int timeout_ms) {
        try { return (int) H_COMM_POP.invokeExact(comm, wordsOut, countsOut, timeoutMs); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_model_next_tokens_device */
    public static int modelNextTokensDevice(long model, MemorySegment dev_out) {
        try { return (int) H_MODEL_NEXT_TOKENS_DEVICE.invokeExact(model, devOut); } catch (Throwable t) { throw rethrow(t); }
    }

    /** jgpt_attn_decode_static_scratch */
    public static int attnDecodeStaticScratch(long pool, int layer, MemorySegment q_dev, MemorySegment seq_ids_dev, MemorySegment rope_pos_dev, MemorySegment lens_dev, int n, int max_len, MemorySegment out_dev) {
        try { return (int) H_ATTN_DECODE_STATIC_SCRATCH.invokeExact(pool, layer, qDev, seqIdsDev, ropePosDev, lensDev, n, maxLen, outDev); } catch (Throwable t) { throw rethrow(t); }
    }

}
