package com.veles.llm.jgpt.b200;

import static com.veles.llm.jgpt.b200.B200Status.check;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;

/**
 * Paged fp16 K/V store of one model on one GPU: fixed blocks of 16 tokens per layer and head, one block table per
 * sequence.  It replaces the per-sequence contiguous fp32 buffers of the reference's {@code KvCacheGpu}
 * (model/KvCacheGpu.java:12-118): many {@link KvCacheGpu} views (one per generated sequence) share one pool.
 * The library owns all device memory behind the handle; the allocator (free list, LRU eviction) lives in the
 * library as well, so Java only forwards.
 */
public final class KvPool implements AutoCloseable {
    public static final int BLOCK_TOKENS = 16;

    private final B200Context ctx;
    private long handle;
    public final int layers, heads, dHead, nBlocks, maxSeqs, maxBlocksPerSeq, maxPositions;

    public KvPool(B200Context ctx, int layers, int heads, int dHead, int nBlocks, int maxSeqs, int maxBlocksPerSeq, int maxPositions) {
        this.ctx = ctx;
        this.layers = layers;
        this.heads = heads;
        this.dHead = dHead;
        this.nBlocks = nBlocks;
        this.maxSeqs = maxSeqs;
        this.maxBlocksPerSeq = maxBlocksPerSeq;
        this.maxPositions = maxPositions;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_LONG);
            // IllegalArgumentException on non-positive dimensions, as the KvCacheGpu constructor
            check(JgptB200.kvpoolCreate(ctx.handle(), layers, heads, dHead, BLOCK_TOKENS, nBlocks, maxSeqs, maxBlocksPerSeq, maxPositions,
                    10000.0f, out));
            handle = out.get(JAVA_LONG, 0);
        }
    }

    public B200Context context() {
        return ctx;
    }

    public long handle() {
        if (handle == 0) throw new IllegalStateException("KV pool is closed");
        return handle;
    }

    private int intOut(java.util.function.ToIntFunction<MemorySegment> call) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT);
            check(call.applyAsInt(out));
            return out.get(JAVA_INT, 0);
        }
    }

    public int freeBlocks() {
        return intOut(o -> JgptB200.kvpoolFreeBlocks(handle(), o));
    }

    /** A new sequence slot (lowest free id first): what {@code new KvCacheGpu(..)} is in the reference. */
    public int seqAlloc() {
        return intOut(o -> JgptB200.seqAlloc(handle(), o));
    }

    public void seqFree(int seq) {
        check(JgptB200.seqFree(handle(), seq));
    }

    /** Maps blocks for positions [0, nTokens); {@link B200Status.PoolExhaustedException} when the pool is full. */
    public void reserve(int seq, int nTokens) {
        check(JgptB200.seqReserve(handle(), seq, nTokens));
    }

    public int length(int seq) {
        return intOut(o -> JgptB200.seqLength(handle(), seq, o));
    }

    public void setLength(int seq, int len) {
        check(JgptB200.seqSetLength(handle(), seq, len));
    }

    public void clear(int seq, boolean zeroFill) {
        check(JgptB200.seqClear(handle(), seq, zeroFill ? 1 : 0));
    }

    /** Rolling window: forget the oldest {@code nBlocks} KV blocks of the sequence (no K/V byte moves, no re-prefill). */
    public void dropFront(int seq, int nBlocks, boolean zeroFill) {
        check(JgptB200.seqDropFront(handle(), seq, nBlocks, zeroFill ? 1 : 0));
    }

    public void markEvictable(int seq, boolean evictable) {
        check(JgptB200.seqMarkEvictable(handle(), seq, evictable ? 1 : 0));
    }

    /** Frees least-recently-used evictable sequences until {@code needFree} blocks are free; returns the victims. */
    public int[] evictLru(int needFree, boolean zeroFill) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment victims = a.allocate(JAVA_INT, maxSeqs), n = a.allocate(JAVA_INT);
            check(JgptB200.kvEvictLru(handle(), needFree, zeroFill ? 1 : 0, victims, maxSeqs, n));
            return victims.asSlice(0, 4L * n.get(JAVA_INT, 0)).toArray(JAVA_INT);
        }
    }

    /** Logical block -> physical block of a sequence (host allocator's view; the device mirror is identical). */
    public int[] blockTable(int seq) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT, maxBlocksPerSeq), n = a.allocate(JAVA_INT);
            check(JgptB200.blockTableCopyOut(handle(), seq, out, maxBlocksPerSeq, n));
            return out.asSlice(0, 4L * n.get(JAVA_INT, 0)).toArray(JAVA_INT);
        }
    }

    /** Contiguous fp32 [heads, maxSeqLen, dHead] planes of one layer of one sequence, as {@code getK/getV} expose them. */
    public void gather(int layer, int seq, int len, int maxSeqLen, long kOutDev, long vOutDev) {
        check(JgptB200.kvGather(handle(), layer, seq, len, maxSeqLen, MemorySegment.ofAddress(kOutDev), MemorySegment.ofAddress(vOutDev)));
    }

    @Override
    public void close() {
        if (handle != 0) {
            JgptB200.kvpoolDestroy(handle);
            handle = 0;
        }
    }
}
