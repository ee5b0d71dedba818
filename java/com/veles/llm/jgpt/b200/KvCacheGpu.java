package com.veles.llm.jgpt.b200;

/**
 * Drop-in for the reference's {@code model.KvCacheGpu} over the paged store: same constructor arguments, same public
 * methods, same exceptions (model/KvCacheGpu.java:12-118) -- but one instance is a sequence of a shared
 * {@link KvPool} instead of 2 x numLayers private fp32 buffers.
 *
 * <ul>
 *   <li>{@code new KvCacheGpu(layers, heads, dHead, maxSeqLen)} creates a private single-sequence pool (the reference's
 *       ownership model); {@code new KvCacheGpu(pool, maxSeqLen)} takes a slot of an existing pool (batched serving).
 *   <li>{@link #getK}/{@link #getV} return a gathered fp32 copy in the reference's layout
 *       {@code h*maxSeqLen*dHead + pos*dHead + j} (zero beyond {@code length()}), not the live storage.
 *   <li>{@link #clear} zero-fills and resets the length, {@link #setLength} rejects values outside [0, maxSeqLen].
 * </ul>
 * Not thread-safe, like the reference: one inference thread per cache.
 */
public final class KvCacheGpu implements AutoCloseable {
    private final KvPool pool;
    private final boolean ownsPool;
    private final int seq, maxSeqLen;
    private boolean closed;

    public KvCacheGpu(B200Context ctx, int numLayers, int numHeads, int dHead, int maxSeqLen) {
        if (numLayers <= 0) throw new IllegalArgumentException("numLayers must be positive, got " + numLayers);
        if (numHeads <= 0) throw new IllegalArgumentException("numHeads must be positive, got " + numHeads);
        if (dHead <= 0) throw new IllegalArgumentException("dHead must be positive, got " + dHead);
        if (maxSeqLen <= 0) throw new IllegalArgumentException("maxSeqLen must be positive, got " + maxSeqLen);
        int blocks = (maxSeqLen + KvPool.BLOCK_TOKENS - 1) / KvPool.BLOCK_TOKENS;
        this.pool = new KvPool(ctx, numLayers, numHeads, dHead, blocks, 1, blocks, maxSeqLen);
        this.ownsPool = true;
        this.maxSeqLen = maxSeqLen;
        this.seq = pool.seqAlloc();
    }

    /** The reference's constructor signature: device 0, private pool. IllegalStateException when no GPU is usable. */
    public KvCacheGpu(int numLayers, int numHeads, int dHead, int maxSeqLen) {
        this(requireGpu(), numLayers, numHeads, dHead, maxSeqLen);
    }

    private static B200Context requireGpu() {
        if (!B200Context.isGpuAvailable()) throw new IllegalStateException("GPU not available for KvCacheGpu");
        return B200Context.shared();
    }

    public KvCacheGpu(KvPool pool, int maxSeqLen) {
        if (maxSeqLen <= 0 || maxSeqLen > pool.maxBlocksPerSeq * KvPool.BLOCK_TOKENS)
            throw new IllegalArgumentException("maxSeqLen must be in [1, " + pool.maxBlocksPerSeq * KvPool.BLOCK_TOKENS + "], got " + maxSeqLen);
        this.pool = pool;
        this.ownsPool = false;
        this.maxSeqLen = maxSeqLen;
        this.seq = pool.seqAlloc();
    }

    public KvPool pool() {
        return pool;
    }

    /** Sequence slot inside the pool (what the batched forward calls take). */
    public int seq() {
        return seq;
    }

    private int checkLayer(int layer) {
        if (layer < 0 || layer >= pool.layers)
            throw new IndexOutOfBoundsException("layer " + layer + " out of range [0, " + pool.layers + ")");
        return layer;
    }

    private float[] plane(int layer, boolean wantK) {
        checkLayer(layer);
        B200Context ctx = pool.context();
        long n = (long) pool.heads * maxSeqLen * pool.dHead;
        long kd = ctx.devAlloc(4 * n), vd = ctx.devAlloc(4 * n);
        try {
            pool.gather(layer, seq, length(), maxSeqLen, kd, vd);
            float[] out = new float[(int) n];
            ctx.copyToHost(out, wantK ? kd : vd, (int) n);
            return out;
        } finally {
            ctx.devFree(kd);
            ctx.devFree(vd);
        }
    }

    /** fp32 [numHeads, maxSeqLen, dHead] copy of the layer's keys (post-RoPE, as stored). */
    public float[] getK(int layer) {
        return plane(layer, true);
    }

    public float[] getV(int layer) {
        return plane(layer, false);
    }

    public int length() {
        return pool.length(seq);
    }

    public void setLength(int len) {
        if (len < 0 || len > maxSeqLen) throw new IllegalArgumentException("len must be in [0, " + maxSeqLen + "], got " + len);
        if (len > 0) pool.reserve(seq, len);
        pool.setLength(seq, len);
    }

    public int maxSeqLen() {
        return maxSeqLen;
    }

    public int remainingCapacity() {
        return maxSeqLen - length();
    }

    public boolean isFull() {
        return length() >= maxSeqLen;
    }

    public void clear() {
        pool.clear(seq, true);
    }

    public int numLayers() {
        return pool.layers;
    }

    @Override
    public String toString() {
        return String.format("KvCacheGpu{paged, layers=%d, maxSeqLen=%d, len=%d, seq=%d, closed=%b}", pool.layers, maxSeqLen,
                closed ? 0 : length(), seq, closed);
    }

    /** Idempotent. */
    @Override
    public void close() {
        if (closed) return;
        closed = true;
        if (ownsPool) pool.close();
        else pool.seqFree(seq);
    }
}
