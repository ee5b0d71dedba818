package com.veles.llm.jgpt.b200;

import static com.veles.llm.jgpt.b200.B200Status.check;
import static java.lang.foreign.ValueLayout.JAVA_FLOAT;
import static java.lang.foreign.ValueLayout.JAVA_INT;
import static java.lang.foreign.ValueLayout.JAVA_LONG;

import java.lang.foreign.Arena;
import java.lang.foreign.MemorySegment;

/**
 * Device-resident weights and step workspace of one decoder-only model: the native side of what the reference's
 * {@code GPTModel} does on its KV path (GPTModel.java:1525-1556, 1894-1910, 1944).  A {@code GPTModel} that is
 * {@code gpuResident} would own one of these and hand its parameters over once ({@link #setParameter} in
 * {@code getParameters()} order, or {@link #loadWeights} for a {@code veles.weights.v1} file); afterwards a forward
 * step is ONE native call (token ids in, logits or sampled ids out), not one call per tensor op.
 */
public final class B200Model implements AutoCloseable {
    private final B200Context ctx;
    private long handle;
    public final int vocabSize, maxSeqLen, dModel, numHeads, numLayers, dIntermediate, maxRows;

    public B200Model(B200Context ctx, int vocabSize, int maxSeqLen, int dModel, int numHeads, int numLayers, int dIntermediate,
            float rmsNormEps, int maxRows) {
        this.ctx = ctx;
        this.vocabSize = vocabSize;
        this.maxSeqLen = maxSeqLen;
        this.dModel = dModel;
        this.numHeads = numHeads;
        this.numLayers = numLayers;
        this.dIntermediate = dIntermediate;
        this.maxRows = maxRows;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_LONG);
            check(JgptB200.modelCreate(ctx.handle(), vocabSize, maxSeqLen, dModel, numHeads, numLayers, dIntermediate, rmsNormEps, maxRows, out));
            handle = out.get(JAVA_LONG, 0);
        }
    }

    public long handle() {
        if (handle == 0) throw new IllegalStateException("model is closed");
        return handle;
    }

    public B200Context context() {
        return ctx;
    }

    public int numTensors() {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT);
            check(JgptB200.modelNumTensors(handle(), out));
            return out.get(JAVA_INT, 0);
        }
    }

    /** Tensor {@code idx} in {@code getParameters()} order: tok, pos, per layer Wq,Wk,Wv,Wo,W1,W2,W3,norm1,norm2, normFinal, lmHead. */
    public void setParameter(int idx, float[] rowMajor) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment h = a.allocateFrom(JAVA_FLOAT, rowMajor);
            check(JgptB200.modelSetTensor(handle(), idx, h, rowMajor.length));
        }
    }

    /** {@code GPTModel.loadWeights(path)} for the {@code veles.weights.v1} format (model/GptModelWeightsLoader.java:58-81). */
    public void loadWeights(String path) {
        try (Arena a = Arena.ofConfined()) {
            check(JgptB200.modelLoadWeights(handle(), a.allocateFrom(path)));
        }
    }

    public KvPool newPool(int nBlocks, int maxSeqs) {
        return new KvPool(ctx, numLayers, numHeads, dModel / numHeads, nBlocks, maxSeqs, (maxSeqLen + 15) / 16, maxSeqLen);
    }

    /** Prefill of one prompt; returns logits [S * vocab] (all rows, as the reference does) and sets the cache length to S. */
    public float[] forwardPrefill(int[] ids, KvCacheGpu cache, int ropeOffset) {
        int S = ids.length;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment in = a.allocateFrom(JAVA_INT, ids), out = a.allocate(JAVA_FLOAT, (long) S * vocabSize);
            check(JgptB200.forwardPrefill(handle(), cache.pool().handle(), cache.seq(), in, S, ropeOffset, out, MemorySegment.NULL, MemorySegment.NULL));
            return out.toArray(JAVA_FLOAT);
        }
    }

    /**
     * One decode step for n independent sequences (additive overload of the reference's batch-1 call): logits
     * [n * vocab] when {@code wantLogits}, and the greedy next tokens in {@code nextOut}.
     */
    public float[] forwardDecode(KvPool pool, int[] seqs, int[] ids, int[] cacheLenBefore, int[] ropePositions, boolean wantLogits, int[] nextOut) {
        int n = seqs.length;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment sq = a.allocateFrom(JAVA_INT, seqs), tk = a.allocateFrom(JAVA_INT, ids), lb = a.allocateFrom(JAVA_INT, cacheLenBefore),
                    rp = a.allocateFrom(JAVA_INT, ropePositions), nx = a.allocate(JAVA_INT, n);
            MemorySegment lg = wantLogits ? a.allocate(JAVA_FLOAT, (long) n * vocabSize) : MemorySegment.NULL;
            check(JgptB200.forwardDecode(handle(), pool.handle(), sq, tk, lb, rp, n, lg, nx));
            if (nextOut != null) MemorySegment.copy(nx, JAVA_INT, 0, nextOut, 0, n);
            return wantLogits ? lg.toArray(JAVA_FLOAT) : null;
        }
    }

    /** The same with {@code sampleNextToken(logits, temperature, topK)} done on the device from the given uniform draws. */
    public int[] forwardDecodeSample(KvPool pool, int[] seqs, int[] ids, int[] cacheLenBefore, int[] ropePositions, float temperature, int topK,
            float[] u01) {
        int n = seqs.length;
        try (Arena a = Arena.ofConfined()) {
            MemorySegment nx = a.allocate(JAVA_INT, n);
            check(JgptB200.forwardDecodeSample(handle(), pool.handle(), a.allocateFrom(JAVA_INT, seqs), a.allocateFrom(JAVA_INT, ids),
                    a.allocateFrom(JAVA_INT, cacheLenBefore), a.allocateFrom(JAVA_INT, ropePositions), n, temperature, topK,
                    a.allocateFrom(JAVA_FLOAT, u01), nx));
            return nx.toArray(JAVA_INT);
        }
    }

    /** {@code sampleNextToken} on host logits with the caller's uniform draw (GptAutoregressiveGenerator.java:208-286). */
    public static int sampleNextToken(float[] logits, float temperature, int topK, float u01) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT);
            check(JgptB200.sampleNextToken(a.allocateFrom(JAVA_FLOAT, logits), logits.length, temperature, topK, u01, out));
            return out.get(JAVA_INT, 0);
        }
    }

    /**
     * {@code generateGpuKv(ids, maxNew, temperature <= 0, topK)}: the whole greedy loop inside the library (stop on
     * sampled id 0, zero tail, the reference's sliding-window re-prefill once the context is full).  Returns
     * [S + maxNew] ids.
     */
    public int[] generateGreedy(KvPool pool, int[] prompt, int maxNewTokens) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT, prompt.length + maxNewTokens), n = a.allocate(JAVA_INT);
            check(JgptB200.generateGreedy(handle(), pool.handle(), a.allocateFrom(JAVA_INT, prompt), prompt.length, maxNewTokens, out, n));
            return out.toArray(JAVA_INT);
        }
    }

    /**
     * Greedy generation with the block-granular rolling window instead of the reference's clear-and-re-prefill.  The pool
     * must have a RoPE table of at least {@code prompt.length + maxNewTokens - 1} positions.  Not an exact-parity mode once
     * the context has filled.
     */
    public int[] generateGreedyRolling(KvPool pool, int[] prompt, int maxNewTokens) {
        try (Arena a = Arena.ofConfined()) {
            MemorySegment out = a.allocate(JAVA_INT, prompt.length + maxNewTokens), n = a.allocate(JAVA_INT);
            check(JgptB200.generateGreedyRolling(handle(), pool.handle(), a.allocateFrom(JAVA_INT, prompt), prompt.length, maxNewTokens, out, n));
            return out.toArray(JAVA_INT);
        }
    }

    @Override
    public void close() {
        if (handle != 0) {
            JgptB200.modelDestroy(handle);
            handle = 0;
        }
    }
}
