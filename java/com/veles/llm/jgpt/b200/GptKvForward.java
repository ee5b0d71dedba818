package com.veles.llm.jgpt.b200;

import com.veles.llm.jgpt.core.Tensor;
import java.util.concurrent.ThreadLocalRandom;

/**
 * The forward-step calls of the reference's {@code model.GptKvForward} (model/GptKvForward.java:46-90, 129-170) and the
 * generation loop of {@code GptAutoregressiveGenerator.generateGpuKv} (:108-206) over the native model: same argument
 * meaning, same shapes ({@code Tensor} ids carried as floats, logits {@code [1,S,V]} / {@code [1,1,V]}), same exceptions in
 * the same order.  {@code GPTModel.forwardPrefill / forwardDecode / generateGpuKv} delegate here when the B200 path is on.
 */
public final class GptKvForward {
    private GptKvForward() {}

    private static int[] idsOf(Tensor t, int vocab) {
        float[] f = t.internalBuffer();
        int[] ids = new int[t.size()];
        for (int i = 0; i < ids.length; i++) {
            int id = (int) f[i];
            if (id < 0 || id >= vocab) throw new IllegalArgumentException("token id " + id + " outside [0, " + vocab + ")");
            ids[i] = id;
        }
        return ids;
    }

    /** ids [1,S] -> logits [1,S,V]; afterwards {@code cache.length() == S}. */
    public static Tensor forwardPrefillGpu(B200Model m, Tensor inputTokens, KvCacheGpu cache, int ropeOffset) {
        int[] shape = inputTokens.getShape();
        if (shape.length != 2 || shape[0] != 1) throw new IllegalArgumentException("forwardPrefill supports batch_size=1 only");
        int S = shape[1];
        if (S > m.maxSeqLen) throw new IllegalArgumentException("seq_len " + S + " > max_seq_len " + m.maxSeqLen);
        if (cache.numLayers() != m.numLayers) throw new IllegalArgumentException("KvCacheGpu layer count mismatch");
        if (S > cache.maxSeqLen()) throw new IllegalArgumentException("seq_len " + S + " > KvCacheGpu.maxSeqLen " + cache.maxSeqLen());
        float[] logits = m.forwardPrefill(idsOf(inputTokens, m.vocabSize), cache, ropeOffset);
        return Tensor.wrap(logits, new int[] {1, S, m.vocabSize});
    }

    /** ids [1,1] -> logits [1,1,V]; IllegalStateException unless {@code cache.length() == cacheLenBefore} and the cache has room. */
    public static Tensor forwardDecodeGpu(B200Model m, Tensor inputTokens, KvCacheGpu cache, int cacheLenBefore, int ropePosition) {
        int[] shape = inputTokens.getShape();
        if (shape.length != 2 || shape[0] != 1 || shape[1] != 1) throw new IllegalArgumentException("forwardDecode expects [1, 1] token indices");
        if (cache.length() != cacheLenBefore)
            throw new IllegalStateException("KV cache length " + cache.length() + " != cacheLenBefore " + cacheLenBefore);
        if (cacheLenBefore >= cache.maxSeqLen()) throw new IllegalStateException("KV cache is full");
        float[] logits = m.forwardDecode(cache.pool(), new int[] {cache.seq()}, idsOf(inputTokens, m.vocabSize), new int[] {cacheLenBefore},
                new int[] {ropePosition}, true, null);
        return Tensor.wrap(logits, new int[] {1, 1, m.vocabSize});
    }

    /** Batched decode (additive overload): ids [B,1] and per-sequence caches of one pool -> logits [B,1,V]. */
    public static Tensor forwardDecodeGpu(B200Model m, Tensor inputTokens, KvCacheGpu[] caches, int[] cacheLenBefore, int[] ropePositions) {
        int B = caches.length;
        int[] seqs = new int[B];
        for (int i = 0; i < B; i++) {
            if (caches[i].pool() != caches[0].pool()) throw new IllegalArgumentException("all caches of one step must share a pool");
            if (caches[i].length() != cacheLenBefore[i])
                throw new IllegalStateException("KV cache length " + caches[i].length() + " != cacheLenBefore " + cacheLenBefore[i]);
            seqs[i] = caches[i].seq();
        }
        float[] logits = m.forwardDecode(caches[0].pool(), seqs, idsOf(inputTokens, m.vocabSize), cacheLenBefore, ropePositions, true, null);
        return Tensor.wrap(logits, new int[] {B, 1, m.vocabSize});
    }

    /**
     * {@code GPTModel.generateGpuKv(ids [1,S], maxNew, temperature, topK)} -> Tensor [1, S + maxNew], prompt kept, zero tail
     * after an early stop on sampled id 0.  Greedy runs inside the library; with a temperature the loop runs here, the
     * decode step samples on the device and the uniform numbers come from ThreadLocalRandom as in the reference
     * ({@code (float) nextDouble()}).
     */
    public static Tensor generateGpuKv(B200Model m, Tensor inputTokens, int maxNewTokens, float temperature, int topK) {
        int[] shape = inputTokens.getShape();
        if (shape.length != 2 || shape[0] != 1) throw new IllegalArgumentException("generate supports batch_size=1 only");
        int[] prompt = idsOf(inputTokens, m.vocabSize);
        int S = prompt.length;
        float[] out = new float[S + maxNewTokens];
        for (int i = 0; i < S; i++) out[i] = prompt[i];
        if (maxNewTokens == 0) return Tensor.wrap(out, new int[] {1, S});
        try (KvPool pool = m.newPool((m.maxSeqLen + 15) / 16, 1)) {
            if (temperature <= 0f) {
                int[] ids = m.generateGreedy(pool, prompt, maxNewTokens);
                for (int i = 0; i < ids.length; i++) out[i] = ids[i];
                return Tensor.wrap(out, new int[] {1, S + maxNewTokens});
            }
            try (KvCacheGpu cache = new KvCacheGpu(pool, m.maxSeqLen)) {
                ThreadLocalRandom rnd = ThreadLocalRandom.current();
                float[] logits = m.forwardPrefill(prompt, cache, 0);
                float[] last = java.util.Arrays.copyOfRange(logits, (S - 1) * m.vocabSize, S * m.vocabSize);
                int tok = B200Model.sampleNextToken(last, temperature, topK, (float) rnd.nextDouble());
                out[S] = tok;
                for (int j = 1; j < maxNewTokens && tok != 0; j++) {
                    int cur = S + j;
                    if (cur > m.maxSeqLen) { // the reference's sliding window: clear and re-prefill out[start, maxSeqLen)
                        int start = cur - m.maxSeqLen, len = m.maxSeqLen - start;
                        if (len <= 0) throw new IllegalStateException("sliding window: startIdx=" + start + " maxSeqLen=" + m.maxSeqLen);
                        pool.clear(cache.seq(), false);
                        int[] window = new int[len];
                        for (int i = 0; i < len; i++) window[i] = (int) out[start + i];
                        float[] lg = m.forwardPrefill(window, cache, start);
                        last = java.util.Arrays.copyOfRange(lg, (len - 1) * m.vocabSize, len * m.vocabSize);
                        tok = B200Model.sampleNextToken(last, temperature, topK, (float) rnd.nextDouble());
                    } else {
                        tok = m.forwardDecodeSample(pool, new int[] {cache.seq()}, new int[] {(int) out[cur - 1]}, new int[] {cache.length()},
                                new int[] {cur - 1}, temperature, topK, new float[] {(float) rnd.nextDouble()})[0];
                    }
                    out[cur] = tok;
                }
            }
        }
        return Tensor.wrap(out, new int[] {1, S + maxNewTokens});
    }
}
