"""Host-side mirror of the reference's ``GPTModel`` KV entry points over the C ABI.

Method names follow src/main/java/com/veles/llm/jgpt/model/GPTModel.java: ``forwardPrefill`` (:1525-1536),
``forwardDecode`` (:1545-1556), ``generateGpuKv`` (:1908), ``loadWeights`` (:1944), with the error contract of
model/GptKvForward.java (ValueError = IllegalArgumentException, RuntimeError = IllegalStateException).
Token ids are int32 arrays here (the reference carries them as floats inside ``Tensor``).
"""
from __future__ import annotations

import ctypes as C
import os

import numpy as np

from . import binding as B
from .kv_cache import KvCacheGpu, KvPool
from .runtime import Context


class GPTModel:
    def __init__(self, ctx: Context, vocabSize, maxSeqLen, dModel, numHeads, numLayers, dIntermediate, rmsNormEps=1e-5,
                 maxRows=None):
        self.ctx, self._lib = ctx, ctx._lib
        self.vocabSize, self.maxSeqLen, self.dModel = vocabSize, maxSeqLen, dModel
        self.numHeads, self.numLayers, self.dIntermediate = numHeads, numLayers, dIntermediate
        self.maxRows = maxRows or maxSeqLen
        h = C.c_uint64()
        B.check(self._lib.jgpt_model_create(ctx.handle, vocabSize, maxSeqLen, dModel, numHeads, numLayers, dIntermediate,
                                            rmsNormEps, self.maxRows, C.byref(h)))
        self.handle = h.value

    # ---- weights -------------------------------------------------------------------------------
    def numTensors(self) -> int:
        n = C.c_int32()
        B.check(self._lib.jgpt_model_num_tensors(self.handle, C.byref(n)))
        return n.value

    def setParameters(self, tensors):
        """Tensors in ``getParameters()`` order: tok, pos, per layer Wq,Wk,Wv,Wo,W1,W2,W3,norm1,norm2, normFinal, lmHead."""
        tensors = list(tensors)
        if len(tensors) != self.numTensors():
            raise ValueError(f"expected {self.numTensors()} tensors, got {len(tensors)}")
        for i, t in enumerate(tensors):
            t = np.ascontiguousarray(t, np.float32)
            B.check(self._lib.jgpt_model_set_tensor(self.handle, i, t.ctypes.data, t.size))

    def loadWeights(self, path):
        B.check(self._lib.jgpt_model_load_weights(self.handle, os.fsencode(path)))

    def saveWeights(self, path):
        """Writes the parameters as ``veles.weights.v1`` (what ``GptModelWeightsLoader`` reads)."""
        B.check(self._lib.jgpt_model_save_weights(self.handle, os.fsencode(path)))

    def newPool(self, n_blocks, max_seqs, max_blocks_per_seq=None, max_positions=None) -> KvPool:
        """``max_positions`` > maxSeqLen sizes the RoPE table for the rolling-window mode (positions beyond the context)."""
        mbs = max_blocks_per_seq or -(-self.maxSeqLen // 16)
        return KvPool(self.ctx, self.numLayers, self.numHeads, self.dModel // self.numHeads, n_blocks, max_seqs, mbs,
                      max_positions=max_positions or self.maxSeqLen)

    # ---- forward step --------------------------------------------------------------------------
    def forwardPrefill(self, inputTokens, cache: KvCacheGpu, ropeOffset=0, all_rows=True):
        """ids [1,S] -> logits [S, vocab] (or the last row only).  Sets ``cache.length()`` to S."""
        ids = np.ascontiguousarray(inputTokens, np.int32)
        if ids.ndim == 2:
            if ids.shape[0] != 1:
                raise ValueError("forwardPrefill supports batch_size=1 only")
            ids = ids[0]
        S = ids.size
        if cache.numLayers() != self.numLayers:
            raise ValueError("KvCacheGpu layer count mismatch")
        if S > cache.maxSeqLen():
            raise ValueError(f"seq_len {S} > KvCacheGpu.maxSeqLen {cache.maxSeqLen()}")
        logits = np.empty((S if all_rows else 1, self.vocabSize), np.float32)
        B.check(self._lib.jgpt_forward_prefill(self.handle, cache.pool.handle, cache.seq, ids.ctypes.data, S, ropeOffset,
                                               logits.ctypes.data if all_rows else None,
                                               None if all_rows else logits.ctypes.data, None))
        return logits

    def forwardPrefillBatch(self, pool: KvPool, seqs, prompts, ropeOffsets=None):
        """Several prompts in one call -> (last-row logits [n, vocab], greedy next tokens [n])."""
        n = len(seqs)
        starts = np.zeros(n + 1, np.int32)
        starts[1:] = np.cumsum([len(p) for p in prompts])
        ids = np.ascontiguousarray(np.concatenate([np.asarray(p, np.int32) for p in prompts]), np.int32)
        ro = np.zeros(n, np.int32) if ropeOffsets is None else np.ascontiguousarray(ropeOffsets, np.int32)
        sq = np.ascontiguousarray(seqs, np.int32)
        logits = np.empty((n, self.vocabSize), np.float32)
        nxt = np.empty(n, np.int32)
        B.check(self._lib.jgpt_forward_prefill_batch(self.handle, pool.handle, sq.ctypes.data, starts.ctypes.data, ids.ctypes.data,
                                                     ro.ctypes.data, n, None, logits.ctypes.data, nxt.ctypes.data))
        return logits, nxt

    def forwardDecode(self, inputTokens, cache: KvCacheGpu, cacheLenBefore, ropePosition):
        """ids [1,1] -> logits [vocab].  RuntimeError if ``cache.length() != cacheLenBefore`` or the cache is full."""
        ids = np.ascontiguousarray(inputTokens, np.int32).reshape(-1)
        if ids.size != 1:
            raise ValueError("forwardDecode expects [1, 1] token indices")
        logits, _ = self.forwardDecodeBatch(cache.pool, [cache.seq], ids, [cacheLenBefore], [ropePosition])
        return logits[0]

    def forwardDecodeBatch(self, pool: KvPool, seqs, tokens, cacheLenBefore, ropePositions, want_logits=True):
        """One decode step for n independent sequences -> (logits [n, vocab] or None, greedy next tokens [n])."""
        sq = np.ascontiguousarray(seqs, np.int32)
        tk = np.ascontiguousarray(tokens, np.int32)
        lb = np.ascontiguousarray(cacheLenBefore, np.int32)
        rp = np.ascontiguousarray(ropePositions, np.int32)
        n = sq.size
        logits = np.empty((n, self.vocabSize), np.float32) if want_logits else None
        nxt = np.empty(n, np.int32)
        B.check(self._lib.jgpt_forward_decode(self.handle, pool.handle, sq.ctypes.data, tk.ctypes.data, lb.ctypes.data,
                                              rp.ctypes.data, n, logits.ctypes.data if want_logits else None, nxt.ctypes.data))
        return logits, nxt

    def forwardDecodeSampleBatch(self, pool: KvPool, seqs, tokens, cacheLenBefore, ropePositions, temperature, topK, u01):
        """One decode step + ``sampleNextToken(logits, temperature, topK)`` per row, sampled on the device with the
        uniform draws ``u01`` -> next tokens [n].  Same token as the host sampler picks from the same logits and draw."""
        sq = np.ascontiguousarray(seqs, np.int32)
        tk = np.ascontiguousarray(tokens, np.int32)
        lb = np.ascontiguousarray(cacheLenBefore, np.int32)
        rp = np.ascontiguousarray(ropePositions, np.int32)
        u = np.ascontiguousarray(u01, np.float32)
        n = sq.size
        if u.size != n:
            raise ValueError("one uniform draw per row")
        nxt = np.empty(n, np.int32)
        B.check(self._lib.jgpt_forward_decode_sample(self.handle, pool.handle, sq.ctypes.data, tk.ctypes.data, lb.ctypes.data,
                                                     rp.ctypes.data, n, float(temperature), int(topK), u.ctypes.data, nxt.ctypes.data))
        return nxt

    # ---- generation ----------------------------------------------------------------------------
    def generateGpuKv(self, inputTokens, maxNewTokens, temperature=0.0, topK=0, pool: KvPool | None = None, rng=None):
        """Returns ids [S + maxNewTokens]: prompt kept, zero tail after an early stop on sampled id 0
        (model/GptAutoregressiveGenerator.java:108-206).  Greedy runs entirely inside the library; with a
        temperature the loop runs here and draws the uniform numbers from ``rng`` (default: numpy default_rng())."""
        prompt = np.ascontiguousarray(inputTokens, np.int32).reshape(-1)
        own = pool is None
        if own:
            pool = self.newPool(-(-self.maxSeqLen // 16), 1)
        try:
            if temperature <= 0:
                out = np.zeros(prompt.size + maxNewTokens, np.int32)
                n = C.c_int32()
                B.check(self._lib.jgpt_generate_greedy(self.handle, pool.handle, prompt.ctypes.data, prompt.size, maxNewTokens,
                                                       out.ctypes.data, C.byref(n)))
                return out
            return self._generate_sampled(pool, prompt, maxNewTokens, temperature, topK, rng or np.random.default_rng())
        finally:
            if own:
                pool.close()

    def generateGpuKvRolling(self, inputTokens, maxNewTokens, pool: KvPool):
        """Greedy generation with the block-granular rolling window instead of the clear-and-re-prefill: when the
        context is full the oldest KV block is dropped and decoding continues.  ``pool`` must have been made with
        ``max_positions >= len(prompt) + maxNewTokens - 1``.  Returns ids [S + maxNewTokens]."""
        prompt = np.ascontiguousarray(inputTokens, np.int32).reshape(-1)
        out = np.zeros(prompt.size + maxNewTokens, np.int32)
        n = C.c_int32()
        B.check(self._lib.jgpt_generate_greedy_rolling(self.handle, pool.handle, prompt.ctypes.data, prompt.size, maxNewTokens,
                                                       out.ctypes.data, C.byref(n)))
        return out

    def sampleNextToken(self, logits, temperature, topK, u01) -> int:
        lg = np.ascontiguousarray(logits, np.float32)
        t = C.c_int32()
        B.check(self._lib.jgpt_sample_next_token(lg.ctypes.data, lg.size, temperature, topK, u01, C.byref(t)))
        return t.value

    def _generate_sampled(self, pool, prompt, max_new, temperature, top_k, rng):
        S = prompt.size
        out = np.zeros(S + max_new, np.int32)
        out[:S] = prompt
        if max_new == 0:
            return out
        cache = KvCacheGpu(self.numLayers, self.numHeads, self.dModel // self.numHeads, self.maxSeqLen, pool=pool)
        try:
            logits = self.forwardPrefill(prompt, cache, 0, all_rows=False)[0]
            tok = self.sampleNextToken(logits, temperature, top_k, float(rng.random()))
            out[S] = tok
            for j in range(1, max_new):
                if tok == 0:
                    break
                cur = S + j
                if cur > self.maxSeqLen:
                    start = cur - self.maxSeqLen
                    ln = self.maxSeqLen - start
                    if ln <= 0:
                        raise RuntimeError(f"sliding window: startIdx={start} maxSeqLen={self.maxSeqLen}")
                    pool.clear(cache.seq, zero_fill=False)
                    logits = self.forwardPrefill(out[start:start + ln], cache, start, all_rows=False)[0]
                    tok = self.sampleNextToken(logits, temperature, top_k, float(rng.random()))
                else:  # the decode step samples on the device: no logits come back
                    tok = int(self.forwardDecodeSampleBatch(pool, [cache.seq], out[cur - 1:cur], [cache.length()], [cur - 1],
                                                            temperature, top_k, [np.float32(rng.random())])[0])
                out[cur] = tok
            return out
        finally:
            cache.close()

    def close(self):
        if self.handle:
            self._lib.jgpt_model_destroy(self.handle)
            self.handle = 0
