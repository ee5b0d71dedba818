"""The CUDA path against the committed fixtures (tests/golden/oracle_vectors.npz), through the C ABI:
logits of the KvCacheTest geometry, the sliding-window greedy streams, fused append + decode attention,
and the allocator trace.  No oracle code runs here."""
import os

import numpy as np
import pytest

from jgpt_b200 import GPTModel, KvCacheGpu, KvPool

pytestmark = pytest.mark.gpu
GOLD = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "oracle_vectors.npz"))


def _random_parameters(vocab, max_seq, d, layers, dff, seed, std):
    """oracle.Model.init_random restated: every matrix N(0, std) from default_rng(seed) in file order, gammas 1."""
    rng = np.random.default_rng(seed)
    shapes = [(vocab, d), (max_seq, d)]
    for _ in range(layers):
        shapes += [(d, d)] * 4 + [(d, dff), (dff, d), (d, dff), (d,), (d,)]
    shapes += [(d,), (d, vocab)]
    return [rng.normal(0.0, std, size=s).astype(np.float32) if len(s) == 2 else np.ones(s, np.float32) for s in shapes]


def test_tiny_model_logits_match_the_frozen_vectors(ctx):
    gm = GPTModel(ctx, 64, 32, 32, 4, 2, 64, rmsNormEps=1e-6)
    gm.setParameters(_random_parameters(64, 32, 32, 2, 64, seed=3, std=0.2))
    cache = KvCacheGpu(2, 4, 8, 32, ctx=ctx)
    try:
        got = gm.forwardPrefill(GOLD["tiny_ids"], cache, 0)
        assert np.abs(got - GOLD["tiny_prefill_logits"]).max() < 5e-4
        tok = 11
        for step in range(3):
            lb = cache.length()
            lg = gm.forwardDecode([tok], cache, lb, lb)
            assert np.abs(lg - GOLD["tiny_decode_logits"][step]).max() < 5e-4
            tok = int(np.argmax(GOLD["tiny_decode_logits"][step]))
        k1 = cache.getK(1).to_host()[:, :19]
        ulp = np.maximum(np.abs(GOLD["tiny_k_layer1"]), 2.0 ** -14) * 2.0 ** -10
        assert (np.abs(k1 - GOLD["tiny_k_layer1"]) <= ulp + 2e-4).all()
    finally:
        cache.close(), gm.close()


def test_sliding_window_greedy_streams_match_the_frozen_vectors(ctx):
    gm = GPTModel(ctx, 64, 12, 32, 4, 2, 64, rmsNormEps=1e-6)
    gm.setParameters(_random_parameters(64, 12, 32, 2, 64, seed=5, std=0.3))
    try:
        for name in ("a", "b"):
            want = GOLD[f"greedy_{name}"]
            assert np.array_equal(gm.generateGpuKv(want[:5], 12), want), name
    finally:
        gm.close()


def test_fused_append_decode_attention_matches_the_frozen_vectors(ctx):
    H, Dh, MS = 2, 16, 48
    kc, vc, lens = GOLD["attn_kc"], GOLD["attn_vc"], GOLD["attn_lens"]
    pool = KvPool(ctx, 1, H, Dh, 9, 3, 3, max_positions=64)
    try:
        seqs = []
        for i in range(3):
            s = pool.seq_alloc()
            pool.reserve(s, MS)
            seqs.append(s)
            L = int(lens[i])
            if L:  # load the cached prefix: the fixture holds fp16-exact values, RoPE at position 0 is the identity
                rows = np.ascontiguousarray(kc[i, :, :L].transpose(1, 0, 2).reshape(L, H * Dh))
                vrows = np.ascontiguousarray(vc[i, :, :L].transpose(1, 0, 2).reshape(L, H * Dh))
                ids = ctx.from_host(np.full(L, s, np.int32))
                pool.append(0, ctx.from_host(rows), ctx.from_host(vrows), ids, ctx.from_host(np.arange(L, dtype=np.int32)),
                            ctx.from_host(np.zeros(L, np.int32)), L)
        out = pool.attn_decode_append_host(0, 1, GOLD["attn_q"], GOLD["attn_k"], GOLD["attn_v"], seqs, GOLD["attn_rope"], lens + 1)
        assert np.abs(out - GOLD["attn_out"]).max() < 2e-5
        for i in range(3):
            kd, vd = ctx.alloc((H, MS, Dh)), ctx.alloc((H, MS, Dh))
            pool.gather(0, seqs[i], int(lens[i]) + 1, MS, kd, vd)
            L1 = int(lens[i]) + 1
            assert np.array_equal(kd.to_host()[:, :L1], GOLD["attn_kc_after"][i, :, :L1])
            assert np.array_equal(vd.to_host()[:, :L1], GOLD["attn_vc_after"][i, :, :L1])
    finally:
        pool.close()


def test_allocator_trace_matches_the_frozen_vectors(ctx):
    tr = [[int(x) for x in row if x >= 0] for row in GOLD["alloc_trace"]]
    pool = KvPool(ctx, 1, 2, 16, 12, 4, 6)
    try:
        s0, s1 = pool.seq_alloc(), pool.seq_alloc()
        pool.reserve(s0, 40), pool.reserve(s1, 16), pool.reserve(s0, 49)
        assert pool.block_table(s0).tolist() == tr[0] and pool.block_table(s1).tolist() == tr[1]
        pool.mark_evictable(s0), pool.set_length(s1, 16), pool.mark_evictable(s1)
        assert pool.evict_lru(10) == tr[2]
        s2 = pool.seq_alloc()
        pool.reserve(s2, 96)
        assert pool.block_table(s2).tolist() == tr[3] and pool.block_table(s2, device=True).tolist() == tr[3]
        assert pool.free_blocks() == len(tr[4])
    finally:
        pool.close()
