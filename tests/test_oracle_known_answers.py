"""Pins the CPU oracle to what the reference's own tests state for this path.

The reference ships no golden vectors; what it does hold are literal known-answer cases
(src/test/java/com/veles/llm/jgpt/ops/TensorOpsTest.java:70-196) and path-vs-path invariants
(src/test/java/com/veles/llm/jgpt/model/KvCacheTest.java:14-118,
 src/test/java/com/veles/llm/jgpt/model/GreedyGenerateParityTest.java:54-87).  Both are replayed here.
"""
import math
import os

import numpy as np
import pytest

import oracle as O


# ---- TensorOpsTest literals ---------------------------------------------------------------------
def test_rmsnorm_known_answer():  # TensorOpsTest.testRmsNorm :97-109
    out = O.rmsnorm(np.array([3.0, 4.0]), np.array([1.0, 1.0]), 1e-6)
    rms = math.sqrt((9 + 16) / 2)
    assert abs(out[0] - 3 / rms) < 1e-5 and abs(out[1] - 4 / rms) < 1e-5


def test_matmul_known_answer():  # TensorOpsTest.testMatmul :113-123
    c = O.matmul(np.array([[1, 2, 3], [4, 5, 6.0]]), np.array([[7, 8], [9, 10], [11, 12.0]]))
    assert c.tolist() == [[58.0, 64.0], [139.0, 154.0]]


def test_sigmoid_known_answers():  # TensorOpsTest.testSigmoid / testSigmoidEdgeCases :70-83
    s = O.sigmoid(np.array([0.0, 20.0, -20.0, 25.0, -25.0]))
    assert abs(s[0] - 0.5) < 1e-3 and s[1] == 1.0 and s[2] == 0.0 and s[3] == 1.0 and s[4] == 0.0


def test_split_concat_roundtrip():  # TensorOpsTest.testSplitConcatHeadsRoundtrip :156-167
    x = np.array([1, 2, 3, 4, 5, 6, 7, 8], np.float32).reshape(1, 2, 4)
    sp = O.split_heads(x, 2)
    assert sp.shape == (1, 2, 2, 2) and sp[0, 1, 0].tolist() == [3.0, 4.0]
    assert np.array_equal(O.concat_heads(sp), x)


def test_softmax_rows_sum_to_one():  # TensorOpsTest.testSoftmaxLastDim :169-196
    p = O.softmax_last_dim(np.array([[[1, 2, 3], [4, 5, 6.0]]]))
    assert np.allclose(p.sum(-1), 1.0, atol=1e-5) and (p >= 0).all() and (p <= 1).all()
    e = np.exp(np.array([1, 2, 3.0]) - 3)
    assert np.allclose(p[0, 0], e / e.sum(), atol=1e-6)
    # long rows take the block kernel's 1/max(sum, 1e-12) form; same values
    x = np.random.default_rng(0).standard_normal((3, 200)).astype(np.float32)
    ref = np.exp(x - x.max(-1, keepdims=True))
    assert np.allclose(O.softmax_last_dim(x), ref / ref.sum(-1, keepdims=True), atol=1e-6)


def test_rope_is_the_interleaved_pair_rotation():
    """rope_4d_kernel (jgpt_cuda_extra_kernels_launches.inl:1127-1159) against float64 arithmetic."""
    rng = np.random.default_rng(1)
    x = rng.standard_normal((1, 3, 5, 16)).astype(np.float32)
    y = O.rope_4d(x, pos_base_offset=2)
    for i in range(5):
        for j in range(8):
            th = np.float32(i + 2) / np.float32(10000.0) ** np.float32(2.0 * j / 16)
            c, s = math.cos(float(th)), math.sin(float(th))
            assert np.allclose(y[0, :, i, 2 * j], x[0, :, i, 2 * j] * c - x[0, :, i, 2 * j + 1] * s, atol=2e-6)
            assert np.allclose(y[0, :, i, 2 * j + 1], x[0, :, i, 2 * j] * s + x[0, :, i, 2 * j + 1] * c, atol=2e-6)
    # explicit positions override the offset (decode passes {ropePosition})
    y2 = O.rope_4d(x[:, :, :1], positions=[4])
    assert np.array_equal(y2[0, :, 0], O.rope_4d(x, pos_base_offset=4)[0, :, 0] * 0 + O.rope_4d(
        np.repeat(x[:, :, :1], 5, axis=2), pos_base_offset=4)[0, :, 0])
    assert np.array_equal(O.rope_4d(x, pos_base_offset=0)[0, :, 0], x[0, :, 0])  # position 0 = identity


def test_round_fp16_is_rne_and_matches_c():
    x = np.array([1.0 + 2 ** -11, 1.0 + 3 * 2 ** -11, 65504.0, 1e-8, -0.1], np.float32)
    want = x.astype(np.float16).astype(np.float32)
    got = np.array([O.lib().og_round_fp16(float(v)) for v in x], np.float32)
    assert np.array_equal(got, want) and got[0] == 1.0 and got[1] == np.float32(1.0 + 2 ** -9)


# ---- AttentionForwardGpuTest.referenceForward: the reference's own scalar attention loops ----------
def test_causal_attention_against_float64_loops():
    rng = np.random.default_rng(55)
    H, S, Dh, scale = 3, 20, 16, 0.19
    q, k, v = (rng.uniform(-1, 1, (H, S, Dh)).astype(np.float32) for _ in range(3))
    out = O.attn_prefill_causal(q, k, v, scale)
    for h in range(H):
        sc = (q[h].astype(np.float64) @ k[h].astype(np.float64).T) * scale
        sc[np.triu_indices(S, 1)] = -np.inf
        p = np.exp(sc - sc.max(-1, keepdims=True))
        p /= p.sum(-1, keepdims=True)
        assert np.abs(out[h] - p @ v[h].astype(np.float64)).max() < 8e-4  # the reference test's tolerance
    # single-query attention over the prefix equals the last causal row
    last = O.attn_query_one(q[1, S - 1], k[1], v[1], scale)
    assert np.abs(last - out[1, S - 1]).max() < 1e-6


# ---- KvCacheTest invariants ---------------------------------------------------------------------
@pytest.fixture(scope="module")
def tiny():
    m = O.Model(64, 32, 32, 4, 2, 64, eps=1e-6).init_random(seed=3, std=0.2)
    yield m
    m.close()


def test_prefill_matches_forward(tiny):  # KvCacheTest.prefillMatchesForward :14-34 (tol 1e-3)
    ids = np.array([(i + 3) % 64 for i in range(5)], np.int32)
    c = tiny.new_cache()
    assert np.abs(tiny.forward(ids) - tiny.forward_prefill(ids, c)).max() < 1e-3
    assert c.length() == 5


def test_decode_matches_second_token_logits(tiny):  # KvCacheTest.decodeMatchesSecondTokenLogits :36-70
    c = tiny.new_cache()
    tiny.forward_prefill(np.array([7], np.int32), c)
    d = tiny.forward_decode(11, c, 1, 1)
    full = tiny.forward(np.array([7, 11], np.int32))
    assert np.abs(full[1] - d).max() < 1e-3 and c.length() == 2
    with pytest.raises(RuntimeError):  # cache.length() != cacheLenBefore -> IllegalStateException
        tiny.forward_decode(11, c, 1, 2)


def test_cache_contract(tiny):  # KvCacheTest ctor / bounds / length / clear :80-118
    with pytest.raises(ValueError):
        O.KvCache(0, 4, 8, 32)
    c = tiny.new_cache()
    with pytest.raises(ValueError):
        c.set_length(33)
    with pytest.raises(IndexError):
        c.k(2)
    tiny.forward_prefill(np.array([1, 2, 3], np.int32), c)
    assert c.k(0)[:, :3].any() and not c.k(0)[:, 3:].any()
    c.clear()
    assert c.length() == 0 and not c.k(0).any() and not c.v(1).any()
    with pytest.raises(ValueError):  # token id outside the vocabulary -> IllegalArgumentException
        tiny.forward_prefill(np.array([64], np.int32), c)


def test_cache_layout_is_head_major_contiguous(tiny):
    """K is stored after RoPE, V raw, at h*maxSeq*Dh + pos*Dh + j (KvCacheGpu.java:7-8, 36-44)."""
    c = tiny.new_cache()
    ids = np.array([5, 9, 13, 2], np.int32)
    tiny.forward_prefill(ids, c, rope_offset=0)
    t = tiny.tensors()
    x = t[0][ids] + t[1][:4]
    n1 = O.rmsnorm(x, t[2 + 7], tiny.eps)
    k = O.matmul(n1, t[2 + 1]).reshape(1, 4, 32)
    v = O.matmul(n1, t[2 + 2]).reshape(1, 4, 32)
    assert np.array_equal(c.k(0)[:, :4], O.rope_4d(O.split_heads(k, 4))[0])
    assert np.array_equal(c.v(0)[:, :4], O.split_heads(v, 4)[0])


# ---- generation loop ----------------------------------------------------------------------------
def test_greedy_generation_rules():
    """Prompt kept, tail zero after an early stop on id 0, lowest index wins ties, sliding window
    re-prefill of out[cur-maxSeq : maxSeq) (GreedyGenerateParityTest geometry: maxSeq 12, prompt 5, 12 new)."""
    m = O.Model(64, 12, 32, 4, 2, 64, eps=1e-6).init_random(seed=5, std=0.3)
    prompt = np.array([(i * 7 + 3) % 64 for i in range(5)], np.int32)
    out, n = m.generate_greedy(prompt, 12)
    assert out.shape == (17,) and np.array_equal(out[:5], prompt)
    # replay by hand: decode until position 12, then the shrinking-window prefill
    c = m.new_cache()
    logits = m.forward_prefill(prompt, c)
    toks = [int(O.argmax(logits[-1]))]
    for j in range(1, 12):
        cur = 5 + j
        if toks[-1] == 0:
            break
        if cur > 12:
            start = cur - 12
            c.clear()
            seq = np.concatenate([prompt, np.array(toks, np.int32)])
            lg = m.forward_prefill(seq[start:12], c, rope_offset=start)
            toks.append(int(O.argmax(lg[-1])))
        else:
            toks.append(int(O.argmax(m.forward_decode(toks[-1], c, c.length(), cur - 1))))
    assert out[5:5 + len(toks)].tolist() == toks and n == len(toks)
    assert not out[5 + len(toks):].any()
    assert O.argmax(np.array([1.0, 3.0, 3.0, 2.0])) == 1
    m.close()
    # cur >= 2*maxSeq: the window is empty -> IllegalStateException, unless id 0 was sampled before that
    raised = 0
    for seed in range(4):
        m = O.Model(64, 12, 32, 4, 2, 64, eps=1e-6).init_random(seed=seed, std=0.3)
        try:
            out, n = m.generate_greedy(prompt, 30)
            assert n < 19 + 1 and out[5 + n - 1] == 0
        except RuntimeError:
            raised += 1
        m.close()
    assert raised >= 1


def test_sampler_rules():
    lg = np.array([0.1, 2.0, 2.0, -1.0, 1.5], np.float32)
    assert O.sample_next_token(lg, 0.0, 0, 0.5) == 1  # greedy
    assert O.sample_next_token(lg, 1.0, 1, 0.99) == 1  # top-1 keeps the lowest index of the tie
    p = np.exp(lg - lg.max())
    p /= p.sum()
    cdf = np.cumsum(p)
    for u in (0.01, 0.3, 0.6, 0.95):
        assert O.sample_next_token(lg, 1.0, 0, u) == int(np.searchsorted(cdf, u))
    assert O.sample_next_token(lg, 1.0, 2, 0.999) in (1, 2)


def test_weights_file_roundtrip(tmp_path):
    """veles.weights.v1: writeUTF tag, int32 BE count, per tensor rank/dims/BE floats
    (GptModelWeightsLoader.java:58-81)."""
    m = O.Model(20, 8, 16, 2, 1, 24).init_random(seed=9)
    p = os.path.join(tmp_path, "w.bin")
    m.save(p)
    raw = open(p, "rb").read()
    assert raw[:18] == b"\x00\x10veles.weights.v1" and int.from_bytes(raw[18:22], "big") == 13
    assert int.from_bytes(raw[22:26], "big") == 2 and int.from_bytes(raw[26:30], "big") == 20
    assert np.frombuffer(raw[34:38], ">f4")[0] == m.tensors()[0][0, 0]
    m2 = O.Model(20, 8, 16, 2, 1, 24)
    m2.load(p)
    for a, b in zip(m.tensors(), m2.tensors()):
        assert np.array_equal(a, b)
    with pytest.raises(OSError):
        O.Model(20, 8, 16, 2, 2, 24).load(p)


def test_decode_attn_batch_equals_model_attention_core(tiny):
    """The microbenchmark's CPU step is the attention core of forward_decode: same RoPE, append index and softmax."""
    rng = np.random.default_rng(2)
    H, Dh, MS = 4, 8, 32
    kc = rng.standard_normal((2, H, MS, Dh)).astype(np.float32)
    vc = rng.standard_normal((2, H, MS, Dh)).astype(np.float32)
    q, k, v = (rng.standard_normal((2, H * Dh)).astype(np.float32) for _ in range(3))
    lens, rope = np.array([3, 17], np.int32), np.array([5, 17], np.int32)
    kc0, vc0 = kc.copy(), vc.copy()
    out = O.decode_attn_batch(q, k, v, kc, vc, lens, rope, H, Dh, MS, kv_fp16=False)
    for i in range(2):
        kr = O.rope_4d(O.split_heads(k[i].reshape(1, 1, -1), H), positions=[rope[i]])[0, :, 0]
        qr = O.rope_4d(O.split_heads(q[i].reshape(1, 1, -1), H), positions=[rope[i]])[0, :, 0]
        assert np.array_equal(kc[i, :, lens[i]], kr) and np.array_equal(vc[i, :, lens[i]], v[i].reshape(H, Dh))
        kc0[i, :, lens[i]], vc0[i, :, lens[i]] = kr, v[i].reshape(H, Dh)
        for h in range(H):
            want = O.attn_query_one(qr[h], kc0[i, h, :lens[i] + 1], vc0[i, h, :lens[i] + 1], 1 / math.sqrt(Dh))
            assert np.array_equal(out[i, h * Dh:(h + 1) * Dh], want)


def test_rolling_window_specification():
    """The block-granular rolling window (no reference counterpart): until the context first fills it is the ordinary
    generator; afterwards a decode step over the shifted cache equals a step over a cache that was built with only the
    surviving tokens -- same keys (RoPE at their absolute positions), same position rows (position mod maxSeq)."""
    V, MS = 50, 32
    om = O.Model(V, MS, 32, 4, 2, 64, eps=1e-6).init_random(seed=8, std=0.2)
    try:
        prompt = np.array([(i * 3 + 1) % V for i in range(20)], np.int32)
        plain, n_plain = om.generate_greedy(prompt, MS - 20 + 1)
        roll, n_roll = om.generate_greedy_rolling(prompt, MS - 20 + 1)
        assert n_plain == n_roll and np.array_equal(plain, roll)  # nothing dropped yet: identical
        # run past the context: 2 full windows more
        out, n = om.generate_greedy_rolling(prompt, 3 * MS)
        assert n >= 1 and (n == 3 * MS or out[20 + n - 1] == 0)
        # one step by hand: cache of 32 tokens, drop 16, decode at absolute position 32
        c = om.new_cache()
        ids = np.array([(i * 5 + 2) % V for i in range(MS)], np.int32)
        om.forward_prefill(ids, c)
        k_before = c.k(0).copy()
        c.drop_front(16)
        assert c.length() == 16 and np.array_equal(c.k(0)[:, :16], k_before[:, 16:32]) and not c.k(0)[:, 16:].any()
        got = om.forward_decode_rolling(7, c, 16, MS)  # position 32 -> row 0
        assert c.length() == 17
        with pytest.raises(ValueError):
            c.drop_front(18)
        # the same step through the ordinary call is refused: position 32 has no row in the table
        c2 = om.new_cache()
        with pytest.raises(ValueError):
            om.forward_decode(7, c2, 0, MS)
        assert np.isfinite(got).all()
    finally:
        om.close()
    a = O.PagedAllocatorRef(n_blocks=6, block_tokens=16, max_seqs=2, max_blocks_per_seq=4)
    s = a.seq_alloc()
    assert a.reserve(s, 50) and a.tables[s] == [0, 1, 2, 3]
    a.length[s] = 50
    assert a.drop_front(s, 2) and a.tables[s] == [2, 3] and a.length[s] == 18 and a.free[-2:] == [0, 1]
    assert not a.drop_front(s, 2)  # only one full block left in 18 tokens
    assert a.reserve(s, 40) and a.tables[s] == [2, 3, 1]  # the block dropped last comes back first
