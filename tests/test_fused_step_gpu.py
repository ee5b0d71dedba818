"""The decode step of one to four rows as ONE cooperative launch (csrc/decode_fused.cu), and greedy generation with
several steps per launch, against the multi-launch step of the same library (JGPT_B200_FUSED_STEP=0), the CPU oracle
and the allocator specification.

Tolerances: logits of the two step forms within 1e-4 of each other on the same cache payload (both compute fp32 products
with different summation orders: split-TF32 tensor-core tiles against plain FMA chains) and within 2e-3 of the oracle run with the
fp16-rounded cache (over 20 steps the one-ulp differences of appended payloads add up on this toy geometry); K/V payloads within one fp16 ulp
(the fp32 value being rounded differs in its last bits) plus 5e-5 absolute (the projections' own fp32 noise, which a sum that
cancels or RoPE's difference of products leaves standing next to a small result);
greedy token streams identical; block tables and free lists identical."""
import numpy as np
import pytest

import oracle as O
from helpers import exact_prefill
from jgpt_b200 import GPTModel

pytestmark = pytest.mark.gpu
GEOM = (96, 80, 64, 4, 3, 128)  # vocab, max_seq, d_model, heads (d_head 16), layers, d_ff


def _three(ctx, geom, seed, std, monkeypatch):
    """The oracle, a model that takes the fused step, a model that does not."""
    om = O.Model(*geom, eps=1e-5).init_random(seed=seed, std=std)
    with exact_prefill():
        fused = GPTModel(ctx, *geom, rmsNormEps=1e-5, maxRows=256)
        monkeypatch.setenv("JGPT_B200_FUSED_STEP", "0")
        plain = GPTModel(ctx, *geom, rmsNormEps=1e-5, maxRows=256)
        monkeypatch.delenv("JGPT_B200_FUSED_STEP")
    fused.setParameters(om.tensors()), plain.setParameters(om.tensors())
    return om, fused, plain


@pytest.mark.parametrize("n", [1, 2, 3, 4])
def test_fused_step_against_the_multi_launch_step_and_the_oracle(ctx, n, monkeypatch):
    om, fused, plain = _three(ctx, GEOM, 4, 0.15, monkeypatch)
    V, MS = GEOM[0], GEOM[1]
    plens = (31, 3, 47, 16)[:n]  # steps below cross 16-token block boundaries for every row
    prompts = [np.array([(i * 7 + 3 * s) % V for i in range(p)], np.int32) for s, p in enumerate(plens)]
    pools = [g.newPool(n_blocks=n * 5, max_seqs=n) for g in (fused, plain)]
    caches = [om.new_cache(kv_fp16=True) for _ in range(n)]
    try:
        seqs = [[pool.seq_alloc() for _ in range(n)] for pool in pools]
        toks = None
        for g, pool, sq in zip((fused, plain), pools, seqs):
            _, t = g.forwardPrefillBatch(pool, sq, prompts)
            assert toks is None or np.array_equal(toks, t)
            toks = t
        for i in range(n):
            om.forward_prefill(prompts[i], caches[i])
        lens = np.array(plens, np.int32)
        for step in range(20):
            lf, tf = fused.forwardDecodeBatch(pools[0], seqs[0], toks, lens, lens)
            lp, tp = plain.forwardDecodeBatch(pools[1], seqs[1], toks, lens, lens)
            # step 0: both read the same prefilled payload; later the payloads appended by the two forms differ by fp16 ulps
            assert np.abs(lf - lp).max() < (1e-4 if step == 0 else 2e-3), (step, float(np.abs(lf - lp).max()))
            for i in range(n):
                want = om.forward_decode(int(toks[i]), caches[i], int(lens[i]), int(lens[i]))
                assert np.abs(lf[i] - want).max() < 2e-3, (step, i)
                assert tf[i] == int(np.argmax(lf[i]))  # the kernel's own argmax: first index of the maximum
            top = np.sort(lp, axis=1)[:, ::-1]
            assert np.array_equal(tf, tp) or (top[:, 0] - top[:, 1]).min() < 1e-4
            toks, lens = tp, lens + 1
        for layer in (0, GEOM[4] - 1):  # what the step appended, as the store holds it
            for i in range(n):
                planes = []
                for pool, sq in zip(pools, seqs):
                    kd, vd = ctx.alloc((GEOM[3], MS, 16)), ctx.alloc((GEOM[3], MS, 16))
                    pool.gather(layer, sq[i], int(lens[i]), MS, kd, vd)
                    planes.append((kd.to_host(), vd.to_host()))
                for a, b in zip(planes[0], planes[1]):
                    if layer == 0:
                        assert np.all(np.abs(a - b) <= np.abs(b) * 2.0 ** -10 + 5e-5), float(np.abs(a - b).max())
                    else:
                        assert np.abs(a - b).max() < 4e-3, float(np.abs(a - b).max())
                ok = caches[i].k(layer)[:, :lens[i]]  # the oracle's payload
                gk = planes[0][0][:, :lens[i]]
                if layer == 0:  # first layer: the inputs of the projection are the oracle's own
                    assert np.all(np.abs(gk - ok) <= np.abs(ok) * 2.0 ** -10 + 5e-5), float(np.abs(gk - ok).max())
                else:  # deeper layers see the earlier layers' one-ulp payload differences through the attention
                    assert np.abs(gk - ok).max() < 4e-3, float(np.abs(gk - ok).max())
    finally:
        for pool in pools:
            pool.close()
        for c in caches:
            c.close()
        fused.close(), plain.close(), om.close()


@pytest.mark.parametrize("max_seq,prompt_len,max_new", [(80, 10, 60), (48, 9, 55), (80, 79, 1), (80, 78, 2)])
def test_generation_with_many_steps_per_launch(ctx, max_seq, prompt_len, max_new, monkeypatch):
    """jgpt_generate_greedy runs the steps up to the point where the window starts to slide in one launch (each step's
    argmax feeds the next): the stream of the one-step-per-call loop and of the oracle, the allocator left as that
    loop leaves it."""
    geom = (96, max_seq, 64, 4, 3, 128)
    om, fused, plain = _three(ctx, geom, 4, 0.15, monkeypatch)
    pools = [g.newPool(n_blocks=12, max_seqs=2) for g in (fused, plain)]
    try:
        for mult in (7, 11):
            prompt = np.array([(i * mult + 3) % 96 for i in range(prompt_len)], np.int32)
            want, _ = om.generate_greedy(prompt, max_new, kv_fp16=True)
            got_f = fused.generateGpuKv(prompt, max_new, pool=pools[0])
            got_p = plain.generateGpuKv(prompt, max_new, pool=pools[1])
            assert np.array_equal(got_f, got_p), (got_f, got_p)
            assert np.array_equal(got_f, want)
            assert pools[0].free_blocks() == pools[1].free_blocks() == 12
            tables = []
            for pool in pools:  # the next sequence gets the same blocks in the same order
                s = pool.seq_alloc()
                pool.reserve(s, min(70, max_seq))
                tables.append(pool.block_table(s).tolist())
                pool.seq_free(s)
            assert tables[0] == tables[1]
    finally:
        for pool in pools:
            pool.close()
        fused.close(), plain.close(), om.close()


def test_a_sampled_zero_ends_the_launch(ctx, monkeypatch):
    """Generation stops after id 0 (the reference's end marker); inside a launch of many steps the kernel itself
    stops there.  A vocabulary of 8 makes a zero likely; the seed is searched on the CPU."""
    geom = (8, 64, 32, 2, 2, 64)
    prompt = np.array([3, 5, 1, 7, 2], np.int32)
    found = None
    for seed in range(200):
        om = O.Model(*geom, eps=1e-5).init_random(seed=seed, std=0.3)
        want, n = om.generate_greedy(prompt, 40, kv_fp16=True)
        om.close()
        if 4 <= n < 40:
            found = (seed, want, n)
            break
    assert found, "no seed with an early stop"
    seed, want, n = found
    om, fused, plain = _three(ctx, geom, seed, 0.3, monkeypatch)
    pool = fused.newPool(n_blocks=8, max_seqs=1)
    try:
        got = fused.generateGpuKv(prompt, 40, pool=pool)
        assert np.array_equal(got, want) and got[5 + n - 1] == 0 and not got[5 + n:].any()
        assert np.array_equal(plain.generateGpuKv(prompt, 40), want)
        assert pool.free_blocks() == 8
    finally:
        pool.close(), fused.close(), plain.close(), om.close()


@pytest.mark.parametrize("n,geom,std", [(5, GEOM, 0.15), (17, GEOM, 0.15), (40, (96, 320, 64, 4, 2, 128), 0.15),
                                        (9, (512, 256, 384, 24, 2, 768), 0.05)])
def test_fused_batch_step_against_the_multi_launch_step_and_the_oracle(ctx, n, geom, std, monkeypatch):
    """Five rows and up: tile products and a warp per attention unit inside one launch (csrc/decode_batch.cu), against the
    multi-launch step (JGPT_B200_FUSED_BATCH=0) and the oracle.  Ragged lengths (1 token up to several chunks), steps that
    cross block and chunk boundaries."""
    om = O.Model(*geom, eps=1e-5).init_random(seed=6, std=std)
    V, MS = geom[0], geom[1]
    with exact_prefill():
        monkeypatch.setenv("JGPT_B200_FUSED_BATCH", "1")
        fused = GPTModel(ctx, *geom, rmsNormEps=1e-5, maxRows=2048)
        monkeypatch.setenv("JGPT_B200_FUSED_BATCH", "0")
        plain = GPTModel(ctx, *geom, rmsNormEps=1e-5, maxRows=2048)
        monkeypatch.delenv("JGPT_B200_FUSED_BATCH")
    fused.setParameters(om.tensors()), plain.setParameters(om.tensors())
    rng = np.random.default_rng(n)
    plens = [int(x) for x in rng.integers(1, MS - 12, n)]
    plens[0], plens[1] = 1, MS - 12
    prompts = [rng.integers(0, V, p).astype(np.int32) for p in plens]
    blocks = sum(-(-(p + 12) // 16) for p in plens)
    pools = [g.newPool(n_blocks=blocks, max_seqs=n) for g in (fused, plain)]
    n_check = min(n, 6)  # rows followed in the oracle
    caches = [om.new_cache(kv_fp16=True) for _ in range(n_check)]
    try:
        seqs = [[pool.seq_alloc() for _ in range(n)] for pool in pools]
        toks = None
        for g, pool, sq in zip((fused, plain), pools, seqs):
            for i0 in range(0, n, 8):  # prefill in groups that fit the workspace
                _, t = g.forwardPrefillBatch(pool, sq[i0:i0 + 8], prompts[i0:i0 + 8])
                toks_g = t if i0 == 0 else np.concatenate([toks_g, t])
            assert toks is None or np.array_equal(toks, toks_g)
            toks = toks_g
        for i in range(n_check):
            om.forward_prefill(prompts[i], caches[i])
        lens = np.array(plens, np.int32)
        for step in range(10):
            lf, tf = fused.forwardDecodeBatch(pools[0], seqs[0], toks, lens, lens)
            lp, tp = plain.forwardDecodeBatch(pools[1], seqs[1], toks, lens, lens)
            assert np.abs(lf - lp).max() < (1e-4 if step == 0 else 2e-3), (step, float(np.abs(lf - lp).max()))
            for i in range(n_check):
                want = om.forward_decode(int(toks[i]), caches[i], int(lens[i]), int(lens[i]))
                assert np.abs(lf[i] - want).max() < 2e-3, (step, i, float(np.abs(lf[i] - want).max()))
            assert np.array_equal(tf, np.argmax(lf, axis=1))
            toks, lens = tp, lens + 1
        for i in (0, 1, n - 1):  # appended payload of the first layer: the multi-launch step's, up to one fp16 ulp
            planes = []
            for pool, sq in zip(pools, seqs):
                kd, vd = ctx.alloc((geom[3], MS, 16)), ctx.alloc((geom[3], MS, 16))
                pool.gather(0, sq[i], int(lens[i]), MS, kd, vd)
                planes.append((kd.to_host(), vd.to_host()))
            for a, b in zip(planes[0], planes[1]):
                assert np.all(np.abs(a - b) <= np.abs(b) * 2.0 ** -10 + 5e-5), float(np.abs(a - b).max())
    finally:
        for pool in pools:
            pool.close()
        for c in caches:
            c.close()
        fused.close(), plain.close(), om.close()


def test_a_refused_cooperative_launch_falls_back_to_the_multi_launch_step(ctx, monkeypatch):
    """A device that cannot keep one CTA per SM resident (MPS with a thread percentage, a green context) refuses the
    cooperative launch.  Injected on the host (JGPT_B200_FUSED_REFUSE=1): the call must still succeed, through the
    multi-launch step, bit for bit; generation likewise, with the allocator left clean."""
    om, fused, plain = _three(ctx, GEOM, 4, 0.15, monkeypatch)
    pools = [g.newPool(n_blocks=10, max_seqs=2) for g in (fused, plain)]
    try:
        prompt = np.array([(i * 7 + 3) % GEOM[0] for i in range(20)], np.int32)
        monkeypatch.setenv("JGPT_B200_FUSED_REFUSE", "1")
        outs = []
        for g, pool in zip((fused, plain), pools):
            s = pool.seq_alloc()
            _, t = g.forwardPrefillBatch(pool, [s], [prompt])
            lg, nx = g.forwardDecodeBatch(pool, [s], t, [20], [20])
            outs.append((lg, nx))
            pool.seq_free(s)
        assert np.array_equal(outs[0][0], outs[1][0]) and np.array_equal(outs[0][1], outs[1][1])
        a = fused.generateGpuKv(prompt, 30, pool=pools[0])
        b = plain.generateGpuKv(prompt, 30, pool=pools[1])
        assert np.array_equal(a, b) and pools[0].free_blocks() == 10
        monkeypatch.delenv("JGPT_B200_FUSED_REFUSE")
        # the form stays off for this model after a refusal: still the multi-launch answers
        s = pools[0].seq_alloc()
        _, t = fused.forwardPrefillBatch(pools[0], [s], [prompt])
        lg, _ = fused.forwardDecodeBatch(pools[0], [s], t, [20], [20])
        assert np.array_equal(lg, outs[1][0])
    finally:
        for pool in pools:
            pool.close()
        fused.close(), plain.close(), om.close()


def test_a_wait_that_runs_out_is_reported_and_the_next_call_works(ctx, monkeypatch):
    """Every wait inside the one-launch step is bounded.  A test hook lets one CTA withhold a result (nothing faults,
    nothing spins for ever): the units that need it give up after their poll limit (~0.5 s), the launch reports
    wait-timeout through the status word, the call fails without tokens or a length change - and the next call, with
    fresh stamps, runs as if nothing had happened."""
    from jgpt_b200 import JgptError

    om, fused, plain = _three(ctx, GEOM, 4, 0.15, monkeypatch)
    pools = [g.newPool(n_blocks=6, max_seqs=1) for g in (fused, plain)]
    try:
        prompt = np.array([(i * 7 + 3) % GEOM[0] for i in range(20)], np.int32)
        seqs, toks = [], None
        for g, pool in zip((fused, plain), pools):
            s = pool.seq_alloc()
            _, toks = g.forwardPrefillBatch(pool, [s], [prompt])
            seqs.append(s)
        monkeypatch.setenv("JGPT_B200_FUSED_TEST_WITHHOLD", "1")
        with pytest.raises(JgptError, match="wait-timeout"):
            fused.forwardDecodeBatch(pools[0], [seqs[0]], toks, [20], [20])
        assert pools[0].length(seqs[0]) == 20
        monkeypatch.delenv("JGPT_B200_FUSED_TEST_WITHHOLD")
        lf, tf = fused.forwardDecodeBatch(pools[0], [seqs[0]], toks, [20], [20])
        lp, tp = plain.forwardDecodeBatch(pools[1], [seqs[1]], toks, [20], [20])
        assert np.abs(lf - lp).max() < 1e-4 and np.array_equal(tf, tp)
        # generation after an aborted multi-step launch as well
        monkeypatch.setenv("JGPT_B200_FUSED_TEST_WITHHOLD", "1")
        with pytest.raises(JgptError, match="wait-timeout"):
            fused.generateGpuKv(prompt, 12)
        monkeypatch.delenv("JGPT_B200_FUSED_TEST_WITHHOLD")
        assert np.array_equal(fused.generateGpuKv(prompt, 12), plain.generateGpuKv(prompt, 12))
    finally:
        for pool in pools:
            pool.close()
        fused.close(), plain.close(), om.close()
