"""The named configurations at their stated sizes (not toy geometries), through the C ABI.

Config 3: causal prefill of batch 32 x 1024 on the JGPT-35M shapes in ONE `jgpt_forward_prefill_batch` call, the
full paged cache written; last-row logits of several sequences against the oracle's per-sequence prefill (the
reference is batch 1: it would loop), one sequence's whole cache against the oracle's fp16 payload.

Config 4: continuous batching of 256 requests (seed 2: prompt U[32, 512], target U[64, 1024] clipped to the
context) on the JGPT-35M shapes with the pool at 60 % of the demand: admissions, evictions, finishes, block tables
(host and device mirror) and free-block counts, step by step, against the written policy
(`oracle.ContinuousBatchRef`).  The policy depends on a request's tokens only through their number and an early
stop on id 0; the reference streams are the ones this model produced in a first run of the same job (a request's
tokens do not depend on what it is batched with), and two short requests are checked against the oracle's own
greedy generation so that the streams themselves are anchored.

Tolerances as everywhere: logits <= 2e-3 against the fp32-cache oracle, <= 5e-4 against the fp16-payload
oracle; payload within one fp16 step; integers bit-exact."""
import numpy as np
import pytest

import oracle as O
from jgpt_b200 import ContinuousBatcher, GPTModel
from jgpt_b200 import workloads as W

pytestmark = pytest.mark.gpu


def _oracle_35m():
    om = O.Model(W.VOCAB, W.CTX, W.D_MODEL, W.HEADS, W.LAYERS, W.D_FF, eps=W.EPS)
    for t, src in zip(om.tensors(), W.jgpt35m_parameters()):
        t[...] = src
    return om


def test_config3_prefill_batch_32_by_1024_fills_the_cache_and_matches_oracle(ctx):
    B, S = 32, 1024
    gm = W.make_model(ctx, max_rows=B * S)
    pool = gm.newPool(n_blocks=B * S // 16, max_seqs=B)
    om = _oracle_35m()
    try:
        rng = np.random.default_rng(7)
        prompts = [rng.integers(0, W.VOCAB, S).astype(np.int32) for _ in range(B)]
        seqs = [pool.seq_alloc() for _ in range(B)]
        logits, nxt = gm.forwardPrefillBatch(pool, seqs, prompts)
        assert logits.shape == (B, W.VOCAB) and all(pool.length(s) == S for s in seqs)
        assert pool.free_blocks() == 0  # the whole pool is in use: 32 x 64 blocks
        assert np.array_equal(nxt, logits.argmax(-1))
        checked = (0, 9, 22, 31)
        for i in checked:
            oc32, oc16 = om.new_cache(kv_fp16=False), om.new_cache(kv_fp16=True)
            want32, want16 = om.forward_prefill(prompts[i], oc32)[-1], om.forward_prefill(prompts[i], oc16)[-1]
            assert np.abs(logits[i] - want32).max() < 2e-3, i
            assert np.abs(logits[i] - want16).max() < 5e-4, i
            top = np.sort(want16)[::-1]
            assert int(nxt[i]) == int(np.argmax(want16)) or top[0] - top[1] < 1e-4
            if i == 22:  # this sequence's full paged cache, every layer, against the oracle's fp16 payload
                kd, vd = ctx.alloc((W.HEADS, S, W.DHEAD)), ctx.alloc((W.HEADS, S, W.DHEAD))
                for layer in range(W.LAYERS):
                    pool.gather(layer, seqs[i], S, S, kd, vd)
                    for got_p, want_p in ((kd.to_host(), oc16.k(layer)), (vd.to_host(), oc16.v(layer))):
                        step = np.maximum(np.abs(want_p), 2.0 ** -14) * 2.0 ** -10  # one fp16 step at that magnitude
                        assert (np.abs(got_p - want_p) <= step + (2e-4 if layer == 0 else 1e-3)).all(), layer
                        assert (got_p == want_p).mean() > (0.97 if layer == 0 else 0.6), layer
                kd.close(), vd.close()
    finally:
        pool.close(), gm.close(), om.close()


def _config4_requests(n_requests=256):
    rng = np.random.default_rng(2)
    p_len = rng.integers(32, 513, n_requests)
    t_len = rng.integers(64, 1025, n_requests)
    t_len = np.minimum(t_len, W.CTX - p_len + 1)
    prompts = [rng.integers(0, W.VOCAB, int(n)).astype(np.int32) for n in p_len]
    return prompts, [int(t) for t in t_len]


def test_config4_continuous_batching_256_requests_matches_policy_step_by_step(ctx):
    prompts, t_len = _config4_requests()
    n_req = len(prompts)
    demand = sum(-(-(p.size + t - 1) // 16) for p, t in zip(prompts, t_len))
    n_blocks = max(int(0.6 * demand), W.CTX // 16)
    max_seqs, max_running, max_rows = n_req + 1, n_req, 4096
    gm = W.make_model(ctx, max_rows=max_rows)
    try:
        # first run: the streams this model produces (also the throughput run of the benchmark's `contbatch` leg)
        pool = gm.newPool(n_blocks=n_blocks, max_seqs=max_seqs)
        sched = ContinuousBatcher(gm, pool, max_running=max_running, max_rows_per_call=max_rows)
        for p, t in zip(prompts, t_len):
            sched.submit(p, t)
        steps_first = sched.run()
        streams = [sched.result(r)[0] for r in range(n_req)]
        events_first = sched.events()
        sched.close(), pool.close()
        assert all(len(s) == t or (len(s) < t and s[-1] == 0) for s, t in zip(streams, t_len))
        assert sum(1 for e in events_first if e[0] == 2) > 50, "a pool at 60 % of the demand must evict"

        # anchor the streams: the two requests with the least work, generated by the oracle on the host
        om = _oracle_35m()
        try:
            for rid in sorted(range(n_req), key=lambda r: prompts[r].size + t_len[r])[:2]:
                out, n = om.generate_greedy(prompts[rid], t_len[rid], kv_fp16=True)
                want = out[prompts[rid].size:prompts[rid].size + n]
                # identical streams (greedy, fp16-payload oracle: the cache the store really holds)
                m = min(len(want), len(streams[rid]))
                first_diff = next((j for j in range(m) if want[j] != streams[rid][j]), None)
                assert first_diff is None and len(want) == len(streams[rid]), (rid, first_diff)
        finally:
            om.close()

        # second run, in lockstep with the written policy driven by those streams
        pool = gm.newPool(n_blocks=n_blocks, max_seqs=max_seqs)
        sched = ContinuousBatcher(gm, pool, max_running=max_running, max_rows_per_call=max_rows)
        ref = O.ContinuousBatchRef(O.PagedAllocatorRef(n_blocks, 16, max_seqs, W.CTX // 16), max_running, max_rows, streams)
        try:
            for p, t in zip(prompts, t_len):
                assert sched.submit(p, t) == ref.submit(p.size, t)
            n_events = 0
            for step in range(steps_first + 5):
                pairs, nr, nw = sched.step()
                want = ref.step()
                assert [tuple(x) for x in pairs.tolist()] == want, step
                assert (nr, nw) == (len(ref.running), len(ref.waiting)), step
                assert pool.free_blocks() == len(ref.a.free), step
                if len(ref.events) != n_events or step % 64 == 0:  # something was admitted / evicted / finished
                    n_events = len(ref.events)
                    for rid in ref.running:
                        seq = ref.reqs[rid]["seq"]
                        assert pool.block_table(seq).tolist() == ref.a.tables[seq], (step, rid)
                        assert pool.block_table(seq, device=True).tolist() == ref.a.tables[seq], (step, rid)
                        assert pool.length(seq) == ref.a.length[seq], (step, rid)
                if nr == 0 and nw == 0:
                    break
            assert step + 1 == steps_first
            assert sched.events() == ref.events == events_first
            for rid in range(n_req):
                toks, state, _ = sched.result(rid)
                assert state == 2 and np.array_equal(toks, streams[rid]), rid
        finally:
            sched.close(), pool.close()
    finally:
        gm.close()
