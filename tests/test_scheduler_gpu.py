"""Continuous batching on the GPU against the written policy (oracle.ContinuousBatchRef) and the oracle's
per-request greedy streams: admissions, evictions and block tables bit-exact, token streams identical."""
import numpy as np
import pytest

import oracle as O
from helpers import exact_prefill
from jgpt_b200 import ContinuousBatcher, GPTModel

pytestmark = pytest.mark.gpu


def test_continuous_batching_matches_policy_and_oracle_streams(ctx):
    V, MS = 96, 80
    om = O.Model(V, MS, 64, 4, 3, 128, eps=1e-5).init_random(seed=4, std=0.15)
    with exact_prefill():  # toy weights: identical token streams need the exact prefill attention
        gm = GPTModel(ctx, V, MS, 64, 4, 3, 128, rmsNormEps=1e-5, maxRows=96)
    gm.setParameters(om.tensors())
    rng = np.random.default_rng(2)
    n_req = 28
    p_len = rng.integers(4, 41, n_req)
    t_len = rng.integers(2, 31, n_req)
    prompts = [rng.integers(0, V, int(n)).astype(np.int32) for n in p_len]
    demand = sum(-(-(int(p) + int(t) - 1) // 16) for p, t in zip(p_len, t_len))
    n_blocks = int(0.6 * demand)  # pool sized at 60 % of the total demand
    max_seqs, max_running = 10, 6
    pool = gm.newPool(n_blocks=n_blocks, max_seqs=max_seqs)
    sched = ContinuousBatcher(gm, pool, max_running=max_running)
    try:
        streams = []
        for p, t in zip(prompts, t_len):  # a request's tokens do not depend on the batch it runs in
            out, n = om.generate_greedy(p, int(t), kv_fp16=True)
            streams.append(out[p.size:p.size + n])
        ref = O.ContinuousBatchRef(O.PagedAllocatorRef(n_blocks, 16, max_seqs, -(-MS // 16)), max_running, 96, streams)
        for p, t in zip(prompts, t_len):
            assert sched.submit(p, int(t)) == ref.submit(p.size, int(t))
        with pytest.raises(ValueError):  # no sliding window while batching
            sched.submit(prompts[0], MS)
        for step in range(10_000):
            pairs, nr, nw = sched.step()
            want = ref.step()
            assert [tuple(x) for x in pairs.tolist()] == want, step
            assert (nr, nw) == (len(ref.running), len(ref.waiting))
            for rid in ref.running:  # block tables of everything running: library == specification
                seq = ref.reqs[rid]["seq"]
                assert pool.block_table(seq).tolist() == ref.a.tables[seq]
                assert pool.block_table(seq, device=True).tolist() == ref.a.tables[seq]
                assert pool.length(seq) == ref.a.length[seq]
            assert pool.free_blocks() == len(ref.a.free)
            if nr == 0 and nw == 0:
                break
        assert sched.events() == ref.events
        assert any(e[0] == 2 for e in ref.events), "the pool was sized so that evictions must happen"
        for rid in range(n_req):
            toks, state, _ = sched.result(rid)
            assert state == 2 and np.array_equal(toks, streams[rid]), rid
    finally:
        sched.close(), pool.close(), gm.close(), om.close()
