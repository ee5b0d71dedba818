"""GPU-side runners for the secondary benchmark workloads (`bench.py --workload ...`): the JGPT-35M greedy
decode, the batch-32 x 1024 prefill, continuous batching of 256 requests and the long-context decode
attention.  Each returns a dict that bench.py prints as one JSON line.  Inputs are seeded synthetic tensors
of the stated shapes (there is no trained checkpoint or dataset)."""
from __future__ import annotations

import time

import numpy as np

from . import binding as B
from .kv_cache import KvPool
from .model import GPTModel
from .runtime import Event
from .scheduler import ContinuousBatcher, TokenGather, shard_requests

VOCAB, CTX, D_MODEL, HEADS, LAYERS, D_FF, EPS = 8000, 1024, 384, 24, 12, 768, 1e-5
DHEAD = D_MODEL // HEADS


def jgpt35m_parameters(seed=0, std=0.02, max_seq=CTX):
    """Parameter tensors in file order: every matrix N(0, std) from numpy default_rng(seed), RMSNorm gammas 1."""
    rng = np.random.default_rng(seed)
    shapes = [(VOCAB, D_MODEL), (max_seq, D_MODEL)]
    for _ in range(LAYERS):
        shapes += [(D_MODEL, D_MODEL)] * 4 + [(D_MODEL, D_FF), (D_FF, D_MODEL), (D_MODEL, D_FF), (D_MODEL,), (D_MODEL,)]
    shapes += [(D_MODEL,), (D_MODEL, VOCAB)]
    return [rng.normal(0.0, std, size=s).astype(np.float32) if len(s) == 2 else np.ones(s, np.float32) for s in shapes]


def make_model(ctx, max_rows, max_seq=CTX):
    m = GPTModel(ctx, VOCAB, max_seq, D_MODEL, HEADS, LAYERS, D_FF, rmsNormEps=EPS, maxRows=max_rows)
    m.setParameters(jgpt35m_parameters(max_seq=max_seq))
    return m


def run_decode35m(ctx, steps_new=128, prompt_len=64, repeats=3):
    """Batch 1: prompt of 64 ids (seed 1), 128 greedy tokens with the KV cache, through generateGpuKv."""
    model = make_model(ctx, max_rows=CTX)
    pool = model.newPool(n_blocks=CTX // 16, max_seqs=1)
    prompt = np.random.default_rng(1).integers(0, VOCAB, prompt_len).astype(np.int32)
    try:
        model.generateGpuKv(prompt, 8, pool=pool)  # warm-up (module load, scratch sizing)
        best_total = best_prefill = 1e30
        out = None
        for _ in range(repeats):
            t0 = time.perf_counter()
            out1 = model.generateGpuKv(prompt, 1, pool=pool)
            t1 = time.perf_counter()
            out = model.generateGpuKv(prompt, steps_new, pool=pool)
            t2 = time.perf_counter()
            best_prefill = min(best_prefill, t1 - t0)
            best_total = min(best_total, t2 - t1)
            assert out[prompt_len] == out1[prompt_len]
        n_sampled = int(np.count_nonzero(out[prompt_len:])) if 0 in out[prompt_len:] else steps_new
        decode_s = max(best_total - best_prefill, 1e-9)
        return {
            "workload": "JGPT-35M greedy decode, batch 1, prompt 64 (seed 1) + 128 new tokens, weights N(0,0.02) seed 0",
            "tokens_sampled": n_sampled, "prefill_ms": best_prefill * 1e3, "total_ms": best_total * 1e3,
            "decode_ms_per_token": decode_s / max(steps_new - 1, 1) * 1e3,
            "decode_tokens_per_s": (steps_new - 1) / decode_s, "first_tokens": out[prompt_len:prompt_len + 8].tolist(),
            "timing": "host wall clock around generateGpuKv (prefill, then the greedy steps inside the library: one launch for up to 256 steps "
                      "when the fused step applies, else one synchronising call per step), best of %d" % repeats,
        }
    finally:
        pool.close(), model.close()


def run_decode_step(ctx, batch=64, ctx_len=512, steps=50):
    """Batched decode steps of the full model: `batch` sequences prefilled with `ctx_len` ids, then `steps`
    forwardDecode steps (sampled ids fed back).  Host clock around the step (it synchronises to read the ids)."""
    model = make_model(ctx, max_rows=8192)
    pool = model.newPool(n_blocks=batch * (-(-(ctx_len + steps + 8) // 16)), max_seqs=batch)
    rng = np.random.default_rng(0)
    seqs = [pool.seq_alloc() for _ in range(batch)]
    prompts = [rng.integers(0, VOCAB, ctx_len).astype(np.int32) for _ in range(batch)]
    per_call = max(1, 8192 // ctx_len)
    try:
        toks = np.zeros(batch, np.int32)
        for i in range(0, batch, per_call):
            _, toks[i:i + per_call] = model.forwardPrefillBatch(pool, seqs[i:i + per_call], prompts[i:i + per_call])
        lens = np.full(batch, ctx_len, np.int32)
        seq_ids = np.asarray(seqs, np.int32)  # converted once: a Python list costs ~5 us per call to turn into an array
        for _ in range(3):
            _, toks = model.forwardDecodeBatch(pool, seq_ids, toks, lens, lens, want_logits=False)
            lens += 1
        ctx.synchronize()
        t0 = time.perf_counter()
        for _ in range(steps):
            _, toks = model.forwardDecodeBatch(pool, seq_ids, toks, lens, lens, want_logits=False)
            lens += 1
        el = (time.perf_counter() - t0) / steps
        return {"workload": f"JGPT-35M batched decode step: batch {batch}, context {ctx_len}+, sampled ids fed back",
                "ms_per_step": el * 1e3, "tokens_per_s": batch / el, "steps": steps,
                "timing": "host wall clock around forwardDecodeBatch (each step reads the sampled ids back)"}
    finally:
        pool.close(), model.close()


def run_prefill(ctx, batch=32, seq_len=1024, repeats=3):
    """Batch 32 x 1024 prompt tokens through the full model; the paged cache of all 12 layers is written."""
    model = make_model(ctx, max_rows=batch * seq_len)
    pool = model.newPool(n_blocks=batch * seq_len // 16, max_seqs=batch)
    rng = np.random.default_rng(7)
    prompts = [rng.integers(0, VOCAB, seq_len).astype(np.int32) for _ in range(batch)]
    seqs = [pool.seq_alloc() for _ in range(batch)]
    try:
        model.forwardPrefillBatch(pool, seqs, prompts)  # warm-up
        e0, e1 = Event(ctx), Event(ctx)
        best = 1e30
        for _ in range(repeats):
            for s in seqs:
                pool.clear(s, zero_fill=False)
            ctx.synchronize()
            e0.record()
            _, nxt = model.forwardPrefillBatch(pool, seqs, prompts)
            e1.record()
            best = min(best, e0.elapsed_ms(e1))
        # attention alone on the same shapes: the exact mode (fp16 high + low operands, the standalone entry point's
        # default) and the single-fp16 mode the model's forward uses
        import os

        n_rows = batch * seq_len
        q = ctx.alloc((n_rows, D_MODEL))
        q.copy_from(rng.standard_normal((n_rows, D_MODEL), dtype=np.float32))
        out = ctx.alloc((n_rows, D_MODEL))
        starts = np.arange(batch + 1, dtype=np.int32) * seq_len
        ro = np.zeros(batch, np.int32)
        attn = {}
        for label, fast in (("exact", "0"), ("fast", "1")):
            old_env = os.environ.get("JGPT_B200_PREFILL_FAST")
            os.environ["JGPT_B200_PREFILL_FAST"] = fast
            try:
                p2 = model.newPool(n_blocks=batch * seq_len // 16, max_seqs=batch)
            finally:
                if old_env is None:
                    os.environ.pop("JGPT_B200_PREFILL_FAST")
                else:
                    os.environ["JGPT_B200_PREFILL_FAST"] = old_env
            s2 = [p2.seq_alloc() for _ in range(batch)]
            for s in s2:
                p2.reserve(s, seq_len)
            for _ in range(2):
                p2.attn_prefill(0, q, q, q, s2, starts, ro, out)
            ctx.synchronize()
            e0.record()
            for layer in range(LAYERS):
                p2.attn_prefill(layer, q, q, q, s2, starts, ro, out)
            e1.record()
            attn[label] = e0.elapsed_ms(e1)
            p2.close()
        attn_ms = attn["fast"]
        flops = 12 * batch * HEADS * 2.0 * seq_len * seq_len * DHEAD  # causal: (4 S^2 Dh)/2 per (seq, head), 12 layers
        return {
            "workload": f"causal prefill filling the paged cache: batch {batch} x {seq_len}, 12 layers, 24 heads, d_head 16 (ids seed 7)",
            "full_model_ms": best, "prompt_tokens_per_s": n_rows / (best * 1e-3),
            "attention_append_12_layers_ms": attn_ms, "attention_append_12_layers_ms_exact_mode": attn["exact"],
            "attention_tflops_causal": flops / (attn_ms * 1e-3) / 1e12,
            "next_tokens_head": nxt[:4].tolist(), "timing": "CUDA events on the library stream, best of %d" % repeats,
        }
    finally:
        pool.close(), model.close()


def run_contbatch(ctx, rank, world, unique_id=None, n_requests=256, pool_fraction=0.6, max_steps=100_000, gather_depth=4):
    """256 requests (seed 2): prompt U[32,512], target U[64,1024] new tokens clipped to the 1024 context; pool sized
    at 60 % of the rank's total block demand; requests dealt round-robin to the ranks; sampled ids all-gathered."""
    rng = np.random.default_rng(2)
    p_len = rng.integers(32, 513, n_requests)
    t_len = rng.integers(64, 1025, n_requests)
    t_len = np.minimum(t_len, CTX - p_len + 1)
    prompts = [rng.integers(0, VOCAB, int(n)).astype(np.int32) for n in p_len]
    mine = shard_requests(n_requests, world, rank)
    demand = sum(-(-(int(p_len[i]) + int(t_len[i]) - 1) // 16) for i in mine)
    n_blocks = max(int(pool_fraction * demand), CTX // 16)
    model = make_model(ctx, max_rows=4096)
    pool = model.newPool(n_blocks=n_blocks, max_seqs=len(mine) + 1)
    sched = ContinuousBatcher(model, pool, max_running=len(mine), max_rows_per_call=4096)
    try:
        for i in mine:
            sched.submit(prompts[i], int(t_len[i]))
        ctx.synchronize()
        total_tokens, steps, done, all_done = 0, 0, False, False
        gather = TokenGather(ctx, world, rank, max_pairs=-(-n_requests // world) + 2, unique_id=unique_id, depth=gather_depth)

        def account(allp):
            nonlocal total_tokens, all_done
            total_tokens += sum(1 for r, _ in allp if r >= 0)
            all_done = all_done or sum(1 for r, _ in allp if r < 0) == world

        t0 = time.perf_counter()
        t_step = t_submit = t_pop = 0.0
        while steps < max_steps and not all_done:
            ta = time.perf_counter()
            if not done:
                pairs, nr, nw = sched.step()
                done = nr == 0 and nw == 0
            else:
                pairs = np.zeros((0, 2), np.int32)
            tb = time.perf_counter()
            # the ids of step t are all-gathered while steps t+1 .. t+depth run; a finished rank keeps reporting (-1, 1)
            gather.submit([(mine[int(r)], int(t)) for r, t in pairs], done=done)
            tc = time.perf_counter()
            steps += 1
            while gather.ready() and not all_done:
                account(gather.pop())
            td = time.perf_counter()
            t_step += tb - ta
            t_submit += tc - tb
            t_pop += td - tc
        for allp in gather.drain():
            account(allp)
        el = time.perf_counter() - t0
        gather.close()
        ev = sched.events()
        return {
            "workload": f"continuous batching: {n_requests} requests (seed 2), prompt U[32,512], target U[64,1024] clipped to the "
                        f"1024 context, KV pool {pool_fraction:.0%} of demand, round-robin over {world} GPU(s), token ids all-gathered by the library's "
                        f"NCCL communicator (asynchronously, read {gather_depth} steps later)",
            "generated_tokens": total_tokens, "steps": steps, "seconds": el, "tokens_per_s": total_tokens / el,
            "seconds_in": {"scheduler_steps": t_step, "gather_submit": t_submit, "gather_read": t_pop},
            "pool_blocks_rank0": n_blocks, "demand_blocks_rank0": demand, "evictions_rank0": sum(1 for e in ev if e[0] == 2),
            "timing": "host wall clock over the whole run (prefills included)",
        }
    finally:
        sched.close(), pool.close(), model.close()


def run_kvstore(ctx, batch=64, ctx_len=1024, n_blocks=4096, repeats=7):
    """The three K/V store kernels on their own at the microbenchmark's size (12 layers x 24 heads x d_head 16, 64
    sequences x 1024 tokens, 4096-block pool, seeded random block table): append of all 65,536 tokens of one layer
    (RoPE + fp16 conversion), gather of the 64 sequences of one layer into contiguous fp32 planes, and the eviction
    scrub of the whole pool.  CUDA events on the library's stream, median of `repeats`; algorithmic bytes per unit:
    append = per token H*DH*(4*2 read + 2*2 written) + 12 index bytes; gather = per (head, position) DH*(2*2 read +
    4*2 written); scrub = per freed block layers*H*64*DH bytes written."""
    import json
    import os
    import statistics

    try:
        peak = float(json.load(open(os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "MEASURED_PEAKS.json")))["hbm_gbs"])
        kind = "of measured"
    except Exception:
        peak, kind = 6650.0, "of fallback"
    pool = KvPool(ctx, LAYERS, HEADS, DHEAD, n_blocks, batch, ctx_len // 16, max_positions=ctx_len)
    rng = np.random.default_rng(1234)
    perm = rng.permutation(n_blocks).astype(np.int32).reshape(batch, ctx_len // 16)
    try:
        seqs = []
        for i in range(batch):
            s = pool.seq_alloc()
            pool.set_block_table(s, perm[i])
            pool.set_length(s, ctx_len)
            seqs.append(s)
        tot = batch * ctx_len
        k = ctx.from_host(rng.standard_normal((tot, D_MODEL), dtype=np.float32))
        v = ctx.from_host(rng.standard_normal((tot, D_MODEL), dtype=np.float32))
        sid = ctx.from_host(np.repeat(np.asarray(seqs, np.int32), ctx_len))
        pos = ctx.from_host(np.tile(np.arange(ctx_len, dtype=np.int32), batch))
        e0, e1 = Event(ctx), Event(ctx)

        def timed(fn, reps=repeats):
            fn()
            ctx.synchronize()
            ts = []
            for _ in range(reps):
                e0.record()
                fn()
                e1.record()
                ts.append(e0.elapsed_ms(e1))
            return statistics.median(ts)

        out = {}
        # append: a different layer each repeat, so the written lines are not the ones just written (1.2 GB pool > L2)
        layer_it = iter(range(10 ** 9))
        ms = timed(lambda: pool.append(next(layer_it) % LAYERS, k, v, sid, pos, pos, tot))
        alg = tot * (HEADS * DHEAD * (4 * 2 + 2 * 2) + 12)
        out["kv_append_kernel"] = {"ms": ms, "algorithmic_bytes": alg, "GBps": alg / ms / 1e6, "frac": alg / ms / 1e6 / peak,
                                   "unit": f"{tot} tokens of one layer per launch"}
        # gather: 64 launches (one per sequence, the reference's getK/getV granularity), timed as one region
        kd = [ctx.alloc((HEADS, ctx_len, DHEAD)) for _ in range(2)]
        gl = iter(range(10 ** 9))

        def gather_all():
            layer = next(gl) % LAYERS
            for s in seqs:
                pool.gather(layer, s, ctx_len, ctx_len, kd[0], kd[1])

        ms = timed(gather_all)
        alg = batch * HEADS * ctx_len * DHEAD * (2 * 2 + 4 * 2)
        out["kv_gather_kernel"] = {"ms": ms, "algorithmic_bytes": alg, "GBps": alg / ms / 1e6, "frac": alg / ms / 1e6 / peak,
                                   "launches": batch, "unit": "64 sequences x 1024 positions of one layer, one launch per sequence "
                                   "(4.7 MB each: launch-bound)"}
        kb = [ctx.alloc((batch, HEADS, ctx_len, DHEAD)) for _ in range(2)]
        gb = iter(range(10 ** 9))
        ms = timed(lambda: pool.gather_batch(next(gb) % LAYERS, seqs, [ctx_len] * batch, ctx_len, kb[0], kb[1]))
        out["kv_gather_kernel_batched"] = {"ms": ms, "algorithmic_bytes": alg, "GBps": alg / ms / 1e6, "frac": alg / ms / 1e6 / peak,
                                           "launches": 1, "unit": "the same 64 sequences in one launch (jgpt_kv_gather_batch)"}
        for b in kb:
            b.close()
        # scrub: free every sequence with zero fill (all 4096 blocks x 12 layers), then map them again
        def scrub_all():
            for s in seqs:
                pool.mark_evictable(s, True)
            pool.evict_lru(n_blocks, zero_fill=True)

        def remap():
            seqs.clear()
            for i in range(batch):
                s = pool.seq_alloc()
                pool.set_block_table(s, perm[i])
                pool.set_length(s, ctx_len)
                seqs.append(s)

        ts = []
        for _ in range(max(3, repeats // 2)):
            ctx.synchronize()
            e0.record()
            scrub_all()
            e1.record()
            ts.append(e0.elapsed_ms(e1))
            remap()
        ms = statistics.median(ts)
        alg = n_blocks * LAYERS * HEADS * 64 * DHEAD
        out["kv_scrub_kernel"] = {"ms": ms, "algorithmic_bytes": alg, "GBps": alg / ms / 1e6, "frac": alg / ms / 1e6 / peak,
                                  "unit": "all 4096 blocks x 12 layers zero-filled by one eviction call (host allocator work included)"}
        return {"workload": "K/V store kernels standalone: 12 layers x 24 heads x d_head 16, 64 x 1024 tokens, 4096-block pool",
                "peak_GBps": peak, "peak_kind": kind, "kernels": out, "timing": f"CUDA events on the library's stream, median of {repeats}"}
    finally:
        pool.close()


def run_phases(ctx, pool, seqs, batch, layers, d_model, ctx_len, overlap=2):
    """Where the time of a per-layer decode-attention launch goes: needs the library built by
    ``python -m jgpt_b200.build --trace`` (loaded through JGPT_B200_LIB).  Runs the per-layer chain as a CUDA graph, then
    reads the per-CTA timestamps of the last two launches: start and end on the global timer, and inside a CTA the
    cycle counts to "barriers initialised", "first K/V slab consumed", "block loop done", "exit"."""
    import ctypes as C

    lib = ctx._lib
    if not hasattr(lib, "jgpt_debug_decode_trace"):
        raise RuntimeError("this library was not built with --trace (python -m jgpt_b200.build --trace; JGPT_B200_LIB=...)")
    lib.jgpt_debug_decode_trace.restype = C.c_int
    rng = np.random.default_rng(5)
    q, k, v = (ctx.from_host(rng.standard_normal((layers, batch, d_model), dtype=np.float32)) for _ in range(3))
    out = ctx.alloc((layers, batch, d_model))
    seq_d = ctx.from_host(np.asarray(seqs, np.int32))
    lens_d, rope_d = ctx.from_host(np.full(batch, ctx_len, np.int32)), ctx.from_host(np.full(batch, ctx_len - 1, np.int32))
    slab = batch * d_model * 4
    pool.set_tuning(launch_overlap=overlap)

    def chain():
        for layer in range(layers):
            pool.attn_decode_append(layer, 1, q.ptr + layer * slab, k.ptr + layer * slab, v.ptr + layer * slab, seq_d, rope_d, lens_d,
                                    batch, ctx_len, out.ptr + layer * slab)

    chain()
    ctx.synchronize()
    g = ctx.capture(chain)
    for _ in range(3):
        g.launch()
    e0, e1 = Event(ctx), Event(ctx)
    e0.record()
    for _ in range(20):
        g.launch()
    e1.record()
    us_layer = e0.elapsed_ms(e1) / 20 / layers * 1e3
    ctx.synchronize()
    g.close()
    buf = np.zeros((65536, 8), np.int64)
    n = lib.jgpt_debug_decode_trace(buf.ctypes.data_as(C.c_void_p), 65536)
    a, b = buf[:n], buf[32768:32768 + n]
    if a[:, 0].min() > b[:, 0].min():
        a, b = b, a  # a = the earlier of the two launches
    g0 = a[:, 0].min()
    res = {"us_per_layer_with_tracing": us_layer, "ctas_per_launch": int(n), "launch_overlap": overlap, "launches": []}
    for t in (a, b):
        start, end = (t[:, 0] - g0) / 1e3, (t[:, 1] - g0) / 1e3
        ph = t[:, 2:6] / 1.9e3  # cycles -> us at 1.9 GHz
        res["launches"].append({
            "cta_start_us": [float(start.min()), float(np.median(start)), float(start.max())],
            "cta_end_us": [float(end.min()), float(np.median(end)), float(end.max())],
            "per_cta_median_us": {"barriers_ready": float(np.median(ph[:, 0])), "first_slab_consumed": float(np.median(ph[:, 1])),
                                  "block_loop_done": float(np.median(ph[:, 2])), "exit": float(np.median(ph[:, 3]))}})
    return res


def run_fused_phases(ctx, prompt_len=900, new_tokens=33):
    """Where the time of one layer of the one-launch decode step (1-4 rows) goes: needs the library built by
    ``python -m jgpt_b200.build --trace`` (loaded through JGPT_B200_LIB).  Generates ``new_tokens`` greedy tokens after a
    prompt (one launch for all steps after the first) and reads every CTA's SM-cycle marks of the second layer of the
    last step: medians over the CTAs that have a unit in the phase."""
    import ctypes as C

    lib = ctx._lib
    if not hasattr(lib, "jgpt_debug_fused_trace_read"):
        raise RuntimeError("this library was not built with --trace (python -m jgpt_b200.build --trace; JGPT_B200_LIB=...)")
    model = make_model(ctx, max_rows=1024)
    try:
        prompt = np.random.default_rng(1).integers(1, VOCAB, prompt_len).astype(np.int32)
        best = 1e9
        for _ in range(3):
            t0 = time.perf_counter()
            model.generateGpuKv(prompt, new_tokens)
            best = min(best, time.perf_counter() - t0)
        buf = np.zeros((256, 24), np.int64)  # the trace array's size; CTAs that do not exist leave their rows zero
        B.check(lib.jgpt_debug_fused_trace_read(buf.ctypes.data_as(C.c_void_p), 256))
        buf = buf[buf.any(axis=1)]
        ns = np.zeros((256, 24), np.int64)  # the same marks on the global timer: comparable across CTAs (0.256 us steps)
        B.check(lib.jgpt_debug_fused_trace_read_ns(ns.ctypes.data_as(C.c_void_p), 256))
        ns = ns[ns.any(axis=1)]
    finally:
        model.close()
    marks = [0, 2, 1, 7, 3, 4, 5, 12, 13, 6, 8, 9, 10, 11]
    names = ["A: wait for the W2 partials + norm", "A: Q,K,V products", "A: sum of the k slices", "A: store + prefetch of Wo",
             "B: attention (incl. the wait for q)", "C: wait for the partials + merge", "C: Wo products", "C: sum of the k slices",
             "C: store + prefetch of W1/W3", "D: wait for the Wo partials + norm", "D: W1/W3 + SwiGLU + store", "E: wait for the activation",
             "E: W2 + store"]
    d = np.diff(buf[:, marks], axis=1).astype(np.float64)
    out = {"workload": f"one-launch decode step, JGPT-35M, batch 1, context ~{prompt_len + new_tokens}: SM-cycle marks of one layer",
           "generate_ms": best * 1e3, "layer_cycles_median": float(np.median(buf[:, 11] - buf[:, 0])), "segments_cycles_median": {}}
    for i, nm in enumerate(names):
        col = d[:, i]
        col = col[(col > 0) & (col < 1e7)]  # CTAs without a unit in the phase leave a mark unset
        out["segments_cycles_median"][nm] = float(np.median(col)) if col.size else None
    # when, over all CTAs, each point of the layer is reached (us after the first CTA starts the layer)
    t0 = ns[:, 0].min()
    points = [(0, "previous layer's W2 results stored"), (2, "A: inputs complete, norm done"), (3, "A: Q,K,V stored"),
              (4, "B: attention partial stored"), (5, "C: partials complete, merged"), (6, "C: Wo results stored"),
              (8, "D: inputs complete, norm done"), (9, "D: activation stored"), (10, "E: activation slice complete"), (11, "E: W2 results stored")]
    out["timeline_us_min_median_max"] = {}
    for mk, nm in points:
        col = ns[:, mk].astype(np.float64)
        col = (col[col > 0] - t0) / 1e3
        out["timeline_us_min_median_max"][nm] = [float(col.min()), float(np.median(col)), float(col.max())]
    # the step's tail: final norm + LM head (1000 units of 8 columns over the CTAs) + argmax
    t0 = ns[:, 16].min()
    points = [(16, "last layer's W2 results stored"), (17, "final norm done"), (18, "logits and per-CTA candidates stored"),
              (19, "tokens picked")]
    out["tail_timeline_us_min_median_max"] = {}
    for mk, nm in points:
        col = ns[:, mk].astype(np.float64)
        col = (col[col > 0] - t0) / 1e3
        out["tail_timeline_us_min_median_max"][nm] = [float(col.min()), float(np.median(col)), float(col.max())]
    return out


def run_step_timeline(ctx, batch=64, ctx_len=512):
    """When each launch of one multi-launch decode step runs: needs the library built by ``python -m jgpt_b200.build
    --trace`` (loaded through JGPT_B200_LIB).  Every projection and attention kernel of that build records, on the global
    timer, when its first CTA came in, when its last CTA was past the wait for the previous kernel and when its last CTA
    left, and which SM each of its first 256 CTAs ran on.  Reported per kind of launch (medians over layers 1..):
    ``early_us`` = how long before the previous kernel's end the first CTA came in (negative: a gap), ``busy_us`` = from
    the later of (own start, previous kernel's end) to the own end, how the CTAs were spread over the SMs, and for the
    projections the split of their time at the end of the k loop (last CTA)."""
    import ctypes as C

    lib = ctx._lib
    if not hasattr(lib, "jgpt_debug_timeline_read"):
        raise RuntimeError("this library was not built with --trace (python -m jgpt_b200.build --trace; JGPT_B200_LIB=...)")
    model = make_model(ctx, max_rows=8192)
    pool = model.newPool(n_blocks=batch * (-(-(ctx_len + 64) // 16)), max_seqs=batch)
    rng = np.random.default_rng(0)
    seqs = [pool.seq_alloc() for _ in range(batch)]
    prompts = [rng.integers(0, VOCAB, ctx_len).astype(np.int32) for _ in range(batch)]
    per_call = max(1, 8192 // ctx_len)
    try:
        toks = np.zeros(batch, np.int32)
        for i in range(0, batch, per_call):
            _, toks[i:i + per_call] = model.forwardPrefillBatch(pool, seqs[i:i + per_call], prompts[i:i + per_call])
        lens = np.full(batch, ctx_len, np.int32)
        for _ in range(10):
            _, toks = model.forwardDecodeBatch(pool, seqs, toks, lens, lens, want_logits=False)
            lens += 1
        ctx.synchronize()
        t0 = time.perf_counter()
        for _ in range(20):
            _, toks = model.forwardDecodeBatch(pool, seqs, toks, lens, lens, want_logits=False)
            lens += 1
        ms = (time.perf_counter() - t0) / 20 * 1e3
        lib.jgpt_debug_timeline_reset()
        model.forwardDecodeBatch(pool, seqs, toks, lens, lens, want_logits=False)
        buf = np.zeros((256, 4), np.uint64)
        n = int(lib.jgpt_debug_timeline_read(buf.ctypes.data_as(C.c_void_p), 256))
        sms = np.zeros((256, 256), np.uint64)
        lib.jgpt_debug_timeline_read_sms(sms.ctypes.data_as(C.c_void_p), 256)
    finally:
        pool.close(), model.close()
    t = buf[:n].astype(np.int64)
    kinds = ["Q,K,V", "attention", "Wo", "W1/W3", "W2"]
    n_layer_launches = n - 1  # the last one is the LM head
    rows = {}
    for i in range(n):
        kind = kinds[i % 5] if i < n_layer_launches else "LM head"
        start, end = t[i, 0], t[i, 2]
        prev_end = t[i - 1, 2] if i else start
        ids = sms[i][sms[i] > 0].astype(np.int64) - 1
        per_sm = np.bincount(ids, minlength=1)
        if i >= 5 or kind == "LM head":
            rows.setdefault(kind, []).append(((prev_end - start) / 1e3, (end - max(prev_end, start)) / 1e3, int(ids.size),
                                              int(np.sum(per_sm > 0)), int(per_sm.max()) if ids.size else 0,
                                              (t[i, 1] - prev_end) / 1e3, (t[i, 3] - t[i, 1]) / 1e3 if t[i, 3] else 0.0, (end - t[i, 3]) / 1e3 if t[i, 3] else 0.0))
    out = {"workload": f"timeline of one multi-launch decode step, JGPT-35M, batch {batch}, context {ctx_len}+ (trace build)",
           "ms_per_step_trace_build": ms, "launches_recorded": n,
           "first_start_to_last_end_us": float((t[n - 1, 2] - t[0, 0]) / 1e3), "per_launch_kind": {}}
    for kind, v in rows.items():
        a = np.asarray(v, np.float64)
        out["per_launch_kind"][kind] = {"launches": len(v), "early_us_median": float(np.median(a[:, 0])), "busy_us_median": float(np.median(a[:, 1])),
                                        "ctas_recorded": int(a[-1, 2]), "sms_used": int(a[-1, 3]), "max_ctas_on_one_sm": int(a[-1, 4]),
                                        "wait_passed_after_prev_end_us": float(np.median(a[:, 5])), "wait_to_k_loop_end_us": float(np.median(a[:, 6])),
                                        "k_loop_end_to_end_us": float(np.median(a[:, 7]))}
    return out


def run_longctx(ctx, rank, world, n_seqs_total=512, steps=20, warmup=3):
    """Decode attention + append at long context: 512 sequences (seed 3) with lengths U[1024, 8192], RoPE positions
    to 8192, dealt in contiguous shards to the ranks; one fused 12-layer launch per step."""
    rng = np.random.default_rng(3)
    lens_all = rng.integers(1024, 8193, n_seqs_total).astype(np.int32)
    per = n_seqs_total // world
    lens = lens_all[rank * per:(rank + 1) * per]
    n = lens.size
    blocks = [-(-int(l) // 16) for l in lens]
    pool = KvPool(ctx, LAYERS, HEADS, DHEAD, sum(blocks), n, 512, max_positions=8192)
    try:
        seqs = []
        for b in blocks:
            s = pool.seq_alloc()
            pool.reserve(s, b * 16)
            seqs.append(s)
        # fill with N(0,1) through the append kernel, one 32768-row slab reused for every chunk of tokens
        slab_rows = 32768
        ks = ctx.from_host(rng.standard_normal((slab_rows, D_MODEL), dtype=np.float32))
        vs = ctx.from_host(rng.standard_normal((slab_rows, D_MODEL), dtype=np.float32))
        seq_of = np.repeat(np.asarray(seqs, np.int32), lens)
        pos_of = np.concatenate([np.arange(l, dtype=np.int32) for l in lens])
        sd, pd = ctx.alloc((slab_rows,), np.int32), ctx.alloc((slab_rows,), np.int32)
        for c0 in range(0, seq_of.size, slab_rows):
            c1 = min(c0 + slab_rows, seq_of.size)
            pad = slab_rows - (c1 - c0)
            sd.copy_from(np.pad(seq_of[c0:c1], (0, pad)))
            pd.copy_from(np.pad(pos_of[c0:c1], (0, pad)))
            for layer in range(LAYERS):
                pool.append(layer, ks, vs, sd, pd, pd, c1 - c0)
        ctx.synchronize()
        q = ctx.from_host(rng.standard_normal((LAYERS, n, D_MODEL), dtype=np.float32))
        k = ctx.from_host(rng.standard_normal((LAYERS, n, D_MODEL), dtype=np.float32))
        v = ctx.from_host(rng.standard_normal((LAYERS, n, D_MODEL), dtype=np.float32))
        out = ctx.alloc((LAYERS, n, D_MODEL))
        seq_d, lens_d = ctx.from_host(np.asarray(seqs, np.int32)), ctx.from_host(lens)
        rope_d = ctx.from_host(lens - 1)
        max_len = int(lens.max())

        def step():
            pool.attn_decode_append(0, LAYERS, q, k, v, seq_d, rope_d, lens_d, n, max_len, out)

        for _ in range(warmup):
            step()
        ctx.synchronize()
        e0, e1 = Event(ctx), Event(ctx)
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        ms = e0.elapsed_ms(e1) / steps
        ctx.synchronize()
        alg = LAYERS * (int(sum(HEADS * (int(l) * DHEAD * 4 + DHEAD * 4 + DHEAD * 4) for l in lens)) + 4 * sum(blocks))
        return {"n_seqs_rank": n, "mean_len": float(lens.mean()), "pool_GB": pool.storage()[1] / 1e9, "ms_per_step": ms,
                "algorithmic_bytes_per_step": alg, "GBps": alg / (ms * 1e-3) / 1e9, "tokens_per_s_rank": n / (ms * 1e-3)}
    finally:
        pool.close()
