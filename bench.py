#!/usr/bin/env python
"""Benchmark of the KV-append + decode-attention hot path (one rank per GPU).

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl reference]

Workload (fixed): 12 layers x 24 heads x d_head 16, fp16 paged K/V in blocks of 16 tokens, 64
sequences per GPU at cached length 1024, block table = seeded permutation of a 4096-block pool,
K/V/Q ~ N(0,1).  One step = for every layer, append one new token per sequence (RoPE fused,
re-written at slot 1023 so the length stays 1024 and the pool stays exactly full) and run
single-query attention over the 1024 keys.  Metric: decode-attention tokens/s (sequences advanced
per second), whole job over all ranks.

Prints ONE JSON line on rank 0.  `value` is timed with the step's inputs resident in HBM;
`e2e` goes through the host-buffer entry point (pinned host q/k/v in, output back, every step).
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import statistics
import subprocess
import sys
import threading
import time

import numpy as np

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

LAYERS, HEADS, DHEAD, BATCH, CTX_LEN, BLOCK, POOL_BLOCKS = 12, 24, 16, 64, 1024, 16, 4096
D = HEADS * DHEAD
TABLE_SEED, VALUE_SEED = 1234, 1235
# Algorithmic bytes of one layer of one step: K+V read (fp16), new K,V written, q read + o written
# (counted as fp16 rows), block table read once.
ALG_BYTES_LAYER = BATCH * HEADS * (CTX_LEN * DHEAD * 2 * 2 + DHEAD * 2 * 2 + DHEAD * 2 * 2) + BATCH * (CTX_LEN // BLOCK) * 4
ALG_BYTES_STEP = ALG_BYTES_LAYER * LAYERS
# dram__bytes_read.sum + dram__bytes_write.sum of one 12-layer launch of attn_decode_kernel<16,true>, from an ncu
# capture of this same workload (the launch holds 1.3 GB on the device, so it was captured at full size).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1_231_777_616
MIN_TIMED_MS = 50.0   # every timed figure covers at least this much device time ...
MIN_REPEATS = 5       # ... in at least this many repeats of the --steps region; the median repeat is reported


def measured_peak_gbs():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    try:
        return float(json.load(open(p))["hbm_gbs"]), "measured"
    except Exception:
        return 6650.0, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    Q = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,"
         "clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap")

    def __init__(self, index: int):
        self.rows, self.proc, self.thread = [], None, None
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", str(index), f"--query-gpu={self.Q}", "--format=csv,noheader,nounits",
                                          "-lms", "25"], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except Exception:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            self.rows.append((time.time(), line.strip()))

    def stop(self, t0, t1):
        if not self.proc:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=2)
        except Exception:
            self.proc.kill()
        sm, mx, reasons, n_in = [], None, set(), 0
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        rows = [r for r in self.rows if t0 - 0.15 <= r[0] <= t1 + 0.15] or self.rows
        for _, line in rows:
            f = [x.strip() for x in line.split(",")]
            if len(f) < 7:
                continue
            try:
                sm.append(float(f[0]))
                mx = float(f[1])
            except ValueError:
                continue
            n_in += 1
            for name, val in zip(names, f[3:7]):
                if val.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(sm) if sm else None, "sm_max_mhz": mx, "reasons": sorted(reasons), "samples": n_in}


def pinned_array(lib, shape, dtype):
    n = int(np.prod(shape)) * np.dtype(dtype).itemsize
    p = C.c_void_p()
    rc = lib.jgpt_host_alloc_pinned(n, C.byref(p))
    if rc:
        raise MemoryError("pinned host allocation failed")
    buf = (C.c_char * n).from_address(p.value)
    return np.frombuffer(buf, dtype=dtype).reshape(shape)


# ------------------------------------------------------------------------------------------------
# CPU arm: the oracle (C restatement of the reference path) timed on the host cores.
# ------------------------------------------------------------------------------------------------
def cpu_arm(budget_s: float, threads: int | None = None, timing_build: bool = True):
    """Times oracle append + single-query attention on a bounded sample of the workload: one layer of
    the 64 x 24 x 1024 step per repetition; a full step is 12 such layers.  Returns tokens/s.

    threads = None: every host core (set explicitly: a launcher such as torchrun exports OMP_NUM_THREADS=1 to
    its ranks).  timing_build: the same C file compiled -O3 -march=native on this machine, used for TIMING only;
    the strict-floating-point build stays the checker."""
    import oracle as O

    if timing_build:
        O.use_timing_build()
    O.set_num_threads(threads or os.cpu_count() or 1)
    nthreads = O.num_threads()
    rng = np.random.default_rng(VALUE_SEED)
    kc = O.round_fp16(rng.standard_normal((BATCH, HEADS, CTX_LEN, DHEAD), dtype=np.float32))
    vc = O.round_fp16(rng.standard_normal((BATCH, HEADS, CTX_LEN, DHEAD), dtype=np.float32))
    q, k, v = (rng.standard_normal((BATCH, D), dtype=np.float32) for _ in range(3))
    lens = np.full(BATCH, CTX_LEN - 1, np.int32)
    rope = np.full(BATCH, CTX_LEN - 1, np.int32)
    O.decode_attn_batch(q, k, v, kc, vc, lens, rope, HEADS, DHEAD, CTX_LEN)  # warm
    reps, t0 = 0, time.perf_counter()
    while True:
        O.decode_attn_batch(q, k, v, kc, vc, lens, rope, HEADS, DHEAD, CTX_LEN)
        reps += 1
        el = time.perf_counter() - t0
        if el > budget_s or reps >= 2000:
            break
    layer_s = el / reps
    return {
        "value": BATCH / (layer_s * LAYERS), "unit": "tokens/s", "cores": nthreads, "kind": "port",
        "sample": f"{reps} repetitions of one layer (64 seqs x 24 heads x 1024 keys, append + attention) of the "
                  f"12-layer step, {el:.1f} s on {nthreads} host thread(s); step time = 12 x layer time; C restatement "
                  f"of the reference path built {'-O3 -march=native' if timing_build else 'as the checker (-O2, strict fp)'}",
        "layer_ms": layer_s * 1e3,
    }


def cpu_baseline_block(budget_s: float):
    """All-core and single-thread figures of the CPU restatement (the reference runs one inference thread)."""
    multi = cpu_arm(budget_s * 0.6)
    single = cpu_arm(budget_s * 0.4, threads=1)
    out = {k: multi[k] for k in ("value", "unit", "cores", "kind", "sample")}
    out["single_thread"] = {k: single[k] for k in ("value", "unit", "cores", "sample")}
    return out


def run_reference(args, rank):
    if rank != 0:
        return
    cb = cpu_arm(budget_s=min(20.0, max(2.0, 2.0 * args.steps)))
    step_ms = cb["layer_ms"] * LAYERS
    line = {
        "impl": "reference", "metric": "decode_attention_tokens_per_s", "value": cb["value"], "unit": "tokens/s",
        "n_gpus": args.gpus, "steps": args.steps, "warmup": args.warmup, "ms_per_step": step_ms,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32", "data": "synthetic",
        "config": workload_config(args.gpus),
        "cpu_baseline": {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")},
        "e2e": {"value": cb["value"], "unit": "tokens/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "note": "the reference's own Java path cannot run here (no JDK; every op is a JNI call into CUDA): this arm times "
                "the C restatement of that path (oracle/) on all host cores of the box (one CPU job however many GPUs "
                "the other arm uses)",
    }
    print(json.dumps(line), flush=True)


def workload_config(n_gpus):
    return {
        "workload": "kv_append+decode_attention microbench: 12 layers x 24 heads x d_head 16, fp16 paged KV (16-token blocks, "
                    "seeded permutation of a 4096-block pool), batch 64 per GPU, cached length 1024, 1 token appended per "
                    "sequence per step then single-query attention",
        "layers": LAYERS, "heads": HEADS, "d_head": DHEAD, "batch_per_gpu": BATCH, "context": CTX_LEN, "block_tokens": BLOCK,
        "pool_blocks": POOL_BLOCKS, "layers_per_launch": LAYERS, "parallelism": f"sequence-sharded x{n_gpus}, no data-path collective",
        "l2": "inputs larger than L2 (1.2 GB of K/V touched per step)", "table_seed": TABLE_SEED, "value_seed": VALUE_SEED,
    }


# ------------------------------------------------------------------------------------------------
# GPU arm
# ------------------------------------------------------------------------------------------------
def build_workload(ctx, rank):
    import jgpt_b200 as J

    pool = J.KvPool(ctx, LAYERS, HEADS, DHEAD, POOL_BLOCKS, BATCH, CTX_LEN // BLOCK, max_positions=CTX_LEN)
    perm = np.random.default_rng(TABLE_SEED + rank).permutation(POOL_BLOCKS).astype(np.int32).reshape(BATCH, CTX_LEN // BLOCK)
    seqs = []
    for i in range(BATCH):
        s = pool.seq_alloc()
        pool.set_block_table(s, perm[i])
        pool.set_length(s, CTX_LEN)
        seqs.append(s)
    rng = np.random.default_rng(VALUE_SEED + rank)
    # Fill the cache through the append kernel: all 1024 positions of all 64 sequences, every layer.
    tot = BATCH * CTX_LEN
    seq_ids = ctx.from_host(np.repeat(np.asarray(seqs, np.int32), CTX_LEN))
    pos = ctx.from_host(np.tile(np.arange(CTX_LEN, dtype=np.int32), BATCH))
    kslab = rng.standard_normal((tot, D), dtype=np.float32)
    vslab = rng.standard_normal((tot, D), dtype=np.float32)
    kd, vd = ctx.alloc((tot, D)), ctx.alloc((tot, D))
    for layer in range(LAYERS):
        kd.copy_from(np.roll(kslab, layer * 17, axis=0))
        vd.copy_from(np.roll(vslab, layer * 29, axis=0))
        pool.append(layer, kd, vd, seq_ids, pos, pos, tot)
    ctx.synchronize()
    kd.close(), vd.close(), seq_ids.close(), pos.close()
    return pool, seqs, rng


class Ranks:
    """Barrier and small reductions between the ranks of one job through the library's own NCCL communicator
    (`jgpt_comm_*`): an all-gather that every rank must join is a barrier; doubles travel as two int32 words."""

    def __init__(self, ctx, rank, world):
        from jgpt_b200.scheduler import TokenGather, rendezvous_unique_id

        self.ctx, self.rank, self.world, self.g, self.uid = ctx, rank, world, None, None
        if world > 1:
            key = f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}"  # same for the ranks of one launch, new per launch
            self.uid = rendezvous_unique_id(rank, world, key)
            self.g = TokenGather(ctx, world, rank, max_pairs=15, unique_id=self.uid, depth=0, timeout_ms=180000)
            if rank == 0:  # every rank has joined by now
                from jgpt_b200.scheduler import rendezvous_cleanup

                rendezvous_cleanup(key)

    def all_gather_f64(self, values):
        v = np.asarray(values, np.float64).reshape(-1)
        if not self.g:
            return v[None, :].copy()
        w = v.view(np.int32)
        self.g.submit_words(w)
        words, counts = self.g.pop_words()
        return np.stack([np.ascontiguousarray(words[r, :counts[r]]).view(np.float64) for r in range(self.world)])

    def barrier(self):
        self.ctx.synchronize()
        if self.g:
            self.all_gather_f64([0.0])

    def max(self, x):
        return float(self.all_gather_f64([x]).max())

    def close(self):
        if self.g:
            self.g.close()


def timed_median(ctx, ranks, step, steps, est_ms=None):
    """Median over repeats of the device time of `steps` back-to-back calls of `step`, each repeat bracketed by CUDA
    events on the library's stream and reduced with max over ranks.  At least MIN_REPEATS repeats, and enough of them
    that the timed regions add up to MIN_TIMED_MS.  Returns (ms per step, repeats, [ms per step of every repeat])."""
    from jgpt_b200.runtime import Event

    e0, e1 = Event(ctx), Event(ctx)
    if est_ms is None:
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        est_ms = ranks.max(e0.elapsed_ms(e1)) / steps
    repeats = int(min(200, max(MIN_REPEATS, np.ceil(MIN_TIMED_MS / max(est_ms * steps, 1e-6)))))
    per = []
    for _ in range(repeats):
        ranks.barrier()
        e0.record()
        for _ in range(steps):
            step()
        e1.record()
        per.append(ranks.max(e0.elapsed_ms(e1)) / steps)
    ranks.barrier()
    return statistics.median(per), repeats, per


def run_model_decode(ctx, ranks, batch=64, ctx_len=512, steps=40):
    """Full-model decode step (JGPT-35M shapes): token ids in, sampled ids out, then the ids of every rank gathered by
    the library's communicator straight from the device buffer the sampler wrote.  Host clock: the step synchronises."""
    from jgpt_b200 import binding as B
    from jgpt_b200 import workloads as W
    from jgpt_b200.scheduler import TokenGather

    model = W.make_model(ctx, max_rows=8192)
    pool = model.newPool(n_blocks=batch * (-(-(ctx_len + steps + 16) // 16)), max_seqs=batch)
    rng = np.random.default_rng(100 + ranks.rank)
    seqs = [pool.seq_alloc() for _ in range(batch)]
    prompts = [rng.integers(0, W.VOCAB, ctx_len).astype(np.int32) for _ in range(batch)]
    per_call = max(1, 8192 // ctx_len)
    gather = TokenGather(ctx, ranks.world, ranks.rank, max_pairs=batch // 2, unique_id=None, depth=4) if ranks.world == 1 else None
    if ranks.world > 1:
        # a second communicator for the ids (the first one carries the bench's barriers): same rendezvous route
        from jgpt_b200.scheduler import rendezvous_unique_id

        key = f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}_ids"
        uid = rendezvous_unique_id(ranks.rank, ranks.world, key)
        gather = TokenGather(ctx, ranks.world, ranks.rank, max_pairs=batch // 2, unique_id=uid, depth=4, timeout_ms=120000)
    try:
        toks = np.zeros(batch, np.int32)
        for i in range(0, batch, per_call):
            _, toks[i:i + per_call] = model.forwardPrefillBatch(pool, seqs[i:i + per_call], prompts[i:i + per_call])
        lens = np.full(batch, ctx_len, np.int32)
        seq_ids = np.asarray(seqs, np.int32)  # converted once, not per step
        dev_next = C.c_void_p()
        B.check(ctx._lib.jgpt_model_next_tokens_device(model.handle, C.byref(dev_next)))
        gathered = 0

        def one_step():
            nonlocal toks, gathered
            _, toks = model.forwardDecodeBatch(pool, seq_ids, toks, lens, lens, want_logits=False)
            lens[:] += 1
            gather.submit_device(dev_next.value, batch)
            while gather.ready():
                _, counts = gather.pop_words()
                gathered += int(counts.sum())

        for _ in range(4):
            one_step()
        ranks.barrier()
        t0 = time.perf_counter()
        for _ in range(steps):
            one_step()
        while gather.in_flight():
            _, counts = gather.pop_words()
            gathered += int(counts.sum())
        el = ranks.max(time.perf_counter() - t0) / steps
        # the reference's own use: one sequence, greedy, prompt 64 + 128 tokens through generateGpuKv (every rank its own)
        pool1 = model.newPool(n_blocks=W.CTX // 16, max_seqs=1)
        try:
            prompt = np.random.default_rng(1).integers(0, W.VOCAB, 64).astype(np.int32)
            model.generateGpuKv(prompt, 8, pool=pool1)
            ranks.barrier()
            best_total = best_prefill = 1e30
            for _ in range(3):
                ta = time.perf_counter()
                model.generateGpuKv(prompt, 1, pool=pool1)
                tb = time.perf_counter()
                model.generateGpuKv(prompt, 128, pool=pool1)
                tc = time.perf_counter()
                best_prefill, best_total = min(best_prefill, tb - ta), min(best_total, tc - tb)
            per_tok = ranks.max(max(best_total - best_prefill, 1e-9) / 127)
        finally:
            pool1.close()
        return {"what": f"JGPT-35M full decode step through jgpt_forward_decode: batch {batch} per GPU, context {ctx_len}+, ids in, "
                        "sampled ids out and fed back; every rank's ids all-gathered by jgpt_comm_submit_device (read 4 steps later)",
                "ms_per_step": el * 1e3, "tokens_per_s": ranks.world * batch / el, "steps": steps, "ids_gathered": gathered,
                "timing": "host wall clock over the steps (each step synchronises to read its ids), max over ranks",
                "greedy_batch1": {"what": "one sequence per GPU, prompt 64 (seed 1) + 128 greedy tokens through jgpt_generate_greedy "
                                          "(decode part: total minus a prefill-only call; best of 3, max over ranks)",
                                  "ms_per_token": per_tok * 1e3, "tokens_per_s": ranks.world / per_tok}}
    finally:
        gather.close(), pool.close(), model.close()


def run_gpu(args, rank, world, local_rank):
    import jgpt_b200 as J
    from jgpt_b200.runtime import Event

    from jgpt_b200.runtime import bind_host_near_gpu

    numa = bind_host_near_gpu(local_rank)  # before any page-locked allocation: the host buffers land next to the GPU
    ctx = J.Context(local_rank)
    lib = ctx._lib
    ranks = Ranks(ctx, rank, world)
    pool, seqs, rng = build_workload(ctx, rank)

    q_h = pinned_array(lib, (LAYERS, BATCH, D), np.float32)
    k_h = pinned_array(lib, (LAYERS, BATCH, D), np.float32)
    v_h = pinned_array(lib, (LAYERS, BATCH, D), np.float32)
    o_h = pinned_array(lib, (LAYERS, BATCH, D), np.float32)
    for a in (q_h, k_h, v_h):
        a[...] = rng.standard_normal(a.shape, dtype=np.float32)
    q_d, k_d, v_d = ctx.from_host(q_h), ctx.from_host(k_h), ctx.from_host(v_h)
    out_d = ctx.alloc((LAYERS, BATCH, D))
    seq_np = np.asarray(seqs, np.int32)
    lens_np = np.full(BATCH, CTX_LEN, np.int32)
    rope_np = np.full(BATCH, CTX_LEN - 1, np.int32)
    seq_d, lens_d, rope_d = ctx.from_host(seq_np), ctx.from_host(lens_np), ctx.from_host(rope_np)

    def step_device():
        pool.attn_decode_append(0, LAYERS, q_d, k_d, v_d, seq_d, rope_d, lens_d, BATCH, CTX_LEN, out_d)

    def step_host():
        pool.attn_decode_append_host(0, LAYERS, q_h, k_h, v_h, seq_np, rope_np, lens_np, out=o_h)

    # ---- device-resident timing -------------------------------------------------------------
    sampler = ClockSampler(local_rank) if rank == 0 else None
    warm = max(args.warmup, 3)
    for _ in range(warm):
        step_device()
    ctx.synchronize()
    # keep the GPU under the same load for ~0.4 s more so the clock samples describe steady state
    t_w = time.time()
    while not args.quick and time.time() - t_w < 0.4:
        for _ in range(16):
            step_device()
        ctx.synchronize()
    ranks.barrier()
    t_wall0 = time.time() - 0.3
    if args.quick:
        slab_q = BATCH * D * 4

        def step_quick_per_layer():
            for layer in range(LAYERS):
                pool.attn_decode_append(layer, 1, q_d.ptr + layer * slab_q, k_d.ptr + layer * slab_q, v_d.ptr + layer * slab_q,
                                        seq_d, rope_d, lens_d, BATCH, CTX_LEN, out_d.ptr + layer * slab_q)

        if args.per_layer:
            pool.set_tuning(launch_overlap=args.launch_overlap)
            step_device = step_quick_per_layer
            step_device()
            ctx.synchronize()
        e0, e1 = Event(ctx), Event(ctx)
        e0.record()
        for _ in range(args.steps):
            step_device()
        e1.record()
        ms_step = e0.elapsed_ms(e1) / args.steps
        if rank == 0:
            print(json.dumps({"quick": True, "ms_per_step": ms_step, "GBps": ALG_BYTES_STEP / (ms_step * 1e-3) / 1e9}), flush=True)
        pool.close(), ranks.close(), ctx.close()
        return
    ms_step, repeats, per_repeat = timed_median(ctx, ranks, step_device, args.steps)
    t_wall1 = time.time()
    launches = args.steps  # one 12-layer attn_decode_kernel<16,true> launch per step (per timed repeat)
    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None

    # ---- the same step as the model's forward issues it: one launch per layer, replayed as a CUDA graph
    slab = BATCH * D * 4

    def step_per_layer():
        for layer in range(LAYERS):
            pool.attn_decode_append(layer, 1, q_d.ptr + layer * slab, k_d.ptr + layer * slab, v_d.ptr + layer * slab,
                                    seq_d, rope_d, lens_d, BATCH, CTX_LEN, out_d.ptr + layer * slab)

    # In this loop the kernel in front of every attention launch is another layer's attention: it writes neither this
    # layer's K/V nor the tables nor the index arrays, which is what launch_overlap = 2 asks the caller to promise (in
    # the model's step the kernel in front is the Q,K,V projection: the same holds).
    pool.set_tuning(launch_overlap=2)
    step_per_layer()  # sizes the split scratch outside the capture
    ctx.synchronize()
    graph = ctx.capture(step_per_layer)
    for _ in range(8):
        graph.launch()
    per_layer_ms, _, _ = timed_median(ctx, ranks, graph.launch, args.steps)
    graph.close()

    # ---- end to end through the host-buffer entry point -------------------------------------
    for _ in range(12):  # the entry point spends its first nine calls measuring which transfer path is fastest here
        step_host()
    e2e_steps = max(8, min(args.steps, 64))
    e2e_per = []
    for _ in range(MIN_REPEATS):
        ranks.barrier()
        t0 = time.perf_counter()
        e2, e3 = Event(ctx), Event(ctx)
        e2.record()
        for _ in range(e2e_steps):
            step_host()
        e3.record()
        dev_ms = e2.elapsed_ms(e3) / e2e_steps
        wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
        e2e_per.append(ranks.max(max(dev_ms, wall_ms)))
    e2e_ms = statistics.median(e2e_per)
    ranks.barrier()

    # sanity: the device and the host paths computed the same thing
    step_device()
    same = bool(np.array_equal(out_d.to_host(), o_h))
    pool.close()

    # ---- the path a generation loop takes: full-model decode step + token-id gather; continuous batching ----
    extras = {}
    if not args.no_model:
        from jgpt_b200 import workloads as W

        extras["model_decode"] = run_model_decode(ctx, ranks)
        uid2 = None
        if world > 1:
            from jgpt_b200.scheduler import rendezvous_unique_id

            uid2 = rendezvous_unique_id(rank, world, f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}_cb")
        ranks.barrier()
        cb = W.run_contbatch(ctx, rank, world, unique_id=uid2, gather_depth=args.gather_depth)
        cb_s = ranks.max(cb["seconds"])
        extras["contbatch"] = {"what": cb["workload"], "generated_tokens": cb["generated_tokens"], "seconds": cb_s,
                               "tokens_per_s": cb["generated_tokens"] / cb_s, "steps_rank0": cb["steps"],
                               "evictions_rank0": cb["evictions_rank0"], "scaling": "strong (256 requests in total)",
                               "timing": cb["timing"] + ", max over ranks"}

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        achieved = ALG_BYTES_STEP / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "decode_attention_tokens_per_s", "value": world * BATCH / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "repeats": repeats, "ms_per_step_min_max": [min(per_repeat), max(per_repeat)],
            "timing": f"median of {repeats} repeats of the {args.steps}-step region (CUDA events on the library's stream, max over "
                      f"ranks per repeat); the repeats cover >= {MIN_TIMED_MS:.0f} ms of device time",
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate",
            "data": "synthetic", "config": workload_config(world), "gpu_launches": launches,
            "e2e": {"value": world * BATCH / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(q_h.nbytes + k_h.nbytes + v_h.nbytes + 3 * seq_np.nbytes),
                    "d2h_bytes_per_step": int(o_h.nbytes), "steps": e2e_steps, "repeats": MIN_REPEATS, "host_equals_device": same,
                    "transfer": "jgpt_attn_decode_append_host on pinned host q/k/v/out; the library picks, from its first calls, the "
                                "fastest of: zero-copy (the kernel reads and writes the host buffers over PCIe itself), inputs copied + "
                                "result written in place, staged copies pipelined over layer groups (JGPT_B200_HOST_ZEROCOPY=0/1/2 pins one)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / 8000.0,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "kernel": "attn_decode_kernel<16,true>",
                         "algorithmic_bytes_per_launch": ALG_BYTES_STEP, "launch_ms": ms_step},
            "per_layer_launches": {"ms_per_step": per_layer_ms, "launches_per_step": LAYERS, "how": "12 single-layer launches "
                                   "replayed as one CUDA graph (the form the model's forward step uses), each a programmatic "
                                   "dependent launch whose copy warp fetches tables and K/V while the previous layer drains "
                                   "(jgpt_kvpool_set_tuning launch_overlap = 2)",
                                   "GBps": ALG_BYTES_STEP / (per_layer_ms * 1e-3) / 1e9,
                                   "frac_of_measured": ALG_BYTES_STEP / (per_layer_ms * 1e-3) / 1e9 / peak,
                                   "frac_of_nominal_8TBs": ALG_BYTES_STEP / (per_layer_ms * 1e-3) / 1e9 / 8000.0},
            "host_binding": numa, "clocks": clocks, "ranks_joined_by": "jgpt_comm (NCCL inside the library)" if world > 1 else "single rank",
        }
        line.update(extras)
        if not args.no_cpu:
            line["cpu_baseline"] = cpu_baseline_block(args.cpu_seconds)
        print(json.dumps(line), flush=True)
    ranks.barrier()
    ranks.close()
    ctx.close()


def run_secondary(args, rank, world, local_rank):
    """The other named configurations: JGPT-35M batch-1 decode, batch-32 prefill, continuous batching, long context,
    and the standalone K/V store kernels."""
    import jgpt_b200 as J
    from jgpt_b200 import workloads as W

    ctx = J.Context(local_rank)
    ranks = Ranks(ctx, rank, world)
    line = {"workload_name": args.workload, "n_gpus": world, "data": "synthetic"}
    if args.workload == "decode35m":
        line.update(W.run_decode35m(ctx))
        if rank == 0 and not args.no_cpu:
            import oracle as O  # CPU baseline leg: the same 35M decode on the host cores, bounded to 16 tokens

            O.use_timing_build()
            O.set_num_threads(os.cpu_count() or 1)
            om = O.Model(W.VOCAB, W.CTX, W.D_MODEL, W.HEADS, W.LAYERS, W.D_FF, eps=W.EPS)
            for t, src in zip(om.tensors(), W.jgpt35m_parameters()):
                t[...] = src
            prompt = np.random.default_rng(1).integers(0, W.VOCAB, 64).astype(np.int32)
            res = {}
            for label, nthr in (("all_cores", os.cpu_count() or 1), ("single_thread", 1)):
                O.set_num_threads(nthr)
                t0 = time.perf_counter()
                om.generate_greedy(prompt, 1)
                t1 = time.perf_counter()
                out, n = om.generate_greedy(prompt, 17)
                t2 = time.perf_counter()
                dec = max((t2 - t1) - (t1 - t0), 1e-9) / 16
                res[label] = {"value": 1.0 / dec, "unit": "tokens/s", "cores": O.num_threads(), "ms_per_token": dec * 1e3,
                              "prefill_ms": (t1 - t0) * 1e3}
            line["cpu_baseline"] = {**res["all_cores"], "kind": "port", "single_thread": res["single_thread"],
                                    "sample": "prompt 64 + 16 decode steps of the oracle (fp32, contiguous cache), -O3 -march=native",
                                    "first_tokens": out[64:72].tolist()}
    elif args.workload == "decodestep":
        line.update(W.run_decode_step(ctx, batch=args.batch, steps=max(args.steps if args.steps != 256 else 50, 2)))
    elif args.workload == "prefill":
        line.update(W.run_prefill(ctx))
    elif args.workload == "kvstore":
        line.update(W.run_kvstore(ctx))
    elif args.workload == "phases":
        pool, seqs, _ = build_workload(ctx, rank)
        line["workload"] = "per-CTA phase timing of per-layer decode-attention launches (batch 64, context 1024; trace build)"
        line["overlap_2"] = W.run_phases(ctx, pool, seqs, BATCH, LAYERS, D, CTX_LEN, overlap=2)
        line["overlap_0"] = W.run_phases(ctx, pool, seqs, BATCH, LAYERS, D, CTX_LEN, overlap=0)
        pool.close()
    elif args.workload == "fusedphases":
        line.update(W.run_fused_phases(ctx))
    elif args.workload == "steptimeline":
        line.update(W.run_step_timeline(ctx, batch=args.batch))
    elif args.workload == "contbatch":
        uid = None
        if world > 1:
            from jgpt_b200.scheduler import rendezvous_unique_id

            uid = rendezvous_unique_id(rank, world, f"{os.environ.get('MASTER_PORT', '0')}_{os.getppid()}_cb")
        ranks.barrier()
        r = W.run_contbatch(ctx, rank, world, unique_id=uid, gather_depth=args.gather_depth)
        sec = ranks.max(r["seconds"])
        r["seconds_max_over_ranks"], r["tokens_per_s"] = sec, r["generated_tokens"] / sec
        line.update(r)
    else:
        r = W.run_longctx(ctx, rank, world, steps=max(args.steps // 8, 5))
        g = ranks.all_gather_f64([r["ms_per_step"], r["algorithmic_bytes_per_step"], r["n_seqs_rank"], r["mean_len"], r["pool_GB"]])
        ms, alg = float(g[:, 0].max()), float(g[:, 1].sum())
        peak, kind = measured_peak_gbs()
        line.update({"workload": "long-context decode attention + append: 512 sequences (seed 3), lengths U[1024, 8192], fp16 paged KV, "
                                 "12 layers x 24 heads x d_head 16, contiguous shards over the GPUs",
                     "ms_per_step_max_over_ranks": ms, "tokens_per_s": float(g[:, 2].sum()) / (ms * 1e-3),
                     "aggregate_GBps": alg / (ms * 1e-3) / 1e9, "per_gpu_GBps": alg / world / (ms * 1e-3) / 1e9,
                     "per_gpu_frac_of_peak": alg / world / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}",
                     "ranks": [{"ms_per_step": float(a[0]), "n_seqs": int(a[2]), "mean_len": float(a[3]), "pool_GB": float(a[4])} for a in g]})
    if rank == 0:
        print(json.dumps(line), flush=True)
    ranks.barrier()
    ranks.close()
    ctx.close()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--no-model", action="store_true", help="skip the full-model decode step and continuous-batching legs")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--quick", action="store_true", help="device-resident timing only (used under a profiler)")
    ap.add_argument("--per-layer", action="store_true", help="with --quick: one launch per layer instead of one per step")
    ap.add_argument("--launch-overlap", type=int, default=2, help="with --quick --per-layer: 0 ordinary launches, 1 / 2 overlapped")
    ap.add_argument("--batch", type=int, default=64, help="sequences per step for --workload decodestep")
    ap.add_argument("--gather-depth", type=int, default=4, help="continuous batching: steps a rank may run ahead of the token-id gather")
    ap.add_argument("--workload", default="microbench", choices=["microbench", "decode35m", "decodestep", "prefill", "contbatch", "longctx", "kvstore", "phases", "fusedphases", "steptimeline"],
                    help="microbench (default) is the headline KV-append + decode-attention step; the others are the "
                         "remaining named configurations (reported, not the contract line)")
    args = ap.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    if args.impl == "reference":
        run_reference(args, rank)
        return
    if world == 1 and args.gpus > 1:
        # launched without torchrun: re-launch one rank per GPU
        cmd = [sys.executable, "-m", "torch.distributed.run", "--nnodes=1", f"--nproc-per-node={args.gpus}",
               "--master-addr", "127.0.0.1", "--master-port", os.environ.get("MASTER_PORT", "29511"), os.path.abspath(__file__),
               "--gpus", str(args.gpus), "--steps", str(args.steps), "--warmup", str(args.warmup)]
        if args.no_cpu:
            cmd.append("--no-cpu")
        if args.no_model:
            cmd.append("--no-model")
        cmd += ["--workload", args.workload]
        sys.exit(subprocess.call(cmd))
    if args.workload != "microbench":
        run_secondary(args, rank, world, local_rank)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
