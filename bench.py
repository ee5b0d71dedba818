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
# dram__bytes_read.sum + dram__bytes_write.sum of one 12-layer launch of attn_decode_kernel<16,true>
# (ncu capture summarised in profiles/attn_decode_b64_ctx1024.md).
NCU_TRAFFIC_BYTES_PER_LAUNCH = 1_229_597_784


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
def cpu_arm(budget_s: float, threads: int | None = None):
    """Times oracle append + single-query attention on a bounded sample of the workload: one layer of
    the 64 x 24 x 1024 step per repetition; a full step is 12 such layers.  Returns tokens/s."""
    import oracle as O

    if threads:
        O.set_num_threads(threads)
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
                  f"12-layer step, {el:.1f} s on {nthreads} host threads; step time = 12 x layer time",
        "layer_ms": layer_s * 1e3,
    }


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
                "the C restatement of that path (oracle/) on the host cores",
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


def run_gpu(args, rank, world, local_rank):
    import jgpt_b200 as J
    from jgpt_b200.runtime import Event

    dist = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod

        torch.cuda.set_device(local_rank)
        dist_mod.init_process_group("nccl", device_id=torch.device("cuda", local_rank))
        dist = dist_mod

    ctx = J.Context(local_rank)
    lib = ctx._lib
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

    def barrier():
        ctx.synchronize()
        if dist:
            dist.barrier()
            import torch
            torch.cuda.synchronize()

    def max_over_ranks(x):
        if not dist:
            return x
        import torch
        t = torch.tensor([x], dtype=torch.float64, device="cuda")
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

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
    barrier()
    e0, e1 = Event(ctx), Event(ctx)
    t_wall0 = time.time() - 0.3
    e0.record()
    for _ in range(args.steps):
        step_device()
    e1.record()
    ms_total = e0.elapsed_ms(e1)
    barrier()
    t_wall1 = time.time()
    # keep the sampler alive over the end-to-end region as well, then read it for the device region
    ms_total = max_over_ranks(ms_total)
    ms_step = ms_total / args.steps
    launches = args.steps  # one 12-layer attn_decode_kernel<16,true> launch per step

    clocks = sampler.stop(t_wall0, t_wall1) if sampler else None
    if args.quick:
        if rank == 0:
            print(json.dumps({"quick": True, "ms_per_step": ms_step, "GBps": ALG_BYTES_STEP / (ms_step * 1e-3) / 1e9}), flush=True)
        pool.close()
        ctx.close()
        return

    # ---- the same step as the model's forward issues it: one launch per layer, replayed as a CUDA graph
    slab = BATCH * D * 4

    def step_per_layer():
        for layer in range(LAYERS):
            pool.attn_decode_append(layer, 1, q_d.ptr + layer * slab, k_d.ptr + layer * slab, v_d.ptr + layer * slab,
                                    seq_d, rope_d, lens_d, BATCH, CTX_LEN, out_d.ptr + layer * slab)

    step_per_layer()  # sizes the split scratch outside the capture
    ctx.synchronize()
    graph = ctx.capture(step_per_layer)
    for _ in range(8):
        graph.launch()
    barrier()
    e4, e5 = Event(ctx), Event(ctx)
    e4.record()
    for _ in range(args.steps):
        graph.launch()
    e5.record()
    per_layer_ms = max_over_ranks(e4.elapsed_ms(e5) / args.steps)
    barrier()
    graph.close()

    # ---- end to end through the host-buffer entry point -------------------------------------
    for _ in range(12):  # the entry point spends its first nine calls measuring which transfer path is fastest here
        step_host()
    barrier()
    e2e_steps = max(8, min(args.steps, 64))
    t0 = time.perf_counter()
    e2, e3 = Event(ctx), Event(ctx)
    e2.record()
    for _ in range(e2e_steps):
        step_host()
    e3.record()
    e2e_ms = e2.elapsed_ms(e3) / e2e_steps
    e2e_wall_ms = (time.perf_counter() - t0) * 1e3 / e2e_steps
    e2e_ms = max_over_ranks(max(e2e_ms, e2e_wall_ms))
    barrier()

    # sanity: the device and the host paths computed the same thing
    step_device()
    same = bool(np.array_equal(out_d.to_host(), o_h))

    if rank == 0:
        peak, peak_kind = measured_peak_gbs()
        achieved = ALG_BYTES_STEP / (ms_step * 1e-3) / 1e9
        line = {
            "metric": "decode_attention_tokens_per_s", "value": world * BATCH / (ms_step * 1e-3), "unit": "tokens/s",
            "n_gpus": world, "steps": args.steps, "warmup": max(args.warmup, 3), "ms_per_step": ms_step,
            "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16 storage, f32 accumulate",
            "data": "synthetic", "config": workload_config(world), "gpu_launches": launches,
            "e2e": {"value": world * BATCH / (e2e_ms * 1e-3), "unit": "tokens/s", "ms_per_step": e2e_ms,
                    "h2d_bytes_per_step": int(q_h.nbytes + k_h.nbytes + v_h.nbytes + 3 * seq_np.nbytes),
                    "d2h_bytes_per_step": int(o_h.nbytes), "steps": e2e_steps, "host_equals_device": same,
                    "transfer": "jgpt_attn_decode_append_host on pinned host q/k/v/out; the library picks, from its first calls, the "
                                "fastest of: zero-copy (the kernel reads and writes the host buffers over PCIe itself), inputs copied + "
                                "result written in place, staged copies pipelined over layer groups (JGPT_B200_HOST_ZEROCOPY=0/1/2 pins one)"},
            "roofline": {"bound": "hbm", "achieved": achieved, "peak": peak, "unit": "GB/s", "frac": achieved / peak,
                         "peak_kind": f"of {peak_kind}", "frac_of_nominal_8TBs": achieved / 8000.0,
                         "traffic": NCU_TRAFFIC_BYTES_PER_LAUNCH, "kernel": "attn_decode_kernel<16,true>",
                         "algorithmic_bytes_per_launch": ALG_BYTES_STEP, "launch_ms": ms_step},
            "per_layer_launches": {"ms_per_step": per_layer_ms, "launches_per_step": LAYERS, "how": "12 single-layer launches "
                                   "replayed as one CUDA graph (the form the model's forward step uses)",
                                   "GBps": ALG_BYTES_STEP / (per_layer_ms * 1e-3) / 1e9},
            "clocks": clocks,
        }
        if world == 1 and not args.no_cpu:
            cb = cpu_arm(budget_s=args.cpu_seconds)
            line["cpu_baseline"] = {k: cb[k] for k in ("value", "unit", "cores", "kind", "sample")}
        print(json.dumps(line), flush=True)
    pool.close()
    ctx.close()
    if dist:
        dist.destroy_process_group()


def run_secondary(args, rank, world, local_rank):
    """The other named configurations: JGPT-35M batch-1 decode, batch-32 prefill, continuous batching, long context."""
    import jgpt_b200 as J
    from jgpt_b200 import workloads as W

    dist = device = None
    if world > 1:
        import torch
        import torch.distributed as dist_mod

        torch.cuda.set_device(local_rank)
        device = torch.device("cuda", local_rank)
        dist_mod.init_process_group("nccl", device_id=device)
        dist = dist_mod
    ctx = J.Context(local_rank)
    line = {"workload_name": args.workload, "n_gpus": world, "data": "synthetic"}
    if args.workload == "decode35m":
        line.update(W.run_decode35m(ctx))
        if rank == 0 and not args.no_cpu:
            import oracle as O  # CPU baseline leg: the same 35M decode on the host cores, bounded to 16 tokens

            om = O.Model(W.VOCAB, W.CTX, W.D_MODEL, W.HEADS, W.LAYERS, W.D_FF, eps=W.EPS)
            for t, src in zip(om.tensors(), W.jgpt35m_parameters()):
                t[...] = src
            prompt = np.random.default_rng(1).integers(0, W.VOCAB, 64).astype(np.int32)
            t0 = time.perf_counter()
            om.generate_greedy(prompt, 1)
            t1 = time.perf_counter()
            out, n = om.generate_greedy(prompt, 17)
            t2 = time.perf_counter()
            dec = max((t2 - t1) - (t1 - t0), 1e-9) / 16
            line["cpu_baseline"] = {"value": 1.0 / dec, "unit": "tokens/s", "cores": O.num_threads(), "kind": "port",
                                    "sample": "prompt 64 + 16 decode steps of the oracle (fp32, contiguous cache)",
                                    "prefill_ms": (t1 - t0) * 1e3, "first_tokens": out[64:72].tolist()}
    elif args.workload == "decodestep":
        line.update(W.run_decode_step(ctx, batch=args.batch, steps=max(args.steps if args.steps != 256 else 50, 2)))
    elif args.workload == "prefill":
        line.update(W.run_prefill(ctx))
    elif args.workload == "contbatch":
        line.update(W.run_contbatch(ctx, rank, world, dist=dist, device=device))
    else:
        r = W.run_longctx(ctx, rank, world, steps=max(args.steps // 8, 5))
        vals = [r]
        if dist:
            vals = [None] * world
            dist.all_gather_object(vals, r)
        ms = max(v["ms_per_step"] for v in vals)
        alg = sum(v["algorithmic_bytes_per_step"] for v in vals)
        peak, kind = measured_peak_gbs()
        line.update({"workload": "long-context decode attention + append: 512 sequences (seed 3), lengths U[1024, 8192], fp16 paged KV, "
                                 "12 layers x 24 heads x d_head 16, contiguous shards over the GPUs",
                     "ms_per_step_max_over_ranks": ms, "tokens_per_s": sum(v["n_seqs_rank"] for v in vals) / (ms * 1e-3),
                     "aggregate_GBps": alg / (ms * 1e-3) / 1e9, "per_gpu_GBps": alg / world / (ms * 1e-3) / 1e9,
                     "per_gpu_frac_of_peak": alg / world / (ms * 1e-3) / 1e9 / peak, "peak_kind": f"of {kind}", "ranks": vals})
    if rank == 0:
        print(json.dumps(line), flush=True)
    ctx.close()
    if dist:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=8)
    ap.add_argument("--impl", default="b200", choices=["b200", "reference"])
    ap.add_argument("--no-cpu", action="store_true", help="skip the CPU baseline leg")
    ap.add_argument("--cpu-seconds", type=float, default=12.0)
    ap.add_argument("--quick", action="store_true", help="device-resident timing only (used under a profiler)")
    ap.add_argument("--batch", type=int, default=64, help="sequences per step for --workload decodestep")
    ap.add_argument("--workload", default="microbench", choices=["microbench", "decode35m", "decodestep", "prefill", "contbatch", "longctx"],
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
        cmd += ["--workload", args.workload]
        sys.exit(subprocess.call(cmd))
    if args.workload != "microbench":
        run_secondary(args, rank, world, local_rank)
        return
    run_gpu(args, rank, world, local_rank)


if __name__ == "__main__":
    main()
