"""The library's token-id gather (`jgpt_comm_*`, NCCL opened at run time) through the C ABI.

One rank: the ring of in-flight steps, ordering, device-side submission and the argument checks, on one
GPU (a single rank needs no NCCL).  Two ranks: child processes on two GPUs over NCCL (skipped on a
one-GPU box): identical results in (rank, local order) on both ranks, a finished rank that keeps reporting
the sentinel, and the host-side timeout -- a rank that submits LATE makes the other rank's bounded read
return TimeoutError instead of blocking, and the same read succeeds once the late rank has arrived.  No
rank ever stays away from a collective, so no kernel is left waiting on the GPU.  NVLS is switched off
for the children."""
import os
import subprocess
import sys

import numpy as np
import pytest

import jgpt_b200 as J
from jgpt_b200.scheduler import TokenGather

pytestmark = pytest.mark.gpu
ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_single_rank_ring_order_and_checks(ctx):
    g = TokenGather(ctx, 1, 0, max_pairs=4, depth=2)
    try:
        assert g.in_flight() == 0 and not g.ready()
        with pytest.raises(RuntimeError, match="no step is in flight"):
            g.pop()
        g.submit([(3, 7)]), g.submit([(5, 0), (6, 1)])
        assert g.in_flight() == 2 and not g.ready()
        g.submit([], done=True)
        assert g.ready()  # more than `depth` in flight: read one before the next submit
        g.submit([(9, 9)])  # the ring has depth + 2 slots
        with pytest.raises(RuntimeError, match="in flight"):
            g.submit([(1, 1)])
        assert g.pop() == [(3, 7)] and g.pop() == [(5, 0), (6, 1)] and g.pop() == [(-1, 1)]
        assert g.drain() == [[(9, 9)]]
        with pytest.raises(ValueError, match="exceed the gather buffer"):
            g.submit([(i, i) for i in range(6)])
        # words that a kernel leaves on the device: gathered after the stream's earlier work, no host round trip
        dev = ctx.from_host(np.array([11, 22, 33, 44], np.int32))
        g.submit_device(dev.ptr, 4)
        words, counts = g.pop_words()
        assert counts.tolist() == [4] and words[0, :4].tolist() == [11, 22, 33, 44] and (words[0, 4:] == -1).all()
    finally:
        g.close()


def test_device_submit_carries_the_sampled_ids_of_a_forward_step(ctx):
    """jgpt_model_next_tokens_device + jgpt_comm_submit_device: what forward_decode sampled is what the gather returns."""
    import ctypes as C
    from jgpt_b200 import binding as B

    import oracle as O

    om = O.Model(64, 32, 32, 4, 2, 64, eps=1e-6).init_random(seed=5, std=0.2)
    m = J.GPTModel(ctx, 64, 32, 32, 4, 2, 64, rmsNormEps=1e-6)
    m.setParameters(om.tensors())
    om.close()
    pool = m.newPool(n_blocks=8, max_seqs=3)
    g = TokenGather(ctx, 1, 0, max_pairs=8, depth=1)
    try:
        seqs = [pool.seq_alloc() for _ in range(3)]
        prompts = [np.array([1, 2, 3], np.int32), np.array([4, 5], np.int32), np.array([6], np.int32)]
        _, nxt = m.forwardPrefillBatch(pool, seqs, prompts)
        lens = [3, 2, 1]
        _, nxt2 = m.forwardDecodeBatch(pool, seqs, nxt, lens, lens)
        p = C.c_void_p()
        B.check(ctx._lib.jgpt_model_next_tokens_device(m.handle, C.byref(p)))
        g.submit_device(p.value, 3)
        words, counts = g.pop_words()
        assert counts.tolist() == [3] and words[0, :3].tolist() == list(nxt2)
    finally:
        g.close(), pool.close(), m.close()


_WORKER = r"""
import os, sys, time
sys.path.insert(0, {root!r})
import numpy as np
import jgpt_b200 as J
from jgpt_b200.scheduler import TokenGather, shard_requests
rank, world, n_req = int(sys.argv[1]), 2, 11
uid = bytes.fromhex(sys.argv[2])
ctx = J.Context(rank)
g = TokenGather(ctx, world, rank, max_pairs=8, unique_id=uid, depth=3, timeout_ms=20000)
mine = shard_requests(n_req, world, rank)
my_steps = 9 if rank == 0 else 5            # rank 1 finishes earlier and keeps reporting "done"
seen, all_done, step = [], False, 0
def account(pairs):
    global all_done
    seen.append([p for p in pairs if p[0] >= 0])
    all_done = all_done or sum(1 for p in pairs if p[0] < 0) == world
while not all_done:
    done = step >= my_steps
    local = [] if done else [(r, (r * 31 + step * 7) % 100) for r in mine if (r + step) % 3 != 0]
    if rank == 1 and step % 2 == 0:
        time.sleep(0.02)                    # uneven step times: the ranks drift within the window
    g.submit(local, done=done)
    step += 1
    while g.ready() and not all_done:
        account(g.pop())
for pairs in g.drain():
    account(pairs)
want = [[(r, (r * 31 + t * 7) % 100) for rk in range(world) for r in shard_requests(n_req, world, rk)
         if t < (9 if rk == 0 else 5) and (r + t) % 3 != 0] for t in range(len(seen))]
ok = seen == want and len(seen) >= 10 and step == len(seen)

# host-side timeout: rank 1 arrives 1.5 s late; rank 0's 200 ms read gives up, stays usable, and then succeeds
timed_out = False
if rank == 1:
    time.sleep(1.5)
g.submit([(100 + rank, 7)])
if rank == 0:
    try:
        g.pop(timeout_ms=200)
    except TimeoutError:
        timed_out = True
    late = g.pop(timeout_ms=20000)
    ok = ok and timed_out and late == [(100, 7), (101, 7)]
else:
    ok = ok and g.pop(timeout_ms=20000) == [(100, 7), (101, 7)]
g.close()
ctx.close()
print("OK" if ok else "MISMATCH %r %r %r" % (seen, want, timed_out), flush=True)
"""


def test_two_ranks_over_nccl_with_a_late_rank(tmp_path):
    import ctypes as C

    n = C.c_int32()
    J.binding.check(J.load().jgpt_device_count(C.byref(n)))
    if n.value < 2:
        pytest.skip("needs two GPUs (run with a two-GPU allocation)")
    uid = TokenGather.unique_id().hex()
    script = os.path.join(tmp_path, "worker.py")
    open(script, "w").write(_WORKER.format(root=ROOT))
    env = dict(os.environ, NCCL_NVLS_ENABLE="0")
    procs = [subprocess.Popen([sys.executable, script, str(r), uid], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True, env=env)
             for r in range(2)]
    outs = [p.communicate(timeout=300) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-3000:]
        assert o.strip().endswith("OK"), (o, e[-3000:])
