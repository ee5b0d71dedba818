"""Multi-rank host logic on CPU: round-robin sharding of requests and the gather of sampled token ids
(gloo, world size 2), plus the continuous-batching policy specification itself."""
import os
import subprocess
import sys

import numpy as np

import oracle as O
from jgpt_b200.scheduler import gather_step_tokens, shard_requests

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_round_robin_sharding_partitions_the_requests():
    for n, w in [(256, 8), (10, 4), (3, 8), (0, 2)]:
        parts = [shard_requests(n, w, r) for r in range(w)]
        assert sorted(x for p in parts for x in p) == list(range(n))
        assert all(all(x % w == r for x in p) for r, p in enumerate(parts))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1
    assert gather_step_tokens([(3, 7), (5, 0)], 1, 0, 4) == [(3, 7), (5, 0)]


_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch.distributed as dist
from jgpt_b200.scheduler import gather_step_tokens, shard_requests
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank, world, n_req = dist.get_rank(), 2, 11
mine = shard_requests(n_req, world, rank)
ok = True
for step in range(5):
    live = [r for r in mine if (r + step) % 3 != 0]          # a different subset produces a token each step
    local = [(r, (r * 31 + step * 7) % 100) for r in live]
    got = gather_step_tokens(local, world, rank, max_pairs=8, dist=dist)
    want = [(r, (r * 31 + step * 7) % 100) for rk in range(world) for r in shard_requests(n_req, world, rk) if (r + step) % 3 != 0]
    ok = ok and got == want
dist.barrier()
dist.destroy_process_group()
print("OK" if ok else "MISMATCH", flush=True)
"""


def test_token_id_gather_two_ranks_gloo(tmp_path):
    port = 29500 + (os.getpid() % 400)
    script = os.path.join(tmp_path, "worker.py")
    open(script, "w").write(_WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, script, str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
        assert o.strip().endswith("OK"), (o, e[-2000:])


_WORKER_LAGGED = r"""
import os, sys, time
sys.path.insert(0, {root!r})
import numpy as np, torch.distributed as dist
from jgpt_b200.scheduler import StepTokenGather, shard_requests
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank, world, n_req = dist.get_rank(), 2, 11
mine = shard_requests(n_req, world, rank)
my_steps = 9 if rank == 0 else 5            # rank 1 finishes earlier and keeps reporting "done"
g = StepTokenGather(world, rank, max_pairs=8, dist=dist, depth=3)
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
    g.submit(local + ([(-1, 1)] if done else []))
    step += 1
    while g.ready() and not all_done:
        account(g.pop())
for pairs in g.drain():
    account(pairs)
want = []
for t in range(len(seen)):
    want.append([(r, (r * 31 + t * 7) % 100) for rk in range(world) for r in shard_requests(n_req, world, rk)
                 if t < (9 if rk == 0 else 5) and (r + t) % 3 != 0])
ok = seen == want and len(seen) >= 10 and step == len(seen)
dist.barrier()
dist.destroy_process_group()
print("OK" if ok else "MISMATCH %r %r" % (seen, want), flush=True)
"""


def test_lagged_token_id_gather_two_ranks_gloo(tmp_path):
    """The asynchronous form: results arrive in step order, identical on both ranks, while the ranks run up to
    `depth` steps apart; both stop on the same gathered step and have issued the same number of collectives."""
    from jgpt_b200.scheduler import StepTokenGather
    g = StepTokenGather(1, 0, 4)  # single rank: nothing is communicated, results still come `depth` steps later
    g.submit([(3, 7)]), g.submit([(5, 0)])
    assert not g.ready() and g.drain() == [[(3, 7)], [(5, 0)]]
    port = 29900 + (os.getpid() % 90)
    script = os.path.join(tmp_path, "worker_lagged.py")
    open(script, "w").write(_WORKER_LAGGED.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, script, str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
        assert o.strip().endswith("OK"), (o, e[-2000:])


def test_continuous_batching_policy_specification():
    """FIFO admission with up-front reservation, LRU eviction of finished sequences, no overtaking."""
    streams = [[5, 6, 7], [8, 0, 9], [1, 2, 3, 4], [9, 9]]
    a = O.PagedAllocatorRef(n_blocks=4, block_tokens=16, max_seqs=2, max_blocks_per_seq=4)
    s = O.ContinuousBatchRef(a, max_running=2, max_rows=64, streams=streams)
    for plen, mx in [(20, 3), (10, 3), (40, 4), (5, 2)]:
        s.submit(plen, mx)  # blocks needed: 2, 1, 3, 1
    assert s.step() == [(0, 5), (1, 8)] and s.events == [(1, 0, 0), (1, 1, 1)]
    assert s.step() == [(0, 6), (1, 0)]  # request 1 stops on token 0 ...
    assert s.events[-1] == (3, 1, 2) and s.running == [0]
    # ... its slot and block are reclaimed only when request 2 (3 blocks) needs them; 2 + 3 > 4: still blocked
    assert s.step() == [(0, 7)] and s.events[-2:] == [(2, 1, 1), (3, 0, 3)] and s.waiting == [2, 3]
    # step 4: evict finished request 0, admit request 2 (3 blocks, slot 0) and, behind it, request 3 (1 block, slot 1)
    assert s.step() == [(2, 1), (3, 9)] and s.events[-3:] == [(2, 0, 0), (1, 2, 0), (1, 3, 1)] and s.waiting == []
    assert s.step() == [(2, 2), (3, 9)] and s.events[-1] == (3, 3, 2)
    assert s.step() == [(2, 3)] and s.step() == [(2, 4)] and s.events[-1] == (3, 2, 4)
    assert [r["out"] for r in s.reqs] == [[5, 6, 7], [8, 0], [1, 2, 3, 4], [9, 9]] and not s.running and not s.waiting
