"""Multi-rank host logic on CPU: round-robin sharding of requests and the wire format + ordering of the gather
of sampled token ids (two gloo ranks standing in for the NCCL transport, which needs GPUs), plus the
continuous-batching policy specification itself.  The NCCL transport of the library (`jgpt_comm_*`) is covered by
tests/test_comm_gpu.py."""
import os
import subprocess
import sys

import numpy as np

import oracle as O
from jgpt_b200.scheduler import pack_pairs, rendezvous_unique_id, shard_requests, unpack_pairs

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_round_robin_sharding_partitions_the_requests():
    for n, w in [(256, 8), (10, 4), (3, 8), (0, 2)]:
        parts = [shard_requests(n, w, r) for r in range(w)]
        assert sorted(x for p in parts for x in p) == list(range(n))
        assert all(all(x % w == r for x in p) for r, p in enumerate(parts))
        assert max(len(p) for p in parts) - min(len(p) for p in parts) <= 1


def test_pair_wire_format_round_trips():
    w0, w1 = pack_pairs([(3, 7), (5, 0)]), pack_pairs([], done=True)
    assert w0.dtype == np.int32 and w0.tolist() == [3, 7, 5, 0] and w1.tolist() == [-1, 1]
    words = np.full((2, 8), -1, np.int32)
    words[0, :4], words[1, :2] = w0, w1
    assert unpack_pairs(words, [4, 2]) == [(3, 7), (5, 0), (-1, 1)]
    assert unpack_pairs(words, [0, 0]) == []
    assert rendezvous_unique_id(0, 1, "unused") is None  # a single rank has nobody to meet


_WORKER = r"""
import os, sys
sys.path.insert(0, {root!r})
import numpy as np, torch, torch.distributed as dist
from jgpt_b200.scheduler import pack_pairs, shard_requests, unpack_pairs
dist.init_process_group("gloo", init_method="tcp://127.0.0.1:{port}", rank=int(sys.argv[1]), world_size=2)
rank, world, n_req, max_words = dist.get_rank(), 2, 11, 18

def gather(pairs, done=False):
    # the library's collective shape: every rank sends 1 count + max_words words, padded with -1
    w = pack_pairs(pairs, done)
    buf = np.full(1 + max_words, -1, np.int32)
    buf[0], buf[1:1 + w.size] = w.size, w
    recv = [torch.empty(1 + max_words, dtype=torch.int32) for _ in range(world)]
    dist.all_gather(recv, torch.from_numpy(buf))
    rows = np.stack([t.numpy() for t in recv])
    return unpack_pairs(rows[:, 1:], rows[:, 0])

mine = shard_requests(n_req, world, rank)
my_steps = 9 if rank == 0 else 5            # rank 1 finishes earlier and keeps reporting "done"
ok, step, all_done, seen = True, 0, False, []
while not all_done:
    done = step >= my_steps
    local = [] if done else [(r, (r * 31 + step * 7) % 100) for r in mine if (r + step) % 3 != 0]
    got = gather(local, done)
    seen.append([p for p in got if p[0] >= 0])
    all_done = sum(1 for p in got if p[0] < 0) == world
    step += 1
want = [[(r, (r * 31 + t * 7) % 100) for rk in range(world) for r in shard_requests(n_req, world, rk)
         if t < (9 if rk == 0 else 5) and (r + t) % 3 != 0] for t in range(len(seen))]
ok = seen == want and len(seen) == 10
dist.barrier()
dist.destroy_process_group()
print("OK" if ok else "MISMATCH %r %r" % (seen, want), flush=True)
"""


def test_token_id_gather_protocol_two_ranks_gloo(tmp_path):
    """Both ranks see the same pairs in (rank, local order), a finished rank keeps reporting the sentinel, and both
    stop on the same step."""
    port = 29500 + (os.getpid() % 400)
    script = os.path.join(tmp_path, "worker.py")
    open(script, "w").write(_WORKER.format(root=ROOT, port=port))
    procs = [subprocess.Popen([sys.executable, script, str(r)], stdout=subprocess.PIPE, stderr=subprocess.PIPE, text=True) for r in range(2)]
    outs = [p.communicate(timeout=180) for p in procs]
    for p, (o, e) in zip(procs, outs):
        assert p.returncode == 0, e[-2000:]
        assert o.strip().endswith("OK"), (o, e[-2000:])


def test_unique_id_file_rendezvous(tmp_path):
    """Rank 0's id reaches a rank that started earlier and polls for it (the id itself comes from NCCL; here a
    stand-in file written the way rank 0 writes it)."""
    import threading
    import time

    got = {}
    t = threading.Thread(target=lambda: got.setdefault("id", rendezvous_unique_id(1, 2, "k1", str(tmp_path), timeout_s=20)))
    t.start()
    time.sleep(0.2)
    tmp = os.path.join(tmp_path, "x.tmp")
    open(tmp, "wb").write(bytes(range(128)))
    os.replace(tmp, os.path.join(tmp_path, "jgpt_b200_rdzv_k1"))
    t.join(timeout=30)
    assert got.get("id") == bytes(range(128))
    try:
        rendezvous_unique_id(1, 2, "missing", str(tmp_path), timeout_s=0.2)
        assert False, "expected a timeout"
    except TimeoutError:
        pass


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
