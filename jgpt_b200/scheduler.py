"""Continuous-batching scheduler (host mirror of the ``jgpt_sched_*`` entry points) and the multi-GPU
sharding helpers: requests are dealt round-robin to the ranks (``request % world``), every rank runs its own
scheduler on its own GPU and pool, and only the sampled token ids are gathered (``TokenGather``: NCCL inside the
library, no PyTorch)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import binding as B

EV_ADMIT, EV_EVICT, EV_FINISH = 1, 2, 3


class ContinuousBatcher:
    def __init__(self, model, pool, max_running, max_rows_per_call=None):
        self.model, self.pool, self._lib = model, pool, model._lib
        h = C.c_uint64()
        B.check(self._lib.jgpt_sched_create(model.handle, pool.handle, max_running, max_rows_per_call or model.maxRows,
                                            model.maxSeqLen, C.byref(h)))
        self.handle = h.value
        self.n_requests = 0

    def submit(self, prompt, max_new) -> int:
        p = np.ascontiguousarray(prompt, np.int32)
        rid = C.c_int32()
        B.check(self._lib.jgpt_sched_submit(self.handle, p.ctypes.data, p.size, max_new, C.byref(rid)))
        self.n_requests += 1
        return rid.value

    def step(self):
        """Returns (pairs [(request, token), ...], n_running, n_waiting)."""
        cap = self.pool.max_seqs + 8
        buf = np.empty(2 * cap, np.int32)
        n, nr, nw = C.c_int32(), C.c_int32(), C.c_int32()
        B.check(self._lib.jgpt_sched_step(self.handle, buf.ctypes.data, cap, C.byref(n), C.byref(nr), C.byref(nw)))
        return buf[: 2 * n.value].reshape(-1, 2).copy(), nr.value, nw.value

    def result(self, rid):
        n, st, sq = C.c_int32(), C.c_int32(), C.c_int32()
        B.check(self._lib.jgpt_sched_result(self.handle, rid, None, 0, C.byref(n), C.byref(st), C.byref(sq)))
        out = np.empty(max(n.value, 1), np.int32)
        B.check(self._lib.jgpt_sched_result(self.handle, rid, out.ctypes.data, out.size, C.byref(n), C.byref(st), C.byref(sq)))
        return out[: n.value].copy(), st.value, sq.value

    def events(self):
        n = C.c_int32()
        B.check(self._lib.jgpt_sched_events(self.handle, None, 0, C.byref(n)))
        out = np.empty(max(n.value, 1), np.int32)
        B.check(self._lib.jgpt_sched_events(self.handle, out.ctypes.data, out.size, C.byref(n)))
        return [tuple(int(x) for x in t) for t in out[: n.value].reshape(-1, 3)]

    def run(self, max_steps=1_000_000):
        """Steps until nothing is running or waiting; returns the number of steps taken."""
        steps = 0
        while steps < max_steps:
            _, nr, nw = self.step()
            steps += 1
            if nr == 0 and nw == 0:
                break
        return steps

    def close(self):
        if self.handle:
            self._lib.jgpt_sched_destroy(self.handle)
            self.handle = 0


# ---------------------------------------------------------------------------------------------------
# Sequence sharding across GPUs
# ---------------------------------------------------------------------------------------------------
def shard_requests(n_requests: int, world: int, rank: int):
    """Global request ids owned by ``rank``: round-robin, request % world == rank."""
    return list(range(rank, n_requests, world))


def rendezvous_unique_id(rank: int, world: int, key: str, directory: str | None = None, timeout_s: float = 120.0) -> bytes | None:
    """Hands rank 0's NCCL unique id to the other ranks of one box through a file: a launcher that has no store of
    its own needs nothing else.  ``key`` must be the same on all ranks of a job and differ between jobs (e.g. the
    launcher's port or run id).  Returns None for a single rank."""
    import os
    import time

    if world <= 1:
        return None
    directory = directory or os.environ.get("JGPT_B200_RDZV_DIR", "/tmp")
    path = os.path.join(directory, f"jgpt_b200_rdzv_{key}")
    if rank == 0:
        uid = TokenGather.unique_id()
        tmp = f"{path}.{os.getpid()}.tmp"
        with open(tmp, "wb") as f:
            f.write(uid)
        os.replace(tmp, path)  # appears atomically
        return uid
    deadline = time.time() + timeout_s
    while time.time() < deadline:
        try:
            with open(path, "rb") as f:
                uid = f.read()
            if len(uid) == 128:
                return uid
        except FileNotFoundError:
            pass
        time.sleep(0.01)
    raise TimeoutError(f"rank {rank}: no unique id at {path} after {timeout_s} s")


def rendezvous_cleanup(key: str, directory: str | None = None):
    """Removes the rendezvous file of ``key`` (rank 0, once every rank has joined the communicator)."""
    import os

    try:
        os.remove(os.path.join(directory or os.environ.get("JGPT_B200_RDZV_DIR", "/tmp"), f"jgpt_b200_rdzv_{key}"))
    except OSError:
        pass


def pack_pairs(pairs, done: bool = False):
    """(request id, token) pairs of one step as the flat int32 words a rank contributes to the gather.  A rank
    that has nothing left to do appends the sentinel pair (-1, 1): when every rank has sent it the job is over."""
    a = np.asarray(pairs, np.int32).reshape(-1, 2)
    if done:
        a = np.concatenate([a, np.array([[-1, 1]], np.int32)])
    return np.ascontiguousarray(a.reshape(-1))


def unpack_pairs(words, counts):
    """Inverse of ``pack_pairs`` over the gathered rows: the pairs of all ranks ordered by (rank, local order)."""
    out = []
    for r, c in enumerate(counts):
        w = words[r]
        out.extend((int(w[2 * i]), int(w[2 * i + 1])) for i in range(int(c) // 2))
    return out


class TokenGather:
    """All-gather of every rank's sampled token ids over NCCL, inside the library (``jgpt_comm_*``).

    One per rank.  ``submit`` hands in this step's pairs and returns at once; the collective runs on a stream of
    its own and its result is read up to ``depth`` steps later (``ready`` says when one has to be read), so the
    ranks never meet after every step.  Results come back in step order, identical on every rank.  Every rank
    must submit once per step and stop by the same rule on the gathered results, then ``drain``.

    ``unique_id`` is the 128-byte rendezvous id made by rank 0 (``TokenGather.unique_id()``) and handed to the
    other ranks by the launcher; with ``world == 1`` nothing is communicated and no NCCL is needed."""

    def __init__(self, ctx, world: int, rank: int, max_pairs: int, unique_id: bytes | None = None, depth: int = 4,
                 timeout_ms: int = 30000):
        self._lib, self.ctx = ctx._lib, ctx
        self.world, self.rank, self.max_words, self.depth, self.timeout_ms = world, rank, 2 * (max_pairs + 1), depth, timeout_ms
        h = C.c_uint64()
        B.check(self._lib.jgpt_comm_create(ctx.handle, unique_id, world, rank, self.max_words, depth, timeout_ms, C.byref(h)))
        self.handle = h.value

    @staticmethod
    def unique_id() -> bytes:
        buf = C.create_string_buffer(128)
        B.check(B.load().jgpt_comm_unique_id(buf, 128))
        return buf.raw

    def submit(self, pairs, done: bool = False):
        self.submit_words(pack_pairs(pairs, done))

    def submit_words(self, words):
        w = np.ascontiguousarray(words, np.int32).reshape(-1)
        B.check(self._lib.jgpt_comm_submit(self.handle, w.ctypes.data, w.size))

    def submit_device(self, words_dev, n_words: int):
        """Gathers n_words int32 words that work already enqueued on the context's stream leaves at ``words_dev``."""
        B.check(self._lib.jgpt_comm_submit_device(self.handle, words_dev, n_words))

    def in_flight(self) -> int:
        n, m = C.c_int32(), C.c_int32()
        B.check(self._lib.jgpt_comm_in_flight(self.handle, C.byref(n), C.byref(m)))
        return n.value

    def ready(self) -> bool:
        n, m = C.c_int32(), C.c_int32()
        B.check(self._lib.jgpt_comm_in_flight(self.handle, C.byref(n), C.byref(m)))
        return bool(m.value)

    def pop_words(self, timeout_ms: int | None = None):
        """(words [world, max_words], counts [world]) of the oldest step; TimeoutError leaves it in flight."""
        words = np.empty((self.world, self.max_words), np.int32)
        counts = np.empty(self.world, np.int32)
        B.check(self._lib.jgpt_comm_pop(self.handle, words.ctypes.data, counts.ctypes.data,
                                        self.timeout_ms if timeout_ms is None else timeout_ms))
        return words, counts

    def pop(self, timeout_ms: int | None = None):
        return unpack_pairs(*self.pop_words(timeout_ms))

    def drain(self):
        out = []
        while self.in_flight():
            out.append(self.pop())
        return out

    def close(self):
        if self.handle:
            self._lib.jgpt_comm_destroy(self.handle)
            self.handle = 0
