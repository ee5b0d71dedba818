"""Continuous-batching scheduler (host mirror of the ``jgpt_sched_*`` entry points) and the multi-GPU
sharding helpers: requests are dealt round-robin to the ranks (``request % world``), every rank runs its own
scheduler on its own GPU and pool, and only the sampled token ids are gathered."""
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


def gather_step_tokens(local_pairs, world: int, rank: int, max_pairs: int, dist=None, device=None):
    """All-gathers one step's (global request id, token) pairs.  Every rank contributes a fixed-size int32
    buffer (count, then pairs, padded with -1) so that the collective has the same shape on every rank.
    Returns the pairs of all ranks ordered by (rank, local order).  ``dist`` is ``torch.distributed`` (NCCL on
    GPUs, gloo in CPU tests); with world == 1 nothing is communicated."""
    local_pairs = np.asarray(local_pairs, np.int32).reshape(-1, 2)
    if local_pairs.shape[0] > max_pairs:
        raise ValueError(f"{local_pairs.shape[0]} pairs exceed the gather buffer of {max_pairs}")
    if world == 1 or dist is None:
        return [tuple(int(x) for x in p) for p in local_pairs]
    import torch

    buf = np.full(1 + 2 * max_pairs, -1, np.int32)
    buf[0] = local_pairs.shape[0]
    buf[1:1 + local_pairs.size] = local_pairs.reshape(-1)
    send = torch.from_numpy(buf)
    if device is not None:
        send = send.to(device)
    recv = [torch.empty_like(send) for _ in range(world)]
    dist.all_gather(recv, send)
    out = []
    for r in range(world):
        a = recv[r].cpu().numpy()
        out.extend((int(a[1 + 2 * i]), int(a[2 + 2 * i])) for i in range(int(a[0])))
    return out
