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


class StepTokenGather:
    """The same all-gather, issued asynchronously and read ``depth`` steps later: the collective of step t overlaps
    the decode steps t+1 .. t+depth of every rank, and ranks may drift up to ``depth`` steps apart instead of meeting
    after every step (one rank's prefill no longer stalls the others' decode steps).  Results come back in step
    order, each the pairs of all ranks ordered by (rank, local order), exactly what ``gather_step_tokens`` returns.

    Every rank must ``submit`` once per step and stop by the same rule on the gathered results (e.g. "all ranks
    reported done"), then ``drain``; since results are read in the same order everywhere, all ranks then have issued
    the same number of collectives."""

    def __init__(self, world: int, rank: int, max_pairs: int, dist=None, device=None, depth: int = 4):
        self.world, self.rank, self.max_pairs, self.dist, self.device = world, rank, max_pairs, dist, device
        self.depth = max(0, int(depth))
        self._inflight = []  # (work or None, slot or None, pairs or None)
        self._slots, self._free = [], []
        if world > 1 and dist is not None and device is not None:
            # a ring of page-locked staging buffers and device tensors: a step's submit is one small copy and one launch
            import torch

            n = 1 + 2 * max_pairs
            for _ in range(self.depth + 2):
                self._slots.append({
                    "send_host": torch.empty(n, dtype=torch.int32, pin_memory=True),
                    "send_dev": torch.empty(n, dtype=torch.int32, device=device),
                    "recv_dev": torch.empty(world * n, dtype=torch.int32, device=device),
                    "recv_host": torch.empty(world * n, dtype=torch.int32, pin_memory=True),
                })
            self._free = list(range(len(self._slots)))

    def submit(self, local_pairs):
        local_pairs = np.asarray(local_pairs, np.int32).reshape(-1, 2)
        if local_pairs.shape[0] > self.max_pairs:
            raise ValueError(f"{local_pairs.shape[0]} pairs exceed the gather buffer of {self.max_pairs}")
        if self.world == 1 or self.dist is None:
            self._inflight.append((None, None, [tuple(int(x) for x in p) for p in local_pairs]))
            return
        import torch

        if self._slots:
            slot_id = self._free.pop(0)
            slot = self._slots[slot_id]
            buf = slot["send_host"].numpy()
            buf[:] = -1
            buf[0] = local_pairs.shape[0]
            buf[1:1 + local_pairs.size] = local_pairs.reshape(-1)
            slot["send_dev"].copy_(slot["send_host"], non_blocking=True)
            work = self.dist.all_gather_into_tensor(slot["recv_dev"], slot["send_dev"], async_op=True)
            self._inflight.append((work, slot_id, None))
            return
        buf = np.full(1 + 2 * self.max_pairs, -1, np.int32)
        buf[0] = local_pairs.shape[0]
        buf[1:1 + local_pairs.size] = local_pairs.reshape(-1)
        send = torch.from_numpy(buf)
        recv = [torch.empty_like(send) for _ in range(self.world)]
        work = self.dist.all_gather(recv, send, async_op=True)
        self._inflight.append((work, None, recv))

    def ready(self) -> bool:
        """True when a result must be read now to keep at most ``depth`` collectives in flight."""
        return len(self._inflight) > self.depth

    def pop(self):
        """Waits for the oldest step's collective and returns its pairs."""
        work, slot_id, payload = self._inflight.pop(0)
        if work is None:
            return payload
        work.wait()
        n = 1 + 2 * self.max_pairs
        if slot_id is not None:
            import torch

            slot = self._slots[slot_id]
            slot["recv_host"].copy_(slot["recv_dev"], non_blocking=True)
            torch.cuda.current_stream().synchronize()
            flat = slot["recv_host"].numpy()
            rows = [flat[r * n:(r + 1) * n] for r in range(self.world)]
            self._free.append(slot_id)
        else:
            rows = [t.cpu().numpy() for t in payload]
        out = []
        for a in rows:
            out.extend((int(a[1 + 2 * i]), int(a[2 + 2 * i])) for i in range(int(a[0])))
        return out

    def drain(self):
        """Results of every step still in flight, oldest first."""
        out = []
        while self._inflight:
            out.append(self.pop())
        return out
