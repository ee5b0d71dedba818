"""Context (one GPU + one stream) and device buffers.

Mirrors, on the reference side, ``TensorOpsGPU`` initialisation / ``synchronizeStream`` and
``GpuFloatBuffer`` / ``GpuIntBuffer`` (src/main/java/com/veles/llm/jgpt/GpuFloatBuffer.java).
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import binding as B


class Context:
    """One GPU and its stream.  The reference has one process-global stream on device 0."""

    def __init__(self, device: int = 0):
        self._lib = B.load()
        h = C.c_uint64()
        B.check(self._lib.jgpt_ctx_create(device, C.byref(h)))
        self.handle = h.value
        self.device = device

    def synchronize(self):
        """``TensorOpsGPU.synchronizeStream``; raises if a kernel recorded a failed self-check."""
        B.check(self._lib.jgpt_sync(self.handle))

    def mem_info(self):
        """(free bytes, total bytes) of the context's device."""
        f, t = C.c_uint64(), C.c_uint64()
        B.check(self._lib.jgpt_mem_info(self.handle, C.byref(f), C.byref(t)))
        return f.value, t.value

    @property
    def stream(self) -> int:
        p = C.c_void_p()
        B.check(self._lib.jgpt_ctx_stream(self.handle, C.byref(p)))
        return p.value or 0

    def alloc(self, shape, dtype=np.float32) -> "DeviceBuffer":
        return DeviceBuffer(self, shape, dtype)

    def from_host(self, arr) -> "DeviceBuffer":
        arr = np.ascontiguousarray(arr)
        buf = DeviceBuffer(self, arr.shape, arr.dtype)
        buf.copy_from(arr)
        return buf

    def pinned_array(self, shape, dtype=np.float32) -> np.ndarray:
        """A numpy view of page-locked host memory (``jgpt_host_alloc_pinned``): the host-buffer entry points read and
        write such buffers in place, without staging copies.  Lives until the process ends."""
        n = int(np.prod(shape, dtype=np.int64)) * np.dtype(dtype).itemsize
        p = C.c_void_p()
        B.check(self._lib.jgpt_host_alloc_pinned(max(n, 1), C.byref(p)))
        buf = (C.c_char * n).from_address(p.value)
        return np.frombuffer(buf, dtype=dtype).reshape(shape)

    def matmul(self, a: "DeviceBuffer", b: "DeviceBuffer", c: "DeviceBuffer", M: int, K: int, N: int):
        """``TensorOpsGPU.matmulGpuDevice(a, b, c, M, K, N)``: C[M,N] = A[M,K] . B[K,N] on device buffers."""
        B.check(self._lib.jgpt_matmul_device(self.handle, a.ptr, b.ptr, c.ptr, M, K, N))

    def capture(self, fn) -> "Graph":
        """Records everything ``fn()`` enqueues on this context into a CUDA graph."""
        B.check(self._lib.jgpt_graph_begin_capture(self.handle))
        try:
            fn()
        finally:
            h = C.c_uint64()
            rc = self._lib.jgpt_graph_end_capture(self.handle, C.byref(h))
        B.check(rc)
        return Graph(self, h.value)

    def close(self):
        if self.handle:
            self._lib.jgpt_ctx_destroy(self.handle)
            self.handle = 0

    def __enter__(self):
        return self

    def __exit__(self, *a):
        self.close()


class Graph:
    def __init__(self, ctx: Context, handle: int):
        self.ctx, self.handle = ctx, handle

    def launch(self):
        B.check(self.ctx._lib.jgpt_graph_launch(self.ctx.handle, self.handle))

    def close(self):
        if self.handle:
            self.ctx._lib.jgpt_graph_destroy(self.handle)
            self.handle = 0


def bind_host_near_gpu(device: int) -> dict:
    """Pins the calling process to the CPUs of the NUMA node the GPU hangs off, so that page-locked buffers allocated
    afterwards (first touch) and the thread that fills them sit next to it.  With one rank per GPU on a two-socket box
    this keeps every rank's PCIe traffic off the inter-socket link.  Returns what it found; does nothing when the
    platform does not say (no sysfs entry, node -1, or an affinity mask that excludes the node)."""
    import os

    lib = B.load()
    buf = C.create_string_buffer(32)
    info = {"device": device, "bound": False}
    if lib.jgpt_device_pci_bus_id(device, buf, 32) != 0:
        return info
    info["pci"] = buf.value.decode()
    try:
        node = int(open(f"/sys/bus/pci/devices/{info['pci']}/numa_node").read().strip())
        info["numa_node"] = node
        if node < 0:
            return info
        cpus = set()
        for part in open(f"/sys/devices/system/node/node{node}/cpulist").read().strip().split(","):
            lo, _, hi = part.partition("-")
            cpus.update(range(int(lo), int(hi or lo) + 1))
        allowed = cpus & os.sched_getaffinity(0)
        if allowed:
            os.sched_setaffinity(0, allowed)
            info["bound"], info["cpus"] = True, len(allowed)
    except (OSError, ValueError):
        pass
    return info


class Event:
    def __init__(self, ctx: Context):
        self.ctx = ctx
        h = C.c_uint64()
        B.check(ctx._lib.jgpt_event_create(C.byref(h)))
        self.handle = h.value

    def record(self):
        B.check(self.ctx._lib.jgpt_event_record(self.ctx.handle, self.handle))

    def elapsed_ms(self, later: "Event") -> float:
        ms = C.c_float()
        B.check(self.ctx._lib.jgpt_event_elapsed_ms(self.handle, later.handle, C.byref(ms)))
        return ms.value

    def __del__(self):
        try:
            if self.handle:
                self.ctx._lib.jgpt_event_destroy(self.handle)
        except Exception:
            pass


class DeviceBuffer:
    """Typed device allocation (``GpuFloatBuffer.allocate`` / ``copyFrom`` / ``copyTo`` / ``clear``)."""

    def __init__(self, ctx: Context, shape, dtype=np.float32):
        self.ctx = ctx
        self.shape = tuple(int(s) for s in (shape if hasattr(shape, "__len__") else (shape,)))
        self.dtype = np.dtype(dtype)
        self.nbytes = int(np.prod(self.shape, dtype=np.int64)) * self.dtype.itemsize
        p = C.c_void_p()
        B.check(ctx._lib.jgpt_dev_alloc(ctx.handle, max(self.nbytes, 1), C.byref(p)))
        self.ptr = p.value

    def copy_from(self, arr):
        arr = np.ascontiguousarray(arr, dtype=self.dtype)
        if arr.nbytes != self.nbytes:
            raise ValueError(f"size mismatch: {arr.nbytes} != {self.nbytes}")
        B.check(self.ctx._lib.jgpt_h2d(self.ctx.handle, self.ptr, arr.ctypes.data, arr.nbytes))
        return self

    def to_host(self) -> np.ndarray:
        out = np.empty(self.shape, self.dtype)
        B.check(self.ctx._lib.jgpt_d2h(self.ctx.handle, out.ctypes.data, self.ptr, self.nbytes))
        return out

    def fill_bytes(self, value: int):
        B.check(self.ctx._lib.jgpt_dev_memset(self.ctx.handle, self.ptr, value, self.nbytes))
        return self

    def close(self):
        if self.ptr:
            self.ctx._lib.jgpt_dev_free(self.ctx.handle, self.ptr)
            self.ptr = None

    def __del__(self):
        try:
            if self.ptr and self.ctx.handle:
                self.close()
        except Exception:
            pass
