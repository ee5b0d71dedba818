"""Paged KV store and the ``KvCacheGpu`` facade the reference's generation loop expects.

``KvPool`` owns the physical blocks of a model (all sequences); ``KvCacheGpu`` is one sequence
of it with the public methods of the reference class
(src/main/java/com/veles/llm/jgpt/model/KvCacheGpu.java:12-118): ``getK/getV`` (a gathered,
contiguous fp32 view ``[heads, maxSeqLen, dHead]``), ``length``, ``setLength``, ``maxSeqLen``,
``remainingCapacity``, ``isFull``, ``clear``, ``numLayers``, ``close``.
"""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import binding as B
from .runtime import Context, DeviceBuffer

BLOCK_TOKENS = 16


def _ptr(x):
    if x is None:
        return None
    if isinstance(x, DeviceBuffer):
        return x.ptr
    return int(x)


class KvPool:
    def __init__(self, ctx: Context, layers, heads, dhead, n_blocks, max_seqs, max_blocks_per_seq,
                 max_positions=None, rope_base=10000.0):
        self.ctx, self._lib = ctx, ctx._lib
        self.layers, self.heads, self.dhead = layers, heads, dhead
        self.n_blocks, self.max_seqs, self.max_blocks_per_seq = n_blocks, max_seqs, max_blocks_per_seq
        self.max_positions = max_positions if max_positions is not None else max_blocks_per_seq * BLOCK_TOKENS
        h = C.c_uint64()
        B.check(self._lib.jgpt_kvpool_create(ctx.handle, layers, heads, dhead, BLOCK_TOKENS, n_blocks, max_seqs,
                                             max_blocks_per_seq, self.max_positions, rope_base, C.byref(h)))
        self.handle = h.value

    # ---- allocator -------------------------------------------------------------------------
    def free_blocks(self) -> int:
        n = C.c_int32()
        B.check(self._lib.jgpt_kvpool_free_blocks(self.handle, C.byref(n)))
        return n.value

    def storage(self):
        p, n = C.c_void_p(), C.c_uint64()
        B.check(self._lib.jgpt_kvpool_storage(self.handle, C.byref(p), C.byref(n)))
        return p.value, n.value

    def set_tuning(self, chunk_blocks=0, stages=0, head_group=0, persistent=-1, launch_overlap=1):
        """Launch shape of the decode-attention kernel on this pool (results do not depend on it)."""
        B.check(self._lib.jgpt_kvpool_set_tuning(self.handle, chunk_blocks, stages, head_group, persistent, launch_overlap))

    def table_device(self):
        """(device address, row stride) of the block-table mirror, int32 [max_seqs][row stride]."""
        p, n = C.c_void_p(), C.c_int32()
        B.check(self._lib.jgpt_kvpool_table_device(self.handle, C.byref(p), C.byref(n)))
        return p.value, n.value

    def seq_alloc(self) -> int:
        s = C.c_int32()
        B.check(self._lib.jgpt_seq_alloc(self.handle, C.byref(s)))
        return s.value

    def seq_free(self, seq):
        B.check(self._lib.jgpt_seq_free(self.handle, seq))

    def reserve(self, seq, n_tokens):
        B.check(self._lib.jgpt_seq_reserve(self.handle, seq, n_tokens))

    def length(self, seq) -> int:
        n = C.c_int32()
        B.check(self._lib.jgpt_seq_length(self.handle, seq, C.byref(n)))
        return n.value

    def set_length(self, seq, n):
        B.check(self._lib.jgpt_seq_set_length(self.handle, seq, n))

    def clear(self, seq, zero_fill=True):
        B.check(self._lib.jgpt_seq_clear(self.handle, seq, 1 if zero_fill else 0))

    def drop_front(self, seq, n_blocks=1, zero_fill=False):
        """Rolling window: forget the oldest n_blocks KV blocks of the sequence (no K/V byte moves)."""
        B.check(self._lib.jgpt_seq_drop_front(self.handle, seq, n_blocks, 1 if zero_fill else 0))

    def set_block_table(self, seq, blocks):
        b = np.ascontiguousarray(blocks, np.int32)
        B.check(self._lib.jgpt_seq_set_block_table(self.handle, seq, b.ctypes.data, b.size))

    def block_table(self, seq, device=False) -> np.ndarray:
        out = np.empty(self.max_blocks_per_seq, np.int32)
        n = C.c_int32()
        fn = self._lib.jgpt_block_table_copy_out_device if device else self._lib.jgpt_block_table_copy_out
        B.check(fn(self.handle, seq, out.ctypes.data, out.size, C.byref(n)))
        return out[: n.value].copy()

    def mark_evictable(self, seq, flag=True):
        B.check(self._lib.jgpt_seq_mark_evictable(self.handle, seq, 1 if flag else 0))

    def evict_lru(self, need_free, zero_fill=False):
        out = np.empty(self.max_seqs, np.int32)
        n = C.c_int32()
        B.check(self._lib.jgpt_kv_evict_lru(self.handle, need_free, 1 if zero_fill else 0, out.ctypes.data, out.size,
                                            C.byref(n)))
        return out[: n.value].tolist()

    # ---- kernels ---------------------------------------------------------------------------
    def append(self, layer, k_dev, v_dev, seq_ids_dev, slot_pos_dev, rope_pos_dev, n):
        B.check(self._lib.jgpt_kv_append(self.handle, layer, _ptr(k_dev), _ptr(v_dev), _ptr(seq_ids_dev),
                                         _ptr(slot_pos_dev), _ptr(rope_pos_dev), n))

    def gather(self, layer, seq, length, max_seq_len, k_out_dev, v_out_dev):
        B.check(self._lib.jgpt_kv_gather(self.handle, layer, seq, length, max_seq_len, _ptr(k_out_dev), _ptr(v_out_dev)))

    def gather_batch(self, layer, seqs, lens, max_seq_len, k_out_dev, v_out_dev):
        """``gather`` for several sequences in one launch: outputs [n, H, max_seq_len, Dh]."""
        sq, ln = np.ascontiguousarray(seqs, np.int32), np.ascontiguousarray(lens, np.int32)
        B.check(self._lib.jgpt_kv_gather_batch(self.handle, layer, sq.ctypes.data, ln.ctypes.data, sq.size, max_seq_len,
                                               _ptr(k_out_dev), _ptr(v_out_dev)))

    def attn_decode(self, layer0, n_layers, q_dev, seq_ids_dev, rope_pos_dev, lens_dev, n, max_len, out_dev):
        B.check(self._lib.jgpt_attn_decode(self.handle, layer0, n_layers, _ptr(q_dev), _ptr(seq_ids_dev),
                                           _ptr(rope_pos_dev), _ptr(lens_dev), n, max_len, _ptr(out_dev)))

    def attn_prefill(self, layer, q_dev, k_dev, v_dev, seq_ids, seq_starts, rope_offsets, out_dev):
        """Causal prefill attention over packed prompts that also fills the cache (host index arrays)."""
        seq_ids = np.ascontiguousarray(seq_ids, np.int32)
        seq_starts = np.ascontiguousarray(seq_starts, np.int32)
        rope_offsets = np.ascontiguousarray(rope_offsets, np.int32)
        if seq_starts.size != seq_ids.size + 1 or rope_offsets.size != seq_ids.size:
            raise ValueError("seq_starts needs n_seqs + 1 entries, rope_offsets n_seqs")
        B.check(self._lib.jgpt_attn_prefill(self.handle, layer, _ptr(q_dev), _ptr(k_dev), _ptr(v_dev), seq_ids.ctypes.data,
                                            seq_starts.ctypes.data, rope_offsets.ctypes.data, seq_ids.size, _ptr(out_dev)))

    def attn_decode_static_scratch(self, layer, q_dev, seq_ids_dev, rope_pos_dev, lens_dev, n, max_len, out_dev):
        """Single-layer decode attention that never allocates (scratch in a fixed array of the library)."""
        B.check(self._lib.jgpt_attn_decode_static_scratch(self.handle, layer, _ptr(q_dev), _ptr(seq_ids_dev),
                                                          _ptr(rope_pos_dev), _ptr(lens_dev), n, max_len, _ptr(out_dev)))

    def attn_decode_append(self, layer0, n_layers, q_dev, k_dev, v_dev, seq_ids_dev, rope_pos_dev, lens_dev, n, max_len,
                           out_dev):
        B.check(self._lib.jgpt_attn_decode_append(self.handle, layer0, n_layers, _ptr(q_dev), _ptr(k_dev), _ptr(v_dev),
                                                  _ptr(seq_ids_dev), _ptr(rope_pos_dev), _ptr(lens_dev), n, max_len,
                                                  _ptr(out_dev)))

    def attn_decode_append_host(self, layer0, n_layers, q, k, v, seq_ids, rope_pos, lens, out=None):
        """Host-buffer form: numpy in, numpy out (H2D, kernel, D2H, synchronise)."""
        q = np.ascontiguousarray(q, np.float32)
        k = np.ascontiguousarray(k, np.float32)
        v = np.ascontiguousarray(v, np.float32)
        seq_ids = np.ascontiguousarray(seq_ids, np.int32)
        rope_pos = np.ascontiguousarray(rope_pos, np.int32)
        lens = np.ascontiguousarray(lens, np.int32)
        n = seq_ids.size
        if out is None:
            out = np.empty_like(q)
        B.check(self._lib.jgpt_attn_decode_append_host(self.handle, layer0, n_layers, q.ctypes.data, k.ctypes.data,
                                                       v.ctypes.data, seq_ids.ctypes.data, rope_pos.ctypes.data,
                                                       lens.ctypes.data, n, out.ctypes.data))
        return out

    def close(self):
        if self.handle:
            self._lib.jgpt_kvpool_destroy(self.handle)
            self.handle = 0


class KvCacheGpu:
    """One sequence of a :class:`KvPool` behind the reference's ``KvCacheGpu`` methods."""

    def __init__(self, num_layers, num_heads, d_head, max_seq_len, pool: KvPool | None = None, ctx: Context | None = None):
        if num_layers <= 0 or num_heads <= 0 or d_head <= 0 or max_seq_len <= 0:
            raise ValueError("KvCacheGpu dimensions must be positive")  # reference ctor: IAE
        self._own_pool = pool is None
        if pool is None:
            if ctx is None:
                raise RuntimeError("KvCacheGpu requires a CUDA context")  # reference: ISE without a GPU
            nb = -(-max_seq_len // BLOCK_TOKENS)
            pool = KvPool(ctx, num_layers, num_heads, d_head, nb, 1, nb, max_positions=max_seq_len)
        if (pool.layers, pool.heads, pool.dhead) != (num_layers, num_heads, d_head):
            raise ValueError("pool geometry differs from the requested cache geometry")
        self.pool = pool
        self._layers, self._max_seq = num_layers, max_seq_len
        self.seq = pool.seq_alloc()
        self._closed = False

    def _gather(self, layer, which):
        if not 0 <= layer < self._layers:
            raise IndexError(f"layer {layer}")  # reference: IndexOutOfBoundsException
        H, Dh = self.pool.heads, self.pool.dhead
        k = self.pool.ctx.alloc((H, self._max_seq, Dh))
        v = self.pool.ctx.alloc((H, self._max_seq, Dh))
        self.pool.gather(layer, self.seq, self.length(), self._max_seq, k, v)
        return k if which == "k" else v

    def getK(self, layer) -> DeviceBuffer:
        return self._gather(layer, "k")

    def getV(self, layer) -> DeviceBuffer:
        return self._gather(layer, "v")

    def length(self) -> int:
        return self.pool.length(self.seq)

    def setLength(self, n: int):
        if n < 0 or n > self._max_seq:
            raise ValueError(f"length {n} outside [0, {self._max_seq}]")
        self.pool.reserve(self.seq, n)
        self.pool.set_length(self.seq, n)

    def maxSeqLen(self) -> int:
        return self._max_seq

    def remainingCapacity(self) -> int:
        return self._max_seq - self.length()

    def isFull(self) -> bool:
        return self.length() >= self._max_seq

    def clear(self):
        self.pool.clear(self.seq, zero_fill=True)

    def numLayers(self) -> int:
        return self._layers

    def close(self):
        if self._closed:
            return
        self._closed = True
        if self.pool.handle:
            self.pool.seq_free(self.seq)
            if self._own_pool:
                self.pool.close()

    def __repr__(self):
        return f"KvCacheGpu(layers={self._layers}, length={self.length()}, maxSeqLen={self._max_seq}, seq={self.seq})"
