"""ctypes front end of ``libjgpt_oracle.so`` (the C restatement in ``jgpt_oracle.c``) plus the
pure-Python reference of the paged block allocator.

Test infrastructure only: the shipped library never loads this module.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess
from collections import OrderedDict

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
_LIB_PATH = os.path.join(_HERE, "libjgpt_oracle.so")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_i32p = np.ctypeslib.ndpointer(dtype=np.int32, flags="C_CONTIGUOUS")


def build(force: bool = False) -> str:
    """Compile the oracle with the committed Makefile (gcc only; no GPU, no reference sources)."""
    if force or not os.path.exists(_LIB_PATH) or os.path.getmtime(_LIB_PATH) < os.path.getmtime(
        os.path.join(_HERE, "jgpt_oracle.c")
    ):
        subprocess.run(["make", "-B", "-C", _HERE], check=True, capture_output=True)
    return _LIB_PATH


_lib = None
_FAST_PATH = os.path.join(_HERE, "libjgpt_oracle_fast.so")
_use_fast = False


def use_timing_build(on: bool = True):
    """Switches this module to ``libjgpt_oracle_fast.so``: the same C file compiled ``-O3 -march=native`` on THIS
    machine (always rebuilt: a copy built on another CPU may use instructions this one lacks).  For timing the CPU
    baseline only; parity checks use the strict build (``-ffp-contract=off``), which stays the default."""
    global _lib, _use_fast
    if on:
        subprocess.run(["make", "-B", "-C", _HERE, "timing"], check=True, capture_output=True)
    if on != _use_fast:
        _use_fast, _lib = on, None


def lib():
    global _lib
    if _lib is not None:
        return _lib
    if not _use_fast:
        build()
    L = C.CDLL(_FAST_PATH if _use_fast else _LIB_PATH)
    vp, ci, cf = C.c_void_p, C.c_int, C.c_float
    sig = {
        "og_rmsnorm": (None, [_f32p, _f32p, _f32p, ci, ci, cf]),
        "og_matmul": (None, [_f32p, _f32p, _f32p, ci, ci, ci]),
        "og_softmax_last_dim": (None, [_f32p, _f32p, C.c_long, ci]),
        "og_sigmoid": (None, [_f32p, _f32p, ci]),
        "og_split_heads": (None, [_f32p, _f32p, ci, ci, ci, ci]),
        "og_concat_heads": (None, [_f32p, _f32p, ci, ci, ci, ci]),
        "og_rope_4d": (None, [_f32p, _f32p, ci, ci, ci, ci, vp, ci, ci]),
        "og_round_fp16": (cf, [cf]),
        "og_cache_create": (vp, [ci, ci, ci, ci]),
        "og_cache_free": (None, [vp]),
        "og_cache_clear": (None, [vp]),
        "og_cache_length": (ci, [vp]),
        "og_cache_set_length": (ci, [vp, ci]),
        "og_cache_set_kv_fp16": (None, [vp, ci]),
        "og_cache_drop_front": (ci, [vp, ci]),
        "og_forward_decode_rolling": (ci, [vp, ci, vp, ci, ci, _f32p]),
        "og_generate_greedy_rolling": (ci, [vp, _i32p, ci, ci, ci, ci, _i32p]),
        "og_cache_k": (C.POINTER(C.c_float), [vp, ci]),
        "og_cache_v": (C.POINTER(C.c_float), [vp, ci]),
        "og_attn_query_one": (None, [_f32p, _f32p, _f32p, ci, ci, cf, _f32p, _f32p]),
        "og_attn_prefill_causal": (None, [_f32p, _f32p, _f32p, _f32p, ci, ci, ci, cf]),
        "og_model_create": (vp, [ci, ci, ci, ci, ci, ci, cf]),
        "og_model_free": (None, [vp]),
        "og_model_num_tensors": (ci, [vp]),
        "og_model_tensor": (C.POINTER(C.c_float), [vp, ci, C.POINTER(ci), C.POINTER(ci), C.POINTER(ci)]),
        "og_model_save": (ci, [vp, C.c_char_p]),
        "og_model_load": (ci, [vp, C.c_char_p]),
        "og_forward_prefill": (ci, [vp, _i32p, ci, vp, ci, _f32p]),
        "og_forward": (ci, [vp, _i32p, ci, _f32p]),
        "og_forward_decode": (ci, [vp, ci, vp, ci, ci, _f32p]),
        "og_argmax": (ci, [_f32p, ci]),
        "og_sample_next_token": (ci, [_f32p, ci, cf, ci, cf]),
        "og_generate_greedy": (ci, [vp, _i32p, ci, ci, ci, _i32p, vp]),
        "og_decode_attn_batch": (None, [_f32p, _f32p, _f32p, _f32p, _f32p, _i32p, _i32p, ci, ci, ci, ci, ci, _f32p]),
        "og_num_threads": (ci, []),
        "og_set_num_threads": (None, [ci]),
    }
    for name, (res, args) in sig.items():
        fn = getattr(L, name)
        fn.restype, fn.argtypes = res, args
    _lib = L
    return L


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


# ---------------------------------------------------------------- elementary ops
def rmsnorm(x, gamma, eps):
    x = _f32(x)
    out = np.empty_like(x)
    D = x.shape[-1]
    lib().og_rmsnorm(x, _f32(gamma), out, x.size // D, D, eps)
    return out


def matmul(a, b):
    a, b = _f32(a), _f32(b)
    M, K = a.shape
    K2, N = b.shape
    assert K == K2
    c = np.empty((M, N), np.float32)
    lib().og_matmul(a, b, c, M, K, N)
    return c


def softmax_last_dim(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().og_softmax_last_dim(x, out, x.size // x.shape[-1], x.shape[-1])
    return out


def sigmoid(x):
    x = _f32(x)
    out = np.empty_like(x)
    lib().og_sigmoid(x, out, x.size)
    return out


def split_heads(x, H):
    x = _f32(x)
    B, S, D = x.shape
    out = np.empty((B, H, S, D // H), np.float32)
    lib().og_split_heads(x, out, B, S, D, H)
    return out


def concat_heads(x):
    x = _f32(x)
    B, H, S, Dh = x.shape
    out = np.empty((B, S, H * Dh), np.float32)
    lib().og_concat_heads(x, out, B, H, S, Dh)
    return out


def rope_4d(x, positions=None, pos_base_offset=0):
    x = _f32(x)
    B, H, S, Dh = x.shape
    out = np.empty_like(x)
    if positions is None:
        lib().og_rope_4d(x, out, B, H, S, Dh, None, 0, pos_base_offset)
    else:
        p = np.ascontiguousarray(positions, dtype=np.int32)
        lib().og_rope_4d(x, out, B, H, S, Dh, p.ctypes.data, p.size, pos_base_offset)
    return out


def round_fp16(x):
    """binary16 round-to-nearest-even, back in fp32 (numpy's conversion is RNE as well)."""
    return np.asarray(x, np.float32).astype(np.float16).astype(np.float32)


def attn_query_one(q, k, v, scale):
    q, k, v = _f32(q), _f32(k), _f32(v)
    L, Dh = k.shape
    out = np.empty(Dh, np.float32)
    lib().og_attn_query_one(q, k, v, L, Dh, scale, out, np.empty(L, np.float32))
    return out


def attn_prefill_causal(q, k, v, scale):
    q, k, v = _f32(q), _f32(k), _f32(v)
    H, S, Dh = q.shape
    out = np.empty_like(q)
    lib().og_attn_prefill_causal(q, k, v, out, H, S, Dh, scale)
    return out


def decode_attn_batch(q, k, v, kc, vc, lens, rope_pos, H, Dh, max_seq, kv_fp16=True):
    """Append one token per sequence into contiguous planes kc/vc [n,H,max_seq,Dh] (updated in
    place) and attend over lens[i]+1 keys.  Returns [n, H*Dh]."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    assert kc.dtype == np.float32 and vc.dtype == np.float32 and kc.flags.c_contiguous and vc.flags.c_contiguous
    n = q.shape[0]
    out = np.empty((n, H * Dh), np.float32)
    lib().og_decode_attn_batch(
        q, k, v, kc, vc, np.ascontiguousarray(lens, np.int32), np.ascontiguousarray(rope_pos, np.int32),
        n, H, Dh, max_seq, 1 if kv_fp16 else 0, out,
    )
    return out


# ---------------------------------------------------------------- cache + model objects
class KvCache:
    """Contiguous fp32 cache [H, maxSeq, Dh] per layer (reference: model/KvCache.java)."""

    def __init__(self, layers, heads, dhead, max_seq, kv_fp16=False):
        self._h = lib().og_cache_create(layers, heads, dhead, max_seq)
        if not self._h:
            raise ValueError("KvCache dims must be positive")
        self.layers, self.heads, self.dhead, self.max_seq = layers, heads, dhead, max_seq
        lib().og_cache_set_kv_fp16(self._h, 1 if kv_fp16 else 0)

    def _plane(self, fn, layer):
        p = fn(self._h, layer)
        if not p:
            raise IndexError(layer)
        return np.ctypeslib.as_array(p, shape=(self.heads, self.max_seq, self.dhead))

    def k(self, layer):
        return self._plane(lib().og_cache_k, layer)

    def v(self, layer):
        return self._plane(lib().og_cache_v, layer)

    def length(self):
        return lib().og_cache_length(self._h)

    def set_length(self, n):
        if lib().og_cache_set_length(self._h, n):
            raise ValueError("length out of range")

    def clear(self):
        lib().og_cache_clear(self._h)

    def drop_front(self, n_tokens):
        """Rolling window: forget the oldest n_tokens (rows shift to the front, payload untouched)."""
        if lib().og_cache_drop_front(self._h, n_tokens):
            raise ValueError("cannot drop more tokens than the cache holds")

    def close(self):
        if self._h:
            lib().og_cache_free(self._h)
            self._h = None

    def __del__(self):
        self.close()


class Model:
    """fp32 JGPT decoder (reference: model/GPTModel.java, GptKvForward.java)."""

    def __init__(self, vocab, max_seq, d_model, heads, layers, d_ff, eps=1e-5):
        self._h = lib().og_model_create(vocab, max_seq, d_model, heads, layers, d_ff, eps)
        if not self._h:
            raise ValueError("bad model geometry")
        self.vocab, self.max_seq, self.d_model, self.heads = vocab, max_seq, d_model, heads
        self.layers, self.d_ff, self.eps = layers, d_ff, eps
        self.dhead = d_model // heads

    def tensors(self):
        """Views of the parameter tensors in file order (tok, pos, 9 per layer, normFinal, lmHead)."""
        out = []
        r, d0, d1 = C.c_int(), C.c_int(), C.c_int()
        for i in range(lib().og_model_num_tensors(self._h)):
            p = lib().og_model_tensor(self._h, i, C.byref(r), C.byref(d0), C.byref(d1))
            shape = (d0.value, d1.value) if r.value == 2 else (d0.value,)
            out.append(np.ctypeslib.as_array(p, shape=shape))
        return out

    def init_random(self, seed=0, std=0.02):
        """Every 2-D tensor N(0, std) from numpy default_rng(seed) in file order; RMSNorm gammas 1."""
        rng = np.random.default_rng(seed)
        for t in self.tensors():
            if t.ndim == 2:
                t[...] = rng.normal(0.0, std, size=t.shape).astype(np.float32)
            else:
                t[...] = 1.0
        return self

    def save(self, path):
        if lib().og_model_save(self._h, os.fsencode(path)):
            raise OSError(path)

    def load(self, path):
        rc = lib().og_model_load(self._h, os.fsencode(path))
        if rc:
            raise OSError(f"{path}: rc={rc}")

    def new_cache(self, kv_fp16=False):
        return KvCache(self.layers, self.heads, self.dhead, self.max_seq, kv_fp16)

    def forward(self, ids):
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty((ids.size, self.vocab), np.float32)
        rc = lib().og_forward(self._h, ids, ids.size, out)
        if rc:
            raise ValueError(f"forward rc={rc}")
        return out

    def forward_prefill(self, ids, cache, rope_offset=0):
        ids = np.ascontiguousarray(ids, np.int32)
        out = np.empty((ids.size, self.vocab), np.float32)
        rc = lib().og_forward_prefill(self._h, ids, ids.size, cache._h, rope_offset, out)
        if rc:
            raise ValueError(f"forward_prefill rc={rc}")
        return out

    def forward_decode(self, tok, cache, cache_len_before, rope_position):
        out = np.empty(self.vocab, np.float32)
        rc = lib().og_forward_decode(self._h, int(tok), cache._h, cache_len_before, rope_position, out)
        if rc == -2:
            raise RuntimeError("cache length mismatch or cache full")
        if rc:
            raise ValueError(f"forward_decode rc={rc}")
        return out

    def forward_decode_rolling(self, tok, cache, cache_len_before, rope_position):
        """Decode step of the rolling-window mode: RoPE at the absolute position, position row = position mod maxSeq."""
        out = np.empty(self.vocab, np.float32)
        rc = lib().og_forward_decode_rolling(self._h, int(tok), cache._h, cache_len_before, rope_position, out)
        if rc == -2:
            raise RuntimeError("cache length mismatch or cache full")
        if rc:
            raise ValueError(f"forward_decode_rolling rc={rc}")
        return out

    def generate_greedy_rolling(self, prompt, max_new, kv_fp16=False, block=16):
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(prompt.size + max_new, np.int32)
        n = lib().og_generate_greedy_rolling(self._h, prompt, prompt.size, max_new, 1 if kv_fp16 else 0, block, out)
        if n < 0:
            raise ValueError(f"generate_rolling rc={n}")
        return out, n

    def generate_greedy(self, prompt, max_new, kv_fp16=False, trace=False):
        prompt = np.ascontiguousarray(prompt, np.int32)
        out = np.zeros(prompt.size + max_new, np.int32)
        tr = np.zeros((max_new, self.vocab), np.float32) if trace else None
        n = lib().og_generate_greedy(
            self._h, prompt, prompt.size, max_new, 1 if kv_fp16 else 0, out, tr.ctypes.data if trace else None
        )
        if n == -2:
            raise RuntimeError("sliding window empty")
        if n < 0:
            raise ValueError(f"generate rc={n}")
        return (out, n, tr) if trace else (out, n)

    def close(self):
        if self._h:
            lib().og_model_free(self._h)
            self._h = None

    def __del__(self):
        self.close()


def argmax(logits):
    logits = _f32(logits)
    return lib().og_argmax(logits, logits.size)


def sample_next_token(logits, temperature, top_k, u01):
    logits = _f32(logits)
    return lib().og_sample_next_token(logits, logits.size, temperature, top_k, u01)


def num_threads():
    return lib().og_num_threads()


def set_num_threads(n):
    lib().og_set_num_threads(int(n))


# ---------------------------------------------------------------- paged allocator reference
class PagedAllocatorRef:
    """Written specification of the block allocator the CUDA library implements on the host.

    The reference has no paged cache; this class is the definition the library's block tables,
    append indices and eviction results are compared with bit for bit.

    Policy (deterministic):
      * physical blocks 0..n_blocks-1; the free list is a LIFO stack initialised so that block 0
        is handed out first, then 1, 2, ...; freed blocks are pushed in ascending logical order of
        the freed sequence, so the most recently freed block is reused first;
      * sequence slots: lowest free slot id first;
      * ``reserve(seq, n_tokens)`` grows the sequence's table to ceil(n_tokens/block_tokens) blocks,
        all or nothing;
      * every ``touch`` (append / attention on the sequence) stamps the sequence with a
        monotonically increasing tick; ``evict_lru(need)`` frees whole sequences marked evictable
        (finished) in ascending (tick, seq id) order until ``need`` blocks are free.
    """

    def __init__(self, n_blocks, block_tokens, max_seqs, max_blocks_per_seq):
        self.n_blocks, self.bt = n_blocks, block_tokens
        self.max_seqs, self.mbs = max_seqs, max_blocks_per_seq
        self.free = list(range(n_blocks - 1, -1, -1))  # pop() from the end -> 0 first
        self.tables: dict[int, list[int]] = {}
        self.length: dict[int, int] = {}
        self.tick: dict[int, int] = {}
        self.evictable: dict[int, bool] = {}
        self.clock = 0

    def seq_alloc(self):
        for s in range(self.max_seqs):
            if s not in self.tables:
                self.tables[s], self.length[s], self.evictable[s] = [], 0, False
                self.clock += 1
                self.tick[s] = self.clock
                return s
        return -1

    def seq_free(self, s):
        for b in self.tables.pop(s):
            self.free.append(b)
        del self.length[s], self.tick[s], self.evictable[s]

    def reserve(self, s, n_tokens):
        need = -(-n_tokens // self.bt) - len(self.tables[s])
        if need <= 0:
            return True
        if len(self.tables[s]) + need > self.mbs or need > len(self.free):
            return False
        for _ in range(need):
            self.tables[s].append(self.free.pop())
        return True

    def set_table(self, s, blocks):
        """Explicit table (microbenchmark: a seeded permutation of the pool)."""
        blocks = [int(b) for b in blocks]
        fs = set(self.free)
        if any(b not in fs for b in blocks) or len(set(blocks)) != len(blocks):
            return False
        for b in self.tables[s]:
            self.free.append(b)
        for b in blocks:
            self.free.remove(b)
        self.tables[s] = blocks
        return True

    def drop_front(self, s, n_blocks):
        """Rolling window: the oldest n_blocks blocks of s go back to the free list (in table order, so the first
        dropped block is handed out last), the table shifts left, the length drops by n_blocks * block_tokens."""
        if n_blocks < 0 or n_blocks > len(self.tables[s]) or self.length[s] < n_blocks * self.bt:
            return False
        for b in self.tables[s][:n_blocks]:
            self.free.append(b)
        del self.tables[s][:n_blocks]
        self.length[s] -= n_blocks * self.bt
        self.touch(s)
        return True

    def touch(self, s):
        self.clock += 1
        self.tick[s] = self.clock

    def append_index(self, s, pos):
        """(physical block, slot in block) of token position pos."""
        return self.tables[s][pos // self.bt], pos % self.bt

    def mark_evictable(self, s, flag=True):
        self.evictable[s] = flag

    def evict_lru(self, need_free):
        victims = []
        order = sorted((t, s) for s, t in self.tick.items() if self.evictable[s])
        for _, s in order:
            if len(self.free) >= need_free:
                break
            victims.append(s)
            self.seq_free(s)
        return victims


class ContinuousBatchRef:
    """Written specification of the continuous-batching policy, driven by precomputed per-request token
    streams (a request's tokens do not depend on what it is batched with).

    step(): FIFO admission reserving ceil((prompt + max_new - 1)/bt) blocks at once, evicting finished
    sequences least-recently-used first (one at a time, lower slot on ties) until blocks and a sequence slot
    are available, no overtaking; the admitted requests get their first token (prefill); the requests that
    were already running get one more token; a request finishes at max_new tokens or on token 0.
    Events: (1, request, slot) admit, (2, slot, request) evict, (3, request, n_tokens) finish."""

    def __init__(self, alloc: PagedAllocatorRef, max_running, max_rows, streams):
        self.a, self.max_running, self.max_rows, self.streams = alloc, min(max_running, max_rows), max_rows, streams
        self.reqs, self.waiting, self.running, self.events = [], [], [], []
        self.owner = {}

    def submit(self, prompt_len, max_new):
        self.reqs.append(dict(S=prompt_len, max_new=max_new, out=[], seq=-1, state=0))
        self.waiting.append(len(self.reqs) - 1)
        return len(self.reqs) - 1

    def _make_room(self, need):
        a = self.a
        while True:
            slot_ok = len(a.tables) < a.max_seqs
            if len(a.free) >= need and slot_ok:
                return True
            cand = sorted((t, s) for s, t in a.tick.items() if a.evictable[s])
            if not cand:
                return False
            victim = cand[0][1]
            self.events.append((2, victim, self.owner.pop(victim)))
            a.seq_free(victim)

    def step(self):
        a, produced = self.a, []
        decoding = list(self.running)
        admitted = []
        while self.waiting and len(self.running) < self.max_running:
            rid = self.waiting[0]
            r = self.reqs[rid]
            need = -(-(r["S"] + r["max_new"] - 1) // a.bt)
            if not self._make_room(need):
                break
            seq = a.seq_alloc()
            assert a.reserve(seq, r["S"] + r["max_new"] - 1)
            r["seq"], r["state"] = seq, 1
            self.owner[seq] = rid
            self.waiting.pop(0)
            self.running.append(rid)
            admitted.append(rid)
            self.events.append((1, rid, seq))
        for rid in admitted:  # prefill: set_length in admission order
            r = self.reqs[rid]
            a.touch(r["seq"])
            a.length[r["seq"]] = r["S"]
        for rid in admitted:
            r = self.reqs[rid]
            r["out"].append(int(self.streams[rid][0]))
            produced.append((rid, r["out"][-1]))
        for rid in decoding:
            r = self.reqs[rid]
            a.touch(r["seq"])
            a.length[r["seq"]] += 1
        for rid in decoding:
            r = self.reqs[rid]
            r["out"].append(int(self.streams[rid][len(r["out"])]))
            produced.append((rid, r["out"][-1]))
        still = []
        for rid in self.running:
            r = self.reqs[rid]
            if len(r["out"]) >= r["max_new"] or r["out"][-1] == 0:
                r["state"] = 2
                a.mark_evictable(r["seq"])
                self.events.append((3, rid, len(r["out"])))
            else:
                still.append(rid)
        self.running = still
        return produced


_ = OrderedDict  # (kept for callers that build ordered fixtures)
