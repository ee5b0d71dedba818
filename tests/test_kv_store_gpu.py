"""GPU parity of the paged KV store (append with fused RoPE, gather, block tables, eviction) against
the CPU oracle, through the C ABI.  Integer results are bit-exact; K/V payloads equal
fp16_rn(oracle fp32) bit for bit (both sides take cos/sin from the host libm and keep the
multiplies and the add/sub of the rotation as separate roundings)."""
import numpy as np
import pytest

import oracle as O
from jgpt_b200 import KvCacheGpu, KvPool, PoolExhausted
from helpers import PagedCase

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("Dh,H", [(16, 24), (16, 2), (8, 4), (4, 4), (32, 3)])
@pytest.mark.parametrize("lens", [[1], [15, 16, 17, 33], [0, 5, 64]])
def test_append_then_gather_matches_oracle_bit_exact(ctx, Dh, H, lens):
    case = PagedCase(ctx, lens, H=H, Dh=Dh, layers=2, seed=3, rope_pos_offset=2)
    try:
        for layer in range(2):
            for i, l in enumerate(lens):
                kd = ctx.alloc((H, case.max_seq, Dh))
                vd = ctx.alloc((H, case.max_seq, Dh))
                kd.fill_bytes(0x7F), vd.fill_bytes(0x7F)
                case.pool.gather(layer, case.seqs[i], l, case.max_seq, kd, vd)
                k, v = kd.to_host(), vd.to_host()
                assert np.array_equal(k.view(np.uint32), case.kc[layer, i].view(np.uint32)), (Dh, H, layer, i)
                assert np.array_equal(v.view(np.uint32), case.vc[layer, i].view(np.uint32))
        ctx.synchronize()
    finally:
        case.close()


def test_block_tables_follow_the_allocator_specification(ctx):
    """reserve / free / reuse order, host table == device mirror == written specification."""
    ref = O.PagedAllocatorRef(n_blocks=40, block_tokens=16, max_seqs=6, max_blocks_per_seq=12)
    pool = KvPool(ctx, 1, 2, 16, 40, 6, 12)
    try:
        rng = np.random.default_rng(7)
        live = {}
        for step in range(200):
            op = rng.integers(0, 4)
            if op == 0 and len(live) < 6:
                s_ref, s = ref.seq_alloc(), pool.seq_alloc()
                assert s == s_ref
                live[s] = 0
            elif op == 1 and live:
                s = int(rng.choice(list(live)))
                want = live[s] + int(rng.integers(1, 40))
                ok_ref = ref.reserve(s, want)
                try:
                    pool.reserve(s, want)
                    ok = True
                except (PoolExhausted, ValueError):
                    ok = False
                assert ok == ok_ref
                if ok:
                    live[s] = want
            elif op == 2 and live:
                s = int(rng.choice(list(live)))
                ref.seq_free(s), pool.seq_free(s)
                del live[s]
            for s in live:
                t = pool.block_table(s)
                assert t.tolist() == ref.tables[s], (step, s)
                assert pool.block_table(s, device=True).tolist() == ref.tables[s]
            assert pool.free_blocks() == len(ref.free)
    finally:
        pool.close()


def test_append_index_is_block_table_lookup(ctx):
    """Token at position p of a sequence lands in physical block table[p // 16], slot p % 16, for
    every layer and head; nothing else in the pool is touched."""
    H, Dh, L = 3, 16, 2
    pool = KvPool(ctx, L, H, Dh, 8, 2, 4)
    try:
        s = pool.seq_alloc()
        pool.set_block_table(s, [5, 2, 7])
        ptr, nbytes = pool.storage()
        pos = 37
        k = np.arange(H * Dh, dtype=np.float32).reshape(1, -1) + 1
        v = -k
        pool.append(1, ctx.from_host(k), ctx.from_host(v), ctx.from_host(np.array([s], np.int32)),
                    ctx.from_host(np.array([pos], np.int32)), ctx.from_host(np.array([0], np.int32)), 1)
        raw = np.empty(nbytes // 2, np.float16)
        from jgpt_b200 import binding as B
        B.check(ctx._lib.jgpt_d2h(ctx.handle, raw.ctypes.data, ptr, nbytes))
        raw = raw.reshape(L, 8, H, 2, 16, Dh)
        expect = np.zeros_like(raw)
        expect[1, 7, :, 0, pos % 16] = k.reshape(H, Dh)  # RoPE at position 0 is the identity
        expect[1, 7, :, 1, pos % 16] = v.reshape(H, Dh)
        assert np.array_equal(raw, expect)
        ref = O.PagedAllocatorRef(8, 16, 2, 4)
        rs = ref.seq_alloc()
        assert ref.set_table(rs, [5, 2, 7]) and ref.append_index(rs, pos) == (7, 5)
    finally:
        pool.close()


def test_lru_eviction_matches_specification_and_scrubs(ctx):
    ref = O.PagedAllocatorRef(n_blocks=12, block_tokens=16, max_seqs=5, max_blocks_per_seq=6)
    pool = KvPool(ctx, 2, 2, 16, 12, 5, 6)
    try:
        seqs = []
        for need in (33, 16, 48, 20):  # 3 + 1 + 3 + 2 = 9 blocks
            s, r = pool.seq_alloc(), ref.seq_alloc()
            assert s == r
            pool.reserve(s, need), ref.reserve(r, need)
            pool.set_length(s, need), ref.touch(r)
            seqs.append(s)
        # poison the whole pool so that scrubbed blocks are recognisable
        ptr, nbytes = pool.storage()
        ctx._lib.jgpt_dev_memset(ctx.handle, ptr, 0x3C, nbytes)
        for s in (seqs[0], seqs[2], seqs[3]):
            pool.mark_evictable(s), ref.mark_evictable(s)
        pool.set_length(seqs[0], 33), ref.touch(seqs[0])  # seq 0 becomes the most recently used
        victims = pool.evict_lru(8, zero_fill=True)
        assert victims == ref.evict_lru(8)
        assert victims == [seqs[2], seqs[3]]
        assert pool.free_blocks() == len(ref.free) == 8
        # blocks come back in the specified order
        s_new, r_new = pool.seq_alloc(), ref.seq_alloc()
        assert s_new == r_new == seqs[2]
        pool.reserve(s_new, 16 * 6), ref.reserve(r_new, 16 * 6)
        assert pool.block_table(s_new).tolist() == ref.tables[r_new]
        assert pool.block_table(s_new, device=True).tolist() == ref.tables[r_new]
        raw = np.empty(nbytes // 2, np.uint16)
        from jgpt_b200 import binding as B
        B.check(ctx._lib.jgpt_d2h(ctx.handle, raw.ctypes.data, ptr, nbytes))
        raw = raw.reshape(2, 12, -1)
        freed = [4, 5, 6, 7, 8]  # blocks of seqs[2] (3) and seqs[3] (2): handed out in order 0..8
        for b in range(12):
            if b in freed:
                assert not raw[:, b].any(), b
            else:
                assert (raw[:, b] == 0x3C3C).all(), b
        with pytest.raises(PoolExhausted):
            pool.evict_lru(12)
    finally:
        pool.close()


def test_kv_cache_gpu_facade_contract(ctx):
    """Argument checks, length bookkeeping and clear() of the reference class
    (KvCacheTest ctor/bounds/length/clear cases, src/test/java/com/veles/llm/jgpt/model/KvCacheTest.java:80-118)."""
    with pytest.raises(ValueError):
        KvCacheGpu(0, 4, 16, 32, ctx=ctx)
    with pytest.raises(ValueError):
        KvCacheGpu(2, 4, 16, -1, ctx=ctx)
    c = KvCacheGpu(2, 4, 16, 40, ctx=ctx)
    try:
        assert (c.numLayers(), c.maxSeqLen(), c.length(), c.remainingCapacity(), c.isFull()) == (2, 40, 0, 40, False)
        with pytest.raises(ValueError):
            c.setLength(41)
        with pytest.raises(ValueError):
            c.setLength(-1)
        with pytest.raises(IndexError):
            c.getK(2)
        c.setLength(40)
        assert c.isFull() and c.remainingCapacity() == 0
        k = np.ones((3, 4 * 16), np.float32)
        ids = ctx.from_host(np.full(3, c.seq, np.int32))
        pos = ctx.from_host(np.arange(3, dtype=np.int32))
        c.pool.append(0, ctx.from_host(k), ctx.from_host(k), ids, pos, pos, 3)
        c.setLength(3)
        assert c.getV(0).to_host()[:, :3].min() == 1.0
        c.clear()
        assert c.length() == 0
        c.setLength(3)  # new blocks; the old ones were scrubbed
        assert not c.getK(0).to_host().any() and not c.getV(0).to_host().any()
    finally:
        c.close()
        c.close()  # idempotent


def test_batched_gather_equals_per_sequence_gather(ctx):
    """jgpt_kv_gather_batch: n caches in one launch give exactly the planes of n single gathers (ragged lengths, one empty)."""
    lens = [40, 0, 16, 129]
    case = PagedCase(ctx, lens, H=6, Dh=16, layers=2, seed=9)
    try:
        ms = case.max_seq
        kb, vb = ctx.alloc((len(lens), 6, ms, 16)), ctx.alloc((len(lens), 6, ms, 16))
        kb.fill_bytes(0x7F), vb.fill_bytes(0x7F)
        case.pool.gather_batch(1, case.seqs, lens, ms, kb, vb)
        ctx.synchronize()
        K, V = kb.to_host(), vb.to_host()
        k1, v1 = ctx.alloc((6, ms, 16)), ctx.alloc((6, ms, 16))
        for i, (s, l) in enumerate(zip(case.seqs, lens)):
            case.pool.gather(1, s, l, ms, k1, v1)
            assert np.array_equal(K[i], k1.to_host()) and np.array_equal(V[i], v1.to_host()), i
            assert np.array_equal(K[i], case.kc[1, i]) and np.array_equal(V[i], case.vc[1, i]), i
        with pytest.raises(ValueError):
            case.pool.gather_batch(1, case.seqs, [ms + 1] * 4, ms, kb, vb)
    finally:
        case.close()
