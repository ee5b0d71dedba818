"""GPU parity of single-query decode attention (plain and fused with the append) against the CPU
oracle, through the C ABI.  The oracle attends over the same fp16-rounded payload the paged store
holds, so the comparison isolates the kernel: tolerance 2e-5 max-abs on outputs of magnitude ~1
(fp32 accumulation order and exp2f vs expf).  The end-to-end logits budget is 2e-3."""
import os

import numpy as np
import pytest

import oracle as O
from helpers import PagedCase, oracle_decode as _oracle_decode

pytestmark = pytest.mark.gpu
TOL = 2e-5


@pytest.mark.parametrize("Dh,H", [(16, 24), (16, 5), (8, 4), (4, 2), (32, 6)])
def test_decode_attention_matches_oracle_ragged(ctx, Dh, H):
    lens = [1, 15, 16, 17, 33, 130, 257, 0]
    case = PagedCase(ctx, lens, H=H, Dh=Dh, layers=2, seed=11)
    try:
        rng = np.random.default_rng(5)
        n = case.n
        rope_pos = np.array([max(l - 1, 0) for l in lens], np.int32)
        for layer in range(2):
            q = rng.standard_normal((n, H * Dh)).astype(np.float32)
            out = ctx.alloc((n, H * Dh))
            out.fill_bytes(0x7F)
            case.pool.attn_decode(layer, 1, ctx.from_host(q), case.seq_ids_dev(), ctx.from_host(rope_pos),
                                  ctx.from_host(case.lens), n, int(max(lens)), out)
            ctx.synchronize()
            got = out.to_host()
            want = _oracle_decode(case, layer, q, lens, rope_pos)
            assert np.abs(got - want).max() < TOL, (Dh, H, layer, np.abs(got - want).max())
            assert not got[-1].any()  # empty sequence -> zero row
    finally:
        case.close()


@pytest.mark.parametrize("chunk_blocks,stages,persistent", [(1, 2, 0), (4, 3, 0), (8, 4, 1), (32, 8, 2), (1, 3, 2), (2, 4, 1)])
def test_split_and_pipeline_settings_agree(ctx, chunk_blocks, stages, persistent):
    """Every split / pipeline configuration gives the oracle's answer (split-K merge, ring wrap-around, one CTA
    per item, and the dynamic work queue: with 1- or 2-block items the launch has more items than resident
    CTAs, so CTAs claim several items each through the item ring)."""
    os.environ["JGPT_B200_CHUNK_BLOCKS"] = str(chunk_blocks)
    os.environ["JGPT_B200_STAGES"] = str(stages)
    os.environ["JGPT_B200_PERSISTENT"] = str(persistent)
    try:
        lens = [700, 3, 512, 129, 1024, 16]
        case = PagedCase(ctx, lens, H=24, Dh=16, layers=1, seed=21)
    finally:
        for k in ("JGPT_B200_CHUNK_BLOCKS", "JGPT_B200_STAGES", "JGPT_B200_PERSISTENT"):
            os.environ.pop(k)
    try:
        rng = np.random.default_rng(6)
        n, H, Dh = case.n, 24, 16
        q = rng.standard_normal((n, H * Dh)).astype(np.float32)
        rope_pos = np.array([l - 1 for l in lens], np.int32)
        out = ctx.alloc((n, H * Dh))
        for rep in range(2):  # twice: the arrival counters must have reset themselves
            out.fill_bytes(0x7F)
            case.pool.attn_decode(0, 1, ctx.from_host(q), case.seq_ids_dev(), ctx.from_host(rope_pos),
                                  ctx.from_host(case.lens), n, 1024, out)
            ctx.synchronize()
            got = out.to_host()
            want = _oracle_decode(case, 0, q, lens, rope_pos)
            assert np.abs(got - want).max() < TOL, (rep, np.abs(got - want).max())
    finally:
        case.close()


@pytest.mark.parametrize("fused", [False, True])
def test_tensor_core_consumer_matches_oracle(ctx, fused):
    """JGPT_B200_DECODE_MMA=1: scores and P.V on mma.sync with fp16 hi/lo split operands (d_head 16).  Same tolerance
    as the scalar consumer; ragged lengths, split-K, odd head count, dead slots in the last block poisoned with NaN."""
    os.environ["JGPT_B200_DECODE_MMA"] = "1"
    os.environ["JGPT_B200_CHUNK_BLOCKS"] = "4"
    try:
        lens0 = [1, 15, 16, 17, 33, 130, 257, 700]
        case = PagedCase(ctx, lens0, H=5, Dh=16, layers=1, seed=51, spare_tokens=2)
    finally:
        os.environ.pop("JGPT_B200_DECODE_MMA"), os.environ.pop("JGPT_B200_CHUNK_BLOCKS")
    try:
        rng = np.random.default_rng(52)
        n, H, Dh = case.n, 5, 16
        lens = np.array(lens0, np.int32)
        # poison everything beyond each sequence's tokens: the kernel must not let it reach the output
        ptr, nbytes = case.pool.storage()
        raw = np.empty(nbytes // 2, np.uint16)
        from jgpt_b200 import binding as B
        B.check(ctx._lib.jgpt_d2h(ctx.handle, raw.ctypes.data, ptr, nbytes))
        tiles = raw.reshape(1, case.n_blocks, H, 2, 16, Dh)
        for i, l in enumerate(lens0):
            blk, slot = case.tables[i][l // 16], l % 16
            if l // 16 < len(case.tables[i]):
                tiles[0, blk, :, :, slot:, :] = 0x7E00  # fp16 NaN
        B.check(ctx._lib.jgpt_h2d(ctx.handle, ptr, raw.ctypes.data, nbytes))
        q = rng.standard_normal((n, H * Dh)).astype(np.float32)
        out = ctx.alloc((n, H * Dh))
        if fused:
            k, v = (rng.standard_normal((n, H * Dh)).astype(np.float32) for _ in range(2))
            rope = (lens + 1).astype(np.int32)
            case.pool.attn_decode_append(0, 1, ctx.from_host(q), ctx.from_host(k), ctx.from_host(v), case.seq_ids_dev(),
                                         ctx.from_host(rope), ctx.from_host(lens + 1), n, int(lens.max()) + 1, out)
            want = O.decode_attn_batch(q, k, v, case.kc[0], case.vc[0], lens, rope, H, Dh, case.max_seq, kv_fp16=True)
        else:
            rope = (lens - 1).astype(np.int32)
            case.pool.attn_decode(0, 1, ctx.from_host(q), case.seq_ids_dev(), ctx.from_host(rope), ctx.from_host(lens), n,
                                  int(lens.max()), out)
            want = _oracle_decode(case, 0, q, lens0, rope)
        ctx.synchronize()
        got = out.to_host()
        assert np.isfinite(got).all() and np.abs(got - want).max() < TOL, np.abs(got - want).max()
    finally:
        case.close()


@pytest.mark.parametrize("Dh,H", [(16, 24), (8, 4)])
def test_fused_append_decode_matches_oracle_step_by_step(ctx, Dh, H):
    """Three decode steps of the fused kernel == oracle append + attend (payload bit-exact, outputs within TOL),
    and == the unfused pair (append kernel, then attention kernel) bit for bit on the payload."""
    lens0 = [0, 14, 15, 16, 47, 200]
    case = PagedCase(ctx, lens0, H=H, Dh=Dh, layers=2, seed=31, spare_tokens=4)
    try:
        rng = np.random.default_rng(8)
        n = case.n
        lens = np.array(lens0, np.int32)
        for step in range(3):
            rope_pos = (lens + 3).astype(np.int32)  # RoPE position differs from the slot on purpose
            q = rng.standard_normal((2, n, H * Dh)).astype(np.float32)
            k = rng.standard_normal((2, n, H * Dh)).astype(np.float32)
            v = rng.standard_normal((2, n, H * Dh)).astype(np.float32)
            out = ctx.alloc((2, n, H * Dh))
            # both layers in one launch (independent queries per layer)
            case.pool.attn_decode_append(0, 2, ctx.from_host(q), ctx.from_host(k), ctx.from_host(v), case.seq_ids_dev(),
                                         ctx.from_host(rope_pos), ctx.from_host(lens + 1), n, int(lens.max()) + 1, out)
            ctx.synchronize()
            got = out.to_host()
            for layer in range(2):
                want = O.decode_attn_batch(q[layer], k[layer], v[layer], case.kc[layer], case.vc[layer], lens, rope_pos,
                                           H, Dh, case.max_seq, kv_fp16=True)
                assert np.abs(got[layer] - want).max() < TOL, (step, layer, np.abs(got[layer] - want).max())
                for i in range(n):
                    kd, vd = ctx.alloc((H, case.max_seq, Dh)), ctx.alloc((H, case.max_seq, Dh))
                    case.pool.gather(layer, case.seqs[i], int(lens[i]) + 1, case.max_seq, kd, vd)
                    assert np.array_equal(kd.to_host().view(np.uint32), case.kc[layer, i].view(np.uint32))
                    assert np.array_equal(vd.to_host().view(np.uint32), case.vc[layer, i].view(np.uint32))
            lens = lens + 1
    finally:
        case.close()


def test_host_buffer_entry_point_equals_device_entry_point(ctx):
    lens0 = [31, 32, 100]
    a = PagedCase(ctx, lens0, H=24, Dh=16, layers=1, seed=41, spare_tokens=2)
    b = PagedCase(ctx, lens0, H=24, Dh=16, layers=1, seed=41, spare_tokens=2)
    try:
        rng = np.random.default_rng(9)
        n, D = 3, 24 * 16
        q, k, v = (rng.standard_normal((n, D)).astype(np.float32) for _ in range(3))
        lens1 = np.array(lens0, np.int32) + 1
        rope = np.array(lens0, np.int32)
        out_h = a.pool.attn_decode_append_host(0, 1, q, k, v, a.seqs, rope, lens1)
        out_d = ctx.alloc((n, D))
        b.pool.attn_decode_append(0, 1, ctx.from_host(q), ctx.from_host(k), ctx.from_host(v), b.seq_ids_dev(),
                                  ctx.from_host(rope), ctx.from_host(lens1), n, int(lens1.max()), out_d)
        assert np.array_equal(out_h, out_d.to_host())
        # page-locked buffers: the kernel reads and writes them in place (no staging copies); same bits
        c = PagedCase(ctx, lens0, H=24, Dh=16, layers=1, seed=41, spare_tokens=2)
        try:
            qp, kp, vp, op = (ctx.pinned_array((n, D)) for _ in range(4))
            qp[:], kp[:], vp[:] = q, k, v
            op[:] = np.nan
            # the first calls on a pool take turns between the transfer paths (kernel reading / writing the host
            # buffers itself; inputs copied + result written in place; staged copies): same bits from each.  The
            # same token is appended to the same slot every time, so the calls are idempotent.
            for _ in range(4):
                op[:] = np.nan
                got = c.pool.attn_decode_append_host(0, 1, qp, kp, vp, c.seqs, rope, lens1, out=op)
                assert got is op or np.shares_memory(got, op)
                assert np.array_equal(op, out_h)
            # the token appended from the page-locked k / v is the one the device path appended: a second query
            # over the grown caches (no append) sees the same keys and values
            q2 = ctx.from_host(rng.standard_normal((n, D)).astype(np.float32))
            o_b, o_c = ctx.alloc((n, D)), ctx.alloc((n, D))
            for case, o in ((b, o_b), (c, o_c)):
                case.pool.attn_decode(0, 1, q2, case.seq_ids_dev(), ctx.from_host(rope), ctx.from_host(lens1), n,
                                      int(lens1.max()), o)
            assert np.array_equal(o_b.to_host(), o_c.to_host())
        finally:
            c.close()
        with pytest.raises(RuntimeError):  # length beyond the reserved blocks -> IllegalState
            a.pool.attn_decode_append_host(0, 1, q, k, v, a.seqs, rope, lens1 + 64)
        with pytest.raises(IndexError):
            a.pool.attn_decode_append_host(0, 1, q, k, v, [0, 1, 7], rope, lens1)
    finally:
        a.close(), b.close()


@pytest.mark.parametrize("way", [0, 1, 2])
def test_every_way_of_moving_the_host_buffers_gives_the_same_bits(ctx, way, monkeypatch):
    """JGPT_B200_HOST_ZEROCOPY pins how the host-buffer entry point moves its bytes (0 staged copies pipelined over layer
    groups, 1 the kernel reads / writes the page-locked buffers itself, 2 inputs copied + result in place): six layers,
    page-locked buffers, same bits as the device entry point and the same appended token."""
    lens0 = [31, 32, 100, 7]
    layers, n, D = 6, 4, 24 * 16
    a = PagedCase(ctx, lens0, H=24, Dh=16, layers=layers, seed=43, spare_tokens=2)
    b = PagedCase(ctx, lens0, H=24, Dh=16, layers=layers, seed=43, spare_tokens=2)
    try:
        rng = np.random.default_rng(11)
        q, k, v = (rng.standard_normal((layers, n, D)).astype(np.float32) for _ in range(3))
        lens1 = np.array(lens0, np.int32) + 1
        rope = np.array(lens0, np.int32)
        out_d = ctx.alloc((layers, n, D))
        b.pool.attn_decode_append(0, layers, ctx.from_host(q), ctx.from_host(k), ctx.from_host(v), b.seq_ids_dev(),
                                  ctx.from_host(rope), ctx.from_host(lens1), n, int(lens1.max()), out_d)
        qp, kp, vp, op = (ctx.pinned_array((layers, n, D)) for _ in range(4))
        qp[:], kp[:], vp[:] = q, k, v
        monkeypatch.setenv("JGPT_B200_HOST_ZEROCOPY", str(way))
        for _ in range(2):  # idempotent: the same token goes to the same slot
            op[:] = np.nan
            a.pool.attn_decode_append_host(0, layers, qp, kp, vp, a.seqs, rope, lens1, out=op)
            assert np.array_equal(op, out_d.to_host())
        q2 = ctx.from_host(rng.standard_normal((layers, n, D)).astype(np.float32))
        o_a, o_b = ctx.alloc((layers, n, D)), ctx.alloc((layers, n, D))
        for case, o in ((a, o_a), (b, o_b)):
            case.pool.attn_decode(0, layers, q2, case.seq_ids_dev(), ctx.from_host(rope), ctx.from_host(lens1), n, int(lens1.max()), o)
        assert np.array_equal(o_a.to_host(), o_b.to_host())
    finally:
        a.close(), b.close()


def test_device_self_checks_report_instead_of_faulting(ctx):
    """A block table entry outside the pool is recorded in the status word (read by synchronize), the access
    is redirected inside the pool, nothing faults."""
    case = PagedCase(ctx, [40], H=2, Dh=16, layers=1, seed=1)
    try:
        q = np.zeros((1, 32), np.float32)
        out = ctx.alloc((1, 32))
        # lens says 40 tokens but claim a bound of 16: flagged, clamped
        case.pool.attn_decode(0, 1, ctx.from_host(q), case.seq_ids_dev(), ctx.from_host(np.array([0], np.int32)),
                              ctx.from_host(case.lens), 1, 16, out)
        from jgpt_b200 import JgptError
        with pytest.raises(JgptError, match="len-over-bound"):
            ctx.synchronize()
        ctx.synchronize()  # status word was cleared; the context stays usable
        # sequence id outside the pool
        case.pool.attn_decode(0, 1, ctx.from_host(q), ctx.from_host(np.array([99], np.int32)),
                              ctx.from_host(np.array([0], np.int32)), ctx.from_host(case.lens), 1, 64, out)
        with pytest.raises(JgptError, match="bad-seq-id"):
            ctx.synchronize()
        ctx.synchronize()
    finally:
        case.close()


@pytest.mark.parametrize("overlap", [1, 2])
def test_overlapped_launches_give_the_same_result(ctx, overlap):
    """Decode attention as a programmatic dependent launch: a chain of per-layer fused append + attention launches
    (eager and replayed as a CUDA graph) whose kernels start while their predecessor drains -- with overlap 2 the copy
    warp already fetches tables and K/V slabs -- gives the outputs of ordinary launches (within the kernel's tolerance: the launch shape differs), bit-identical cache
    contents, and the oracle's answer."""
    lens = [700, 3, 512, 129, 1023, 16, 333, 64]
    L = 4
    cases = [PagedCase(ctx, lens, H=24, Dh=16, layers=L, seed=31, spare_tokens=1) for _ in range(2)]
    try:
        rng = np.random.default_rng(32)
        n, D = len(lens), 24 * 16
        q, k, v = (rng.standard_normal((L, n, D)).astype(np.float32) for _ in range(3))
        new_lens = np.asarray(lens, np.int32) + 1
        rope = np.asarray(lens, np.int32)
        outs = []
        for case, ov in zip(cases, (0, overlap)):
            case.pool.set_tuning(launch_overlap=ov)
            qd, kd, vd = ctx.from_host(q), ctx.from_host(k), ctx.from_host(v)
            out = ctx.alloc((L, n, D))
            sd, rd, ld = case.seq_ids_dev(), ctx.from_host(rope), ctx.from_host(new_lens)
            slab = n * D * 4

            def chain():
                for layer in range(L):
                    case.pool.attn_decode_append(layer, 1, qd.ptr + layer * slab, kd.ptr + layer * slab, vd.ptr + layer * slab,
                                                 sd, rd, ld, n, 1024, out.ptr + layer * slab)

            chain()
            ctx.synchronize()
            eager = out.to_host()
            g = ctx.capture(chain)  # the appended token is rewritten with the same payload: same answer
            out.fill_bytes(0x7F)
            for _ in range(3):
                g.launch()
            ctx.synchronize()
            g.close()
            assert np.array_equal(out.to_host(), eager)
            outs.append(eager)
        # the overlapped launch picks its own head grouping and ring depth, so the split-K merge order differs:
        # equal within the kernel's tolerance, not bit for bit
        assert np.abs(outs[0] - outs[1]).max() < TOL
        # against the oracle (layer 2), and the payload the overlapped chain appended
        c = cases[1]
        kc, vc = np.ascontiguousarray(c.kc[2]), np.ascontiguousarray(c.vc[2])
        want = O.decode_attn_batch(q[2], k[2], v[2], kc, vc, np.asarray(lens, np.int32), rope, 24, 16, c.max_seq)
        assert np.abs(outs[1][2] - want).max() < TOL
        kd2, vd2 = ctx.alloc((24, c.max_seq, 16)), ctx.alloc((24, c.max_seq, 16))
        c.pool.gather(2, c.seqs[0], lens[0] + 1, c.max_seq, kd2, vd2)
        assert np.array_equal(kd2.to_host(), kc[0]) and np.array_equal(vd2.to_host(), vc[0])
    finally:
        for c in cases:
            c.close()
