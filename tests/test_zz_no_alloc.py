"""The allocation-free decode-attention entry point, through the C ABI.

`jgpt_attn_decode_static_scratch` is for hosts that cannot call cudaMalloc while they generate (the
device is already full of their own buffers, or an allocation stall is unacceptable): its split-K
scratch is a fixed array inside the library.  It must give what `jgpt_attn_decode` gives, and what the
CPU oracle gives, and it must leave the device's free memory exactly where it found it.  The file is
named so that pytest collects it last: a run that stops at the first failure has then already run
everything else.  It passes on its own in a fresh process and after the other tests (the shared array
keeps old contents between calls, so two calls in a row are checked)."""
import numpy as np
import pytest

from helpers import PagedCase, oracle_decode

pytestmark = pytest.mark.gpu
TOL = 2e-5


def test_static_scratch_decode_equals_ordinary_decode_and_the_oracle_twice_in_a_row(ctx):
    lens = [700, 3, 512, 129, 1024, 16, 0, 333]
    case = PagedCase(ctx, lens, H=24, Dh=16, layers=2, seed=77)
    try:
        rng = np.random.default_rng(78)
        n, D = case.n, 24 * 16
        rope_pos = np.array([max(l - 1, 0) for l in lens], np.int32)
        seq_d, rope_d, lens_d = case.seq_ids_dev(), ctx.from_host(rope_pos), ctx.from_host(case.lens)
        # set-up only (n = 0): this is where the GPU takes the array and loads the kernel
        case.pool.attn_decode_static_scratch(0, None, None, None, None, 0, 1024, None)
        want_d, got_d = ctx.alloc((n, D)), ctx.alloc((n, D))
        q_d = ctx.alloc((n, D))
        for call in range(2):
            layer = call  # second call: other layer, other queries, same shared scratch
            q = rng.standard_normal((n, D)).astype(np.float32)
            q_d.copy_from(q)
            want_d.fill_bytes(0x7F), got_d.fill_bytes(0x7F)
            case.pool.attn_decode(layer, 1, q_d, seq_d, rope_d, lens_d, n, 1024, want_d)
            ctx.synchronize()
            free_before, _ = ctx.mem_info()
            case.pool.attn_decode_static_scratch(layer, q_d, seq_d, rope_d, lens_d, n, 1024, got_d)
            ctx.synchronize()
            free_after, _ = ctx.mem_info()
            # sequences of 1024 tokens are split into chunks here, so the scratch is in use; nothing was allocated for it
            assert free_after == free_before, (call, free_before - free_after)
            w, g = want_d.to_host(), got_d.to_host()
            assert np.isfinite(g).all()
            assert np.abs(g - w).max() < TOL, (call, np.abs(g - w).max())
            o = oracle_decode(case, layer, q, lens, rope_pos)
            assert np.abs(g - o).max() < TOL, (call, np.abs(g - o).max())
            assert not g[6].any()  # the empty sequence gets a zero row
    finally:
        case.close()


def test_static_scratch_does_not_allocate_where_the_ordinary_call_must_grow_its_scratch(ctx):
    """A fresh pool has no split-K scratch yet: the ordinary entry point would cudaMalloc it on this very call.
    The static one serves the same request with the device's free memory unchanged."""
    lens = [1024] * 6
    case = PagedCase(ctx, lens, H=24, Dh=16, layers=1, seed=80)
    try:
        rng = np.random.default_rng(81)
        n, D = case.n, 24 * 16
        rope_pos = np.array([l - 1 for l in lens], np.int32)
        seq_d, rope_d, lens_d = case.seq_ids_dev(), ctx.from_host(rope_pos), ctx.from_host(case.lens)
        q = rng.standard_normal((n, D)).astype(np.float32)
        q_d, got_d = ctx.from_host(q), ctx.alloc((n, D))
        case.pool.attn_decode_static_scratch(0, None, None, None, None, 0, 1024, None)  # set-up, once per device
        # one unsplit launch (a single 16-token chunk touches no scratch at all), so that whatever the driver sets
        # up at a kernel's very first launch in a process is not counted against the call under test
        short_d = ctx.from_host(np.full(n, 16, np.int32))
        case.pool.attn_decode_static_scratch(0, q_d, seq_d, rope_d, short_d, 1, 16, got_d)
        ctx.synchronize()
        free_before, _ = ctx.mem_info()
        case.pool.attn_decode_static_scratch(0, q_d, seq_d, rope_d, lens_d, n, 1024, got_d)
        ctx.synchronize()
        free_after, _ = ctx.mem_info()
        assert free_after == free_before, free_before - free_after
        assert np.abs(got_d.to_host() - oracle_decode(case, 0, q, lens, rope_pos)).max() < TOL
    finally:
        case.close()


def test_static_scratch_rejects_requests_beyond_its_size(ctx):
    case = PagedCase(ctx, [16], H=24, Dh=16, layers=1, seed=79, max_seq=8192)
    try:
        q = ctx.alloc((1, 384))
        one = ctx.from_host(np.zeros(1, np.int32))
        # 5000 rows x 24 heads x 18 words x several chunks is far beyond 1 Mi partial words (pointers are not touched)
        with pytest.raises(ValueError, match="static scratch holds"):
            case.pool.attn_decode_static_scratch(0, q, one, one, one, 5000, 8192, q)
        ctx.synchronize()
    finally:
        case.close()
