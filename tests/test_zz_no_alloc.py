"""The allocation-free decode-attention entry point against the ordinary one, through the C ABI.

`jgpt_attn_decode_static_scratch` is for hosts that cannot call cudaMalloc while they generate (the
device is already full of their own buffers, or an allocation stall is unacceptable): its split-K
scratch is a fixed array inside the library.  It must give what `jgpt_attn_decode` gives.  The file is
named so that pytest collects it last: a run that stops at the first failure has then already run
everything else.  It passes on its own in a fresh process and after the other tests (the shared array
keeps old contents between calls, so two calls in a row are checked)."""
import numpy as np
import pytest

from helpers import PagedCase

pytestmark = pytest.mark.gpu
TOL = 2e-5


def test_static_scratch_decode_equals_ordinary_decode_twice_in_a_row(ctx):
    lens = [700, 3, 512, 129, 1024, 16, 0, 333]
    case = PagedCase(ctx, lens, H=24, Dh=16, layers=2, seed=77)
    try:
        rng = np.random.default_rng(78)
        n, D = case.n, 24 * 16
        rope_pos = np.array([max(l - 1, 0) for l in lens], np.int32)
        seq_d, rope_d, lens_d = case.seq_ids_dev(), ctx.from_host(rope_pos), ctx.from_host(case.lens)
        for call in range(2):
            layer = call  # second call: other layer, other queries, same shared scratch
            q = ctx.from_host(rng.standard_normal((n, D)).astype(np.float32))
            want, got = ctx.alloc((n, D)), ctx.alloc((n, D))
            want.fill_bytes(0x7F), got.fill_bytes(0x7F)
            case.pool.attn_decode(layer, 1, q, seq_d, rope_d, lens_d, n, 1024, want)
            case.pool.attn_decode_static_scratch(layer, q, seq_d, rope_d, lens_d, n, 1024, got)
            ctx.synchronize()
            w, g = want.to_host(), got.to_host()
            assert np.isfinite(g).all()
            assert np.abs(g - w).max() < TOL, (call, np.abs(g - w).max())
    finally:
        case.close()


def test_static_scratch_rejects_requests_beyond_its_size(ctx):
    case = PagedCase(ctx, [16], H=24, Dh=16, layers=1, seed=79, max_seq=8192)
    try:
        q = ctx.alloc((1, 384))
        one = ctx.from_host(np.zeros(1, np.int32))
        # 5000 rows x 24 heads x 18 words x >= 1 chunk is far beyond 1 Mi partial words (pointers are not touched)
        with pytest.raises(ValueError, match="static scratch holds"):
            case.pool.attn_decode_static_scratch(0, q, one, one, one, 5000, 8192, q)
        ctx.synchronize()
    finally:
        case.close()
