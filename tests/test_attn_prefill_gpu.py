"""GPU parity of the causal prefill attention that fills the paged cache (tensor-core kernel at d_head 16,
SIMT kernel otherwise) against the CPU oracle, through the C ABI.  The oracle attends over the fp16-rounded
RoPE'd K and V the store holds; the cache contents themselves must be bit-exact."""
import numpy as np
import pytest

import oracle as O
from jgpt_b200 import KvPool

pytestmark = pytest.mark.gpu
TOL = 2e-5


def _run_case(ctx, H, Dh, S_list, rope_offsets, seed, layers=2, layer=1, poison=False):
    D = H * Dh
    n = len(S_list)
    blocks = [-(-S // 16) for S in S_list]
    pool = KvPool(ctx, layers, H, Dh, sum(blocks) + 3, n, max(blocks), max_positions=max(S + r for S, r in zip(S_list, rope_offsets)))
    try:
        rng = np.random.default_rng(seed)
        perm = rng.permutation(sum(blocks) + 3).astype(np.int32)
        seqs, off = [], 0
        for b in blocks:
            s = pool.seq_alloc()
            pool.set_block_table(s, perm[off:off + b])
            off += b
            seqs.append(s)
        if poison:  # stale but finite garbage everywhere, as a long-running pool would hold
            ptr, nbytes = pool.storage()
            ctx._lib.jgpt_dev_memset(ctx.handle, ptr, 0x5B, nbytes)
        starts = np.concatenate([[0], np.cumsum(S_list)]).astype(np.int32)
        n_rows = int(starts[-1])
        q, k, v = (rng.standard_normal((n_rows, D)).astype(np.float32) for _ in range(3))
        out = ctx.alloc((n_rows, D))
        out.fill_bytes(0x7F)
        pool.attn_prefill(layer, ctx.from_host(q), ctx.from_host(k), ctx.from_host(v), seqs, starts, rope_offsets, out)
        ctx.synchronize()
        got = out.to_host()
        scale = 1.0 / np.sqrt(Dh)
        worst = 0.0
        for i, S in enumerate(S_list):
            sl = slice(starts[i], starts[i + 1])
            qh = O.rope_4d(O.split_heads(q[sl].reshape(1, S, D), H), pos_base_offset=rope_offsets[i])[0]
            kh = O.round_fp16(O.rope_4d(O.split_heads(k[sl].reshape(1, S, D), H), pos_base_offset=rope_offsets[i])[0])
            vh = O.round_fp16(O.split_heads(v[sl].reshape(1, S, D), H)[0])
            want = O.concat_heads(O.attn_prefill_causal(qh, kh, vh, scale)[None])[0]
            worst = max(worst, float(np.abs(got[sl] - want).max()))
            # the cache holds exactly the oracle's payload, zero beyond the prompt
            ms = blocks[i] * 16
            kd, vd = ctx.alloc((H, ms, Dh)), ctx.alloc((H, ms, Dh))
            pool.gather(layer, seqs[i], S, ms, kd, vd)
            kg, vg = kd.to_host(), vd.to_host()
            assert np.array_equal(kg[:, :S], kh) and np.array_equal(vg[:, :S], vh), (i, S)
            assert not kg[:, S:].any() and not vg[:, S:].any()
        return worst
    finally:
        pool.close()


@pytest.mark.parametrize("S_list", [[1], [15, 16, 17], [64, 65, 130], [200, 3, 1024]])
def test_prefill_tensor_core_kernel_matches_oracle(ctx, S_list):
    worst = _run_case(ctx, H=24, Dh=16, S_list=S_list, rope_offsets=[0, 5, 2][:len(S_list)], seed=100 + len(S_list))
    assert worst < TOL, worst


def test_prefill_over_stale_pool_contents(ctx):
    assert _run_case(ctx, H=3, Dh=16, S_list=[5, 33, 70], rope_offsets=[0, 0, 9], seed=7, poison=True) < TOL


@pytest.mark.parametrize("Dh,H", [(8, 4), (4, 2), (32, 3)])
def test_prefill_simt_kernel_matches_oracle(ctx, Dh, H):
    assert _run_case(ctx, H=H, Dh=Dh, S_list=[1, 17, 40], rope_offsets=[2, 0, 0], seed=5) < TOL


def test_prefill_then_decode_continues_the_same_sequence(ctx):
    """Prefill S tokens, then one fused decode step: equals the oracle's causal row S over S+1 keys."""
    H, Dh, S = 24, 16, 77
    D = H * Dh
    pool = KvPool(ctx, 1, H, Dh, 8, 1, 8, max_positions=128)
    try:
        s = pool.seq_alloc()
        pool.reserve(s, S + 1)
        rng = np.random.default_rng(3)
        q, k, v = (rng.standard_normal((S + 1, D)).astype(np.float32) for _ in range(3))
        out = ctx.alloc((S, D))
        pool.attn_prefill(0, ctx.from_host(q[:S]), ctx.from_host(k[:S]), ctx.from_host(v[:S]), [s], [0, S], [0], out)
        got = pool.attn_decode_append_host(0, 1, q[S:], k[S:], v[S:], [s], [S], [S + 1])
        qh = O.rope_4d(O.split_heads(q.reshape(1, S + 1, D), H))[0]
        kh = O.round_fp16(O.rope_4d(O.split_heads(k.reshape(1, S + 1, D), H))[0])
        vh = O.round_fp16(O.split_heads(v.reshape(1, S + 1, D), H)[0])
        want = O.concat_heads(O.attn_prefill_causal(qh, kh, vh, 0.25)[None])[0]
        assert np.abs(out.to_host() - want[:S]).max() < TOL
        assert np.abs(got[0] - want[S]).max() < TOL
    finally:
        pool.close()


def test_prefill_argument_checks(ctx):
    pool = KvPool(ctx, 1, 2, 16, 4, 2, 2, max_positions=32)
    try:
        s = pool.seq_alloc()
        pool.reserve(s, 16)
        buf = ctx.alloc((40, 32))
        with pytest.raises(RuntimeError):  # more prompt tokens than reserved blocks -> IllegalState
            pool.attn_prefill(0, buf, buf, buf, [s], [0, 17], [0], buf)
        with pytest.raises(ValueError):  # RoPE positions beyond the table -> IllegalArgument
            pool.attn_prefill(0, buf, buf, buf, [s], [0, 16], [17], buf)
        with pytest.raises(IndexError):
            pool.attn_prefill(0, buf, buf, buf, [1], [0, 16], [0], buf)
        with pytest.raises(IndexError):
            pool.attn_prefill(1, buf, buf, buf, [s], [0, 16], [0], buf)
    finally:
        pool.close()


def test_fast_operand_mode_stays_inside_its_stated_tolerance(ctx, monkeypatch):
    """JGPT_B200_PREFILL_FAST=1: the probabilities go to the tensor cores as single fp16 values (q keeps its fp16
    high + low split, so the scores are exact).  The cache payload is still bit-exact (the append does not change);
    attention outputs on N(0,1) inputs stay within 6e-4 of the oracle (2^-11 relative on every probability, measured
    3.9e-4; the exact mode: 2e-5).  The forward step of the model uses this mode by default and is held to the logits budget by the
    model tests."""
    monkeypatch.setenv("JGPT_B200_PREFILL_FAST", "1")
    worst = _run_case(ctx, 24, 16, [64, 65, 130, 1024], [0, 3, 0, 0], seed=41)
    assert worst < 6e-4, worst
    monkeypatch.delenv("JGPT_B200_PREFILL_FAST")
    exact = _run_case(ctx, 24, 16, [64, 65, 130, 1024], [0, 3, 0, 0], seed=41)
    assert exact < TOL, exact
