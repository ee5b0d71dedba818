"""GPU parity of the projection primitive (TensorOpsGPU.matmulGpuDevice) through the C ABI, on both of its
paths: the tcgen05 / tensor-memory kernel that prefill-sized products take and the mma.sync kernel for
decode-sized ones.  Both split every fp32 operand into two TF32 parts and accumulate three products in fp32.

Tolerance: max |C - C64| <= 2e-5 * max |C64| against a float64 product (K up to 2048; the tensor cores
truncate when they add into the fp32 accumulator, which leaves about 3e-9 * K of the largest element; a
k-ordered fp32 loop sits at about 6e-7).  Plain TF32, what the reference runs these GEMMs with, is ~1e-3."""
import os

import numpy as np
import pytest

import oracle as O
from jgpt_b200 import GPTModel, KvCacheGpu

pytestmark = pytest.mark.gpu
REL_TOL = 2e-5


class _env:
    def __init__(self, **kv):
        self.kv = {k: str(v) for k, v in kv.items()}

    def __enter__(self):
        self.old = {k: os.environ.get(k) for k in self.kv}
        os.environ.update(self.kv)

    def __exit__(self, *a):
        for k, v in self.old.items():
            if v is None:
                os.environ.pop(k, None)
            else:
                os.environ[k] = v


def _matmul(ctx, a, b, min_rows):
    M, K = a.shape
    N = b.shape[1]
    da, db, dc = ctx.from_host(a), ctx.from_host(b), ctx.alloc((M, N))
    dc.fill_bytes(0xFF)  # NaN: every element must be written
    with _env(JGPT_B200_UMMA_MIN_ROWS=min_rows):
        ctx.matmul(da, db, dc, M, K, N)
    ctx.synchronize()
    out = dc.to_host()
    da.close(), db.close(), dc.close()
    return out


@pytest.mark.parametrize("M,K,N", [
    (128, 16, 256),      # one tile, one pipeline stage
    (1, 16, 4),          # far inside one tile
    (129, 80, 260),      # ragged in M and N, K = 5 stages (wraps the 4-stage ring)
    (1000, 512, 8000),   # LM-head shape: N not a multiple of the 256-column tile
    (2048, 512, 2048),   # FFN up
    (2048, 2048, 512),   # FFN down
])
def test_tcgen05_path_matches_float64_and_the_mma_sync_path(ctx, M, K, N):
    rng = np.random.default_rng(M * 7 + K * 3 + N)
    a = rng.standard_normal((M, K), dtype=np.float32)
    b = rng.standard_normal((K, N), dtype=np.float32)
    ref = a.astype(np.float64) @ b.astype(np.float64)
    scale = np.abs(ref).max()
    big = _matmul(ctx, a, b, min_rows=1)          # tcgen05 path
    small = _matmul(ctx, a, b, min_rows=10 ** 8)  # mma.sync path
    assert np.isfinite(big).all() and np.isfinite(small).all()
    assert np.abs(big - ref).max() <= REL_TOL * scale
    assert np.abs(small - ref).max() <= REL_TOL * scale
    assert np.abs(big - small).max() <= 2e-6 * scale


def test_operand_layout_is_exact_on_integers(ctx):
    """Small integers are exact in TF32, so any mistake in the operand images or the accumulator read-back
    shows as a wrong integer: C[m, n] = sum_k (m + k) * (k == n mod K ? 1 : 0) style selector product."""
    M, K, N = 256, 64, 512
    a = (np.arange(M)[:, None] * 3 + np.arange(K)[None, :]).astype(np.float32)
    b = np.zeros((K, N), np.float32)
    b[np.arange(N) % K, np.arange(N)] = 1.0
    b[(np.arange(N) * 5 + 1) % K, np.arange(N)] += 2.0
    want = a.astype(np.float64) @ b.astype(np.float64)
    got = _matmul(ctx, a, b, min_rows=1)
    assert (got == want).all()


def test_unaligned_k_falls_back_to_the_small_kernel(ctx):
    rng = np.random.default_rng(5)
    a, b = rng.standard_normal((300, 20), dtype=np.float32), rng.standard_normal((20, 36), dtype=np.float32)
    got = _matmul(ctx, a, b, min_rows=1)  # K % 16 != 0
    ref = a.astype(np.float64) @ b.astype(np.float64)
    assert np.abs(got - ref).max() <= REL_TOL * np.abs(ref).max()


def test_matmul_argument_contract(ctx):
    d = ctx.alloc((16,))
    with pytest.raises(ValueError):  # IllegalArgumentException
        ctx.matmul(d, d, d, 0, 4, 4)
    d.close()


def test_forward_step_on_the_tcgen05_projections(ctx):
    """The whole forward step with every projection forced onto the tcgen05 kernel: logits and greedy tokens
    as with the default kernels and as the oracle's; weight images follow a weight update."""
    V, MS, D, H, L, F = 96, 80, 64, 4, 3, 128
    om = O.Model(V, MS, D, H, L, F, eps=1e-5).init_random(seed=4, std=0.15)
    gm_def = GPTModel(ctx, V, MS, D, H, L, F, rmsNormEps=1e-5)
    with _env(JGPT_B200_UMMA_MIN_ROWS=1):
        gm_big = GPTModel(ctx, V, MS, D, H, L, F, rmsNormEps=1e-5)
    gm_def.setParameters(om.tensors()), gm_big.setParameters(om.tensors())
    ids = np.array([(i * 5 + 1) % V for i in range(40)], np.int32)
    c1, c2 = (KvCacheGpu(L, H, om.dhead, MS, ctx=ctx) for _ in range(2))
    try:
        a, b = gm_def.forwardPrefill(ids, c1), gm_big.forwardPrefill(ids, c2)
        want = om.forward_prefill(ids, om.new_cache(kv_fp16=True))
        assert np.abs(a - b).max() < 5e-5
        assert np.abs(b - want).max() < 5e-4
        tok = int(np.argmax(b[-1]))
        for _ in range(8):
            da = gm_def.forwardDecode([tok], c1, c1.length(), c1.length())
            db = gm_big.forwardDecode([tok], c2, c2.length(), c2.length())
            assert np.abs(da - db).max() < 5e-5
            tok = int(np.argmax(db))
        # new weights: the cached weight images must be rebuilt
        om2 = O.Model(V, MS, D, H, L, F, eps=1e-5).init_random(seed=9, std=0.15)
        gm_big.setParameters(om2.tensors())
        c2.clear()
        b2 = gm_big.forwardPrefill(ids, c2)
        want2 = om2.forward_prefill(ids, om2.new_cache(kv_fp16=True))
        assert np.abs(b2 - want2).max() < 5e-4
        om2.close()
    finally:
        c1.close(), c2.close(), gm_def.close(), gm_big.close(), om.close()
