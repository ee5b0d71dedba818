"""Pins the CPU oracle to the REFERENCE'S OWN CUDA kernels, run on the GPU on identical seeded inputs.

The reference ships no golden vectors for this path, and its Java side cannot run without a JDK; what
can run is its kernel file (src/main/cpp/jgpt_cuda_extra_kernels_launches.inl), compiled for sm_100a
behind ``oracle/ref_harness/ref_kernels.cu``.  Each test feeds the same arrays to a reference kernel
(or launch helper) and to the oracle's restatement of it, so a misreading in the oracle shows up here
rather than being inherited by every GPU-vs-oracle parity test.

Tolerances, per operation (the oracle is plain C on the host, the reference is device code compiled with
nvcc's defaults, i.e. fused multiply-add on and no fast-math):
  * pure data movement (cache write, split/concat heads) and the embedding sum: bit-exact;
  * RoPE: the device's powf/sinf/cosf are not bit-identical to the host libm.  CUDA documents powf at
    <= 4 ulp and sinf/cosf at <= 2 ulp over the full range; an ulp error in powf moves theta by the same
    relative amount, so |diff| <= (|x1|+|x2|) * (6 ulp(theta) + 4 ulp(1));
  * softmax / RMSNorm / sigmoid: expf <= 2 ulp and a different summation order: 2e-6 relative;
  * the reference's FlashAttention-2 forward uses __expf and __frcp_rn (documented error of __expf:
    2 + |1.16 x| ulp): 1e-4 absolute on outputs of magnitude ~1, 2e-5 on the log-sum-exp relative;
  * anything that goes through the reference's cuBLAS handle runs in TF32 tensor-op math mode (10-bit
    mantissas), as the reference sets it: 3e-3 absolute on uniform[-1,1) inputs, the tolerance the
    reference's own KvPrefillDecodeGpuResidentTest uses for the same reason.
"""
import numpy as np
import pytest

import oracle as O
from oracle import ref_kernels as R

pytestmark = pytest.mark.gpu

EPS32 = float(np.finfo(np.float32).eps)


@pytest.fixture(scope="module", autouse=True)
def _harness():
    if not R.available():
        if R.reference_present():
            R.build()
        else:
            pytest.skip("reference checkout absent and oracle/_ref not prebuilt: nothing to compare the oracle with")
    assert R.lib().ref_device_count() >= 1, "the reference harness sees no CUDA device"


def _rope_bound(x, positions, dhead):
    """Per-element bound of the RoPE comparison, see the module docstring."""
    j = np.arange(dhead // 2, dtype=np.float32)
    theta = positions[:, None].astype(np.float32) / np.power(np.float32(10000.0), 2.0 * j / dhead)  # [S, Dh/2]
    pair = np.abs(x[..., 0::2]) + np.abs(x[..., 1::2])  # [B,H,S,Dh/2]
    b = pair * (6.0 * theta * EPS32 + 4.0 * EPS32)
    return np.repeat(b, 2, axis=-1)


@pytest.mark.parametrize("S,base", [(1, 0), (1, 1023), (37, 2), (64, 960), (16, 8176)])
def test_rope_matches_rope_4d_kernel(S, base):  # jgpt_cuda_extra_kernels_launches.inl:1127-1159
    rng = np.random.default_rng(10 + S + base)
    x = rng.standard_normal((2, 24, S, 16)).astype(np.float32)
    want = R.rope_4d(x, pos_base_offset=base)
    got = O.rope_4d(x, pos_base_offset=base)
    pos = np.arange(S, dtype=np.int32) + base
    bound = _rope_bound(x, pos, 16)
    assert (np.abs(got - want) <= bound).all(), float(np.abs(got - want).max())
    # explicit positions (the decode call passes {ropePosition}); entries past posLen fall back to i + base
    p = np.array([base + 5], np.int32)
    want = R.rope_4d(x[:, :, :1], positions=p, pos_base_offset=0)
    got = O.rope_4d(x[:, :, :1], positions=p, pos_base_offset=0)
    assert (np.abs(got - want) <= _rope_bound(x[:, :, :1], p, 16)).all()


def test_rope_head_dims_other_than_16():
    rng = np.random.default_rng(3)
    for dh in (8, 32, 64):
        x = rng.standard_normal((1, 4, 9, dh)).astype(np.float32)
        want, got = R.rope_4d(x, pos_base_offset=100), O.rope_4d(x, pos_base_offset=100)
        assert (np.abs(got - want) <= _rope_bound(x, np.arange(9, dtype=np.int32) + 100, dh)).all()


def test_cache_write_matches_kv_heads4d_to_cache_kernel():  # :1085-1099, dst = h*maxSeq*Dh + pos*Dh + j
    rng = np.random.default_rng(4)
    H, Dh, max_seq = 24, 16, 48
    n = 1
    # prefill of 20 rows at position 0, then single-token decode writes at 20, 21
    kc = np.zeros((n, H, max_seq, Dh), np.float32)
    vc = np.zeros_like(kc)
    ref_k = np.zeros((H, max_seq, Dh), np.float32)
    ref_v = np.zeros_like(ref_k)
    for step, length in enumerate([0] + [20, 21]):
        S = 20 if step == 0 else 1
        k = rng.standard_normal((1, S, H * Dh)).astype(np.float32)
        v = rng.standard_normal((1, S, H * Dh)).astype(np.float32)
        kh, vh = R.split_heads(k, H), R.split_heads(v, H)
        kr = R.rope_4d(kh, pos_base_offset=length)
        ref_k = R.kv_heads4d_to_cache(kr[0], ref_k, max_seq, pos_offset=length)
        ref_v = R.kv_heads4d_to_cache(vh[0], ref_v, max_seq, pos_offset=length)
        # the oracle's append, one token at a time, through the decode entry point (fp32 cache)
        for s in range(S):
            q = np.zeros((n, H * Dh), np.float32)
            lens = np.array([length + s], np.int32)
            O.decode_attn_batch(q, k[:, s], v[:, s], kc, vc, lens, lens, H, Dh, max_seq, kv_fp16=False)
    assert np.array_equal(vc[0], ref_v), "V rows or their positions differ"
    pos = np.arange(max_seq, dtype=np.int32)
    # K went through RoPE on both sides: same bound as the RoPE test, on the rotated values' own magnitude
    # |x1|+|x2| <= sqrt(2) (|y1|+|y2|) for a rotation: widen by 1.5
    bound = 1.5 * _rope_bound(np.maximum(np.abs(kc[0]), np.abs(ref_k))[None], pos, Dh)[0] + 1e-30
    assert (np.abs(kc[0] - ref_k) <= bound).all()
    assert np.array_equal(kc[0][:, 22:], np.zeros((H, max_seq - 22, Dh), np.float32)) and not ref_k[:, 22:].any()


def test_split_concat_embed_are_bit_exact():  # :1063-1125, :937-955, :1020-1032
    rng = np.random.default_rng(5)
    x = rng.standard_normal((3, 7, 384)).astype(np.float32)
    assert np.array_equal(O.split_heads(x, 24), R.split_heads(x, 24))
    h = rng.standard_normal((3, 24, 7, 16)).astype(np.float32)
    assert np.array_equal(O.concat_heads(h), R.concat_heads(h))
    tok = rng.standard_normal((50, 32)).astype(np.float32)
    pos = rng.standard_normal((12, 32)).astype(np.float32)
    ids = rng.integers(0, 50, (1, 7))
    want = R.embed_pos(ids, tok, pos, pos_row_start=3)
    # x[b,s,:] = tok[id] + pos[posRowStart + s]: one fp32 add per element, so the statement itself is the check
    assert np.array_equal((tok[ids[0]] + pos[3:10])[None], want)
    # and through the oracle's forward pass: with identity-free weights the first thing it does is this sum;
    # an out-of-range id is rejected there where the kernel writes zeros
    m = O.Model(50, 12, 32, 4, 1, 64)
    try:
        with pytest.raises(Exception):
            m.forward(np.array([50], np.int32))
    finally:
        m.close()


@pytest.mark.parametrize("inner", [3, 17, 63, 64, 65, 200, 1025])
def test_softmax_matches_both_reference_branches(inner):  # thread-per-row < 64 <= block-per-row, :13-34, :176-201
    rng = np.random.default_rng(inner)
    x = (rng.standard_normal((29, inner)) * 3).astype(np.float32)
    want = R.softmax_last_dim(x)
    got = O.softmax_last_dim(x)
    assert np.abs(got - want).max() <= 2e-6 * max(1.0, float(want.max())), float(np.abs(got - want).max())
    assert np.allclose(want.sum(-1), 1.0, atol=1e-5)


@pytest.mark.parametrize("D", [2, 32, 63, 64, 384, 1000])
def test_rmsnorm_matches_both_reference_branches(D):  # :668-713
    rng = np.random.default_rng(D)
    x = rng.standard_normal((11, D)).astype(np.float32)
    g = rng.standard_normal(D).astype(np.float32)
    x[3] = 0.0  # rms = sqrt(eps): still finite
    want, got = R.rmsnorm(x, g, 1e-5), O.rmsnorm(x, g, 1e-5)
    assert np.abs(got - want).max() <= 2e-6 * float(np.abs(want).max() + 1.0)
    # the non-finite guard: a row with an inf gives inv = 0 on both sides (0 * inf = nan where the inf sits)
    x[5, 0] = np.inf
    want, got = R.rmsnorm(x, g, 1e-5), O.rmsnorm(x, g, 1e-5)
    assert np.array_equal(np.isnan(want), np.isnan(got))
    assert np.array_equal(np.nan_to_num(want[5]), np.nan_to_num(got[5]))


def test_sigmoid_and_swiglu_gate():  # :799-815 (clamp at +-20), :832
    x = np.concatenate([np.linspace(-30, 30, 1001), [20.0, -20.0, 19.999, -19.999]]).astype(np.float32)
    want, got = R.sigmoid(x), O.sigmoid(x)
    assert np.abs(got - want).max() <= 3e-7
    assert want[x >= 20].min() == 1.0 and want[x <= -20].max() == 0.0
    assert np.array_equal(want[np.abs(x) >= 20], got[np.abs(x) >= 20])


@pytest.mark.parametrize("S", [1, 5, 128, 129, 300])
def test_causal_attention_matches_flash_attn_fwd_kernel(S):  # :1916-2050, tile 128
    rng = np.random.default_rng(S)
    BH = 6
    q, k, v = (rng.standard_normal((BH, S, 16)).astype(np.float32) for _ in range(3))
    want, lse = R.flash_attn_fwd(q, k, v, 0.25)
    got = O.attn_prefill_causal(q, k, v, 0.25)
    assert np.abs(got - want).max() <= 1e-4, float(np.abs(got - want).max())
    # log-sum-exp of the scaled causal scores, float64 on the host
    z = np.einsum("bid,bjd->bij", q.astype(np.float64), k.astype(np.float64)) * 0.25
    z = np.where(np.tril(np.ones((S, S), bool)), z, -np.inf)
    m = z.max(-1)
    lse64 = m + np.log(np.exp(z - m[..., None]).sum(-1))
    assert np.abs(lse - lse64).max() <= 2e-5 * (1 + np.abs(lse64).max())


def test_masked_softmax_matches_fused_kernel_and_the_oracles_mask_orientation():  # :239-276
    rng = np.random.default_rng(8)
    S = 70
    scores = rng.standard_normal((4 * S, S)).astype(np.float32)
    mask = np.where(np.triu(np.ones((S, S), bool), 1), -np.inf, 0.0).astype(np.float32)  # createCausalMask: j > i
    want = R.softmax_scaled_masked(scores, mask, 0.25)
    z = scores.reshape(4, S, S) * np.float32(0.25) + mask
    got = np.stack([O.softmax_last_dim(z[b]) for b in range(4)]).reshape(4 * S, S)
    assert np.abs(got - want).max() <= 2e-6
    assert not want.reshape(4, S, S)[:, np.triu(np.ones((S, S), bool), 1)].any()


def test_prefill_attention_matches_attn_fwd_run_core_under_tf32():  # :1840-1870 (two cuBLAS products + fused softmax)
    rng = np.random.default_rng(9)
    B, S, d = 5, 64, 16
    q, k, v = (rng.uniform(-1, 1, (B, S, d)).astype(np.float32) for _ in range(3))
    mask = np.where(np.triu(np.ones((S, S), bool), 1), -np.inf, 0.0).astype(np.float32)
    want = R.attn_fwd_core(q, k, v, mask, 0.25)
    got = O.attn_prefill_causal(q, k, v, 0.25)
    assert np.abs(got - want).max() <= 3e-3, float(np.abs(got - want).max())


def test_single_query_attention_composed_the_way_the_reference_composes_it():
    """TensorOps.scaledDotProductAttentionQueryOne (ops/TensorOps.java:1088-1140): transpose K, q.K^T,
    multiply by the scale, softmax over the last dimension, .V -- built here from the reference's own
    matmul and softmax and compared with the oracle's single routine.  Lengths on both sides of the
    64-column softmax branch."""
    rng = np.random.default_rng(11)
    for L in (1, 5, 63, 64, 333, 1024):
        q = rng.uniform(-1, 1, (1, 16)).astype(np.float32)
        k = rng.uniform(-1, 1, (L, 16)).astype(np.float32)
        v = rng.uniform(-1, 1, (L, 16)).astype(np.float32)
        scores = R.matmul(q, np.ascontiguousarray(k.T))  # [1, L]
        probs = R.softmax_last_dim(R.mul(scores, np.full_like(scores, 0.25)))
        want = R.matmul(probs, v)[0]
        got = O.attn_query_one(q[0], k, v, 0.25)
        assert np.abs(got - want).max() <= 3e-3, (L, float(np.abs(got - want).max()))


def test_projection_convention_y_equals_x_times_w_row_major():  # jgpt_cuda_jni_init_matmul.inl:67, TF32 math mode
    rng = np.random.default_rng(12)
    a = rng.uniform(-1, 1, (7, 384)).astype(np.float32)
    w = rng.uniform(-1, 1, (384, 96)).astype(np.float32) * 0.05
    want, got = R.matmul(a, w), O.matmul(a, w)
    assert np.abs(got - want).max() <= 3e-3
