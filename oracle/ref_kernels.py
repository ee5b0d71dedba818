"""ctypes front end of ``_ref/libjgpt_ref_kernels.so``: the reference's own CUDA kernels behind the
small harness ``ref_harness/ref_kernels.cu``.

Test infrastructure only.  It exists so that a GPU test can check the CPU oracle against what the
reference's kernels compute on the same inputs; nothing in the shipped package loads it.  The
library is built (``make -C oracle ref``) where the reference checkout is present and travels as a
prebuilt file otherwise.  Every function takes and returns host numpy arrays.
"""
from __future__ import annotations

import ctypes as C
import os
import subprocess

import numpy as np

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "_ref", "libjgpt_ref_kernels.so")
REFERENCE_DIR = os.environ.get("JGPT_REFERENCE_DIR", "/root/reference")
_KERNEL_FILE = os.path.join(REFERENCE_DIR, "src", "main", "cpp", "jgpt_cuda_extra_kernels_launches.inl")

_f32p = np.ctypeslib.ndpointer(dtype=np.float32, flags="C_CONTIGUOUS")
_lib = None


def reference_present() -> bool:
    return os.path.exists(_KERNEL_FILE)


def build(force: bool = False) -> str | None:
    """Compile the harness if the reference checkout is there; returns the library path or None."""
    if not reference_present():
        return LIB_PATH if os.path.exists(LIB_PATH) else None
    args = ["make", "-C", _HERE, f"REF={REFERENCE_DIR}", "ref"]
    if force:
        args.insert(1, "-B")
    subprocess.run(args, check=True, capture_output=True)
    return LIB_PATH


def available() -> bool:
    return os.path.exists(LIB_PATH)


def lib():
    global _lib
    if _lib is None:
        L = C.CDLL(LIB_PATH)
        ci, cf, vp, ll = C.c_int, C.c_float, C.c_void_p, C.c_longlong
        sig = {
            "ref_device_count": [],
            "ref_rope_4d": [_f32p, _f32p, ci, ci, ci, ci, vp, ci, ci],
            "ref_kv_heads4d_to_cache": [_f32p, _f32p, ci, ci, ci, ci, ci],
            "ref_softmax_last_dim": [_f32p, _f32p, ll, ci, ci],
            "ref_softmax_scaled_masked": [_f32p, _f32p, vp, cf, ll, ci],
            "ref_rms_norm": [_f32p, _f32p, _f32p, ci, ci, cf],
            "ref_sigmoid": [_f32p, _f32p, ci],
            "ref_mul": [_f32p, _f32p, _f32p, ci],
            "ref_embed_pos": [_f32p, _f32p, _f32p, _f32p, ci, ci, ci, ci, ci, ci],
            "ref_split_heads": [_f32p, _f32p, ci, ci, ci, ci],
            "ref_concat_heads": [_f32p, _f32p, ci, ci, ci, ci],
            "ref_flash_attn_fwd": [_f32p, _f32p, _f32p, _f32p, _f32p, ci, ci, cf],
            "ref_attn_fwd_core": [_f32p, _f32p, _f32p, vp, _f32p, vp, ci, ci, ci, ci, cf],
            "ref_matmul_row_major": [_f32p, _f32p, _f32p, ci, ci, ci, ci],
        }
        for name, args in sig.items():
            fn = getattr(L, name)
            fn.restype, fn.argtypes = ci, args
        _lib = L
    return _lib


def _f32(a):
    return np.ascontiguousarray(a, dtype=np.float32)


def _ok(rc, what):
    if rc != 0:
        raise RuntimeError(f"reference harness: {what} returned {rc}")


def rope_4d(x, positions=None, pos_base_offset=0):
    x = _f32(x)
    B, H, S, Dh = x.shape
    out = np.empty_like(x)
    if positions is None:
        rc = lib().ref_rope_4d(x, out, B, H, S, Dh, None, 0, pos_base_offset)
    else:
        p = np.ascontiguousarray(positions, np.int32)
        rc = lib().ref_rope_4d(x, out, B, H, S, Dh, p.ctypes.data, p.size, pos_base_offset)
    _ok(rc, "rope_4d")
    return out


def kv_heads4d_to_cache(src, cache, max_seq, pos_offset=0):
    """src [H, S, Dh] written into cache [H, max_seq, Dh] (returned copy) at rows pos_offset.."""
    src, cache = _f32(src), _f32(cache).copy()
    H, S, Dh = src.shape
    _ok(lib().ref_kv_heads4d_to_cache(src, cache, H, S, max_seq, Dh, pos_offset), "kv_heads4d_to_cache")
    return cache


def softmax_last_dim(x, fp16_branch=False):
    x = _f32(x)
    out = np.empty_like(x)
    _ok(lib().ref_softmax_last_dim(x, out, x.size // x.shape[-1], x.shape[-1], int(fp16_branch)), "softmax_last_dim")
    return out


def softmax_scaled_masked(scores, mask, scale):
    scores = _f32(scores)
    out = np.empty_like(scores)
    inner = scores.shape[-1]
    m = None if mask is None else _f32(mask)
    rc = lib().ref_softmax_scaled_masked(scores, out, None if m is None else m.ctypes.data, scale, scores.size // inner, inner)
    _ok(rc, "softmax_scaled_masked")
    return out


def rmsnorm(x, gamma, eps):
    x = _f32(x)
    out = np.empty_like(x)
    D = x.shape[-1]
    _ok(lib().ref_rms_norm(x, _f32(gamma), out, x.size // D, D, eps), "rms_norm")
    return out


def sigmoid(x):
    x = _f32(x)
    out = np.empty_like(x)
    _ok(lib().ref_sigmoid(x, out, x.size), "sigmoid")
    return out


def mul(a, b):
    a, b = _f32(a), _f32(b)
    out = np.empty_like(a)
    _ok(lib().ref_mul(a, b, out, a.size), "mul")
    return out


def embed_pos(ids, tok, pos, pos_row_start):
    """ids [B, S] (carried as floats, as the reference does); returns tok[id] + pos[pos_row_start + s]."""
    idf = _f32(ids)
    B, S = idf.shape
    tok, pos = _f32(tok), _f32(pos)
    out = np.empty((B, S, tok.shape[1]), np.float32)
    _ok(lib().ref_embed_pos(idf, tok, pos, out, B, S, tok.shape[1], tok.shape[0], pos.shape[0], pos_row_start), "embed_pos")
    return out


def split_heads(x, H):
    x = _f32(x)
    B, S, D = x.shape
    out = np.empty((B, H, S, D // H), np.float32)
    _ok(lib().ref_split_heads(x, out, B, S, D, H), "split_heads")
    return out


def concat_heads(x):
    x = _f32(x)
    B, H, S, Dh = x.shape
    out = np.empty((B, S, H * Dh), np.float32)
    _ok(lib().ref_concat_heads(x, out, B, H, S, Dh), "concat_heads")
    return out


def flash_attn_fwd(q, k, v, scale):
    """q, k, v [BH, S, 16]; returns (o [BH, S, 16], lse [BH, S])."""
    q, k, v = _f32(q), _f32(k), _f32(v)
    BH, S, Dh = q.shape
    assert Dh == 16
    o, lse = np.empty_like(q), np.empty((BH, S), np.float32)
    _ok(lib().ref_flash_attn_fwd(q, k, v, o, lse, BH, S, scale), "flash_attn_fwd")
    return o, lse


def attn_fwd_core(q, k, v, mask, scale):
    q, k, v = _f32(q), _f32(k), _f32(v)
    B, S, dk = q.shape
    dv = v.shape[2]
    out = np.empty((B, S, dv), np.float32)
    m = None if mask is None else _f32(mask)
    rc = lib().ref_attn_fwd_core(q, k, v, None if m is None else m.ctypes.data, out, None, B, S, dk, dv, scale)
    _ok(rc, "attn_fwd_core")
    return out


def matmul(a, b):
    a, b = _f32(a), _f32(b)
    if a.ndim == 2:
        a, b = a[None], b[None]
    Bt, M, K = a.shape
    N = b.shape[2]
    c = np.empty((Bt, M, N), np.float32)
    _ok(lib().ref_matmul_row_major(a, b, c, Bt, M, K, N), "matmul_row_major")
    return c if Bt > 1 else c[0]
