"""ctypes binding of ``libjgpt_b200.so``: the same symbols a JNI shim or a Java FFM downcall binds.

The argument lists are parsed from ``include/jgpt_b200.h`` so the binding cannot drift from the
header.  There is no fallback: if the shared library is missing the import fails loudly.
"""
from __future__ import annotations

import ctypes as C
import os
import re

_HERE = os.path.dirname(os.path.abspath(__file__))
HEADER = os.path.normpath(os.path.join(_HERE, "..", "include", "jgpt_b200.h"))
LIB_PATH = os.environ.get("JGPT_B200_LIB", os.path.join(_HERE, "lib", "libjgpt_b200.so"))

OK = 0
ERR_INVALID_ARGUMENT, ERR_ILLEGAL_STATE, ERR_OUT_OF_RANGE, ERR_OUT_OF_MEMORY = 1, 2, 3, 4
ERR_POOL_EXHAUSTED, ERR_BAD_HANDLE, ERR_CUDA, ERR_UNSUPPORTED, ERR_DEVICE_CHECK, ERR_IO = 5, 6, 7, 8, 9, 10
ERR_NCCL, ERR_TIMEOUT = 11, 12


class JgptError(RuntimeError):
    def __init__(self, code, msg):
        super().__init__(f"[{code}] {msg}")
        self.code = code


class PoolExhausted(JgptError):
    pass


def raise_for(code: int, msg: str):
    """Maps a status code to the Python counterpart of the exception the reference throws."""
    if code == ERR_INVALID_ARGUMENT:
        raise ValueError(msg)  # IllegalArgumentException
    if code == ERR_ILLEGAL_STATE:
        raise RuntimeError(msg)  # IllegalStateException
    if code == ERR_OUT_OF_RANGE:
        raise IndexError(msg)  # IndexOutOfBoundsException
    if code == ERR_OUT_OF_MEMORY:
        raise MemoryError(msg)  # OutOfMemoryError
    if code == ERR_POOL_EXHAUSTED:
        raise PoolExhausted(code, msg)
    if code == ERR_TIMEOUT:
        raise TimeoutError(msg)
    raise JgptError(code, msg)


_CTYPES = {
    "int32_t": C.c_int32, "uint64_t": C.c_uint64, "float": C.c_float, "jgpt_ctx": C.c_uint64,
    "jgpt_kvpool": C.c_uint64, "jgpt_model": C.c_uint64, "void": None, "char": C.c_char,
}


def _parse_type(t: str):
    t = t.replace("const", "").strip()
    stars = t.count("*")
    base = t.replace("*", "").strip()
    if stars == 0:
        return _CTYPES[base]
    if base == "char" and stars == 1:
        return C.c_char_p
    return C.c_void_p  # every pointer travels as an address


def declared_functions(header: str = HEADER):
    """[(name, restype, [argtypes])] for every JGPT_API declaration of the header."""
    src = open(header).read()
    src = re.sub(r"/\*.*?\*/", "", src, flags=re.S)
    out = []
    for m in re.finditer(r"JGPT_API\s+([\w\s\*]+?)\s*\b(jgpt_\w+)\s*\(([^)]*)\)\s*;", src):
        ret, name, args = m.group(1).strip(), m.group(2), m.group(3).strip()
        argtypes = []
        if args and args != "void":
            for a in args.split(","):
                a = a.strip()
                ty = re.sub(r"\b\w+$", "", a).strip() if not a.endswith("*") else a
                argtypes.append(_parse_type(ty))
        out.append((name, _parse_type(ret), argtypes))
    return out


_lib = None


def load():
    """Loads the shared library (once) and types every declared entry point."""
    global _lib
    if _lib is not None:
        return _lib
    if not os.path.exists(LIB_PATH):
        raise ImportError(
            f"{LIB_PATH} not found: build it with `python -m jgpt_b200.build` (needs nvcc). "
            "jgpt_b200 has no CPU or PyTorch fallback."
        )
    lib = C.CDLL(LIB_PATH)
    for name, res, args in declared_functions():
        fn = getattr(lib, name)  # AttributeError here = header/library drift
        fn.restype, fn.argtypes = res, args
    _lib = lib
    return lib


def check(code: int):
    if code != OK:
        raise_for(code, load().jgpt_last_error().decode("utf-8", "replace"))
