"""CPU-side checks: the C-ABI library loads and exports every symbol the header declares, entry points
fail loudly without a GPU (no fallback), the allocator specification behaves, the CPU arm of the benchmark
prints a well-formed line."""
import ctypes as C
import json
import os
import subprocess
import sys

import numpy as np
import pytest

import oracle as O

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_library_exports_every_declared_symbol():
    from jgpt_b200 import binding as B

    decl = B.declared_functions()
    names = [n for n, _, _ in decl]
    assert len(names) >= 40 and len(set(names)) == len(names)
    lib = C.CDLL(B.LIB_PATH)
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/jgpt_b200.h but not exported"
    # nothing else with the public prefix is exported behind the header's back
    out = subprocess.run(["nm", "-D", "--defined-only", B.LIB_PATH], capture_output=True, text=True).stdout
    exported = {l.split()[-1] for l in out.splitlines() if " T " in l and l.split()[-1].startswith("jgpt_")}
    assert exported == set(names), exported ^ set(names)


def test_no_gpu_means_loud_failure_not_fallback():
    """On a machine without a usable GPU creating a context raises (the reference's requireCuda throws
    IllegalStateException); with a GPU this test has nothing to check."""
    import jgpt_b200 as J
    from jgpt_b200 import binding as B

    n = C.c_int32()
    assert B.load().jgpt_device_count(C.byref(n)) == 0
    if n.value == 0:
        with pytest.raises(RuntimeError, match="no CPU fallback"):
            J.Context(0)


def test_bad_handles_and_arguments_are_rejected_without_a_gpu():
    from jgpt_b200 import binding as B

    lib = B.load()
    out = C.c_uint64()
    assert lib.jgpt_sync(12345) == B.ERR_BAD_HANDLE
    assert lib.jgpt_kvpool_create(12345, 1, 1, 16, 16, 1, 1, 1, 16, 10000.0, C.byref(out)) == B.ERR_BAD_HANDLE
    assert lib.jgpt_seq_alloc(999, C.byref(C.c_int32())) == B.ERR_BAD_HANDLE
    assert b"handle" in lib.jgpt_last_error()
    assert lib.jgpt_ctx_create(0, None) == B.ERR_INVALID_ARGUMENT


def test_product_package_never_touches_the_oracle():
    """The shipped package must not import, load or link the oracle (or any CPU fallback)."""
    pkg = os.path.join(ROOT, "jgpt_b200")
    for dirpath, _, files in os.walk(pkg):
        for f in files:
            if f.endswith((".py", ".cu", ".cuh", ".cpp", ".h")):
                text = open(os.path.join(dirpath, f)).read()
                assert "oracle" not in text.lower(), f"{f} mentions the oracle"
    from jgpt_b200 import binding as B

    ldd = subprocess.run(["ldd", B.LIB_PATH], capture_output=True, text=True).stdout
    assert "oracle" not in ldd and "torch" not in ldd


def test_allocator_specification_basics():
    a = O.PagedAllocatorRef(n_blocks=6, block_tokens=16, max_seqs=3, max_blocks_per_seq=4)
    s0, s1 = a.seq_alloc(), a.seq_alloc()
    assert (s0, s1) == (0, 1)
    assert a.reserve(s0, 17) and a.tables[s0] == [0, 1]
    assert a.reserve(s1, 1) and a.tables[s1] == [2]
    assert a.reserve(s0, 20) and a.tables[s0] == [0, 1]  # already covered
    assert not a.reserve(s1, 16 * 5)  # per-sequence limit
    assert not a.reserve(s1, 16 * 4 + 1)
    assert a.reserve(s1, 64) and a.tables[s1] == [2, 3, 4, 5]
    assert not a.reserve(s0, 33)  # pool exhausted, all or nothing
    assert a.tables[s0] == [0, 1]
    a.seq_free(s1)
    assert a.free == [2, 3, 4, 5]
    assert a.reserve(s0, 48) and a.tables[s0] == [0, 1, 5]  # most recently freed block first
    assert a.append_index(s0, 37) == (5, 5)
    assert a.seq_alloc() == 1


def test_reference_arm_prints_the_contract_line():
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--steps", "1", "--warmup", "1"],
                       capture_output=True, text=True, timeout=120)
    assert r.returncode == 0, r.stderr
    line = json.loads(r.stdout.strip().splitlines()[-1])
    assert line["impl"] == "reference" and line["unit"] == "tokens/s" and line["value"] > 0
    assert line["cpu_baseline"]["kind"] == "port" and line["cpu_baseline"]["cores"] >= 1
    assert line["e2e"]["h2d_bytes_per_step"] == 0 and line["config"]["workload"].startswith("kv_append")
    # a non-zero rank exits 0 without output
    env = dict(os.environ, RANK="1", WORLD_SIZE="2", LOCAL_RANK="1")
    r = subprocess.run([sys.executable, os.path.join(ROOT, "bench.py"), "--impl", "reference", "--gpus", "2", "--steps", "1"],
                       capture_output=True, text=True, timeout=60, env=env)
    assert r.returncode == 0 and r.stdout.strip() == ""


def test_algorithmic_bytes_figure():
    sys.path.insert(0, ROOT)
    import bench

    assert bench.ALG_BYTES_LAYER == 100_876_288 and bench.ALG_BYTES_STEP == 1_210_515_456


def test_java_ffm_bindings_cover_every_declared_symbol_with_matching_arity():
    """java/.../JgptB200.java is what a Java host binds (no JDK here to compile it): it must name every entry point
    the header declares, with one layout per C argument plus the return value."""
    import re

    from jgpt_b200 import binding

    src = open(os.path.join(ROOT, "java", "com", "veles", "llm", "jgpt", "b200", "JgptB200.java")).read()
    bound = {m.group(1): m.group(2) for m in re.finditer(r'bind\("(jgpt_\w+)", FunctionDescriptor\.of\(([^)]*)\)\)', src)}
    for name, _res, args in binding.declared_functions():
        assert name in bound, f"{name} has no FFM handle"
        assert len([x for x in bound[name].split(",") if x.strip()]) == 1 + len(args), name
    assert len(bound) == len(binding.declared_functions())


def test_env_config_follows_the_reference_parsing_rules(monkeypatch):
    """jgpt_env_config needs no GPU: JGPT_RMSNORM_EPS in (0, 1e-2] else the default (1e-5 with JGPT_FP16_MATMUL, 1e-6
    without: TensorOpsGpuInit.resolveRmsNormEps), JGPT_MAX_SEQ_LEN positive or ignored, this library's own keys."""
    from jgpt_b200 import binding

    lib = binding.load()

    def read():
        bt, pb, ms, be = C.c_int32(), C.c_int32(), C.c_int32(), C.c_int32()
        eps = C.c_float()
        assert lib.jgpt_env_config(C.byref(bt), C.byref(pb), C.byref(ms), C.byref(eps), C.byref(be)) == 0
        return bt.value, pb.value, ms.value, eps.value, be.value

    for k in ("JGPT_KV_BLOCK_TOKENS", "JGPT_KV_POOL_BLOCKS", "JGPT_MAX_SEQ_LEN", "JGPT_RMSNORM_EPS", "JGPT_FP16_MATMUL", "JGPT_KV_BACKEND"):
        monkeypatch.delenv(k, raising=False)
    assert read() == (16, 0, 0, np.float32(1e-6), 1)
    monkeypatch.setenv("JGPT_FP16_MATMUL", "TRUE")
    assert read()[3] == np.float32(1e-5)
    monkeypatch.setenv("JGPT_RMSNORM_EPS", " 3e-4 ")
    assert read()[3] == np.float32(3e-4)
    for bad in ("0", "-1e-5", "0.5", "nan", "inf", "abc", ""):
        monkeypatch.setenv("JGPT_RMSNORM_EPS", bad)
        assert read()[3] == np.float32(1e-5), bad
    monkeypatch.setenv("JGPT_MAX_SEQ_LEN", "512")
    monkeypatch.setenv("JGPT_KV_POOL_BLOCKS", "4096")
    monkeypatch.setenv("JGPT_KV_BACKEND", "Reference")
    assert read()[:3] == (16, 4096, 512) and read()[4] == 0
    monkeypatch.setenv("JGPT_MAX_SEQ_LEN", "-7")
    monkeypatch.setenv("JGPT_KV_BACKEND", "b200")
    assert read()[2] == 0 and read()[4] == 1
    assert lib.jgpt_env_config(None, None, None, None, None) == 0
