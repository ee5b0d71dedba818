"""The committed fixtures: (a) the literal known-answer cases of the reference's own op tests, (b) frozen
oracle outputs (tests/golden/oracle_vectors.npz, made by tests/golden/make_golden.py).  The oracle must
reproduce both on the CPU."""
import importlib.util
import json
import os

import numpy as np

import oracle as O

HERE = os.path.dirname(os.path.abspath(__file__))
GOLD = os.path.join(HERE, "golden")


def test_oracle_reproduces_the_reference_known_answers():
    ka = json.load(open(os.path.join(GOLD, "reference_known_answers.json")))
    c = ka["rmsnorm"]
    assert np.abs(O.rmsnorm(np.array(c["x"]), np.array(c["gamma"]), c["eps"]) - np.array(c["expected"])).max() < c["tol"]
    c = ka["matmul"]
    assert np.array_equal(O.matmul(np.array(c["a"], float), np.array(c["b"], float)), np.array(c["expected"], np.float32))
    c = ka["sigmoid"]
    assert np.abs(O.sigmoid(np.array(c["x"])) - np.array(c["expected"])).max() < c["tol"]
    c = ka["split_concat"]
    x = np.array(c["x"], np.float32).reshape(c["shape"])
    assert np.array_equal(O.concat_heads(O.split_heads(x, c["heads"])), x)
    c = ka["softmax_rows"]
    assert np.abs(O.softmax_last_dim(np.array(c["x"])).sum(-1) - c["row_sum"]).max() < c["tol"]


def test_oracle_reproduces_the_frozen_vectors_bit_for_bit():
    spec = importlib.util.spec_from_file_location("make_golden", os.path.join(GOLD, "make_golden.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    fresh = mod.build()
    gold = np.load(os.path.join(GOLD, "oracle_vectors.npz"))
    assert sorted(gold.files) == sorted(fresh)
    for name in gold.files:
        a, b = gold[name], np.asarray(fresh[name])
        if a.dtype.kind == "f":
            # same compiler flags, same libm -> identical; allow the last ulp of expf/cosf for another libm build
            assert np.allclose(a, b, rtol=2e-6, atol=2e-6), name
        else:
            assert np.array_equal(a, b), name
