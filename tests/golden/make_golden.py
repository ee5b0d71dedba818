"""Generates tests/golden/oracle_vectors.npz from the CPU oracle (run from the repository root:
`python tests/golden/make_golden.py`).

The reference holds no golden vectors for this path and cannot be executed where this repository is built
(no JDK; its arithmetic is CUDA behind JNI), so these vectors are outputs of the C restatement in oracle/,
frozen so that (a) a change of the oracle shows up as a diff and (b) the GPU tests have fixed targets that
do not depend on rebuilding the oracle.  The literal cases of the reference's own tests are kept separately
in reference_known_answers.json.
"""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
sys.path.insert(0, ROOT)
import oracle as O  # noqa: E402


def build():
    out = {}
    # 1. KvCacheTest geometry: prefill + 3 decode steps (fp16-payload cache, what the paged store holds)
    m = O.Model(64, 32, 32, 4, 2, 64, eps=1e-6).init_random(seed=3, std=0.2)
    ids = np.array([(i * 7 + 3) % 64 for i in range(16)], np.int32)
    c = m.new_cache(kv_fp16=True)
    out["tiny_ids"] = ids
    out["tiny_prefill_logits"] = m.forward_prefill(ids, c)
    dec, tok = [], 11
    for step in range(3):
        lg = m.forward_decode(tok, c, c.length(), c.length())
        dec.append(lg)
        tok = int(O.argmax(lg))
    out["tiny_decode_logits"] = np.stack(dec)
    out["tiny_k_layer1"] = c.k(1)[:, :19].copy()
    # 2. GreedyGenerateParityTest geometry (sliding window): maxSeq 12, prompt 5, 12 new tokens
    g = O.Model(64, 12, 32, 4, 2, 64, eps=1e-6).init_random(seed=5, std=0.3)
    for name, (mult, add) in (("a", (7, 3)), ("b", (11, 2))):
        prompt = np.array([(i * mult + add) % 64 for i in range(5)], np.int32)
        stream, n = g.generate_greedy(prompt, 12, kv_fp16=True)
        out[f"greedy_{name}"] = stream
    # 3. single-query attention + append, one head group, ragged lengths
    rng = np.random.default_rng(11)
    H, Dh, MS = 2, 16, 48
    kc = O.round_fp16(rng.standard_normal((3, H, MS, Dh)).astype(np.float32))
    vc = O.round_fp16(rng.standard_normal((3, H, MS, Dh)).astype(np.float32))
    q, k, v = (rng.standard_normal((3, H * Dh)).astype(np.float32) for _ in range(3))
    lens, rope = np.array([0, 15, 33], np.int32), np.array([2, 15, 40], np.int32)
    out.update(attn_kc=kc.copy(), attn_vc=vc.copy(), attn_q=q, attn_k=k, attn_v=v, attn_lens=lens, attn_rope=rope)
    out["attn_out"] = O.decode_attn_batch(q, k, v, kc, vc, lens, rope, H, Dh, MS, kv_fp16=True)
    out["attn_kc_after"], out["attn_vc_after"] = kc, vc
    # 4. allocator specification trace
    a = O.PagedAllocatorRef(12, 16, 4, 6)
    trace = []
    s0, s1 = a.seq_alloc(), a.seq_alloc()
    a.reserve(s0, 40), a.reserve(s1, 16), a.reserve(s0, 49)
    trace += [a.tables[s0][:], a.tables[s1][:]]
    a.mark_evictable(s0), a.touch(s1), a.mark_evictable(s1)
    victims = a.evict_lru(10)
    s2 = a.seq_alloc()
    a.reserve(s2, 96)
    trace += [victims, a.tables[s2][:], a.free[:]]
    out["alloc_trace"] = np.array([x + [-1] * (8 - len(x)) for x in trace], np.int32)
    return out


if __name__ == "__main__":
    path = os.path.join(ROOT, "tests", "golden", "oracle_vectors.npz")
    np.savez_compressed(path, **build())
    print("wrote", path, os.path.getsize(path), "bytes")
