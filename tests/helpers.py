"""Shared builders for the GPU parity tests: a paged pool filled through the C ABI next to the
oracle's contiguous planes holding the same (fp16-rounded) payload."""
from __future__ import annotations

import numpy as np

import oracle as O
from jgpt_b200 import KvPool

BT = 16


class exact_prefill:
    """Models created inside use the exact prefill attention (fp16 high + low probabilities): what the toy geometries
    need to stay within their tight tolerances.  The default mode (single fp16 probabilities) is tested on its own."""

    def __enter__(self):
        import os

        self.old = os.environ.get("JGPT_B200_PREFILL_EXACT")
        os.environ["JGPT_B200_PREFILL_EXACT"] = "1"

    def __exit__(self, *a):
        import os

        if self.old is None:
            os.environ.pop("JGPT_B200_PREFILL_EXACT", None)
        else:
            os.environ["JGPT_B200_PREFILL_EXACT"] = self.old


class PagedCase:
    """n sequences of given lengths, K/V ~ N(0,1), block tables = a seeded permutation of the pool."""

    def __init__(self, ctx, lens, H=24, Dh=16, layers=1, seed=0, max_seq=None, extra_blocks=0, spare_tokens=1,
                 rope_pos_offset=0):
        self.ctx, self.H, self.Dh, self.layers = ctx, H, Dh, layers
        self.lens = np.asarray(lens, np.int32)
        n = self.n = len(lens)
        self.max_seq = max_seq or int(-(-(int(self.lens.max()) + spare_tokens) // BT) * BT)
        self.mbs = self.max_seq // BT
        need = [-(-(int(l) + spare_tokens) // BT) for l in lens]
        self.n_blocks = sum(need) + extra_blocks
        rng = np.random.default_rng(seed)
        self.pool = KvPool(ctx, layers, H, Dh, self.n_blocks, n, self.mbs, max_positions=self.max_seq + rope_pos_offset + 8)
        perm = rng.permutation(self.n_blocks).astype(np.int32)
        self.tables, off = [], 0
        self.seqs = []
        for i in range(n):
            s = self.pool.seq_alloc()
            self.seqs.append(s)
            self.pool.set_block_table(s, perm[off:off + need[i]])
            self.tables.append(perm[off:off + need[i]].copy())
            off += need[i]
        # contiguous oracle planes [layer][n, H, max_seq, Dh]
        self.kc = np.zeros((layers, n, H, self.max_seq, Dh), np.float32)
        self.vc = np.zeros((layers, n, H, self.max_seq, Dh), np.float32)
        self.rope_pos_offset = rope_pos_offset
        for layer in range(layers):
            tot = int(self.lens.sum())
            if tot == 0:
                continue
            k = rng.standard_normal((tot, H * Dh)).astype(np.float32)
            v = rng.standard_normal((tot, H * Dh)).astype(np.float32)
            seq_ids = np.concatenate([np.full(l, self.seqs[i], np.int32) for i, l in enumerate(self.lens)])
            slot = np.concatenate([np.arange(l, dtype=np.int32) for l in self.lens])
            rope = slot + rope_pos_offset
            self.pool.append(layer, ctx.from_host(k), ctx.from_host(v), ctx.from_host(seq_ids), ctx.from_host(slot),
                             ctx.from_host(rope), tot)
            off = 0
            for i, l in enumerate(self.lens):
                l = int(l)
                if l == 0:
                    continue
                kh = O.split_heads(k[off:off + l].reshape(1, l, H * Dh), H)  # [1,H,l,Dh]
                vh = O.split_heads(v[off:off + l].reshape(1, l, H * Dh), H)
                kr = O.rope_4d(kh, positions=np.arange(l, dtype=np.int32) + rope_pos_offset)
                self.kc[layer, i, :, :l] = O.round_fp16(kr[0])
                self.vc[layer, i, :, :l] = O.round_fp16(vh[0])
                off += l
        ctx.synchronize()

    def seq_ids_dev(self):
        return self.ctx.from_host(np.asarray(self.seqs, np.int32))

    def close(self):
        self.pool.close()


def oracle_decode(case, layer, q, lens, rope_pos):
    """Attention only (no append): run the oracle's append+attend on a copy with the cached last token as 'new'."""
    n, H, Dh = case.n, case.H, case.Dh
    out = np.zeros((n, H * Dh), np.float32)
    scale = 1.0 / np.sqrt(Dh)
    qh = O.split_heads(q.reshape(n, 1, H * Dh), H)  # [n,H,1,Dh]
    for i in range(n):
        L = int(lens[i])
        if L == 0:
            continue
        qr = O.rope_4d(qh[i:i + 1], positions=np.array([rope_pos[i]], np.int32))[0, :, 0]
        for h in range(H):
            out[i, h * Dh:(h + 1) * Dh] = O.attn_query_one(qr[h], case.kc[layer, i, h, :L], case.vc[layer, i, h, :L], scale)
    return out
