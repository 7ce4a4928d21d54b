"""Seeded inputs shared by the golden-vector generator and the tests that replay them."""
import hashlib

import numpy as np


def config1_inputs():
    """Config 1 of the benchmark spec: one Llama-3-8B attention layer decode step, 32 q / 8 kv heads,
    head_dim 128, batch 4, context lengths uniform in 256..1024, page size 16, page ids a random
    permutation of a 512-page pool, q/K/V fp32 ~ N(0,1).  Returns a dict of numpy arrays."""
    rng = np.random.default_rng(1)
    lens = rng.integers(256, 1025, 4).astype(np.int32)
    perm = rng.permutation(512).astype(np.int32)
    hq, hkv, d, ps = 32, 8, 128, 16
    pages = [(int(n) + ps - 1) // ps for n in lens]
    bt = np.zeros((4, max(pages)), np.int32)
    off = 0
    for b, n in enumerate(pages):
        bt[b, :n] = perm[off:off + n]
        off += n
    q = rng.standard_normal((4, hq, d)).astype(np.float32)
    K = [rng.standard_normal((int(n), hkv, d)).astype(np.float32) for n in lens]
    V = [rng.standard_normal((int(n), hkv, d)).astype(np.float32) for n in lens]
    h = hashlib.sha256()
    for a in [lens, bt, q] + K + V:
        h.update(np.ascontiguousarray(a).tobytes())
    return dict(seq_lens=lens, block_table=bt, q=q, K=K, V=V, hq=hq, hkv=hkv, d=d, ps=ps, sha256=h.hexdigest())
