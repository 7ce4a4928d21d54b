"""The N > 1 path on CPU: two gloo ranks shard one decode layer by kv heads and by batch, each
computes its shard (the CPU oracle stands in for the GPU kernel here: this test is about the
partitioning and the gather), and the gathered result must equal the unsharded layer."""
import os
import socket
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _problem():
    rng = np.random.default_rng(31)
    B, hq, hkv, d, ps = 5, 16, 4, 128, 16
    lens = [40, 7, 129, 64, 300]
    pages = [(n + ps - 1) // ps for n in lens]
    perm = rng.permutation(sum(pages) + 2).astype(np.int32)
    bt = np.zeros((B, max(pages)), np.int32)
    off = 0
    for b, n in enumerate(pages):
        bt[b, :n] = perm[off:off + n]
        off += n
    K = [rng.standard_normal((n, hkv, d), dtype=np.float32).astype(np.float16) for n in lens]
    V = [rng.standard_normal((n, hkv, d), dtype=np.float32).astype(np.float16) for n in lens]
    q = rng.standard_normal((B, hq, d), dtype=np.float32).astype(np.float16)
    return B, hq, hkv, d, ps, lens, bt, K, V, q, len(perm)


def _decode(q, K, V, bt, lens, hq, hkv, d, ps, num_pages):
    """Oracle append + decode for the given (possibly sharded) heads / rows."""
    import oracle_lib as ol
    kc = np.zeros(num_pages * hkv * ps * d, np.uint16)
    vc = np.zeros_like(kc)
    for b in range(len(lens)):
        ol.append(0, np.ascontiguousarray(K[b]).view(np.uint16), np.ascontiguousarray(V[b]).view(np.uint16), kc, vc,
                  bt[b], 0, hkv, d, ps)
    return ol.paged_decode(1, 0, np.ascontiguousarray(q).view(np.uint16), kc, vc, bt, lens, hq, hkv, d, ps)


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    import torch
    import torch.distributed as dist
    from paged_attention_b200 import sharding
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        B, hq, hkv, d, ps, lens, bt, K, V, q, num_pages = _problem()
        full = _decode(q, K, V, bt, lens, hq, hkv, d, ps, num_pages)
        # --- kv-head sharding: replicated table and lengths, local pool holds Hkv/N heads
        sh = sharding.shard_heads(rank, world, hq, hkv)
        q_local = sharding.local_query(torch.from_numpy(q), sh).numpy()
        K_local = [sharding.local_kv(torch.from_numpy(k), sh).numpy() for k in K]
        V_local = [sharding.local_kv(torch.from_numpy(v), sh).numpy() for v in V]
        out_local = _decode(q_local, K_local, V_local, bt, lens, sh.num_q_heads, sh.num_kv_heads, d, ps, num_pages)
        got = sharding.gather_outputs(torch.from_numpy(out_local), "heads").numpy()
        assert got.shape == full.shape
        assert np.array_equal(got, full), "head-sharded result differs from the unsharded layer"
        # --- batch sharding with ragged shards (5 rows over 2 ranks: 3 + 2)
        begin, end = sharding.shard_batch(rank, world, B)
        rows = [e - b for b, e in (sharding.shard_batch(r, world, B) for r in range(world))]
        out_rows = _decode(q[begin:end], K[begin:end], V[begin:end], bt[begin:end], lens[begin:end], hq, hkv, d, ps, num_pages)
        got = sharding.gather_outputs(torch.from_numpy(out_rows), "batch", rows=rows).numpy()
        assert np.array_equal(got, full), "batch-sharded result differs from the unsharded layer"
        # --- timing is the max over ranks: the reduction bench.py uses
        t = torch.tensor([1.0 + rank], dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        assert t.item() == float(world)
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_shard_arithmetic():
    sys.path.insert(0, os.path.dirname(HERE))
    from paged_attention_b200 import sharding
    s = sharding.shard_heads(3, 4, 64, 8)
    assert (s.kv_begin, s.kv_end, s.q_begin, s.q_end, s.num_kv_heads, s.num_q_heads) == (6, 8, 48, 64, 2, 16)
    assert [sharding.shard_batch(r, 3, 8) for r in range(3)] == [(0, 3), (3, 6), (6, 8)]
    with pytest.raises(ValueError):
        sharding.shard_heads(0, 3, 32, 8)       # 8 kv heads do not divide over 3 ranks
    with pytest.raises(ValueError):
        sharding.shard_heads(0, 2, 30, 8)
    with pytest.raises(ValueError):
        sharding.shard_batch(2, 2, 8)


def test_two_gloo_ranks_shard_and_gather(tmp_path):
    import torch.multiprocessing as mp
    port = _free_port()
    mp.spawn(_worker, args=(2, port, str(tmp_path)), nprocs=2, join=True)
    assert os.path.exists(tmp_path / "ok0") and os.path.exists(tmp_path / "ok1")
