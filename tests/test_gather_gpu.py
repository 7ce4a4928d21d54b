"""Gathered outputs by peer stores (pd_paged_decode_gather / pd_gather_wait).

One rank: the gathered buffer equals the ordinary decode's output (the flag protocol runs against
itself).  Two or more GPUs (skipped otherwise): one process per GPU, kv-head sharding and batch
sharding of one fixed layer; after decode_gather + wait every rank's buffer must hold the full
layer, equal to the CPU oracle over the unsharded inputs.  Ranks exchange IPC handles over a gloo
group; no collective touches the data."""
import os
import socket
import sys

import numpy as np
import pytest

HERE = os.path.dirname(os.path.abspath(__file__))
pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _view(torch, ptr, nbytes):
    from common import device_view
    return device_view(ptr, nbytes, torch)


def _layer(seed=5):
    rng = np.random.default_rng(seed)
    B, hq, hkv, d, ps = 6, 32, 8, 128, 16
    lens = [700, 33, 2049, 1, 1500, 64]
    K = [rng.standard_normal((n, hkv, d), dtype=np.float32).astype(np.float16) for n in lens]
    V = [rng.standard_normal((n, hkv, d), dtype=np.float32).astype(np.float16) for n in lens]
    q = rng.standard_normal((B, hq, d), dtype=np.float32).astype(np.float16)
    return B, hq, hkv, d, ps, lens, K, V, q


def _build(torch, pa, K, V, lens, hkv, ps, shuffle):
    pages = [(n + ps - 1) // ps for n in lens]
    cfg = pa.PagedKVCache.Config(num_pages=sum(pages) + 2, page_size=ps, num_kv_heads=hkv, head_dim=128,
                                 max_slots=len(lens), max_pages_per_slot=max(pages))
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(shuffle)
    for b, n in enumerate(lens):
        assert cache.admit() == b
        assert cache.append(b, torch.from_numpy(np.ascontiguousarray(K[b])).cuda(),
                            torch.from_numpy(np.ascontiguousarray(V[b])).cuda(), n)
    return cache, cfg


def _oracle_full():
    import oracle_lib as ol
    B, hq, hkv, d, ps, lens, K, V, q = _layer()
    pages = [(n + ps - 1) // ps for n in lens]
    bt = np.zeros((B, max(pages)), np.int32)
    off = 0
    for b, n in enumerate(pages):
        bt[b, :n] = np.arange(off, off + n)
        off += n
    kc = np.zeros(off * hkv * ps * d, np.uint16)
    vc = np.zeros_like(kc)
    for b in range(B):
        ol.append(0, K[b].view(np.uint16), V[b].view(np.uint16), kc, vc, bt[b], 0, hkv, d, ps)
    return ol.paged_decode(1, 0, q.view(np.uint16), kc, vc, bt, lens, hq, hkv, d, ps)


def _run_rank(rank, world, torch, pa, sharding, mode):
    """Decode this rank's shard with gathered output, three steps; returns the local gathered buffer."""
    B, hq, hkv, d, ps, lens, K, V, q = _layer()
    if mode == "heads":
        sh = sharding.shard_heads(rank, world, hq, hkv)
        Kl = [k[:, sh.kv_begin:sh.kv_end] for k in K]
        Vl = [v[:, sh.kv_begin:sh.kv_end] for v in V]
        ql, lens_l, l_hq, l_hkv = q[:, sh.q_begin:sh.q_end], lens, sh.num_q_heads, sh.num_kv_heads
        head_off, row_off = sh.q_begin, 0
    else:
        b0, b1 = sharding.shard_batch(rank, world, B)
        Kl, Vl, ql, lens_l, l_hq, l_hkv = K[b0:b1], V[b0:b1], q[b0:b1], lens[b0:b1], hq, hkv
        head_off, row_off = 0, b0
    cache, cfg = _build(torch, pa, Kl, Vl, lens_l, l_hkv, ps, shuffle=3 + rank)
    dq = torch.from_numpy(np.ascontiguousarray(ql)).cuda()
    plan = pa.make_plan(pa.KVDtype.FP16, lens_l, l_hq, l_hkv, d, 40)      # forces split rows: in-kernel merge
    dplan = pa.DevicePlan()
    dplan.upload(plan, l_hq // l_hkv, d)
    p = cache.params()
    p.q, p.out = dq.data_ptr(), None
    p.batch, p.num_q_heads = len(lens_l), l_hq
    dplan.bind(p)
    full_bytes = B * hq * d * 2
    gg = sharding.GatherGroup(full_bytes)
    got = None
    for step in range(6):                          # more steps than buffers in the rotation
        # alternately: announce only + separate wait kernel, and announce-and-wait in one kernel
        gg.decode(pa.KVDtype.FP16, p, hq, head_off, row_off, 0, cfg.num_pages, sync=bool(step & 1))
        if not step & 1:
            gg.wait(0)
        torch.cuda.synchronize()
        assert pa.kernel_status() == 0
        buf = _view(torch, gg.buffer_ptr(-1), full_bytes).view(torch.float16).view(B, hq, d)
        got = buf.float().cpu().numpy()
        if step == 0:
            first = got.copy()
        assert np.array_equal(got, first)          # every buffer, every step: the same bits
    return got, gg, cache


def test_gather_single_rank(torch_cuda, pa):
    from common import TOL
    from paged_attention_b200 import sharding
    got, gg, cache = _run_rank(0, 1, torch_cuda, pa, sharding, "heads")
    assert np.abs(got - _oracle_full()).max() < TOL
    gg.close()
    cache.close()


def test_wait_for_a_flag_nobody_sets_times_out_and_the_context_survives(torch_cuda, pa):
    """Failure detection without a fault: the bounded wait for a step that no rank ever signals gives up
    after about a second, the status word reports which peer was missing, and the next decode on the same
    context works."""
    import time
    from common import TOL
    from paged_attention_b200 import sharding
    torch = torch_cuda
    got, gg, cache = _run_rank(0, 1, torch, pa, sharding, "heads")
    t0 = time.time()
    gg.wait_epoch(gg.epoch + 1)            # nothing will ever raise the flag to this value
    with pytest.raises(pa.decode._lib.KernelTimeout, match="wait 5"):
        pa.kernel_status()
    assert 0.2 < time.time() - t0 < 10.0
    assert pa.kernel_status() == 0          # reading the status re-arms it
    got2, gg2, cache2 = _run_rank(0, 1, torch, pa, sharding, "batch")
    assert np.abs(got2 - _oracle_full()).max() < TOL
    for x in (gg, gg2, cache, cache2):
        x.close()


def _worker(rank, world, port, out_dir):
    sys.path.insert(0, HERE)
    sys.path.insert(0, os.path.dirname(HERE))
    os.environ["NCCL_NVLS_ENABLE"] = "0"
    import torch
    import torch.distributed as dist
    import paged_attention_b200 as pa
    from common import TOL
    from paged_attention_b200 import sharding
    torch.cuda.set_device(rank)
    os.environ["MASTER_ADDR"], os.environ["MASTER_PORT"] = "127.0.0.1", str(port)
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        want = _oracle_full()
        for mode in ("heads", "batch"):
            got, gg, cache = _run_rank(rank, world, torch, pa, sharding, mode)
            assert np.abs(got - want).max() < TOL, f"rank {rank} {mode}: gathered layer differs from the oracle"
            dist.barrier()          # nobody frees its block while a peer may still store into it
            gg.close()
            cache.close()
        open(os.path.join(out_dir, f"ok{rank}"), "w").close()
    finally:
        dist.destroy_process_group()


def test_gather_across_gpus(torch_cuda, pa, tmp_path):
    torch = torch_cuda
    world = min(torch.cuda.device_count(), 4)
    if world < 2:
        pytest.skip("needs at least two GPUs")
    if world == 3:
        world = 2
    import torch.multiprocessing as mp
    mp.spawn(_worker, args=(world, _free_port(), str(tmp_path)), nprocs=world, join=True)
    for r in range(world):
        assert os.path.exists(tmp_path / f"ok{r}")
