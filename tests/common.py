"""Shared helpers of the GPU parity tests: the reference's decode-test driver
(tests/test_paged_decode.cu:50-151 of the reference) restated over the C ABI,
with the oracle as the checker."""
import os
import sys

import numpy as np

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
if ROOT not in sys.path:
    sys.path.insert(0, ROOT)

import oracle_lib as ol  # noqa: E402

# Stated tolerance of the path: outputs within 2e-3 max-abs of the reference.
TOL = 2e-3


def seeded_kv(seq_lens, hkv, d, seed=1234):
    """Per-sequence K/V and q as fp16 values N(0,1): K[b], V[b] are [len][hkv][d]."""
    rng = np.random.default_rng(seed)
    K = [rng.standard_normal((n, hkv, d), dtype=np.float32).astype(np.float16) for n in seq_lens]
    V = [rng.standard_normal((n, hkv, d), dtype=np.float32).astype(np.float16) for n in seq_lens]
    return K, V


class Case:
    def __init__(self, dtype, hq, hkv, page_size, seq_lens, num_ctas=0, chunk=0, d=128, seed=1234, shuffle=None,
                 extra_pages=3, scale=None):
        self.dtype, self.hq, self.hkv, self.ps, self.seq_lens = dtype, hq, hkv, page_size, list(seq_lens)
        self.num_ctas, self.chunk, self.d, self.seed, self.shuffle = num_ctas, chunk, d, seed, shuffle
        self.extra_pages = extra_pages
        # |x| <= 4 fits: the reference's test scale (tests/test_paged_decode.cu:79)
        self.scale = scale if scale is not None else (4.0 / 448.0 if dtype == 1 else 1.0)


def build_cache(case, K, V, torch, pa):
    """Create an engine cache, append the sequences (whole or in round-robin chunks) and
    return (cache, model) where model is the oracle's allocator driven in lock step."""
    B = len(case.seq_lens)
    pages = [(n + case.ps - 1) // case.ps for n in case.seq_lens]
    cfg = pa.PagedKVCache.Config(num_pages=sum(pages) + case.extra_pages, page_size=case.ps, num_kv_heads=case.hkv,
                                 head_dim=case.d, max_slots=B, max_pages_per_slot=max(pages),
                                 dtype=pa.KVDtype(case.dtype), k_scale=case.scale, v_scale=case.scale)
    cache = pa.PagedKVCache(cfg)
    model = ol.PoolModel(cfg.num_pages, case.ps, B, max(pages))
    if case.shuffle is not None:
        cache.shuffle_free_pages(case.shuffle)
        model.shuffle(case.shuffle)
    dK = [torch.from_numpy(k.view(np.int16)).cuda().view(torch.float16) for k in K]
    dV = [torch.from_numpy(v.view(np.int16)).cuda().view(torch.float16) for v in V]
    for b in range(B):
        assert cache.admit() == b
        assert model.admit() == b
    done = [0] * B
    progress = True
    while progress:
        progress = False
        for b in range(B):
            n = min(case.chunk if case.chunk > 0 else case.seq_lens[b], case.seq_lens[b] - done[b])
            if n <= 0:
                continue
            assert cache.append(b, dK[b][done[b]:], dV[b][done[b]:], n)
            assert model.append(b, n)
            done[b] += n
            progress = True
    return cache, model, cfg


class _DeviceBytes:
    """Zero-copy view of raw device memory for torch.as_tensor."""

    def __init__(self, ptr, nbytes):
        self.__cuda_array_interface__ = {"shape": (nbytes,), "typestr": "|u1", "data": (int(ptr), False), "version": 2}


def device_view(ptr, nbytes, torch):
    return torch.as_tensor(_DeviceBytes(ptr, nbytes), device="cuda")


def cache_bytes(cache, cfg, torch):
    """Device pools copied back as numpy arrays (uint16 for fp16, uint8 for fp8)."""
    p = cache.params()
    elems = cfg.num_pages * cfg.num_kv_heads * cfg.page_size * cfg.head_dim
    np_dt = np.uint16 if int(cfg.dtype) == 0 else np.uint8
    nbytes = elems * np.dtype(np_dt).itemsize
    return [device_view(ptr, nbytes, torch).cpu().numpy().view(np_dt) for ptr in (p.k_cache, p.v_cache)]


def oracle_cache(case, cfg, K, V, model):
    """The oracle's cache bytes for the same appends (tables from the allocator model)."""
    np_dt = np.uint16 if case.dtype == 0 else np.uint8
    elems = cfg.num_pages * cfg.num_kv_heads * cfg.page_size * cfg.head_dim
    kc, vc = np.zeros(elems, np_dt), np.zeros(elems, np_dt)
    for b, n in enumerate(case.seq_lens):
        ol.append(case.dtype, K[b].view(np.uint16), V[b].view(np.uint16), kc, vc, model.table(b), 0, case.hkv, case.d,
                  case.ps, case.scale, case.scale)
    return kc, vc


def block_table_matrix(model, B, max_pages):
    bt = np.zeros((B, max_pages), np.int32)
    for b in range(B):
        t = model.table(b)
        bt[b, :len(t)] = t
    return bt


def run_case(case, torch, pa, check_bytes=True, precision=1):
    """Runs one case through the engine and returns (max abs error vs the oracle, output).
    Also asserts the allocator decisions and (optionally) the cache bytes bit-exactly."""
    B = len(case.seq_lens)
    K, V = seeded_kv(case.seq_lens, case.hkv, case.d, case.seed)
    rng = np.random.default_rng(case.seed + 1)
    q = rng.standard_normal((B, case.hq, case.d), dtype=np.float32).astype(np.float16)
    cache, model, cfg = build_cache(case, K, V, torch, pa)
    for b in range(B):
        assert (cache.block_table(b) == model.table(b)).all(), "block table differs from the allocator model"
        assert cache.seq_len(b) == model.seq_len(b)
    assert cache.free_pages() == model.free_pages()
    kc, vc = oracle_cache(case, cfg, K, V, model)
    if check_bytes:
        gk, gv = cache_bytes(cache, cfg, torch)
        assert (gk == kc).all() and (gv == vc).all(), "cache bytes differ from the oracle append"
    dq = torch.from_numpy(q.view(np.int16)).cuda().view(torch.float16)
    dout = torch.zeros_like(dq)
    cache.decode(dq, dout, B, case.hq, case.num_ctas)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    out = dout.cpu().numpy().astype(np.float32)
    assert np.isfinite(out).all()
    bt = block_table_matrix(model, B, cfg.max_pages_per_slot)
    want = ol.paged_decode(precision, case.dtype, q.view(np.uint16), kc, vc, bt, case.seq_lens, case.hq, case.hkv,
                           case.d, case.ps, k_scale=case.scale, v_scale=case.scale, threads=0)
    err = float(np.abs(out - want).max())
    plan = cache.last_plan()
    info = dict(num_ctas=plan.num_ctas, segments=plan.num_segments)
    cache.close()
    return err, out, want, info


def raw_decode(torch, pa, dtype, dq, k_cache, v_cache, block_table, seq_lens, hq, hkv, ps, k_scale=1.0, v_scale=1.0,
               num_ctas=0, slot_ids=None, num_pages=0, d=128):
    """Drives the kernel directly on caller-owned buffers, as the reference's torch binding does
    (bindings/torch_decode.cu:21-59): plan from host lengths, upload, fill DecodeParams by hand, decode.
    k_cache / v_cache / dq are torch CUDA tensors; block_table a numpy int32 matrix. Returns the output tensor."""
    B = dq.shape[0]
    lens = np.ascontiguousarray(seq_lens, np.int32)
    rows = lens if slot_ids is None else lens[np.asarray(slot_ids)]
    plan = pa.make_plan(pa.KVDtype(dtype), rows, hq, hkv, d, num_ctas)
    dp = pa.DevicePlan()
    dp.upload(plan, hq // hkv, d)
    d_bt = torch.from_numpy(np.ascontiguousarray(block_table, np.int32)).cuda()
    d_lens = torch.from_numpy(lens).cuda()
    d_slots = torch.from_numpy(np.ascontiguousarray(slot_ids, np.int32)).cuda() if slot_ids is not None else None
    out = torch.zeros_like(dq)
    p = pa.DecodeParams()
    p.q, p.out = dq.data_ptr(), out.data_ptr()
    p.k_cache, p.v_cache = k_cache.data_ptr(), v_cache.data_ptr()
    p.block_table, p.seq_lens = d_bt.data_ptr(), d_lens.data_ptr()
    p.slot_ids = d_slots.data_ptr() if d_slots is not None else None
    p.block_table_stride = d_bt.shape[1]
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.page_size = B, hq, hkv, d, ps
    p.sm_scale = 1.0 / float(np.sqrt(np.float32(d)))
    p.k_scale, p.v_scale = k_scale, v_scale
    dp.bind(p)
    pa.paged_decode(pa.KVDtype(dtype), p, 0, num_pages)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    return out, plan
