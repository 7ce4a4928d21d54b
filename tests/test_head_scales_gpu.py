"""One fp8 scale per kv head (pd_append_tokens_scaled, pd_paged_decode_scaled, pd_cache_set_head_scales).

The reference quantises with one scale per tensor (src/decode/paged_kv_cache.cu:20-21, DecodeParams
k_scale / v_scale); its README notes per-head scales as the next accuracy step.  The oracle is used
unchanged: a layer with per-head scales is num_kv_heads independent single-kv-head layers, each with its
own per-tensor scale, so the oracle runs head by head on slices of the same tensors.

Checked: cache bytes bit-exact against the oracle's append per head; outputs within the path's tolerance
of the oracle's decode per head; equal scales reproduce the per-tensor path bit for bit; the cache object
applies the scales in append, batched append and run, and refuses to change them once it holds tokens;
and on heads of very different magnitude per-head scales are more accurate than one scale per tensor.
"""
import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, cache_bytes, device_view

pytestmark = pytest.mark.gpu

FP16, FP8 = 0, 1
HQ, HKV, D, PS = 32, 8, 128, 16
G = HQ // HKV


def _layer(torch, lens, head_gain, seed=0):
    """K/V whose kv head h is N(0,1) * head_gain[h]; a scattered block table; q."""
    rng = np.random.default_rng(seed)
    gain = np.asarray(head_gain, np.float32)[None, :, None]
    K = [(rng.standard_normal((n, HKV, D), dtype=np.float32) * gain).astype(np.float16) for n in lens]
    V = [(rng.standard_normal((n, HKV, D), dtype=np.float32) * gain).astype(np.float16) for n in lens]
    q = rng.standard_normal((len(lens), HQ, D), dtype=np.float32).astype(np.float16)
    pages = [(n + PS - 1) // PS for n in lens]
    num_pages = sum(pages) + 1
    perm = rng.permutation(num_pages).astype(np.int32)
    bt = np.zeros((len(lens), max(pages)), np.int32)
    at = 0
    for b, n in enumerate(pages):
        bt[b, :n] = perm[at:at + n]
        at += n
    return K, V, q, bt, num_pages


def _engine_append(torch, pa, dtype, K, V, bt, num_pages, scale, k_scales=None, v_scales=None):
    elem = torch.float16 if dtype == FP16 else torch.uint8
    kc = torch.zeros(num_pages * HKV * PS * D, dtype=elem, device="cuda")
    vc = torch.zeros_like(kc)
    d_bt = torch.from_numpy(bt).cuda()
    dks = torch.tensor(k_scales, dtype=torch.float32, device="cuda") if k_scales is not None else None
    dvs = torch.tensor(v_scales, dtype=torch.float32, device="cuda") if v_scales is not None else None
    for b in range(len(K)):
        dk = torch.from_numpy(K[b].view(np.int16)).cuda()
        dv = torch.from_numpy(V[b].view(np.int16)).cuda()
        pa.append_tokens(dtype, dk, dv, kc, vc, d_bt[b], 0, K[b].shape[0], HKV, D, PS, scale, scale,
                         d_k_scales=dks, d_v_scales=dvs)
    torch.cuda.synchronize()
    return kc, vc, d_bt, dks, dvs


def _oracle_per_head(dtype, K, V, q, bt, num_pages, lens, k_scales, v_scales):
    """The oracle's cache bytes and outputs, one kv head at a time with that head's scale."""
    np_dt = np.uint16 if dtype == FP16 else np.uint8
    kc_all = np.zeros((num_pages, HKV, PS, D), np_dt)
    vc_all = np.zeros_like(kc_all)
    out = np.zeros((len(lens), HQ, D), np.float32)
    for h in range(HKV):
        kc = np.zeros(num_pages * PS * D, np_dt)
        vc = np.zeros_like(kc)
        for b in range(len(lens)):
            ol.append(dtype, K[b][:, h:h + 1].copy().view(np.uint16), V[b][:, h:h + 1].copy().view(np.uint16), kc, vc, bt[b],
                      0, 1, D, PS, float(k_scales[h]), float(v_scales[h]))
        kc_all[:, h] = kc.reshape(num_pages, PS, D)
        vc_all[:, h] = vc.reshape(num_pages, PS, D)
        if dtype == FP8:
            o = ol.paged_decode(1, dtype, q[:, h * G:(h + 1) * G].copy().view(np.uint16), kc, vc, bt, lens, G, 1, D, PS,
                                k_scale=float(k_scales[h]), v_scale=float(v_scales[h]), threads=0)
        else:
            # the oracle reads an fp16 cache unscaled (as the reference's test does); the kernel applies
            # k_scale / v_scale to either cache type, which for fp16 is sm_scale * k_scale and out * v_scale
            o = ol.paged_decode(1, dtype, q[:, h * G:(h + 1) * G].copy().view(np.uint16), kc, vc, bt, lens, G, 1, D, PS,
                                sm_scale=float(np.float32(k_scales[h]) / np.sqrt(np.float32(D))), threads=0)
            o = o * np.float32(v_scales[h])
        out[:, h * G:(h + 1) * G] = o
    return kc_all, vc_all, out


def _decode(torch, pa, dtype, q, kc, vc, d_bt, lens, num_pages, scale, dks=None, dvs=None, ctas=0):
    dq = torch.from_numpy(q.view(np.int16)).cuda().view(torch.float16)
    out = torch.zeros_like(dq)
    plan = pa.make_plan(pa.KVDtype(dtype), lens, HQ, HKV, D, ctas)
    dp = pa.DevicePlan()
    dp.upload(plan, G, D)
    d_lens = torch.tensor(lens, dtype=torch.int32, device="cuda")
    p = pa.DecodeParams()
    p.q, p.out, p.k_cache, p.v_cache = dq.data_ptr(), out.data_ptr(), kc.data_ptr(), vc.data_ptr()
    p.block_table, p.seq_lens, p.block_table_stride = d_bt.data_ptr(), d_lens.data_ptr(), d_bt.shape[1]
    p.batch, p.num_q_heads, p.num_kv_heads, p.head_dim, p.page_size = len(lens), HQ, HKV, D, PS
    p.sm_scale = 1.0 / float(np.sqrt(np.float32(D)))
    p.k_scale = p.v_scale = scale
    dp.bind(p)
    pa.paged_decode(pa.KVDtype(dtype), p, 0, num_pages, d_k_scales=dks, d_v_scales=dvs)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    return out


@pytest.mark.parametrize("ctas", [0, 40])
def test_per_head_scales_against_the_oracle_head_by_head(ctas, torch_cuda, pa):
    torch = torch_cuda
    lens = [700, 33, 2049, 1]
    gains = [1.0, 0.25, 4.0, 0.02, 2.0, 0.5, 8.0, 0.1]
    K, V, q, bt, num_pages = _layer(torch, lens, gains, seed=3)
    ks = [4.5 * g / 448.0 for g in gains]
    vs = [5.0 * g / 448.0 for g in gains]
    kc, vc, d_bt, dks, dvs = _engine_append(torch, pa, FP8, K, V, bt, num_pages, 1.0, ks, vs)
    want_k, want_v, want = _oracle_per_head(FP8, K, V, q, bt, num_pages, lens, ks, vs)
    assert (kc.cpu().numpy().reshape(want_k.shape) == want_k).all(), "K bytes differ from the oracle's per-head append"
    assert (vc.cpu().numpy().reshape(want_v.shape) == want_v).all(), "V bytes differ from the oracle's per-head append"
    out = _decode(torch, pa, FP8, q, kc, vc, d_bt, lens, num_pages, 1.0, dks, dvs, ctas)
    err = float(np.abs(out.float().cpu().numpy() - want).max())
    assert err <= TOL * max(gains), err       # outputs of head h scale with gains[h]; TOL is quoted at unit magnitude
    rel = np.abs(out.float().cpu().numpy() - want).reshape(len(lens), HKV, G, D).max(axis=(0, 2, 3)) / np.asarray(gains)
    assert rel.max() <= TOL, rel


@pytest.mark.parametrize("dtype", [FP16, FP8])
def test_equal_head_scales_reproduce_the_per_tensor_path(dtype, torch_cuda, pa):
    torch = torch_cuda
    lens = [513, 64, 3000]
    K, V, q, bt, num_pages = _layer(torch, lens, [1.0] * HKV, seed=5)
    s = 4.0 / 448.0 if dtype == FP8 else 0.75       # for an fp16 cache the scales are plain multipliers
    kc0, vc0, d_bt, _, _ = _engine_append(torch, pa, dtype, K, V, bt, num_pages, s)
    kc1, vc1, _, dks, dvs = _engine_append(torch, pa, dtype, K, V, bt, num_pages, 123.0, [s] * HKV, [s] * HKV)
    assert torch.equal(kc0, kc1) and torch.equal(vc0, vc1)
    for mode in (0, 2):                               # both schedules of the fp16 kernel
        before = pa.head_fused()
        pa.set_head_fused(mode)
        try:
            a = _decode(torch, pa, dtype, q, kc0, vc0, d_bt, lens, num_pages, s)
            b = _decode(torch, pa, dtype, q, kc0, vc0, d_bt, lens, num_pages, 123.0, dks, dvs)
        finally:
            pa.set_head_fused(before)
        assert torch.equal(a, b), f"schedule mode {mode}"


def test_fp16_cache_with_different_head_scales_in_both_schedules(torch_cuda, pa):
    torch = torch_cuda
    lens = [900, 17, 4100]
    K, V, q, bt, num_pages = _layer(torch, lens, [1.0] * HKV, seed=8)
    ks = [1.0, 0.5, 2.0, 0.25, 1.5, 0.75, 3.0, 0.125]
    vs = [2.0, 1.0, 0.5, 4.0, 0.25, 1.25, 0.75, 1.0]
    kc, vc, d_bt, _, _ = _engine_append(torch, pa, FP16, K, V, bt, num_pages, 1.0)
    _, _, want = _oracle_per_head(FP16, K, V, q, bt, num_pages, lens, ks, vs)
    dks = torch.tensor(ks, dtype=torch.float32, device="cuda")
    dvs = torch.tensor(vs, dtype=torch.float32, device="cuda")
    before = pa.head_fused()
    try:
        for mode in (0, 2):
            pa.set_head_fused(mode)
            out = _decode(torch, pa, FP16, q, kc, vc, d_bt, lens, num_pages, 1.0, dks, dvs)
            rel = np.abs(out.float().cpu().numpy() - want).reshape(len(lens), HKV, G, D).max(axis=(0, 2, 3)) / np.asarray(vs)
            assert rel.max() <= TOL, (mode, rel)
    finally:
        pa.set_head_fused(before)


def test_cache_object_applies_head_scales(torch_cuda, pa):
    torch = torch_cuda
    lens = [300, 1000, 45]
    gains = [1.0, 0.1, 3.0, 0.03, 1.0, 0.3, 10.0, 0.01]
    K, V, q, _, _ = _layer(torch, lens, gains, seed=11)
    ks = [4.5 * g / 448.0 for g in gains]
    vs = [4.5 * g / 448.0 for g in gains]
    pages = [(n + PS - 1) // PS for n in lens]
    cfg = pa.PagedKVCache.Config(num_pages=sum(pages) + 8, page_size=PS, num_kv_heads=HKV, head_dim=D, max_slots=len(lens),
                                 max_pages_per_slot=max(pages) + 1, dtype=pa.KVDtype.FP8_E4M3, k_scale=1.0, v_scale=1.0)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(2)
    with pytest.raises(pa.InvalidArgument):
        cache.set_head_scales(ks, None)
    with pytest.raises(pa.InvalidArgument):
        cache.set_head_scales([0.0] * HKV, vs)
    cache.set_head_scales(ks, vs)
    dK = [torch.from_numpy(k.view(np.int16)).cuda().view(torch.float16) for k in K]
    dV = [torch.from_numpy(v.view(np.int16)).cuda().view(torch.float16) for v in V]
    for b in range(len(lens)):
        assert cache.admit() == b
    # all but the last token of every sequence one by one, the last tokens as one batched step
    for b, n in enumerate(lens):
        assert cache.append(b, dK[b], dV[b], n - 1)
    cache.append_batch(list(range(len(lens))), [dK[b][n - 1:] for b, n in enumerate(lens)],
                       [dV[b][n - 1:] for b, n in enumerate(lens)], [1] * len(lens))
    torch.cuda.synchronize()
    with pytest.raises(pa.InvalidArgument, match="already holds tokens"):
        cache.set_head_scales(None, None)
    bt = np.zeros((len(lens), cfg.max_pages_per_slot), np.int32)
    for b in range(len(lens)):
        t = cache.block_table(b)
        bt[b, :len(t)] = t
    want_k, want_v, want = _oracle_per_head(FP8, K, V, q, bt, cfg.num_pages, lens, ks, vs)
    gk, gv = cache_bytes(cache, cfg, torch)
    assert (gk.reshape(want_k.shape) == want_k).all() and (gv.reshape(want_v.shape) == want_v).all()
    dq = torch.from_numpy(q.view(np.int16)).cuda().view(torch.float16)
    out = torch.zeros_like(dq)
    cache.decode(dq, out, len(lens), HQ)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    rel = np.abs(out.float().cpu().numpy() - want).reshape(len(lens), HKV, G, D).max(axis=(0, 2, 3)) / np.asarray(gains)
    assert rel.max() <= TOL, rel
    cache.close()


def test_per_head_scales_are_more_accurate_on_uneven_heads(torch_cuda, pa):
    """Heads whose magnitudes differ by more than E4M3's dynamic range (2^-9 .. 448): with one scale per
    tensor the small heads fall below its smallest subnormal and are stored as zeros; with one scale per
    head every head keeps full fp8 precision."""
    torch = torch_cuda
    lens = [2048, 500]
    gains = [3000.0, 0.01, 1.0, 0.01, 100.0, 0.02, 3000.0, 0.05]
    K, V, q, bt, num_pages = _layer(torch, lens, gains, seed=13)
    kc16, vc16, d_bt, _, _ = _engine_append(torch, pa, FP16, K, V, bt, num_pages, 1.0)
    truth = _decode(torch, pa, FP16, q, kc16, vc16, d_bt, lens, num_pages, 1.0).float().cpu().numpy()
    tensor_scale = 4.5 * max(gains) / 448.0
    kc, vc, _, _, _ = _engine_append(torch, pa, FP8, K, V, bt, num_pages, tensor_scale)
    per_tensor = _decode(torch, pa, FP8, q, kc, vc, d_bt, lens, num_pages, tensor_scale).float().cpu().numpy()
    hs = [4.5 * g / 448.0 for g in gains]
    kc, vc, _, dks, dvs = _engine_append(torch, pa, FP8, K, V, bt, num_pages, 1.0, hs, hs)
    per_head = _decode(torch, pa, FP8, q, kc, vc, d_bt, lens, num_pages, 1.0, dks, dvs).float().cpu().numpy()

    def head_rel_err(x):
        e = np.abs(x - truth).reshape(len(lens), HKV, G, D).max(axis=(0, 2, 3))
        return e / np.abs(truth).reshape(len(lens), HKV, G, D).max(axis=(0, 2, 3))
    e_tensor, e_head = head_rel_err(per_tensor), head_rel_err(per_head)
    small = [h for h, g in enumerate(gains) if g < 0.1]
    assert all(e_head[h] < 0.1 for h in small), e_head
    assert all(e_head[h] * 4 < e_tensor[h] for h in small), (e_tensor, e_head)
