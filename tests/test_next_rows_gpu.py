"""GPU parity tests of the rows next to the decode path: the batched multi-slot append (the step
before the path; src/decode/paged_kv_cache.cu:95-136 of the reference run once per slot) and the
`Decoder` torch-tensor binding (bindings/torch_decode.cu:14-81)."""
import math

import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, cache_bytes

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [0, 1])
def test_append_batch_equals_per_slot_appends(dtype, torch_cuda, pa):
    """A serving loop: prefill six slots, then 40 decode steps of one new token per slot (plus a
    release / re-admit in the middle).  Cache A takes each step with one append_batch call, cache B
    with one append per slot, the oracle's allocator model follows along: block tables, lengths,
    free lists and all cache bytes must be identical."""
    torch = torch_cuda
    hkv, d, ps, B = 4, 128, 16, 6
    scale = 4.0 / 448.0 if dtype else 1.0
    mk = lambda: pa.PagedKVCache(pa.PagedKVCache.Config(num_pages=40, page_size=ps, num_kv_heads=hkv, head_dim=d,
                                                        max_slots=B, max_pages_per_slot=12, dtype=pa.KVDtype(dtype),
                                                        k_scale=scale, v_scale=scale))
    A, Bc, model = mk(), mk(), ol.PoolModel(40, ps, B, 12)
    for pool in (A, Bc):
        pool.shuffle_free_pages(9)
    model.shuffle(9)
    gen = torch.Generator(device="cuda").manual_seed(4)
    rnd = lambda n: torch.randn(n, hkv, d, device="cuda", dtype=torch.float16, generator=gen)
    lens0 = [5, 16, 31, 1, 47, 100]
    for b, n in enumerate(lens0):
        assert A.admit() == Bc.admit() == model.admit() == b
    ks, vs = [rnd(n) for n in lens0], [rnd(n) for n in lens0]
    assert A.append_batch(list(range(B)), ks, vs, lens0)            # the prefill as one batch
    for b in range(B):
        assert Bc.append(b, ks[b], vs[b], lens0[b]) and model.append(b, lens0[b])
    for step in range(40):
        slots = [b for b in range(B) if not (step % 7 == 3 and b == 2)]     # some steps skip a slot
        k1, v1 = [rnd(1) for _ in slots], [rnd(1) for _ in slots]
        assert A.append_batch(slots, k1, v1, [1] * len(slots))
        for i, b in enumerate(slots):
            assert Bc.append(b, k1[i], v1[i], 1) and model.append(b, 1)
        if step == 20:   # a sequence finishes and a new one takes its slot
            for pool in (A, Bc, model):
                pool.release(4)
                assert pool.admit() == 4
            k2, v2 = rnd(33), rnd(33)
            assert A.append_batch([4], [k2], [v2], [33])
            assert Bc.append(4, k2, v2, 33) and model.append(4, 33)
    torch.cuda.synchronize()
    for b in range(B):
        assert A.block_table(b).tolist() == Bc.block_table(b).tolist() == model.table(b).tolist()
        assert A.seq_len(b) == Bc.seq_len(b) == model.seq_len(b)
    assert A.free_list().tolist() == Bc.free_list().tolist() == model.free_list().tolist()
    (ak, av), (bk, bv) = cache_bytes(A, A.config(), torch), cache_bytes(Bc, Bc.config(), torch)
    assert (ak == bk).all() and (av == bv).all()
    # the device-side tables and lengths were updated by the batch path too: decode both and compare
    q = torch.randn(B, 16, d, device="cuda", dtype=torch.float16, generator=gen)
    oa, ob = torch.zeros_like(q), torch.zeros_like(q)
    A.decode(q, oa, B, 16, 13)
    Bc.decode(q, ob, B, 16, 13)
    torch.cuda.synchronize()
    assert torch.equal(oa, ob)

    # all-or-nothing when the pool cannot hold every slot's tokens; bad batches change nothing
    free_before, lens_before = A.free_pages(), [A.seq_len(b) for b in range(B)]
    big = [rnd(16 * 12) for _ in range(B)]
    assert A.free_pages() < 3 * B
    assert not A.append_batch(list(range(B)), big, big, [16 * 3] * B)      # 18 more pages than the pool has
    with pytest.raises(pa.InvalidArgument, match="twice"):
        A.append_batch([0, 0], big[:2], big[:2], [1, 1])
    with pytest.raises(pa.LengthError):
        A.append_batch([0], big[:1], big[:1], [16 * 12])
    assert A.free_pages() == free_before and [A.seq_len(b) for b in range(B)] == lens_before
    A.close()
    Bc.close()


def test_release_waits_for_a_batched_append_on_another_stream(torch_cuda, pa):
    """append_batch is stream-ordered and does not wait; release() hands the slot's pages back and zeroes its
    device-side length with a memset that is not ordered with that stream.  On a non-blocking stream (every
    torch stream is one) the scatter may still be pending: release must wait for it, so that the freed pages
    are not rewritten later and the slot's device length ends at zero (a device-side plan reads it)."""
    torch = torch_cuda
    from common import device_view
    hkv, d, ps = 8, 128, 16
    cfg = pa.PagedKVCache.Config(num_pages=600, page_size=ps, num_kv_heads=hkv, head_dim=d, max_slots=3,
                                 max_pages_per_slot=300)
    cache = pa.PagedKVCache(cfg)
    gen = torch.Generator(device="cuda").manual_seed(1)
    n = 4096
    k0 = torch.randn(n, hkv, d, device="cuda", dtype=torch.float16, generator=gen)
    k1 = torch.randn(n, hkv, d, device="cuda", dtype=torch.float16, generator=gen)
    k2 = torch.randn(64, hkv, d, device="cuda", dtype=torch.float16, generator=gen)
    assert cache.admit() == 0 and cache.admit() == 1
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    busy = torch.empty(256 << 20, dtype=torch.uint8, device="cuda")
    with torch.cuda.stream(side):
        for _ in range(8):
            busy.fill_(1)                       # keeps the side stream occupied while the host runs ahead
        assert cache.append_batch([0, 1], [k0, k1], [k0, k1], [n, n], side.cuda_stream)
    cache.release(0)                            # host-side at once; must not overtake the scatter on `side`
    assert cache.admit() == 0
    assert cache.append(0, k2, k2, 64)          # reuses the pages slot 0 had (default stream)
    torch.cuda.synchronize()
    lens = device_view(cache.params().seq_lens, 12, torch).view(torch.int32).tolist()
    assert lens == [64, n, 0]
    # slot 0's new tokens are what its pages hold now, not the released sequence's scatter arriving late
    q = torch.randn(2, 32, d, device="cuda", dtype=torch.float16, generator=gen)
    out = torch.zeros_like(q)
    cache.plan_device(2, 32)
    cache.run(q, out)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    K = [k2.cpu().numpy(), k1.cpu().numpy()]
    kc = np.zeros(cfg.num_pages * hkv * ps * d, np.uint16)
    vc = np.zeros_like(kc)
    bt = np.zeros((2, cfg.max_pages_per_slot), np.int32)
    for b in range(2):
        t = cache.block_table(b)
        bt[b, :len(t)] = t
        ol.append(0, K[b].view(np.uint16), K[b].view(np.uint16), kc, vc, t, 0, hkv, d, ps)
    want = ol.paged_decode(1, 0, q.cpu().numpy().view(np.uint16), kc, vc, bt, [64, n], 32, hkv, d, ps)
    assert float(np.abs(out.float().cpu().numpy() - want).max()) <= TOL
    cache.close()


@pytest.mark.parametrize("fp8", [False, True])
def test_decoder_binding_on_raw_tensors(fp8, torch_cuda, pa):
    """Inputs built the way the reference's FlashInfer harness builds them
    (scripts/compare_flashinfer.py:80-101): random pools, per-tensor scale amax/448, scattered table."""
    torch = torch_cuda
    from paged_attention_b200.torch_decode import Decoder
    hq, hkv, dim, page, batch, seq_len = 32, 8, 128, 16, 5, 1000
    g = torch.Generator(device="cuda").manual_seed(0)
    pages_per_seq = math.ceil(seq_len / page)
    num_pages = batch * pages_per_seq
    k = torch.randn(num_pages, hkv, page, dim, device="cuda", dtype=torch.float16, generator=g)
    v = torch.randn(num_pages, hkv, page, dim, device="cuda", dtype=torch.float16, generator=g)
    k_scale = v_scale = 1.0
    if fp8:
        k_scale, v_scale = k.abs().max().item() / 448.0, v.abs().max().item() / 448.0
        k, v = (k / k_scale).to(torch.float8_e4m3fn), (v / v_scale).to(torch.float8_e4m3fn)
    block_table = torch.randperm(num_pages, device="cuda", generator=g).to(torch.int32).view(batch, pages_per_seq).contiguous()
    q = torch.randn(batch, hq, dim, device="cuda", dtype=torch.float16, generator=g)
    lens = torch.full((batch,), seq_len, dtype=torch.int32)
    dec = Decoder(hq, hkv, dim, page, fp8)
    dec.plan(lens, 50)
    out = dec.run(q, k, v, block_table, lens.cuda(), k_scale, v_scale)
    torch.cuda.synchronize()
    assert dec.num_ctas > 0 and dec.num_segments >= batch * hkv
    np_dt = np.uint8 if fp8 else np.uint16
    kc = k.view(torch.uint8 if fp8 else torch.int16).cpu().numpy().view(np_dt).reshape(-1)
    vc = v.view(torch.uint8 if fp8 else torch.int16).cpu().numpy().view(np_dt).reshape(-1)
    want = ol.paged_decode(1, int(fp8), q.cpu().numpy().view(np.uint16), kc, vc, block_table.cpu().numpy(),
                           lens.numpy(), hq, hkv, dim, page, k_scale=k_scale, v_scale=v_scale)
    assert np.abs(out.float().cpu().numpy() - want).max() < TOL
    with pytest.raises(ValueError):
        dec.run(q[:2].contiguous(), k, v, block_table, lens.cuda(), k_scale, v_scale)
    with pytest.raises(TypeError):
        dec.plan(lens.cuda())
