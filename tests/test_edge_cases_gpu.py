"""Edges of the supported domain (the reference supports any page size >= 1 and any length >= 1,
src/decode/decode.cu:24-36,79): an empty batch, thousands of one-token sequences, and a sequence of a
million tokens.  The long case is checked through a size-independent property: attention over a sequence
that repeats a block of tokens r times equals attention over the block once (every key appears r times
with the same score, so the softmax weights of its copies add up to the weight it has in the block), which
the oracle can compute on the short block.
"""
import numpy as np
import pytest

import oracle_lib as ol
from common import TOL, Case, run_case, seeded_kv

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("dtype", [0, 1])
def test_empty_batch_is_a_no_op(dtype, torch_cuda, pa):
    torch = torch_cuda
    cfg = pa.PagedKVCache.Config(num_pages=8, page_size=16, num_kv_heads=8, head_dim=128, max_slots=4,
                                 max_pages_per_slot=4, dtype=pa.KVDtype(dtype), k_scale=0.01, v_scale=0.01)
    cache = pa.PagedKVCache(cfg)
    q = torch.zeros(0, 32, 128, dtype=torch.float16, device="cuda")
    out = torch.zeros_like(q)
    cache.plan([], 32)
    assert cache.last_plan().num_segments == 0
    cache.run(q, out)
    cache.decode(q, out, 0, 32)
    dp = pa.DevicePlan()
    dp.build(dtype, torch.zeros(1, dtype=torch.int32, device="cuda"), 0, 32, 8, 128, 0)
    assert dp.info()[:2] == (0, 0)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    cache.close()


@pytest.mark.parametrize("dtype", [0, 1])
def test_thousands_of_one_token_sequences(dtype, torch_cuda, pa):
    # attention over a single token returns that token's V (dequantised): no softmax to speak of
    err, out, want, info = run_case(Case(dtype, 8, 8, 16, [1] * 3000, shuffle=5, seed=9, extra_pages=0), torch_cuda, pa)
    assert err <= TOL
    assert info["segments"] == 3000 * 8


@pytest.mark.parametrize("dtype,ps", [(0, 16), (1, 16), (0, 4096)])
def test_million_token_sequence_equals_its_repeating_block(dtype, ps, torch_cuda, pa):
    torch = torch_cuda
    hq, hkv, block, repeats = 32, 8, 4096, 256          # 1 048 576 tokens: 4 GiB of fp16 K+V
    L = block * repeats
    K, V = seeded_kv([block], hkv, 128, 77)
    scale = 4.5 / 448.0 if dtype == 1 else 1.0
    pages = (L + ps - 1) // ps
    cfg = pa.PagedKVCache.Config(num_pages=pages, page_size=ps, num_kv_heads=hkv, head_dim=128, max_slots=1,
                                 max_pages_per_slot=pages, dtype=pa.KVDtype(dtype), k_scale=scale, v_scale=scale)
    cache = pa.PagedKVCache(cfg)
    cache.shuffle_free_pages(1)
    dK = torch.from_numpy(K[0].view(np.int16)).cuda().view(torch.float16)
    dV = torch.from_numpy(V[0].view(np.int16)).cuda().view(torch.float16)
    assert cache.admit() == 0
    for _ in range(repeats):
        assert cache.append(0, dK, dV, block)
    assert cache.seq_len(0) == L
    q = torch.randn(1, hq, 128, dtype=torch.float16, generator=torch.Generator().manual_seed(2)).cuda()
    out = torch.zeros_like(q)
    cache.decode(q, out, 1, hq)
    torch.cuda.synchronize()
    assert pa.kernel_status() == 0
    plan = cache.last_plan()
    assert plan.num_segments > 8, "one sequence spread over the whole grid"
    cache.close()

    # the oracle on one block, stored through the oracle's own append
    np_dt = np.uint16 if dtype == 0 else np.uint8
    bp = (block + 15) // 16
    kc, vc = np.zeros(bp * hkv * 16 * 128, np_dt), np.zeros(bp * hkv * 16 * 128, np_dt)
    table = np.arange(bp, dtype=np.int32)
    ol.append(dtype, K[0].view(np.uint16), V[0].view(np.uint16), kc, vc, table, 0, hkv, 128, 16, scale, scale)
    want = ol.paged_decode(1, dtype, q.cpu().numpy().view(np.uint16), kc, vc, table[None, :], [block], hq, hkv, 128, 16,
                           k_scale=scale, v_scale=scale, threads=0)
    err = float(np.abs(out.float().cpu().numpy() - want).max())
    assert err <= TOL, err
