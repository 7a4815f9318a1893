"""Accepted-path KV compaction on the GPU: bit-exact against the reference's golden checksums and the oracle."""
import pytest
import torch

from oracle import kv_oracle as ko
from subspec_b200 import kv_cache as kc
from subspec_b200 import synthetic
from tests import golden_io

pytestmark = pytest.mark.gpu


def test_golden_pool_reorder_through_request_object(cuda_lib):
    for c in golden_io.kv_cases():
        pool = kc.KvCachePool(c["pages"], c["layers"], c["heads"], c["head_dim"], c["page_len"],
                              golden_io.DT[c["dtype"]], "cuda")
        pool.cache_data.copy_(golden_io.kv_pool(c))
        req = kc.RequestKvCache(pool, c["page_len"], c["offset"] + c["tree_n"])
        req.reorder_cache_with_offset(torch.tensor(c["beam"]), offset=c["offset"] + 1 if c["offset"] else 0)
        assert ko.checksum(pool.cache_data.cpu()) == c["after"], c["seed"]
        assert (req.kv_len, req.kv_last_page_len, len(req.kv_page_indices)) == (
            c["kv_len"], c["kv_last_page_len"], c["n_pages"])
        assert int(pool.num_free_pages()) == c["free_pages"]


def test_batched_random_page_table(cuda_lib):
    """Config-5 layout at reduced length: random page table, several sequences, device-side n/offset/beam."""
    B, L, H, D, page_len, pages_per_seq = 6, 28, 4, 128, 16, 12
    gen = torch.Generator().manual_seed(41)
    table = synthetic.random_page_table(B, pages_per_seq, gen)
    pool = torch.randn(L, B * pages_per_seq, 2, page_len, H, D, generator=gen).to(torch.bfloat16)
    tokens = pages_per_seq * page_len
    offs, ns, beams = [], [], torch.zeros(B, 16, dtype=torch.int64)
    expect = pool.clone()
    for b in range(B):
        off = tokens - 64 - b
        n = 1 + (b * 3) % 11
        beam = torch.cat([torch.zeros(1, dtype=torch.long),
                          torch.sort(torch.randperm(63, generator=gen)[:n - 1] + 1).values])
        offs.append(off)
        ns.append(n)
        beams[b, :n] = beam
        ko.paged_reorder(expect, beam, off, page_table=table[b].tolist())
    dpool = pool.cuda()
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    kc.compact_paged(dpool, page_table=table.cuda(), offset=torch.tensor(offs, dtype=torch.int32).cuda(),
                     n=torch.tensor(ns, dtype=torch.int32).cuda(), beam=beams.cuda(), status=status)
    assert int(status.item()) == 0
    assert torch.equal(dpool.cpu(), expect)


def test_destination_aliases_a_later_source(cuda_lib):
    """beam = [0, 2, 5, 6, ...]: destination 2 is the source of element 1; more rows than one staging chunk."""
    pool = kc.KvCachePool(8, 2, 2, 64, 8, torch.float16, "cuda")
    gen = torch.Generator().manual_seed(3)
    pool.cache_data.copy_(torch.randn(pool.cache_data.shape, generator=gen).to(torch.float16))
    expect = pool.cache_data.cpu().clone()
    beam = torch.tensor([0, 2, 5, 6, 7, 9, 12, 13, 17, 18, 19, 20, 22, 23, 24, 26, 27, 30, 31, 33])
    ko.paged_reorder(expect, beam, 10)
    pool.reorder_cache_with_offset(beam, offset=10)
    assert torch.equal(pool.cache_data.cpu(), expect)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_hf_layout_static_and_dynamic(cuda_lib, dtype):
    gen = torch.Generator().manual_seed(17)
    layers, H, T, D = 5, 4, 96, 128
    cache = kc.TreeStaticCache(num_layers=layers, num_kv_heads=H, head_dim=D, max_cache_len=T, device="cuda",
                               dtype=dtype, max_batch_size=1)
    ks = [torch.randn(1, H, T, D, generator=gen).to(dtype) for _ in range(layers)]
    vs = [torch.randn(1, H, T, D, generator=gen).to(dtype) for _ in range(layers)]
    for i in range(layers):
        cache.key_cache[i].copy_(ks[i])
        cache.value_cache[i].copy_(vs[i])
    ptrs = [t.data_ptr() for t in cache.key_cache]
    beam = torch.tensor([0, 1, 4, 9, 30])
    mgr = kc.KVManager(cache)
    mgr.reorder_cache_with_offset(beam, new_chunk_len=5, offset=40)
    ko.hf_static_reorder(ks, vs, beam, 40)
    for i in range(layers):
        assert torch.equal(cache.key_cache[i].cpu(), ks[i]) and torch.equal(cache.value_cache[i].cpu(), vs[i])
    assert ptrs == [t.data_ptr() for t in cache.key_cache]  # static addresses survive

    dyn = kc.TreeDynamicCache()
    ks = [torch.randn(1, H, 70, D, generator=gen).to(dtype) for _ in range(layers)]
    vs = [torch.randn(1, H, 70, D, generator=gen).to(dtype) for _ in range(layers)]
    for i in range(layers):
        dyn.update(ks[i].cuda(), vs[i].cuda(), i)
    dyn.reorder_cache_with_offset(beam, offset=38)
    ko.hf_dynamic_reorder(ks, vs, beam, 38)
    for i in range(layers):
        assert dyn.key_cache[i].shape == ks[i].shape
        assert torch.equal(dyn.key_cache[i].cpu(), ks[i]) and torch.equal(dyn.value_cache[i].cpu(), vs[i])


def test_golden_hf_layout_reorders(cuda_lib):
    """The HF-layout caches against checksums left by the reference's own TreeStaticCache /
    TreeDynamicCache.reorder_cache_with_offset (tests/golden/kv_hf_cases.json), called the way the generators
    call them: through KVManager with dim=2 (generators/classic_sd.py:254)."""
    cases = golden_io.kv_hf_cases()
    assert len(cases) >= 12
    for c in cases:
        dt = golden_io.DT[c["dtype"]]
        ks, vs = golden_io.kv_hf_tensors(c)
        beam = torch.tensor(c["beam"])
        cache = kc.TreeStaticCache(num_layers=c["layers"], num_kv_heads=c["heads"], head_dim=c["head_dim"],
                                   max_cache_len=c["tokens"], device="cuda", dtype=dt, max_batch_size=1)
        for i in range(c["layers"]):
            cache.key_cache[i].copy_(ks[i])
            cache.value_cache[i].copy_(vs[i])
        kc.KVManager(cache).reorder_cache_with_offset(beam, new_chunk_len=c["tree_n"], offset=c["offset"], dim=2)
        got = torch.stack([t.cpu() for t in list(cache.key_cache) + list(cache.value_cache)])
        assert ko.checksum(got) == c["static_after"], c["seed"]
        dyn = kc.TreeDynamicCache()
        for i in range(c["layers"]):
            dyn.update(ks[i].cuda(), vs[i].cuda(), i)
        kc.KVManager(dyn).reorder_cache_with_offset(beam, new_chunk_len=c["tree_n"], offset=c["offset"], dim=2)
        got = torch.stack([t.cpu() for t in list(dyn.key_cache) + list(dyn.value_cache)])
        assert got.shape[3] == c["dynamic_tokens"]
        assert ko.checksum(got) == c["dynamic_after"], c["seed"]


def test_bad_indices_are_reported(cuda_lib):
    pool = kc.KvCachePool(4, 1, 1, 8, 4, torch.float32, "cuda")
    with pytest.raises(ValueError):
        pool.reorder_cache_with_offset(torch.tensor([0, 40]), offset=2)  # source beyond the pool
    with pytest.raises(ValueError):
        pool.reorder_cache_with_offset(torch.arange(70), offset=0)  # more rows than one step can keep
    # full-size property: compaction is idempotent once the kept rows are in place (beam = 0..n-1)
    before = pool.cache_data.clone()
    pool.reorder_cache_with_offset(torch.arange(5), offset=3)
    assert torch.equal(pool.cache_data, before)


def test_flashinfer_cache_holder(cuda_lib):
    """FlashInferCache builds the pool the reference builds (cache_manager.py:419-466): fp16, one page."""
    from types import SimpleNamespace
    cfg = SimpleNamespace(hidden_size=512, num_attention_heads=8, num_hidden_layers=3, num_key_value_heads=2)
    c = kc.FlashInferCache(cfg, max_tokens=100, PAGE_LEN=16)
    assert c.max_cache_len == 100 and c.config is cfg
    assert tuple(c.kvCachePool.cache_data.shape) == (3, 1, 2, 16, 2, 64) and c.kvCachePool.cache_data.dtype == torch.float16
    c.kvCachePool.cache_data.fill_(1.0)
    c.reset()
    assert float(c.kvCachePool.cache_data.abs().sum()) == 0.0
    big = kc.FlashInferCache(cfg, max_tokens=100, PAGE_LEN=16, max_pages=7)
    assert big.kvCachePool.max_pages == 7 and int(big.kvCachePool.num_free_pages()) == 7
