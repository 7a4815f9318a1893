"""Tree attention over the paged cache and the K / V append, against the full-precision restatement."""
import pytest
import torch

from oracle import attention_oracle as ao
from subspec_b200 import synthetic
from subspec_b200.attention import append_paged_kv, tree_attention_paged, tree_attention_static
from subspec_b200.tree import Tree
from tests import golden_io

pytestmark = pytest.mark.gpu


def _case(seed, B, QL, HQ, HKV, prefix_lens, n_qs, page_len=16, layers=2, layer=1, dtype=torch.bfloat16, D=128):
    gen = torch.Generator().manual_seed(seed)
    pages_per_seq = max((p + QL + page_len - 1) // page_len for p in prefix_lens) + 1
    P = B * pages_per_seq
    table = synthetic.random_page_table(B, pages_per_seq, gen)
    pool = torch.randn(layers, P, 2, page_len, HKV, D, generator=gen).to(dtype)
    q = torch.randn(B, QL, HQ, D, generator=gen).to(dtype)
    k = torch.randn(B, QL, HKV, D, generator=gen).to(dtype)
    v = torch.randn(B, QL, HKV, D, generator=gen).to(dtype)
    kv_len = [p + n for p, n in zip(prefix_lens, n_qs)]
    cols = max(kv_len) + 5
    mask = torch.zeros(B, QL, cols, dtype=torch.bool)
    for b in range(B):
        st = synthetic.random_tree(n_qs[b], 6, 3, 1000, gen)
        tree = Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())
        mask[b, :n_qs[b], :kv_len[b]] = tree.create_attention_mask(prefix_length=prefix_lens[b])[0, 0]
    return dict(B=B, QL=QL, table=table, pool=pool, q=q, k=k, v=v, kv_len=kv_len, n_q=n_qs, mask=mask,
                prefix=prefix_lens, layer=layer, page_len=page_len)


def _run_and_check(c, tol=2e-2, kv_splits=None):
    dev = "cuda"
    pool = c["pool"].to(dev)
    table = c["table"].to(dev)
    kv_len = torch.tensor(c["kv_len"], dtype=torch.int32, device=dev)
    n_q = torch.tensor(c["n_q"], dtype=torch.int32, device=dev)
    status = torch.zeros(1, dtype=torch.int32, device=dev)
    append_paged_kv(pool, c["layer"], c["k"].to(dev), c["v"].to(dev), page_table=table, kv_len=kv_len, n_q=n_q,
                    status=status)
    out = tree_attention_paged(c["q"].to(dev), pool, c["layer"], page_table=table, kv_len=kv_len,
                               mask=c["mask"].to(dev), n_q=n_q, status=status, kv_splits=kv_splits)
    assert int(status.item()) == 0
    # the append: exactly the tree's rows changed, and they hold k / v bit for bit
    want_pool = c["pool"].clone()
    for b in range(c["B"]):
        for i in range(c["n_q"][b]):
            pos = c["prefix"][b] + i
            pg, slot = int(c["table"][b, pos // c["page_len"]]), pos % c["page_len"]
            want_pool[c["layer"], pg, 0, slot] = c["k"][b, i]
            want_pool[c["layer"], pg, 1, slot] = c["v"][b, i]
    assert torch.equal(pool.cpu(), want_pool)
    worst = 0.0
    for b in range(c["B"]):
        n, nq = c["kv_len"][b], c["n_q"][b]
        pages = c["table"][b].tolist()
        kk, vv = ao.gather_rows(want_pool, c["layer"], pages, n)
        ref = ao.tree_attention(c["q"][b, :nq], kk, vv, c["mask"][b, :nq, :n])
        got = out[b, :nq].double().cpu()
        err = float((got - ref).abs().max() / ref.abs().max())
        worst = max(worst, err)
        # no worse than what rounding P to bf16 and the output to bf16 allows
        assert err < tol, (b, err)
    return worst


def test_small_trees_grouped_heads(cuda_lib):
    """Qwen2.5-7B's head layout (28 query heads on 4 KV heads), ragged prefixes that end inside a page and inside
    a 64-row tile, trees smaller than the buffers, a request with an empty prefix."""
    c = _case(1, B=4, QL=24, HQ=28, HKV=4, prefix_lens=[0, 37, 64, 131], n_qs=[24, 9, 17, 24])
    assert _run_and_check(c) < 1e-2


def test_single_kv_head_and_one_token(cuda_lib):
    c = _case(2, B=2, QL=8, HQ=4, HKV=1, prefix_lens=[5, 300], n_qs=[1, 8], page_len=8)
    _run_and_check(c)
    c = _case(3, B=1, QL=64, HQ=8, HKV=8, prefix_lens=[1000], n_qs=[64], layers=1, layer=0)
    _run_and_check(c)


@pytest.mark.parametrize("page_len", [4, 8, 24, 32, 64, 128, 192])
def test_page_lengths(cuda_lib, page_len):
    """Pages that tile the 64-row tiles of the kernel (8, 32, 64), pages that hold whole tiles (128, 192: tensor
    copies of 64 rows at an offset inside the page) and pages that do neither (4, 24: the row-by-row copies);
    prefixes that end on a tile boundary, one row before and one row after it; more than 128 query rows per KV
    head in one request (two row blocks) and fewer (one)."""
    c = _case(10 + page_len, B=3, QL=40, HQ=8, HKV=2, prefix_lens=[600, 64 * 5 - 1 - 40, 64 * 7 + 1 - 40],
              n_qs=[40, 40, 40], page_len=page_len)
    c["kv_len"] = [p + n for p, n in zip(c["prefix"], c["n_q"])]
    _run_and_check(c)
    c = _case(20 + page_len, B=2, QL=16, HQ=4, HKV=4, prefix_lens=[64 * 3 - 16, 1], n_qs=[16, 5], page_len=page_len)
    _run_and_check(c)


@pytest.mark.parametrize("seed", range(16))
def test_random_shapes(cuda_lib, seed):
    """Seeded random geometry: batch, tree size, head layout, page length, prefixes, partly filled trees, type."""
    g = torch.Generator().manual_seed(1000 + seed)
    r = lambda lo, hi: int(torch.randint(lo, hi + 1, (1,), generator=g))
    B, QL = r(1, 3), r(1, 70)
    HKV = [1, 2, 4][r(0, 2)]
    HQ = HKV * [1, 2, 4, 7][r(0, 3)]
    page_len = [1, 8, 16, 16, 40, 64, 256][r(0, 6)]
    prefix = [r(0, 700) for _ in range(B)]
    n_q = [r(1, QL) for _ in range(B)]
    dtype = [torch.bfloat16, torch.float16][r(0, 1)]
    c = _case(2000 + seed, B=B, QL=QL, HQ=HQ, HKV=HKV, prefix_lens=prefix, n_qs=n_q, page_len=page_len, dtype=dtype)
    _run_and_check(c)


@pytest.mark.parametrize("kv_splits", [1, 2, 5, 16, 40])
def test_split_cache_ranges(cuda_lib, kv_splits):
    """The cache rows of a request cut into ranges for several CTAs and merged (what a lone request with a long
    cache gets by default): one range (no merge), ranges that end inside the prefix and inside the tree, more
    ranges than tiles (empty ones), a request with an empty prefix beside a long one."""
    c = _case(30 + kv_splits, B=2, QL=40, HQ=14, HKV=2, prefix_lens=[1500, 0], n_qs=[40, 23])
    _run_and_check(c, kv_splits=kv_splits)
    c = _case(31 + kv_splits, B=1, QL=64, HQ=28, HKV=4, prefix_lens=[4032], n_qs=[64], dtype=torch.float16)
    _run_and_check(c, tol=4e-3, kv_splits=kv_splits)


@pytest.mark.parametrize("kv_splits", [1, None, 3])
def test_head_dim_64(cuda_lib, kv_splits):
    """The head dimension of the small draft models of the classic-SD generators (Llama-3.2-1B: 32 query heads
    on 8 KV heads of 64): one 64-dim half per tile, half as many MMA steps, O half as wide."""
    c = _case(40, B=2, QL=48, HQ=32, HKV=8, prefix_lens=[700, 1], n_qs=[48, 30], D=64)
    _run_and_check(c, kv_splits=kv_splits)
    c = _case(41, B=1, QL=9, HQ=6, HKV=2, prefix_lens=[133], n_qs=[9], page_len=24, dtype=torch.float16, D=64)
    _run_and_check(c, tol=4e-3, kv_splits=kv_splits)


def test_fp16_pool(cuda_lib):
    """The reference's FlashInferCache allocates its pool in fp16 (cache_manager.py:462): same kernel, the
    tensor core's other 16-bit format, P and the output rounded to fp16."""
    c = _case(7, B=3, QL=40, HQ=28, HKV=4, prefix_lens=[900, 63, 0], n_qs=[40, 13, 40], dtype=torch.float16)
    assert _run_and_check(c, tol=4e-3) < 4e-3
    c = _case(8, B=1, QL=16, HQ=4, HKV=4, prefix_lens=[333], n_qs=[16], page_len=24, dtype=torch.float16)
    _run_and_check(c, tol=4e-3)


def test_long_stream_and_peaked_rows(cuda_lib):
    """A few thousand cache rows behind one request (the ring of tiles goes round many times), and queries
    scaled so that single keys dominate rows: the running maximum moves by far more than the margin the
    rescaling of the accumulator allows itself, many times."""
    c = _case(5, B=1, QL=48, HQ=6, HKV=2, prefix_lens=[5000], n_qs=[48], page_len=16, layers=1, layer=0)
    c["q"] = (c["q"].float() * 6).to(torch.bfloat16)
    _run_and_check(c, tol=3e-2)


def test_benchmark_shape(cuda_lib):
    """One request of the sharded-step workload: a 64-node tree behind 4032 cached rows (4096 in all, page 16),
    28 query heads on 4 KV heads; linearity in V as a size-independent check beside the oracle."""
    c = _case(4, B=2, QL=64, HQ=28, HKV=4, prefix_lens=[4032, 2000], n_qs=[64, 64])
    _run_and_check(c)
    dev = "cuda"
    pool = c["pool"].to(dev)
    table, kv_len = c["table"].to(dev), torch.tensor(c["kv_len"], dtype=torch.int32, device=dev)
    o1 = tree_attention_paged(c["q"].to(dev), pool, c["layer"], page_table=table, kv_len=kv_len, mask=c["mask"].to(dev))
    pool[:, :, 1] *= 2   # V doubled: the output doubles exactly (powers of two commute with every rounding)
    o2 = tree_attention_paged(c["q"].to(dev), pool, c["layer"], page_table=table, kv_len=kv_len, mask=c["mask"].to(dev))
    assert torch.equal(o2.float(), o1.float() * 2)
    with pytest.raises(ValueError):
        tree_attention_paged(c["q"].to(dev)[..., :64].contiguous(), pool, 0, page_table=table, kv_len=kv_len,
                             mask=c["mask"].to(dev))  # a head dimension other than the pool's


def test_inside_a_cuda_graph(cuda_lib):
    """Append + attention captured once and replayed on new queries and a longer cache: the kernel reads the
    lengths, the page table and the mask from device memory at run time, and the tensor map of the pool is a
    launch parameter that the capture keeps."""
    c = _case(6, B=2, QL=32, HQ=8, HKV=2, prefix_lens=[700, 130], n_qs=[32, 32])
    dev = "cuda"
    pool, table = c["pool"].to(dev), c["table"].to(dev)
    kv_len = torch.tensor(c["kv_len"], dtype=torch.int32, device=dev)
    q, k, v, mask = (c[n].to(dev) for n in ("q", "k", "v", "mask"))
    out = torch.empty_like(q)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        for _ in range(2):  # warm-up outside the capture (function attributes, the driver entry point)
            append_paged_kv(pool, c["layer"], k, v, page_table=table, kv_len=kv_len)
            tree_attention_paged(q, pool, c["layer"], page_table=table, kv_len=kv_len, mask=mask, out=out)
    torch.cuda.current_stream().wait_stream(side)
    g = torch.cuda.CUDAGraph()
    with torch.cuda.graph(g):
        append_paged_kv(pool, c["layer"], k, v, page_table=table, kv_len=kv_len)
        tree_attention_paged(q, pool, c["layer"], page_table=table, kv_len=kv_len, mask=mask, out=out)
    for step in range(2):
        q.copy_(torch.randn_like(q.float()).to(torch.bfloat16))
        if step == 1:  # the requests have grown by three rows: same graph, new lengths
            kv_len += 3
            mask.copy_(torch.roll(mask, 3, dims=2))
            mask[:, :, :3] = True
        g.replay()
        want = torch.empty_like(q)
        append_paged_kv(pool, c["layer"], k, v, page_table=table, kv_len=kv_len)
        tree_attention_paged(q, pool, c["layer"], page_table=table, kv_len=kv_len, mask=mask, out=want)
        assert torch.equal(out, want)


def test_against_sdpa_goldens(cuda_lib):
    """The kernel against torch SDPA on the reference's masks (tests/golden/attention_*): the rows laid out in
    pages of 16 through a random page table."""
    for case in golden_io.attention_cases():
        if case["dtype"] == "float32":
            continue  # the kernel takes the 16-bit types
        st, q, k, v, mask, exact, native = golden_io.attention_golden(case)
        n_q, n, page_len, dev = case["n_q"], case["prefix"] + case["n_q"], 16, "cuda"
        pages = (n + page_len - 1) // page_len + 1
        gen = torch.Generator().manual_seed(case["seed"])
        table = synthetic.random_page_table(1, pages, gen)
        pool = torch.zeros(1, pages, 2, page_len, case["kv_heads"], 128, dtype=q.dtype)
        for pos in range(n):
            pg = int(table[0, pos // page_len])
            pool[0, pg, 0, pos % page_len], pool[0, pg, 1, pos % page_len] = k[pos], v[pos]
        out = tree_attention_paged(q[None].to(dev), pool.to(dev), 0, page_table=table.to(dev),
                                   kv_len=torch.tensor([n], dtype=torch.int32, device=dev), mask=mask[None].to(dev))
        got = out[0].float().cpu()
        tol = 2e-2 if case["dtype"] == "bfloat16" else 3e-3
        assert float((got - exact).abs().max()) < tol * float(exact.abs().max()), case["name"]
        assert float((got - native).abs().max()) < 2 * tol * float(exact.abs().max()), case["name"]


@pytest.mark.parametrize("mask_dtype", [torch.bool, torch.float32, torch.bfloat16, torch.float16])
def test_static_caches_against_sdpa_goldens(cuda_lib, mask_dtype):
    """The Hugging Face layout -- q [batch, heads, tokens, dim], key / value caches [batch, kv_heads, rows, dim],
    the mask in the `[1, 1, max_verify, max_cache_len]` buffer, bool or as invert_mask leaves it -- against torch
    SDPA on the reference's masks.  Cache lengths that are multiples of 64 (tensor copies) and not."""
    dev = "cuda"
    for case in golden_io.attention_cases():
        if case["dtype"] == "float32":
            continue
        st, q, k, v, mask, exact, native = golden_io.attention_golden(case)
        n_q, n = case["n_q"], case["prefix"] + case["n_q"]
        for max_len in (((n + 63) // 64 + 1) * 64, n + 5):
            B = 2  # the request sits in entry 1 of a two-entry cache; entry 0 holds another, shorter one
            kc = torch.randn(B, case["kv_heads"], max_len, 128).to(q.dtype)
            vc = torch.randn(B, case["kv_heads"], max_len, 128).to(q.dtype)
            kc[1, :, :n], vc[1, :, :n] = k.permute(1, 0, 2), v.permute(1, 0, 2)
            qq = torch.randn(B, case["q_heads"], n_q, 128).to(q.dtype)
            qq[1] = q.permute(1, 0, 2)
            buf = torch.zeros(1, 1, n_q + 3, max_len, dtype=torch.bool)  # a static buffer larger than the tree
            buf[0, 0, :n_q, :n] = mask
            if mask_dtype != torch.bool:
                buf = (~buf).to(mask_dtype) * torch.finfo(mask_dtype).min  # invert_mask
            kv_len = torch.tensor([min(n, 7), n], dtype=torch.int32, device=dev)
            nq = torch.tensor([min(n_q, min(n, 7)), n_q], dtype=torch.int32, device=dev)
            out = tree_attention_static(qq.to(dev), kc.to(dev), vc.to(dev), kv_len=kv_len, n_q=nq, mask=buf.to(dev))
            got = out[1].permute(1, 0, 2).float().cpu()
            tol = 2e-2 if case["dtype"] == "bfloat16" else 3e-3
            assert float((got - exact).abs().max()) < tol * float(exact.abs().max()), (case["name"], max_len)
