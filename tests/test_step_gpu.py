"""The batched, device-resident step (verify -> accepted-path KV compaction, no host round trip in between)
against the CPU oracle, eagerly and from a captured CUDA graph."""
import pytest
import torch

from oracle import kv_oracle as ko
from oracle import verify_oracle as vo
from subspec_b200 import synthetic
from subspec_b200.step import SpeculativeStepBatch
from subspec_b200.tree import Tree
from subspec_b200.verify import flatten_tree

pytestmark = pytest.mark.gpu

LOSSY_KW = {"threshold_method": "entropy", "threshold": 0.3, "window_size": 2}
B, NODES, VOCAB = 6, 32, 4099
KV = dict(kv_layers=3, kv_heads=2, head_dim=64, page_len=16, pages_per_seq=8)
TOKENS = KV["pages_per_seq"] * KV["page_len"]


def _case(seed):
    gen = torch.Generator().manual_seed(seed)
    trees = [synthetic.random_tree(NODES, 8, 4, VOCAB, gen) for _ in range(B)]
    logits = torch.stack([synthetic.verify_logits(t, VOCAB, gen, dtype=torch.bfloat16, peaked=True) for t in trees])
    flats = []
    for st in trees:
        tok, off, idx = flatten_tree(Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist()), 0, limit=st.n,
                                     restrict=True)
        flats.append((tok, off, idx, st.n, 0))
    return trees, logits, flats


def _batch(table, pool_cpu):
    sb = SpeculativeStepBatch(B, NODES, "cuda", page_table=table, **KV)
    sb.pool.copy_(pool_cpu)
    sb.set_kv_offsets([TOKENS - NODES] * B)
    return sb


def _expected(trees, logits, pool_cpu, table):
    """Oracle: exact and lossy verification per sequence, then the reference's reorder with the lossy path."""
    pool = pool_cpu.clone()
    exact, lossy = [], []
    for b, st in enumerate(trees):
        kw = dict(logits=logits[b], token_ids=st.token_ids.tolist(), children=st.children(), upcast=True)
        exact.append(vo.verify(method="exact", **kw))
        r = vo.verify(method="lossy", threshold=LOSSY_KW["threshold"], window=LOSSY_KW["window_size"],
                      threshold_method="entropy", **kw)
        lossy.append(r)
        ko.paged_reorder(pool, torch.tensor(r.hidden), TOKENS - NODES, page_table=table[b].tolist())
    return exact, lossy, pool


def _check(out, exact, lossy):
    for b in range(B):
        for pre, want in (("out2", exact[b]), ("out", lossy[b])):
            L = int(out[pre + "_meta"][b, 0])
            assert out[pre + "_tokens"][b, :L].tolist() == want.tokens
            assert out[pre + "_hidden"][b, :L].tolist() == want.hidden
            assert int(out[pre + "_meta"][b, 1]) == want.accept_len


def test_step_matches_the_oracle(cuda_lib):
    trees, logits, flats = _case(5)
    gen = torch.Generator().manual_seed(6)
    table = synthetic.random_page_table(B, KV["pages_per_seq"], gen)
    pool_cpu = torch.randn(KV["kv_layers"], B * KV["pages_per_seq"], 2, KV["page_len"], KV["kv_heads"], KV["head_dim"],
                           generator=gen).to(torch.bfloat16)
    sb = _batch(table, pool_cpu)
    sb.set_trees(flats)
    sb.verify(logits.cuda(), verify_method="exact+lossy", verify_kwargs=LOSSY_KW)
    sb.compact_kv()
    out = sb.results()
    exact, lossy, pool_want = _expected(trees, logits, pool_cpu, table)
    _check(out, exact, lossy)
    assert sum(r.accept_len for r in lossy) > B  # the peaked inputs make the walks go somewhere
    assert torch.equal(sb.pool.cpu(), pool_want)


def test_step_from_a_cuda_graph(cuda_lib):
    """verify + compaction captured once and replayed on new logits: no allocation, no synchronisation, no host
    value baked into the launches besides the buffers' addresses."""
    gen = torch.Generator().manual_seed(16)
    table = synthetic.random_page_table(B, KV["pages_per_seq"], gen)
    pool_cpu = torch.randn(KV["kv_layers"], B * KV["pages_per_seq"], 2, KV["page_len"], KV["kv_heads"], KV["head_dim"],
                           generator=gen).to(torch.bfloat16)
    sb = _batch(table, pool_cpu)
    static_logits = torch.zeros(B, NODES, VOCAB, dtype=torch.bfloat16, device="cuda")
    trees0, logits0, flats0 = _case(21)
    sb.set_trees(flats0)
    static_logits.copy_(logits0)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):  # warm-up outside the capture (module load, function attributes)
        sb.verify(static_logits, verify_method="exact+lossy", verify_kwargs=LOSSY_KW)
        sb.compact_kv()
    torch.cuda.current_stream().wait_stream(side)
    torch.cuda.synchronize()
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        sb.verify(static_logits, verify_method="exact+lossy", verify_kwargs=LOSSY_KW)
        sb.compact_kv()
    for seed in (21, 22, 23):
        trees, logits, flats = _case(seed)
        sb.set_trees(flats)          # host -> device copy of the tree arrays into the same buffers
        sb.pool.copy_(pool_cpu)
        static_logits.copy_(logits)
        graph.replay()
        out = sb.results()
        exact, lossy, pool_want = _expected(trees, logits, pool_cpu, table)
        _check(out, exact, lossy)
        assert torch.equal(sb.pool.cpu(), pool_want)
