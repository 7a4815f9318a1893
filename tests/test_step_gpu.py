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


def test_loop_runs_without_host_round_trips(cuda_lib):
    """SpeculativeLoopBatch: five steps of grow -> verify -> re-root -> delayed reorder -> trim for four
    requests, launched back to back; only the test looks at the device state in between.  Against the oracle's
    verification, the delayed-reorder bookkeeping and the reference's pool reorder."""
    from oracle import postverify_oracle as po
    from subspec_b200.step import SpeculativeLoopBatch

    Bn, n, rows, vocab = 4, 16, 9, 997   # the trees reach past the decoded rows, as after a post-speculation
    gen = torch.Generator().manual_seed(44)
    init = [5, 17, 32, 9]
    loop = SpeculativeLoopBatch(Bn, n, "cuda", kv_layers=2, kv_heads=2, head_dim=64, page_len=16, pages_per_seq=12,
                                init_len=torch.tensor(init))
    loop.pool.copy_(torch.randn(loop.pool.shape, generator=gen).to(torch.bfloat16))
    want_pool = loop.pool.cpu().clone()
    oracle = [po.DelayedReorder(x) for x in init]
    pending = [0] * Bn   # rows of earlier trees still waiting for their reorder
    deferred = 0
    for step in range(5):
        sts = [synthetic.random_tree(n, 5, 3, vocab, gen) for _ in range(Bn)]
        logits = torch.stack([synthetic.verify_logits(s, vocab, gen, dtype=torch.bfloat16, peaked=True, boost_frac=0.9)
                              for s in sts])
        flats = []
        for s in sts:
            tok, off, idx = flatten_tree(Tree.from_arrays(s.token_ids.tolist(), s.parents.tolist()), 0)
            flats.append((tok, off, idx, rows, 0))
        pos = loop.begin_step(rows)
        assert pos.seq_indptr.tolist() == [b * rows for b in range(Bn + 1)]
        assert loop.pages.kv_len.tolist() == [oracle[b].kv_len + pending[b] + rows for b in range(Bn)]
        table = loop.pages.page_table.cpu()
        loop.set_trees(flats)
        if step == 4:
            loop.state.finished.fill_(1)
        loop.end_step(logits[:, :rows].contiguous().cuda())
        loop.check()
        for b, s in enumerate(sts):
            target = vo.target_probs(logits[b, :rows], upcast=True).argmax(-1).tolist()
            r = vo.exact_walk(target=target + [-1] * (n - rows), token_ids=s.token_ids.tolist(),
                              children=s.children(), root=0, n_rows=rows, eos=None)
            root = po.find_child_index(s.token_ids.tolist(), s.children(), r.hidden[-1], r.tokens[-1])
            assert int(loop.state.next_root[b]) == (root + pending[b] if root >= 0 else -1)
            beam, at = oracle[b].step([h + pending[b] for h in r.hidden], root, finished=step == 4)
            if beam is None:
                deferred += 1
                pending[b] += rows
            else:
                ko.paged_reorder(want_pool, torch.tensor(beam), at, page_table=table[b].tolist())
                pending[b] = 0
            assert int(loop.state.kv_len[b]) == oracle[b].kv_len
            assert int(loop.pages.kv_len[b]) == oracle[b].kv_len + pending[b]
            assert int(loop.pages.n_pages[b]) == -(-(oracle[b].kv_len + pending[b]) // 16)
        assert torch.equal(loop.pool.cpu(), want_pool), step
    assert deferred >= 1 and pending == [0] * Bn
