"""The benchmark configurations at their literal sizes on the GPU, against the CPU oracle.

Everything else in the GPU suite runs small cases; these run the launches the benchmark times: a full wave of
the sharded step (64 sequences x 64 nodes x 152064 bf16 logits through the unsplit-row path, greedy and lossy
results from one pass, then compaction of 4096-token caches behind a random page table) and the stochastic batch
(64 sequences x 128-node trees)."""
import pytest
import torch

from oracle import kv_oracle as ko
from oracle import verify_oracle as vo
from subspec_b200 import synthetic
from subspec_b200.step import SpeculativeStepBatch
from subspec_b200.tree import Tree
from subspec_b200.verify import flatten_tree, verify_tree_batched

pytestmark = pytest.mark.gpu

VOCAB, NODES, WAVE = 152064, 64, 64
LOSSY_KW = {"threshold_method": "entropy", "threshold": 0.3, "window_size": 6}
KV = dict(kv_layers=28, kv_heads=4, head_dim=128, page_len=16, pages_per_seq=256)   # 4096 tokens per sequence
TOKENS = KV["pages_per_seq"] * KV["page_len"]


def _flats(trees):
    out = []
    for st in trees:
        tok, off, idx = flatten_tree(Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist()), 0, limit=st.n,
                                     restrict=True)
        out.append((tok, off, idx, st.n, 0))
    return out


@pytest.mark.parametrize("variant", ["literal", "peaked"])
def test_sharded_step_full_wave(cuda_lib, variant):
    """One wave of the sharded step exactly as the benchmark launches it.  All 64 sequences: the greedy result
    (out2_*) and the lossy result (out_*) against the oracle, then the KV pool: the accepted rows of every
    sequence against the oracle's reorder, every other row of the 15 GB pool untouched."""
    free, _ = torch.cuda.mem_get_info()
    if free < 50 << 30:
        pytest.skip("needs ~35 GB of device memory")
    dev = torch.device("cuda", torch.cuda.current_device())
    ids = list(range(1000, 1000 + WAVE))
    trees, logits = synthetic.config5_wave(ids, variant, dev, nodes=NODES, vocab=VOCAB)
    gen = torch.Generator().manual_seed(77)
    table = synthetic.random_page_table(WAVE, KV["pages_per_seq"], gen)
    sb = SpeculativeStepBatch(WAVE, NODES, dev, page_table=table, **KV)
    for layer in range(KV["kv_layers"]):
        sb.pool[layer].normal_()
    before = sb.pool.clone()
    offset = TOKENS - NODES
    sb.set_trees(_flats(trees))
    sb.set_kv_offsets([offset] * WAVE)
    assert WAVE * NODES >= 4 * 148   # enough rows that no row is split over CTAs: the path the benchmark times
    sb.verify(logits, verify_method="exact+lossy", verify_kwargs=LOSSY_KW)
    sb.compact_kv()
    out = sb.results()

    accepted = moved = undecided = 0
    may_change = torch.zeros(WAVE * KV["pages_per_seq"], KV["page_len"], dtype=torch.bool)
    tail_pages = NODES // KV["page_len"]   # the tree's 64 rows are the last four pages of a sequence
    for b, st in enumerate(trees):
        lg = logits[b].cpu()
        kw = dict(logits=lg, token_ids=st.token_ids.tolist(), children=st.children(), upcast=True)
        want_exact = vo.verify(method="exact", **kw)
        want_lossy = vo.verify(method="lossy", threshold=LOSSY_KW["threshold"], window=LOSSY_KW["window_size"],
                               threshold_method="entropy", **kw)
        if want_lossy.min_gate_margin <= 1e-5:   # a gate within rounding of its threshold: not pinned by fp32
            undecided += 1
        for pre, want in (("out2", want_exact), ("out", want_lossy)):
            if pre == "out" and want_lossy.min_gate_margin <= 1e-5:
                continue
            L = int(out[pre + "_meta"][b, 0])
            assert out[pre + "_tokens"][b, :L].tolist() == want.tokens, (variant, b, pre)
            assert out[pre + "_hidden"][b, :L].tolist() == want.hidden, (variant, b, pre)
            assert (int(out[pre + "_meta"][b, 1]), int(out[pre + "_meta"][b, 2])) == \
                (want.accept_len, want.total_len), (variant, b, pre)
        accepted += want_lossy.accept_len
        # KV: rows offset + i <- offset + hidden[i]; all of them live in the sequence's last four pages
        pages = table[b, -tail_pages:].long()
        sub = before[:, pages.to(dev)].cpu()
        L = int(out["out_meta"][b, 0])
        ko.paged_reorder(sub, torch.tensor(out["out_hidden"][b, :L]), 0)   # (= the oracle's path, checked above)
        assert torch.equal(sb.pool[:, pages.to(dev)].cpu(), sub), (variant, b)
        for i, h in enumerate(out["out_hidden"][b, :L].tolist()):
            pos = offset + i
            may_change[int(table[b, pos // KV["page_len"]]), pos % KV["page_len"]] = True
            moved += int(h != i)
    # everything outside the accepted rows' destinations is bit-identical to what it was
    same = (sb.pool == before).all(dim=-1).all(dim=-1)          # [layers, pages, 2, page_len]
    untouched_ok = same | may_change.to(dev)[None, :, None, :]
    assert bool(untouched_ok.all())
    assert undecided <= 3
    if variant == "peaked":
        assert accepted > WAVE // 4 and moved > 5   # walks go down the trees and rows really move
    else:
        assert accepted >= 0


class _LazyTargets:
    """Sampled target tokens of one sequence, computed by the oracle only for the contexts a walk asks for."""

    def __init__(self, logits_dev, uniforms, temperature, top_p):
        self.logits, self.u, self.t, self.p = logits_dev, uniforms, temperature, top_p
        self.seen = {}
        self.margin = {}

    def __getitem__(self, u):
        if u not in self.seen:
            row = self.logits[u:u + 1].cpu()
            probs = vo.target_probs(row, True, self.t, self.p, upcast=True)
            self.seen[u] = vo.inverse_cdf_pick(probs[0], float(self.u[u]))
            self.margin[u] = vo.sampling_margins(row, self.t, self.p, [float(self.u[u])])[0]
        return self.seen[u]

    def __len__(self):
        return self.logits.shape[0]

    def __iter__(self):
        return iter(self.seen.get(u, -1) for u in range(len(self)))


def test_stochastic_batch_full_size(cuda_lib):
    """Config 2 at its size: 64 sequences x 128-node trees, bf16 logits N(0, 2.5^2) over 152064 tokens with the
    drafted child boosted (so that walks move), temperature 1, top-p 0.9, injected uniforms.  The walk-driven
    launch against the oracle's sample-and-match walk for every sequence whose draws are not decided by rounding;
    the every-row launch against the walk-driven one (same draws wherever both drew) and, for four sequences,
    all 128 draws against the oracle."""
    from transformers.generation.logits_process import LogitsProcessorList, TopPLogitsWarper
    from subspec_b200.verify import get_workspace

    B, N, T, TOP_P = 64, 128, 1.0, 0.9
    dev = torch.device("cuda", torch.cuda.current_device())
    cgen = torch.Generator().manual_seed(202)
    dgen = torch.Generator(device=dev).manual_seed(203)
    sts = [synthetic.random_tree(N, 10, 8, VOCAB, cgen) for _ in range(B)]
    logits = torch.empty(B, N, VOCAB, dtype=torch.bfloat16, device=dev)
    for b, st in enumerate(sts):
        x = torch.randn(N, VOCAB, generator=dgen, device=dev) * 2.5
        ch = st.children()
        for u in range(N):   # the first child of most inner nodes is likely enough to be drawn
            if ch[u] and (u + b) % 4:
                x[u, int(st.token_ids[ch[u][0]])] = 17.0
        logits[b] = x.to(torch.bfloat16)
    uniforms = torch.rand(B, N, generator=cgen)
    procs = LogitsProcessorList([TopPLogitsWarper(top_p=TOP_P)])
    trees = [Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist()) for st in sts]
    kw = dict(trees=trees, root_inds=[0] * B, logits=logits, eos_token_id=None, logits_processor=procs,
              do_sample=True, verify_method="stochastic", uniforms=uniforms)
    walk = verify_tree_batched(**kw)
    walk_targets = get_workspace(B, N, dev).fetch()["node_target"].copy()
    every = verify_tree_batched(verify_kwargs={"sample_all_nodes": True}, **kw)
    every_targets = get_workspace(B, N, dev).fetch()["node_target"].copy()

    checked = accepted = 0
    for b, st in enumerate(sts):
        lazy = _LazyTargets(logits[b], uniforms[b].tolist(), T, TOP_P)
        r = vo.exact_walk(target=lazy, token_ids=st.token_ids.tolist(), children=st.children(), root=0, n_rows=N,
                          eos=None)
        decided = all(mb > 1e-3 and mp > 1e-6 for mb, mp in lazy.margin.values())
        if decided:
            assert walk[b].sampled_tokens.squeeze(0).tolist() == r.tokens, b
            assert walk[b].hidden_indices.tolist() == r.hidden, b
            assert (walk[b].total_len, walk[b].accept_len) == (r.total_len, r.accept_len), b
            checked += 1
            accepted += r.accept_len
        # the two launches agree with each other on everything, draw for draw
        assert every[b].sampled_tokens.tolist() == walk[b].sampled_tokens.tolist(), b
        assert every[b].hidden_indices.tolist() == walk[b].hidden_indices.tolist(), b
        visited = walk_targets[b] >= 0
        assert (every_targets[b][visited] == walk_targets[b][visited]).all(), b
    assert checked >= B * 3 // 4 and accepted > B
    for b in range(4):   # every one of the 128 draws of a few sequences
        lg = logits[b].cpu()
        probs = vo.target_probs(lg, True, T, TOP_P, upcast=True)
        want = vo.target_tokens(probs, True, uniforms[b].tolist())
        margins = vo.sampling_margins(lg, T, TOP_P, uniforms[b].tolist())
        safe = [mb > 1e-3 and mp > 1e-6 for mb, mp in margins]
        assert sum(safe) >= N * 3 // 4
        for u in range(N):
            if safe[u]:
                assert int(every_targets[b, u]) == want[u], (b, u, margins[u])
