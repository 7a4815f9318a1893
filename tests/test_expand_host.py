"""Expansion: the CPU oracle and the host-side tree classes against vectors produced by the reference."""
import torch

from oracle import expand_oracle as eo
from subspec_b200.draft import DraftParams, TreeData, TreeMaskCache, invert_mask
from subspec_b200.tree import Tree
from tests import golden_io

DT = golden_io.DT


def _replay(case, topk_fn):
    """Run the depth loop with `topk_fn(probs, parent_probs, k)`; returns per-step outputs."""
    dt = DT[case["dtype"]]
    parent_probs = torch.ones(1, 1, dtype=dt)
    outs = []
    for d in range(case["depth"]):
        probs = eo.draft_probs(golden_io.expand_logits(case, d), case["temperature"])
        tok, val, par = topk_fn(probs, parent_probs, case["k"])
        outs.append((probs, parent_probs, tok, val, par))
        parent_probs = val
    return outs


def test_oracle_topk_matches_reference():
    for case in golden_io.expand_cases():
        for d, (probs, pp, tok, val, par) in enumerate(_replay(case, eo.topk_flatten)):
            g = case["steps"][d]
            assert val.float().tolist() == g["probs"], (case["name"], d)
            assert tok.tolist() == g["tokens"] and par.tolist() == g["parents"], (case["name"], d)


def test_oracle_tree_matches_reference():
    for case in golden_io.expand_cases():
        dt = DT[case["dtype"]]
        t = eo.FlatTree(7)
        toks = torch.tensor([[s["tokens"][0] for s in case["steps"]]])
        pars = torch.tensor([[s["parents"][0] for s in case["steps"]]])
        probs = torch.tensor([[s["probs"][0] for s in case["steps"]]]).to(dt)
        t.add_nodes(toks, probs, pars)
        assert t.token == case["full"]["token_ids"] and t.parent == case["full"]["parent_indices"]
        assert t.depth == case["full"]["depths"]
        assert t.mask().to(torch.uint8).tolist() == [row[3:] for row in case["full"]["mask"]]
        keep = t.prune_to_top_n(case["keep"], dt)
        g = case["pruned"]
        assert keep == g["keep_idx"] and t.token == g["token_ids"] and t.parent == g["parent_indices"]
        assert t.children == g["children"] and t.leaves == g["leaves"]
        assert t.mask().to(torch.uint8).tolist() == g["mask"]
        # draft-side incremental mask
        prev = torch.ones(1, 5, dtype=torch.bool)
        for s in case["steps"]:
            prev = eo.mask_rows(prev, s["parents"][0])
            assert prev.to(torch.uint8).tolist() == s["mask"]


def test_product_tree_matches_reference():
    """subspec_b200.Tree: add_nodes numbering, get_tree_data, create_attention_mask, prune_to_top_n, leaves."""
    for case in golden_io.expand_cases():
        dt = DT[case["dtype"]]
        data = TreeData()
        for s in case["steps"]:
            data.update(torch.tensor(s["tokens"]), torch.tensor(s["probs"]).to(dt), torch.tensor(s["parents"]))
        tree = Tree(torch.tensor(7), dt)
        tree.add_nodes(*data.get_data())
        full = tree.get_tree_data()
        g = case["full"]
        assert full["token_ids"].tolist() == g["token_ids"] and full["depths"].tolist() == g["depths"]
        assert full["parent_indices"].tolist() == g["parent_indices"]
        assert full["cumulative_probabilities"].float().tolist() == g["probs"]
        assert tree.create_attention_mask(prefix_length=3)[0, 0].to(torch.uint8).tolist() == g["mask"]
        assert tree.size() == len(g["token_ids"]) and int(tree.get_depth()) == case["depth"]
        keep = tree.prune_to_top_n(case["keep"])
        p = case["pruned"]
        if case["probs_distinct"]:
            assert keep.tolist() == p["keep_idx"]
            assert [list(n.children) for n in tree.nodes] == p["children"]
            assert tree.available_leaves == p["leaves"]
            assert tree.create_attention_mask()[0, 0].to(torch.uint8).tolist() == p["mask"]
            assert tree.get_tree_data()["parent_indices"].tolist() == p["parent_indices"]
        else:  # tied probabilities: the kept multiset of probabilities is pinned, the order inside ties is not
            assert sorted(tree.get_tree_data()["cumulative_probabilities"].float().tolist()) == sorted(p["probs"])
        # structural invariants after pruning
        for i, n in enumerate(tree.nodes):
            for c in n.children:
                assert tree.nodes[c].parent == i
        assert tree.find_child_index(0, tree.nodes[tree.nodes[0].children[0]].token_id) == tree.nodes[0].children[0]
        assert tree.find_child_index(0, -5) == -1


def test_product_mask_cache_and_params():
    for case in golden_io.expand_cases():
        for static in (False, True):
            cache = TreeMaskCache(prefix_len=5, sample_len=case["k"],
                                  max_cache_len=5 + case["k"] * case["depth"] if static else None,
                                  dtype=torch.float32, device="cpu")
            for d, s in enumerate(case["steps"]):
                m = cache.update_tree_mask(torch.tensor(s["parents"]), return_invert=False)
                got = m[0, 0, :, :5 + case["k"] * (d + 1)] if static else m[0, 0]
                want = torch.tensor(s["mask"], dtype=torch.bool)
                if d == 0 and static:
                    got = got[:want.shape[0]]
                assert torch.equal(got[:want.shape[0]], want), (case["name"], d, static)
            inv = cache.get_tree_mask(return_invert=True)
            assert inv.dtype == torch.float32 and float(inv.min()) == torch.finfo(torch.float32).min
    assert torch.equal(invert_mask(torch.tensor([True, False]), torch.float16),
                       torch.tensor([0.0, torch.finfo(torch.float16).min], dtype=torch.float16))
    p = DraftParams(temperature=0.2, max_depth=32, topk_len=6)
    assert p.max_sample_tokens == 193 and p.max_verify_tokens == 193
    assert DraftParams(max_depth=8, topk_len=6, max_verify_tokens=40).max_verify_tokens == 40


def test_prune_to_depth_and_tree_views():
    t = Tree.from_arrays([1, 2, 3, 4, 5, 6], [-1, 0, 0, 1, 3, 3])
    assert [n.depth for n in t.nodes] == [0, 1, 1, 2, 3, 3]
    kept = t.prune_to_depth(2)
    assert kept.tolist() == [0, 1, 2, 3] and t.size() == 4
    assert t.available_leaves == [2, 3] and t.nodes[3].has_been_sampled is False
    assert t.prune_to_depth(10).tolist() == [0, 1, 2, 3]
    assert t.get_children_indices(0).tolist() == [1, 2] and t.get_children_ids(1).tolist() == [4]


def test_masks_with_prefix_and_skipped_rows_match_reference():
    """create_attention_mask(prefix_length, skip_nodes), get_tree_data(skip_nodes) and the static draft-side
    mask buffer, against what the reference's classes returned (also for trees that prune_to_top_n leaves alone)."""
    no_prune = 0
    for case in golden_io.expand_cases():
        dt = DT[case["dtype"]]
        data = TreeData()
        for s in case["steps"]:
            data.update(torch.tensor(s["tokens"]), torch.tensor(s["probs"]).to(dt), torch.tensor(s["parents"]))
        tree = Tree(torch.tensor(7), dt)
        tree.add_nodes(*data.get_data())
        keep = tree.prune_to_top_n(case["keep"])
        p = case["pruned"]
        if tree.size() == len(case["full"]["token_ids"]):
            no_prune += 1
            assert keep.tolist() == list(range(tree.size())) == p["keep_idx"]
            assert tree.get_tree_data()["parent_indices"].tolist() == case["full"]["parent_indices"]
        if case["probs_distinct"] or tree.size() == len(case["full"]["token_ids"]):
            m = tree.create_attention_mask(prefix_length=p["prefix"], skip_nodes=p["skip"])
            assert m[0, 0].to(torch.uint8).tolist() == p["mask_prefix_skip"]
            d = tree.get_tree_data(p["skip"])
            for key in ("token_ids", "depths", "parent_indices"):
                assert d[key].tolist() == p["data_skip"][key]
        cache = TreeMaskCache(prefix_len=5, sample_len=case["k"], max_cache_len=5 + case["k"] * case["depth"] + 3,
                              dtype=torch.float32, device="cpu")
        for s in case["steps"]:
            got = cache.update_tree_mask(torch.tensor(s["parents"]), return_invert=False)
            assert got[0, 0].to(torch.uint8).tolist() == s["static_mask"]
    assert no_prune >= 4


def test_oracle_reproduces_reference_expansion_chains():
    """Ten levels at the benchmark's vocabulary (a subset of the golden sequences, to keep the CPU suite short):
    the restated top-k gives the reference's values at every level, and where torch.topk's open tie order played
    no part (`rule_agrees`) the ordered variant gives its indices and its pruned tree too."""
    chain = golden_io.expand_chain()
    V, k = chain["vocab"], chain["k"]
    assert len(chain["sequences"]) == 36 and sum(s["dtype"] == "bfloat16" for s in chain["sequences"]) == 32
    picked = [s for s in chain["sequences"] if s["dtype"] == "bfloat16"][:2] + \
        [s for s in chain["sequences"] if s["rule_agrees_prune"]][:1]
    assert len(picked) == 3
    for seq in picked:
        dt = DT[seq["dtype"]]
        pp = torch.ones(1, 1, dtype=dt)
        tree = eo.FlatTree(chain["root_token"])
        for d, g in enumerate(seq["levels"]):
            probs = eo.draft_probs(golden_io.chain_logits(chain, seq, d), 1.0)
            tok, val, par = eo.topk_flatten_ordered(probs, pp, k)
            assert val[0].float().tolist() == g["probs"], (seq["seed"], d)
            scores = (probs * pp.unsqueeze(-1)).view(1, -1)
            assert eo.same_topk(scores, torch.tensor([g["probs"]]).to(dt), val, par * V + tok)
            if seq["rule_agrees"]:
                assert tok[0].tolist() == g["tokens"] and par[0].tolist() == g["parents"]
            tree.add_nodes(tok.unsqueeze(0), val.unsqueeze(0), par.unsqueeze(0))
            pp = val
        keep = tree.prune_to_top_n(chain["keep"], dt, ordered=True)
        assert sorted(tree.prob, reverse=True) == sorted(seq["pruned"]["probs"], reverse=True)
        if seq["rule_agrees_prune"]:
            assert keep == seq["pruned"]["keep_idx"] and tree.parent == seq["pruned"]["parent_indices"]
            rows = [int(sum(1 << j for j in range(len(keep)) if bool(m[j]))) for m in tree.mask()]
            assert rows == seq["pruned"]["mask_rows"]
