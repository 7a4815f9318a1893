"""The CPU oracle against vectors produced by the reference itself (tests/golden/make_golden.py)."""
import pytest
import torch

from oracle import verify_oracle as vo
from tests import golden_io


def _run_oracle(case, upcast):
    tree, logits = golden_io.verify_input(case)
    skip, rows = case["skip_nodes"], case["rows"]
    ch_all = tree.children()
    n_loc = tree.n - skip
    ch = [[c - skip for c in ch_all[v + skip] if c - skip >= 0] for v in range(n_loc)]
    tok = tree.token_ids[skip:].tolist()
    probs = vo.target_probs(logits, upcast=upcast)
    tgt = probs.argmax(-1).tolist()
    kw = case["kwargs"]
    if case["method"] == "exact":
        r = vo.exact_walk(target=tgt + [-1] * (n_loc - rows), token_ids=tok, children=ch,
                          root=case["root_ind"] - skip, n_rows=rows, eos=case["eos"])
    else:
        n = min(rows, n_loc)
        root = case["root_ind"] - skip
        if root < 0 or root >= n:
            root = 0
        r = vo.lossy_verify(probs=probs[:n], token_ids=tok[:n], children=[[c for c in k if c < n] for k in ch[:n]],
                            root=root, eos=case["eos"], threshold=float(kw.get("threshold", 0.0)),
                            window=int(kw.get("window_size", 1)),
                            use_entropy=kw.get("threshold_method", "prob") == "entropy", target=tgt[:n])
    return dict(tokens=r.tokens, hidden=[h + skip for h in r.hidden], total_len=r.total_len, accept_len=r.accept_len)


@pytest.mark.parametrize("upcast", [False, True])
def test_oracle_matches_reference_verify_tree(upcast):
    cases = golden_io.verify_cases()
    assert len(cases) >= 150
    bad = []
    for case in cases:
        if upcast and not case["upcast_agrees"]:
            continue
        if _run_oracle(case, upcast) != case["expected"]:
            bad.append(case["name"])
    assert not bad, bad


def test_oracle_matches_reference_unit_tests():
    cases = golden_io.lossy_unit_cases()
    assert len(cases) == 8
    for c in cases:
        probs = torch.tensor(c["probs"], dtype=torch.float32)
        r = vo.lossy_verify(probs=probs, token_ids=c["token_ids"], children=c["children_lists"],
                            root=c["root_index"], eos=c["eos_token_id"], threshold=c["threshold"],
                            window=c["window_size"], use_entropy=c["threshold_method"] == "entropy")
        assert r.tokens == c["expected"]["sampled"], c["test"]
        assert r.hidden == c["expected"]["hidden"], c["test"]
        assert r.accept_len == c["expected"]["accept_len"], c["test"]


def test_inverse_cdf_pick_edges():
    row = torch.tensor([0.0, 0.25, 0.0, 0.5, 0.25, 0.0])
    assert vo.inverse_cdf_pick(row, 0.0) == 1
    assert vo.inverse_cdf_pick(row, 0.2499) == 1
    assert vo.inverse_cdf_pick(row, 0.25) == 3
    assert vo.inverse_cdf_pick(row, 0.9999999) == 4
    assert vo.inverse_cdf_pick(row, 1.0) == 4


def test_kv_oracle_matches_reference_pool_reorder():
    from oracle import kv_oracle as ko

    cases = golden_io.kv_cases()
    assert len(cases) >= 12
    for c in cases:
        pool = golden_io.kv_pool(c)
        assert ko.checksum(pool) == c["before"]
        ko.paged_reorder(pool, torch.tensor(c["beam"]), c["offset"])
        assert ko.checksum(pool) == c["after"], c["seed"]


def test_kv_oracle_matches_reference_hf_layout_reorders():
    """hf_static_reorder / hf_dynamic_reorder against checksums left by the reference's own
    TreeStaticCache / TreeDynamicCache.reorder_cache_with_offset (run on a stand-in object by make_golden.py)."""
    from oracle import kv_oracle as ko

    cases = golden_io.kv_hf_cases()
    assert len(cases) >= 12
    for c in cases:
        ks, vs = golden_io.kv_hf_tensors(c)
        assert ko.checksum(torch.stack(ks + vs)) == c["before"]
        beam = torch.tensor(c["beam"])
        sk, sv = [t.clone() for t in ks], [t.clone() for t in vs]
        ko.hf_static_reorder(sk, sv, beam, c["offset"])
        assert ko.checksum(torch.stack(sk + sv)) == c["static_after"], c["seed"]
        dk, dv = [t.clone() for t in ks], [t.clone() for t in vs]
        ko.hf_dynamic_reorder(dk, dv, beam, c["offset"])
        assert dk[0].shape[2] == c["dynamic_tokens"]
        assert ko.checksum(torch.stack(dk + dv)) == c["dynamic_after"], c["seed"]


def test_kv_oracle_page_table_is_consistent_with_identity():
    from oracle import kv_oracle as ko

    gen = torch.Generator().manual_seed(9)
    pool = torch.randn(2, 6, 2, 4, 2, 8, generator=gen)
    ident = pool.clone()
    ko.paged_reorder(ident, torch.tensor([0, 3, 4, 9]), 5)
    # scatter the logical pages over physical pages with a permutation, reorder, and undo the permutation
    perm = torch.tensor([4, 0, 5, 2, 1, 3])
    phys = torch.empty_like(pool)
    phys[:, perm] = pool
    ko.paged_reorder(phys, torch.tensor([0, 3, 4, 9]), 5, page_table=perm.tolist())
    assert torch.equal(phys[:, perm], ident)


@pytest.mark.parametrize("temperature,top_k,top_p", [(1.0, 0, 0.9), (0.7, 50, 1.0), (1.3, 20, 0.8), (1.0, 1, 1.0),
                                                      (0.5, 5000, 0.95)])
def test_oracle_filters_match_transformers_warpers(temperature, top_k, top_p):
    """`target_probs` against the processors the reference's `_sample_token` runs (generators/base.py:42-64,
    109-139): transformers' temperature / top-k / top-p warpers followed by softmax, on tie-free rows."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    gen = torch.Generator().manual_seed(11)
    logits = torch.randn(7, 3001, generator=gen) * 3.0
    procs = LogitsProcessorList()
    if temperature != 1.0:
        procs.append(TemperatureLogitsWarper(temperature))
    if top_k:
        procs.append(TopKLogitsWarper(top_k=top_k))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    want = torch.softmax(procs(None, logits.clone()), dim=-1)
    got = vo.target_probs(logits, True, temperature, top_p, upcast=False, top_k=top_k)
    assert torch.equal(want > 0, got > 0)
    assert torch.allclose(want, got, rtol=1e-6, atol=0)


def test_oracle_matches_reference_sampled_verification():
    """do_sample=True: the reference ran with its own warpers, softmax, walk and lossy verifier, its
    torch.multinomial replaced by the inverse-CDF pick for injected uniforms (tests/golden/make_golden.py).
    The restatement in the reference's arithmetic reproduces every case except those the generator flagged:
    16-bit rows where torch.sort's unspecified order among tied logits decides which of them the nucleus
    keeps (the restatement and the CUDA path drop the lowest vocabulary indices first)."""
    cases = golden_io.sampled_cases()
    flagged = [c for c in cases if not c["oracle_agrees"]]
    assert len(cases) >= 80 and len(flagged) <= 3
    assert all(c["dtype"] != "float32" and (c["top_p"] < 1.0) for c in flagged)
    accepted = 0
    for c in cases:
        if not c["oracle_agrees"]:
            continue
        tree, logits = golden_io.sampled_input(c)
        kw = c["kwargs"]
        r = vo.verify(logits=logits, token_ids=tree.token_ids.tolist(), children=tree.children(), method=c["method"],
                      do_sample=True, temperature=c["temperature"], top_p=c["top_p"], top_k=c["top_k"],
                      uniforms=c["uniforms"], threshold=float(kw.get("threshold", 0.0)),
                      window=int(kw.get("window_size", 1)), threshold_method=kw.get("threshold_method", "prob"),
                      upcast=False)
        got = dict(tokens=r.tokens, hidden=r.hidden, total_len=r.total_len, accept_len=r.accept_len)
        assert got == c["expected"], c["name"]
        accepted += r.accept_len
    assert accepted > 50  # the walks go somewhere


def test_post_verify_oracle_matches_reference_tree_methods():
    """find_child_index and prune_to_depth against the reference's Tree on seeded trees, level-ordered and
    rank-numbered (children lists out of ascending order)."""
    from oracle import postverify_oracle as po

    cases = golden_io.post_cases()
    assert len(cases) == 24 and any(c["ranked"] for c in cases)
    for c in cases:
        t = c["tree"]
        for node, tok, want in c["finds"]:
            assert po.find_child_index(t["token_ids"], t["children"], node, tok) == want
        for pr in c["prunes"]:
            keep, tok, par, dep, ch = po.prune_to_depth(t["token_ids"], t["parents"], t["depths"], t["children"],
                                                        pr["max_depth"])
            assert keep == pr["keep"] and tok == pr["token_ids"] and par == pr["parents"] and dep == pr["depths"]
            assert ch == pr["children"]
            if len(keep) < len(t["token_ids"]):  # an early return leaves the reference's leaf list as it was
                assert [i for i in range(len(keep)) if not ch[i]] == pr["leaves"]


def test_attention_oracle_against_sdpa_on_the_reference_masks():
    """The attention oracle against torch's scaled_dot_product_attention fed the way transformers' SDPA attention
    feeds it on the reference's default path (repeat_kv, additive mask from the reference's
    Tree.create_attention_mask + invert_mask): same numbers to fp32 accuracy, and our Tree builds the same mask."""
    from oracle import attention_oracle as ao
    from subspec_b200.tree import Tree
    for case in golden_io.attention_cases():
        st, q, k, v, mask, exact, native = golden_io.attention_golden(case)
        tree = Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())
        assert torch.equal(tree.create_attention_mask(prefix_length=case["prefix"])[0, 0], mask)
        want = ao.tree_attention(q, k, v, mask)
        assert float((want - exact.double()).abs().max()) < 2e-5 * float(exact.abs().max()), case["name"]
        # the result in the inputs' own type is the fp32 one up to that type's rounding (of P and of the output)
        tol = {"bfloat16": 2e-2, "float16": 3e-3, "float32": 8e-3}[case["dtype"]]  # fp32 case: stored as bf16
        assert float((native.double() - want).abs().max()) < tol * float(want.abs().max()), case["name"]
