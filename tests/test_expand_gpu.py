"""Draft-tree expansion kernels against the reference's golden outputs and the CPU oracle."""
import pytest
import torch

from oracle import expand_oracle as eo
from subspec_b200.draft import DraftTreeBatch, topk_sampling, topk_sampling_from_logits
from tests import golden_io

pytestmark = pytest.mark.gpu
DT = golden_io.DT


def _check_topk(scores_flat, ref_vals, tok, val, par, V, exact_idx=None):
    flat = (par * V + tok).cpu()
    assert eo.same_topk(scores_flat, ref_vals, val.cpu(), flat), (ref_vals, val)
    if exact_idx is not None:  # no ties among the candidates: indices are pinned too
        assert flat.tolist() == exact_idx


def test_golden_steps_probs_in(cuda_lib):
    """topk_sampling(probabilities) == the reference's _topk_flatten on every golden step."""
    for case in golden_io.expand_cases():
        dt = DT[case["dtype"]]
        pp = torch.ones(1, 1, dtype=dt)
        for d, g in enumerate(case["steps"]):
            probs = eo.draft_probs(golden_io.expand_logits(case, d), case["temperature"])
            tok, val, par = topk_sampling(probs.cuda(), pp.cuda(), case["k"])
            assert tok.dtype == torch.int64 and par.dtype == torch.int64 and val.dtype == dt
            scores = (probs * pp.unsqueeze(-1)).view(1, -1)
            ref_vals = torch.tensor(g["probs"]).to(dt)
            uniq = len(set(scores[0].float().tolist())) == scores.numel()
            want_idx = [[p * case["vocab"] + t for p, t in zip(g["parents"][0], g["tokens"][0])]] if uniq else None
            _check_topk(scores, ref_vals, tok, val, par, case["vocab"], want_idx)
            pp = ref_vals


def test_golden_steps_fused_from_logits(cuda_lib):
    """The fused softmax + top-k gives the reference's values from the raw draft logits."""
    for case in golden_io.expand_cases():
        dt = DT[case["dtype"]]
        pp = None
        for d, g in enumerate(case["steps"]):
            logits = golden_io.expand_logits(case, d)
            tok, val, par = topk_sampling_from_logits(logits.cuda(), None if pp is None else pp.cuda(), case["k"],
                                                      case["temperature"])
            probs = eo.draft_probs(logits, case["temperature"])
            ppc = torch.ones(1, 1, dtype=dt) if pp is None else pp
            scores = (probs * ppc.unsqueeze(-1)).view(1, -1)
            ref_vals = torch.tensor(g["probs"]).to(dt)
            if dt == torch.float32:  # fp32: GPU exp/sum vs CPU exp/sum differ in the last bits
                assert torch.allclose(val.cpu(), ref_vals, rtol=1e-5, atol=0)
                assert (par * case["vocab"] + tok).cpu().tolist()[0] == \
                    [p * case["vocab"] + t for p, t in zip(g["parents"][0], g["tokens"][0])]
            else:  # 16-bit: probabilities are rounded to the dtype as the reference does -> bit-equal values
                _check_topk(scores, ref_vals, tok, val, par, case["vocab"])
            pp = ref_vals


def _ordered_tree(case):
    """The tree the stated tie order (value desc, flat index asc) gives on a golden case's probabilities: equal to
    the reference's wherever no scores tie, and the one deterministic answer where they do."""
    dt = DT[case["dtype"]]
    pp = torch.ones(1, 1, dtype=dt)
    t = eo.FlatTree(7)
    levels = []
    for d in range(case["depth"]):
        probs = eo.draft_probs(golden_io.expand_logits(case, d), case["temperature"])
        tok, val, par = eo.topk_flatten_ordered(probs, pp, case["k"])
        t.add_nodes(tok.unsqueeze(0), val.unsqueeze(0), par.unsqueeze(0))
        levels.append((tok[0].tolist(), par[0].tolist(), val[0].float().tolist()))
        pp = val
    return t, levels


def _rows_to_lists(mask2d):
    return mask2d.to(torch.uint8).cpu().tolist()


def test_device_resident_tree_matches_reference(cuda_lib):
    """DraftTreeBatch: expand level by level on the device, finalize = prune_to_top_n + mask + position ids.
    Every golden case, all dtypes, including trees no larger than `keep` (left in insertion order like the
    reference, cpu_tree.py:176-177).  Where cumulative probabilities tie (16-bit cases) the reference's node
    order depends on torch.topk's open tie order: there the values are pinned by the golden and the structure
    by the ordered restatement."""
    seen_no_prune = seen_16bit = 0
    for case in golden_io.expand_cases():
        dt = DT[case["dtype"]]
        tree = DraftTreeBatch(1, case["k"], case["depth"], "cuda", root_tokens=torch.tensor([7]), prefix_len=5,
                              max_cache_len=5 + case["k"] * case["depth"] + 3)
        oracle_tree, levels = _ordered_tree(case)
        exact_ref = case["probs_distinct"] and all(
            lv[0] == g["tokens"][0] and lv[1] == g["parents"][0] for lv, g in zip(levels, case["steps"]))
        for d in range(case["depth"]):
            probs = eo.draft_probs(golden_io.expand_logits(case, d), case["temperature"])
            tok, val, par = tree.expand(probs.cuda(), from_logits=False)
            g = case["steps"][d]
            assert val[0].float().cpu().tolist() == g["probs"][0], (case["name"], d)  # the reference's values
            assert tok[0].tolist() == levels[d][0] and par[0].tolist() == levels[d][1], (case["name"], d)
            # draft-side mask of the level, written by the same kernel into the static buffer
            want = torch.zeros(case["k"], tree.draft_mask.shape[3], dtype=torch.bool)
            rows = torch.tensor(g["static_mask"], dtype=torch.bool) if exact_ref else None
            prev = torch.ones(1, 5, dtype=torch.bool)
            for dd in range(d + 1):
                prev = eo.mask_rows(prev, levels[dd][1])
            want[:, :prev.shape[1]] = prev
            assert torch.equal(tree.get_tree_mask()[0, 0].cpu(), want), (case["name"], d)
            if rows is not None:
                assert torch.equal(tree.get_tree_mask()[0, 0].cpu(), rows), (case["name"], d)
            assert tree.draft_position_ids[0].tolist() == [5 + d] * case["k"]
        out = tree.finalize(case["keep"], position_offset=torch.tensor([11]))
        tree.check_status()
        g = case["pruned"]
        n = len(g["token_ids"])
        no_prune = n == len(case["full"]["token_ids"])
        seen_no_prune += no_prune
        seen_16bit += dt != torch.float32
        assert int(out["n_nodes"][0]) == n
        assert sorted(out["cumulative_probabilities"][0, :n].tolist(), reverse=True) == sorted(g["probs"], reverse=True)
        keep_idx = oracle_tree.prune_to_top_n(case["keep"], dt, ordered=True)
        assert out["keep_idx"][0, :n].tolist() == keep_idx
        assert out["token_ids"][0, :n].tolist() == oracle_tree.token
        assert out["parent_indices"][0, :n].tolist() == oracle_tree.parent
        assert out["depths"][0, :n].tolist() == oracle_tree.depth
        assert out["position_ids"][0, :n].tolist() == [d + 11 for d in oracle_tree.depth]
        assert _rows_to_lists(out["tree_mask"][0, :n, :n]) == _rows_to_lists(oracle_tree.mask())
        off, idx = out["child_off"][0].tolist(), out["child_idx"][0].tolist()
        assert [idx[off[i]:off[i + 1]] for i in range(n)] == oracle_tree.children
        if no_prune:
            assert keep_idx == list(range(n))
        if exact_ref:  # no ties anywhere: the reference's own numbering, node for node
            assert out["keep_idx"][0, :n].tolist() == g["keep_idx"]
            assert out["token_ids"][0, :n].tolist() == g["token_ids"]
            assert out["parent_indices"][0, :n].tolist() == g["parent_indices"]
            assert out["depths"][0, :n].tolist() == g["depths"]
            assert out["cumulative_probabilities"][0, :n].tolist() == g["probs"]
            assert _rows_to_lists(out["tree_mask"][0, :n, :n]) == g["mask"]
            assert [idx[off[i]:off[i + 1]] for i in range(n)] == g["children"]
        # padding behind a tree smaller than `keep`: no node, and a row that attends to itself only
        for r in range(n, case["keep"]):
            assert int(out["keep_idx"][0, r]) == -1
            assert out["tree_mask"][0, r].nonzero().flatten().tolist() == [r]
    assert seen_no_prune >= 4 and seen_16bit >= 4


@pytest.mark.parametrize("mask_dtype", [torch.bool, torch.float32, torch.bfloat16, torch.float16])
def test_finalize_writes_prefix_skip_and_static_buffer(cuda_lib, mask_dtype):
    """The verifier-side mask in the forms the reference's generator hands to the target forward
    (generators/classic_sd.py:33-55, 73-77): prefix columns, rows from skip_nodes, spliced into a preallocated
    [1, 1, max_verify, max_cache_len] buffer, optionally inverted to the additive form (utils/utils.py:4-6)."""
    from subspec_b200.draft import invert_mask

    checked = 0
    for case in golden_io.expand_cases():
        g = case["pruned"]
        n = len(g["token_ids"])
        _, levels = _ordered_tree(case)
        exact_ref = case["probs_distinct"] and all(
            lv[0] == s["tokens"][0] and lv[1] == s["parents"][0] for lv, s in zip(levels, case["steps"]))
        if not exact_ref:
            continue
        checked += 1
        tree = DraftTreeBatch(1, case["k"], case["depth"], "cuda", root_tokens=torch.tensor([7]))
        for d in range(case["depth"]):
            tree.expand(eo.draft_probs(golden_io.expand_logits(case, d), case["temperature"]).cuda(), from_logits=False)
        P, S = g["prefix"], g["skip"]
        max_verify, max_cache_len = case["keep"] + 5, P + case["keep"] + 9
        base = torch.zeros(1, 1, max_verify, max_cache_len, dtype=torch.bool)
        partial = torch.tensor(g["mask_prefix_skip"], dtype=torch.bool)[None, None]
        K, D = partial.shape[2], partial.shape[3]
        want = base[:, :, :K, :].clone()     # the reference's _get_tree_mask: clone the buffer rows, splice
        want[:, :, :K, :D] = partial
        if mask_dtype != torch.bool:
            want = invert_mask(want, mask_dtype)
        buf = torch.full((1, 1, max_verify, max_cache_len), 1, dtype=mask_dtype, device="cuda")  # stale contents
        out = tree.finalize(case["keep"], position_offset=[P], prefix_length=P, skip_nodes=S, mask_out=buf)
        tree.check_status()
        got = buf[:, :, :n - S].cpu()
        assert torch.equal(got.view(torch.uint8) if mask_dtype == torch.bool else
                           got.view(torch.int32 if mask_dtype == torch.float32 else torch.int16),
                           want.view(torch.uint8) if mask_dtype == torch.bool else
                           want.view(torch.int32 if mask_dtype == torch.float32 else torch.int16)), case["name"]
        assert out["token_ids"][0, S:n].tolist() == g["data_skip"]["token_ids"]
        assert out["parent_indices"][0, S:n].tolist() == g["data_skip"]["parent_indices"]
        assert out["position_ids"][0, S:n].tolist() == [d + P for d in g["data_skip"]["depths"]]
        # rows the call does not own keep their contents
        assert bool((buf[:, :, case["keep"] - S:] == 1).all())
        # a dense mask of its own, per-sequence prefix given as a tensor
        dense = tree.finalize(case["keep"], prefix_length=torch.tensor([P]), skip_nodes=S, mask_dtype=mask_dtype)
        assert tuple(dense["tree_mask"].shape) == (1, case["keep"] - S, P + case["keep"])
        assert torch.equal(dense["tree_mask"][0, :n - S, :D].cpu().float(), want[0, 0, :, :D].float())
    assert checked >= 4


def _finalize_restated(tokens, parents, probs, depths, keep):
    """prune_to_top_n + renumbering on the host (cpu_tree.py:168-206): stable order by cumulative probability,
    parents renumbered, ancestor-or-self rows."""
    n = len(tokens)
    pr = [1.0] + [float(x) for x in probs[1:]]
    order = list(range(n)) if n <= keep else sorted(range(n), key=lambda i: (-pr[i], i))[:keep]
    new_of = {o: r for r, o in enumerate(order)}
    par = [new_of.get(int(parents[o]), -1) if o else -1 for o in order]
    mask = torch.zeros(len(order), len(order), dtype=torch.bool)
    for r in range(len(order)):
        cur = r
        while cur >= 0:
            mask[r, cur] = True
            cur = par[cur]
    return order, par, mask


@pytest.mark.parametrize("keep,skip,mask_dtype", [(64, 0, torch.bool), (50, 3, torch.bool), (64, 1, torch.bfloat16),
                                                  (37, 0, torch.float32)])
def test_finalize_mask_rows_shared_between_ctas(cuda_lib, keep, skip, mask_dtype):
    """A static [batch, 1, max_verify, max_cache_len] buffer of a long cache is filled by several CTAs per
    sequence, each owning a range of rows (ranges that do not divide evenly included); a dense mask of the tree's
    own width is filled by one.  Both must say the same, and both must agree with the host restatement."""
    from subspec_b200.draft import invert_mask

    B, k, depth, V, P = 3, 16, 10, 4000, 4032
    g = torch.Generator().manual_seed(keep * 7 + skip)
    tree = DraftTreeBatch(B, k, depth, "cuda")
    for lvl in range(depth):
        tree.expand((torch.randn(B, 1 if lvl == 0 else k, V, generator=g) * 3).cuda())
    prefix = torch.tensor([P, P - 17, 5])
    buf = torch.full((B, 1, 70, 4160), 1, dtype=mask_dtype, device="cuda")
    big = tree.finalize(keep, position_offset=prefix, prefix_length=prefix, skip_nodes=skip, mask_out=buf)
    big = {key: v.clone() for key, v in big.items() if torch.is_tensor(v) and key != "tree_mask"}
    small = tree.finalize(keep, position_offset=prefix, skip_nodes=skip, mask_cols=keep)
    tree.check_status()
    for key in big:
        assert torch.equal(big[key], small[key]), key
    for b in range(B):
        n = tree.n_nodes
        order, par, m = _finalize_restated(tree.tokens[b, :n].tolist(), tree.parents[b, :n].tolist(),
                                           tree.probs[b, :n].tolist(), tree.depths[b, :n].tolist(), keep)
        assert small["keep_idx"][b].tolist() == order and small["parent_indices"][b].tolist() == par
        want = torch.zeros(keep - skip, 4160, dtype=torch.bool)
        pb = int(prefix[b])
        want[:, :pb] = True
        want[:, pb:pb + keep] = m[skip:]
        assert torch.equal(small["tree_mask"][b].cpu(), m[skip:])
        got = buf[b, 0, :keep - skip].cpu()
        if mask_dtype == torch.bool:
            assert torch.equal(got, want), b
        else:
            assert torch.equal(got.float(), invert_mask(want, mask_dtype).float()), b
        assert bool((buf[b, 0, keep - skip:] == 1).all())  # rows past the call's own keep their contents


def test_finalize_largest_tree(cuda_lib):
    """4065 nodes of the 4096 one call takes (more shared memory than a kernel gets by default), 1024 kept."""
    k, depth, V, keep = 32, 127, 300, 1024
    g = torch.Generator().manual_seed(5)
    tree = DraftTreeBatch(2, k, depth, "cuda")
    for lvl in range(depth):
        tree.expand((torch.randn(2, 1 if lvl == 0 else k, V, generator=g) * 2).cuda())
    out = tree.finalize(keep)
    tree.check_status()
    n = 1 + k * depth
    assert n == 4065
    for b in range(2):
        order, par, m = _finalize_restated(tree.tokens[b, :n].tolist(), tree.parents[b, :n].tolist(),
                                           tree.probs[b, :n].tolist(), tree.depths[b, :n].tolist(), keep)
        assert out["keep_idx"][b].tolist() == order
        assert out["parent_indices"][b].tolist() == par
        assert torch.equal(out["tree_mask"][b].cpu(), m)
        assert out["token_ids"][b].tolist() == [int(tree.tokens[b, o]) for o in order]


def test_finalize_rejects_bad_geometry(cuda_lib):
    tree = DraftTreeBatch(2, 4, 2, "cuda")
    probs = torch.rand(2, 1, 50).softmax(-1)
    tree.expand(probs.cuda(), from_logits=False)
    with pytest.raises(ValueError):
        tree.finalize(8, skip_nodes=9)
    with pytest.raises(ValueError):  # the prefix does not fit the columns the caller asked for
        tree.finalize(8, prefix_length=[3, 30], mask_cols=20)
        tree.check_status()
    tree.finalize(8, prefix_length=[3, 12], mask_cols=20)
    tree.check_status()


def test_config3_chain_matches_reference(cuda_lib):
    """Config 3 as a chain: 32 bf16 sequences (and 4 fp32 ones), ten `DraftTreeBatch.expand` levels from raw
    logits at V = 128256 with k = 16, then `finalize(64)`, against what the unmodified reference produced with
    _topk_flatten -> TreeData -> Tree.add_nodes -> prune_to_top_n(64) -> get_tree_data / create_attention_mask
    on the same seeded logits.  bf16: every level's values bit-equal, every chosen candidate carries its value,
    kept probabilities bit-equal; all of these sequences have ties somewhere, where the reference's node order
    is torch.topk's open choice, so the structure is compared with the ordered restatement.  fp32 (no ties):
    the reference's own tokens, parents, kept nodes and mask."""
    chain = golden_io.expand_chain()
    V, k, depth, keep = chain["vocab"], chain["k"], chain["depth"], chain["keep"]
    for dtype in ("bfloat16", "float32"):
        seqs = [s for s in chain["sequences"] if s["dtype"] == dtype]
        B, dt = len(seqs), DT[dtype]
        assert B == (32 if dtype == "bfloat16" else 4)
        tree = DraftTreeBatch(B, k, depth, "cuda", root_tokens=torch.full((B,), chain["root_token"]))
        oracle = [eo.FlatTree(chain["root_token"]) for _ in range(B)]
        pp = [torch.ones(1, 1, dtype=dt) for _ in range(B)]
        for d in range(depth):
            logits = torch.cat([golden_io.chain_logits(chain, s, d) for s in seqs])
            tok, val, par = tree.expand(logits.cuda(), from_logits=True, temperature=1.0)
            tok, val, par = tok.cpu(), val.cpu(), par.cpu()
            for b, s in enumerate(seqs):
                g = s["levels"][d]
                if dtype == "bfloat16":
                    probs = eo.draft_probs(logits[b:b + 1], 1.0)
                    assert val[b].float().tolist() == g["probs"], (s["seed"], d)
                    scores = (probs * pp[b].unsqueeze(-1)).view(1, -1)
                    assert eo.same_topk(scores, torch.tensor([g["probs"]]).to(dt), val[b:b + 1],
                                        (par * V + tok)[b:b + 1]), (s["seed"], d)
                    ot, ov, op = eo.topk_flatten_ordered(probs, pp[b], k)
                    assert tok[b].tolist() == ot[0].tolist() and par[b].tolist() == op[0].tolist(), (s["seed"], d)
                    oracle[b].add_nodes(ot.unsqueeze(0), ov.unsqueeze(0), op.unsqueeze(0))
                    pp[b] = ov
                else:
                    # fp32: torch's CPU softmax is itself up to ~2e-5 (relative) off the exact value on these
                    # rows and the error compounds down the chain, so the yardstick for the values is the exact
                    # (fp64) chain, within the stated 1e-5; the reference's values bound them more loosely and
                    # its indices exactly (no ties, margins audited by the generator)
                    p64 = torch.softmax(logits[b].double(), dim=-1)
                    exact = torch.stack([p64[l, t] * pp[b][0, l].double() for l, t in zip(g["parents"], g["tokens"])])
                    assert torch.allclose(val[b].double(), exact, rtol=1e-5, atol=0), (s["seed"], d)
                    assert torch.allclose(val[b], torch.tensor(g["probs"]), rtol=2e-4, atol=0), (s["seed"], d)
                    assert tok[b].tolist() == g["tokens"] and par[b].tolist() == g["parents"], (s["seed"], d)
                    pp[b] = exact.view(1, -1)
        out = tree.finalize(keep, position_offset=[100 + b for b in range(B)])
        tree.check_status()
        assert out["n_nodes"].tolist() == [keep] * B
        for b, s in enumerate(seqs):
            g = s["pruned"]
            got_rows = [int(sum(1 << j for j in r.nonzero().flatten().tolist())) for r in out["tree_mask"][b].cpu()]
            off, idx = out["child_off"][b].tolist(), out["child_idx"][b].tolist()
            kids = [idx[off[i]:off[i + 1]] for i in range(keep)]
            if dtype == "bfloat16":
                assert out["cumulative_probabilities"][b].tolist() == g["probs"], s["seed"]  # sorted, bit-equal
                keep_idx = oracle[b].prune_to_top_n(keep, dt, ordered=True)
                assert out["keep_idx"][b].tolist() == keep_idx
                assert out["token_ids"][b].tolist() == oracle[b].token
                assert out["parent_indices"][b].tolist() == oracle[b].parent
                assert out["depths"][b].tolist() == oracle[b].depth
                assert got_rows == [int(sum(1 << j for j in range(keep) if bool(m[j]))) for m in oracle[b].mask()]
                assert kids == oracle[b].children
            else:
                assert s["rule_agrees_prune"]
                assert out["keep_idx"][b].tolist() == g["keep_idx"]
                assert out["token_ids"][b].tolist() == g["token_ids"]
                assert out["parent_indices"][b].tolist() == g["parent_indices"]
                assert out["depths"][b].tolist() == g["depths"]
                assert got_rows == g["mask_rows"] and kids == g["children"]
            assert out["position_ids"][b].tolist() == [x + 100 + b for x in out["depths"][b].tolist()]


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float32])
def test_config3_shape_batched(cuda_lib, dtype):
    """Config-3 shape at reduced batch: [B, 16, 128256] logits, k = 16, against the oracle per sequence."""
    B, L, V, k = 3, 16, 128256, 16
    gen = torch.Generator().manual_seed(33)
    logits = (torch.randn(B, L, V, generator=gen) * 3.0).to(dtype)
    pp = torch.rand(B, L, generator=gen).to(dtype)
    tok, val, par = topk_sampling_from_logits(logits.cuda(), pp.cuda(), k, 1.0)
    probs = eo.draft_probs(logits, 1.0)
    _, ref_vals, _ = eo.topk_flatten(probs, pp, k)
    scores = (probs * pp.unsqueeze(-1)).view(B, -1)
    if dtype == torch.float32:
        assert torch.allclose(val.cpu(), ref_vals, rtol=2e-5, atol=0)
        rt, _, rp = eo.topk_flatten(probs, pp, k)
        assert torch.equal((par * V + tok).cpu(), rp * V + rt)
    else:
        _check_topk(scores, ref_vals, tok, val, par, V)
    # probabilities-in path on the same data, unaligned vocabulary (odd row length)
    tok2, val2, par2 = topk_sampling(probs[:, :, :V - 3].contiguous().cuda(), pp.cuda(), k)
    _, ref2, _ = eo.topk_flatten(probs[:, :, :V - 3].contiguous(), pp, k)
    _check_topk((probs[:, :, :V - 3] * pp.unsqueeze(-1)).reshape(B, -1), ref2, tok2, val2, par2, V - 3)


@pytest.mark.parametrize("B,L,V,dtype,temperature", [
    (1, 1, 128256, torch.bfloat16, 1.0), (1, 16, 128256, torch.float16, 0.7), (2, 5, 32000, torch.float32, 1.3),
    (1, 16, 152064, torch.bfloat16, 1.0), (9, 16, 32000, torch.bfloat16, 1.0)])
def test_few_rows_are_cut_into_slices(cuda_lib, B, L, V, dtype, temperature):
    """A launch with few rows cuts every row into slices (one CTA each) whose lists and softmax sums meet behind
    a ticket per row: a single sequence's step, the reference's own setting.  Same answers as the oracle."""
    k = 16
    gen = torch.Generator().manual_seed(B * 100 + L)
    logits = (torch.randn(B, L, V, generator=gen) * 3.0).to(dtype)
    pp = torch.rand(B, L, generator=gen).to(dtype)
    probs = eo.draft_probs(logits, temperature)
    rt, ref_vals, rp = eo.topk_flatten(probs, pp, k)
    scores = (probs * pp.unsqueeze(-1)).view(B, -1)
    for rep in range(2):  # twice: the tickets are cleared by every call
        tok, val, par = topk_sampling_from_logits(logits.cuda(), pp.cuda(), k, temperature)
        if dtype == torch.float32:
            assert torch.allclose(val.cpu(), ref_vals, rtol=2e-5, atol=0)
            assert torch.equal((par * V + tok).cpu(), rp * V + rt)
        else:
            _check_topk(scores, ref_vals, tok, val, par, V)
    tok2, val2, par2 = topk_sampling(probs.cuda(), pp.cuda(), k)   # probabilities in
    _check_topk(scores, ref_vals, tok2, val2, par2, V)


def test_edge_cases(cuda_lib):
    # k larger than the vocabulary is clamped like the reference (min(k, vocab)); ties resolved by flat index
    probs = torch.full((1, 2, 3), 0.25, dtype=torch.float32)
    tok, val, par = topk_sampling(probs.cuda(), torch.ones(1, 2).cuda(), 8)
    assert tok.shape == (1, 3)
    assert (par * 3 + tok).tolist() == [[0, 1, 2]]
    # ascending data: every element beats the running k-th (worst case for the candidate queue)
    V = 5000
    asc = torch.arange(V, dtype=torch.float32).view(1, 1, V) / V
    tok, val, par = topk_sampling(asc.cuda(), torch.ones(1, 1).cuda(), 16)
    assert tok.tolist() == [list(range(V - 1, V - 17, -1))]
    with pytest.raises(ValueError):
        topk_sampling(torch.rand(2, 3), torch.ones(1, 2), 4)
