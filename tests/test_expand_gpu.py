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


def test_device_resident_tree_matches_reference(cuda_lib):
    """DraftTreeBatch: expand level by level on the device, finalize = prune_to_top_n + mask + position ids."""
    for case in golden_io.expand_cases():
        if not case["probs_distinct"] or case["dtype"] != "float32":
            continue
        tree = DraftTreeBatch(1, case["k"], case["depth"], "cuda", root_tokens=torch.tensor([7]))
        for d in range(case["depth"]):
            probs = eo.draft_probs(golden_io.expand_logits(case, d), case["temperature"])
            tree.expand(probs.cuda(), from_logits=False)
        out = tree.finalize(case["keep"], position_offset=torch.tensor([11]))
        g = case["pruned"]
        n = len(g["token_ids"])
        assert int(out["n_nodes"][0]) == n
        assert out["keep_idx"][0, :n].tolist() == g["keep_idx"]
        assert out["token_ids"][0, :n].tolist() == g["token_ids"]
        assert out["parent_indices"][0, :n].tolist() == g["parent_indices"]
        assert out["depths"][0, :n].tolist() == g["depths"]
        assert out["cumulative_probabilities"][0, :n].tolist() == g["probs"]
        assert out["position_ids"][0, :n].tolist() == [d + 11 for d in g["depths"]]
        assert out["tree_mask"][0, :n, :n].to(torch.uint8).tolist() == g["mask"]
        off, idx = out["child_off"][0].tolist(), out["child_idx"][0].tolist()
        assert [idx[off[i]:off[i + 1]] for i in range(n)] == g["children"]


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
