"""Parity of the fused CUDA verifier with the reference's outputs (golden) and with the CPU oracle."""
import pytest
import torch

from oracle import verify_oracle as vo
from subspec_b200 import synthetic
from subspec_b200.tree import Tree
from subspec_b200.verify import lossy_bottom_up_verify, verify_tree, verify_tree_batched
from subspec_b200.wandb_logger import wandb_logger
from tests import golden_io

pytestmark = pytest.mark.gpu


def _tree_of(st: synthetic.SynthTree) -> Tree:
    return Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())


def test_reference_unit_cases_through_the_kernel(cuda_lib):
    """The eight hand-built cases of the reference's own test file, same signature, on the GPU."""
    for c in golden_io.lossy_unit_cases():
        wandb_logger.clear_log_data()
        sampled, hidden, acc = lossy_bottom_up_verify(
            probs=torch.tensor(c["probs"], dtype=torch.float32), token_ids=torch.tensor(c["token_ids"]),
            parent_indices=torch.tensor(c["parent_indices"]), children_lists=c["children_lists"],
            root_index=c["root_index"], eos_token_id=c["eos_token_id"], do_sample=c["do_sample"],
            threshold=c["threshold"], window_size=c["window_size"], threshold_method=c["threshold_method"])
        exp = c["expected"]
        assert sampled.tolist() == exp["sampled"], c["test"]
        assert hidden.tolist() == exp["hidden"], c["test"]
        assert acc == exp["accept_len"], c["test"]
        for key, val in exp["log_data"].items():
            got = wandb_logger.log_data[key]
            if isinstance(val, str):
                assert got == val, (c["test"], key)
            else:
                assert got == pytest.approx(val, rel=1e-6, abs=1e-7), (c["test"], key)


def test_golden_verify_tree(cuda_lib):
    """verify_tree on the GPU reproduces what the reference returned for every golden case, bit for bit."""
    bad = []
    for case in golden_io.verify_cases():
        if not case["upcast_agrees"]:
            continue
        st, logits = golden_io.verify_input(case)
        toks, hidden, (total, acc) = verify_tree(
            tree=_tree_of(st), root_ind=case["root_ind"], logits=logits.unsqueeze(0).cuda(), eos_token_id=case["eos"],
            logits_processor=None, do_sample=False, skip_nodes=case["skip_nodes"], verify_method=case["method"],
            verify_kwargs=case["kwargs"])
        got = dict(tokens=toks.squeeze(0).tolist(), hidden=hidden.tolist(), total_len=total, accept_len=acc)
        if got != case["expected"]:
            bad.append((case["name"], got, case["expected"]))
    assert not bad, bad[:3]


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16, torch.float16])
def test_entropy_and_probabilities_match_fp32_oracle(cuda_lib, dtype):
    """Entropy and P[parent, child token] within 1e-5 relative of the fp32 oracle (the stated tolerance)."""
    from subspec_b200 import _lib
    from subspec_b200.verify import get_workspace, flatten_tree

    st, logits = synthetic.config1_case(77, dtype=dtype, peaked=True)
    tree = _tree_of(st)
    tok, off, idx = flatten_tree(tree, 0, limit=st.n, restrict=True)
    ws = get_workspace(1, st.n, torch.device("cuda", 0))
    ws.set_trees([(tok, off, idx, st.n, 0)])
    ws.run(logits.unsqueeze(0).cuda(), input_kind=_lib.IN_LOGITS, method=_lib.VERIFY_LOSSY, gate=_lib.GATE_ENTROPY,
           threshold=0.3, window=6)
    out = ws.fetch()
    # Exact (fp64) entropy and probabilities of the fp32-upcast logits.  The reference's own fp32 pipeline
    # (torch softmax, entr, sum) sits up to ~5e-5 relative away from these on the same rows, so they, not the
    # fp32 reference values, are the yardstick; the stated tolerance is 1e-5 relative (plus 2e-6 absolute on a
    # quantity that lives in [0, 1] and is compared with thresholds around 0.3).
    probs = torch.softmax(logits.double(), dim=-1)
    ent = torch.tensor(vo.normalised_entropy(probs), dtype=torch.float64)
    got_ent = torch.from_numpy(out["node_entropy"][0, :st.n]).double()
    assert torch.allclose(got_ent, ent, rtol=1e-5, atol=2e-6), (got_ent - ent).abs().max()
    ref32 = torch.tensor(vo.normalised_entropy(vo.target_probs(logits, upcast=True)), dtype=torch.float64)
    assert (got_ent - ent).abs().max() <= (ref32 - ent).abs().max() + 2e-6  # no worse than the fp32 reference path
    assert out["node_target"][0, :st.n].tolist() == probs.argmax(-1).tolist()
    par = st.parents.tolist()
    for c in range(1, st.n):
        ref = float(probs[par[c], int(st.token_ids[c])])
        assert out["node_child_prob"][0, c] == pytest.approx(ref, rel=1e-5, abs=1e-30)


def test_batched_equals_per_sequence(cuda_lib):
    """A batch in one launch gives, per sequence, what the single-sequence call gives (and the oracle)."""
    B, vocab, n = 12, 4099, 33  # vocab not a multiple of 8: exercises the unaligned row path
    gen = torch.Generator().manual_seed(5)
    sts = [synthetic.random_tree(n - (b % 3), 6, 4, vocab, gen) for b in range(B)]
    logits = torch.zeros(B, n, vocab, dtype=torch.bfloat16)
    for b, st in enumerate(sts):
        logits[b, :st.n] = synthetic.verify_logits(st, vocab, gen, dtype=torch.bfloat16, peaked=True)
    trees = [_tree_of(st) for st in sts]
    for method, kw in [("exact", {}), ("lossy", {"threshold_method": "entropy", "threshold": 0.3, "window_size": 1}),
                       ("lossy", {"threshold_method": "prob", "threshold": 0.1, "window_size": 0})]:
        res = verify_tree_batched(trees=trees, root_inds=[0] * B, logits=logits.cuda(), eos_token_id=None,
                                  verify_method=method, verify_kwargs=kw)
        for b, st in enumerate(sts):
            r = vo.verify(logits=logits[b, :st.n], token_ids=st.token_ids.tolist(), children=st.children(),
                          method=method, threshold=kw.get("threshold", 0.0), window=kw.get("window_size", 1),
                          threshold_method=kw.get("threshold_method", "prob"), upcast=True)
            assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens, (method, b)
            assert res[b].hidden_indices.tolist() == r.hidden, (method, b)
            assert (res[b].total_len, res[b].accept_len) == (r.total_len, r.accept_len)


def test_edge_cases(cuda_lib):
    # a single root node: no children, the only output is the bonus token
    t = Tree(torch.tensor(3))
    logits = torch.randn(1, 1, 17)
    toks, hidden, (total, acc) = verify_tree(tree=t, root_ind=0, logits=logits, eos_token_id=None,
                                             logits_processor=None, do_sample=False)
    assert toks.tolist() == [[int(logits[0, 0].argmax())]] and hidden.tolist() == [0] and (total, acc) == (0, 0)
    # argmax ties resolve to the first index, as torch.argmax does
    logits = torch.zeros(1, 1, 40)
    logits[0, 0, 7] = logits[0, 0, 31] = 2.0
    toks, _, _ = verify_tree(tree=t, root_ind=0, logits=logits, eos_token_id=None, logits_processor=None,
                             do_sample=False, verify_method="lossy")
    assert toks.tolist() == [[7]]
    # -inf (masked) logits do not poison the entropy
    logits = torch.full((1, 1, 64), float("-inf"))
    logits[0, 0, 5], logits[0, 0, 9] = 1.0, 1.0
    st = synthetic.SynthTree(torch.tensor([0, 5]), torch.tensor([-1, 0]), torch.tensor([0, 1]))
    toks, hidden, (total, acc) = verify_tree(tree=_tree_of(st), root_ind=0, logits=logits.expand(1, 2, 64).contiguous(),
                                             eos_token_id=None, logits_processor=None, do_sample=False,
                                             verify_method="lossy",
                                             verify_kwargs={"threshold_method": "entropy", "threshold": 0.5,
                                                            "window_size": 0})
    assert toks.tolist() == [[5, 5]] and acc == 1
    with pytest.raises(ValueError):
        verify_tree(tree=t, root_ind=0, logits=torch.randn(1, 1, 17), eos_token_id=None, logits_processor=None,
                    do_sample=False, verify_method="nonsense")
    # an out-of-vocabulary draft token is reported, not read
    st = synthetic.SynthTree(torch.tensor([0, 99]), torch.tensor([-1, 0]), torch.tensor([0, 1]))
    with pytest.raises(ValueError):
        verify_tree(tree=_tree_of(st), root_ind=0, logits=torch.randn(1, 2, 17), eos_token_id=None,
                    logits_processor=None, do_sample=False, verify_method="lossy")


def _sampled_case(seed, batch, nodes, vocab, dtype, sigma):
    gen = torch.Generator().manual_seed(seed)
    sts = [synthetic.random_tree(nodes, 10, 8, vocab, gen) for _ in range(batch)]
    logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=dtype, sigma=sigma, boost=6.0) for st in sts])
    uniforms = torch.rand(batch, nodes, generator=gen)
    return sts, logits, uniforms


@pytest.mark.parametrize("vocab,nodes,dtype,temperature,top_p", [
    (152064, 24, torch.bfloat16, 1.0, 0.9),   # config-2 distribution at reduced node count
    (32000, 40, torch.float16, 0.7, 0.95),
    (4099, 33, torch.bfloat16, 1.3, 1.0),     # no nucleus filter, unaligned rows
    (50, 12, torch.bfloat16, 1.0, 0.5),       # tiny vocabulary: heavy ties at the boundary
])
def test_stochastic_sample_and_match(cuda_lib, vocab, nodes, dtype, temperature, top_p):
    """Sampled targets (temperature, nucleus, injected uniforms) and the sample-and-match walk vs the oracle."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopPLogitsWarper)
    B = 3
    sts, logits, uniforms = _sampled_case(500 + nodes, B, nodes, vocab, dtype, 2.5)
    procs = LogitsProcessorList()
    if temperature != 1.0:
        procs.append(TemperatureLogitsWarper(temperature))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    res = verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                              eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="stochastic",
                              uniforms=uniforms, verify_kwargs={"sample_all_nodes": True})
    from subspec_b200.verify import get_workspace
    targets = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_target"]
    decided_by_rounding = 0
    for b, st in enumerate(sts):
        probs = vo.target_probs(logits[b], True, temperature, top_p, upcast=True)
        want = vo.target_tokens(probs, True, uniforms[b].tolist())
        margins = vo.sampling_margins(logits[b], temperature, top_p, uniforms[b].tolist())
        safe = [mb > 1e-3 and mp > 1e-6 for mb, mp in margins]
        decided_by_rounding += safe.count(False)
        for u in range(st.n):
            if safe[u]:
                assert int(targets[b, u]) == want[u], (b, u, margins[u])
        # the walk itself is integer work: replay it on the kernel's own targets
        r = vo.exact_walk(target=targets[b, :st.n].tolist(), token_ids=st.token_ids.tolist(), children=st.children(),
                          root=0, n_rows=st.n, eos=None)
        assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens
        assert res[b].hidden_indices.tolist() == r.hidden
        assert (res[b].total_len, res[b].accept_len) == (r.total_len, r.accept_len)
    assert decided_by_rounding <= max(2, B * nodes // 10)


def test_stochastic_ties_masks_and_zeros(cuda_lib):
    """Rows made of a handful of distinct values (-inf masks, both zeros, long runs of ties): the sampler's
    count histogram, its tie rule (lowest vocabulary index goes first) and the second sweep's value compares."""
    from transformers.generation.logits_process import LogitsProcessorList, TopPLogitsWarper
    vocab, nodes, B = 3000, 16, 2
    gen = torch.Generator().manual_seed(77)
    sts = [synthetic.random_tree(nodes, 6, 4, vocab, gen) for _ in range(B)]
    levels = torch.tensor([float("-inf"), -3.0, -0.0, 0.0, 0.5, 1.0, 2.5, 4.0])
    weights = torch.tensor([0.3, 0.2, 0.1, 0.1, 0.15, 0.1, 0.04, 0.01])
    idx = torch.multinomial(weights, B * nodes * vocab, replacement=True, generator=gen).reshape(B, nodes, vocab)
    logits = levels[idx].to(torch.bfloat16)
    logits[:, :, 7] = 4.0  # never a row without a finite value
    uniforms = torch.rand(B, nodes, generator=gen)
    checked = 0
    # the ascending cumulative probability passes 1 - top_p inside the run of -3s, of 0.5s, of 2.5s, of 4s;
    # with 0.9 it passes inside the run of zeros, where the kernel orders -0 before +0 and a stable sort on
    # values does not: there only what both agree on is checked (nothing at or below -3 survives)
    for top_p in (0.999, 0.8, 0.5, 0.05, 0.9):
        procs = LogitsProcessorList([TopPLogitsWarper(top_p=top_p)])
        verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                            eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="stochastic",
                            uniforms=uniforms, verify_kwargs={"sample_all_nodes": True})
        from subspec_b200.verify import get_workspace
        targets = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_target"]
        for b, st in enumerate(sts):
            probs = vo.target_probs(logits[b], True, 1.0, top_p, upcast=True)
            want = vo.target_tokens(probs, True, uniforms[b].tolist())
            margins = vo.sampling_margins(logits[b], 1.0, top_p, uniforms[b].tolist())
            for u in range(st.n):
                assert float(logits[b, u, int(targets[b, u])]) > float("-inf")  # never a masked token
                if top_p == 0.9:
                    assert float(logits[b, u, int(targets[b, u])]) >= 0.0
                elif margins[u][0] > 1e-3 and margins[u][1] > 1e-6:
                    assert int(targets[b, u]) == want[u], (top_p, b, u, margins[u])
                    checked += 1
    assert checked >= B * nodes * 2
    # the same rows through the lossy verifier: a child whose token sits in the run of equal values that the
    # nucleus boundary cuts has probability e/Z or 0 according to its place in that run
    cut_children = 0
    for top_p in (0.999, 0.8, 0.5):
        procs = LogitsProcessorList([TopPLogitsWarper(top_p=top_p)])
        verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                            eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="lossy",
                            verify_kwargs={"threshold_method": "prob", "threshold": 0.01, "window_size": 0},
                            uniforms=uniforms)
        cprob = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_child_prob"]
        for b, st in enumerate(sts):
            probs = vo.target_probs(logits[b], True, 1.0, top_p, upcast=True)
            margins = vo.sampling_margins(logits[b], 1.0, top_p, uniforms[b].tolist())
            ch = st.children()
            for u in range(st.n):
                if margins[u][0] <= 1e-3:
                    continue
                row = logits[b, u].float()
                kept = row[probs[u] > 0]
                for c in ch[u]:
                    tok = int(st.token_ids[c])
                    want, got = float(probs[u, tok]), float(cprob[b, c])
                    assert (want == 0.0) == (got == 0.0) and abs(got - want) <= 2e-4 * want, (top_p, b, u, c, got, want)
                    cut_children += int(float(row[tok]) == float(kept.min()) and bool((row == row[tok]).sum() > (kept == kept.min()).sum()))
    assert cut_children > 0  # the partial-run path was exercised


def test_stochastic_counter_overflow_is_reported(cuda_lib):
    """More than 65535 equal finite values in one row do not fit the sampler's 16-bit counters: reported."""
    vocab, nodes = 70016, 2
    st = synthetic.SynthTree(torch.tensor([0, 5]), torch.tensor([-1, 0]), torch.tensor([0, 1]))
    for copies in (65536, 66000):
        logits = torch.randn(1, nodes, vocab).to(torch.bfloat16)
        logits[0, 1, :copies] = 0.75
        with pytest.raises(ValueError, match="65535"):
            verify_tree_batched(trees=[_tree_of(st)], root_inds=[0], logits=logits.cuda(), eos_token_id=None,
                                logits_processor=None, do_sample=True, verify_method="stochastic",
                                uniforms=torch.rand(1, nodes), verify_kwargs={"sample_all_nodes": True})
    # exactly 65535 copies still fit
    logits = torch.randn(1, nodes, vocab).to(torch.bfloat16)
    logits[0, 1, :65535] = 0.75
    logits[0, 1, 65535:][logits[0, 1, 65535:] == 0.75] = 0.5
    verify_tree_batched(trees=[_tree_of(st)], root_inds=[0], logits=logits.cuda(), eos_token_id=None,
                        logits_processor=None, do_sample=True, verify_method="stochastic", uniforms=torch.rand(1, nodes),
                        verify_kwargs={"sample_all_nodes": True})


@pytest.mark.parametrize("vocab,nodes,dtype,temperature,top_k,top_p", [
    (32000, 20, torch.float16, 0.8, 50, 1.0),      # top-k alone
    (152064, 12, torch.bfloat16, 1.0, 40, 0.9),    # the reference's usual trio: temperature, top-k, top-p
    (4099, 16, torch.bfloat16, 1.2, 1, 1.0),       # k = 1: greedy by another name
    (5000, 16, torch.bfloat16, 1.0, 100000, 0.7),  # k beyond the vocabulary: no cut
])
def test_stochastic_top_k(cuda_lib, vocab, nodes, dtype, temperature, top_k, top_p):
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    from subspec_b200.verify import get_workspace
    B = 2
    sts, logits, uniforms = _sampled_case(900 + nodes, B, nodes, vocab, dtype, 2.5)
    procs = LogitsProcessorList()
    if temperature != 1.0:
        procs.append(TemperatureLogitsWarper(temperature))
    procs.append(TopKLogitsWarper(top_k=top_k))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(), eos_token_id=None,
                        logits_processor=procs, do_sample=True, verify_method="stochastic", uniforms=uniforms,
                        verify_kwargs={"sample_all_nodes": True})
    targets = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_target"]
    checked = 0
    for b, st in enumerate(sts):
        probs = vo.target_probs(logits[b], True, temperature, top_p, upcast=True, top_k=min(top_k, vocab))
        want = vo.target_tokens(probs, True, uniforms[b].tolist())
        margins = vo.sampling_margins(logits[b], temperature, top_p, uniforms[b].tolist(), top_k=min(top_k, vocab))
        for u in range(st.n):
            assert float(probs[u, int(targets[b, u])]) > 0.0  # never a token the filters removed
            if margins[u][0] > 1e-3 and margins[u][1] > 1e-6:
                assert int(targets[b, u]) == want[u], (b, u, margins[u])
                checked += 1
    assert checked >= B * nodes // 2
    with pytest.raises(ValueError):  # the reference's order is temperature, top-k, top-p
        verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                            eos_token_id=None, do_sample=True, verify_method="stochastic", uniforms=uniforms,
                            logits_processor=LogitsProcessorList([TopPLogitsWarper(top_p=0.9),
                                                                  TopKLogitsWarper(top_k=5)]))


@pytest.mark.parametrize("gate,threshold", [("entropy", 0.25), ("prob", 0.02)])
@pytest.mark.parametrize("dtype,top_k,top_p", [(torch.bfloat16, 0, 0.9), (torch.float16, 64, 0.95),
                                               (torch.bfloat16, 0, 1.0)])
def test_lossy_on_sampled_targets(cuda_lib, dtype, top_k, top_p, gate, threshold):
    """verify_method='lossy' with do_sample: sampled targets, and the gates (entropy of the filtered
    distribution, filtered probability of the child token) as lossy_tree_verify.py:66-77, 135-146 computes them
    from the processed probabilities."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    from subspec_b200.verify import get_workspace
    B, nodes, vocab, temperature = 3, 24, 32000, 0.9
    sts, logits, uniforms = _sampled_case(1300 + top_k, B, nodes, vocab, dtype, 2.0)
    procs = LogitsProcessorList([TemperatureLogitsWarper(temperature)])
    if top_k:
        procs.append(TopKLogitsWarper(top_k=top_k))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    kw = {"threshold_method": gate, "threshold": threshold, "window_size": 1}
    res = verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                              eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="lossy",
                              verify_kwargs=kw, uniforms=uniforms)
    out = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()
    for b, st in enumerate(sts):
        probs = vo.target_probs(logits[b], True, temperature, top_p, upcast=True, top_k=top_k)
        ent = torch.tensor(vo.normalised_entropy(probs))
        assert torch.allclose(torch.from_numpy(out["node_entropy"][b, :st.n].copy()), ent, rtol=2e-4, atol=2e-6)
        ch = st.children()
        for u in range(st.n):
            for c in ch[u]:
                want = float(probs[u, int(st.token_ids[c])])
                got = float(out["node_child_prob"][b, c])
                assert (want == 0.0) == (got == 0.0) and abs(got - want) <= 2e-4 * want + 1e-9, (b, u, c, got, want)
        # the DP and the walk are integer work on top of these: replay them on the kernel's own targets and gates
        r = vo.lossy_verify(probs=probs, token_ids=st.token_ids.tolist(), children=ch, root=0, eos=None,
                            threshold=threshold, window=1, use_entropy=gate == "entropy",
                            target=out["node_target"][b, :st.n].tolist())
        if r.min_gate_margin > 1e-4:  # no gate decision within rounding of its threshold
            assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens
            assert res[b].hidden_indices.tolist() == r.hidden
            assert (res[b].total_len, res[b].accept_len) == (r.total_len, r.accept_len)


@pytest.mark.parametrize("dtype,vocab", [(torch.bfloat16, 152064), (torch.float32, 4099), (torch.float16, 32000)])
@pytest.mark.parametrize("gate,threshold,window", [("entropy", 0.3, 6), ("prob", 0.05, 1), ("entropy", 0.9, 0)])
def test_exact_and_lossy_in_one_pass(cuda_lib, dtype, vocab, gate, threshold, window):
    """verify_method='exact+lossy' (one pass over the logits) returns exactly what the two separate calls return."""
    B, nodes = 5, 48
    gen = torch.Generator().manual_seed(4242 + vocab)
    sts = [synthetic.random_tree(nodes, 8, 4, vocab, gen) for _ in range(B)]
    logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=dtype, sigma=3.0, boost=18.0) for st in sts])
    kw = {"threshold_method": gate, "threshold": threshold, "window_size": window}
    trees = [_tree_of(st) for st in sts]
    common = dict(trees=trees, root_inds=[0] * B, logits=logits.cuda(), eos_token_id=int(sts[0].token_ids[3]),
                  logits_processor=None, do_sample=False)
    exact = verify_tree_batched(verify_method="exact", **common)
    lossy = verify_tree_batched(verify_method="lossy", verify_kwargs=kw, **common)
    both = verify_tree_batched(verify_method="exact+lossy", verify_kwargs=kw, **common)
    accepted = 0
    for b in range(B):
        for got, want in ((both[b][0], exact[b]), (both[b][1], lossy[b])):
            assert got.sampled_tokens.tolist() == want.sampled_tokens.tolist()
            assert got.hidden_indices.tolist() == want.hidden_indices.tolist()
            assert (got.total_len, got.accept_len) == (want.total_len, want.accept_len)
        accepted += lossy[b].accept_len
    assert accepted > 0
    # a partially decoded tree cannot share one flattening between the two walks
    with pytest.raises(ValueError):
        verify_tree_batched(trees=trees, root_inds=[0] * B, logits=logits[:, :nodes - 3].cuda(), eos_token_id=None,
                            logits_processor=None, do_sample=False, verify_method="exact+lossy", verify_kwargs=kw)


@pytest.mark.parametrize("vocab,nodes,dtype,temperature,top_k,top_p", [
    (152064, 40, torch.bfloat16, 1.0, 0, 0.9), (32000, 64, torch.float16, 0.8, 50, 0.95), (4099, 24, torch.bfloat16, 1.0, 0, 1.0)])
def test_stochastic_walk_samples_only_where_it_stands(cuda_lib, vocab, nodes, dtype, temperature, top_k, top_p):
    """Default stochastic verification draws only at the contexts the walk visits (as the reference's walker
    does): same tokens, contexts and lengths as drawing at every node, and the draws it does make are the same."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    from subspec_b200.verify import get_workspace
    B = 6
    gen = torch.Generator().manual_seed(77 + nodes)
    sts = [synthetic.random_tree(nodes, 10, 6, vocab, gen) for _ in range(B)]
    logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=dtype, sigma=2.5, boost=14.0) for st in sts])
    uniforms = torch.rand(B, nodes, generator=gen)
    procs = LogitsProcessorList()
    if temperature != 1.0:
        procs.append(TemperatureLogitsWarper(temperature))
    if top_k:
        procs.append(TopKLogitsWarper(top_k=top_k))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    common = dict(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                  eos_token_id=int(sts[0].token_ids[2]), logits_processor=procs, do_sample=True,
                  verify_method="stochastic", uniforms=uniforms)
    full = verify_tree_batched(verify_kwargs={"sample_all_nodes": True}, **common)
    t_full = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_target"].copy()
    lazy = verify_tree_batched(**common)
    t_lazy = get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_target"].copy()
    accepted = 0
    for b in range(B):
        assert lazy[b].sampled_tokens.tolist() == full[b].sampled_tokens.tolist()
        assert lazy[b].hidden_indices.tolist() == full[b].hidden_indices.tolist()
        assert (lazy[b].total_len, lazy[b].accept_len) == (full[b].total_len, full[b].accept_len)
        visited = set(lazy[b].hidden_indices.tolist())
        for u in range(sts[b].n):
            if u in visited:
                assert t_lazy[b, u] == t_full[b, u]
            else:
                assert t_lazy[b, u] == -1
        accepted += lazy[b].accept_len
    assert accepted > 0


@pytest.mark.parametrize("vocab,nodes,dtype,temperature,top_k,top_p,draft_t", [
    (4099, 24, torch.bfloat16, 1.0, 0, 1.0, 1.0), (32000, 32, torch.float16, 0.8, 0, 0.9, 1.2),
    (152064, 20, torch.bfloat16, 1.0, 50, 0.9, 1.0)])
def test_residual_acceptance(cuda_lib, vocab, nodes, dtype, temperature, top_k, top_p, draft_t):
    """verify_kwargs={'acceptance': 'residual'}: accept child c with probability min(1, p'(x)/q(x)), subtract q
    from p' after a rejection, draw the bonus from p'.  Against the fp64 restatement (no reference counterpart)."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    B = 8
    gen = torch.Generator().manual_seed(31 + nodes)
    sts = [synthetic.random_tree(nodes, 8, 4, vocab, gen) for _ in range(B)]
    target = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=dtype, sigma=2.0, boost=11.0) for st in sts])
    # a draft that resembles the target, with its own noise, and that also likes the drafted tokens
    draft = (target.float() * 0.7 + torch.randn(target.shape, generator=gen) * 1.0).to(dtype)
    u_draw = torch.rand(B, nodes, generator=gen)
    u_acc = torch.rand(B, nodes, generator=gen)
    procs = LogitsProcessorList()
    if temperature != 1.0:
        procs.append(TemperatureLogitsWarper(temperature))
    if top_k:
        procs.append(TopKLogitsWarper(top_k=top_k))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    res = verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=target.cuda(),
                              eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="stochastic",
                              verify_kwargs={"acceptance": "residual", "draft_temperature": draft_t},
                              draft_logits=draft.cuda(), uniforms=u_draw, accept_uniforms=u_acc)
    checked = accepted = 0
    trace = {"accept_after_reject": 0, "residual_bonus": 0}
    for b, st in enumerate(sts):
        tr = {}
        r, margin = vo.residual_walk(logits=target[b], draft_logits=draft[b], token_ids=st.token_ids.tolist(),
                                     children=st.children(), accept_uniforms=u_acc[b].tolist(),
                                     uniforms=u_draw[b].tolist(), temperature=temperature, top_p=top_p, top_k=top_k,
                                     draft_temperature=draft_t, trace=tr)
        if margin > 1e-4:  # no accept test or draw within rounding of its threshold
            assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens, (b, margin)
            assert res[b].hidden_indices.tolist() == r.hidden
            assert (res[b].total_len, res[b].accept_len) == (r.total_len, r.accept_len)
            checked += 1
            accepted += r.accept_len
            for key in trace:
                trace[key] += tr[key]
    assert checked >= B // 2 and accepted > 0
    # the branches that set this rule apart from sample-and-match were taken
    assert trace["accept_after_reject"] > 0 and trace["residual_bonus"] > 0, trace
    one = verify_tree(tree=_tree_of(sts[0]), root_ind=0, logits=target[:1].cuda(), eos_token_id=None,
                      logits_processor=procs, do_sample=True, verify_method="stochastic",
                      verify_kwargs={"acceptance": "residual", "draft_temperature": draft_t},
                      draft_logits=draft[0].cuda(), uniforms=u_draw[0], accept_uniforms=u_acc[0])
    assert one[0].squeeze(0).tolist() == res[0].sampled_tokens.squeeze(0).tolist() and one[2][1] == res[0].accept_len
    with pytest.raises(ValueError):  # residual acceptance needs the draft's logits
        verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=target.cuda(),
                            eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="stochastic",
                            verify_kwargs={"acceptance": "residual"})


def _wide_targets(B, nodes):
    from subspec_b200.verify import get_workspace
    return get_workspace(B, nodes, torch.device("cuda", 0)).fetch()["node_target"]


@pytest.mark.parametrize("vocab,nodes,temperature,top_k,top_p", [
    (4099, 20, 1.0, 0, 0.9), (32000, 16, 0.7, 50, 0.95), (152064, 6, 1.0, 0, 1.0), (50, 12, 1.3, 8, 0.5),
    (32000, 10, 1.0, 200, 1.0)])
def test_stochastic_fp32_logits(cuda_lib, vocab, nodes, temperature, top_k, top_p):
    """fp32 logits have no 16-bit histogram: the filters' boundaries come from searches over the key space.
    Same semantics, same oracle, same margins as the 16-bit pipeline; both the every-row and the walk-driven
    launch."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    B = 3
    sts, logits, uniforms = _sampled_case(900 + nodes, B, nodes, vocab, torch.float32, 2.5)
    procs = LogitsProcessorList()
    if temperature != 1.0:
        procs.append(TemperatureLogitsWarper(temperature))
    if top_k:
        procs.append(TopKLogitsWarper(top_k=top_k))
    if top_p < 1.0:
        procs.append(TopPLogitsWarper(top_p=top_p))
    kw = dict(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(), eos_token_id=None,
              logits_processor=procs, do_sample=True, verify_method="stochastic", uniforms=uniforms)
    res = verify_tree_batched(verify_kwargs={"sample_all_nodes": True}, **kw)
    targets = _wide_targets(B, nodes).copy()
    checked = 0
    for b, st in enumerate(sts):
        probs = vo.target_probs(logits[b], True, temperature, top_p, upcast=True, top_k=top_k)
        want = vo.target_tokens(probs, True, uniforms[b].tolist())
        margins = vo.sampling_margins(logits[b], temperature, top_p, uniforms[b].tolist(), top_k=top_k)
        for u in range(st.n):
            if margins[u][0] > 1e-3 and margins[u][1] > 1e-6:
                assert int(targets[b, u]) == want[u], (b, u, margins[u])
                checked += 1
        r = vo.exact_walk(target=targets[b, :st.n].tolist(), token_ids=st.token_ids.tolist(), children=st.children(),
                          root=0, n_rows=st.n, eos=None)
        assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens
        assert res[b].hidden_indices.tolist() == r.hidden
    assert checked >= B * nodes * 8 // 10
    lazy = verify_tree_batched(**kw)  # only the contexts the walk stands on
    visited = _wide_targets(B, nodes)
    for b in range(B):
        assert lazy[b].sampled_tokens.tolist() == res[b].sampled_tokens.tolist()
        assert lazy[b].hidden_indices.tolist() == res[b].hidden_indices.tolist()
        seen = visited[b] >= 0
        assert 1 <= int(seen.sum()) <= res[b].accept_len + 1
        assert (visited[b][seen] == targets[b][seen]).all()


def test_stochastic_fp32_ties_and_masks(cuda_lib):
    """fp32 rows made of a few distinct values: the top-p boundary falls inside long runs of ties (cut in
    vocabulary order), -inf masks carry no mass, top-k keeps every tie of the k-th value."""
    from transformers.generation.logits_process import LogitsProcessorList, TopKLogitsWarper, TopPLogitsWarper
    vocab, nodes, B = 3000, 12, 2
    gen = torch.Generator().manual_seed(78)
    sts = [synthetic.random_tree(nodes, 6, 4, vocab, gen) for _ in range(B)]
    levels = torch.tensor([float("-inf"), -3.0, -1.0, 0.25, 0.5, 1.0, 2.5, 4.0])
    weights = torch.tensor([0.3, 0.2, 0.1, 0.1, 0.15, 0.1, 0.04, 0.01])
    idx = torch.multinomial(weights, B * nodes * vocab, replacement=True, generator=gen).reshape(B, nodes, vocab)
    logits = levels[idx].to(torch.float32)
    logits[:, :, 7] = 4.0
    uniforms = torch.rand(B, nodes, generator=gen)
    checked = 0
    for top_k, top_p in ((0, 0.999), (0, 0.8), (0, 0.5), (0, 0.05), (100, 1.0), (400, 0.7)):
        procs = LogitsProcessorList(([TopKLogitsWarper(top_k=top_k)] if top_k else []) +
                                    ([TopPLogitsWarper(top_p=top_p)] if top_p < 1.0 else []))
        verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                            eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="stochastic",
                            uniforms=uniforms, verify_kwargs={"sample_all_nodes": True})
        targets = _wide_targets(B, nodes)
        for b, st in enumerate(sts):
            probs = vo.target_probs(logits[b], True, 1.0, top_p, upcast=True, top_k=top_k)
            want = vo.target_tokens(probs, True, uniforms[b].tolist())
            margins = vo.sampling_margins(logits[b], 1.0, top_p, uniforms[b].tolist(), top_k=top_k)
            for u in range(st.n):
                assert float(logits[b, u, int(targets[b, u])]) > float("-inf")
                if margins[u][0] > 1e-3 and margins[u][1] > 1e-6:
                    assert int(targets[b, u]) == want[u], (top_k, top_p, b, u, margins[u])
                    checked += 1
    assert checked >= B * nodes * 4


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("gate,threshold,window", [("entropy", 0.3, 1), ("prob", 0.05, 0)])
def test_lossy_on_probabilities_with_sampled_targets(cuda_lib, dtype, gate, threshold, window):
    """lossy_bottom_up_verify(probs=..., do_sample=True): the reference draws torch.multinomial(probs)
    (lossy_tree_verify.py:75-77); here the draw is the inverse-CDF pick for injected uniforms, the gates use
    the probabilities as given."""
    vocab, nodes = 4099, 24
    gen = torch.Generator().manual_seed(41)
    checked = accepted = 0
    for trial in range(4):
        st = synthetic.random_tree(nodes, 6, 4, vocab, gen)
        logits = synthetic.verify_logits(st, vocab, gen, dtype=torch.float32, sigma=2.0, boost=14.0)
        probs = torch.softmax(logits, dim=-1).to(dtype)
        u = torch.rand(nodes, generator=gen)
        sampled, hidden, acc = lossy_bottom_up_verify(
            probs=probs.cuda(), token_ids=st.token_ids, parent_indices=st.parents, children_lists=st.children(),
            root_index=0, eos_token_id=None, do_sample=True, threshold=threshold, window_size=window,
            threshold_method=gate, uniforms=u)
        cdf = probs.double().cumsum(-1)
        tot = cdf[:, -1:]
        pick_margin = float(((cdf - u.double().unsqueeze(1) * tot).abs() / tot).min())
        r = vo.verify(logits=probs.float(), token_ids=st.token_ids.tolist(), children=st.children(), method="lossy",
                      do_sample=True, uniforms=u.tolist(), threshold=threshold, window=window,
                      threshold_method=gate, input_is_probs=True)
        if pick_margin > 1e-6 and r.min_gate_margin > 1e-5:
            assert sampled.tolist() == r.tokens, (trial, pick_margin)
            assert hidden.tolist() == r.hidden and acc == r.accept_len
            checked += 1
            accepted += acc
    assert checked >= 3 and accepted > 0


@pytest.mark.parametrize("gate,threshold", [("entropy", 0.25), ("prob", 0.02)])
def test_lossy_on_sampled_targets_fp32_logits(cuda_lib, gate, threshold):
    """fp32 logits, lossy verification with sampled targets and a temperature (no top-k / top-p: those need the
    16-bit pipeline for the gates and are refused)."""
    from transformers.generation.logits_process import LogitsProcessorList, TemperatureLogitsWarper, TopPLogitsWarper
    B, vocab, nodes, temperature = 4, 4099, 24, 0.8
    gen = torch.Generator().manual_seed(43)
    sts = [synthetic.random_tree(nodes, 6, 4, vocab, gen) for _ in range(B)]
    logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=torch.float32, sigma=2.0, boost=14.0)
                          for st in sts])
    uniforms = torch.rand(B, nodes, generator=gen)
    kw = {"threshold_method": gate, "threshold": threshold, "window_size": 1}
    res = verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                              eos_token_id=None, logits_processor=LogitsProcessorList([TemperatureLogitsWarper(temperature)]),
                              do_sample=True, verify_method="lossy", verify_kwargs=kw, uniforms=uniforms)
    checked = 0
    for b, st in enumerate(sts):
        r = vo.verify(logits=logits[b], token_ids=st.token_ids.tolist(), children=st.children(), method="lossy",
                      do_sample=True, temperature=temperature, uniforms=uniforms[b].tolist(), threshold=threshold,
                      window=1, threshold_method=gate, upcast=True)
        margins = vo.sampling_margins(logits[b], temperature, 1.0, uniforms[b].tolist())
        if min(m[1] for m in margins) > 1e-6 and r.min_gate_margin > 1e-5:
            assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens, b
            assert res[b].hidden_indices.tolist() == r.hidden and res[b].accept_len == r.accept_len
            checked += 1
    assert checked >= B // 2
    # with top-k / top-p the gates use the filtered distribution; the sampler computes them itself
    from transformers.generation.logits_process import TopKLogitsWarper
    checked = accepted = 0
    for top_k, top_p in ((0, 0.9), (64, 0.95), (200, 1.0)):
        procs = LogitsProcessorList([TemperatureLogitsWarper(temperature)] +
                                    ([TopKLogitsWarper(top_k=top_k)] if top_k else []) +
                                    ([TopPLogitsWarper(top_p=top_p)] if top_p < 1.0 else []))
        res = verify_tree_batched(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(),
                                  eos_token_id=None, logits_processor=procs, do_sample=True, verify_method="lossy",
                                  verify_kwargs=kw, uniforms=uniforms)
        for b, st in enumerate(sts):
            r = vo.verify(logits=logits[b], token_ids=st.token_ids.tolist(), children=st.children(), method="lossy",
                          do_sample=True, temperature=temperature, top_p=top_p, top_k=top_k,
                          uniforms=uniforms[b].tolist(), threshold=threshold, window=1, threshold_method=gate,
                          upcast=True)
            margins = vo.sampling_margins(logits[b], temperature, top_p, uniforms[b].tolist(), top_k=top_k)
            if (min(m[0] for m in margins) > 1e-3 and min(m[1] for m in margins) > 1e-6 and
                    r.min_gate_margin > 1e-5):
                assert res[b].sampled_tokens.squeeze(0).tolist() == r.tokens, (top_k, top_p, b)
                assert res[b].hidden_indices.tolist() == r.hidden and res[b].accept_len == r.accept_len
                checked += 1
                accepted += r.accept_len
    assert checked >= 6 and accepted > 0
    with pytest.raises(ValueError):  # probabilities in are drawn from as they are: no filter to apply
        lossy = _lib_probs_with_filter(sts[0], logits[0])


def test_golden_sampled_verification(cuda_lib):
    """The reference's own results with do_sample=True (its warpers, softmax, walk and lossy verifier; its
    torch.multinomial replaced by the inverse-CDF pick for injected uniforms) against the CUDA path: every case
    whose outcome does not hang on 16-bit rounding of the probabilities (the kernel computes them in fp32) or
    on a uniform within rounding of a CDF edge."""
    checked = {"exact": 0, "lossy": 0}
    accepted = 0
    left_out = {"sixteen_bit_probabilities": 0, "margins": 0}
    for c in golden_io.sampled_cases():
        decided = (c["upcast_agrees"] and c["boundary_margin"] > 1e-3 and c["pick_margin"] > 1e-6 and
                   (c["gate_margin"] is None or c["gate_margin"] > 1e-5))
        if not decided:
            left_out["margins" if c["upcast_agrees"] else "sixteen_bit_probabilities"] += 1
            continue
        tree, logits = golden_io.sampled_input(c)
        modes = [{}] if c["method"] == "lossy" else [{}, {"sample_all_nodes": True}]
        for extra in modes:
            toks, hidden, (total, acc) = verify_tree(
                tree=_tree_of(tree), root_ind=0, logits=logits.unsqueeze(0).cuda(), eos_token_id=None,
                logits_processor=golden_io.sampled_processors(c), do_sample=True, verify_method=c["method"],
                verify_kwargs={**c["kwargs"], **extra}, uniforms=torch.tensor(c["uniforms"]))
            got = dict(tokens=toks.squeeze(0).tolist(), hidden=hidden.tolist(), total_len=total, accept_len=acc)
            assert got == c["expected"], (c["name"], extra)
        checked[c["method"]] += 1
        accepted += c["expected"]["accept_len"]
    assert checked["exact"] >= 45 and checked["lossy"] >= 20 and accepted > 40, (checked, accepted)
    # The cases left out are a stated deviation (fp32 probabilities where the reference keeps 16 bits) and
    # decisions inside rounding distance; their number is pinned so that it cannot grow unnoticed.
    assert len(golden_io.sampled_cases()) == 104
    assert left_out == {"sixteen_bit_probabilities": 5, "margins": 5}, left_out


def _lib_probs_with_filter(st, logits):
    """Probabilities in together with a nucleus filter: refused by the library."""
    from subspec_b200 import _lib
    from subspec_b200.verify import flatten_tree, get_workspace
    tok, off, idx = flatten_tree(_tree_of(st), 0, limit=st.n, restrict=True)
    ws = get_workspace(1, st.n, torch.device("cuda", 0))
    ws.set_trees([(tok, off, idx, st.n, 0)])
    ws.run(torch.softmax(logits, -1).unsqueeze(0).cuda(), input_kind=_lib.IN_PROBS, method=_lib.VERIFY_LOSSY,
           gate=_lib.GATE_PROB, threshold=0.1, window=1, do_sample=1, temperature=1.0, top_p=0.9)


def test_scratch_tickets_are_left_clean(cuda_lib):
    """Every launch leaves its tickets zero, so a caller who vouches for the buffer (SUBSPEC_VERIFY_SCRATCH_CLEAN,
    what VerifyWorkspace does) needs no clearing operation in front of the kernel; without the flag the
    library clears them itself, whatever the buffer holds.  Split rows (few rows) and whole rows (many)."""
    from subspec_b200.verify import VerifyWorkspace
    for B, nodes, vocab in ((1, 12, 50000), (6, 40, 4099)):
        gen = torch.Generator().manual_seed(B)
        sts = [synthetic.random_tree(nodes, 6, 4, vocab, gen) for _ in range(B)]
        logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=torch.bfloat16, peaked=True) for st in sts])
        ws = VerifyWorkspace(B, nodes, torch.device("cuda", 0))
        kw = dict(trees=[_tree_of(st) for st in sts], root_inds=[0] * B, logits=logits.cuda(), eos_token_id=None,
                  verify_method="exact+lossy", verify_kwargs={"threshold_method": "entropy", "threshold": 0.3,
                                                              "window_size": 1}, workspace=ws)
        ws.scratch.fill_(0xFF)
        ws.scratch_clean = False            # garbage in the buffer: the library has to clear the tickets
        want = verify_tree_batched(**kw)
        tickets = 4 * B * (nodes + 1)
        off = ws._scratch_ptr - ws.scratch.data_ptr()
        assert int(ws.scratch[off:off + tickets].max()) == 0   # ... and the launch left them zero
        ws.scratch_clean = True
        for _ in range(3):
            got = verify_tree_batched(**kw)
            for g, w in zip(got, want):
                for x, y in zip(g, w):
                    assert x.sampled_tokens.tolist() == y.sampled_tokens.tolist()
                    assert x.hidden_indices.tolist() == y.hidden_indices.tolist()
                    assert (x.total_len, x.accept_len) == (y.total_len, y.accept_len)
        assert int(ws.scratch[off:off + tickets].max()) == 0


def test_malformed_trees_are_refused_before_any_launch(cuda_lib):
    """Children lists that are not a forest never reach a kernel: the host layer raises ValueError (the walks
    on the device are bounded as well, but no test feeds them a loop)."""
    probs = torch.softmax(torch.randn(4, 30), -1)
    tok = torch.tensor([1, 2, 3, 4])
    kw = dict(probs=probs, token_ids=tok, parent_indices=torch.tensor([-1, 0, 1, 2]), root_index=0,
              eos_token_id=None, do_sample=False, threshold=0.1, window_size=1, threshold_method="prob")
    for bad in ([[1], [2], [3], [1]],      # node 1 reached from 0 and from 3: a loop 1 -> 2 -> 3 -> 1
                [[0], [], [], []],         # a node that is its own child
                [[1], [9], [], []],        # an index outside the tree
                [[1, 2], [2], [], []]):    # a node with two parents
        with pytest.raises(ValueError):
            lossy_bottom_up_verify(children_lists=bad, **kw)
    sampled, hidden, acc = lossy_bottom_up_verify(children_lists=[[1], [2], [3], []], **kw)  # the same call, valid
    assert len(sampled) == acc + 1
    # more decoded rows than nodes, and more than the logits hold
    from subspec_b200.verify import VerifyWorkspace, _children_csr
    from subspec_b200 import _lib
    ws = VerifyWorkspace(1, 8, torch.device("cuda", 0))
    off, idx = _children_csr([[1], [2], [3], []])
    with pytest.raises(ValueError):
        ws.set_trees([(tok.numpy(), off, idx, 5, 0)])
    ws.set_trees([(tok.numpy(), off, idx, 4, 0)])
    with pytest.raises(ValueError):
        ws.run(torch.randn(1, 3, 30, device="cuda"), input_kind=_lib.IN_LOGITS, method=_lib.VERIFY_EXACT)


@pytest.mark.parametrize("method", ["exact", "lossy", "exact+lossy"])
def test_chain_of_1024_nodes(cuda_lib, method):
    """The longest walk the kernels support: a 1024-node chain whose every draft token is the target's choice.
    The walk takes n - 1 steps, exactly the bound the device loops stop at, and the DP n rounds."""
    n, vocab = 1024, 97
    gen = torch.Generator().manual_seed(8)
    tokens = torch.randint(vocab, (n,), generator=gen)
    st = synthetic.SynthTree(tokens, torch.arange(-1, n - 1), torch.arange(n))
    logits = torch.randn(n, vocab, generator=gen)
    for u in range(n - 1):
        logits[u, int(tokens[u + 1])] = 9.0
    kw = {"threshold_method": "entropy", "threshold": 0.3, "window_size": 2}
    res = verify_tree_batched(trees=[_tree_of(st)], root_inds=[0], logits=logits.unsqueeze(0).cuda(),
                              eos_token_id=None, verify_method=method, verify_kwargs=kw)[0]
    for got, m in zip(res if isinstance(res, tuple) else (res,), ("exact", "lossy") if method == "exact+lossy"
                      else (method,)):
        r = vo.verify(logits=logits, token_ids=tokens.tolist(), children=st.children(), method=m,
                      threshold=0.3, window=2, threshold_method="entropy", upcast=True)
        assert r.accept_len == n - 1
        assert got.sampled_tokens.squeeze(0).tolist() == r.tokens and got.hidden_indices.tolist() == r.hidden
        assert (got.total_len, got.accept_len) == (r.total_len, r.accept_len)


def test_sequence_without_decoded_rows(cuda_lib):
    """A sequence with no decoded row gets an empty result (L = 0) instead of what the previous call left
    in the output block, and the scratch tickets stay clean for the next launch."""
    from subspec_b200 import _lib
    from subspec_b200.verify import VerifyWorkspace, flatten_tree
    vocab, n = 4099, 12
    gen = torch.Generator().manual_seed(4)
    sts = [synthetic.random_tree(n, 5, 3, vocab, gen) for _ in range(3)]
    logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=torch.bfloat16, peaked=True) for st in sts])
    ws = VerifyWorkspace(3, n, torch.device("cuda", 0))
    flats = []
    for st in sts:
        tok, off, idx = flatten_tree(_tree_of(st), 0, limit=n, restrict=True)
        flats.append((tok, off, idx, n, 0))
    for method in (_lib.VERIFY_EXACT, _lib.VERIFY_EXACT_AND_LOSSY):
        ws.set_trees(flats)
        ws.run(logits.cuda(), input_kind=_lib.IN_LOGITS, method=method, gate=_lib.GATE_ENTROPY, threshold=0.3)
        full = {k: v.copy() for k, v in ws.fetch().items()}
        assert all(int(full["out_meta"][b, 0]) >= 1 for b in range(3))
        holed = list(flats)
        holed[1] = (flats[1][0], flats[1][1], flats[1][2], 0, 0)   # the middle sequence has no row this time
        ws.set_trees(holed)
        ws.run(logits.cuda(), input_kind=_lib.IN_LOGITS, method=method, gate=_lib.GATE_ENTROPY, threshold=0.3)
        out = ws.fetch()
        assert out["out_meta"][1].tolist() == [0, 0, 0, 0]
        if method == _lib.VERIFY_EXACT_AND_LOSSY:
            assert out["out2_meta"][1].tolist() == [0, 0, 0, 0]
        for b in (0, 2):
            L = int(full["out_meta"][b, 0])
            assert out["out_meta"][b].tolist() == full["out_meta"][b].tolist()
            assert out["out_tokens"][b, :L].tolist() == full["out_tokens"][b, :L].tolist()
