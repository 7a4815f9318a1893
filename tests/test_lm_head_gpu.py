"""lm_head + verification without the logits (`subspec_lm_head_verify`) against `logits = hidden @ W^T` rounded to
bf16 followed by the verifier: the CPU oracle on small cases, the streaming kernel on the library GEMM's logits
at the size of the benchmark's wave.

A GEMM's accumulation order is its own: an fp32 sum that lies within rounding of a bf16 rounding boundary may
come out one bf16 step apart.  The targets are therefore compared exactly where the reference's two largest
logits of a row differ by more than one bf16 step, and must point at a logit within one step of the maximum
elsewhere; sequences whose rows all agree must give identical outputs.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from oracle import verify_oracle as vo
from subspec_b200 import _lib, synthetic
from subspec_b200.tree import Tree
from subspec_b200.verify import get_workspace, verify_tree_batched

pytestmark = pytest.mark.gpu

METHODS = [("exact", {}),
           ("lossy", {"threshold_method": "entropy", "threshold": 0.3, "window_size": 1}),
           ("lossy", {"threshold_method": "prob", "threshold": 0.05, "window_size": 0})]


def _build(st: synthetic.SynthTree) -> Tree:
    return Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist())


def _case(B, n, dim, vocab, seed, boost=True, dtype=torch.bfloat16):
    gen = torch.Generator().manual_seed(seed)
    sts = [synthetic.random_tree(n - (b % 3), 6, 4, vocab, gen) for b in range(B)]
    hidden = torch.randn(B, n, dim, generator=gen).to(dtype)
    weight = (torch.randn(vocab, dim, generator=gen) * (3.0 / dim ** 0.5)).to(dtype)
    if boost:
        # make the draft right most of the time: the hidden state of a node points at the weight row of its
        # first child's token, so that walks accept and the lossy gates see probabilities that matter
        for b, st in enumerate(sts):
            kids = st.children()
            for u in range(st.n):
                if kids[u] and (u + b) % 4 != 3:
                    hidden[b, u] += (weight[int(st.token_ids[kids[u][0]])].float() * 1.5).to(dtype)
    return sts, hidden, weight


def _ref_logits(hidden, weight):
    B, n, dim = hidden.shape
    return (hidden.float().view(-1, dim) @ weight.float().t()).view(B, n, -1).to(hidden.dtype)


def _bf16_step(x: torch.Tensor, mantissa_bits: int = 7) -> torch.Tensor:
    """The distance from |x| to the next bf16 value above it (with 10 mantissa bits: the next fp16 value; a bf16
    step is never smaller, so it serves as the tolerance for both)."""
    return torch.maximum(x.abs().float(), torch.tensor(2.0 ** -126)).log2().floor().exp2() * 2.0 ** -mantissa_bits


def _check_against(sts, ref_logits, got, out, ref_results, exact_outputs=True):
    B = len(sts)
    for b, st in enumerate(sts):
        lg = ref_logits[b, :st.n].float()
        top = lg.max(-1).values
        tgt = torch.from_numpy(out["node_target"][b, :st.n].astype(np.int64))
        at = lg.gather(1, tgt[:, None]).squeeze(1)
        assert bool((at >= top - _bf16_step(top)).all()), b           # within one step of the maximum, always
        same_rows = bool((tgt == lg.argmax(-1)).all())
        if same_rows and exact_outputs:
            r = ref_results[b]
            assert got[b].sampled_tokens.squeeze(0).tolist() == r[0], b
            assert got[b].hidden_indices.tolist() == r[1], b
            assert (got[b].total_len, got[b].accept_len) == r[2], b


@pytest.mark.parametrize("B,n,dim,vocab,dtype", [
    (4, 33, 512, 5000, torch.bfloat16),      # fewer rows than a tile, ragged last tile
    (3, 64, 264, 255, torch.bfloat16),        # one column tile, dim not a multiple of 64
    (9, 40, 1024, 8192 + 40, torch.bfloat16),
    (1, 64, 768, 40000, torch.bfloat16),      # one request: narrowed column tiles, second row block skipped
    (4, 33, 512, 5000, torch.float16),        # the reference's usual dtype
    (1, 50, 768, 30001, torch.float16),
    (7, 48, 1024, 9000, torch.float16)])
def test_matches_oracle_on_rounded_logits(cuda_lib, B, n, dim, vocab, dtype):
    sts, hidden, weight = _case(B, n, dim, vocab, seed=B * 7 + n, dtype=dtype)
    ref = _ref_logits(hidden, weight)
    trees = [_build(st) for st in sts]
    accepted = 0
    for method, kw in METHODS:
        refs = []
        for b, st in enumerate(sts):
            r = vo.verify(logits=ref[b, :st.n], token_ids=st.token_ids.tolist(), children=st.children(), method=method,
                          threshold=kw.get("threshold", 0.0), window=kw.get("window_size", 1),
                          threshold_method=kw.get("threshold_method", "prob"), upcast=True)
            refs.append((r.tokens, r.hidden, (r.total_len, r.accept_len)))
            accepted += r.accept_len
        got = verify_tree_batched(trees=trees, root_inds=[0] * B, hidden_states=hidden.cuda(),
                                  lm_head_weight=weight.cuda(), eos_token_id=None, verify_method=method, verify_kwargs=kw)
        ws = get_workspace(B, max(st.n for st in sts), torch.device("cuda", torch.cuda.current_device()))
        out = ws.fetch()
        assert int(out["dev_status"][0]) == 0
        _check_against(sts, ref, got, out, refs)
        if method == "lossy":  # entropies and child probabilities against fp64 softmax of the rounded logits
            for b, st in enumerate(sts):
                p = torch.softmax(ref[b, :st.n].double(), -1)
                ent = -(p * torch.log(p.clamp_min(1e-300))).sum(-1) / np.log(vocab)
                assert np.allclose(out["node_entropy"][b, :st.n], ent.numpy(), rtol=2e-2, atol=2e-3)
                kids = st.children()
                for u in range(st.n):
                    for c in kids[u]:
                        want = float(p[u, int(st.token_ids[c])])
                        step = float(_bf16_step(ref[b, u, int(st.token_ids[c])].float()))
                        assert out["node_child_prob"][b, c] == pytest.approx(want, rel=np.expm1(step) * 1.05 + 2e-2,
                                                                             abs=1e-7)
    assert accepted > 0


def test_rows_per_sequence_and_strides(cuda_lib):
    """More rows laid out per sequence than the trees decode; padded row strides of both operands."""
    B, n, dim, vocab = 5, 20, 320, 1500
    sts, hidden, weight = _case(B, n, dim, vocab, seed=11)
    rows = 37
    hpad = torch.zeros(B, rows, dim + 24, dtype=torch.bfloat16)
    hpad[:, :n, :dim] = hidden
    hpad[:, n:, :dim] = 7.0  # rows nobody decodes
    wpad = torch.zeros(vocab, dim + 8, dtype=torch.bfloat16)
    wpad[:, :dim] = weight
    hd, wd = hpad.cuda()[:, :, :dim], wpad.cuda()[:, :dim]
    ref = _ref_logits(hidden, weight)
    trees = [_build(st) for st in sts]
    dev = torch.device("cuda", torch.cuda.current_device())
    ws = get_workspace(B, max(st.n for st in sts), dev)
    from subspec_b200.verify import _prepare_tree
    ws.set_trees([_prepare_tree(t, 0, 0, rows, _lib.VERIFY_EXACT) for t in trees])
    # the wrapper makes operands contiguous; go through the C ABI with the strides as they are
    la = _lib.LmHeadVerifyArgs()
    la.struct_size = C.sizeof(_lib.LmHeadVerifyArgs)
    la.hidden_dim, la.hidden_seq_rows = dim, rows
    la.hidden, la.hidden_row_stride = hd.data_ptr(), hd.stride(1)
    la.weight, la.weight_row_stride = wd.data_ptr(), wd.stride(0)
    ws.run_lm_head(hidden.cuda(), weight.cuda(), method=_lib.VERIFY_EXACT)   # fills a template of the arguments
    want = ws.fetch()["node_target"].copy()
    need = C.c_size_t(0)
    _lib.check(_lib.lib().subspec_lm_head_verify_scratch_bytes(B, ws.max_nodes, rows, vocab, C.byref(need)), "bytes")
    scratch = torch.zeros(need.value + 256, dtype=torch.uint8, device=dev)
    a = la.verify
    a.struct_size = C.sizeof(_lib.VerifyArgs)
    a.batch, a.max_nodes, a.vocab, a.dtype = B, ws.max_nodes, vocab, _lib.torch_dtype_code(torch.bfloat16)
    for name in ("n_nodes", "n_rows", "token_ids", "child_off", "child_idx", "root"):
        setattr(a, name, ws._in_ptr(name))
    a.temperature, a.top_p, a.method, a.gate, a.window, a.eos, a.max_out = 1.0, 1.0, _lib.VERIFY_EXACT, 0, 1, -1, ws.max_out
    for name in ("out_tokens", "out_hidden", "out_meta", "node_target", "node_entropy", "node_child_prob", "node_rowmax",
                 "node_rowsum", "node_exact_after", "node_best_len", "node_best_next", "dev_status", "out2_tokens",
                 "out2_hidden", "out2_meta"):
        setattr(a, name, ws._out_ptr(name))
    a.scratch = (scratch.data_ptr() + 255) // 256 * 256
    a.scratch_bytes = need.value
    ws.dev_view("node_target").fill_(-5)
    stream = torch.cuda.current_stream().cuda_stream
    _lib.check(_lib.lib().subspec_lm_head_verify(C.byref(la), C.c_void_p(stream)), "subspec_lm_head_verify")
    out = ws.fetch()
    assert int(out["dev_status"][0]) == 0
    for b, st in enumerate(sts):
        assert out["node_target"][b, :st.n].tolist() == want[b, :st.n].tolist()
        assert out["node_target"][b, :st.n].tolist() == ref[b, :st.n].float().argmax(-1).tolist()
    # arguments the call refuses: a stride that is not a multiple of 16 bytes, sampled targets, fp32 operands
    la.hidden_row_stride = hd.stride(1) + 1
    assert _lib.lib().subspec_lm_head_verify(C.byref(la), C.c_void_p(stream)) == _lib.EINVAL
    la.hidden_row_stride = hd.stride(1)
    a.do_sample = 1
    assert _lib.lib().subspec_lm_head_verify(C.byref(la), C.c_void_p(stream)) == _lib.EUNSUPPORTED
    a.do_sample = 0
    a.dtype = _lib.torch_dtype_code(torch.float32)
    assert _lib.lib().subspec_lm_head_verify(C.byref(la), C.c_void_p(stream)) == _lib.EUNSUPPORTED
    a.dtype = _lib.torch_dtype_code(torch.bfloat16)
    a.scratch_bytes = need.value - 256
    assert _lib.lib().subspec_lm_head_verify(C.byref(la), C.c_void_p(stream)) == _lib.ESCRATCH
    torch.cuda.synchronize()


def test_wave_of_the_benchmark_against_the_streaming_kernel(cuda_lib):
    """64 trees of 64 nodes, hidden size 3584, vocabulary 152064: the fused call against the library GEMM's bf16
    logits run through `subspec_verify_batched`, greedy and lossy."""
    B, n, dim, vocab = 64, 64, 3584, 152064
    gen = torch.Generator().manual_seed(3)
    sts = [synthetic.random_tree(n, 8, 4, vocab, gen) for _ in range(B)]
    dev = torch.device("cuda", torch.cuda.current_device())
    h = torch.randn(B, n, dim, generator=gen).to(torch.bfloat16).to(dev)
    w = (torch.randn(vocab, dim, generator=gen) * (3.0 / dim ** 0.5)).to(torch.bfloat16).to(dev)
    for b, st in enumerate(sts):  # walks that accept: see _case
        kids = st.children()
        rows = [u for u in range(st.n) if kids[u] and (u + b) % 4]
        toks = [int(st.token_ids[kids[u][0]]) for u in rows]
        h[b, rows] += (w[toks].float() * 2.5).to(torch.bfloat16)
    trees = [_build(st) for st in sts]
    logits = (h.view(-1, dim) @ w.t()).view(B, n, vocab)
    ws = get_workspace(B, n, dev)
    accepted = 0
    for method, kw in METHODS[:2]:
        ref = verify_tree_batched(trees=trees, root_inds=[0] * B, logits=logits, eos_token_id=None, verify_method=method,
                                  verify_kwargs=kw)
        r = ws.fetch()
        ref_ent, ref_cp = r["node_entropy"].copy(), r["node_child_prob"].copy()
        refs = [(x.sampled_tokens.squeeze(0).tolist(), x.hidden_indices.tolist(), (x.total_len, x.accept_len)) for x in ref]
        accepted += sum(x.accept_len for x in ref)
        got = verify_tree_batched(trees=trees, root_inds=[0] * B, hidden_states=h, lm_head_weight=w, eos_token_id=None,
                                  verify_method=method, verify_kwargs=kw)
        out = ws.fetch()
        assert int(out["dev_status"][0]) == 0
        _check_against(sts, logits.cpu(), got, out, refs)
        if method == "lossy":
            assert np.allclose(out["node_entropy"], ref_ent, rtol=1e-3, atol=1e-5)
            # a child's probability moves by the factor e^step when its logit comes out one bf16 step apart
            # (the tail recomputes these few logits as dot products); most must agree to fp32 rounding
            close = total = 0
            for b, st in enumerate(sts):
                par, tok = st.parents[1:].to(dev), st.token_ids[1:].to(dev)
                lg = logits[b, par, tok].float().cpu()
                tol = torch.expm1(_bf16_step(lg)).numpy() * 1.05 + 1e-4
                g, r_ = out["node_child_prob"][b, 1:st.n], ref_cp[b, 1:st.n]
                assert bool((np.abs(g - r_) <= tol * r_ + 1e-12).all()), b
                close += int((np.abs(g - r_) <= 1e-4 * r_ + 1e-12).sum())
                total += st.n - 1
            assert close > 0.95 * total
    assert accepted > B


def test_loop_step_from_hidden_states(cuda_lib):
    """SpeculativeLoopBatch.end_step with hidden states and the lm_head weight leaves the loop in the state that
    the same step with the library GEMM's logits leaves it in (targets, re-rooting, page lists, KV rows)."""
    from subspec_b200.step import SpeculativeLoopBatch
    from subspec_b200.verify import flatten_tree

    Bn, n, dim, vocab = 4, 16, 128, 997
    sts, hidden, weight = _case(Bn, n, dim, vocab, seed=21)
    sts = [synthetic.random_tree(n, 5, 3, vocab, torch.Generator().manual_seed(100 + b)) for b in range(Bn)]
    for b, st in enumerate(sts):
        kids = st.children()
        for u in range(st.n):
            if kids[u]:
                hidden[b, u] += (weight[int(st.token_ids[kids[u][0]])].float() * 2.0).to(torch.bfloat16)
    h, w = hidden.cuda(), weight.cuda()
    logits = (h.view(-1, dim) @ w.t()).view(Bn, n, vocab)
    flats = []
    for s in sts:
        tok, off, idx = flatten_tree(Tree.from_arrays(s.token_ids.tolist(), s.parents.tolist()), 0)
        flats.append((tok, off, idx, n, 0))
    states = []
    for fused in (False, True):
        loop = SpeculativeLoopBatch(Bn, n, "cuda", kv_layers=2, kv_heads=2, head_dim=64, page_len=16, pages_per_seq=12,
                                    init_len=torch.tensor([5, 17, 32, 9]))
        loop.pool.copy_(torch.randn(loop.pool.shape, generator=torch.Generator().manual_seed(1)).to(torch.bfloat16))
        loop.begin_step(n)
        loop.set_trees(flats)
        if fused:
            loop.end_step(hidden_states=h, lm_head_weight=w)
        else:
            loop.end_step(logits)
        loop.check()
        out = loop.ws.fetch()
        states.append((out["node_target"].copy(), out["out_tokens"].copy(), out["out_hidden"].copy(), out["out_meta"].copy(),
                       loop.state.next_root.cpu(), loop.state.kv_len.cpu(), loop.pages.kv_len.cpu(), loop.pool.cpu()))
    assert int(states[0][3][:, 1].sum()) > Bn  # tokens were accepted
    if not np.array_equal(states[0][0], states[1][0]):
        # a target decided by the rounding of two different GEMMs: it must be within one bf16 step of the maximum,
        # and the states behind it are not comparable
        lg = logits.float().cpu()
        at = lg.gather(2, torch.from_numpy(states[1][0].astype(np.int64))[..., None]).squeeze(-1)
        assert bool((at >= lg.max(-1).values - _bf16_step(lg.max(-1).values)).all())
        pytest.skip("a row's two largest logits are within one bf16 step: the two GEMMs chose differently")
    for x, y in zip(*states):
        assert (np.array_equal(x, y) if isinstance(x, np.ndarray) else torch.equal(x, y))


def test_exact_and_lossy_from_one_call(cuda_lib):
    """`verify_method="exact+lossy"` (the pair of results a step that verifies greedily and then lossily needs)
    through the fused call: both results equal those of the streaming kernel on the library GEMM's logits."""
    B, n, dim, vocab = 6, 48, 768, 32000
    sts, hidden, weight = _case(B, n, dim, vocab, seed=5)
    sts = [synthetic.random_tree(n, 6, 4, vocab, torch.Generator().manual_seed(50 + b)) for b in range(B)]  # all rows decoded
    for b, st in enumerate(sts):
        kids = st.children()
        for u in range(st.n):
            if kids[u] and (u + b) % 3:
                hidden[b, u] += (weight[int(st.token_ids[kids[u][0]])].float() * 2.0).to(torch.bfloat16)
    h, w = hidden.cuda(), weight.cuda()
    logits = (h.view(-1, dim) @ w.t()).view(B, n, vocab)
    trees = [_build(st) for st in sts]
    kw = {"threshold_method": "prob", "threshold": 0.02, "window_size": 1}
    dev = torch.device("cuda", torch.cuda.current_device())
    ref = verify_tree_batched(trees=trees, root_inds=[0] * B, logits=logits, eos_token_id=None,
                              verify_method="exact+lossy", verify_kwargs=kw)
    ref_tgt = get_workspace(B, n, dev).fetch()["node_target"].copy()
    got = verify_tree_batched(trees=trees, root_inds=[0] * B, hidden_states=h, lm_head_weight=w, eos_token_id=None,
                              verify_method="exact+lossy", verify_kwargs=kw)
    out = get_workspace(B, n, dev).fetch()
    assert int(out["dev_status"][0]) == 0
    compared = 0
    for b in range(B):
        if not np.array_equal(out["node_target"][b], ref_tgt[b]):
            continue  # a target decided by the rounding of two different GEMMs (checked against the rule elsewhere)
        compared += 1
        for r, g in zip(ref[b], got[b]):  # (exact result, lossy result)
            assert g.sampled_tokens.tolist() == r.sampled_tokens.tolist() and g.hidden_indices.tolist() == r.hidden_indices.tolist()
            assert (g.total_len, g.accept_len) == (r.total_len, r.accept_len)
    assert compared >= B // 2
    assert sum(r[1].accept_len for r in ref) >= sum(r[0].accept_len for r in ref) > 0


def test_single_tree_call(cuda_lib):
    """`verify_tree(..., hidden_states=, lm_head_weight=)`: the reference's call for one tree, fed with the
    target's last hidden states instead of logits."""
    from subspec_b200.verify import verify_tree

    sts, hidden, weight = _case(1, 40, 384, 3000, seed=9)
    st = sts[0]
    ref = _ref_logits(hidden, weight)
    toks, hid, (total, acc) = verify_tree(tree=_build(st), root_ind=0, hidden_states=hidden[0, :st.n].cuda(),
                                          lm_head_weight=weight.cuda(), eos_token_id=None)
    tgt = get_workspace(1, st.n, torch.device("cuda", torch.cuda.current_device())).fetch()["node_target"][0, :st.n]
    lg = ref[0, :st.n].float()
    at = lg.gather(1, torch.from_numpy(tgt.astype(np.int64))[:, None]).squeeze(1)
    assert bool((at >= lg.max(-1).values - _bf16_step(lg.max(-1).values)).all())
    r = vo.exact_walk(target=tgt.tolist(), token_ids=st.token_ids.tolist(), children=st.children(), root=0,
                      n_rows=st.n, eos=None)
    assert toks.squeeze(0).tolist() == r.tokens and hid.tolist() == r.hidden and (total, acc) == (r.total_len, r.accept_len)
    with pytest.raises(ValueError):
        verify_tree(tree=_build(st), root_ind=0, hidden_states=hidden[0, :st.n].cuda(), lm_head_weight=weight.cuda(),
                    eos_token_id=None, do_sample=True)


def test_fused_call_in_a_cuda_graph(cuda_lib):
    """The call captures into a CUDA graph (no allocation, no synchronisation inside) and a replay on new hidden
    states in the same buffer gives that input's results."""
    B, n, dim, vocab = 3, 32, 512, 6000
    sts, hidden, weight = _case(B, n, dim, vocab, seed=13)
    _, hidden2, _ = _case(B, n, dim, vocab, seed=14)
    trees = [_build(st) for st in sts]
    dev = torch.device("cuda", torch.cuda.current_device())
    from subspec_b200.verify import _prepare_tree
    ws = get_workspace(B, max(st.n for st in sts), dev)
    ws.set_trees([_prepare_tree(t, 0, 0, n, _lib.VERIFY_LOSSY) for t in trees])
    h, w = hidden.cuda(), weight.cuda()
    kw = dict(method=_lib.VERIFY_LOSSY, gate=_lib.GATE_ENTROPY, threshold=0.3, window=1)
    side = torch.cuda.Stream()
    side.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(side):
        ws.run_lm_head(h, w, **kw)   # first call outside the capture: sizes the scratch
    torch.cuda.current_stream().wait_stream(side)
    eager = {k: v.copy() for k, v in ws.fetch().items()}
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        ws.run_lm_head(h, w, **kw)
    graph.replay()
    out = ws.fetch()
    for key in ("out_tokens", "out_hidden", "out_meta", "node_target", "node_entropy"):
        assert np.array_equal(out[key], eager[key]), key
    h.copy_(hidden2.cuda())
    graph.replay()
    out2 = {k: v.copy() for k, v in ws.fetch().items()}
    ws.run_lm_head(h, w, **kw)
    want2 = ws.fetch()
    assert not np.array_equal(out2["node_target"], eager["node_target"])
    for key in ("out_tokens", "out_hidden", "out_meta", "node_target", "node_entropy"):
        assert np.array_equal(out2[key], want2[key]), key
