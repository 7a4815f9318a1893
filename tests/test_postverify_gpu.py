"""The SubSpec-v2 steps between two verifications on the device: re-rooting, delayed KV reorder, prune_to_depth."""
import numpy as np
import pytest
import torch

from oracle import kv_oracle as ko
from oracle import postverify_oracle as po
from oracle import verify_oracle as vo
from subspec_b200 import _lib, kv_cache, synthetic
from subspec_b200.postverify import PostVerifyState, post_verify, prune_to_depth_batched
from subspec_b200.tree import Tree
from subspec_b200.verify import VerifyWorkspace, flatten_tree
from tests import golden_io

pytestmark = pytest.mark.gpu


def _csr(children, stride):
    off = np.zeros(stride + 1, dtype=np.int32)
    idx = np.zeros(stride, dtype=np.int32)
    w = 0
    for i, ch in enumerate(children):
        off[i] = w
        for c in ch:
            idx[w] = c
            w += 1
    off[len(children):] = w
    return off, idx


def test_prune_to_depth_matches_reference(cuda_lib):
    """Every golden prune (reference Tree.prune_to_depth), all trees of a depth in one launch."""
    cases = golden_io.post_cases()
    S = max(len(c["tree"]["token_ids"]) for c in cases) + 3
    for d in range(0, 9):
        rows = [(c, next((p for p in c["prunes"] if p["max_depth"] == d), None)) for c in cases]
        rows = [(c, p) for c, p in rows if p is not None]
        if not rows:
            continue
        B = len(rows)
        tok = torch.zeros(B, S, dtype=torch.int32)
        par = torch.full((B, S), -1, dtype=torch.int32)
        dep = torch.zeros(B, S, dtype=torch.int32)
        prb = torch.rand(B, S)
        off = torch.zeros(B, S + 1, dtype=torch.int32)
        idx = torch.zeros(B, S, dtype=torch.int32)
        n = torch.zeros(B, dtype=torch.int32)
        for b, (c, _) in enumerate(rows):
            t = c["tree"]
            m = len(t["token_ids"])
            tok[b, :m] = torch.tensor(t["token_ids"])
            par[b, :m] = torch.tensor(t["parents"])
            dep[b, :m] = torch.tensor(t["depths"])
            o, i = _csr(t["children"], S)
            off[b], idx[b] = torch.from_numpy(o), torch.from_numpy(i)
            n[b] = m
        prb0 = prb.clone()
        trees = {"token_ids": tok.cuda(), "parent_indices": par.cuda(), "depths": dep.cuda(), "n_nodes": n.cuda(),
                 "cumulative_probabilities": prb.cuda(), "child_off": off.cuda(), "child_idx": idx.cuda()}
        status = torch.zeros(1, dtype=torch.int32, device="cuda")
        out = prune_to_depth_batched(trees, d, status=status)
        assert int(status.item()) == 0
        for b, (c, p) in enumerate(rows):
            k = len(p["keep"])
            assert int(out["n_nodes"][b]) == k == int(trees["n_nodes"][b])
            assert out["keep_idx"][b, :k].tolist() == p["keep"]
            assert trees["token_ids"][b, :k].tolist() == p["token_ids"]
            assert trees["parent_indices"][b, :k].tolist() == p["parents"]
            assert trees["depths"][b, :k].tolist() == p["depths"]
            assert trees["cumulative_probabilities"][b, :k].cpu().tolist() == prb0[b, p["keep"]].tolist()
            o, i = trees["child_off"][b].tolist(), trees["child_idx"][b].tolist()
            assert [i[o[r]:o[r + 1]] for r in range(k)] == p["children"]
    with pytest.raises(ValueError):
        prune_to_depth_batched(trees, -1)


def test_rerooting_matches_reference_lookups(cuda_lib):
    """next_root = Tree.find_child_index(last context, bonus token): the golden look-ups, fed through the
    kernel as verify outputs whose last entry is (token, context)."""
    for c in golden_io.post_cases():
        t = c["tree"]
        m = len(t["token_ids"])
        finds = c["finds"]
        B = len(finds)
        ws = VerifyWorkspace(B, m, torch.device("cuda", 0))
        off, idx = _csr(t["children"], m)
        flat = (np.asarray(t["token_ids"], dtype=np.int64), off[:m + 1], idx[:int(off[m])], m, 0)
        ws.set_trees([flat] * B)
        toks = ws.dev_view("out_tokens").view(B, ws.max_out)
        hid = ws.dev_view("out_hidden").view(B, ws.max_out)
        meta = ws.dev_view("out_meta").view(B, 4)
        for b, (node, tok, _) in enumerate(finds):
            L = 1 + b % 3
            meta[b, 0] = L
            toks[b, L - 1], hid[b, L - 1] = tok, node
        st = PostVerifyState(B, 16, "cuda")
        post_verify(ws, st)
        st.check_status()
        assert st.next_root.tolist() == [w for _, _, w in finds]
        assert st.accepted.tolist() == [int(w >= 0) for _, _, w in finds]


def test_delayed_reorder_over_several_steps(cuda_lib):
    """Four steps of the loop on six sequences: verify (real kernel, peaked inputs) -> post_verify -> paged
    compaction driven by reorder_n / reorder_offset / beam_cache, against the oracle's bookkeeping and the
    reference's pool reorder.  A sequence whose bonus token lands on a child of the tree puts its reorder off;
    the others reorder with everything gathered since."""
    B, n, vocab = 6, 24, 997
    L_kv, H, D, page_len, pages = 2, 2, 64, 16, 10
    tokens_kv = pages * page_len
    gen = torch.Generator().manual_seed(12)
    table = synthetic.random_page_table(B, pages, gen)
    pool_cpu = torch.randn(L_kv, B * pages, 2, page_len, H, D, generator=gen).to(torch.bfloat16)
    pool = pool_cpu.cuda()
    want_pool = pool_cpu.clone()
    kv0 = [40 + b for b in range(B)]
    ws = VerifyWorkspace(B, n, torch.device("cuda", 0))
    st = PostVerifyState(B, 4 * (n + 1), "cuda", kv_len=torch.tensor(kv0))
    oracle = [po.DelayedReorder(kv0[b]) for b in range(B)]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    deferred = reordered = 0
    for step in range(4):
        sts = [synthetic.random_tree(n, 6, 3, vocab, gen) for _ in range(B)]
        logits = torch.stack([synthetic.verify_logits(s, vocab, gen, dtype=torch.bfloat16, peaked=True, boost_frac=0.9)
                              for s in sts])
        flats = []
        for s in sts:
            tok, off, idx = flatten_tree(Tree.from_arrays(s.token_ids.tolist(), s.parents.tolist()), 0)
            flats.append((tok, off, idx, n, 0))
        ws.set_trees(flats)
        if step == 3:
            st.finished.fill_(1)   # the last step: every sequence reorders whatever it has gathered
        ws.run(logits.cuda(), input_kind=_lib.IN_LOGITS, method=_lib.VERIFY_EXACT)
        post_verify(ws, st)
        kv_cache.compact_paged(pool, page_table=table.cuda(), offset=st.reorder_offset, n=st.reorder_n,
                               beam=st.beam_cache, status=status)
        out = ws.fetch()
        st.check_status()
        assert int(status.item()) == 0
        for b, s in enumerate(sts):
            r = vo.verify(logits=logits[b], token_ids=s.token_ids.tolist(), children=s.children(), method="exact",
                          upcast=True)
            Lb = int(out["out_meta"][b, 0])
            assert out["out_hidden"][b, :Lb].tolist() == r.hidden
            want_root = po.find_child_index(s.token_ids.tolist(), s.children(), r.hidden[-1], r.tokens[-1])
            assert int(st.next_root[b]) == want_root
            beam, at = oracle[b].step(r.hidden, want_root, finished=step == 3)
            if beam is None:
                deferred += 1
                assert int(st.reorder_n[b]) == 0
            else:
                reordered += 1
                assert int(st.reorder_n[b]) == len(beam) and int(st.reorder_offset[b]) == at
                ko.paged_reorder(want_pool, torch.tensor(beam), at, page_table=table[b].tolist())
            assert int(st.kv_len[b]) == oracle[b].kv_len
            assert int(st.beam_len[b]) == len(oracle[b].cache)
            assert st.beam_cache[b, :len(oracle[b].cache)].tolist() == oracle[b].cache
        assert torch.equal(pool.cpu(), want_pool), step
    assert reordered >= B and tokens_kv > max(o.kv_len for o in oracle) + n
