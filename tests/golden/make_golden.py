"""Generate the golden fixtures under tests/golden/ by running the UNMODIFIED reference.

Usage (only where a read-only checkout of NYCU-EDgeAi/subspec is available):

    python tests/golden/make_golden.py --reference /path/to/subspec [--only verify|sampled|expand|expand_chain|kv|kv_hf|post|pages|lossy_unit]

The reference is imported, never copied.  Two third-party modules it imports but
does not need on this path (`nvtx`, `prettytable`) are replaced by throw-away
stubs in a temporary directory.  Inputs come from `subspec_b200.synthetic`
(seeded); small cases also store their inputs inline so the fixture does not
depend on the RNG stream.  Outputs written:

    verify_cases.json / verify_small.npz   verify_tree (exact, lossy) results
    sampled_cases.json                     verify_tree with do_sample=True and injected uniforms
    lossy_unit_cases.json                  every call made by the reference's tests/test_lossy_tree_verify.py
    expand_cases.json / expand_small.npz   _topk_flatten / Tree / TreeMaskCache results
    expand_chain.json                      ten-level expansions at the benchmark's vocabulary, pruned to 64 nodes
    kv_cases.json                          KvCachePool.reorder_cache_with_offset checksums
    kv_hf_cases.json                       TreeStaticCache / TreeDynamicCache.reorder_cache_with_offset checksums
    post_cases.json                        Tree.prune_to_depth / Tree.find_child_index results
    pages_cases.json                       KvCachePool / RequestKvCache page lists over scripted generation loops
"""
from __future__ import annotations

import argparse
import hashlib
import json
import sys
import tempfile
from pathlib import Path

import numpy as np
import torch

HERE = Path(__file__).resolve().parent
ROOT = HERE.parent.parent
sys.path.insert(0, str(ROOT))

from subspec_b200 import synthetic  # noqa: E402

DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


def import_reference(ref: str):
    stub = Path(tempfile.mkdtemp(prefix="subspec_stub_"))
    (stub / "nvtx.py").write_text(
        "import contextlib\n@contextlib.contextmanager\ndef annotate(*a, **k):\n    yield\n")
    (stub / "prettytable.py").write_text("class PrettyTable:\n    pass\n")
    sys.path.insert(0, str(stub))
    sys.path.insert(0, ref)
    import specdecodes.models.utils.tree_verify as tv
    import specdecodes.models.utils.lossy_tree_verify as ltv
    import specdecodes.models.utils.cpu_tree as ct
    import specdecodes.models.generators.base as gb
    import specdecodes.models.generators.classic_sd as csd
    import specdecodes.models.draft_models.base as db
    import specdecodes.models.utils.flashinfer.cache_manager as cm
    import specdecodes.models.utils.cache_utils as cu
    from specdecodes.models.utils.wandb_logger import wandb_logger
    return dict(tv=tv, ltv=ltv, ct=ct, gb=gb, csd=csd, db=db, cm=cm, cu=cu, wandb_logger=wandb_logger)


def ref_tree(ct, tree: synthetic.SynthTree):
    """Build the reference's Tree by appending TreeNodes directly."""
    t = ct.Tree(tree.token_ids[0], torch.float32)
    for i in range(1, tree.n):
        p = int(tree.parents[i])
        node = ct.TreeNode(parent=p, token_id=int(tree.token_ids[i]), cumulative_probability=1.0,
                           depth=int(tree.depths[i]))
        t.nodes.append(node)
        t.nodes[p].children.append(i)
    t.current_size = tree.n
    return t


def run_ref_verify(ref, tree, logits, *, method, kwargs, eos, skip_nodes, root_ind):
    rt = ref_tree(ref["ct"], tree)
    ref["wandb_logger"].clear_log_data()
    toks, hidden, (total, acc) = ref["tv"].verify_tree(
        tree=rt, root_ind=root_ind, logits=logits.unsqueeze(0),
        sample_token_fn=lambda *a, **k: ref["gb"].GeneratorBase._sample_token(None, *a, **k),
        verify_step_fn=lambda *a, **k: ref["csd"].ClassicSDGeneratorBase._verify_step(None, *a, **k),
        eos_token_id=eos, logits_processor=None, do_sample=False, skip_nodes=skip_nodes,
        verify_method=method, verify_kwargs=kwargs)
    return {"tokens": toks.squeeze(0).tolist(), "hidden": hidden.tolist(), "total_len": int(total),
            "accept_len": int(acc)}


def oracle_upcast(tree, logits, *, method, kwargs, eos, skip_nodes, root_ind):
    """The fp32-upcast restatement, to flag cases whose outcome depends on 16-bit rounding of probabilities."""
    sys.path.insert(0, str(ROOT))
    from oracle import verify_oracle as vo
    rows = logits.shape[0]
    ch_all = tree.children()
    n_loc = tree.n - skip_nodes
    ch = [[c - skip_nodes for c in ch_all[v + skip_nodes] if c - skip_nodes >= 0] for v in range(n_loc)]
    tok = tree.token_ids[skip_nodes:].tolist()
    probs = vo.target_probs(logits, upcast=True)
    tgt = probs.argmax(-1).tolist()
    if method == "exact":
        r = vo.exact_walk(target=tgt + [-1] * (n_loc - rows), token_ids=tok, children=ch, root=root_ind - skip_nodes,
                          n_rows=rows, eos=eos)
    else:
        n = min(rows, n_loc)
        root = root_ind - skip_nodes
        if root < 0 or root >= n:
            root = 0
        r = vo.lossy_verify(probs=probs[:n], token_ids=tok[:n], children=[[c for c in k if c < n] for k in ch[:n]],
                            root=root, eos=eos, threshold=float(kwargs.get("threshold", 0.0)),
                            window=int(kwargs.get("window_size", 1)),
                            use_entropy=str(kwargs.get("threshold_method", "prob")) == "entropy", target=tgt[:n])
    return {"tokens": r.tokens, "hidden": [h + skip_nodes for h in r.hidden], "total_len": r.total_len,
            "accept_len": r.accept_len}, r.min_gate_margin


METHODS = [
    ("exact", {}),
    ("lossy", {"threshold_method": "entropy", "threshold": 0.3, "window_size": 6}),
    ("lossy", {"threshold_method": "entropy", "threshold": 0.3, "window_size": 1}),
    ("lossy", {"threshold_method": "prob", "threshold": 0.05, "window_size": 0}),
    ("lossy", {"threshold_method": "prob", "threshold": 0.2, "window_size": 2}),
]


def gen_verify(ref, out_dir: Path):
    cases, small = [], {}
    skipped = []

    def add(name, tree, logits, *, gen_params, store_inline, eos=None, skip_nodes=0, root_ind=0, rows=None):
        rows = logits.shape[0] if rows is None else rows
        lg = logits[:rows]
        for mi, (method, kwargs) in enumerate(METHODS):
            exp = run_ref_verify(ref, tree, lg, method=method, kwargs=kwargs, eos=eos, skip_nodes=skip_nodes,
                                 root_ind=root_ind)
            up, margin = oracle_upcast(tree, lg, method=method, kwargs=kwargs, eos=eos, skip_nodes=skip_nodes,
                                       root_ind=root_ind)
            case = dict(name=f"{name}/m{mi}", input=name, method=method, kwargs=kwargs, eos=eos,
                        skip_nodes=skip_nodes, root_ind=root_ind, rows=rows, expected=exp,
                        upcast_agrees=(up == exp), gate_margin=None if margin == float("inf") else margin,
                        **gen_params)
            if up != exp:
                skipped.append(case["name"])
            cases.append(case)
        if store_inline:
            small[name + "/logits"] = logits.float().numpy()
            small[name + "/tokens"] = tree.token_ids.numpy()
            small[name + "/parents"] = tree.parents.numpy()

    # --- small vocab, inputs stored inline ---
    k = 0
    for vocab, n_nodes, depth, branch in [(11, 6, 3, 3), (50, 16, 5, 3), (257, 24, 6, 4), (1000, 40, 8, 4)]:
        for dtype in ("float32", "bfloat16", "float16"):
            for rep in range(2):
                seed = 1000 + k
                k += 1
                gen = torch.Generator().manual_seed(seed)
                tree = synthetic.random_tree(n_nodes, depth, branch, vocab, gen)
                logits = synthetic.verify_logits(tree, vocab, gen, dtype=DT[dtype], peaked=True, sigma=2.0)
                eos = int(tree.token_ids[n_nodes // 2]) if rep == 1 else None
                add(f"small/v{vocab}_n{n_nodes}_{dtype}_{rep}", tree, logits,
                    gen_params=dict(dtype=dtype, vocab=vocab, n_nodes=n_nodes, inline=True), store_inline=True,
                    eos=eos)
    # --- skip_nodes / root_ind / fewer rows than nodes (SubSpec v2 post-verify call pattern) ---
    for rep in range(4):
        seed = 2000 + rep
        gen = torch.Generator().manual_seed(seed)
        vocab, n_nodes = 97, 30
        tree = synthetic.random_tree(n_nodes, 6, 3, vocab, gen)
        skip = 1 + rep
        ch = tree.children()
        # root_ind = first node at or after `skip` that has children
        root_ind = next(i for i in range(skip, n_nodes) if ch[i])
        sub = synthetic.SynthTree(tree.token_ids[skip:], tree.parents[skip:] - skip, tree.depths[skip:])
        logits_local = synthetic.verify_logits(sub, vocab, gen, dtype=torch.float32, peaked=True, sigma=2.0)
        rows = logits_local.shape[0] - (rep % 2) * 5
        name = f"skip/v{vocab}_n{n_nodes}_s{skip}_{rep}"
        add(name, tree, logits_local, gen_params=dict(dtype="float32", vocab=vocab, n_nodes=n_nodes, inline=True),
            store_inline=True, skip_nodes=skip, root_ind=root_ind, rows=rows)
    # --- benchmark shapes, regenerated from the seed ---
    for dtype, peaked, seeds in [("float32", False, [1]), ("float32", True, [11, 12, 13]),
                                 ("bfloat16", False, [5]), ("bfloat16", True, [51, 52, 53]),
                                 ("float16", True, [61])]:
        for seed in seeds:
            tree, logits = synthetic.config1_case(seed, dtype=DT[dtype], peaked=peaked)
            add(f"config1/{dtype}_{'peaked' if peaked else 'literal'}_{seed}", tree, logits,
                gen_params=dict(dtype=dtype, vocab=152064, n_nodes=64, inline=False, seed=seed, peaked=peaked),
                store_inline=False)
    (out_dir / "verify_cases.json").write_text(json.dumps(
        {"torch": torch.__version__, "cases": cases, "dtype_sensitive": skipped}, indent=1))
    np.savez_compressed(out_dir / "verify_small.npz", **small)
    print(f"verify: {len(cases)} cases, {len(skipped)} depend on 16-bit probability rounding: {skipped}")


class InjectedDraws:
    """While active, torch.multinomial / Tensor.multinomial (the reference's only source of randomness on this
    path: classic_sd.py:112, tree_verify.py:99, lossy_tree_verify.py:76) return the inverse-CDF pick for the
    uniform injected for that node instead of a draw from the global RNG.  Everything else the reference
    runs is its own code: warpers, softmax, dtype handling, walk, bonus-token rule."""

    def __init__(self, uniforms):
        self.u = [float(x) for x in uniforms]
        self.rows = None  # the probabilities _sample_token returned, [N, V]: a 1-D draw is located among them

    def remember(self, probs):
        self.rows = probs.reshape(-1, probs.shape[-1]).detach().cpu()
        return probs

    def _draw(self, probs, num_samples=1, *a, **k):
        from oracle import verify_oracle as vo
        assert num_samples == 1
        if probs.dim() == 1:
            hits = (self.rows == probs.detach().cpu()).all(dim=-1).nonzero().reshape(-1)
            assert hits.numel() == 1, "cannot tell which node this distribution belongs to"
            return torch.tensor([vo.inverse_cdf_pick(probs, self.u[int(hits[0])])], dtype=torch.long)
        return torch.tensor([[vo.inverse_cdf_pick(probs[i], self.u[i])] for i in range(probs.shape[0])],
                            dtype=torch.long)

    def __enter__(self):
        self._saved = (torch.multinomial, torch.Tensor.multinomial)
        torch.multinomial = self._draw
        torch.Tensor.multinomial = lambda t, *a, **k: self._draw(t, *a, **k)
        return self

    def __exit__(self, *exc):
        torch.multinomial, torch.Tensor.multinomial = self._saved


def gen_sampled(ref, out_dir: Path):
    """do_sample=True through the unmodified reference with injected uniforms: sample-and-match walks and the
    lossy verifier on sampled targets, with the reference's own warper list (generators/base.py:42-64)."""
    sys.path.insert(0, str(ROOT))
    from oracle import verify_oracle as vo
    cases = []
    specs = []
    k = 0
    for vocab, nodes, depth, branch in [(50, 12, 4, 3), (1000, 24, 6, 4), (4099, 24, 6, 4), (32000, 20, 6, 4),
                                        (152064, 12, 5, 3)]:
        for dtype in ("float32", "bfloat16", "float16"):
            for temperature, top_k, top_p in [(1.0, 0, 0.9), (0.7, 50, 0.95), (1.3, 0, 1.0), (1.0, 20, 1.0)]:
                if top_k >= vocab:
                    top_k = vocab // 4
                specs.append(dict(vocab=vocab, nodes=nodes, depth=depth, branch=branch, dtype=dtype,
                                  temperature=temperature, top_k=top_k, top_p=top_p, method="exact", kwargs={},
                                  seed=7000 + k))
                k += 1
        # the lossy verifier on sampled targets: 16-bit logits with filters, fp32 with a temperature only
        for dtype, temperature, top_k, top_p in [("bfloat16", 1.0, 0, 0.9), ("float16", 0.8, 64, 0.95),
                                                 ("float32", 0.8, 0, 1.0), ("float32", 1.0, 0, 1.0)]:
            for kwargs in ({"threshold_method": "entropy", "threshold": 0.3, "window_size": 1},
                           {"threshold_method": "prob", "threshold": 0.05, "window_size": 0}):
                if vocab > 40000:
                    continue
                specs.append(dict(vocab=vocab, nodes=nodes, depth=depth, branch=branch, dtype=dtype,
                                  temperature=temperature, top_k=min(top_k, vocab // 4), top_p=top_p, method="lossy",
                                  kwargs=kwargs, seed=7000 + k))
                k += 1
    # fp32 logits, lossy, with top-k / top-p (gates on the filtered distribution)
    k = 0
    for vocab, nodes, depth, branch in [(1000, 24, 6, 4), (4099, 24, 6, 4), (32000, 20, 6, 4)]:
        for temperature, top_k, top_p in [(1.0, 0, 0.9), (0.8, 64, 0.95)]:
            for kwargs in ({"threshold_method": "entropy", "threshold": 0.3, "window_size": 1},
                           {"threshold_method": "prob", "threshold": 0.05, "window_size": 0}):
                specs.append(dict(vocab=vocab, nodes=nodes, depth=depth, branch=branch, dtype="float32",
                                  temperature=temperature, top_k=top_k, top_p=top_p, method="lossy",
                                  kwargs=kwargs, seed=8000 + k))
                k += 1
    for sp in specs:
        tree, logits, uniforms = synthetic.sampled_case(sp["seed"], sp["nodes"], sp["depth"], sp["branch"],
                                                        sp["vocab"], DT[sp["dtype"]])
        procs = ref["gb"].GeneratorBase._get_logits_processor(None, temperature=sp["temperature"],
                                                              top_k=sp["top_k"], top_p=sp["top_p"])
        rt = ref_tree(ref["ct"], tree)
        ref["wandb_logger"].clear_log_data()
        with InjectedDraws(uniforms.tolist()) as inj:
            toks, hidden, (total, acc) = ref["tv"].verify_tree(
                tree=rt, root_ind=0, logits=logits.unsqueeze(0),
                sample_token_fn=lambda *a, **kw: inj.remember(ref["gb"].GeneratorBase._sample_token(None, *a, **kw)),
                verify_step_fn=lambda *a, **kw: ref["csd"].ClassicSDGeneratorBase._verify_step(None, *a, **kw),
                eos_token_id=None, logits_processor=procs, do_sample=True, skip_nodes=0,
                verify_method=sp["method"], verify_kwargs=sp["kwargs"])
        exp = {"tokens": toks.squeeze(0).tolist(), "hidden": hidden.tolist(), "total_len": int(total),
               "accept_len": int(acc)}
        # the restatement in the reference's arithmetic (probabilities in the logits' type) and in fp32
        okw = dict(logits=logits, token_ids=tree.token_ids.tolist(), children=tree.children(), method=sp["method"],
                   do_sample=True, temperature=sp["temperature"], top_p=sp["top_p"], top_k=sp["top_k"],
                   uniforms=uniforms.tolist(), threshold=float(sp["kwargs"].get("threshold", 0.0)),
                   window=int(sp["kwargs"].get("window_size", 1)),
                   threshold_method=sp["kwargs"].get("threshold_method", "prob"))
        as_ref = vo.verify(upcast=False, **okw)
        up = vo.verify(upcast=True, **okw)
        same = lambda r: {"tokens": r.tokens, "hidden": r.hidden, "total_len": r.total_len,
                          "accept_len": r.accept_len} == exp
        margins = vo.sampling_margins(logits, sp["temperature"], sp["top_p"], uniforms.tolist(), top_k=sp["top_k"])
        used = range(tree.n) if sp["method"] == "lossy" else sorted(set(exp["hidden"]))
        cases.append(dict(name=f"sampled/{sp['method']}_v{sp['vocab']}_{sp['dtype']}_{sp['seed']}", **sp,
                          uniforms=[float(x) for x in uniforms.tolist()], expected=exp,
                          oracle_agrees=bool(same(as_ref)), upcast_agrees=bool(same(up)),
                          boundary_margin=min(margins[u][0] for u in used),
                          pick_margin=min(margins[u][1] for u in used),
                          gate_margin=None if up.min_gate_margin == float("inf") else up.min_gate_margin))
    (out_dir / "sampled_cases.json").write_text(json.dumps({"torch": torch.__version__, "cases": cases}, indent=1))
    n = len(cases)
    print(f"sampled: {n} cases; restatement agrees on {sum(c['oracle_agrees'] for c in cases)}, the fp32 upcast on "
          f"{sum(c['upcast_agrees'] for c in cases)}; accepted tokens in total "
          f"{sum(c['expected']['accept_len'] for c in cases)}")


def gen_lossy_unit(ref, ref_root: str, out_dir: Path):
    """Run the reference's own unit tests of the lossy verifier and record every call they make
    to lossy_bottom_up_verify: inputs, outputs and the wandb_logger metrics left behind."""
    import importlib.util

    spec = importlib.util.spec_from_file_location("ref_test_lossy", str(Path(ref_root) / "tests" /
                                                                      "test_lossy_tree_verify.py"))
    mod = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(mod)
    real = mod.lossy_bottom_up_verify
    records = []
    current = {"name": None}

    def recorder(**kw):
        sampled, hidden, acc = real(**kw)
        log = {k: v for k, v in ref["wandb_logger"].log_data.items() if isinstance(v, (int, float, str))}
        records.append(dict(
            test=current["name"], probs=kw["probs"].tolist(), token_ids=kw["token_ids"].tolist(),
            parent_indices=kw["parent_indices"].tolist(), children_lists=[list(c) for c in kw["children_lists"]],
            root_index=int(kw["root_index"]), eos_token_id=kw["eos_token_id"], do_sample=bool(kw["do_sample"]),
            threshold=float(kw["threshold"]), window_size=int(kw["window_size"]),
            threshold_method=kw.get("threshold_method", "prob"),
            expected=dict(sampled=sampled.tolist(), hidden=hidden.tolist(), accept_len=int(acc), log_data=log)))
        return sampled, hidden, acc

    mod.lossy_bottom_up_verify = recorder
    for name in sorted(n for n in dir(mod) if n.startswith("test_")):
        current["name"] = name
        ref["wandb_logger"].clear_log_data()
        getattr(mod, name)()  # the reference's own assertions run here
    (out_dir / "lossy_unit_cases.json").write_text(json.dumps({"cases": records}, indent=1))
    print(f"lossy unit: {len(records)} recorded calls from {len(set(r['test'] for r in records))} reference tests")


def gen_kv(ref, out_dir: Path):
    """Reorder small pools with the reference's KvCachePool / RequestKvCache and store checksums."""
    sys.path.insert(0, str(ROOT))
    from oracle.kv_oracle import checksum
    cm = ref["cm"]
    cases = []
    shapes = [(3, 8, 16, 4, 128, "bfloat16"), (2, 6, 8, 2, 64, "float16"), (1, 5, 4, 1, 8, "float32"),
              (28, 16, 16, 4, 128, "bfloat16")]
    seed = 300
    for (L, P, page_len, H, D, dtype) in shapes:
        for rep in range(3):
            seed += 1
            gen = torch.Generator().manual_seed(seed)
            pool = cm.KvCachePool(P, L, H, D, page_len, DT[dtype], "cpu")
            pool.cache_data.copy_(torch.randn(pool.cache_data.shape, generator=gen).to(DT[dtype]))
            tokens = P * page_len
            tree_n = min(24, tokens // 2)
            offset = int(torch.randint(0, tokens - tree_n + 1, (1,), generator=gen))
            n = int(torch.randint(1, min(11, tree_n) + 1, (1,), generator=gen))
            beam = torch.sort(torch.randperm(tree_n - 1, generator=gen)[:n - 1] + 1).values
            beam = torch.cat([torch.zeros(1, dtype=torch.long), beam]) if rep != 2 else \
                torch.sort(torch.randperm(tree_n, generator=gen)[:n]).values
            before = checksum(pool.cache_data)
            # through the request object: callers pass kv_len + 1 and the callee subtracts 1
            req = cm.RequestKvCache(pool, page_len, offset + tree_n)
            req.reorder_cache_with_offset(beam, offset=offset + 1 if offset else 0)
            cases.append(dict(seed=seed, layers=L, pages=P, page_len=page_len, heads=H, head_dim=D, dtype=dtype,
                              offset=offset, tree_n=tree_n, beam=beam.tolist(), before=before,
                              after=checksum(pool.cache_data), kv_len=req.kv_len,
                              kv_last_page_len=req.kv_last_page_len, n_pages=len(req.kv_page_indices),
                              free_pages=int(pool.num_free_pages())))
    (out_dir / "kv_cases.json").write_text(json.dumps({"cases": cases}, indent=1))
    print(f"kv: {len(cases)} cases")


def gen_expand(ref, out_dir: Path):
    """Drive the reference's own expansion helpers (one sequence at a time, as the reference does)."""
    from types import SimpleNamespace

    db, ct = ref["db"], ref["ct"]
    cases, small = [], {}
    # the last four keep at least as many nodes as the tree has: prune_to_top_n then leaves the numbering alone
    # (cpu_tree.py:176-177), which is the reference's default (max_verify_tokens = max_depth * topk_len + 1)
    cfgs = [(300, 4, 5, "float32", 1.0, 12), (300, 4, 5, "bfloat16", 1.0, 12), (1000, 6, 4, "float16", 0.7, 16),
            (2048, 16, 3, "float32", 1.0, 32), (97, 3, 6, "float32", 0.2, 10),
            (300, 4, 5, "float32", 1.0, 21), (300, 4, 3, "bfloat16", 1.0, 32), (1000, 6, 4, "float16", 0.7, 25),
            (500, 5, 4, "float32", 1.0, 64)]
    PREFIX, SKIP = 7, 2
    for ci, (V, k, depth, dtype, T, keep) in enumerate(cfgs):
        gen = torch.Generator().manual_seed(700 + ci)
        dt = DT[dtype]
        holder = SimpleNamespace()
        tree_data = db.TreeData()
        mask_cache = db.TreeMaskCache(prefix_len=5, sample_len=k, max_cache_len=None, dtype=torch.float32,
                                      device="cpu")
        static_len = 5 + k * depth + 3
        static_cache = db.TreeMaskCache(prefix_len=5, sample_len=k, max_cache_len=static_len, dtype=torch.float32,
                                        device="cpu")
        assert static_cache.tree_mask_update_method == "static"
        parent_probs = torch.ones(1, 1, dtype=dt)
        steps = []
        for d in range(depth):
            L = 1 if d == 0 else k
            logits = (torch.randn(1, L, V, generator=gen) * 3.0).to(dt)
            probs = torch.softmax(logits / T, dim=-1)
            tok, val, par = db.DraftModelBase._topk_flatten(holder, probs, parent_probs, k)
            tree_data.update(tok, val, par)
            mask = mask_cache.update_tree_mask(par, return_invert=False)
            smask = static_cache.update_tree_mask(par, return_invert=False)
            small[f"c{ci}/logits{d}"] = logits.float().numpy()
            steps.append(dict(tokens=tok.tolist(), parents=par.tolist(), probs=val.float().tolist(),
                              mask=mask[0, 0].to(torch.uint8).tolist(),
                              static_mask=smask[0, 0].to(torch.uint8).tolist()))
            parent_probs = val
        tree = ct.Tree(torch.tensor(7), dt)
        tree.add_nodes(*tree_data.get_data())
        full = tree.get_tree_data()
        full_mask = tree.create_attention_mask(prefix_length=3)
        probs_all = torch.tensor([n.cumulative_probability for n in tree.nodes], dtype=dt)
        distinct = len(set(probs_all.float().tolist())) == len(tree.nodes)
        keep_idx = tree.prune_to_top_n(keep)
        pruned = tree.get_tree_data()
        cases.append(dict(
            name=f"c{ci}", vocab=V, k=k, depth=depth, dtype=dtype, temperature=T, keep=keep, steps=steps,
            full=dict(token_ids=full["token_ids"].tolist(), depths=full["depths"].tolist(),
                      parent_indices=full["parent_indices"].tolist(),
                      probs=full["cumulative_probabilities"].float().tolist(),
                      mask=full_mask[0, 0].to(torch.uint8).tolist()),
            probs_distinct=distinct,
            pruned=dict(keep_idx=keep_idx.tolist(), token_ids=pruned["token_ids"].tolist(),
                        depths=pruned["depths"].tolist(), parent_indices=pruned["parent_indices"].tolist(),
                        probs=pruned["cumulative_probabilities"].float().tolist(),
                        children=[list(n.children) for n in tree.nodes],
                        leaves=list(tree.available_leaves),
                        mask=tree.create_attention_mask()[0, 0].to(torch.uint8).tolist(),
                        prefix=PREFIX, skip=SKIP,
                        mask_prefix_skip=tree.create_attention_mask(prefix_length=PREFIX, skip_nodes=SKIP)[0, 0]
                        .to(torch.uint8).tolist(),
                        data_skip={k_: v_.tolist() for k_, v_ in tree.get_tree_data(SKIP).items()
                                   if k_ != "cumulative_probabilities"})))
    (out_dir / "expand_cases.json").write_text(json.dumps({"cases": cases}))
    np.savez_compressed(out_dir / "expand_small.npz", **small)
    print(f"expand: {len(cases)} cases; cumulative probabilities all distinct: {[c['probs_distinct'] for c in cases]}")


def _rule_topk(scores_flat: torch.Tensor, k: int):
    """The k best flat indices under (value descending, index ascending): the order the CUDA path uses."""
    v = scores_flat.float()
    order = sorted(range(v.numel()), key=lambda i: (-float(v[i]), i)) if v.numel() <= 4096 else None
    if order is None:
        top = torch.topk(v, min(4 * k, v.numel()), sorted=True)
        cand = sorted(zip((-top.values).tolist(), top.indices.tolist()))
        assert cand[k - 1][0] < cand[-1][0] or len(cand) == v.numel(), "the tie at the cut is wider than the margin"
        return [i for _, i in cand[:k]]
    return order[:k]


def _rounding_margin(p64: torch.Tensor, dt: torch.dtype) -> float:
    """Smallest relative distance of the exact probabilities `p64` from a rounding boundary of `dt`: a
    probability computed with a relative error below it rounds to the same 16-bit value."""
    b = p64.to(dt)
    bits = b.view(torch.int16).to(torch.int32)
    up = (bits + 1).to(torch.int16).view(dt).double()
    dn = (bits - 1).to(torch.int16).view(dt).double()
    bd = b.double()
    edge = torch.minimum(((bd + up) / 2 - p64).abs(), ((bd + dn) / 2 - p64).abs())
    return float((edge / p64).min())


def gen_expand_chain(ref, out_dir: Path):
    """Config-3 expansions through the reference: per sequence ten levels of _topk_flatten at V = 128256, k = 16,
    TreeData -> Tree.add_nodes -> prune_to_top_n(64) -> get_tree_data / create_attention_mask.  Inputs are
    rebuilt from seeds (synthetic.expand_level_logits); only results are stored.  `rule_agrees` says whether the
    reference's choices coincide with the (value desc, index asc) order everywhere, i.e. whether torch.topk's
    unspecified tie order played no part: those sequences pin indices and structure, the others values only.

    Margin audit: discrete outputs come from floating-point inputs, so a seed is used only if none of the 2k best
    candidates of any level has an exact (fp64) probability within MARGIN (relative) of a 16-bit rounding
    boundary, and -- fp32, where indices are compared -- no two of them are closer than MARGIN; for 16-bit
    dtypes the reference's own CPU probabilities of those candidates must also equal the exactly rounded ones.
    Other seeds are skipped and the next one is tried.  The smallest margin met is stored."""
    from types import SimpleNamespace

    db, ct = ref["db"], ref["ct"]
    V, k, depth, keep = 128256, 16, 10, 64
    MARGIN = 5e-6
    seqs, skipped = [], []
    for dtype, first, want in (("bfloat16", 3000, 32), ("float32", 3100, 4)):
        dt = DT[dtype]
        seed, have = first - 1, 0
        while have < want:
            seed += 1
            holder = SimpleNamespace()
            tree_data = db.TreeData()
            parent_probs = torch.ones(1, 1, dtype=dt)
            levels, agrees, margin = [], True, float("inf")
            for d in range(depth):
                logits = synthetic.expand_level_logits(seed, d, k, V, dt)
                probs = torch.softmax(logits / 1.0, dim=-1)
                tok, val, par = db.DraftModelBase._topk_flatten(holder, probs, parent_probs, k)
                flat = (par * V + tok)[0].tolist()
                scores = (probs * parent_probs.unsqueeze(-1)).view(-1)
                agrees = agrees and flat == _rule_topk(scores, k)
                p64 = torch.softmax(logits.double(), dim=-1)
                s64 = (p64 * parent_probs.double().unsqueeze(-1)).view(-1)
                top = torch.topk(s64, 2 * k, sorted=True)
                if dt != torch.float32:
                    margin = min(margin, _rounding_margin(p64.view(-1)[top.indices], dt))
                    # torch's CPU softmax of a 16-bit tensor is itself up to ~1e-4 off on peaked rows (it adds up
                    # exponentials already rounded to the dtype), enough to round the other way now and then:
                    # such seeds pin the CPU build's rounding, not the reference's arithmetic, and are skipped
                    if not torch.equal(probs.view(-1)[top.indices], p64.view(-1)[top.indices].to(dt)):
                        margin = 0.0
                else:
                    margin = min(margin, float(((top.values[:-1] - top.values[1:]) / top.values[:-1]).min()))
                tree_data.update(tok, val, par)
                levels.append(dict(tokens=tok[0].tolist(), parents=par[0].tolist(), probs=val[0].float().tolist()))
                parent_probs = val
            if margin < MARGIN:
                skipped.append(seed)
                continue
            have += 1
            tree = ct.Tree(torch.tensor(11), dt)
            tree.add_nodes(*tree_data.get_data())
            cum = torch.tensor([n.cumulative_probability for n in tree.nodes], dtype=dt)
            keep_idx = tree.prune_to_top_n(keep).tolist()
            agrees_prune = keep_idx == _rule_topk(cum, keep)
            data = tree.get_tree_data()
            mask = tree.create_attention_mask()[0, 0]
            rows = [int(sum(1 << j for j in range(mask.shape[1]) if bool(mask[i, j]))) for i in range(mask.shape[0])]
            seqs.append(dict(seed=seed, dtype=dtype, levels=levels, rule_agrees=bool(agrees), min_margin=margin,
                             rule_agrees_prune=bool(agrees and agrees_prune),
                             pruned=dict(keep_idx=keep_idx, token_ids=data["token_ids"].tolist(),
                                         depths=data["depths"].tolist(),
                                         parent_indices=data["parent_indices"].tolist(),
                                         probs=data["cumulative_probabilities"].float().tolist(),
                                         children=[list(n.children) for n in tree.nodes], mask_rows=rows)))
    (out_dir / "expand_chain.json").write_text(json.dumps(
        dict(vocab=V, k=k, depth=depth, keep=keep, root_token=11, margin=MARGIN, skipped_seeds=skipped,
             sequences=seqs)))
    print(f"expand chain: {len(seqs)} sequences ({len(skipped)} seeds skipped by the margin audit, smallest margin "
          f"kept {min(s_['min_margin'] for s_ in seqs):.2e}); tie order irrelevant in "
          f"{sum(s_['rule_agrees'] for s_ in seqs)} expansions and {sum(s_['rule_agrees_prune'] for s_ in seqs)} prunes")


def gen_kv_hf(ref, out_dir: Path):
    """The HF-layout reorders, run by the reference's own methods on a stand-in object that carries the two
    attributes they touch (`key_cache`, `value_cache`; the installed transformers' cache classes no longer
    have them, so the classes themselves cannot be instantiated): TreeStaticCache.reorder_cache_with_offset
    (cache_utils.py:166-208) and TreeDynamicCache.reorder_cache_with_offset (:85-103), called as the
    generators call them (dim=2, classic_sd.py:254)."""
    from types import SimpleNamespace

    sys.path.insert(0, str(ROOT))
    from oracle.kv_oracle import checksum
    cu = ref["cu"]
    cases = []
    seed = 500
    for (layers, H, T, D, dtype) in [(5, 4, 96, 128, "bfloat16"), (3, 2, 40, 64, "float16"), (2, 1, 33, 8, "float32"),
                                      (28, 4, 160, 128, "bfloat16")]:
        for rep in range(3):
            seed += 1
            gen = torch.Generator().manual_seed(seed)
            ks = [torch.randn(1, H, T, D, generator=gen).to(DT[dtype]) for _ in range(layers)]
            vs = [torch.randn(1, H, T, D, generator=gen).to(DT[dtype]) for _ in range(layers)]
            tree_n = min(24, T // 2)
            offset = int(torch.randint(0, T - tree_n + 1, (1,), generator=gen))
            n = int(torch.randint(1, min(11, tree_n) + 1, (1,), generator=gen))
            beam = torch.sort(torch.randperm(tree_n - 1, generator=gen)[:n - 1] + 1).values
            beam = torch.cat([torch.zeros(1, dtype=torch.long), beam]) if rep != 2 else \
                torch.sort(torch.randperm(tree_n, generator=gen)[:n]).values
            before = checksum(torch.stack(ks + vs))
            st = SimpleNamespace(key_cache=[t.clone() for t in ks], value_cache=[t.clone() for t in vs])
            cu.TreeStaticCache.reorder_cache_with_offset(st, beam, new_chunk_len=tree_n, offset=offset, dim=2)
            dy = SimpleNamespace(key_cache=[t.clone() for t in ks], value_cache=[t.clone() for t in vs])
            cu.TreeDynamicCache.reorder_cache_with_offset(dy, beam, new_chunk_len=tree_n, offset=offset, dim=2)
            cases.append(dict(seed=seed, layers=layers, heads=H, tokens=T, head_dim=D, dtype=dtype, offset=offset,
                              tree_n=tree_n, beam=beam.tolist(), before=before,
                              static_after=checksum(torch.stack(st.key_cache + st.value_cache)),
                              dynamic_after=checksum(torch.stack(dy.key_cache + dy.value_cache)),
                              dynamic_tokens=int(dy.key_cache[0].shape[2])))
    (out_dir / "kv_hf_cases.json").write_text(json.dumps({"cases": cases}, indent=1))
    print(f"kv hf: {len(cases)} cases")


def gen_post(ref, out_dir: Path):
    """Tree.prune_to_depth and Tree.find_child_index of the reference on seeded trees: level-ordered ones, as
    Tree.add_nodes builds them, and the same trees after prune_to_top_n, whose nodes are numbered by rank and
    whose children lists are no longer in ascending order."""
    ct = ref["ct"]
    cases = []
    for seed in range(900, 912):
        gen = torch.Generator().manual_seed(seed)
        n = 20 + 7 * (seed % 5)
        st = synthetic.random_tree(n, 7, 4, 50, gen)   # a small vocabulary: siblings' tokens are probed by value
        probs = torch.rand(n, generator=gen).tolist()
        probs[0] = 1.0
        for i in range(1, n):  # cumulative probabilities fall along a path, as in a real draft tree
            probs[i] = probs[int(st.parents[i])] * (0.3 + 0.7 * probs[i])

        def build():
            t = ct.Tree(st.token_ids[0], torch.float32)
            for i in range(1, n):
                p = int(st.parents[i])
                t.nodes.append(ct.TreeNode(parent=p, token_id=int(st.token_ids[i]), cumulative_probability=probs[i],
                                           depth=int(st.depths[i])))
                t.nodes[p].children.append(i)
            t.current_size = n
            return t

        for ranked in (False, True):
            base = build()
            if ranked:
                base.prune_to_top_n(max(4, (2 * n) // 3))
            tree0 = dict(token_ids=[int(x.token_id) for x in base.nodes],
                         parents=[-1 if x.parent is None else int(x.parent) for x in base.nodes],
                         depths=[int(x.depth) for x in base.nodes], children=[list(x.children) for x in base.nodes])
            finds = []
            for node in range(0, len(base.nodes), 3):
                for tok in {int(base.nodes[c].token_id) for c in base.nodes[node].children} | {49, 0}:
                    finds.append([node, tok, int(base.find_child_index(node, tok))])
            prunes = []
            for d in range(0, int(base.get_depth()) + 2):
                t = build()
                if ranked:
                    t.prune_to_top_n(max(4, (2 * n) // 3))
                keep = t.prune_to_depth(d).tolist()
                prunes.append(dict(max_depth=d, keep=keep, token_ids=[int(x.token_id) for x in t.nodes],
                                   parents=[-1 if x.parent is None else int(x.parent) for x in t.nodes],
                                   depths=[int(x.depth) for x in t.nodes], children=[list(x.children) for x in t.nodes],
                                   leaves=list(t.available_leaves)))
            cases.append(dict(seed=seed, ranked=ranked, tree=tree0, finds=finds, prunes=prunes))
    (out_dir / "post_cases.json").write_text(json.dumps({"cases": cases}))
    print(f"post: {len(cases)} trees, {sum(len(c['prunes']) for c in cases)} prunes, "
          f"{sum(len(c['finds']) for c in cases)} child look-ups")


def gen_pages(ref, out_dir: Path):
    """A scripted generation loop over the reference's KvCachePool / RequestKvCache (CPU, a pool of one float per
    row: only the bookkeeping matters): several requests share one pool; every step each request is cropped to
    the length a verification left it with (all requests first), then grows by the next tree (requests in
    order).  Page lists, lengths and the free count after every step are stored."""
    cm = ref["cm"]
    scripts = []
    for seed, (B, num_pages, page_len, tree_n, steps) in enumerate([(3, 40, 4, 7, 6), (8, 200, 16, 24, 8),
                                                                    (1, 30, 16, 64, 5), (16, 600, 16, 64, 6)]):
        gen = torch.Generator().manual_seed(600 + seed)
        pool = cm.KvCachePool(num_pages, 1, 1, 1, page_len, torch.float32, "cpu")
        init = [int(torch.randint(1, 3 * page_len, (1,), generator=gen)) for _ in range(B)]
        reqs = [cm.RequestKvCache(pool, page_len, n) for n in init]
        rec = []

        def snap():
            return dict(pages=[list(r.kv_page_indices) for r in reqs], kv_len=[r.kv_len for r in reqs],
                        last=[r.kv_last_page_len for r in reqs], free=int(pool.num_free_pages()))

        first = snap()
        for _ in range(steps):
            for r in reqs:
                r.increment(tree_n)
            grown = snap()
            kept = [int(torch.randint(1, tree_n + 1, (1,), generator=gen)) for _ in range(B)]
            new_len = [r.kv_len - tree_n + k for r, k in zip(reqs, kept)]
            for r, n in zip(reqs, new_len):
                r.crop(n)
            rec.append(dict(grown=grown, new_len=new_len, cropped=snap()))
        scripts.append(dict(batch=B, num_pages=num_pages, page_len=page_len, tree_n=tree_n, init=init, first=first,
                            steps=rec))
    (out_dir / "pages_cases.json").write_text(json.dumps({"scripts": scripts}))
    print(f"pages: {len(scripts)} scripted loops, {sum(len(s_['steps']) for s_ in scripts)} steps")


ATTN_CASES = [  # (seed, tree nodes, prefix rows, query heads, KV heads, dtype)
    (3100, 12, 37, 4, 2, "bfloat16"), (3101, 16, 0, 4, 4, "bfloat16"), (3102, 20, 150, 7, 1, "float16"),
    (3103, 1, 9, 4, 1, "bfloat16"), (3104, 17, 64, 6, 3, "float32"),
]


def gen_attention(ref, out_dir: Path):
    """The attention the reference's default (HF) path computes over a tree: transformers' SDPA attention --
    `repeat_kv`, then `torch.nn.functional.scaled_dot_product_attention` with an additive mask -- fed with the
    mask the reference builds (`Tree.create_attention_mask(prefix_length)` and `invert_mask`,
    specdecodes/models/utils/cpu_tree.py:263, specdecodes/models/utils/utils.py:4-6).  Stored per case: the
    result computed in fp32 from the inputs (what pins the oracle) and the result in the inputs' own type (what
    the reference's model would hold).  The inputs are regenerated from the seed (synthetic.attention_case)."""
    import specdecodes.models.utils.utils as ru
    arrays, cases = {}, []
    for seed, n_q, prefix, hq, hkv, dt in ATTN_CASES:
        dtype = getattr(torch, dt)
        st, q, k, v = synthetic.attention_case(seed, n_q, prefix, hq, hkv, dtype)
        rt = ref_tree(ref["ct"], st)
        mask = rt.create_attention_mask(prefix_length=prefix)  # bool [1, 1, n_q, prefix + n_q]
        assert tuple(mask.shape) == (1, 1, n_q, prefix + n_q)

        def sdpa(t):
            qq = q.to(t).permute(1, 0, 2)[None]                      # [1, HQ, n_q, D]
            kk = k.to(t).permute(1, 0, 2)[None].repeat_interleave(hq // hkv, dim=1)  # repeat_kv
            vv = v.to(t).permute(1, 0, 2)[None].repeat_interleave(hq // hkv, dim=1)
            o = torch.nn.functional.scaled_dot_product_attention(qq, kk, vv, attn_mask=ru.invert_mask(mask, t))
            return o[0].permute(1, 0, 2).contiguous()                 # [n_q, HQ, D]

        name = f"a{seed}"
        arrays[name + "/exact"] = sdpa(torch.float32).numpy()
        arrays[name + "/native"] = sdpa(dtype).to(torch.float16 if dtype == torch.float16 else torch.bfloat16).view(
            torch.int16).numpy()  # the 16-bit patterns (bf16 for the fp32 case)
        arrays[name + "/mask"] = mask[0, 0].numpy()
        cases.append(dict(name=name, seed=seed, n_q=n_q, prefix=prefix, q_heads=hq, kv_heads=hkv, dtype=dt))
    np.savez_compressed(out_dir / "attention_small.npz", **arrays)
    (out_dir / "attention_cases.json").write_text(json.dumps(dict(
        generator="tests/golden/make_golden.py --only attention", cases=cases), indent=1))
    print(f"attention: {len(cases)} cases")


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--reference", required=True, help="checkout of the unmodified reference repository")
    ap.add_argument("--only", default=None)
    args = ap.parse_args()
    ref = import_reference(args.reference)
    torch.set_num_threads(8)
    if args.only in (None, "verify"):
        gen_verify(ref, HERE)
    if args.only in (None, "expand"):
        gen_expand(ref, HERE)
    if args.only in (None, "expand_chain"):
        gen_expand_chain(ref, HERE)
    if args.only in (None, "kv"):
        gen_kv(ref, HERE)
    if args.only in (None, "kv_hf"):
        gen_kv_hf(ref, HERE)
    if args.only in (None, "post"):
        gen_post(ref, HERE)
    if args.only in (None, "pages"):
        gen_pages(ref, HERE)
    if args.only in (None, "attention"):
        gen_attention(ref, HERE)
    if args.only in (None, "sampled"):
        gen_sampled(ref, HERE)
    if args.only in (None, "lossy_unit"):
        gen_lossy_unit(ref, args.reference, HERE)


if __name__ == "__main__":
    main()
