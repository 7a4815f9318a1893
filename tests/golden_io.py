"""Load the committed golden fixtures (tests/golden/) back into tensors."""
from __future__ import annotations

import json
from functools import lru_cache
from pathlib import Path

import numpy as np
import torch

from subspec_b200 import synthetic

GOLDEN = Path(__file__).resolve().parent / "golden"
DT = {"float32": torch.float32, "bfloat16": torch.bfloat16, "float16": torch.float16}


@lru_cache(maxsize=None)
def verify_cases():
    return json.loads((GOLDEN / "verify_cases.json").read_text())["cases"]


@lru_cache(maxsize=None)
def _verify_small():
    return dict(np.load(GOLDEN / "verify_small.npz"))


@lru_cache(maxsize=4)
def _config1(seed: int, dtype: str, peaked: bool):
    return synthetic.config1_case(seed, dtype=DT[dtype], peaked=peaked)


def verify_input(case):
    """(SynthTree over the whole tree, logits [rows, V] in the case's dtype) for one golden verify case."""
    if case["inline"]:
        z = _verify_small()
        name = case["input"]
        tok = torch.from_numpy(z[name + "/tokens"])
        par = torch.from_numpy(z[name + "/parents"])
        depth = torch.zeros_like(par)
        for i in range(1, len(par)):
            depth[i] = depth[par[i]] + 1
        tree = synthetic.SynthTree(tok, par, depth)
        logits = torch.from_numpy(z[name + "/logits"]).to(DT[case["dtype"]])
    else:
        tree, logits = _config1(case["seed"], case["dtype"], case["peaked"])
    return tree, logits[:case["rows"]]


@lru_cache(maxsize=None)
def lossy_unit_cases():
    return json.loads((GOLDEN / "lossy_unit_cases.json").read_text())["cases"]


@lru_cache(maxsize=None)
def kv_cases():
    return json.loads((GOLDEN / "kv_cases.json").read_text())["cases"]


def kv_pool(case) -> torch.Tensor:
    """The pool contents the golden generator started from (same seed, same draw order)."""
    gen = torch.Generator().manual_seed(case["seed"])
    shape = (case["layers"], case["pages"], 2, case["page_len"], case["heads"], case["head_dim"])
    return torch.randn(shape, generator=gen).to(DT[case["dtype"]])


@lru_cache(maxsize=None)
def post_cases():
    """Tree.prune_to_depth / Tree.find_child_index results of the reference on seeded trees."""
    return json.loads((GOLDEN / "post_cases.json").read_text())["cases"]


@lru_cache(maxsize=None)
def pages_scripts():
    """Page lists the reference's KvCachePool / RequestKvCache went through in scripted generation loops."""
    return json.loads((GOLDEN / "pages_cases.json").read_text())["scripts"]


@lru_cache(maxsize=None)
def kv_hf_cases():
    return json.loads((GOLDEN / "kv_hf_cases.json").read_text())["cases"]


def kv_hf_tensors(case):
    """(key tensors, value tensors), each a list of [1, H, T, D], as the golden generator drew them."""
    gen = torch.Generator().manual_seed(case["seed"])
    shape = (1, case["heads"], case["tokens"], case["head_dim"])
    ks = [torch.randn(shape, generator=gen).to(DT[case["dtype"]]) for _ in range(case["layers"])]
    vs = [torch.randn(shape, generator=gen).to(DT[case["dtype"]]) for _ in range(case["layers"])]
    return ks, vs


@lru_cache(maxsize=None)
def expand_chain():
    """Config-3 expansions run by the reference (ten levels, V = 128256, k = 16, pruned to 64 nodes)."""
    return json.loads((GOLDEN / "expand_chain.json").read_text())


def chain_logits(chain, seq, level: int) -> torch.Tensor:
    """[1, leaves, vocab] draft logits of one level of one golden sequence, rebuilt from its seed."""
    return synthetic.expand_level_logits(seq["seed"], level, chain["k"], chain["vocab"], DT[seq["dtype"]])


@lru_cache(maxsize=None)
def expand_cases():
    return json.loads((GOLDEN / "expand_cases.json").read_text())["cases"]


@lru_cache(maxsize=None)
def _expand_small():
    return dict(np.load(GOLDEN / "expand_small.npz"))


def expand_logits(case, step: int) -> torch.Tensor:
    """[1, leaves, vocab] draft logits of one depth step, in the case's dtype."""
    return torch.from_numpy(_expand_small()[f"{case['name']}/logits{step}"]).to(DT[case["dtype"]])


@lru_cache(maxsize=None)
def sampled_cases():
    return json.loads((GOLDEN / "sampled_cases.json").read_text())["cases"]


def sampled_input(case):
    """(SynthTree, logits [n, V] in the case's dtype) of one sampled-verification case; the uniforms the
    reference ran with are stored in the case itself."""
    tree, logits, _ = synthetic.sampled_case(case["seed"], case["nodes"], case["depth"], case["branch"],
                                             case["vocab"], DT[case["dtype"]])
    return tree, logits


def sampled_processors(case):
    """The warper list the reference builds for these parameters (generators/base.py:42-64)."""
    from transformers.generation.logits_process import (LogitsProcessorList, TemperatureLogitsWarper,
                                                        TopKLogitsWarper, TopPLogitsWarper)
    procs = LogitsProcessorList()
    if case["temperature"] != 1.0:
        procs.append(TemperatureLogitsWarper(case["temperature"]))
    if case["top_k"]:
        procs.append(TopKLogitsWarper(top_k=case["top_k"]))
    if case["top_p"] < 1.0:
        procs.append(TopPLogitsWarper(top_p=case["top_p"]))
    return procs


@lru_cache(maxsize=None)
def attention_cases():
    return json.loads((GOLDEN / "attention_cases.json").read_text())["cases"]


@lru_cache(maxsize=None)
def _attention_small():
    return dict(np.load(GOLDEN / "attention_small.npz"))


def attention_golden(case):
    """(tree, q, k, v in the case's type, bool mask [n_q, prefix + n_q], SDPA result computed in fp32,
    SDPA result computed in the case's own type as fp32 values) of one golden attention case."""
    dtype = DT[case["dtype"]]
    tree, q, k, v = synthetic.attention_case(case["seed"], case["n_q"], case["prefix"], case["q_heads"],
                                             case["kv_heads"], dtype)
    z = _attention_small()
    name = case["name"]
    native16 = torch.from_numpy(z[name + "/native"]).view(torch.float16 if dtype == torch.float16 else torch.bfloat16)
    return tree, q, k, v, torch.from_numpy(z[name + "/mask"]), torch.from_numpy(z[name + "/exact"]), native16.float()
