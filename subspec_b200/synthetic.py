"""Seeded synthetic inputs with the shapes and value distributions of the benchmark configs.

The reference measures on MT-Bench prompts with real checkpoints; neither is
available offline, so these generators stand in: random draft trees, Gaussian
target logits with the drafted child boosted at a fraction of the nodes, random
page tables.  Everything is driven by an explicit `torch.Generator`, so the same
seed gives the same tensors on any machine with the same torch build.
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import List, Optional, Tuple

import torch


@dataclass
class SynthTree:
    token_ids: torch.Tensor  # [n] int64, node 0 is the root
    parents: torch.Tensor    # [n] int64, -1 for the root, parent < child
    depths: torch.Tensor     # [n] int64

    @property
    def n(self) -> int:
        return int(self.token_ids.numel())

    def children(self) -> List[List[int]]:
        ch: List[List[int]] = [[] for _ in range(self.n)]
        for i, p in enumerate(self.parents.tolist()):
            if p >= 0:
                ch[p].append(i)
        return ch


def random_tree(n_nodes: int, max_depth: int, max_branch: int, vocab: int, gen: torch.Generator) -> SynthTree:
    """Grow a tree one node at a time under a uniformly chosen eligible parent
    (fewer than `max_branch` children, depth below `max_depth`), then renumber in
    level order so that parent < child, as the reference's `Tree.add_nodes` numbers its nodes."""
    parent = [-1]
    depth = [0]
    nchild = [0]
    for _ in range(1, n_nodes):
        elig = [i for i in range(len(parent)) if nchild[i] < max_branch and depth[i] < max_depth]
        p = elig[int(torch.randint(len(elig), (1,), generator=gen))]
        parent.append(p)
        depth.append(depth[p] + 1)
        nchild.append(0)
        nchild[p] += 1
    order = sorted(range(n_nodes), key=lambda i: (depth[i], i))
    new_of = {old: new for new, old in enumerate(order)}
    parents = torch.tensor([-1 if parent[o] < 0 else new_of[parent[o]] for o in order], dtype=torch.long)
    depths = torch.tensor([depth[o] for o in order], dtype=torch.long)
    tokens = torch.randint(vocab, (n_nodes,), generator=gen, dtype=torch.long)
    # sibling tokens must differ (a draft never proposes the same token twice under one node)
    seen = {}
    for i in range(1, n_nodes):
        key = int(parents[i])
        used = seen.setdefault(key, set())
        while int(tokens[i]) in used:
            tokens[i] = (int(tokens[i]) + 1) % vocab
        used.add(int(tokens[i]))
    return SynthTree(tokens, parents, depths)


def verify_logits(tree: SynthTree, vocab: int, gen: torch.Generator, *, sigma: float = 3.0, boost: float = 6.0,
                  boost_frac: float = 0.6, dtype: torch.dtype = torch.float32, peaked: bool = False,
                  sharp_frac: float = 0.3, device: Optional[torch.device] = None) -> torch.Tensor:
    """Target logits [n, vocab]: sigma * randn, with one random child's token boosted at
    `boost_frac` of the internal nodes.

    `peaked=False` is the literal benchmark distribution (+`boost` on the child's
    logit).  With V ~ 150k the row maximum sits near 4.4 sigma, so a +6 boost almost
    never wins the argmax and the normalised entropy stays near 0.6: the accept
    walk and the entropy gate are barely exercised.  `peaked=True` is the parity
    variant: the boosted child is set to row_max + 4, and `sharp_frac` of the
    rows are scaled by 4 so their entropy drops below the usual 0.3 threshold.
    """
    n = tree.n
    g_dev = gen.device
    x = torch.randn((n, vocab), generator=gen, device=g_dev, dtype=torch.float32) * sigma
    children = tree.children()
    cpu_gen = gen if g_dev.type == "cpu" else torch.Generator().manual_seed(int(gen.initial_seed()) + 1)
    for u in range(n):
        if not children[u]:
            continue
        if float(torch.rand((), generator=cpu_gen)) < boost_frac:
            c = children[u][int(torch.randint(len(children[u]), (1,), generator=cpu_gen))]
            t = int(tree.token_ids[c])
            if peaked:
                x[u, t] = x[u].max() + 4.0
            else:
                x[u, t] += boost
    if peaked:
        sharp = torch.rand(n, generator=cpu_gen) < sharp_frac
        x[sharp.to(x.device)] *= 4.0
    x = x.to(dtype)
    return x if device is None else x.to(device)


def config1_case(seed: int, *, vocab: int = 152064, n_nodes: int = 64, max_depth: int = 8, max_branch: int = 4,
                 dtype: torch.dtype = torch.float32, peaked: bool = False) -> Tuple[SynthTree, torch.Tensor]:
    """Config 1 / 5 verify input: one 64-node tree and its [n, vocab] target logits."""
    gen = torch.Generator().manual_seed(seed)
    tree = random_tree(n_nodes, max_depth, max_branch, vocab, gen)
    return tree, verify_logits(tree, vocab, gen, dtype=dtype, peaked=peaked)


def sampled_case(seed: int, n_nodes: int, max_depth: int, max_branch: int, vocab: int, dtype: torch.dtype):
    """Input of one sampled verification: a tree, its [n, vocab] target logits (drafted tokens likely enough
    to be drawn now and then) and one uniform per node."""
    gen = torch.Generator().manual_seed(seed)
    tree = random_tree(n_nodes, max_depth, max_branch, vocab, gen)
    logits = verify_logits(tree, vocab, gen, dtype=dtype, peaked=True, sigma=2.0)
    uniforms = torch.rand(n_nodes, generator=gen)
    return tree, logits, uniforms


def expand_level_logits(seed: int, level: int, k: int, vocab: int, dtype: torch.dtype, sigma: float = 3.0) -> torch.Tensor:
    """Draft logits [1, leaves, vocab] of one depth step of one sequence (config 3: sigma * randn; one leaf on
    the first step, k afterwards).  Every (sequence seed, level) has a generator of its own, so a test can
    rebuild any level without drawing the ones before it."""
    gen = torch.Generator().manual_seed(int(seed) * 1000 + int(level))
    leaves = 1 if level == 0 else int(k)
    return (torch.randn(1, leaves, vocab, generator=gen) * sigma).to(dtype)


def config5_wave(seq_ids, variant: str, device, *, nodes: int = 64, vocab: int = 152064, with_logits: bool = True):
    """Trees (host) and bf16 logits [len(seq_ids), nodes, vocab] (on `device`) of the sharded-step workload for
    the given global sequence ids; everything is seeded by the id, so any rank can rebuild any sequence.
    `variant` "literal": 3 * randn with one drafted child boosted by +6 at 60 % of the inner nodes;
    "peaked": that child set to the row maximum + 4, so that walks, gates and compaction have work to do."""
    trees = []
    for sid in seq_ids:
        gen = torch.Generator().manual_seed(1_000_003 * 5 + sid)
        trees.append(random_tree(nodes, 8, 4, vocab, gen))
    if not with_logits:
        return trees, None
    S = len(seq_ids)
    dgen = torch.Generator(device=device).manual_seed(7_000_001 + seq_ids[0])
    logits = torch.empty(S, nodes, vocab, dtype=torch.bfloat16, device=device)
    for b in range(S):  # fp32 noise generated one sequence at a time to bound the transient footprint
        logits[b] = (torch.randn(nodes, vocab, generator=dgen, device=device) * 3.0).to(torch.bfloat16)
    bi, ui, ti = [], [], []
    for b, (sid, st) in enumerate(zip(seq_ids, trees)):
        cgen = torch.Generator().manual_seed(9_000_011 + sid)
        ch = st.children()
        for u in range(st.n):
            if ch[u] and float(torch.rand((), generator=cgen)) < 0.6:
                c = ch[u][int(torch.randint(len(ch[u]), (1,), generator=cgen))]
                bi.append(b)
                ui.append(u)
                ti.append(int(st.token_ids[c]))
    bi, ui, ti = (torch.tensor(x, device=device) for x in (bi, ui, ti))
    if variant == "peaked":
        rowmax = logits.float().amax(dim=-1)
        logits[bi, ui, ti] = (rowmax[bi, ui] + 4.0).to(torch.bfloat16)
    else:
        logits[bi, ui, ti] = (logits[bi, ui, ti].float() + 6.0).to(torch.bfloat16)
    return trees, logits


def random_page_table(batch: int, pages_per_seq: int, gen: torch.Generator) -> torch.Tensor:
    """[batch, pages_per_seq] int32: a random permutation of the pool's pages split across sequences."""
    perm = torch.randperm(batch * pages_per_seq, generator=gen)
    return perm.reshape(batch, pages_per_seq).to(torch.int32)


def w4a16_case(n: int, k: int, m: int, seed: int, group: int = 64):
    """Synthetic HQQ-style 4-bit linear: int32 words of eight nibbles (nibble i of word j = q[n, 8 j + i]),
    scale ~U(0.005, 0.02) and zero ~U(0, 15) in fp16 per group of `group` inputs, activations ~N(0, 1) bf16."""
    gen = torch.Generator().manual_seed(seed)
    q = torch.randint(0, 16, (n, k // 8, 8), generator=gen, dtype=torch.int64)
    qweight = (q << (torch.arange(8) * 4)).sum(-1).to(torch.int32)
    scale = (torch.rand(n, k // group, generator=gen) * 0.015 + 0.005).half()
    zero = (torch.rand(n, k // group, generator=gen) * 15.0).half()
    x = torch.randn(m, k, generator=gen).to(torch.bfloat16)
    return qweight, scale, zero, x


def attention_case(seed: int, n_q: int, prefix: int, q_heads: int, kv_heads: int, dtype: torch.dtype, head_dim: int = 128):
    """Seeded inputs of one tree-attention problem: a random tree of `n_q` nodes behind `prefix` cache rows.

    Returns (tree, q [n_q, q_heads, D], k and v [prefix + n_q, kv_heads, D]) in `dtype`, rows in cache order."""
    gen = torch.Generator().manual_seed(seed)
    tree = random_tree(n_q, 6, 3, 1000, gen)
    n = prefix + n_q
    q = torch.randn(n_q, q_heads, head_dim, generator=gen).to(dtype)
    k = torch.randn(n, kv_heads, head_dim, generator=gen).to(dtype)
    v = torch.randn(n, kv_heads, head_dim, generator=gen).to(dtype)
    return tree, q, k, v
