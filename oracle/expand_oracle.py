"""CPU oracle for draft-tree expansion.  TEST INFRASTRUCTURE ONLY.

Restates the reference's expansion path on torch CPU tensors and plain Python; only tests/,
__graft_entry__.smoke() and bench.py's CPU baseline may import it.  Pinned against the reference:
tests/golden/expand_cases.json + expand_small.npz hold what the reference's own _topk_flatten,
TreeData, TreeMaskCache and Tree (add_nodes, prune_to_top_n, get_tree_data,
create_attention_mask) produce on seeded inputs (tests/golden/make_golden.py);
tests/test_oracle_golden.py checks this module against them.

  draft_probs        softmax(logits / T) in the model dtype      draft_models/classic_sd.py:10-16
  topk_flatten       DraftModelBase._topk_flatten                draft_models/base.py:281-305
  same_topk          the reference's own tie-tolerant check       analysis/bench_topk_sampling.py:146-163
  FlatTree           Tree.add_nodes / prune_to_top_n / get_tree_data / create_attention_mask
                                                                  models/utils/cpu_tree.py:69-117, 175-215, 238-286
  mask_rows          TreeMaskCache.update_tree_mask (dynamic)     draft_models/base.py:93-110
"""
from __future__ import annotations

from typing import List, Sequence, Tuple

import torch


def draft_probs(logits: torch.Tensor, temperature: float = 1.0) -> torch.Tensor:
    return torch.softmax(logits / temperature, dim=-1)


def topk_flatten(sampled_probs: torch.Tensor, parent_probs: torch.Tensor, k: int):
    """(token_ids [B,k], topk_probs [B,k], parent_indices [B,k]); tie order is whatever torch.topk gives."""
    B, L, V = sampled_probs.shape
    k = min(int(k), int(V))
    scores = (sampled_probs * parent_probs.unsqueeze(-1)).view(B, -1)
    vals, idx = torch.topk(scores, k, dim=1, sorted=True)
    return (idx % V).long(), vals, (idx // V).long()


def topk_flatten_ordered(sampled_probs: torch.Tensor, parent_probs: torch.Tensor, k: int):
    """`topk_flatten` with ties in a stated order: (value descending, flat index ascending), the order the CUDA
    path documents.  torch.topk leaves the order of equal values open, so against the reference only the values
    can be compared where scores tie; against this function the indices can be compared too."""
    B, L, V = sampled_probs.shape
    k = min(int(k), int(V))
    scores = (sampled_probs * parent_probs.unsqueeze(-1)).view(B, -1)
    toks, vals, pars = [], [], []
    for b in range(B):
        row = scores[b].float()
        m = min(row.numel(), 8 * k)
        while True:
            top = torch.topk(row, m, sorted=True)
            if m == row.numel() or float(top.values[-1]) < float(top.values[k - 1]):
                break  # every score equal to the k-th is among the m candidates
            m = min(row.numel(), 4 * m)
        order = sorted(range(m), key=lambda i: (-float(top.values[i]), int(top.indices[i])))[:k]
        idx = top.indices[order]
        toks.append(idx % V)
        pars.append(idx // V)
        vals.append(scores[b][idx])
    return torch.stack(toks).long(), torch.stack(vals), torch.stack(pars).long()


def same_topk(scores_flat: torch.Tensor, ref_vals: torch.Tensor, got_vals: torch.Tensor, got_flat_idx: torch.Tensor):
    """Tie-tolerant equality: the sorted values are bit-equal, every returned index really carries its
    value, and no index is returned twice.  (Which members of a tied group appear is not pinned.)"""
    if not torch.equal(ref_vals, got_vals):
        return False
    for b in range(scores_flat.shape[0]):
        if not torch.equal(scores_flat[b][got_flat_idx[b]], got_vals[b]):
            return False
        if len(set(got_flat_idx[b].tolist())) != got_flat_idx.shape[1]:
            return False
    return True


class FlatTree:
    """Parent/child lists only: just enough to restate numbering, pruning and the ancestor mask."""

    def __init__(self, root_token: int):
        self.token = [int(root_token)]
        self.parent = [-1]
        self.depth = [0]
        self.prob = [1.0]
        self.children: List[List[int]] = [[]]
        self.leaves = [0]

    def add_nodes(self, token_ids, token_probs, local_parents) -> None:
        """Inputs [1, depth, k]; the parent of sample i at level d is the local_parents[d][i]-th leaf of level d-1."""
        toks, probs, pars = token_ids[0].tolist(), token_probs[0].tolist(), local_parents[0].tolist()
        for d in range(len(toks)):
            base = len(self.token)
            new = []
            for i, (p_local, t, pr) in enumerate(zip(pars[d], toks[d], probs[d])):
                p = self.leaves[p_local]
                self.token.append(t)
                self.parent.append(p)
                self.depth.append(self.depth[p] + 1)
                self.prob.append(pr)
                self.children.append([])
                self.children[p].append(base + i)
                new.append(base + i)
            self.leaves = new

    def prune_to_top_n(self, n: int, dtype=torch.float32, ordered: bool = False) -> List[int]:
        """`ordered`: ties by ascending node index (the CUDA path's rule) instead of torch.topk's open order."""
        if n == -1 or len(self.token) <= n:
            return list(range(len(self.token)))
        probs = torch.tensor(self.prob, dtype=dtype)
        if ordered:
            keep = sorted(range(len(self.token)), key=lambda i: (-float(probs[i]), i))[:n]
        else:
            keep = torch.topk(probs, k=n, sorted=True).indices.tolist()
        new_of = {o: i for i, o in enumerate(keep)}
        self.children = [[new_of[c] for c in self.children[o] if c in new_of] for o in keep]
        self.parent = [new_of.get(self.parent[o], -1) if self.parent[o] >= 0 else -1 for o in keep]
        self.token = [self.token[o] for o in keep]
        self.depth = [self.depth[o] for o in keep]
        self.prob = [self.prob[o] for o in keep]
        self.leaves = [i for i in range(len(keep)) if not self.children[i]]
        return keep

    def mask(self) -> torch.Tensor:
        n = len(self.token)
        m = torch.zeros(n, n, dtype=torch.bool)
        for i in range(n):
            j = i
            while j >= 0:
                m[i, j] = True
                j = self.parent[j]
        return m


def mask_rows(prev: torch.Tensor, parents: Sequence[int]) -> torch.Tensor:
    """Draft-side mask of a new level: row i = prev[parents[i]] followed by a one-hot for itself."""
    k = len(parents)
    return torch.cat([prev[list(parents)], torch.eye(k, dtype=torch.bool)], dim=1)
