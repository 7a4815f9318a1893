"""Draft token tree: a flat (struct-of-arrays) tree with the reference's `Tree` interface.

The reference keeps a Python list of `TreeNode` objects
(specdecodes/models/utils/cpu_tree.py:4-29, 32-324).  Here the tree is a set of
parallel arrays (token, parent, depth, cumulative probability, children CSR) --
the same arrays the CUDA kernels consume -- and `tree.nodes[i]` is a thin view
onto row i, so code written against the reference (`tree.nodes[v].children`,
`tree.get_tree_data()`, `tree.create_attention_mask()` ...) keeps working.

Node numbering follows the reference: root is 0; `add_nodes` appends level by
level in the order given (cpu_tree.py:87-117); `prune_to_top_n` renumbers by
rank of cumulative probability (cpu_tree.py:175-215); `prune_to_depth` keeps
the original relative order (cpu_tree.py:119-173).
"""
from __future__ import annotations

from typing import Dict, List, Optional

import numpy as np
import torch


class _NodeView:
    """Read/write view of one node; mirrors the fields of the reference's TreeNode."""

    __slots__ = ("_t", "_i")

    def __init__(self, tree: "Tree", index: int):
        self._t = tree
        self._i = index

    @property
    def parent(self) -> Optional[int]:
        p = self._t._parent[self._i]
        return None if p < 0 else p

    @property
    def children(self) -> List[int]:
        return self._t._children[self._i]

    @property
    def depth(self) -> int:
        return self._t._depth[self._i]

    @property
    def token_id(self) -> int:
        return self._t._token[self._i]

    @property
    def cumulative_probability(self) -> float:
        return self._t._prob[self._i]

    @property
    def has_been_sampled(self) -> bool:
        return self._t._sampled[self._i]

    @has_been_sampled.setter
    def has_been_sampled(self, v: bool) -> None:
        self._t._sampled[self._i] = bool(v)

    def __repr__(self) -> str:
        return (f"TreeNode(token_id={self.token_id}, cumulative_probability={self.cumulative_probability:.4f}, "
                f"depth={self.depth}, parent={self.parent})")


class _NodeList:
    __slots__ = ("_t",)

    def __init__(self, tree: "Tree"):
        self._t = tree

    def __len__(self) -> int:
        return self._t.current_size

    def __getitem__(self, i: int) -> _NodeView:
        n = self._t.current_size
        if i < 0:
            i += n
        if not 0 <= i < n:
            raise IndexError(i)
        return _NodeView(self._t, i)

    def __iter__(self):
        return (_NodeView(self._t, i) for i in range(self._t.current_size))


class Tree:
    """Flat draft tree with the interface of the reference's `Tree` (cpu_tree.py:32-324)."""

    def __init__(self, root_token_id, prob_dtype: torch.dtype = torch.float32):
        self.prob_dtype = prob_dtype
        root = int(root_token_id.item()) if hasattr(root_token_id, "item") else int(root_token_id)
        self._token: List[int] = [root]
        self._parent: List[int] = [-1]
        self._depth: List[int] = [0]
        self._prob: List[float] = [1.0]
        self._sampled: List[bool] = [False]
        self._children: List[List[int]] = [[]]
        self.current_size = 1
        self.available_leaves: List[int] = [0]

    # -- construction -----------------------------------------------------------
    @classmethod
    def from_arrays(cls, token_ids, parents, probs=None, prob_dtype: torch.dtype = torch.float32) -> "Tree":
        """Build a tree from flat arrays (parents[0] == -1, parents[i] < i is not required)."""
        token_ids = [int(t) for t in token_ids]
        parents = [int(p) for p in parents]
        t = cls(token_ids[0], prob_dtype)
        n = len(token_ids)
        t._token = token_ids
        t._parent = [-1 if p < 0 else p for p in parents]
        t._prob = [1.0] * n if probs is None else [float(x) for x in probs]
        t._sampled = [False] * n
        t._children = [[] for _ in range(n)]
        for i, p in enumerate(t._parent):
            if p >= 0:
                t._children[p].append(i)
        depth = [0] * n
        for i in range(n):
            d, p, guard = 0, t._parent[i], 0
            while p >= 0:
                d += 1
                p = t._parent[p]
                guard += 1
                if guard > n:
                    raise ValueError("parent array contains a cycle")
            depth[i] = d
        t._depth = depth
        t.current_size = n
        t._refresh_leaves()
        return t

    @property
    def nodes(self) -> _NodeList:
        return _NodeList(self)

    def add_nodes(self, token_ids: torch.Tensor, token_probs: torch.Tensor, local_parent_indices: torch.Tensor):
        """Append `total_depth` levels of `num_samples` nodes (inputs are [1, total_depth, num_samples]).

        The parent of sample i at level d is the `local_parent_indices[0, d, i]`-th
        leaf of the previous level (cpu_tree.py:69-117).
        """
        batch_size, total_depth, _ = token_ids.shape
        assert batch_size == 1, "Currently only batch_size=1 is supported."
        par = local_parent_indices.detach().to("cpu").tolist()[0]
        tok = token_ids.detach().to("cpu").tolist()[0]
        prb = token_probs.detach().to("cpu").tolist()[0]
        for d in range(total_depth):
            for leaf in self.available_leaves:
                self._sampled[leaf] = True
            base = self.current_size
            leaves = self.available_leaves
            new_leaves = []
            for i, (p_local, t, pr) in enumerate(zip(par[d], tok[d], prb[d])):
                p = leaves[p_local]
                idx = base + i
                self._token.append(t)
                self._parent.append(p)
                self._depth.append(self._depth[p] + 1)
                self._prob.append(pr)
                self._sampled.append(False)
                self._children.append([])
                self._children[p].append(idx)
                new_leaves.append(idx)
            self.current_size = len(self._token)
            self.available_leaves = new_leaves

    # -- pruning -----------------------------------------------------------------
    def _refresh_leaves(self) -> None:
        for i in range(self.current_size):
            if not self._children[i]:
                self._sampled[i] = False
        self.available_leaves = [i for i in range(self.current_size) if not self._children[i]]

    def _keep(self, keep: List[int]) -> None:
        """Rebuild the arrays keeping nodes `keep` (old indices) in that order."""
        remap = {old: new for new, old in enumerate(keep)}
        self._children = [[remap[c] for c in self._children[old] if c in remap] for old in keep]
        self._parent = [remap.get(self._parent[old], -1) if self._parent[old] >= 0 else -1 for old in keep]
        self._token = [self._token[old] for old in keep]
        self._depth = [self._depth[old] for old in keep]
        self._prob = [self._prob[old] for old in keep]
        self._sampled = [self._sampled[old] for old in keep]
        self.current_size = len(keep)
        self._refresh_leaves()

    def prune_to_depth(self, max_depth: int) -> torch.Tensor:
        """Keep nodes with depth <= max_depth; returns the kept original indices (cpu_tree.py:119-173)."""
        if max_depth < 0:
            raise ValueError("max_depth must be >= 0")
        if self.current_size == 0:
            return torch.empty(0, dtype=torch.long)
        if max_depth > max(self._depth):
            return torch.arange(self.current_size, device="cpu")
        keep = [i for i in range(self.current_size) if self._depth[i] <= max_depth]
        if len(keep) == self.current_size:
            return torch.arange(self.current_size, device="cpu")
        self._keep(keep)
        return torch.tensor(keep, dtype=torch.long)

    def prune_to_top_n(self, n: int) -> torch.Tensor:
        """Keep the n nodes of largest cumulative probability, renumbered by rank (cpu_tree.py:175-215).

        Ties are ordered by ascending original index (the reference leaves tie
        order to torch.topk).
        """
        if n == -1 or self.current_size <= n:
            return torch.arange(self.current_size, device="cpu")
        probs = torch.tensor(self._prob, dtype=self.prob_dtype).to(torch.float64).numpy()
        order = np.lexsort((np.arange(self.current_size), -probs))
        keep = [int(i) for i in order[:n]]
        self._keep(keep)
        return torch.tensor(keep, dtype=torch.long)

    # -- queries -----------------------------------------------------------------
    def get_node(self, node_index: int) -> _NodeView:
        if node_index < 0 or node_index >= self.current_size:
            raise IndexError(f"Node index {node_index} out of bounds for tree size {self.current_size}.")
        return _NodeView(self, node_index)

    def get_children_indices(self, node_index) -> torch.Tensor:
        return torch.tensor(self._children[int(node_index)], dtype=torch.long, device="cpu")

    def get_children_ids(self, node_index) -> torch.Tensor:
        return torch.tensor([self._token[c] for c in self._children[int(node_index)]], dtype=torch.long, device="cpu")

    def find_child_index(self, node_index: int, match_token_id: int) -> int:
        for c in self._children[int(node_index)]:
            if self._token[c] == match_token_id:
                return c
        return -1

    def get_tree_data(self, skip_nodes: int = 0) -> Dict[str, torch.Tensor]:
        s = int(skip_nodes)
        return {
            "token_ids": torch.tensor(self._token[s:], dtype=torch.long, device="cpu"),
            "cumulative_probabilities": torch.tensor(self._prob[s:], dtype=self.prob_dtype, device="cpu"),
            "depths": torch.tensor(self._depth[s:], dtype=torch.long, device="cpu"),
            "parent_indices": torch.tensor(self._parent[s:], dtype=torch.long, device="cpu"),
        }

    def get_depth(self) -> torch.Tensor:
        return torch.tensor(max(self._depth, default=0), dtype=torch.long, device="cpu")

    def size(self) -> int:
        return self.current_size

    def ancestor_matrix(self) -> np.ndarray:
        """[n, n] bool, M[i, j] = j is i or an ancestor of i."""
        n = self.current_size
        m = np.zeros((n, n), dtype=bool)
        par = self._parent
        if all(par[i] < i for i in range(n)):
            for i in range(n):  # a node's row is its parent's row plus itself
                if par[i] >= 0:
                    m[i] = m[par[i]]
                m[i, i] = True
        else:
            for i in range(n):
                j, guard = i, 0
                while j >= 0 and guard <= n:
                    m[i, j] = True
                    j = par[j]
                    guard += 1
        return m

    def create_attention_mask(self, prefix_length: int = 0, skip_nodes: int = 0, device: str = "cpu") -> torch.Tensor:
        """Tree-attention mask [1, 1, n - skip_nodes, prefix_length + n], True = may attend (cpu_tree.py:263-286)."""
        n = self.current_size
        if n == 0:
            return torch.empty((1, 1, 0, prefix_length), dtype=self.prob_dtype, device=device)
        m = self.ancestor_matrix()
        if prefix_length > 0:
            m = np.concatenate([np.ones((n, prefix_length), dtype=bool), m], axis=1)
        out = torch.from_numpy(m[int(skip_nodes):, :]).to(device)
        return out.unsqueeze(0).unsqueeze(0)

    # -- flat export for the kernels ------------------------------------------------
    def flat_children(self, skip_nodes: int = 0, limit: Optional[int] = None, restrict: bool = False):
        """Token ids and children CSR in local numbering (node v -> v - skip_nodes).

        `limit` cuts the node range to [skip_nodes, skip_nodes + limit).  With
        `restrict`, children outside that range are dropped (the lossy wrapper,
        tree_verify.py:137-145); without it they are kept (the exact walker looks
        at all children and stops on the first one beyond the decoded rows).
        """
        s = int(skip_nodes)
        end = self.current_size if limit is None else min(self.current_size, s + int(limit))
        n_desc = (end - s) if restrict else (self.current_size - s)
        n_desc = max(n_desc, 0)
        tok = np.asarray(self._token[s:s + n_desc], dtype=np.int64)
        off = np.zeros(n_desc + 1, dtype=np.int32)
        idx: List[int] = []
        for v in range(n_desc):
            for c in self._children[s + v]:
                cl = c - s
                if 0 <= cl < n_desc:
                    idx.append(cl)
            off[v + 1] = len(idx)
        return tok, off, np.asarray(idx, dtype=np.int32)

    def print(self, tokenizer=None, show_token_id: bool = True, show_probability: bool = True):
        if not (show_token_id or show_probability):
            raise ValueError("At least one of 'show_token_id' or 'show_probability' must be True.")

        def label(i: int) -> str:
            parts = []
            if show_token_id:
                parts.append(repr(tokenizer.decode([self._token[i]])) if tokenizer else str(self._token[i]))
            if show_probability:
                parts.append(f"({self._prob[i]:.4f})")
            return " ".join(parts)

        print(label(0))
        stack = [(c, "", k == len(self._children[0]) - 1) for k, c in reversed(list(enumerate(self._children[0])))]
        while stack:
            i, prefix, last = stack.pop()
            print(prefix + ("└── " if last else "├── ") + label(i))
            kids = self._children[i]
            for k, c in reversed(list(enumerate(kids))):
                stack.append((c, prefix + ("    " if last else "│   "), k == len(kids) - 1))

    def __repr__(self) -> str:
        return f"Tree(num_nodes={self.current_size}, device='cpu')"
