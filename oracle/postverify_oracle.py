"""CPU oracle for the steps between two verifications of the SubSpec-v2 loop.  TEST INFRASTRUCTURE ONLY.

Plain-Python restatements; only tests/ may import this module.  Pinned against the reference:
tests/golden/post_cases.json holds what the reference's own Tree.prune_to_depth and Tree.find_child_index
returned on seeded trees (tests/golden/make_golden.py), and tests/test_oracle_golden.py checks `prune_to_depth`
and `find_child_index` against them.  `DelayedReorder` restates a few lines of the generator's loop body that
cannot be called on their own (they sit inside generate()); it is checked against the reference by reading only:
parity unpinned for that class alone.

  find_child_index   Tree.find_child_index       specdecodes/models/utils/cpu_tree.py:232-236
  prune_to_depth     Tree.prune_to_depth         cpu_tree.py:119-173
  DelayedReorder     hidden_indices_cache, is_prev_accepted, kv_reorder
                                                 specdecodes/models/generators/subspec_sd_v2.py:223-262
"""
from __future__ import annotations

from typing import List, Optional, Sequence, Tuple


def find_child_index(token_ids: Sequence[int], children: Sequence[Sequence[int]], node: int, token: int) -> int:
    for c in children[node]:
        if int(token_ids[c]) == int(token):
            return int(c)
    return -1


def prune_to_depth(token_ids, parents, depths, children, max_depth: int):
    """Returns (keep list of old indices, token_ids, parents (-1 = none), depths, children) of the pruned tree."""
    if max_depth < 0:
        raise ValueError("max_depth must be >= 0")
    keep = [i for i, d in enumerate(depths) if d <= max_depth]
    new_of = {o: n for n, o in enumerate(keep)}
    tok = [int(token_ids[o]) for o in keep]
    par = [new_of.get(int(parents[o]), -1) if int(parents[o]) >= 0 else -1 for o in keep]
    dep = [int(depths[o]) for o in keep]
    ch = [[new_of[c] for c in children[o] if c in new_of] for o in keep]
    return keep, tok, par, dep, ch


class DelayedReorder:
    """One sequence's bookkeeping across steps: indices gathered while the bonus token keeps landing in the tree."""

    def __init__(self, kv_len: int):
        self.kv_len = int(kv_len)
        self.cache: List[int] = []

    def step(self, hidden: Sequence[int], next_root: int, finished: bool = False
             ) -> Tuple[Optional[List[int]], int]:
        """Returns (indices to reorder with now or None, the offset they apply at)."""
        self.cache = self.cache + [int(h) for h in hidden]
        accepted = next_root >= 0
        if not accepted or finished:
            beam, at = self.cache, self.kv_len
            self.kv_len += len(beam)
            self.cache = []
            return beam, at
        return None, self.kv_len
