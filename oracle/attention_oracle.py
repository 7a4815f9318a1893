"""CPU oracle for tree attention over the paged cache.  TEST INFRASTRUCTURE ONLY.

fp32 / fp64 torch restatement of what the reference obtains from FlashInfer
(BatchPrefillWithPagedKVCacheWrapper with a custom mask after append_paged_kv_cache;
specdecodes/models/utils/flashinfer/attention_wrapper.py:104-151, 234-253, 288-316): per request, the tree
tokens' queries over the request's cache rows, gathered through the page table, under a boolean mask, softmax
in full precision, grouped-query head mapping h -> h // (q_heads // kv_heads).  FlashInfer is a third-party
package (flashinfer-python, requirements.txt of the reference) whose kernels need a GPU, so they cannot be run
where the fixtures are made.  What pins this restatement instead is the attention of the reference's default
(Hugging Face) path over the same trees: torch's scaled_dot_product_attention behind transformers' repeat_kv,
with the additive mask the reference builds (Tree.create_attention_mask + invert_mask,
specdecodes/models/utils/cpu_tree.py:263, specdecodes/models/utils/utils.py:4-6) -- tests/golden/attention_*,
made by tests/golden/make_golden.py --only attention, agree with this function to fp32 accuracy.  The paged
gather (`gather_rows`) follows KvCachePool's layout, which the KV goldens pin.  Only tests/ may import this.
"""
from __future__ import annotations

import math
from typing import Sequence

import torch


def gather_rows(pool: torch.Tensor, layer: int, pages: Sequence[int], n: int):
    """(K, V) [n, kv_heads, head_dim] of a request whose rows live in `pages` in order."""
    page_len = pool.shape[3]
    k = torch.cat([pool[layer, p, 0] for p in pages])[:n]
    v = torch.cat([pool[layer, p, 1] for p in pages])[:n]
    assert k.shape[0] == n and page_len > 0
    return k, v


def tree_attention(q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, mask: torch.Tensor, sm_scale=None,
                   dtype=torch.float64) -> torch.Tensor:
    """q [nq, HQ, D], k / v [n, HKV, D], mask bool [nq, n] -> [nq, HQ, D] in `dtype`."""
    nq, HQ, D = q.shape
    G = HQ // k.shape[1]
    scale = 1.0 / math.sqrt(D) if sm_scale is None else sm_scale
    qd, kd, vd = q.to(dtype), k.to(dtype), v.to(dtype)
    out = torch.empty(nq, HQ, D, dtype=dtype)
    for h in range(HQ):
        s = (qd[:, h] @ kd[:, h // G].T) * scale
        s = s.masked_fill(~mask, float("-inf"))
        out[:, h] = torch.softmax(s, dim=-1) @ vd[:, h // G]
    return out
