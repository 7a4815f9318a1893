"""Host-side rejection of malformed trees: nothing here touches a GPU (the checks run before any launch)."""
import numpy as np
import pytest

from subspec_b200.verify import _children_csr, check_forest


def _csr(children):
    return _children_csr(children)


def test_forests_pass():
    for children in ([[]], [[1, 2], [3], [], []], [[2], [], [1]],  # a child may precede its parent in numbering
                     [[], [0]], [[1], [2], [3], [4], []]):
        off, idx = _csr(children)
        check_forest(off, idx, len(children))
    # a 1024-node chain in reverse numbering: the pointer-jumping path at its longest
    n = 1024
    children = [[] if i == 0 else [i - 1] for i in range(n)]
    off, idx = _csr(children)
    check_forest(off, idx, n)


@pytest.mark.parametrize("children,what", [
    ([[0]], "loop"),                      # a node that is its own child
    ([[1], [0]], "loop"),                 # two nodes that are each other's child
    ([[1], [2], [1]], "more than once"),  # node 1 reached twice
    ([[1, 1], []], "more than once"),
    ([[5], []], "outside"),
    ([[-1], []], "outside"),
    ([[2], [3], [1], [2]], "more than once"),
    ([[], [2], [3], [1]], "loop"),        # a loop that the root does not reach
])
def test_non_forests_are_rejected(children, what):
    off, idx = _csr(children)
    with pytest.raises(ValueError, match=what):
        check_forest(off, idx, len(children))


def test_bad_offsets_are_rejected():
    with pytest.raises(ValueError, match="offsets"):
        check_forest(np.array([0, 2, 1]), np.array([1, 1]), 2)
    with pytest.raises(ValueError, match="offsets"):
        check_forest(np.array([1, 1, 1]), np.array([], dtype=np.int32), 2)
    with pytest.raises(ValueError, match="offsets"):
        check_forest(np.array([0, 0]), np.array([], dtype=np.int32), 2)
    with pytest.raises(ValueError, match="child entries"):
        check_forest(np.array([0, 3, 3]), np.array([1, 1, 1]), 2)


def test_attention_wrapper_rejects_bad_arguments():
    """The checks of `tree_attention_paged` / `append_paged_kv` that run before any launch, on CPU tensors."""
    import torch

    from subspec_b200.attention import append_paged_kv, tree_attention_paged

    L, P, page, H, D, B, QL, HQ = 1, 4, 16, 2, 128, 1, 8, 4
    pool = torch.zeros(L, P, 2, page, H, D, dtype=torch.bfloat16)
    q = torch.zeros(B, QL, HQ, D, dtype=torch.bfloat16)
    table = torch.zeros(B, 4, dtype=torch.int32)
    kv_len = torch.full((B,), 20, dtype=torch.int32)
    mask = torch.ones(B, QL, 32, dtype=torch.bool)
    kw = dict(page_table=table, kv_len=kv_len, mask=mask)
    with pytest.raises(ValueError, match="same type"):  # fp16 queries on a bf16 pool
        tree_attention_paged(q.half(), pool, 0, **kw)
    with pytest.raises(ValueError, match="same type"):
        tree_attention_paged(q.float(), pool.float(), 0, **kw)
    with pytest.raises(ValueError, match="head_dim"):
        tree_attention_paged(q[..., :64].contiguous(), pool, 0, **kw)
    with pytest.raises(ValueError, match="mask"):
        tree_attention_paged(q, pool, 0, page_table=table, kv_len=kv_len, mask=mask.long())
    with pytest.raises(ValueError, match="mask"):
        tree_attention_paged(q, pool, 0, page_table=table, kv_len=kv_len, mask=mask[:, :4])
    with pytest.raises(ValueError, match="page_table"):
        tree_attention_paged(q, pool, 0, page_table=table.long(), kv_len=kv_len, mask=mask)
    with pytest.raises(ValueError, match="out must"):
        tree_attention_paged(q, pool, 0, out=torch.zeros(B, QL, HQ, D, dtype=torch.float16), **kw)
    k = torch.zeros(B, QL, H, D, dtype=torch.bfloat16)
    with pytest.raises(ValueError):
        append_paged_kv(pool, 0, k, k.half(), page_table=table, kv_len=kv_len)
    from subspec_b200.attention import tree_attention_static
    qh = torch.zeros(B, HQ, QL, D, dtype=torch.bfloat16)
    kc = torch.zeros(B, H, 64, D, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="same type"):
        tree_attention_static(qh, kc, kc.half(), kv_len=kv_len, mask=mask)
    with pytest.raises(ValueError, match="one shape"):
        tree_attention_static(qh, kc, kc[:, :, :32], kv_len=kv_len, mask=mask)
    with pytest.raises(ValueError, match="mask"):
        tree_attention_static(qh, kc, kc, kv_len=kv_len, mask=mask.long())


def test_fused_lm_head_arguments_are_checked_before_any_launch():
    """`verify_tree_batched(hidden_states=, lm_head_weight=)`: the argument combinations it refuses are refused
    on the host, before a device is touched."""
    import torch

    from subspec_b200.tree import Tree
    from subspec_b200.verify import verify_tree_batched

    tree = Tree.from_arrays([1, 2, 3], [-1, 0, 0])
    hidden = torch.zeros(1, 3, 64, dtype=torch.bfloat16)
    weight = torch.zeros(100, 64, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="either logits"):
        verify_tree_batched(trees=[tree], root_inds=[0], logits=torch.zeros(1, 3, 100), hidden_states=hidden,
                            lm_head_weight=weight, eos_token_id=None)
    with pytest.raises(ValueError, match="either logits"):
        verify_tree_batched(trees=[tree], root_inds=[0], hidden_states=hidden, eos_token_id=None)
    with pytest.raises(ValueError, match="greedy targets only"):
        verify_tree_batched(trees=[tree], root_inds=[0], hidden_states=hidden, lm_head_weight=weight,
                            eos_token_id=None, do_sample=True)
    with pytest.raises(ValueError, match="hidden_states must be"):
        verify_tree_batched(trees=[tree], root_inds=[0], hidden_states=hidden[0], lm_head_weight=weight,
                            eos_token_id=None)
    with pytest.raises(ValueError, match="logits must be"):
        verify_tree_batched(trees=[tree], root_inds=[0], eos_token_id=None)
