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
