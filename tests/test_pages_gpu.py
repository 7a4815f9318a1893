"""Device-resident page bookkeeping against page lists the reference's KvCachePool / RequestKvCache produced."""
import pytest
import torch

from subspec_b200.pages import DevicePagePool
from tests import golden_io

pytestmark = pytest.mark.gpu


def _check(pool, snap, B):
    n = pool.n_pages.tolist()
    table = pool.page_table.tolist()
    assert n == [len(p) for p in snap["pages"]]
    assert [table[b][:n[b]] for b in range(B)] == snap["pages"]
    assert pool.kv_len.tolist() == snap["kv_len"] and pool.kv_last_page_len.tolist() == snap["last"]
    assert pool.num_free_pages() == snap["free"]


def _check_plan(pos, snap, B, appended):
    indptr = [0]
    for p in snap["pages"]:
        indptr.append(indptr[-1] + len(p))
    assert pos.kv_page_indptr.tolist() == indptr
    assert pos.kv_page_indices[:indptr[-1]].tolist() == [pg for p in snap["pages"] for pg in p]
    assert pos.seq_indptr.tolist() == [b * appended for b in range(B + 1)]
    want_b, want_p = [], []
    for b in range(B):
        want_b += [b] * appended
        want_p += [snap["kv_len"][b] - appended + j for j in range(appended)]
    assert pos.batch_indices[:B * appended].tolist() == want_b
    assert pos.positions[:B * appended].tolist() == want_p


def test_scripted_loops_match_reference(cuda_lib):
    """Every step of the golden loops: grow every request by the next tree, then cut it back to what the
    verification kept.  Page lists (ids and order), lengths, last-page fills, free count and the flattened
    page-table tensors equal the reference's after every call; nothing is read back between calls."""
    for sc in golden_io.pages_scripts():
        B, tree_n = sc["batch"], sc["tree_n"]
        pool = DevicePagePool(B, sc["num_pages"], sc["page_len"], pages_per_seq=sc["num_pages"], device="cuda",
                              max_append=B * tree_n)
        pool.update(set_len=torch.tensor(sc["init"]), mode="prefill")
        _check(pool, sc["first"], B)
        for step in sc["steps"]:
            pos = pool.update(add_all=tree_n, mode="tree", tree_tokens=tree_n)
            _check(pool, step["grown"], B)
            _check_plan(pos, step["grown"], B, tree_n)
            pool.update(set_len=torch.tensor(step["new_len"]), mode="decode")
            _check(pool, step["cropped"], B)
        pool.check_status()


def test_running_out_of_pages_is_reported(cuda_lib):
    pool = DevicePagePool(2, 5, 4, pages_per_seq=5, device="cuda")
    pool.update(set_len=torch.tensor([8, 8]))      # two pages each
    pool.check_status()
    pool.update(add_all=8)                         # two more each: only one page is left
    with pytest.raises(ValueError):
        pool.check_status()
    small = DevicePagePool(1, 64, 4, pages_per_seq=2, device="cuda")
    small.update(set_len=torch.tensor([9]))        # three pages, the request's list holds two
    with pytest.raises(ValueError):
        small.check_status()
    with pytest.raises(ValueError):
        small.update(mode="sideways")
