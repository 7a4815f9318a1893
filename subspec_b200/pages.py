"""Device-resident page bookkeeping for a batch of requests over one paged KV pool.

The reference's `KvCachePool` / `RequestKvCache` / `getKvCacheBatchPosition`
(specdecodes/models/utils/flashinfer/cache_manager.py:35-414) keep the free-page mask on the CPU and the page
lists in Python, so every step of a generation loop passes through the host.  `DevicePagePool` keeps the same
state in device arrays and brings it up to date with one kernel launch per step (`subspec_pages_update`,
include/subspec_b200.h): lengths set after a reorder, pages released, pages allocated for the next tree, and the
flattened page-table tensors of the attention plan rebuilt -- nothing is read back.  The host classes in
`subspec_b200.kv_cache` remain the drop-in mirror of the reference's interface; this is the batched form.
"""
from __future__ import annotations

import ctypes as C
from typing import Optional

import torch

from . import _lib
from .kv_cache import KvCacheBatchPosition

_MODES = {"prefill": _lib.PAGES_PREFILL, "decode": _lib.PAGES_DECODE, "tree": _lib.PAGES_TREE}


class DevicePagePool:
    """`batch` requests sharing `num_pages` physical pages of `page_len` tokens; at most `pages_per_seq` each."""

    def __init__(self, batch: int, num_pages: int, page_len: int, pages_per_seq: int, device, max_append: int = 0):
        dev = torch.device(device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self.batch, self.num_pages, self.page_len, self.pages_per_seq = int(batch), int(num_pages), int(page_len), \
            int(pages_per_seq)
        self.device = dev
        i32 = dict(dtype=torch.int32, device=dev)
        words = (self.num_pages + 31) // 32
        self.free_mask = torch.full((words,), -1, **i32)  # every page free (bits past the pool are ignored)
        self.page_table = torch.full((batch, pages_per_seq), -1, **i32)
        self.n_pages = torch.zeros(batch, **i32)
        self.kv_len = torch.zeros(batch, **i32)
        self.kv_last_page_len = torch.zeros(batch, **i32)
        self.seq_indptr = torch.zeros(batch + 1, **i32)
        self.kv_page_indptr = torch.zeros(batch + 1, **i32)
        self.kv_page_indices = torch.zeros(batch * pages_per_seq, **i32)
        self.max_append = int(max_append)
        self.batch_indices = torch.zeros(max(1, self.max_append), **i32)
        self.positions = torch.zeros(max(1, self.max_append), **i32)
        self.status = torch.zeros(1, **i32)

    @torch.no_grad()
    def update(self, *, set_len: Optional[torch.Tensor] = None, add_len: Optional[torch.Tensor] = None,
               add_all: int = 0, mode: str = "tree", tree_tokens: int = 0) -> KvCacheBatchPosition:
        """One step of bookkeeping on the current stream (no synchronisation).

        kv_len <- (set_len if given else kv_len) + add_len + add_all; surplus pages are released, missing ones
        allocated (lowest free pages first, requests in batch order).  Returns the page-table tensors of
        `getKvCacheBatchPosition(mode, treeTokens=tree_tokens)` as views of buffers this object owns:
        `kv_page_indices` is sized for the worst case, its first `kv_page_indptr[-1]` entries are in use."""
        if mode not in _MODES:
            raise ValueError("invalid mode")
        a = _lib.PagesArgs()
        a.struct_size = C.sizeof(_lib.PagesArgs)
        a.batch, a.num_pages, a.page_len, a.pages_per_seq = self.batch, self.num_pages, self.page_len, self.pages_per_seq
        a.free_mask, a.page_table, a.n_pages = self.free_mask.data_ptr(), self.page_table.data_ptr(), self.n_pages.data_ptr()
        a.kv_len, a.kv_last_page_len = self.kv_len.data_ptr(), self.kv_last_page_len.data_ptr()
        keep = []
        for name, t in (("set_len", set_len), ("add_len", add_len)):
            if t is not None:
                t = t.to(self.device, torch.int32).contiguous()
                if t.numel() != self.batch:
                    raise ValueError(f"{name} must hold one value per request")
                keep.append(t)
                setattr(a, name, t.data_ptr())
        a.add_all, a.mode, a.tree_tokens = int(add_all), _MODES[mode], int(tree_tokens)
        a.seq_indptr, a.kv_page_indptr = self.seq_indptr.data_ptr(), self.kv_page_indptr.data_ptr()
        a.kv_page_indices = self.kv_page_indices.data_ptr()
        if self.max_append > 0:
            a.max_append = self.max_append
            a.batch_indices, a.positions = self.batch_indices.data_ptr(), self.positions.data_ptr()
        a.dev_status = self.status.data_ptr()
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().subspec_pages_update(C.byref(a), C.c_void_p(stream)), "subspec_pages_update")
        return KvCacheBatchPosition(seq_indptr=self.seq_indptr, kv_page_indptr=self.kv_page_indptr,
                                    kv_page_indices=self.kv_page_indices, kv_last_page_len=self.kv_last_page_len,
                                    batch_indices=self.batch_indices, positions=self.positions)

    def num_free_pages(self) -> int:
        """Synchronises: free pages of the pool (bits of the mask inside the pool)."""
        m = self.free_mask.cpu().numpy().view("uint32")
        bits = sum(bin(int(w)).count("1") for w in m[:-1]) if len(m) > 1 else 0
        tail = self.num_pages - 32 * (len(m) - 1)
        last = int(m[-1]) & ((1 << tail) - 1 if tail < 32 else 0xFFFFFFFF)
        return bits + bin(last).count("1")

    def check_status(self) -> None:
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise ValueError("page bookkeeping kernel: " + _lib.dev_status_text(word))
