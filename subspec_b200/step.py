"""Batched, device-resident speculative step: verify a batch of draft trees, then compact the accepted KV rows.

This is the data-parallel form of the reference's per-request loop body
(generators/classic_sd.py:225-257: `_verify` followed by
`kv_reorder` / `reorder_cache_with_offset`): the reference asserts batch size 1
and walks on the CPU between the two; here a batch of independent sequences goes
through two kernel launches with no host round trip in between -- the verify
kernel's `out_hidden` / `out_meta` feed the compaction kernel directly.
"""
from __future__ import annotations

from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from . import _lib, kv_cache
from .verify import VerifyWorkspace, _gate_code, _method_code


class SpeculativeStepBatch:
    """`batch` independent sequences, each with a draft tree of up to `max_nodes` nodes and a paged KV region.

    The KV pool is [layers, batch * pages_per_seq, 2, page_len, heads, head_dim];
    `page_table[b]` lists the physical pages of sequence b.
    """

    def __init__(self, batch: int, max_nodes: int, device, *, kv_layers: int = 0, kv_heads: int = 4,
                 head_dim: int = 128, page_len: int = 16, pages_per_seq: int = 0,
                 kv_dtype: torch.dtype = torch.bfloat16, page_table: Optional[torch.Tensor] = None):
        self.batch, self.max_nodes = int(batch), int(max_nodes)
        self.ws = VerifyWorkspace(batch, max_nodes, torch.device(device))
        self.device = self.ws.device
        self.pool: Optional[torch.Tensor] = None
        self.page_table: Optional[torch.Tensor] = None
        self.kv_offset = torch.zeros(batch, dtype=torch.int32, device=self.device)
        self.status = torch.zeros(1, dtype=torch.int32, device=self.device)
        if kv_layers and pages_per_seq:
            self.pool = torch.empty(kv_layers, batch * pages_per_seq, 2, page_len, kv_heads, head_dim,
                                    dtype=kv_dtype, device=self.device)
            if page_table is None:
                page_table = torch.arange(batch * pages_per_seq, dtype=torch.int32).reshape(batch, pages_per_seq)
            self.page_table = page_table.to(self.device, torch.int32).contiguous()

    @property
    def kv_row_bytes(self) -> int:
        """Bytes of one token's K and V rows over all layers."""
        L, _, _, _, H, D = self.pool.shape
        return int(L * 2 * H * D * self.pool.element_size())

    def set_trees(self, flats: Sequence) -> None:
        self.ws.set_trees(flats)

    def set_kv_offsets(self, offsets) -> None:
        self.kv_offset.copy_(torch.as_tensor(offsets, dtype=torch.int32))

    def verify(self, logits: torch.Tensor, *, verify_method: str = "exact", verify_kwargs: Optional[dict] = None,
               eos_token_id: Optional[int] = None) -> None:
        """Launch the fused verify kernel on the current stream (no synchronisation)."""
        method = _method_code(verify_method)
        vk = dict(verify_kwargs or {})
        gate, threshold, window = _lib.GATE_PROB, 0.0, 1
        if method != _lib.VERIFY_EXACT:
            gate = _gate_code(vk.get("threshold_method", "prob") or "prob")
            threshold = float(vk.get("threshold", 0.0))
            window = max(0, int(vk.get("window_size", 1)))
        self.ws.run(logits, input_kind=_lib.IN_LOGITS, method=method, gate=gate, threshold=threshold, window=window,
                    eos=eos_token_id)

    def verify_from_hidden(self, hidden: torch.Tensor, lm_head_weight: torch.Tensor, *, verify_method: str = "exact",
                           verify_kwargs: Optional[dict] = None, eos_token_id: Optional[int] = None) -> None:
        """`verify(lm_head(hidden))` without the logits: `hidden` [batch, rows, dim] and `lm_head_weight`
        [vocab, dim], bf16; greedy targets (generators/classic_sd.py:100-116 for a batch).  No synchronisation."""
        method = _method_code(verify_method)
        vk = dict(verify_kwargs or {})
        gate, threshold, window = _lib.GATE_PROB, 0.0, 1
        if method != _lib.VERIFY_EXACT:
            gate = _gate_code(vk.get("threshold_method", "prob") or "prob")
            threshold = float(vk.get("threshold", 0.0))
            window = max(0, int(vk.get("window_size", 1)))
        self.ws.run_lm_head(hidden, lm_head_weight, method=method, gate=gate, threshold=threshold, window=window,
                            eos=eos_token_id)

    def compact_kv(self) -> None:
        """Move the accepted path's KV rows into place, reading the verify kernel's outputs on the device."""
        if self.pool is None:
            raise ValueError("this batch was created without a KV pool")
        meta = self.ws.dev_view("out_meta")
        beam = self.ws.dev_view("out_hidden").view(self.batch, self.ws.max_out)
        kv_cache.compact_paged(self.pool, page_table=self.page_table, offset=self.kv_offset, n=meta, beam=beam,
                               status=self.status, n_stride=4)

    def results(self) -> Dict[str, np.ndarray]:
        """Synchronise and fetch every verify output (tokens, hidden indices, lengths, per-node arrays)."""
        out = self.ws.fetch()
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise ValueError("KV compaction rejected its input: " + _lib.dev_status_text(word))
        return out


class SpeculativeLoopBatch(SpeculativeStepBatch):
    """The loop body of the reference's generators for a batch of requests, with nothing read back between steps.

    Per step (generators/subspec_sd_v2.py:170-262, classic_sd.py:225-257, with the paged cache of
    subspec_sd_fi.py): verify the trees, look the bonus token up among the last context's children (re-rooting),
    gather the hidden indices, reorder the KV rows of the requests whose bonus token missed the tree (with all
    the indices gathered since their last reorder), cut their page lists back to the rows kept and grow every
    request by the next tree -- five launches on the current stream.  The reference runs one request, on the
    host, with a device synchronisation at each of those points (`assert batch_size == 1`, classic_sd.py:169).
    """

    def __init__(self, batch: int, max_nodes: int, device, *, kv_layers: int, kv_heads: int = 4, head_dim: int = 128,
                 page_len: int = 16, pages_per_seq: int, num_pages: Optional[int] = None,
                 kv_dtype: torch.dtype = torch.bfloat16, init_len=1):
        from .pages import DevicePagePool
        from .postverify import PostVerifyState

        super().__init__(batch, max_nodes, device)
        num_pages = int(num_pages or batch * pages_per_seq)
        self.pool = torch.empty(kv_layers, num_pages, 2, page_len, kv_heads, head_dim, dtype=kv_dtype,
                                device=self.device)
        self.pages = DevicePagePool(batch, num_pages, page_len, pages_per_seq, self.device,
                                    max_append=batch * max_nodes)
        self.page_table = self.pages.page_table  # the compaction kernel reads the live table
        init = torch.as_tensor(init_len, dtype=torch.int32).expand(batch).contiguous()
        self.pages.update(set_len=init, mode="prefill")
        self.state = PostVerifyState(batch, 4 * (max_nodes + 1), self.device, kv_len=init)
        self.tree_tokens = 0

    def begin_step(self, tree_tokens: int):
        """Room for the next tree in every request's cache (RequestKvCache.increment); returns the page-table
        tensors of the tree-decoding forward (getKvCacheBatchPosition(mode='tree'))."""
        self.tree_tokens = int(tree_tokens)
        return self.pages.update(add_all=self.tree_tokens, mode="tree", tree_tokens=self.tree_tokens)

    def end_step(self, logits: Optional[torch.Tensor] = None, *, verify_method: str = "exact",
                 verify_kwargs: Optional[dict] = None, eos_token_id: Optional[int] = None,
                 hidden_states: Optional[torch.Tensor] = None, lm_head_weight: Optional[torch.Tensor] = None) -> None:
        """verify -> re-root / gather -> delayed KV reorder -> page lists cut back.  No synchronisation.
        With `hidden_states` and `lm_head_weight` instead of `logits` the lm_head product is part of the
        verification call and the logits are never written (`verify_from_hidden`)."""
        from .postverify import post_verify

        st = self.state
        # rows of earlier trees that are still waiting for their reorder sit in front of this tree's rows: the
        # indices that leave this step count from the first of them
        st.skip_nodes.copy_(self.pages.kv_len - self.tree_tokens - st.kv_len)
        if hidden_states is not None:
            if logits is not None or lm_head_weight is None:
                raise ValueError("give either logits, or hidden_states together with lm_head_weight")
            self.verify_from_hidden(hidden_states, lm_head_weight, verify_method=verify_method,
                                    verify_kwargs=verify_kwargs, eos_token_id=eos_token_id)
        else:
            self.verify(logits, verify_method=verify_method, verify_kwargs=verify_kwargs, eos_token_id=eos_token_id)
        post_verify(self.ws, self.state)
        kv_cache.compact_paged(self.pool, page_table=self.page_table, offset=st.reorder_offset, n=st.reorder_n,
                               beam=st.beam_cache, status=self.status)
        # rows kept so far plus, for a request whose reorder is put off, the whole tree it still reads from
        keep = st.kv_len + torch.where(st.reorder_n > 0, 0, self.pages.kv_len - st.kv_len).to(torch.int32)
        self.pages.update(set_len=keep, mode="decode")

    def check(self) -> None:
        """Synchronise and raise if any kernel of the loop reported a problem."""
        self.results()
        self.state.check_status()
        self.pages.check_status()
