"""Between two verifications of the SubSpec-v2 loop, for a batch of sequences, without leaving the device.

Reference (specdecodes/models/generators/subspec_sd_v2.py): after `_verify` the loop looks the bonus token up
among the children of the last accepted node (`tree.find_child_index`, :231-236); while it keeps finding it,
the KV reorder is put off and the hidden indices pile up in `hidden_indices_cache` (:223-229); when it misses,
or the request has finished, `reorder_cache_with_offset` runs once with everything gathered and `seq_len`
grows by that many rows (:250-262).  `_post_verify` prunes the tree to the depth reached
(`tree.prune_to_depth`, :44-45).  Each of these is a `.item()` / `.tolist()` round trip there; here they are
two small kernels that read the verify kernel's outputs in place (`subspec_post_verify`,
`subspec_tree_prune_depth`, include/subspec_b200.h).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional

import torch

from . import _lib
from .verify import VerifyWorkspace


class PostVerifyState:
    """Per-sequence loop state on the device: rows gathered since the last reorder, KV length, next root."""

    def __init__(self, batch: int, beam_stride: int, device, kv_len=0):
        dev = torch.device(device)
        if dev.type == "cuda" and dev.index is None:
            dev = torch.device("cuda", torch.cuda.current_device())
        self.batch, self.beam_stride, self.device = int(batch), int(beam_stride), dev
        z = dict(dtype=torch.int32, device=dev)
        self.next_root = torch.full((batch,), -1, **z)
        self.accepted = torch.zeros(batch, **z)
        self.beam_cache = torch.zeros(batch, beam_stride, dtype=torch.int64, device=dev)
        self.beam_len = torch.zeros(batch, **z)
        self.reorder_n = torch.zeros(batch, **z)
        self.reorder_offset = torch.zeros(batch, **z)
        self.kv_len = torch.zeros(batch, **z)
        self.kv_len += torch.as_tensor(kv_len, dtype=torch.int32, device=dev)
        self.skip_nodes = torch.zeros(batch, **z)
        self.finished = torch.zeros(batch, dtype=torch.uint8, device=dev)
        self.status = torch.zeros(1, **z)

    def check_status(self) -> None:
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise ValueError("post-verify kernel rejected its input: " + _lib.dev_status_text(word))


@torch.no_grad()
def post_verify(ws: VerifyWorkspace, state: PostVerifyState) -> None:
    """Launch on the current stream, right behind `ws.run(...)`: no synchronisation, nothing comes to the host.

    Afterwards `state.next_root` is the root of the next verification (-1: speculate afresh), and
    `state.reorder_n` / `state.reorder_offset` / `state.beam_cache` are what `kv_cache.compact_paged` /
    `compact_hf` take as n / offset / beam."""
    if ws.batch != state.batch or ws.device != state.device:
        raise ValueError("workspace and state describe different batches")
    a = _lib.PostVerifyArgs()
    a.struct_size = C.sizeof(_lib.PostVerifyArgs)
    a.batch, a.max_nodes, a.max_out = ws.batch, ws.max_nodes, ws.max_out
    for name in ("n_nodes", "token_ids", "child_off", "child_idx"):
        setattr(a, name, ws._in_ptr(name))
    for name in ("out_tokens", "out_hidden", "out_meta"):
        setattr(a, name, ws._out_ptr(name))
    a.skip_nodes, a.finished = state.skip_nodes.data_ptr(), state.finished.data_ptr()
    a.next_root, a.accepted = state.next_root.data_ptr(), state.accepted.data_ptr()
    a.beam_cache, a.beam_stride, a.beam_len = state.beam_cache.data_ptr(), state.beam_stride, state.beam_len.data_ptr()
    a.reorder_n, a.reorder_offset = state.reorder_n.data_ptr(), state.reorder_offset.data_ptr()
    a.kv_len, a.dev_status = state.kv_len.data_ptr(), state.status.data_ptr()
    stream = torch.cuda.current_stream(state.device).cuda_stream
    _lib.check(_lib.lib().subspec_post_verify(C.byref(a), C.c_void_p(stream)), "subspec_post_verify")


@torch.no_grad()
def prune_to_depth_batched(trees: Dict[str, torch.Tensor], max_depth, status: Optional[torch.Tensor] = None
                           ) -> Dict[str, torch.Tensor]:
    """Tree.prune_to_depth (cpu_tree.py:119-173) for a batch of device-resident trees, in place.

    `trees` holds int32 [batch, stride] tensors "token_ids", "parent_indices", "depths", the int32 [batch]
    tensor "n_nodes", optionally float32 "cumulative_probabilities" and the children lists "child_off"
    [batch, stride + 1] / "child_idx" [batch, stride] -- the layout `DraftTreeBatch.finalize` returns.
    `max_depth` is an int or one value per sequence.  Returns {"keep_idx": old index of every kept node,
    "n_nodes": nodes kept}; the arrays of `trees` (and its "n_nodes") are updated.
    """
    tok, par, dep, n = (trees[k] for k in ("token_ids", "parent_indices", "depths", "n_nodes"))
    B, S = tok.shape
    dev = tok.device
    for t in (tok, par, dep):
        if t.dtype != torch.int32 or tuple(t.shape) != (B, S) or not t.is_contiguous() or t.device != dev:
            raise ValueError("token_ids / parent_indices / depths must be contiguous int32 [batch, stride] tensors")
    md = torch.as_tensor(max_depth, dtype=torch.int32)
    if bool((md < 0).any()):
        raise ValueError("max_depth must be >= 0")
    md = md.to(dev).expand(B).contiguous() if md.dim() == 0 else md.to(dev).contiguous()
    keep_idx = torch.full((B, S), -1, dtype=torch.int32, device=dev)
    n_out = torch.empty(B, dtype=torch.int32, device=dev)
    a = _lib.TreePruneDepthArgs()
    a.struct_size = C.sizeof(_lib.TreePruneDepthArgs)
    a.batch, a.tree_stride = B, S
    a.n_nodes, a.max_depth = n.data_ptr(), md.data_ptr()
    a.tokens, a.parents, a.depths = tok.data_ptr(), par.data_ptr(), dep.data_ptr()
    probs = trees.get("cumulative_probabilities")
    a.probs = 0 if probs is None else probs.data_ptr()
    a.keep_idx, a.n_out = keep_idx.data_ptr(), n_out.data_ptr()
    if "child_off" in trees:
        off, idx = trees["child_off"], trees["child_idx"]
        if tuple(off.shape) != (B, S + 1) or tuple(idx.shape) != (B, S):
            raise ValueError("child_off must be [batch, stride + 1] and child_idx [batch, stride]")
        a.child_off, a.child_idx = off.data_ptr(), idx.data_ptr()
    a.dev_status = 0 if status is None else status.data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().subspec_tree_prune_depth(C.byref(a), C.c_void_p(stream)), "subspec_tree_prune_depth")
    n.copy_(n_out)
    return {"keep_idx": keep_idx, "n_nodes": n_out}
