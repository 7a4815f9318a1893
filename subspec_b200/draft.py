"""Draft-tree expansion behind the reference's draft-model helpers.

Reference surface mirrored here (specdecodes/models/...):
  draft_models/base.py:267-305   DraftModelBase.topk_sampling / _topk_flatten  -> topk_sampling
  draft_models/classic_sd.py:10-16  softmax(logits / T) in the draft forward    -> topk_sampling_from_logits (fused)
  draft_models/base.py:31-47     TreeData
  draft_models/base.py:49-117    TreeMaskCache
  utils/utils.py:4-17            invert_mask, DraftParams
  utils/cpu_tree.py:175-286      prune_to_top_n / get_tree_data / create_attention_mask -> DraftTreeBatch.finalize

`topk_sampling` keeps the reference's signature (probabilities in).  The fused
form takes the draft LOGITS and never materialises the [leaves, vocab]
probabilities or the scores buffer.  `DraftTreeBatch` keeps the growing trees of
a batch of sequences on the device: `expand` appends one level per call,
`finalize` prunes to the best n nodes and emits parents, tree-attention mask,
position ids and the children lists the verifier consumes -- no host round trip.
"""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass
from typing import Dict, Optional, Tuple

import torch

from . import _lib


def invert_mask(mask: torch.Tensor, dtype: torch.dtype) -> torch.Tensor:
    """bool mask (True = attend) -> additive mask (0 / finfo.min), utils/utils.py:4-6."""
    return (~mask).to(dtype) * torch.finfo(dtype).min


@dataclass
class DraftParams:
    """utils/utils.py:8-17."""

    temperature: float = 1
    max_depth: int = 6
    topk_len: int = 10
    max_verify_tokens: Optional[int] = None

    def __post_init__(self):
        self.max_sample_tokens = self.max_depth * self.topk_len + 1
        self.max_verify_tokens = (min(self.max_sample_tokens, self.max_verify_tokens)
                                  if self.max_verify_tokens is not None else self.max_sample_tokens)


class TreeData:
    """Per-step accumulator of (token_ids, child_probs, parent_indices), each [1, k]; get_data -> 3 x [1, depth, k]."""

    def __init__(self):
        self.token_ids_data, self.child_probs_data, self.parent_indices_data = [], [], []

    def update(self, token_ids: torch.Tensor, child_probs: torch.Tensor, parent_indices: torch.Tensor) -> None:
        self.token_ids_data.append(token_ids)
        self.child_probs_data.append(child_probs)
        self.parent_indices_data.append(parent_indices)

    def get_data(self):
        return tuple(torch.cat(d, dim=0).unsqueeze(0)
                     for d in (self.token_ids_data, self.child_probs_data, self.parent_indices_data))


class TreeMaskCache:
    """Draft-side incremental tree mask (draft_models/base.py:49-117).

    Row i of a new level is the row of its parent in the previous level followed
    by a one-hot for itself.  'static' writes into a preallocated
    [1, 1, sample_len, max_cache_len] bool buffer, 'dynamic' concatenates.
    """

    def __init__(self, prefix_len: int, sample_len: int, max_cache_len: Optional[int], dtype, device):
        self.prefix_len, self.sample_len, self.max_cache_len = prefix_len, sample_len, max_cache_len
        self.dtype, self.device = dtype, device
        static = max_cache_len is not None and int(max_cache_len) >= int(prefix_len) + int(sample_len)
        if static:
            self.tree_mask_update_method = "static"
            self.tree_mask_cache = torch.zeros((1, 1, sample_len, max_cache_len), device=device, dtype=torch.bool)
            self.tree_mask_cache[:, :, 0, :prefix_len] = True
            self.current_len = prefix_len
        else:
            self.tree_mask_update_method = "dynamic"
            self.tree_mask_cache = torch.ones((1, 1, 1, prefix_len), device=device, dtype=torch.bool)
        self.eye_block = torch.eye(sample_len, device=device, dtype=torch.bool)[None, None]

    def update_tree_mask(self, parent_indices: torch.Tensor, return_invert: bool = True) -> torch.Tensor:
        if self.tree_mask_update_method == "static":
            cur = self.current_len
            self.tree_mask_cache[..., :cur] = self.tree_mask_cache[..., parent_indices[0], :cur]
            self.tree_mask_cache[..., cur:cur + self.sample_len] = self.eye_block
            self.current_len += self.sample_len
        else:
            self.tree_mask_cache = torch.cat((self.tree_mask_cache[:, :, parent_indices[0]], self.eye_block), dim=3)
        return self.get_tree_mask(return_invert)

    def get_tree_mask(self, return_invert: bool = True) -> torch.Tensor:
        return invert_mask(self.tree_mask_cache, self.dtype) if return_invert else self.tree_mask_cache


# ---------------------------------------------------------------------------------
# one expansion step
# ---------------------------------------------------------------------------------
_scratch: Dict[Tuple[int, int], torch.Tensor] = {}


def _scratch_for(device: torch.device, batch: int, leaves: int, k: int) -> Tuple[int, int]:
    """One buffer per (device, batch), zeroed when it is made: the ticket words at its start depend on `batch`
    alone and every launch leaves them zero, so the calls can vouch for it (SUBSPEC_EXPAND_SCRATCH_CLEAN) and
    the library puts no clearing operation in front of the kernel.  Like the verify workspaces, a buffer serves
    one stream at a time."""
    need = C.c_size_t(0)
    _lib.check(_lib.lib().subspec_expand_scratch_bytes(batch, leaves, k, C.byref(need)), "subspec_expand_scratch_bytes")
    key = (device.index if device.index is not None else torch.cuda.current_device(), int(batch))
    buf = _scratch.get(key)
    if buf is None or buf.numel() < need.value + 256:
        buf = _scratch[key] = torch.zeros(need.value + 256, dtype=torch.uint8, device=device)
    ptr = (buf.data_ptr() + 255) // 256 * 256
    return ptr, need.value


def _expand(scores: torch.Tensor, parent_probs: Optional[torch.Tensor], k: int, input_kind: int, temperature: float,
            tree: Optional["DraftTreeBatch"] = None, level: int = 0):
    if scores.dim() != 3:
        raise ValueError("scores must be [batch, leaves, vocab]")
    if not scores.is_cuda:
        if not torch.cuda.is_available():
            raise _lib.SubspecError("subspec_b200 needs a CUDA device (sm_100a); there is no CPU path")
        scores = scores.cuda()
    if scores.stride(2) != 1:
        scores = scores.contiguous()
    B, L, V = scores.shape
    k = min(int(k), int(V))
    dev = scores.device
    if parent_probs is not None:
        parent_probs = parent_probs.to(dev, scores.dtype).contiguous()
        if tuple(parent_probs.shape) != (B, L):
            raise ValueError(f"parent_probs must be [{B}, {L}]")
    out_tokens = torch.empty(B, k, dtype=torch.int64, device=dev)
    out_parents = torch.empty(B, k, dtype=torch.int64, device=dev)
    out_probs = torch.empty(B, k, dtype=scores.dtype, device=dev)
    a = _lib.ExpandArgs()
    a.struct_size = C.sizeof(_lib.ExpandArgs)
    a.batch, a.leaves, a.vocab, a.k = B, L, V, k
    a.dtype, a.input_kind = _lib.torch_dtype_code(scores.dtype), input_kind
    a.seq_stride, a.row_stride = int(scores.stride(0)), int(scores.stride(1))
    a.scores = scores.data_ptr()
    a.parent_probs = 0 if parent_probs is None else parent_probs.data_ptr()
    a.temperature = float(temperature)
    a.out_tokens, a.out_probs, a.out_parents = out_tokens.data_ptr(), out_probs.data_ptr(), out_parents.data_ptr()
    if tree is not None:
        a.level, a.tree_stride = int(level), tree.stride
        a.tree_tokens, a.tree_parents = tree.tokens.data_ptr(), tree.parents.data_ptr()
        a.tree_probs, a.tree_depths = tree.probs.data_ptr(), tree.depths.data_ptr()
        a.dev_status = tree.status.data_ptr()
        if tree.draft_mask is not None:
            m = tree.draft_mask
            a.draft_mask, a.draft_mask_kind = m.data_ptr(), tree._mask_kind
            a.draft_mask_cols = int(m.shape[3])
            a.draft_mask_row_stride, a.draft_mask_seq_stride = int(m.stride(2)), int(m.stride(0))
            a.prefix_len = tree.prefix_len.data_ptr()
            a.draft_position_ids = tree.draft_position_ids.data_ptr()
    a.scratch, a.scratch_bytes = _scratch_for(dev, B, L, k)
    a.flags = _lib.EXPAND_SCRATCH_CLEAN
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().subspec_expand_step(C.byref(a), C.c_void_p(stream)), "subspec_expand_step")
    return out_tokens, out_probs, out_parents


@torch.no_grad()
def topk_sampling(sampled_probs: torch.Tensor, parent_probs: torch.Tensor, sample_k: int):
    """Drop-in for DraftModelBase.topk_sampling: (token_ids [B,k] int64, topk_probs [B,k], parent_indices [B,k] int64).

    Ties are ordered by ascending flat index leaf * vocab + token (torch.topk leaves them unspecified).
    """
    return _expand(sampled_probs, parent_probs, sample_k, _lib.IN_PROBS, 1.0)


@torch.no_grad()
def topk_sampling_from_logits(logits: torch.Tensor, parent_probs: Optional[torch.Tensor], sample_k: int,
                              temperature: float = 1.0):
    """softmax(logits / temperature) -> topk_sampling in one pass over the logits."""
    return _expand(logits, parent_probs, sample_k, _lib.IN_LOGITS, temperature)


_MASK_KIND = {torch.bool: _lib.MASK_BOOL, torch.uint8: _lib.MASK_BOOL, torch.float32: _lib.MASK_ADD_F32,
              torch.bfloat16: _lib.MASK_ADD_BF16, torch.float16: _lib.MASK_ADD_F16}


def _mask_kind(dtype: torch.dtype) -> int:
    try:
        return _MASK_KIND[dtype]
    except KeyError:
        raise ValueError(f"mask dtype {dtype}: expected bool (raw mask) or float32 / bfloat16 / float16 (additive)")


def _per_sequence_i32(x, batch: int, device) -> torch.Tensor:
    if isinstance(x, torch.Tensor):
        t = x.to(device=device, dtype=torch.int32).reshape(-1)
    elif isinstance(x, (list, tuple)):
        t = torch.tensor([int(v) for v in x], dtype=torch.int32, device=device)
    else:
        t = torch.full((batch,), int(x), dtype=torch.int32, device=device)
    if t.numel() == 1 and batch > 1:
        t = t.expand(batch)
    if t.numel() != batch:
        raise ValueError(f"expected one value per sequence ({batch}), got {t.numel()}")
    return t.contiguous()


class DraftTreeBatch:
    """Device-resident draft trees of `batch` sequences grown level by level with `k` nodes per level.

    With `prefix_len` (tokens in front of the first level, the root last among them: the draft's `kv_len`,
    draft_models/classic_sd.py:57-63) every `expand` also writes the level's draft-side tree mask and
    position ids -- what `TreeMaskCache.update_tree_mask` / `get_tree_mask` and the speculate loop's
    `position_ids` hold (draft_models/base.py:93-117, classic_sd.py:71-72, 113) -- into `draft_mask`
    [batch, 1, k, cols] and `draft_position_ids` [batch, k]: raw bool for `mask_dtype=torch.bool`, the
    inverted additive form for a float dtype.  `cols` is `max_cache_len` (the reference's static buffer) or,
    without it, `max(prefix_len) + k * max_depth`.
    """

    def __init__(self, batch: int, k: int, max_depth: int, device, root_tokens: Optional[torch.Tensor] = None, *,
                 prefix_len=None, max_cache_len: Optional[int] = None, mask_dtype: torch.dtype = torch.bool):
        self.batch, self.k, self.max_depth = int(batch), int(k), int(max_depth)
        self.device = torch.device(device)
        if self.device.type == "cuda" and self.device.index is None:  # "cuda" means the current device
            self.device = torch.device("cuda", torch.cuda.current_device())
        self.stride = 1 + self.k * self.max_depth
        z = dict(device=self.device)
        self.tokens = torch.zeros(batch, self.stride, dtype=torch.int32, **z)
        self.parents = torch.full((batch, self.stride), -1, dtype=torch.int32, **z)
        self.probs = torch.zeros(batch, self.stride, dtype=torch.float32, **z)
        self.depths = torch.zeros(batch, self.stride, dtype=torch.int32, **z)
        self.probs[:, 0] = 1.0
        if root_tokens is not None:
            self.tokens[:, 0] = root_tokens.to(self.device, torch.int32)
        self.level = 0
        self.parent_probs: Optional[torch.Tensor] = None
        self.status = torch.zeros(1, dtype=torch.int32, **z)
        self.prefix_len: Optional[torch.Tensor] = None
        self.draft_mask: Optional[torch.Tensor] = None
        self.draft_position_ids: Optional[torch.Tensor] = None
        if prefix_len is not None:
            longest = (max(int(v) for v in prefix_len) if isinstance(prefix_len, (list, tuple)) else
                       int(prefix_len.max()) if isinstance(prefix_len, torch.Tensor) else int(prefix_len))
            self.prefix_len = _per_sequence_i32(prefix_len, self.batch, self.device)
            cols = int(max_cache_len) if max_cache_len is not None else longest + self.k * self.max_depth
            if cols < longest + self.k * self.max_depth:
                raise ValueError("max_cache_len is shorter than prefix_len + k * max_depth")
            self._mask_kind = _mask_kind(mask_dtype)
            self._longest_prefix = longest
            self.draft_mask = torch.zeros(batch, 1, self.k, cols, dtype=mask_dtype, **z)
            self.draft_position_ids = torch.zeros(batch, self.k, dtype=torch.int64, **z)

    @property
    def n_nodes(self) -> int:
        return 1 + self.level * self.k

    def get_tree_mask(self) -> torch.Tensor:
        """The draft-side mask after the last `expand`: [batch, 1, k, cols] (all columns of the buffer)."""
        if self.draft_mask is None:
            raise ValueError("this batch was created without prefix_len: no draft-side mask is kept")
        return self.draft_mask

    def check_status(self) -> None:
        """Synchronise and raise if a kernel of this batch rejected its input."""
        word = int(self.status.item())
        if word:
            self.status.zero_()
            raise ValueError("draft-tree kernel rejected its input: " + _lib.dev_status_text(word))

    @torch.no_grad()
    def expand(self, scores: torch.Tensor, *, from_logits: bool = True, temperature: float = 1.0):
        """One depth step.  `scores` is [batch, leaves, vocab]: leaves = 1 on the first step, k afterwards."""
        if self.level >= self.max_depth:
            raise ValueError("tree is already at max_depth")
        kind = _lib.IN_LOGITS if from_logits else _lib.IN_PROBS
        toks, probs, parents = _expand(scores, self.parent_probs, self.k, kind, temperature, tree=self,
                                       level=self.level)
        self.parent_probs = probs
        self.level += 1
        return toks, probs, parents

    @torch.no_grad()
    def finalize(self, keep: int, position_offset=None, *, prefix_length=None, skip_nodes: int = 0,
                 mask_out: Optional[torch.Tensor] = None, mask_dtype: torch.dtype = torch.bool,
                 mask_cols: Optional[int] = None) -> Dict[str, torch.Tensor]:
        """prune_to_top_n(keep) + renumbering + tree mask + position ids + children lists, all on the device.

        `prefix_length` (int, list or [batch] tensor) puts that many may-attend columns in front of the tree
        columns and `skip_nodes` starts the mask rows at that node (Tree.create_attention_mask,
        cpu_tree.py:263-286).  `mask_out` is a caller's preallocated [batch, 1, rows, max_cache_len] buffer
        (generators/classic_sd.py:21-55): rows [0, keep - skip_nodes) are written whole, in the buffer's dtype
        -- bool, or a float dtype for the inverted additive form (utils/utils.py:4-6).  Without it a dense
        [batch, keep - skip_nodes, mask_cols] tensor of `mask_dtype` is returned (`mask_cols` defaults to
        max(prefix_length) + keep, which reads the maximum back from the device if the prefix is a tensor).
        The per-node outputs always describe nodes 0 .. keep - 1; slice them from `skip_nodes` as the
        reference's get_tree_data(skip_nodes) does.
        """
        B, dev = self.batch, self.device
        keep, skip = int(keep), int(skip_nodes)
        if not 0 <= skip <= keep:
            raise ValueError("skip_nodes must be in [0, keep]")
        prefix = None if prefix_length is None else _per_sequence_i32(prefix_length, B, dev)
        if mask_out is not None:
            if mask_out.dim() == 4 and mask_out.shape[1] == 1:
                mview = mask_out[:, 0]
            elif mask_out.dim() == 3:
                mview = mask_out
            else:
                raise ValueError("mask_out must be [batch, 1, rows, cols] or [batch, rows, cols]")
            if mview.shape[0] != B or mview.shape[1] < keep - skip or mview.stride(2) != 1 or mview.device != dev:
                raise ValueError("mask_out does not hold [batch, keep - skip_nodes, cols] rows on this device")
            cols = int(mview.shape[2])
            tree_mask, kind = mview, _mask_kind(mview.dtype)
        else:
            if mask_cols is None:
                mask_cols = keep + (0 if prefix is None else int(prefix.max()))
            cols = int(mask_cols)
            tree_mask = torch.empty(B, keep - skip, cols, dtype=mask_dtype, device=dev)
            kind = _mask_kind(mask_dtype)
        out = {
            "keep_idx": torch.empty(B, keep, dtype=torch.int32, device=dev),
            "token_ids": torch.empty(B, keep, dtype=torch.int32, device=dev),
            "parent_indices": torch.empty(B, keep, dtype=torch.int32, device=dev),
            "depths": torch.empty(B, keep, dtype=torch.int32, device=dev),
            "cumulative_probabilities": torch.empty(B, keep, dtype=torch.float32, device=dev),
            "position_ids": torch.empty(B, keep, dtype=torch.int64, device=dev),
            "tree_mask": tree_mask,
            "child_off": torch.empty(B, keep + 1, dtype=torch.int32, device=dev),
            "child_idx": torch.zeros(B, keep, dtype=torch.int32, device=dev),
            "n_nodes": torch.empty(B, dtype=torch.int32, device=dev),
        }
        a = _lib.TreeFinalizeArgs()
        a.struct_size = C.sizeof(_lib.TreeFinalizeArgs)
        a.batch, a.n_nodes, a.tree_stride, a.keep = B, self.n_nodes, self.stride, keep
        a.tree_tokens, a.tree_parents = self.tokens.data_ptr(), self.parents.data_ptr()
        a.tree_probs, a.tree_depths = self.probs.data_ptr(), self.depths.data_ptr()
        if position_offset is not None:
            position_offset = _per_sequence_i32(position_offset, B, dev)
            a.position_offset = position_offset.data_ptr()
        a.keep_idx, a.tokens, a.parents = (out[n].data_ptr() for n in ("keep_idx", "token_ids", "parent_indices"))
        a.depths, a.probs = out["depths"].data_ptr(), out["cumulative_probabilities"].data_ptr()
        a.position_ids, a.mask = out["position_ids"].data_ptr(), tree_mask.data_ptr()
        a.child_off, a.child_idx, a.n_out = (out[n].data_ptr() for n in ("child_off", "child_idx", "n_nodes"))
        a.dev_status = self.status.data_ptr()
        a.prefix_length = 0 if prefix is None else prefix.data_ptr()
        a.skip_nodes, a.mask_kind = skip, kind
        a.mask_cols = cols
        a.mask_row_stride, a.mask_seq_stride = int(tree_mask.stride(1)), int(tree_mask.stride(0))
        stream = torch.cuda.current_stream(dev).cuda_stream
        _lib.check(_lib.lib().subspec_tree_finalize(C.byref(a), C.c_void_p(stream)), "subspec_tree_finalize")
        return out
