"""Tree attention over the paged KV cache: the FlashInfer calls of the reference's paged generators.

Reference (specdecodes/models/utils/flashinfer/attention_wrapper.py:104-151, 234-253, 288-316 and
attention.py:26-102): per layer, `append_paged_kv_cache` writes the tree tokens' K / V rows into the request's
pages and `BatchPrefillWithPagedKVCacheWrapper.run` evaluates the tree tokens' queries over the request's cache
under a custom mask.  Here both are kernels of the C-ABI library (`subspec_kv_append_paged`,
`subspec_tree_attention_paged`) that take the pool, the page table and the mask as the other kernels of this
package leave them: `KvCachePool.cache_data`, `DevicePagePool.page_table` / `kv_len`, and the
[rows, prefix + tree columns] mask `DraftTreeBatch.finalize` writes.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import Optional

import torch

from . import _lib


def _i32(t: Optional[torch.Tensor], dev, n: int, what: str) -> int:
    if t is None:
        return 0
    if t.dtype != torch.int32 or t.device != dev or t.numel() != n or not t.is_contiguous():
        raise ValueError(f"{what} must be a contiguous int32 [{n}] tensor on the pool's device")
    return t.data_ptr()


_MASK_KINDS = {torch.bool: _lib.MASK_BOOL, torch.uint8: _lib.MASK_BOOL, torch.float32: _lib.MASK_ADD_F32,
               torch.bfloat16: _lib.MASK_ADD_BF16, torch.float16: _lib.MASK_ADD_F16}


_SMS = 148  # B200


def _split_cache(a, batch: int, q_heads: int, kv_heads: int, q_len: int, cap_rows: int, device, kv_splits):
    """Few requests with long caches would keep batch * kv_heads CTAs busy: cut the cache rows of each into
    `kv_splits` ranges (partial results combined by a second kernel).  None: as many as fill the SMs once, at
    most one per four 64-row tiles of the cache's capacity and at most 16 (measured: a lone request behind 4096
    rows 75 -> 25 us; more CTAs than SMs, or ranges of a tile or two, cost more than they bring).  Returns the
    scratch tensor to keep alive."""
    ctas = batch * kv_heads * ((q_heads // kv_heads * q_len + 255) // 256)
    if kv_splits is None:
        kv_splits = max(1, min(_SMS // max(ctas, 1), (cap_rows + 63) // 64 // 4, 16))
    kv_splits = int(kv_splits)
    if kv_splits < 1 or kv_splits > 1024:
        raise ValueError("kv_splits must be between 1 and 1024")
    if kv_splits == 1:
        return None
    scratch = torch.empty(batch * q_heads * q_len * kv_splits * 130, dtype=torch.float32, device=device)
    a.kv_splits, a.split_scratch = kv_splits, scratch.data_ptr()
    return scratch


@torch.no_grad()
def append_paged_kv(pool: torch.Tensor, layer: int, k: torch.Tensor, v: torch.Tensor, *, page_table: torch.Tensor,
                    kv_len: torch.Tensor, n_q: Optional[torch.Tensor] = None,
                    status: Optional[torch.Tensor] = None) -> None:
    """k, v [batch, q_len, kv_heads, head_dim] -> cache rows kv_len[b] - n_q[b] + i of layer `layer`.

    `kv_len` counts the rows AFTER the append (grow the requests first, as `RequestKvCache.increment` does)."""
    L, P, _, page_len, H, D = pool.shape
    B, QL = int(k.shape[0]), int(k.shape[1])
    if k.shape != v.shape or tuple(k.shape[2:]) != (H, D) or k.dtype != pool.dtype or v.dtype != pool.dtype or \
            k.stride() != v.stride() or pool.element_size() != 2:
        raise ValueError("k and v must be [batch, q_len, kv_heads, head_dim] tensors of the pool's (16-bit) dtype and one layout")
    if k.stride(3) != 1 or k.stride(2) != D:
        k, v = k.contiguous(), v.contiguous()
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or not page_table.is_contiguous():
        raise ValueError("page_table must be a contiguous int32 [batch, pages_per_seq] tensor")
    a = _lib.KvAppendArgs()
    a.struct_size = C.sizeof(_lib.KvAppendArgs)
    a.batch, a.q_len, a.num_kv_heads, a.head_dim = B, QL, int(H), int(D)
    a.layer, a.layers, a.num_pages, a.page_len = int(layer), int(L), int(P), int(page_len)
    a.pages_per_seq = int(page_table.shape[1])
    a.pool, a.page_table = pool.data_ptr(), page_table.data_ptr()
    a.kv_len = _i32(kv_len, pool.device, B, "kv_len")
    a.n_q = _i32(n_q, pool.device, B, "n_q")
    a.k, a.v = k.data_ptr(), v.data_ptr()
    a.batch_stride, a.token_stride = int(k.stride(0)), int(k.stride(1))
    a.dev_status = 0 if status is None else status.data_ptr()
    stream = torch.cuda.current_stream(pool.device).cuda_stream
    _lib.check(_lib.lib().subspec_kv_append_paged(C.byref(a), C.c_void_p(stream)), "subspec_kv_append_paged")


@torch.no_grad()
def tree_attention_paged(q: torch.Tensor, pool: torch.Tensor, layer: int, *, page_table: torch.Tensor,
                         kv_len: torch.Tensor, mask: torch.Tensor, n_q: Optional[torch.Tensor] = None,
                         prefix_len: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None,
                         status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                         kv_splits: Optional[int] = None) -> torch.Tensor:
    """q [batch, q_len, q_heads, head_dim (64 or 128)] bf16 or fp16 (as the pool) -> attention output of the same shape (into `out` when given: a
    captured graph needs a buffer that outlives the capture).

    `mask` is bool / uint8 [batch or 1, q_len, cols >= kv_len] (a singleton head axis after the batch axis is
    accepted), or the additive form `invert_mask` makes of it (0 = visible) in float32 / bfloat16 / float16: row i
    of request b marks the cache rows its query i may read; rows below `prefix_len[b]` (default kv_len - n_q) are
    read without looking at the mask."""
    if q.dtype not in (torch.bfloat16, torch.float16) or pool.dtype != q.dtype or q.dim() != 4:
        raise ValueError("q must be bf16 or fp16 [batch, q_len, q_heads, head_dim] and the pool of the same type")
    L, P, _, page_len, H, D = pool.shape
    B, QL, HQ, Dq = (int(x) for x in q.shape)
    if Dq != D or q.stride(3) != 1 or D not in (64, 128):
        raise ValueError("q's head_dim must equal the pool's, be contiguous and be 64 or 128")
    if mask.dim() == 4 and mask.shape[1] == 1:
        mask = mask[:, 0]
    if mask.dim() != 3 or mask.shape[0] not in (1, B) or mask.shape[1] < QL or mask.stride(2) != 1 or \
            mask.dtype not in _MASK_KINDS:
        raise ValueError("mask must be [batch or 1, q_len, cols] with contiguous columns: bool / uint8, or the "
                         "additive form (0 = visible) in float32 / bfloat16 / float16")
    if page_table.dtype != torch.int32 or page_table.dim() != 2 or not page_table.is_contiguous():
        raise ValueError("page_table must be a contiguous int32 [batch, pages_per_seq] tensor")
    if out is None:
        out = torch.empty_like(q)
    elif out.dtype != q.dtype or out.shape != q.shape or out.device != q.device or out.stride(3) != 1:
        raise ValueError("out must be a tensor of q's type and shape on q's device with contiguous head_dim")
    a = _lib.TreeAttnArgs()
    a.struct_size = C.sizeof(_lib.TreeAttnArgs)
    a.batch, a.q_len, a.num_q_heads, a.num_kv_heads, a.head_dim = B, QL, HQ, int(H), int(D)
    a.layer, a.layers, a.num_pages, a.page_len = int(layer), int(L), int(P), int(page_len)
    a.pages_per_seq = int(page_table.shape[1])
    a.pool, a.page_table = pool.data_ptr(), page_table.data_ptr()
    a.kv_len = _i32(kv_len, pool.device, B, "kv_len")
    a.n_q = _i32(n_q, pool.device, B, "n_q")
    a.prefix_len = _i32(prefix_len, pool.device, B, "prefix_len")
    a.mask, a.mask_row_stride = mask.data_ptr(), int(mask.stride(1))
    a.mask_batch_stride = int(mask.stride(0)) if mask.shape[0] == B else 0
    a.mask_kind = _MASK_KINDS[mask.dtype]
    a.q, a.q_batch_stride, a.q_token_stride, a.q_head_stride = q.data_ptr(), *(int(q.stride(i)) for i in range(3))
    a.out, a.o_batch_stride, a.o_token_stride, a.o_head_stride = out.data_ptr(), *(int(out.stride(i)) for i in range(3))
    a.sm_scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
    a.dtype = _lib.BF16 if q.dtype == torch.bfloat16 else _lib.F16
    a.dev_status = 0 if status is None else status.data_ptr()
    scratch = _split_cache(a, B, HQ, int(H), QL, int(page_table.shape[1]) * int(page_len), pool.device, kv_splits)
    stream = torch.cuda.current_stream(pool.device).cuda_stream
    _lib.check(_lib.lib().subspec_tree_attention_paged(C.byref(a), C.c_void_p(stream)),
               "subspec_tree_attention_paged")
    del scratch  # (torch's allocator keeps the block for this stream until the kernels have passed)
    return out


@torch.no_grad()
def tree_attention_static(q: torch.Tensor, key_cache: torch.Tensor, value_cache: torch.Tensor, *, kv_len: torch.Tensor,
                          mask: torch.Tensor, n_q: Optional[torch.Tensor] = None,
                          prefix_len: Optional[torch.Tensor] = None, sm_scale: Optional[float] = None,
                          status: Optional[torch.Tensor] = None, out: Optional[torch.Tensor] = None,
                          kv_splits: Optional[int] = None) -> torch.Tensor:
    """The same kernel over the static caches of the reference's default (Hugging Face) path: what
    `scaled_dot_product_attention(q, repeat_kv(k), repeat_kv(v), attn_mask=mask)` computes for the tree's tokens.

    q [batch, q_heads, q_len, 128], key_cache / value_cache [batch, kv_heads, max_cache_len, 128] of one layer
    (TreeStaticCache, specdecodes/models/utils/cache_utils.py; the tree's own K / V rows already written at
    kv_len - n_q ...), all bf16 or fp16; `mask` [batch or 1, 1, q_len, cols >= kv_len] bool or additive (the
    `[1, 1, max_verify, max_cache_len]` buffer the tree finaliser fills); kv_len[b] = rows of request b incl. the
    tree's.  Returns [batch, q_heads, q_len, 128] (or fills `out`)."""
    if q.dim() != 4 or key_cache.dim() != 4 or key_cache.shape != value_cache.shape or \
            key_cache.stride() != value_cache.stride():
        raise ValueError("q must be [batch, q_heads, q_len, head_dim] and the caches two [batch, kv_heads, rows, "
                         "head_dim] tensors of one shape and layout")
    if q.dtype not in (torch.bfloat16, torch.float16) or key_cache.dtype != q.dtype or value_cache.dtype != q.dtype:
        raise ValueError("q and the caches must be bf16 or fp16, all of the same type")
    B, HQ, QL, D = (int(x) for x in q.shape)
    Bk, H, S, Dk = (int(x) for x in key_cache.shape)
    if Bk < B or Dk != D or q.stride(3) != 1 or key_cache.stride(3) != 1 or D not in (64, 128):
        raise ValueError("the caches must hold the batch, share q's head_dim (64 or 128), and head_dim must be contiguous")
    if mask.dim() == 4 and mask.shape[1] == 1:
        mask = mask[:, 0]
    if mask.dim() != 3 or mask.shape[0] not in (1, B) or mask.shape[1] < QL or mask.stride(2) != 1 or \
            mask.dtype not in _MASK_KINDS:
        raise ValueError("mask must be [batch or 1, (1,) q_len, cols] with contiguous columns, bool or additive")
    if out is None:
        out = torch.empty_like(q)
    elif out.dtype != q.dtype or out.shape != q.shape or out.device != q.device or out.stride(3) != 1:
        raise ValueError("out must be a tensor of q's type and shape on q's device with contiguous head_dim")
    a = _lib.TreeAttnArgs()
    a.struct_size = C.sizeof(_lib.TreeAttnArgs)
    a.batch, a.q_len, a.num_q_heads, a.num_kv_heads, a.head_dim = B, QL, HQ, H, D
    a.layer, a.layers, a.num_pages, a.page_len, a.pages_per_seq = 0, 1, Bk, S, 1
    a.pool, a.v_cache, a.page_table = key_cache.data_ptr(), value_cache.data_ptr(), 0
    a.kv_batch_stride, a.kv_head_stride, a.kv_row_stride = (int(key_cache.stride(i)) for i in range(3))
    a.kv_len = _i32(kv_len, q.device, B, "kv_len")
    a.n_q = _i32(n_q, q.device, B, "n_q")
    a.prefix_len = _i32(prefix_len, q.device, B, "prefix_len")
    a.mask, a.mask_row_stride = mask.data_ptr(), int(mask.stride(1))
    a.mask_batch_stride = int(mask.stride(0)) if mask.shape[0] == B else 0
    a.mask_kind = _MASK_KINDS[mask.dtype]
    a.q, a.q_batch_stride, a.q_head_stride, a.q_token_stride = q.data_ptr(), *(int(q.stride(i)) for i in range(3))
    a.out, a.o_batch_stride, a.o_head_stride, a.o_token_stride = out.data_ptr(), *(int(out.stride(i)) for i in range(3))
    a.sm_scale = float(sm_scale) if sm_scale is not None else 1.0 / math.sqrt(D)
    a.dtype = _lib.BF16 if q.dtype == torch.bfloat16 else _lib.F16
    a.dev_status = 0 if status is None else status.data_ptr()
    scratch = _split_cache(a, B, HQ, H, QL, S, q.device, kv_splits)
    stream = torch.cuda.current_stream(q.device).cuda_stream
    _lib.check(_lib.lib().subspec_tree_attention_paged(C.byref(a), C.c_void_p(stream)),
               "subspec_tree_attention_paged")
    del scratch
    return out
