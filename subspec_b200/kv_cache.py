"""KV-cache managers with the reference's call surface, backed by the TMA compaction kernel.

Reference classes mirrored here (specdecodes/models/utils/...):
  cache_utils.py:41-60     KVManager
  cache_utils.py:62-109    TreeDynamicCache   (HF layout, tensors grow)
  cache_utils.py:112-208   TreeStaticCache    (HF layout, preallocated [B, H, T, D] per layer)
  flashinfer/cache_manager.py:9-33    KvCacheBatchPosition
  flashinfer/cache_manager.py:35-213  KvCachePool  ([L, pages, 2, page_len, H, D])
  flashinfer/cache_manager.py:216-348 RequestKvCache
  flashinfer/cache_manager.py:350-414 getKvCacheBatchPosition

What changes is what sits behind `reorder_cache_with_offset`: the reference
clones / re-stacks the entire cache and copies it back every step; here one
kernel launch moves only the accepted rows (`subspec_kv_compact_paged` /
`subspec_kv_compact_hf`).  The bytes that end up in rows [offset, offset + n)
are identical; rows beyond stay as they were, as in the reference.

Page tables.  The reference's pool-level reorder maps a logical position p to
physical page p // page_len, i.e. it assumes the request owns pages 0, 1, 2, ...
(`KvCachePool.reorder_cache_with_offset`, cache_manager.py:144-153) and ignores
`RequestKvCache.kv_page_indices`.  `KvCachePool.reorder_cache_with_offset` keeps
exactly that meaning.  `RequestKvCache.reorder_cache_with_offset` translates
through the request's own page list, which is the same thing whenever the
request owns the leading pages (the only layout the reference works with) and is
what a pool shared by several requests needs.
"""
from __future__ import annotations

import ctypes as C
import math
from typing import List, Optional, Sequence

import torch

from . import _lib

MAX_BEAM = 1025


def _elem_bytes(dtype: torch.dtype) -> int:
    if dtype in (torch.bfloat16, torch.float16):
        return 2
    if dtype == torch.float32:
        return 4
    raise ValueError(f"unsupported KV dtype {dtype}")


def _status_word(device) -> torch.Tensor:
    return torch.zeros(1, dtype=torch.int32, device=device)


def _check_status(status: torch.Tensor) -> None:
    word = int(status.item())
    if word:
        raise ValueError("KV compaction rejected its input: " + _lib.dev_status_text(word))


def _beam_tensor(beam_idx, device) -> torch.Tensor:
    beam = torch.as_tensor(beam_idx, dtype=torch.int64).reshape(1, -1)
    if beam.shape[1] > MAX_BEAM:
        raise ValueError(f"at most {MAX_BEAM} rows can be kept per step, got {beam.shape[1]}")
    return beam.to(device).contiguous()


def compact_paged(pool: torch.Tensor, *, page_table: Optional[torch.Tensor], offset: torch.Tensor, n: torch.Tensor,
                  beam: torch.Tensor, status: Optional[torch.Tensor] = None, n_stride: int = 1) -> None:
    """Batched accepted-path compaction of a paged pool [L, pages, 2, page_len, H, D], in place.

    offset / n are int32 [batch] and beam int64 [batch, max_beam] DEVICE tensors
    (the verifier's out_meta / out_hidden can be passed as they are); page_table is
    int32 [batch, pages_per_seq] or None for the identity table.  Runs on the
    current stream and does not synchronise.
    """
    if pool.dim() != 6 or pool.shape[2] != 2 or not pool.is_contiguous():
        raise ValueError("pool must be a contiguous [layers, pages, 2, page_len, heads, head_dim] tensor")
    L, P, _, page_len, H, D = pool.shape
    a = _lib.KvPagedArgs()
    a.struct_size = C.sizeof(_lib.KvPagedArgs)
    a.batch = int(offset.numel())
    a.layers, a.num_pages, a.page_len, a.heads, a.head_dim = int(L), int(P), int(page_len), int(H), int(D)
    a.elem_bytes = _elem_bytes(pool.dtype)
    a.pool = pool.data_ptr()
    if page_table is not None:
        if page_table.dtype != torch.int32 or not page_table.is_contiguous() or page_table.dim() != 2:
            raise ValueError("page_table must be a contiguous int32 [batch, pages_per_seq] tensor")
        a.page_table, a.pages_per_seq = page_table.data_ptr(), int(page_table.shape[1])
    for t, dt in ((offset, torch.int32), (n, torch.int32), (beam, torch.int64)):
        if t.dtype != dt or (not t.is_contiguous() and t is not n) or t.device != pool.device:
            raise ValueError("offset/n must be int32 and beam int64, contiguous, on the pool's device")
    a.offset, a.n, a.beam = offset.data_ptr(), n.data_ptr(), beam.data_ptr()
    a.max_beam = int(beam.shape[1])
    a.n_stride = int(n_stride)
    a.dev_status = 0 if status is None else status.data_ptr()
    stream = torch.cuda.current_stream(pool.device).cuda_stream
    _lib.check(_lib.lib().subspec_kv_compact_paged(C.byref(a), C.c_void_p(stream)), "subspec_kv_compact_paged")


def compact_hf(tensors: Sequence[torch.Tensor], *, offset: torch.Tensor, n: torch.Tensor, beam: torch.Tensor,
               ptr_table: Optional[torch.Tensor] = None, status: Optional[torch.Tensor] = None) -> None:
    """Batched compaction of HF-layout caches: `tensors` are [B, H, T, D] K/V tensors of identical shape/strides."""
    t0 = tensors[0]
    B, H, T, D = t0.shape
    for t in tensors:
        if t.shape != t0.shape or t.stride() != t0.stride() or t.dtype != t0.dtype or t.stride(3) != 1:
            raise ValueError("all cache tensors must share shape, strides and dtype, with head_dim contiguous")
        if t.data_ptr() % 16:
            raise ValueError("cache tensors must be 16-byte aligned")
    if ptr_table is None:
        ptr_table = torch.tensor([t.data_ptr() for t in tensors], dtype=torch.int64, device=t0.device)
    a = _lib.KvHfArgs()
    a.struct_size = C.sizeof(_lib.KvHfArgs)
    a.batch, a.num_tensors, a.heads, a.tokens, a.head_dim = int(B), len(tensors), int(H), int(T), int(D)
    a.elem_bytes = _elem_bytes(t0.dtype)
    a.batch_stride, a.head_stride, a.token_stride = (int(s) for s in t0.stride()[:3])
    a.layer_ptrs = ptr_table.data_ptr()
    a.offset, a.n, a.beam = offset.data_ptr(), n.data_ptr(), beam.data_ptr()
    a.max_beam = int(beam.shape[1])
    a.n_stride = 1
    a.dev_status = 0 if status is None else status.data_ptr()
    stream = torch.cuda.current_stream(t0.device).cuda_stream
    _lib.check(_lib.lib().subspec_kv_compact_hf(C.byref(a), C.c_void_p(stream)), "subspec_kv_compact_hf")
    del ptr_table


# ---------------------------------------------------------------------------------
# HF layout
# ---------------------------------------------------------------------------------
class KVManager:
    """cache_utils.py:41-60."""

    def __init__(self, cache):
        self.cache = cache
        self.seq_len = 0

    def get_seq_length(self) -> int:
        return self.seq_len

    def crop(self, start: int, end: Optional[int] = None, dim: int = 2) -> None:
        if end is None:
            end = self.get_seq_length()
        self.cache.crop(start, end, dim)

    def reorder_cache_with_offset(self, beam_idx, new_chunk_len=1, offset=0, dim=0):
        self.cache.reorder_cache_with_offset(beam_idx, new_chunk_len, offset, dim)

    def reset(self):
        self.cache.reset()
        self.seq_len = 0


class _HfLayoutCache:
    """key_cache / value_cache lists of [B, H, T, D] tensors (the attribute names the reference relies on)."""

    def __init__(self) -> None:
        self.key_cache: List[torch.Tensor] = []
        self.value_cache: List[torch.Tensor] = []
        self._ptr_table: Optional[torch.Tensor] = None
        self._ptr_key = None

    def __len__(self) -> int:
        return len(self.key_cache)

    def _interleaved(self) -> List[torch.Tensor]:
        out: List[torch.Tensor] = []
        for k, v in zip(self.key_cache, self.value_cache):
            out.extend((k, v))
        return out

    def _compact(self, beam_idx, offset: int) -> int:
        tensors = self._interleaved()
        if not tensors:
            return 0
        dev = tensors[0].device
        beam = _beam_tensor(beam_idx, dev)
        n = int(beam.shape[1])
        B = tensors[0].shape[0]
        beam = beam.expand(B, n).contiguous()
        off = torch.full((B,), int(offset), dtype=torch.int32, device=dev)
        cnt = torch.full((B,), n, dtype=torch.int32, device=dev)
        key = tuple(t.data_ptr() for t in tensors)
        if self._ptr_key != key:
            self._ptr_table = torch.tensor(key, dtype=torch.int64, device=dev)
            self._ptr_key = key
        status = _status_word(dev)
        compact_hf(tensors, offset=off, n=cnt, beam=beam, ptr_table=self._ptr_table, status=status)
        _check_status(status)
        return n


class TreeStaticCache(_HfLayoutCache):
    """Preallocated cache; `reorder_cache_with_offset` keeps every tensor's address (cache_utils.py:112-208)."""

    def __init__(self, config=None, max_cache_len: Optional[int] = None, device=None, dtype=torch.float32,
                 max_batch_size: Optional[int] = None, *, num_layers: Optional[int] = None,
                 num_kv_heads: Optional[int] = None, head_dim: Optional[int] = None) -> None:
        super().__init__()
        if config is not None:
            num_layers = num_layers or config.num_hidden_layers
            num_kv_heads = num_kv_heads or getattr(config, "num_key_value_heads", config.num_attention_heads)
            head_dim = head_dim or getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        if None in (num_layers, num_kv_heads, head_dim, max_cache_len):
            raise ValueError("config (or num_layers/num_kv_heads/head_dim) and max_cache_len must be provided")
        self.max_cache_len = int(max_cache_len)
        self.max_batch_size = int(max_batch_size or 1)
        shape = (self.max_batch_size, int(num_kv_heads), self.max_cache_len, int(head_dim))
        for _ in range(int(num_layers)):
            self.key_cache.append(torch.zeros(shape, dtype=dtype, device=device))
            self.value_cache.append(torch.zeros(shape, dtype=dtype, device=device))
        self._seen = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return self._seen

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs=None):
        pos = (cache_kwargs or {}).get("cache_position")
        if pos is None:
            pos = torch.arange(self._seen, self._seen + key_states.shape[2], device=key_states.device)
        self.key_cache[layer_idx].index_copy_(2, pos, key_states)
        self.value_cache[layer_idx].index_copy_(2, pos, value_states)
        if layer_idx == len(self.key_cache) - 1:
            self._seen = int(pos[-1]) + 1
        return self.key_cache[layer_idx], self.value_cache[layer_idx]

    def reset(self):
        for k, v in zip(self.key_cache, self.value_cache):
            k.zero_()
            v.zero_()
        self._seen = 0

    def crop(self, start: int, end: Optional[int] = None, dim: int = 2) -> None:
        """Zero the token range [start, end) (negative start counts from `end`), cache_utils.py:136-164."""
        if end is None:
            end = self.get_seq_length()
        if start < 0:
            start = end + start
        if end <= start:
            return
        for k, v in zip(self.key_cache, self.value_cache):
            k[:, :, start:end].zero_()
            v[:, :, start:end].zero_()

    def reorder_cache_with_offset(self, beam_idx, new_chunk_len: int = 1, offset: int = 0, dim: int = 0) -> None:
        self._compact(beam_idx, offset)


class TreeDynamicCache(_HfLayoutCache):
    """Growing cache (cache_utils.py:62-109).  After a reorder each tensor is a view of its first offset + n rows."""

    def __init__(self) -> None:
        super().__init__()
        self._seen_tokens = 0

    def get_seq_length(self, layer_idx: int = 0) -> int:
        return 0 if not self.key_cache else int(self.key_cache[layer_idx].shape[2])

    def update(self, key_states, value_states, layer_idx: int, cache_kwargs=None):
        if layer_idx == 0:
            self._seen_tokens += key_states.shape[2]
        if len(self.key_cache) <= layer_idx:
            self.key_cache.append(key_states.contiguous())
            self.value_cache.append(value_states.contiguous())
        else:
            self.key_cache[layer_idx] = torch.cat([self.key_cache[layer_idx], key_states], dim=2)
            self.value_cache[layer_idx] = torch.cat([self.value_cache[layer_idx], value_states], dim=2)
        return self.key_cache[layer_idx], self.value_cache[layer_idx]

    def crop(self, start: int, end: Optional[int] = None, dim: int = 2) -> None:
        if end is not None and start < 0:
            start = end - abs(start)
        self._seen_tokens = start
        for i in range(len(self.key_cache)):
            self.key_cache[i] = self.key_cache[i][..., :start, :]
            self.value_cache[i] = self.value_cache[i][..., :start, :]

    def reorder_cache_with_offset(self, beam_idx, new_chunk_len: int = 1, offset: int = 0, dim: int = 0) -> None:
        n = self._compact(beam_idx, offset)
        keep = int(offset) + n
        for i in range(len(self.key_cache)):
            self.key_cache[i] = self.key_cache[i][..., :keep, :]
            self.value_cache[i] = self.value_cache[i][..., :keep, :]

    def reset(self):
        self._seen_tokens = 0
        self.key_cache = []
        self.value_cache = []
        self._ptr_key = None


def create_kv_cache(cache_implementation: str = "dynamic", max_cache_len: Optional[int] = None,
                    max_batch_size: Optional[int] = None, config=None, device="cpu", dtype="float16") -> KVManager:
    """cache_utils.py:6-39."""
    if isinstance(dtype, str):
        if not hasattr(torch, dtype):
            raise ValueError(f"Unsupported dtype string: {dtype}")
        dtype = getattr(torch, dtype)
    if cache_implementation == "dynamic":
        cache = TreeDynamicCache()
    elif cache_implementation == "static":
        if config is None:
            raise ValueError("config must be provided for static cache")
        cache = TreeStaticCache(config=config, max_cache_len=max_cache_len, max_batch_size=max_batch_size,
                                device=device, dtype=dtype)
    else:
        raise ValueError(f"Unsupported cache_implementation: {cache_implementation}")
    return KVManager(cache)


# ---------------------------------------------------------------------------------
# paged layout
# ---------------------------------------------------------------------------------
class KvCacheBatchPosition:
    """cache_manager.py:9-33."""

    def __init__(self, seq_indptr, kv_page_indptr, kv_page_indices, kv_last_page_len, batch_indices, positions):
        self.batch_indices = batch_indices
        self.kv_page_indices = kv_page_indices
        self.positions = positions
        self.kv_page_indptr = kv_page_indptr
        self.kv_last_page_len = kv_last_page_len
        self.seq_indptr = seq_indptr

    def print_info(self):
        for name in ("seq_indptr", "kv_page_indptr", "kv_page_indices", "kv_last_page_len", "batch_indices",
                     "positions"):
            print(f"  {name}: {getattr(self, name)}")


class KvCachePool:
    """Paged pool [layers, max_pages, 2, page_len, heads, head_dim] with a host-side free-page map."""

    def __init__(self, max_pages: int, num_layers: int, num_heads: int, head_dim: int, page_len: int,
                 dtype: torch.dtype, device):
        self.cache_data = torch.zeros(num_layers, max_pages, 2, page_len, num_heads, head_dim, dtype=dtype,
                                      device=device)
        self.num_layers = num_layers
        self.device = device
        self.max_pages = max_pages
        self.page_len = page_len
        self.free_page_mask = torch.ones(max_pages, dtype=torch.bool, device="cpu")
        self.num_heads = num_heads
        self.head_dims = head_dim
        self.dtype = dtype

    def reset(self):
        self.cache_data.zero_()

    def num_free_pages(self):
        return self.free_page_mask.sum()

    def allocate(self, num_pages: int) -> List[int]:
        free = self.free_page_mask.nonzero().squeeze(1)
        assert len(free) >= num_pages, (
            f"Out of available cache pages: asked {num_pages}, only {len(free)} free pages")
        got = free[:num_pages]
        self.free_page_mask[got] = False
        return got.tolist()

    def deallocate(self, kv_page_indices: List[int]):
        self.free_page_mask[kv_page_indices] = True

    def crop(self, seq_len: int) -> None:
        """Zero everything after `seq_len` tokens and free the fully unused pages (cache_manager.py:76-118)."""
        cap = self.max_pages * self.page_len
        if not 0 <= seq_len <= cap:
            raise ValueError(f"seq_len={seq_len} is outside the [0, {cap}] range.")
        full, rem = divmod(seq_len, self.page_len)
        keep = full + (1 if rem else 0)
        if rem:
            self.cache_data[:, full, :, rem:].zero_()
        if keep < self.max_pages:
            self.cache_data[:, keep:].zero_()
        self.free_page_mask.zero_()
        if keep < self.max_pages:
            self.free_page_mask[keep:] = True

    def _reorder(self, beam_idx, offset: int, page_table: Optional[torch.Tensor], num_new_tokens: int = 0) -> int:
        dev = self.cache_data.device
        beam = _beam_tensor(beam_idx, dev)
        n = int(beam.shape[1])
        total_pages = (int(offset) + int(num_new_tokens) + self.page_len - 1) // self.page_len
        if total_pages > self.max_pages:
            raise ValueError(
                f"Cache does not have enough pages ({self.max_pages}) for total tokens ({offset + num_new_tokens}).")
        status = _status_word(dev)
        compact_paged(self.cache_data, page_table=page_table,
                      offset=torch.full((1,), int(offset), dtype=torch.int32, device=dev),
                      n=torch.full((1,), n, dtype=torch.int32, device=dev), beam=beam, status=status)
        _check_status(status)
        return n

    def reorder_cache_with_offset(self, beam_idx, offset=0, num_new_tokens=0):
        """Pool-level reorder under the identity page table (cache_manager.py:119-213)."""
        self._reorder(beam_idx, int(offset), None, int(num_new_tokens))


class RequestKvCache:
    """Per-request page list and length bookkeeping (cache_manager.py:216-348)."""

    def __init__(self, kvCachePool: KvCachePool, page_len: int, seq_init_len: int):
        self.kvCachePool = kvCachePool
        self.page_len = page_len
        init_num_pages = math.ceil(seq_init_len / self.page_len)
        self.kv_last_page_len = seq_init_len - (init_num_pages - 1) * self.page_len
        self.kv_page_indices = kvCachePool.allocate(init_num_pages)
        self.kv_len = seq_init_len
        self.is_released = False

    def get_seq_length(self):
        return self.kv_len

    def increment(self, num_tokens: int = 1):
        self.kv_len += num_tokens
        self.kv_last_page_len += num_tokens
        while self.kv_last_page_len > self.page_len:
            self.kv_last_page_len -= self.page_len
            self.kv_page_indices.extend(self.kvCachePool.allocate(1))

    def release(self):
        self.kvCachePool.deallocate(self.kv_page_indices)
        self.is_released = True

    def _last_page_len(self) -> int:
        return 0 if self.kv_len == 0 else (self.kv_len - 1) % self.page_len + 1

    def _trim_pages(self) -> None:
        need = (self.kv_len + self.page_len - 1) // self.page_len
        have = len(self.kv_page_indices)
        if have > need:
            self.kvCachePool.deallocate(self.kv_page_indices[need:])
            self.kv_page_indices = self.kv_page_indices[:need]
        elif have < need:
            self.kv_page_indices.extend(self.kvCachePool.allocate(need - have))
            raise ValueError("a reorder never lengthens a request: it had fewer pages than its kept rows need")

    def decrement(self, num_tokens: int = 1):
        if num_tokens <= 0:
            return
        self.kv_len -= min(num_tokens, self.kv_len)
        need = (self.kv_len + self.page_len - 1) // self.page_len if self.kv_len > 0 else 0
        while len(self.kv_page_indices) > need:
            self.kvCachePool.deallocate([self.kv_page_indices.pop()])
        self.kv_last_page_len = self._last_page_len()

    def crop(self, start: int, end=None, dim=0):
        if end is None:
            end = self.get_seq_length()
        if start < 0:
            start = end - abs(start)
        if end <= start:
            return
        self.kv_len = start
        self.kv_last_page_len = self._last_page_len()
        self._trim_pages()

    def page_table(self, device=None) -> torch.Tensor:
        return torch.tensor([self.kv_page_indices], dtype=torch.int32, device=device or self.kvCachePool.device)

    def reorder_cache_with_offset(self, beam_idx, offset=0, num_new_tokens=0):
        """Keep rows offset + beam_idx of this request (callers pass offset = kv_len + 1, cache_manager.py:318-319)."""
        if offset != 0:
            offset -= 1
        self.kvCachePool._reorder(beam_idx, int(offset), self.page_table(), int(num_new_tokens))
        self.kv_len = offset + int(torch.as_tensor(beam_idx).numel())
        self.kv_last_page_len = self._last_page_len()
        self._trim_pages()


def getKvCacheBatchPosition(request_kv_caches: List[RequestKvCache], mode: str, device, treeTokens: int = 0
                            ) -> KvCacheBatchPosition:
    """Page-table tensors for a batch of requests (cache_manager.py:350-414).

    `batch_indices` / `positions` restate flashinfer.get_batch_indices_positions
    for the single append segment the reference builds (kv_append_indptr =
    [0, total appended]): every appended token belongs to request 0 and sits at
    position kv_len(request 0) - total + i.
    """
    page_indices: List[int] = []
    page_indptr, seq_indptr, last_len, seq_lens = [], [], [], []
    cum_pages = cum_seq = 0
    for r in request_kv_caches:
        page_indices.extend(r.kv_page_indices)
        page_indptr.append(cum_pages)
        seq_indptr.append(cum_seq)
        last_len.append(r.kv_last_page_len)
        seq_lens.append(r.kv_len)
        cum_pages += len(r.kv_page_indices)
        if mode == "prefill":
            cum_seq += r.kv_len
        elif mode == "decode":
            cum_seq += 1
        elif mode == "tree":
            cum_seq += treeTokens
        else:
            raise ValueError("invalid mode")
    page_indptr.append(cum_pages)
    seq_indptr.append(cum_seq)

    def i32(x):
        return torch.tensor(x, dtype=torch.int32, device=device)

    batch_indices = torch.zeros(cum_seq, dtype=torch.int32, device=device)
    positions = (torch.arange(cum_seq, dtype=torch.int32, device=device) + (seq_lens[0] - cum_seq)
                 if seq_lens else torch.zeros(0, dtype=torch.int32, device=device))
    return KvCacheBatchPosition(seq_indptr=i32(seq_indptr), kv_page_indptr=i32(page_indptr),
                                kv_page_indices=i32(page_indices), kv_last_page_len=i32(last_len),
                                batch_indices=batch_indices, positions=positions)


class FlashInferCache:
    """The reference's holder of the paged pool (flashinfer/cache_manager.py:419-466): same constructor
    (`config`, `max_tokens`, `PAGE_LEN`), same attributes (`config`, `max_cache_len`, `kvCachePool`), same
    memory check (`CUDA_MEMORY_FRACTION`), fp16 pool on the current device.

    The reference sizes the pool at ONE page whatever `max_tokens` says (its line 451); `max_pages` is an
    addition that lets a caller get a pool that holds something, and defaults to the reference's value.
    """

    def __init__(self, config, max_tokens: Optional[int] = None, PAGE_LEN: int = 16,
                 max_pages: Optional[int] = None) -> None:
        import os

        device = torch.device("cuda", torch.cuda.current_device())
        dtype_size = torch.tensor([], dtype=torch.float16).element_size()
        self.config = config
        head_dim = getattr(config, "head_dim", config.hidden_size // config.num_attention_heads)
        fraction = float(os.getenv("CUDA_MEMORY_FRACTION", "1.0"))
        self.max_cache_len = max_tokens
        page_bytes = 2 * PAGE_LEN * config.num_hidden_layers * config.num_key_value_heads * head_dim * dtype_size
        free_now, _ = torch.cuda.mem_get_info(device)
        total = torch.cuda.get_device_properties(device).total_memory
        free = max(0, free_now - (1 - fraction) * total)
        if free < page_bytes:
            raise RuntimeError(
                f"Not enough GPU memory to allocate even a single cache page "
                f"({page_bytes / (1024**2):.2f} MiB required, {free / (1024**2):.2f} MiB available).")
        self.kvCachePool = KvCachePool(max_pages=1 if max_pages is None else int(max_pages),
                                       num_layers=config.num_hidden_layers, num_heads=config.num_key_value_heads,
                                       head_dim=head_dim, page_len=PAGE_LEN, dtype=torch.float16, device=device)

    def reset(self):
        self.kvCachePool.reset()
