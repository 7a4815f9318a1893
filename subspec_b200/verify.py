"""Tree verify + accept behind the reference's `verify_tree` / `lossy_bottom_up_verify` signatures.

The arithmetic runs in one fused sm_100a kernel per batch
(`subspec_verify_batched`, include/subspec_b200.h); this module only flattens
trees into the kernel's arrays, launches, and turns the outputs back into the
tuples the reference's generators expect:

  verify_tree(...)            -> (sampled_tokens [1, L], hidden_indices [L], (total_len, accept_len))
                                 specdecodes/models/utils/tree_verify.py:7-163
  lossy_bottom_up_verify(...) -> (sampled [L], hidden [L], accept_len)
                                 specdecodes/models/utils/lossy_tree_verify.py:9-343

`verify_tree_batched` is the same operation over a batch of independent
sequences in one launch.  There is no CPU fallback: tensors are moved to the GPU
if they are not there already, and a missing CUDA library raises.
"""
from __future__ import annotations

import ctypes as C
import math
from dataclasses import dataclass
from typing import Any, Dict, List, Optional, Sequence, Tuple

import numpy as np
import torch

from . import _lib
from .wandb_logger import wandb_logger

_I32 = np.dtype(np.int32)


def _align(x: int, a: int) -> int:
    return (x + a - 1) // a * a


def _device_of(t: Optional[torch.Tensor]) -> torch.device:
    if t is not None and t.is_cuda:
        return t.device
    if not torch.cuda.is_available():
        raise _lib.SubspecError("subspec_b200 needs a CUDA device (sm_100a); there is no CPU path")
    return torch.device("cuda", torch.cuda.current_device())


class VerifyWorkspace:
    """Device + pinned-host buffers for verifying `batch` trees of up to `max_nodes` nodes.

    All small inputs travel in one host->device copy and all outputs come back in
    one device->host copy.  A workspace is tied to one device and must not be used
    by two launches that overlap on the GPU (they share the scratch area).
    """

    def __init__(self, batch: int, max_nodes: int, device: torch.device):
        if not 1 <= max_nodes <= 1024:
            raise ValueError("max_nodes must be in [1, 1024]")
        device = torch.device(device)
        if device.type == "cuda" and device.index is None:  # "cuda" means the current device
            device = torch.device("cuda", torch.cuda.current_device())
        self.batch, self.max_nodes, self.device = int(batch), int(max_nodes), device
        B, N = self.batch, self.max_nodes
        self.max_out = N + 1
        # ---- int32 inputs, one block ----
        self._in_off: Dict[str, Tuple[int, int]] = {}
        cur = 0
        for name, cnt in (("n_nodes", B), ("n_rows", B), ("root", B), ("token_ids", B * N),
                          ("child_off", B * (N + 1)), ("child_idx", B * N)):
            self._in_off[name] = (cur, cnt)
            cur += _align(cnt, 4)
        self._in_host = torch.zeros(cur, dtype=torch.int32).pin_memory()
        self._in_dev = torch.zeros(cur, dtype=torch.int32, device=self.device)
        # ---- outputs, one block of bytes ----
        self._out_off: Dict[str, Tuple[int, int, np.dtype]] = {}
        cur = 0
        for name, cnt, dt in (("out_tokens", B * self.max_out, np.int64), ("out_hidden", B * self.max_out, np.int64),
                              ("out_meta", B * 4, np.int32), ("node_target", B * N, np.int32),
                              ("node_entropy", B * N, np.float32), ("node_child_prob", B * N, np.float32),
                              ("node_rowmax", B * N, np.float32), ("node_rowsum", B * N, np.float32),
                              ("node_exact_after", B * N, np.int32), ("node_best_len", B * N, np.int32),
                              ("node_best_next", B * N, np.int32), ("dev_status", 1, np.uint32),
                              # results of the exact walk when one launch verifies exactly AND lossily
                              ("out2_tokens", B * self.max_out, np.int64), ("out2_hidden", B * self.max_out, np.int64),
                              ("out2_meta", B * 4, np.int32)):
            dt = np.dtype(dt)
            self._out_off[name] = (cur, cnt, dt)
            cur += _align(cnt * dt.itemsize, 16)
        self._out_dev = torch.zeros(cur, dtype=torch.uint8, device=self.device)
        self._out_host = torch.zeros(cur, dtype=torch.uint8).pin_memory()
        self.uniforms = torch.zeros(B * N, dtype=torch.float32, device=self.device)
        self.accept_uniforms = torch.zeros(B * N, dtype=torch.float32, device=self.device)  # residual acceptance
        need = C.c_size_t(0)
        _lib.check(_lib.lib().subspec_verify_scratch_bytes(B, N, C.byref(need)), "subspec_verify_scratch_bytes")
        # zeroed once: every launch leaves the ticket words at its start zero, and run() says so to the
        # library (SUBSPEC_VERIFY_SCRATCH_CLEAN), which then puts no clearing operation in front of the kernel
        self.scratch = torch.zeros(need.value + 256, dtype=torch.uint8, device=self.device)
        self.scratch_clean = True  # False: the library clears the tickets itself before every launch
        self._scratch_ptr = _align(self.scratch.data_ptr(), 256)
        self._scratch_bytes = need.value

    # -- inputs -------------------------------------------------------------------
    def host_view(self, name: str) -> np.ndarray:
        off, cnt = self._in_off[name]
        return self._in_host.numpy()[off:off + cnt]

    def set_trees(self, flats: Sequence[Tuple[np.ndarray, np.ndarray, np.ndarray, int, int]]) -> None:
        """Stage `batch` flattened trees: (token_ids, child_off, child_idx, n_rows, root) per sequence.

        Children lists that are not a forest (an index outside the tree, a node listed twice, a loop) are
        rejected here with ValueError, before anything is launched; so are row counts beyond the node count."""
        B, N = self.batch, self.max_nodes
        if len(flats) != B:
            raise ValueError(f"expected {B} trees, got {len(flats)}")
        tok = self.host_view("token_ids").reshape(B, N)
        off = self.host_view("child_off").reshape(B, N + 1)
        idx = self.host_view("child_idx").reshape(B, N)
        nn, nr, rt = self.host_view("n_nodes"), self.host_view("n_rows"), self.host_view("root")
        for b, (t, o, i, n_rows, root) in enumerate(flats):
            n = int(t.shape[0])
            if n > N:
                raise ValueError(f"tree {b} has {n} nodes; workspace holds {N}")
            if n and (int(t.min()) < 0 or int(t.max()) > 0x7FFFFFFF):
                raise ValueError("token ids must fit in int32")
            if not 0 <= int(n_rows) <= n:
                raise ValueError(f"tree {b}: {int(n_rows)} decoded rows for {n} nodes")
            check_forest(o, i, n, b)
            tok[b, :n] = t
            off[b, :n + 1] = o
            off[b, n + 1:] = o[-1] if n else 0
            idx[b, :len(i)] = i
            nn[b], nr[b], rt[b] = n, int(n_rows), int(root)
        self.upload()

    def upload(self, stream: Optional[torch.cuda.Stream] = None) -> None:
        with torch.cuda.stream(stream or torch.cuda.current_stream(self.device)):
            self._in_dev.copy_(self._in_host, non_blocking=True)

    def _in_ptr(self, name: str) -> int:
        return self._in_dev.data_ptr() + 4 * self._in_off[name][0]

    def _out_ptr(self, name: str) -> int:
        return self._out_dev.data_ptr() + self._out_off[name][0]

    def dev_view(self, name: str) -> torch.Tensor:
        """Device tensor view of one output array (no copy)."""
        off, cnt, dt = self._out_off[name]
        tdt = {np.dtype(np.int64): torch.int64, np.dtype(np.int32): torch.int32,
               np.dtype(np.float32): torch.float32, np.dtype(np.uint32): torch.int32}[dt]
        return self._out_dev[off:off + cnt * dt.itemsize].view(tdt)

    # -- launch ---------------------------------------------------------------------
    def run(self, logits: torch.Tensor, *, input_kind: int, method: int, gate: int = _lib.GATE_PROB,
            threshold: float = 0.0, window: int = 1, eos: Optional[int] = None, do_sample: bool = False,
            temperature: float = 1.0, top_p: float = 1.0, top_k: int = 0,
            draft_logits: Optional[torch.Tensor] = None, draft_temperature: float = 1.0) -> None:
        """Launch the fused kernel on the current stream.  `logits` is [batch, rows, vocab] on this device.
        With `draft_logits` (same shape and dtype) the sampled exact walk uses residual acceptance."""
        B, N = self.batch, self.max_nodes
        if logits.dim() != 3 or logits.shape[0] != B:
            raise ValueError(f"logits must be [batch={B}, rows, vocab], got {tuple(logits.shape)}")
        if logits.device != self.device:
            raise ValueError("logits live on another device than the workspace")
        if logits.stride(2) != 1:
            logits = logits.contiguous()
        if int(self.host_view("n_rows").max(initial=0)) > int(logits.shape[1]):
            raise ValueError(f"a tree has more decoded rows than logits has rows ({int(logits.shape[1])})")
        a = _lib.VerifyArgs()
        a.struct_size = C.sizeof(_lib.VerifyArgs)
        a.batch, a.max_nodes, a.vocab = B, N, int(logits.shape[2])
        a.dtype = _lib.torch_dtype_code(logits.dtype)
        a.input_kind = int(input_kind)
        a.seq_stride, a.row_stride = int(logits.stride(0)), int(logits.stride(1))
        a.logits = logits.data_ptr()
        for name in ("n_nodes", "n_rows", "token_ids", "child_off", "child_idx", "root"):
            setattr(a, name, self._in_ptr(name))
        a.do_sample = int(do_sample)  # 0 / 1 (every row draws) / 2 (only the contexts the exact walk visits)
        a.top_k = int(top_k)
        a.temperature, a.top_p = float(temperature), float(top_p)
        a.uniforms = self.uniforms.data_ptr()
        if draft_logits is not None:
            if draft_logits.shape != logits.shape or draft_logits.dtype != logits.dtype or \
                    draft_logits.device != self.device:
                raise ValueError("draft_logits must match logits in shape, dtype and device")
            if draft_logits.stride(2) != 1:
                draft_logits = draft_logits.contiguous()
            a.acceptance = 1
            a.draft_logits = draft_logits.data_ptr()
            a.draft_seq_stride, a.draft_row_stride = int(draft_logits.stride(0)), int(draft_logits.stride(1))
            a.draft_temperature = float(draft_temperature)
            a.accept_uniforms = self.accept_uniforms.data_ptr()
            self._keepalive_draft = draft_logits
        a.method, a.gate = int(method), int(gate)
        a.threshold, a.window = float(threshold), int(window)
        a.eos = -1 if eos is None else int(eos)
        a.max_out = self.max_out
        for name in ("out_tokens", "out_hidden", "out_meta", "node_target", "node_entropy", "node_child_prob",
                     "node_rowmax", "node_rowsum", "node_exact_after", "node_best_len", "node_best_next",
                     "dev_status", "out2_tokens", "out2_hidden", "out2_meta"):
            setattr(a, name, self._out_ptr(name))
        a.scratch, a.scratch_bytes = self._scratch_ptr, self._scratch_bytes
        a.flags = _lib.VERIFY_SCRATCH_CLEAN if self.scratch_clean else 0
        self._rows = int(logits.shape[1])
        self._keepalive = logits
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().subspec_verify_batched(C.byref(a), C.c_void_p(stream)), "subspec_verify_batched")

    def run_lm_head(self, hidden: torch.Tensor, weight: torch.Tensor, *, method: int, gate: int = _lib.GATE_PROB,
                    threshold: float = 0.0, window: int = 1, eos: Optional[int] = None) -> None:
        """lm_head and verification in one call (greedy targets): `hidden` [batch, rows, dim] (bf16 or fp16) are the
        target's last hidden states of the tree rows, `weight` [vocab, dim] (same dtype) the lm_head's weight.  Stands
        for `logits = lm_head(hidden)` (generators/classic_sd.py:100-109) followed by `run(logits, ...)`;
        the logits are never written.  Results as `run`'s, up to the rounding of a different GEMM."""
        B, N = self.batch, self.max_nodes
        if hidden.dim() != 3 or hidden.shape[0] != B or weight.dim() != 2 or weight.shape[1] != hidden.shape[2]:
            raise ValueError(f"hidden must be [batch={B}, rows, dim] and weight [vocab, dim], got "
                             f"{tuple(hidden.shape)} and {tuple(weight.shape)}")
        if hidden.dtype not in (torch.bfloat16, torch.float16) or weight.dtype != hidden.dtype:
            raise ValueError("hidden and weight must both be bfloat16 or both float16")
        if hidden.device != self.device or weight.device != self.device:
            raise ValueError("hidden / weight live on another device than the workspace")
        if not hidden.is_contiguous():
            hidden = hidden.contiguous()
        if weight.stride(1) != 1:
            weight = weight.contiguous()
        rows, dim, vocab = int(hidden.shape[1]), int(hidden.shape[2]), int(weight.shape[0])
        if int(self.host_view("n_rows").max(initial=0)) > rows:
            raise ValueError(f"a tree has more decoded rows than hidden has rows ({rows})")
        key = (rows, vocab)
        if getattr(self, "_lm_key", None) != key:
            need = C.c_size_t(0)
            _lib.check(_lib.lib().subspec_lm_head_verify_scratch_bytes(B, N, rows, vocab, C.byref(need)),
                       "subspec_lm_head_verify_scratch_bytes")
            self._lm_scratch = torch.zeros(need.value + 256, dtype=torch.uint8, device=self.device)
            self._lm_key, self._lm_bytes = key, need.value
        la = _lib.LmHeadVerifyArgs()
        la.struct_size = C.sizeof(_lib.LmHeadVerifyArgs)
        la.hidden_dim, la.hidden_seq_rows = dim, rows
        la.hidden, la.hidden_row_stride = hidden.data_ptr(), int(hidden.stride(1))
        la.weight, la.weight_row_stride = weight.data_ptr(), int(weight.stride(0))
        a = la.verify
        a.struct_size = C.sizeof(_lib.VerifyArgs)
        a.batch, a.max_nodes, a.vocab = B, N, vocab
        a.dtype, a.input_kind = _lib.torch_dtype_code(hidden.dtype), _lib.IN_LOGITS
        for name in ("n_nodes", "n_rows", "token_ids", "child_off", "child_idx", "root"):
            setattr(a, name, self._in_ptr(name))
        a.temperature, a.top_p = 1.0, 1.0
        a.method, a.gate = int(method), int(gate)
        a.threshold, a.window = float(threshold), int(window)
        a.eos = -1 if eos is None else int(eos)
        a.max_out = self.max_out
        for name in ("out_tokens", "out_hidden", "out_meta", "node_target", "node_entropy", "node_child_prob",
                     "node_rowmax", "node_rowsum", "node_exact_after", "node_best_len", "node_best_next",
                     "dev_status", "out2_tokens", "out2_hidden", "out2_meta"):
            setattr(a, name, self._out_ptr(name))
        a.scratch, a.scratch_bytes = _align(self._lm_scratch.data_ptr(), 256), self._lm_bytes
        a.flags = _lib.VERIFY_SCRATCH_CLEAN if self.scratch_clean else 0
        self._rows = rows
        self._keepalive = (hidden, weight)
        stream = torch.cuda.current_stream(self.device).cuda_stream
        _lib.check(_lib.lib().subspec_lm_head_verify(C.byref(la), C.c_void_p(stream)), "subspec_lm_head_verify")

    def clear_status(self) -> None:
        self.dev_view("dev_status").zero_()

    # -- outputs --------------------------------------------------------------------
    def fetch(self) -> Dict[str, np.ndarray]:
        """Copy every output to the host (one transfer), synchronise, and return numpy views."""
        self._out_host.copy_(self._out_dev, non_blocking=True)
        torch.cuda.current_stream(self.device).synchronize()
        raw = self._out_host.numpy()
        B, N = self.batch, self.max_nodes
        out: Dict[str, np.ndarray] = {}
        for name, (off, cnt, dt) in self._out_off.items():
            arr = raw[off:off + cnt * dt.itemsize].view(dt)
            if name in ("out_tokens", "out_hidden", "out2_tokens", "out2_hidden"):
                arr = arr.reshape(B, self.max_out)
            elif name in ("out_meta", "out2_meta"):
                arr = arr.reshape(B, 4)
            elif name != "dev_status":
                arr = arr.reshape(B, N)
            out[name] = arr
        status = int(out["dev_status"][0])
        if status:
            self.clear_status()
            self.scratch.zero_()  # a launch that gave up may have left tickets behind
            raise ValueError("verify kernel rejected its input: " + _lib.dev_status_text(status))
        return out


_workspaces: Dict[Tuple[int, int, int], VerifyWorkspace] = {}


def get_workspace(batch: int, n_nodes: int, device: torch.device) -> VerifyWorkspace:
    """Cached workspace, node capacity rounded up to a multiple of 64.

    One workspace per (device, batch, capacity) serves every caller of `verify_tree` / `verify_tree_batched`
    in the process: it is meant for one stream and one host thread at a time, as the reference's generators run
    (calls that overlap on the GPU would share its scratch and output blocks; give those a `VerifyWorkspace`
    of their own through the `workspace` argument)."""
    cap = min(1024, max(64, _align(int(n_nodes), 64)))
    if n_nodes > 1024:
        raise ValueError("trees of more than 1024 nodes are not supported")
    dev = torch.device(device)
    index = dev.index if dev.index is not None else torch.cuda.current_device()  # "cuda" = the current device
    key = (int(index), int(batch), cap)
    ws = _workspaces.get(key)
    if ws is None:
        ws = _workspaces[key] = VerifyWorkspace(batch, cap, device)
    return ws


# ---------------------------------------------------------------------------------
# tree flattening
# ---------------------------------------------------------------------------------
def flatten_tree(tree, skip_nodes: int = 0, limit: Optional[int] = None, restrict: bool = False):
    """(token_ids, child_off, child_idx) in local numbering for any tree with the reference's interface."""
    if hasattr(tree, "flat_children"):
        return tree.flat_children(skip_nodes, limit, restrict)
    s = int(skip_nodes)
    size = int(tree.current_size)
    end = size if limit is None else min(size, s + int(limit))
    n = max((end - s) if restrict else (size - s), 0)
    tok = np.asarray([int(tree.nodes[s + v].token_id) for v in range(n)], dtype=np.int64)
    off = np.zeros(n + 1, dtype=np.int32)
    idx: List[int] = []
    for v in range(n):
        for c in tree.nodes[s + v].children:
            cl = int(c) - s
            if 0 <= cl < n:
                idx.append(cl)
        off[v + 1] = len(idx)
    return tok, off, np.asarray(idx, dtype=np.int32)


def check_forest(child_off: np.ndarray, child_idx: np.ndarray, n: int, which: int = 0) -> None:
    """Raise ValueError unless the children lists (CSR over n nodes) describe a forest: offsets ascending from 0,
    every child index inside [0, n), no node listed as a child twice, no loop.  The kernels bound their walks
    anyway; a malformed tree is refused here so that no launch ever sees one."""
    off = np.asarray(child_off, dtype=np.int64).reshape(-1)
    if off.shape[0] != n + 1 or (n + 1 and off[0] != 0) or np.any(np.diff(off) < 0):
        raise ValueError(f"tree {which}: children offsets must ascend from 0 over {n} nodes")
    m = int(off[-1]) if n + 1 else 0
    idx = np.asarray(child_idx, dtype=np.int64).reshape(-1)
    if m > n or idx.shape[0] < m:
        raise ValueError(f"tree {which}: {m} child entries for {n} nodes")
    if m == 0:
        return
    idx = idx[:m]
    if idx.min() < 0 or idx.max() >= n:
        raise ValueError(f"tree {which}: a child index lies outside [0, {n})")
    if np.bincount(idx, minlength=n).max() > 1:
        raise ValueError(f"tree {which}: a node is listed as a child more than once")
    parent = np.full(n, -1, dtype=np.int64)
    parent[idx] = np.repeat(np.arange(n, dtype=np.int64), np.diff(off))
    if np.all(parent < np.arange(n)):  # children behind their parents, the usual numbering: no loop possible
        return
    up = parent.copy()  # pointer jumping: after ceil(log2 n) + 1 doublings every node of a forest has left it
    for _ in range(max(1, int(n).bit_length()) + 1):
        live = up >= 0
        if not live.any():
            return
        up = np.where(live, up[np.where(live, up, 0)], -1)
    if (up >= 0).any():
        raise ValueError(f"tree {which}: the children lists contain a loop")


def _children_csr(children_lists: Sequence[Sequence[int]]):
    off = np.zeros(len(children_lists) + 1, dtype=np.int32)
    idx: List[int] = []
    for v, ch in enumerate(children_lists):
        idx.extend(int(c) for c in ch)
        off[v + 1] = len(idx)
    return off, np.asarray(idx, dtype=np.int32)


def _sampling_params(logits_processor, do_sample: bool) -> Tuple[float, int, float]:
    """Temperature, top-k and nucleus top-p out of a HF LogitsProcessorList, in the order the reference
    builds it: temperature, top-k, top-p (generators/base.py:42-64).  top_k = 0 means off."""
    temperature, top_k, top_p = 1.0, 0, 1.0
    if not do_sample or not logits_processor:
        return temperature, top_k, top_p
    stage = 0
    for proc in logits_processor:
        kind = type(proc).__name__
        order = {"TemperatureLogitsWarper": 1, "TopKLogitsWarper": 2, "TopPLogitsWarper": 3}.get(kind)
        if order is None:
            raise ValueError(f"logits processor {kind} is not supported by the fused verifier "
                             "(supported: TemperatureLogitsWarper, TopKLogitsWarper, TopPLogitsWarper)")
        if order <= stage:
            raise ValueError("logits processors must come in the order temperature, top-k, top-p, each at most once")
        stage = order
        if order == 1:
            temperature = float(proc.temperature)
        elif order == 2:
            top_k = int(proc.top_k)  # transformers has already folded min_tokens_to_keep into it
            if float(getattr(proc, "filter_value", -float("inf"))) != -float("inf"):
                raise ValueError("TopKLogitsWarper.filter_value other than -inf is not supported")
        else:
            top_p = float(proc.top_p)
            if int(getattr(proc, "min_tokens_to_keep", 1)) != 1:
                raise ValueError("TopPLogitsWarper.min_tokens_to_keep != 1 is not supported")
    return temperature, top_k, top_p


def _method_code(verify_method) -> int:
    m = str(verify_method or "exact").strip().lower()
    if m in ("exact", "greedy", "stochastic"):
        return _lib.VERIFY_EXACT
    if m == "lossy":
        return _lib.VERIFY_LOSSY
    if m in ("exact+lossy", "greedy+lossy"):
        return _lib.VERIFY_EXACT_AND_LOSSY
    raise ValueError(f"Unsupported verify_method: {verify_method!r} (supported: 'exact', 'lossy')")


def _gate_code(threshold_method) -> int:
    g = str(threshold_method or "entropy").strip().lower()
    if g == "entropy":
        return _lib.GATE_ENTROPY
    if g == "prob":
        return _lib.GATE_PROB
    raise ValueError(f"Unsupported threshold_method: {threshold_method!r} (supported: 'entropy', 'prob')")


# ---------------------------------------------------------------------------------
# diagnostics of the lossy verifier (host side, from the kernel's per-node outputs)
# ---------------------------------------------------------------------------------
def _welford_push(key: str, x: float) -> None:
    st = wandb_logger.internal_data.get(key) or {"n": 0, "mean": 0.0, "M2": 0.0}
    n = int(st["n"]) + 1
    d = x - float(st["mean"])
    mean = float(st["mean"]) + d / n
    wandb_logger.internal_data[key] = {"n": n, "mean": mean, "M2": float(st["M2"]) + d * (x - mean)}


def _welford_read(key: str) -> Tuple[float, float]:
    st = wandb_logger.internal_data.get(key)
    if not st or int(st.get("n", 0)) <= 0:
        return 0.0, 0.0
    return float(st["mean"]), math.sqrt(max(float(st["M2"]) / int(st["n"]), 0.0))


def log_lossy_diagnostics(*, token_ids, child_off, child_idx, target, entropy, child_prob, exact_after,
                          best_next, hidden, n_out: int, accept_len: int, use_entropy: bool,
                          threshold: float, window: int) -> None:
    """Reproduce the reference's `wandb_logger` side effects (lossy_tree_verify.py:171-194, 249-337)."""
    need = max(0, int(window))

    def kids(u: int):
        return child_idx[child_off[u]:child_off[u + 1]]

    def mismatch(u: int) -> bool:
        ch = kids(u)
        return len(ch) > 0 and all(int(token_ids[c]) != int(target[u]) for c in ch)

    def window_ok_gate(u: int) -> Optional[float]:
        if not mismatch(u):
            return None
        ok = [int(c) for c in kids(u) if int(exact_after[c]) >= need]
        if not ok:
            return None
        return float(entropy[u]) if use_entropy else max(float(child_prob[c]) for c in ok)

    def blocks(v: float) -> bool:
        return v >= threshold if use_entropy else v < threshold

    mm = elig = drop = mm_acc = mm_acc_nomatch = 0
    visited = [int(hidden[i]) for i in range(accept_len)]
    if n_out > accept_len:
        visited.append(int(hidden[n_out - 1]))
    for step, ctx in enumerate(visited):
        if mismatch(ctx):
            mm += 1
            g = window_ok_gate(ctx)
            if g is not None:
                elig += 1
                _welford_push("lossy/window_ok_gate", g)
                if blocks(g):
                    drop += 1
                    _welford_push("lossy/window_ok_drop_gate", g)
        if step < accept_len:
            nxt = int(best_next[ctx])
            if int(token_ids[nxt]) != int(target[ctx]):
                mm_acc += 1
                p = float(child_prob[nxt])
                _welford_push("verify/mm_acc_p", p)
                _welford_push("lossy/accept_gate", float(entropy[ctx]) if use_entropy else p)
                if mismatch(ctx):
                    mm_acc_nomatch += 1

    store = wandb_logger.internal_data
    for key, val in (("lossy/accept_tokens", accept_len), ("lossy/mm_ctx", mm), ("lossy/mm_elig_ctx", elig),
                     ("lossy/mm_drop_ctx", drop), ("lossy/mm_acc_steps", mm_acc),
                     ("lossy/mm_acc_nomatch_steps", mm_acc_nomatch)):
        store[key] = float(store.get(key, 0.0)) + float(val)
    acc_tokens = float(store["lossy/accept_tokens"])
    mm_acc_total = float(store["lossy/mm_acc_steps"])
    log = wandb_logger.log_data
    log["verify_accept_tokens"] = acc_tokens
    log["verify_lossy_accept_tokens"] = mm_acc_total
    log["verify_lossy_accept_rate"] = mm_acc_total / acc_tokens if acc_tokens > 0 else 0.0
    e, d = float(store["lossy/mm_elig_ctx"]), float(store["lossy/mm_drop_ctx"])
    log["lossy_window_ok_drop_rate"] = d / e if e > 0 else 0.0
    m, nm = float(store["lossy/mm_ctx"]), float(store["lossy/mm_acc_nomatch_steps"])
    log["lossy_accept_rate_when_no_match"] = nm / m if m > 0 else 0.0
    log["lossy_window_ok_gate_mean"], log["lossy_window_ok_gate_std"] = _welford_read("lossy/window_ok_gate")
    log["lossy_window_ok_drop_gate_mean"], log["lossy_window_ok_drop_gate_std"] = _welford_read(
        "lossy/window_ok_drop_gate")
    log["lossy_threshold_method"] = "entropy" if use_entropy else "prob"
    log["lossy_accepted_prob_mean"], log["lossy_accepted_prob_std"] = _welford_read("verify/mm_acc_p")
    log["lossy_accepted_gate_mean"], log["lossy_accepted_gate_std"] = _welford_read("lossy/accept_gate")


# ---------------------------------------------------------------------------------
# public API
# ---------------------------------------------------------------------------------
@dataclass
class VerifyOutput:
    """Per-sequence result of a batched verify."""

    sampled_tokens: torch.Tensor  # [1, L] int64 (CPU)
    hidden_indices: torch.Tensor  # [L] int64 (CPU), original tree indexing
    total_len: int
    accept_len: int

    def as_tuple(self):
        return self.sampled_tokens, self.hidden_indices, (self.total_len, self.accept_len)


def _run_single_flat(*, values: torch.Tensor, input_kind: int, tok, off, idx, n_rows: int, root: int,
                     method: int, gate: int, threshold: float, window: int, eos, do_sample: bool,
                     temperature: float, top_p: float, uniforms=None):
    device = _device_of(values)
    values = values.to(device)
    if values.dim() == 2:
        values = values.unsqueeze(0)
    ws = get_workspace(1, max(len(tok), 1), device)
    ws.set_trees([(tok, off, idx, n_rows, root)])
    if do_sample:
        if uniforms is None:
            ws.uniforms.uniform_()
        else:
            u = torch.as_tensor(uniforms, dtype=torch.float32).reshape(-1)
            ws.uniforms[:u.numel()].copy_(u.to(device))
    ws.run(values, input_kind=input_kind, method=method, gate=gate, threshold=threshold, window=window, eos=eos,
           do_sample=do_sample, temperature=temperature, top_p=top_p)
    return ws.fetch()


@torch.no_grad()
def lossy_bottom_up_verify(*, probs: torch.Tensor, token_ids: torch.Tensor, parent_indices: torch.Tensor,
                           children_lists: Sequence[Sequence[int]], root_index: int, eos_token_id: Optional[int],
                           do_sample: bool, threshold: float, window_size: int, threshold_method: str = "prob",
                           uniforms=None) -> Tuple[torch.Tensor, torch.Tensor, int]:
    """Lossy bottom-up verification over a tree chunk given target PROBABILITIES [N, V].

    Same contract as the reference (lossy_tree_verify.py:9-343), including the
    `wandb_logger` diagnostics.  `parent_indices` is accepted for signature
    compatibility; like the reference, the structure is taken from `children_lists`.
    With do_sample the target token of each node is the inverse-CDF pick for
    `uniforms[u]` (fresh uniforms are drawn on the device when not given).
    """
    gate = _gate_code(threshold_method if threshold_method else "entropy")
    tok = np.asarray(token_ids.detach().cpu().numpy() if isinstance(token_ids, torch.Tensor) else token_ids,
                     dtype=np.int64).reshape(-1)
    n = int(probs.shape[0])
    off, idx = _children_csr(list(children_lists)[:n])
    out = _run_single_flat(values=probs, input_kind=_lib.IN_PROBS, tok=tok[:n], off=off, idx=idx, n_rows=n,
                           root=int(root_index), method=_lib.VERIFY_LOSSY, gate=gate, threshold=float(threshold),
                           window=max(0, int(window_size)), eos=eos_token_id, do_sample=do_sample,
                           temperature=1.0, top_p=1.0, uniforms=uniforms)
    L, acc = int(out["out_meta"][0, 0]), int(out["out_meta"][0, 1])
    hidden = out["out_hidden"][0, :L]
    log_lossy_diagnostics(token_ids=tok, child_off=off, child_idx=idx, target=out["node_target"][0],
                          entropy=out["node_entropy"][0], child_prob=out["node_child_prob"][0],
                          exact_after=out["node_exact_after"][0], best_next=out["node_best_next"][0],
                          hidden=hidden, n_out=L, accept_len=acc, use_entropy=gate == _lib.GATE_ENTROPY,
                          threshold=float(threshold), window=int(window_size))
    return (torch.from_numpy(out["out_tokens"][0, :L].copy()), torch.from_numpy(hidden.copy()), acc)


def _prepare_tree(tree, root_ind: int, skip_nodes: int, rows: int, method: int):
    skip = int(skip_nodes)
    if method == _lib.VERIFY_EXACT_AND_LOSSY:
        # one flattening has to serve both walks: that is the case when every node is decoded
        tok, off, idx = flatten_tree(tree, skip, restrict=False)
        root = int(root_ind) - skip
        if len(tok) > rows or not 0 <= root < len(tok):
            raise ValueError("verify_method='exact+lossy' needs logits for every tree node and a root inside them")
        return tok, off, idx, len(tok), root
    if method == _lib.VERIFY_LOSSY:
        tok, off, idx = flatten_tree(tree, skip, limit=rows, restrict=True)
        n_rows = len(tok)
        root = int(root_ind) - skip
        if root < 0 or root >= n_rows:
            root = 0  # tree_verify.py:133-135
    else:
        tok, off, idx = flatten_tree(tree, skip, restrict=False)
        n_rows = min(rows, len(tok))
        root = int(root_ind) - skip
    return tok, off, idx, n_rows, root


@torch.no_grad()
def verify_tree_batched(*, trees: Sequence[Any], root_inds: Sequence[int], logits: Optional[torch.Tensor] = None,
                        eos_token_id: Optional[int], logits_processor=None, do_sample: bool = False,
                        skip_nodes=0, verify_method: str = "exact", verify_kwargs: Optional[dict] = None,
                        uniforms: Optional[torch.Tensor] = None, workspace: Optional[VerifyWorkspace] = None,
                        log_diagnostics: bool = False, draft_logits: Optional[torch.Tensor] = None,
                        accept_uniforms: Optional[torch.Tensor] = None,
                        hidden_states: Optional[torch.Tensor] = None,
                        lm_head_weight: Optional[torch.Tensor] = None) -> List[VerifyOutput]:
    """Verify `len(trees)` independent draft trees against `logits` [batch, rows, vocab] in one launch.

    Instead of `logits`, `hidden_states` [batch, rows, dim] and `lm_head_weight` [vocab, dim] (both bf16 or fp16) may be
    given (greedy targets only): the lm_head product and the verification then run as one call that never
    writes the logits (`VerifyWorkspace.run_lm_head`).

    Per sequence the result equals the reference's `verify_tree` on
    `logits[b:b+1]` (tree_verify.py:7-163).  `verify_method="exact+lossy"` returns, per sequence, the pair
    (exact result, lossy result) of the two calls a step that verifies greedily and then lossily makes, from
    one pass over the logits; it needs logits for every tree node.

    `verify_kwargs={"acceptance": "residual", "draft_temperature": T}` with `draft_logits` [batch, rows, vocab]
    (an extension, not in the reference): sampled verification accepts child c of a context with probability
    min(1, p'(x_c) / q(x_c)) in list order, p' being the filtered target distribution from which q is
    subtracted (and the rest renormalised) after every rejection; the bonus token is drawn from p'.
    `accept_uniforms` [batch, nodes] are the uniforms of the accept tests, `uniforms` those of the draws.
    """
    method = _method_code(verify_method)
    vk = dict(verify_kwargs or {})
    B = len(trees)
    fused = hidden_states is not None
    if fused:
        if logits is not None or lm_head_weight is None:
            raise ValueError("give either logits, or hidden_states together with lm_head_weight")
        if do_sample:
            raise ValueError("hidden_states / lm_head_weight: greedy targets only (sampling needs the whole row)")
        if hidden_states.dim() != 3 or hidden_states.shape[0] != B:
            raise ValueError(f"hidden_states must be [batch={B}, rows, dim]")
        device = _device_of(hidden_states)
        hidden_states, lm_head_weight = hidden_states.to(device), lm_head_weight.to(device)
        rows = int(hidden_states.shape[1])
    else:
        if logits is None or logits.dim() != 3 or logits.shape[0] != B:
            raise ValueError(f"logits must be [batch={B}, rows, vocab]")
        device = _device_of(logits)
        logits = logits.to(device)
        rows = int(logits.shape[1])
    skips = [int(skip_nodes)] * B if isinstance(skip_nodes, int) else [int(s) for s in skip_nodes]
    flats = [_prepare_tree(t, r, s, rows, method) for t, r, s in zip(trees, root_inds, skips)]
    gate, threshold, window = _lib.GATE_PROB, 0.0, 1
    if method != _lib.VERIFY_EXACT:
        gate = _gate_code(vk.get("threshold_method", "prob") or "prob")
        threshold = float(vk.get("threshold", 0.0))
        window = max(0, int(vk.get("window_size", 1)))
    temperature, top_k, top_p = _sampling_params(logits_processor, do_sample)
    n_max = max(max(len(f[0]) for f in flats), 1)
    ws = workspace or get_workspace(B, n_max, device)
    ws.set_trees(flats)
    if do_sample:
        if uniforms is None:
            ws.uniforms.uniform_()
        else:
            u = torch.as_tensor(uniforms, dtype=torch.float32, device=device)
            ws.uniforms.view(B, ws.max_nodes)[:, :u.shape[1]].copy_(u)
    # Sampled targets: the exact walk only needs them at the contexts it visits (mode 2); the lossy DP, and a
    # caller who asks for every node's draw (`verify_kwargs={"sample_all_nodes": True}`), need all rows (mode 1).
    sample_mode = 0
    if do_sample:
        sample_mode = 2 if (method == _lib.VERIFY_EXACT and not vk.get("sample_all_nodes", False)) else 1
    acceptance = str(vk.get("acceptance", "match") or "match").strip().lower()
    if acceptance not in ("match", "residual"):
        raise ValueError(f"Unsupported acceptance: {acceptance!r} (supported: 'match', 'residual')")
    if acceptance == "residual":
        if not do_sample or method != _lib.VERIFY_EXACT or draft_logits is None:
            raise ValueError("residual acceptance needs do_sample=True, the exact/stochastic method and draft_logits")
        draft_logits = draft_logits.to(device)
        if accept_uniforms is None:
            ws.accept_uniforms.uniform_()
        else:
            au = torch.as_tensor(accept_uniforms, dtype=torch.float32, device=device)
            ws.accept_uniforms.view(B, ws.max_nodes)[:, :au.shape[1]].copy_(au)
    else:
        draft_logits = None
    if fused:
        ws.run_lm_head(hidden_states, lm_head_weight, method=method, gate=gate, threshold=threshold, window=window,
                       eos=eos_token_id)
    else:
        ws.run(logits, input_kind=_lib.IN_LOGITS, method=method, gate=gate, threshold=threshold, window=window,
               eos=eos_token_id, do_sample=sample_mode, temperature=temperature, top_p=top_p, top_k=top_k,
               draft_logits=draft_logits, draft_temperature=float(vk.get("draft_temperature", 1.0)))
    out = ws.fetch()
    results: List[Any] = []
    for b in range(B):
        L, acc, total = (int(x) for x in out["out_meta"][b, :3])
        hidden_local = out["out_hidden"][b, :L]
        if log_diagnostics and method != _lib.VERIFY_EXACT:
            tok, off, idx = flats[b][:3]
            log_lossy_diagnostics(token_ids=tok, child_off=off, child_idx=idx, target=out["node_target"][b],
                                  entropy=out["node_entropy"][b], child_prob=out["node_child_prob"][b],
                                  exact_after=out["node_exact_after"][b], best_next=out["node_best_next"][b],
                                  hidden=hidden_local, n_out=L, accept_len=acc,
                                  use_entropy=gate == _lib.GATE_ENTROPY, threshold=threshold, window=window)
        res = VerifyOutput(
            sampled_tokens=torch.from_numpy(out["out_tokens"][b, :L].copy()).unsqueeze(0),
            hidden_indices=torch.from_numpy(hidden_local + skips[b]),
            total_len=total, accept_len=acc)
        if method == _lib.VERIFY_EXACT_AND_LOSSY:  # (exact result, lossy result)
            L2, acc2, total2 = (int(x) for x in out["out2_meta"][b, :3])
            res = (VerifyOutput(
                sampled_tokens=torch.from_numpy(out["out2_tokens"][b, :L2].copy()).unsqueeze(0),
                hidden_indices=torch.from_numpy(out["out2_hidden"][b, :L2] + skips[b]),
                total_len=total2, accept_len=acc2), res)
        results.append(res)
    return results


@torch.no_grad()
def verify_tree(*, tree, root_ind: int, logits: Optional[torch.Tensor] = None, sample_token_fn=None,
                verify_step_fn=None, eos_token_id: Optional[int], logits_processor=None, do_sample: bool = False,
                skip_nodes: int = 0, verify_method: str = "exact", verify_kwargs: Optional[dict] = None,
                uniforms: Optional[torch.Tensor] = None, draft_logits: Optional[torch.Tensor] = None,
                accept_uniforms: Optional[torch.Tensor] = None, hidden_states: Optional[torch.Tensor] = None,
                lm_head_weight: Optional[torch.Tensor] = None):
    """Drop-in for the reference's `verify_tree` (tree_verify.py:7-163).

    `sample_token_fn` and `verify_step_fn` are accepted so call sites need not
    change, but are not called: softmax, target-token choice, child matching,
    the accept walk and the lossy DP all happen inside the fused kernel.  With
    `do_sample=True` the per-node draw is the inverse-CDF pick for `uniforms[u]`
    (drawn on the device when not supplied) instead of `torch.multinomial`.
    `draft_logits` [rows, vocab] and `accept_uniforms` [nodes] serve
    `verify_kwargs={"acceptance": "residual"}` (see `verify_tree_batched`).
    `hidden_states` [1, rows, dim] with `lm_head_weight` [vocab, dim] instead of `logits` (greedy targets): the
    lm_head product is part of the call and the logits are never written.
    """
    if hidden_states is not None and hidden_states.dim() == 2:
        hidden_states = hidden_states.unsqueeze(0)
    if draft_logits is not None and draft_logits.dim() == 2:
        draft_logits = draft_logits.unsqueeze(0)
    if accept_uniforms is not None:
        accept_uniforms = torch.as_tensor(accept_uniforms).reshape(1, -1)
    res = verify_tree_batched(trees=[tree], root_inds=[int(root_ind)], logits=logits, eos_token_id=eos_token_id,
                              logits_processor=logits_processor, do_sample=do_sample, skip_nodes=int(skip_nodes),
                              verify_method=verify_method, verify_kwargs=verify_kwargs,
                              uniforms=None if uniforms is None else torch.as_tensor(uniforms).reshape(1, -1),
                              log_diagnostics=True, draft_logits=draft_logits, accept_uniforms=accept_uniforms,
                              hidden_states=hidden_states, lm_head_weight=lm_head_weight)
    return res[0].as_tuple()
