"""ctypes binding of `libsubspec_b200.so` (declared in include/subspec_b200.h).

There is no CPU fallback: if the CUDA library has not been built, importing a
compute entry point raises.  Build it with `python -m subspec_b200.build`.
"""
from __future__ import annotations

import ctypes as C
from pathlib import Path

_LIB_PATH = Path(__file__).resolve().parent / "lib" / "libsubspec_b200.so"

OK, EINVAL, EUNSUPPORTED, ECUDA, ESCRATCH, ETOOLARGE = 0, -1, -2, -3, -4, -5
STATIC_SCRATCH_MAX_ROWS = 4096
F32, BF16, F16 = 0, 1, 2
IN_LOGITS, IN_PROBS = 0, 1
VERIFY_EXACT, VERIFY_LOSSY, VERIFY_EXACT_AND_LOSSY = 0, 1, 2
VERIFY_SCRATCH_CLEAN = 1  # SUBSPEC_VERIFY_SCRATCH_CLEAN
EXPAND_SCRATCH_CLEAN = 1  # SUBSPEC_EXPAND_SCRATCH_CLEAN
GATE_PROB, GATE_ENTROPY = 0, 1
DEV_BAD_TOKEN, DEV_BAD_CHILD, DEV_BAD_ROOT, DEV_BAD_PAGE, DEV_BAD_INDEX, DEV_TIMEOUT, DEV_HIST_OVERFLOW = 1, 2, 4, 8, 16, 32, 64
DEV_BAD_PARENT, DEV_BAD_COUNT = 128, 256
MASK_BOOL, MASK_ADD_F32, MASK_ADD_BF16, MASK_ADD_F16 = 0, 1, 2, 3

_STATUS_TEXT = {
    EINVAL: "invalid argument",
    EUNSUPPORTED: "unsupported shape",
    ECUDA: "CUDA error",
    ESCRATCH: "scratch buffer too small or misaligned",
    ETOOLARGE: "batch * max_nodes exceeds the built-in scratch of the no-allocation entry point (4096 rows)",
}

_DEV_TEXT = {
    DEV_BAD_TOKEN: "draft token id outside [0, vocab)",
    DEV_BAD_CHILD: "child index outside the tree",
    DEV_BAD_ROOT: "root index outside the decoded rows",
    DEV_BAD_PAGE: "page id outside the pool",
    DEV_BAD_INDEX: "accepted-path index out of range",
    DEV_TIMEOUT: "a bounded device-side wait ran out",
    DEV_HIST_OVERFLOW: "sampling: one finite logit value occurs more than 65535 times in a row",
    DEV_BAD_PARENT: "a parent index was not smaller than the node's own",
    DEV_BAD_COUNT: "a node / row count or a children offset was out of range",
}

_vp, _i32, _i64, _u32, _f32, _f64 = C.c_void_p, C.c_int32, C.c_int64, C.c_uint32, C.c_float, C.c_double


class VerifyArgs(C.Structure):
    """Mirror of `subspec_verify_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("max_nodes", _i32), ("vocab", _i32), ("dtype", _i32),
        ("input_kind", _i32), ("seq_stride", _i64), ("row_stride", _i64), ("logits", _vp),
        ("n_nodes", _vp), ("n_rows", _vp), ("token_ids", _vp), ("child_off", _vp), ("child_idx", _vp),
        ("root", _vp),
        ("do_sample", _i32), ("top_k", _i32), ("temperature", _f64), ("top_p", _f64), ("uniforms", _vp),
        ("method", _i32), ("gate", _i32), ("threshold", _f64), ("window", _i32), ("eos", _i64),
        ("max_out", _i32), ("out_tokens", _vp), ("out_hidden", _vp), ("out_meta", _vp),
        ("node_target", _vp), ("node_entropy", _vp), ("node_child_prob", _vp), ("node_rowmax", _vp),
        ("node_rowsum", _vp), ("node_exact_after", _vp), ("node_best_len", _vp), ("node_best_next", _vp),
        ("dev_status", _vp), ("scratch", _vp), ("scratch_bytes", C.c_size_t),
        ("out2_tokens", _vp), ("out2_hidden", _vp), ("out2_meta", _vp),
        ("acceptance", _i32), ("draft_logits", _vp), ("draft_seq_stride", _i64), ("draft_row_stride", _i64),
        ("draft_temperature", _f64), ("accept_uniforms", _vp), ("flags", _u32),
    ]


class LmHeadVerifyArgs(C.Structure):
    """Mirror of `subspec_lm_head_verify_args`."""

    _fields_ = [
        ("struct_size", _u32), ("hidden_dim", _i32), ("hidden", _vp), ("hidden_row_stride", _i64),
        ("weight", _vp), ("weight_row_stride", _i64), ("hidden_seq_rows", _i32), ("reserved", _i32),
        ("verify", VerifyArgs),
    ]


class KvPagedArgs(C.Structure):
    """Mirror of `subspec_kv_paged_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("layers", _i32), ("num_pages", _i32), ("page_len", _i32),
        ("heads", _i32), ("head_dim", _i32), ("elem_bytes", _i32), ("pool", _vp), ("page_table", _vp),
        ("pages_per_seq", _i32), ("offset", _vp), ("n", _vp), ("beam", _vp), ("max_beam", _i32),
        ("n_stride", _i32), ("dev_status", _vp),
    ]


class KvHfArgs(C.Structure):
    """Mirror of `subspec_kv_hf_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("num_tensors", _i32), ("heads", _i32), ("tokens", _i32),
        ("head_dim", _i32), ("elem_bytes", _i32), ("batch_stride", _i64), ("head_stride", _i64),
        ("token_stride", _i64), ("layer_ptrs", _vp), ("offset", _vp), ("n", _vp), ("beam", _vp),
        ("max_beam", _i32), ("n_stride", _i32), ("dev_status", _vp),
    ]


class ExpandArgs(C.Structure):
    """Mirror of `subspec_expand_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("leaves", _i32), ("vocab", _i32), ("k", _i32), ("dtype", _i32),
        ("input_kind", _i32), ("seq_stride", _i64), ("row_stride", _i64), ("scores", _vp), ("parent_probs", _vp),
        ("temperature", _f64), ("out_tokens", _vp), ("out_probs", _vp), ("out_parents", _vp), ("level", _i32),
        ("tree_stride", _i32), ("tree_tokens", _vp), ("tree_parents", _vp), ("tree_probs", _vp),
        ("tree_depths", _vp), ("scratch", _vp), ("scratch_bytes", C.c_size_t), ("dev_status", _vp),
        ("draft_mask", _vp), ("draft_mask_kind", _i32), ("draft_mask_cols", _i64), ("draft_mask_row_stride", _i64),
        ("draft_mask_seq_stride", _i64), ("prefix_len", _vp), ("draft_position_ids", _vp),
        ("flags", _u32), ("reserved", _u32),
    ]


class TreeFinalizeArgs(C.Structure):
    """Mirror of `subspec_tree_finalize_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("n_nodes", _i32), ("tree_stride", _i32), ("keep", _i32),
        ("tree_tokens", _vp), ("tree_parents", _vp), ("tree_probs", _vp), ("tree_depths", _vp),
        ("position_offset", _vp), ("keep_idx", _vp), ("tokens", _vp), ("parents", _vp), ("depths", _vp),
        ("probs", _vp), ("position_ids", _vp), ("mask", _vp), ("child_off", _vp), ("child_idx", _vp),
        ("n_out", _vp), ("dev_status", _vp), ("prefix_length", _vp), ("skip_nodes", _i32), ("mask_kind", _i32),
        ("mask_cols", _i64), ("mask_row_stride", _i64), ("mask_seq_stride", _i64),
    ]


class W4A16Args(C.Structure):
    """Mirror of `subspec_w4a16_args`."""

    _fields_ = [
        ("struct_size", _u32), ("m", _i32), ("n", _i32), ("k", _i32), ("x", _vp), ("x_stride", _i64),
        ("packed", _vp), ("y", _vp), ("y_stride", _i64), ("scratch", _vp), ("scratch_bytes", C.c_size_t),
        ("dev_status", _vp),
    ]


class PostVerifyArgs(C.Structure):
    """Mirror of `subspec_post_verify_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("max_nodes", _i32), ("max_out", _i32), ("n_nodes", _vp),
        ("token_ids", _vp), ("child_off", _vp), ("child_idx", _vp), ("out_tokens", _vp), ("out_hidden", _vp),
        ("out_meta", _vp), ("skip_nodes", _vp), ("finished", _vp), ("next_root", _vp), ("accepted", _vp),
        ("beam_cache", _vp), ("beam_stride", _i32), ("beam_len", _vp), ("reorder_n", _vp), ("reorder_offset", _vp),
        ("kv_len", _vp), ("dev_status", _vp),
    ]


class TreePruneDepthArgs(C.Structure):
    """Mirror of `subspec_tree_prune_depth_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("tree_stride", _i32), ("n_nodes", _vp), ("max_depth", _vp),
        ("tokens", _vp), ("parents", _vp), ("depths", _vp), ("probs", _vp), ("keep_idx", _vp), ("n_out", _vp),
        ("child_off", _vp), ("child_idx", _vp), ("dev_status", _vp),
    ]


PAGES_PREFILL, PAGES_DECODE, PAGES_TREE = 0, 1, 2


class PagesArgs(C.Structure):
    """Mirror of `subspec_pages_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("num_pages", _i32), ("page_len", _i32), ("pages_per_seq", _i32),
        ("free_mask", _vp), ("page_table", _vp), ("n_pages", _vp), ("kv_len", _vp), ("kv_last_page_len", _vp),
        ("set_len", _vp), ("add_len", _vp), ("add_all", _i32), ("mode", _i32), ("tree_tokens", _i32),
        ("max_append", _i32), ("seq_indptr", _vp), ("kv_page_indptr", _vp), ("kv_page_indices", _vp),
        ("batch_indices", _vp), ("positions", _vp), ("dev_status", _vp),
    ]


class TreeAttnArgs(C.Structure):
    """Mirror of `subspec_tree_attn_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("q_len", _i32), ("num_q_heads", _i32), ("num_kv_heads", _i32),
        ("head_dim", _i32), ("layer", _i32), ("layers", _i32), ("num_pages", _i32), ("page_len", _i32),
        ("pages_per_seq", _i32), ("pool", _vp), ("page_table", _vp), ("kv_len", _vp), ("n_q", _vp),
        ("prefix_len", _vp), ("mask", _vp), ("mask_batch_stride", _i64), ("mask_row_stride", _i64), ("q", _vp),
        ("q_batch_stride", _i64), ("q_token_stride", _i64), ("q_head_stride", _i64), ("out", _vp),
        ("o_batch_stride", _i64), ("o_token_stride", _i64), ("o_head_stride", _i64), ("sm_scale", _f64),
        ("dev_status", _vp), ("dtype", _i32), ("mask_kind", _i32), ("v_cache", _vp),
        ("kv_batch_stride", _i64), ("kv_head_stride", _i64), ("kv_row_stride", _i64),
        ("kv_splits", _i32), ("reserved", _i32), ("split_scratch", _vp),
    ]


class KvAppendArgs(C.Structure):
    """Mirror of `subspec_kv_append_args`."""

    _fields_ = [
        ("struct_size", _u32), ("batch", _i32), ("q_len", _i32), ("num_kv_heads", _i32), ("head_dim", _i32),
        ("layer", _i32), ("layers", _i32), ("num_pages", _i32), ("page_len", _i32), ("pages_per_seq", _i32),
        ("pool", _vp), ("page_table", _vp), ("kv_len", _vp), ("n_q", _vp), ("k", _vp), ("v", _vp),
        ("batch_stride", _i64), ("token_stride", _i64), ("dev_status", _vp),
    ]


W4A16_MAX_GROUP = 4


class W4A16GroupArgs(C.Structure):
    """Mirror of `subspec_w4a16_group_args`."""

    _fields_ = [
        ("struct_size", _u32), ("m", _i32), ("k", _i32), ("count", _i32), ("x", _vp), ("x_stride", _i64),
        ("packed", _vp * W4A16_MAX_GROUP), ("n", _i32 * W4A16_MAX_GROUP), ("y", _vp * W4A16_MAX_GROUP),
        ("y_stride", _i64 * W4A16_MAX_GROUP), ("scratch", _vp), ("scratch_bytes", C.c_size_t), ("dev_status", _vp),
    ]


# every symbol include/subspec_b200.h declares: name -> (restype, argtypes)
SYMBOLS = {
    "subspec_version": (C.c_char_p, []),
    "subspec_last_cuda_error": (C.c_char_p, []),
    "subspec_verify_scratch_bytes": (C.c_int, [_i32, _i32, C.POINTER(C.c_size_t)]),
    "subspec_verify_batched": (C.c_int, [C.POINTER(VerifyArgs), _vp]),
    "subspec_verify_batched_static_scratch": (C.c_int, [C.POINTER(VerifyArgs), _vp]),
    "subspec_lm_head_verify_scratch_bytes": (C.c_int, [_i32, _i32, _i32, _i32, C.POINTER(C.c_size_t)]),
    "subspec_lm_head_verify": (C.c_int, [C.POINTER(LmHeadVerifyArgs), _vp]),
    "subspec_kv_compact_paged": (C.c_int, [C.POINTER(KvPagedArgs), _vp]),
    "subspec_kv_compact_hf": (C.c_int, [C.POINTER(KvHfArgs), _vp]),
    "subspec_expand_scratch_bytes": (C.c_int, [_i32, _i32, _i32, C.POINTER(C.c_size_t)]),
    "subspec_expand_step": (C.c_int, [C.POINTER(ExpandArgs), _vp]),
    "subspec_tree_finalize": (C.c_int, [C.POINTER(TreeFinalizeArgs), _vp]),
    "subspec_post_verify": (C.c_int, [C.POINTER(PostVerifyArgs), _vp]),
    "subspec_pages_update": (C.c_int, [C.POINTER(PagesArgs), _vp]),
    "subspec_tree_attention_paged": (C.c_int, [C.POINTER(TreeAttnArgs), _vp]),
    "subspec_kv_append_paged": (C.c_int, [C.POINTER(KvAppendArgs), _vp]),
    "subspec_tree_prune_depth": (C.c_int, [C.POINTER(TreePruneDepthArgs), _vp]),
    "subspec_w4a16_packed_bytes": (C.c_int, [_i32, _i32, C.POINTER(C.c_size_t)]),
    "subspec_w4a16_pack": (C.c_int, [_vp, _vp, _vp, _vp, _i32, _i32, _vp]),
    "subspec_w4a16_scratch_bytes": (C.c_int, [_i32, _i32, _i32, C.POINTER(C.c_size_t)]),
    "subspec_w4a16_gemm": (C.c_int, [C.POINTER(W4A16Args), _vp]),
    "subspec_w4a16_gemm_grouped": (C.c_int, [C.POINTER(W4A16GroupArgs), _vp]),
}

_lib = None


class SubspecError(RuntimeError):
    pass


def lib_path() -> Path:
    return _LIB_PATH


def lib() -> C.CDLL:
    """Load the CUDA library (once).  Raises if it has not been built."""
    global _lib
    if _lib is None:
        if not _LIB_PATH.exists():
            raise SubspecError(
                f"{_LIB_PATH} is missing: build the sm_100a kernels with `python -m subspec_b200.build`. "
                "subspec_b200 has no CPU or PyTorch fallback."
            )
        handle = C.CDLL(str(_LIB_PATH))
        for name, (res, args) in SYMBOLS.items():
            fn = getattr(handle, name)
            fn.restype = res
            fn.argtypes = args
        _lib = handle
    return _lib


def check(rc: int, what: str) -> None:
    if rc == OK:
        return
    msg = _STATUS_TEXT.get(rc, f"status {rc}")
    if rc == ECUDA:
        msg += ": " + lib().subspec_last_cuda_error().decode()
    if rc in (EINVAL, EUNSUPPORTED, ESCRATCH, ETOOLARGE):
        raise ValueError(f"{what}: {msg}")
    raise SubspecError(f"{what}: {msg}")


def dev_status_text(word: int) -> str:
    return "; ".join(t for bit, t in _DEV_TEXT.items() if word & bit)


def torch_dtype_code(dtype) -> int:
    import torch

    if dtype == torch.float32:
        return F32
    if dtype == torch.bfloat16:
        return BF16
    if dtype == torch.float16:
        return F16
    raise ValueError(f"unsupported dtype {dtype}: expected float32, bfloat16 or float16")
