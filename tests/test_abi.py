"""The C-ABI library builds for sm_100a, loads, and exports every symbol the header declares (no GPU needed)."""
import ctypes as C
import re
from pathlib import Path

from subspec_b200 import _lib

HEADER = Path(__file__).resolve().parent.parent / "include" / "subspec_b200.h"


def _declared():
    text = HEADER.read_text()
    return set(re.findall(r"SUBSPEC_API\s+[\w\s\*]+?\b(subspec_\w+)\s*\(", text))


def test_header_symbols_are_exported(cuda_lib):
    declared = _declared()
    assert declared, "no SUBSPEC_API declarations found"
    assert declared == set(_lib.SYMBOLS), (declared ^ set(_lib.SYMBOLS))
    for name in declared:
        assert hasattr(cuda_lib, name), name
    assert b"sm_100a" in cuda_lib.subspec_version()


def test_struct_sizes_are_checked(cuda_lib):
    a = _lib.VerifyArgs()
    a.struct_size = C.sizeof(_lib.VerifyArgs) - 8
    assert cuda_lib.subspec_verify_batched(C.byref(a), None) == _lib.EINVAL
    # a correctly sized, empty batch is accepted without touching the device
    a.struct_size = C.sizeof(_lib.VerifyArgs)
    a.batch, a.max_nodes, a.vocab, a.max_out = 0, 8, 16, 9
    assert cuda_lib.subspec_verify_batched(C.byref(a), None) == _lib.OK
    k = _lib.KvPagedArgs()
    k.struct_size = C.sizeof(_lib.KvPagedArgs)
    k.batch, k.layers, k.num_pages, k.page_len, k.heads, k.head_dim, k.elem_bytes = 0, 1, 1, 16, 4, 128, 2
    assert cuda_lib.subspec_kv_compact_paged(C.byref(k), None) == _lib.OK
    k.elem_bytes = 3
    assert cuda_lib.subspec_kv_compact_paged(C.byref(k), None) == _lib.EINVAL
    h = _lib.KvHfArgs()
    h.struct_size = 4
    assert cuda_lib.subspec_kv_compact_hf(C.byref(h), None) == _lib.EINVAL


def test_argument_validation(cuda_lib):
    n = C.c_size_t(0)
    assert cuda_lib.subspec_verify_scratch_bytes(4, 64, C.byref(n)) == _lib.OK and n.value > 0
    assert cuda_lib.subspec_verify_scratch_bytes(4, 5000, C.byref(n)) == _lib.EINVAL
    a = _lib.VerifyArgs()
    a.struct_size = C.sizeof(_lib.VerifyArgs)
    a.batch, a.max_nodes, a.vocab, a.max_out = 1, 8, 16, 9
    # null pointers are rejected before any launch
    assert cuda_lib.subspec_verify_batched(C.byref(a), None) == _lib.EINVAL
    a.max_nodes = 4096
    assert cuda_lib.subspec_verify_batched(C.byref(a), None) == _lib.EUNSUPPORTED
    # lm_head + verify: sizes, the embedded verify arguments, what the fused path does not take
    assert cuda_lib.subspec_lm_head_verify_scratch_bytes(4, 64, 64, 152064, C.byref(n)) == _lib.OK
    assert n.value >= 4 * 64 * 594 * 20
    assert cuda_lib.subspec_lm_head_verify_scratch_bytes(4, 64, 0, 152064, C.byref(n)) == _lib.EINVAL
    la = _lib.LmHeadVerifyArgs()
    la.struct_size = C.sizeof(_lib.LmHeadVerifyArgs)
    assert cuda_lib.subspec_lm_head_verify(C.byref(la), None) == _lib.EINVAL  # verify.struct_size not set
    v = la.verify
    v.struct_size = C.sizeof(_lib.VerifyArgs)
    v.batch, v.max_nodes, v.vocab, v.max_out, v.dtype = 1, 8, 512, 9, _lib.torch_dtype_code(__import__("torch").bfloat16)
    la.hidden_dim, la.hidden_seq_rows = 64, 8
    assert cuda_lib.subspec_lm_head_verify(C.byref(la), None) == _lib.EINVAL  # null pointers
    la.hidden_dim = 60
    assert cuda_lib.subspec_lm_head_verify(C.byref(la), None) == _lib.EUNSUPPORTED
    la.hidden_dim = 64
    v.do_sample = 1
    assert cuda_lib.subspec_lm_head_verify(C.byref(la), None) == _lib.EUNSUPPORTED
    v.do_sample, v.batch = 0, 0
    assert cuda_lib.subspec_lm_head_verify(C.byref(la), None) == _lib.OK  # an empty batch touches nothing


def test_header_is_plain_c_and_matches_the_ctypes_mirror(tmp_path):
    """The header compiles as C99 on its own, and every argument struct has the size and field offsets the
    ctypes mirror in subspec_b200/_lib.py assumes (a host in another language binds against the same layout)."""
    import shutil
    import subprocess

    gcc = shutil.which("gcc")
    assert gcc, "gcc is part of the toolchain"
    structs = {"subspec_verify_args": _lib.VerifyArgs, "subspec_kv_paged_args": _lib.KvPagedArgs,
               "subspec_kv_hf_args": _lib.KvHfArgs, "subspec_expand_args": _lib.ExpandArgs,
               "subspec_tree_finalize_args": _lib.TreeFinalizeArgs, "subspec_w4a16_args": _lib.W4A16Args,
               "subspec_w4a16_group_args": _lib.W4A16GroupArgs,
               "subspec_post_verify_args": _lib.PostVerifyArgs, "subspec_pages_args": _lib.PagesArgs,
               "subspec_tree_attn_args": _lib.TreeAttnArgs, "subspec_kv_append_args": _lib.KvAppendArgs,
               "subspec_tree_prune_depth_args": _lib.TreePruneDepthArgs,
               "subspec_lm_head_verify_args": _lib.LmHeadVerifyArgs}
    lines = ['#include <stdio.h>', '#include <stddef.h>', '#include "subspec_b200.h"', 'int main(void) {']
    for cname, mirror in structs.items():
        lines.append(f'  printf("{cname} %zu\\n", sizeof({cname}));')
        for field, _ in mirror._fields_:
            lines.append(f'  printf("{cname}.{field} %zu\\n", offsetof({cname}, {field}));')
    lines += ["  return 0;", "}"]
    src = tmp_path / "layout.c"
    src.write_text("\n".join(lines) + "\n")
    exe = tmp_path / "layout"
    subprocess.run([gcc, "-std=c99", "-Wall", "-Wextra", "-Werror", "-pedantic", "-I", str(HEADER.parent), str(src),
                    "-o", str(exe)], check=True)
    got = dict(line.rsplit(" ", 1) for line in subprocess.run([str(exe)], check=True, capture_output=True,
                                                             text=True).stdout.splitlines())
    for cname, mirror in structs.items():
        assert int(got[cname]) == C.sizeof(mirror), cname
        for field, _ in mirror._fields_:
            assert int(got[f"{cname}.{field}"]) == getattr(mirror, field).offset, (cname, field)
