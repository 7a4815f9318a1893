"""The no-allocation verify entry point gives the same answers as the one that takes a caller-owned scratch buffer.

`subspec_verify_batched_static_scratch` is for hosts that cannot hand the library a scratch buffer -- a serving
loop that gave all device memory to its own pools at start-up, or a thin binding without a device allocator.
It keeps its scratch in an array inside the library image.  Both entry points are called here directly through
the C ABI with the same argument struct, twice in a row (a lossy verify, then an exact verify over different
trees and logits), so the second call meets whatever the first one left in the shared array.
This file sorts last on purpose: a `-x` run has already executed every other test when it gets here.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from subspec_b200 import _lib, synthetic
from subspec_b200.tree import Tree
from subspec_b200.verify import VerifyWorkspace, flatten_tree

pytestmark = pytest.mark.gpu

OUTPUTS = ("out_tokens", "out_hidden", "out_meta", "node_target", "node_entropy", "node_child_prob", "node_rowmax",
           "node_rowsum", "node_exact_after", "node_best_len", "node_best_next")


def _args(ws: VerifyWorkspace, logits: torch.Tensor, method: int, gate: int) -> _lib.VerifyArgs:
    a = _lib.VerifyArgs()
    a.struct_size = C.sizeof(_lib.VerifyArgs)
    a.batch, a.max_nodes, a.vocab = ws.batch, ws.max_nodes, int(logits.shape[2])
    a.dtype, a.input_kind = _lib.torch_dtype_code(logits.dtype), _lib.IN_LOGITS
    a.seq_stride, a.row_stride, a.logits = int(logits.stride(0)), int(logits.stride(1)), logits.data_ptr()
    for name in ("n_nodes", "n_rows", "token_ids", "child_off", "child_idx", "root"):
        setattr(a, name, ws._in_ptr(name))
    a.temperature, a.top_p, a.uniforms = 1.0, 1.0, ws.uniforms.data_ptr()
    a.method, a.gate, a.threshold, a.window, a.eos = method, gate, 0.3, 1, -1
    a.max_out = ws.max_out
    for name in OUTPUTS + ("dev_status",):
        setattr(a, name, ws._out_ptr(name))
    return a


def _case(seed: int, batch: int, nodes: int, vocab: int, dtype):
    gen = torch.Generator().manual_seed(seed)
    sts = [synthetic.random_tree(nodes, 6, 4, vocab, gen) for _ in range(batch)]
    logits = torch.stack([synthetic.verify_logits(st, vocab, gen, dtype=dtype, peaked=True) for st in sts]).cuda()
    flats = []
    for st in sts:
        tok, off, idx = flatten_tree(Tree.from_arrays(st.token_ids.tolist(), st.parents.tolist()), 0, st.n, True)
        flats.append((tok, off, idx, st.n, 0))
    return flats, logits


def _valid(out, flats):
    """Copies of the defined parts of every output (entries past a sequence's length are never written)."""
    got = {}
    for b, f in enumerate(flats):
        n, L = len(f[0]), int(out["out_meta"][b, 0])
        for name in OUTPUTS:
            arr = out[name][b]
            if name in ("out_tokens", "out_hidden"):
                arr = arr[:L]
            elif name == "node_child_prob":
                arr = arr[1:n]  # the root has no parent
            elif name != "out_meta":
                arr = arr[:n]
            got[(name, b)] = np.array(arr, copy=True)
    return got


def test_static_scratch_entry_matches_caller_scratch_entry(cuda_lib):
    dev = torch.device("cuda", 0)
    torch.cuda.set_device(dev)
    stream = C.c_void_p(torch.cuda.current_stream(dev).cuda_stream)
    calls = [
        # few rows: every row is split over several CTAs, so the partials area of the scratch is exercised
        dict(seed=901, batch=3, nodes=24, vocab=32000, dtype=torch.bfloat16, method=_lib.VERIFY_LOSSY,
             gate=_lib.GATE_ENTROPY),
        dict(seed=902, batch=40, nodes=64, vocab=4099, dtype=torch.float32, method=_lib.VERIFY_EXACT,
             gate=_lib.GATE_PROB),
    ]
    for c in calls:
        flats, logits = _case(c["seed"], c["batch"], c["nodes"], c["vocab"], c["dtype"])
        ws = VerifyWorkspace(c["batch"], c["nodes"], dev)
        ws.set_trees(flats)
        a = _args(ws, logits, c["method"], c["gate"])
        # reference run: caller-owned scratch
        a.scratch, a.scratch_bytes = ws._scratch_ptr, ws._scratch_bytes
        assert cuda_lib.subspec_verify_batched(C.byref(a), stream) == _lib.OK
        want = _valid(ws.fetch(), flats)
        ws._out_dev.zero_()
        # the entry point under test: no scratch passed at all
        a.scratch, a.scratch_bytes = None, 0
        assert cuda_lib.subspec_verify_batched_static_scratch(C.byref(a), stream) == _lib.OK
        got = _valid(ws.fetch(), flats)
        for key in want:
            if want[key].dtype.kind == "f":  # same kernel, same reduction order: the tolerance is there for form
                assert np.allclose(got[key], want[key], rtol=1e-5, atol=1e-7), key
            else:
                assert np.array_equal(got[key], want[key]), key
        assert int(want[("out_meta", 0)][0]) >= 1


def test_static_scratch_entry_rejects_oversized_batches(cuda_lib):
    a = _lib.VerifyArgs()
    a.struct_size = C.sizeof(_lib.VerifyArgs)
    a.batch, a.max_nodes, a.vocab, a.max_out = 65, 64, 1000, 65  # 4160 rows > 4096
    assert cuda_lib.subspec_verify_batched_static_scratch(C.byref(a), None) == _lib.ETOOLARGE
    with pytest.raises(ValueError, match="4096"):
        _lib.check(_lib.ETOOLARGE, "subspec_verify_batched_static_scratch")
