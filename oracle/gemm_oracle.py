"""CPU oracle for the W4A16 group-wise dequant GEMM.  TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the arithmetic lives in two third-party packages the reference imports but does
not vendor (hqq==0.2.6, HQQLinear with nbits=4, group_size=64, axis=1; gemlite==0.5.1.post1, the
A16W4 kernel HQQ's `prepare_for_inference(backend="gemlite")` patches in --
specdecodes/helpers/quantizers/hqq/__init__.py:5-8, 65-66, 119; requirements.txt:7-8).  Neither is
installed here and the reference has no test or golden vector at that boundary.  This module states
the published definition of that format: w = (q - zero[group]) * scale[group] with groups of 64
along the input dimension, y = x @ w^T, and the benchmark config's value ranges.

Only tests/, __graft_entry__.smoke() and bench.py's CPU baseline may import this module.
"""
from __future__ import annotations

import torch

GROUP = 64


def unpack_nibbles(qweight: torch.Tensor) -> torch.Tensor:
    """int32 [N, K/8] -> int64 [N, K]; value i of word j sits in bits 4i..4i+3."""
    shifts = torch.arange(8, dtype=torch.int64) * 4
    q = (qweight.to(torch.int64).unsqueeze(-1) >> shifts) & 0xF
    return q.reshape(qweight.shape[0], -1)


def dequant(qweight: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """fp32 [N, K] weights."""
    q = unpack_nibbles(qweight).float()
    N, K = q.shape
    return ((q.reshape(N, K // GROUP, GROUP) - zero.float().unsqueeze(-1)) * scale.float().unsqueeze(-1)).reshape(N, K)


def w4a16_matmul(x: torch.Tensor, qweight: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """fp32 [M, N] = x.float() @ dequant(W)^T."""
    return x.float() @ dequant(qweight, scale, zero).t()


def config4_case(n: int, k: int, m: int, seed: int):
    """The HQQ-style synthetic linear of the GEMM benchmark: uint4 weights, scale ~U(0.005, 0.02), zero ~U(0, 15) in fp16, x ~N(0, 1) bf16."""
    from subspec_b200.synthetic import w4a16_case

    return w4a16_case(n, k, m, seed, GROUP)
