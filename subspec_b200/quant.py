"""HQQ-style 4-bit draft linears on the tcgen05 W4A16 GEMM, behind the reference's quantizer hook.

Reference surface (specdecodes/helpers/...):
  quantizers/hqq/__init__.py:17-119   HqqQuantizer.quantize_model(model, quant_config, compute_dtype, device)
  recipes/subspec/hqq_4bit_postspec.py:21-34   quant_config: layer name -> BaseQuantizeConfig(nbits=4, group_size=64, axis=1)
  recipes/base_recipe.py:44-53        apply_quantization -> quantizer.quantize_model(...)

The reference delegates the arithmetic to two third-party packages (hqq's HQQLinear and gemlite's
A16W4 Triton kernel).  Here the replacement module holds the 4-bit weights in the tiled layout of
`subspec_w4a16_gemm` and runs y = x @ dequant(W)^T on the tensor cores.  Quantisation itself is plain
round-to-nearest affine per group of 64 input features (hqq additionally refines the zero point
with a few proximal iterations; the storage format and the forward arithmetic are the same).
"""
from __future__ import annotations

import ctypes as C
from typing import Dict, Optional, Tuple

import torch
import torch.nn as nn

from . import _lib

GROUP = 64


def BaseQuantizeConfig(nbits: int = 4, group_size: int = 64, axis: int = 1, **_unused) -> dict:
    """Same shape of result as hqq's helper of that name: a dict with 'weight_quant_params'."""
    return {"weight_quant_params": {"nbits": nbits, "group_size": group_size, "axis": axis}}


def _check_config(cfg) -> None:
    p = cfg.get("weight_quant_params", cfg) if isinstance(cfg, dict) else vars(cfg)
    nbits, gs, axis = p.get("nbits", 4), p.get("group_size", 64), p.get("axis", 1)
    if (nbits, gs, axis) != (4, GROUP, 1):
        raise ValueError(f"only nbits=4, group_size=64, axis=1 is supported, got {(nbits, gs, axis)}")


@torch.no_grad()
def quantize_weight(weight: torch.Tensor) -> Tuple[torch.Tensor, torch.Tensor, torch.Tensor]:
    """[N, K] float -> (qweight int32 [N, K/8], scale fp16 [N, K/64], zero fp16 [N, K/64]).

    Group-wise affine along the input dimension: w ~ (q - zero) * scale, q in 0..15.
    qweight packs 8 values per int32, value i of word j in bits 4i..4i+3.
    """
    N, K = weight.shape
    if K % GROUP:
        raise ValueError("in_features must be a multiple of 64")
    w = weight.float().reshape(N, K // GROUP, GROUP)
    lo, hi = w.amin(-1, keepdim=True), w.amax(-1, keepdim=True)
    scale = ((hi - lo) / 15.0).clamp_min(1e-8).half()
    zero = (-lo / scale.float()).half()
    q = torch.clamp(torch.round(w / scale.float() + zero.float()), 0, 15).to(torch.int32).reshape(N, K // 8, 8)
    shifts = torch.arange(8, device=weight.device, dtype=torch.int32) * 4
    qweight = (q << shifts).sum(-1).to(torch.int32)
    return qweight.contiguous(), scale.squeeze(-1).contiguous(), zero.squeeze(-1).contiguous()


@torch.no_grad()
def pack(qweight: torch.Tensor, scale: torch.Tensor, zero: torch.Tensor) -> torch.Tensor:
    """Interchange tensors (on the GPU) -> the kernel's tiled layout (uint8 buffer)."""
    N, K = int(qweight.shape[0]), int(qweight.shape[1]) * 8
    if not qweight.is_cuda:
        raise _lib.SubspecError("pack() runs on the GPU: move the tensors to a CUDA device first")
    qweight = qweight.to(torch.int32).contiguous()
    scale, zero = scale.half().contiguous(), zero.half().contiguous()
    if tuple(scale.shape) != (N, K // GROUP) or tuple(zero.shape) != (N, K // GROUP):
        raise ValueError("scale and zero must be [N, K/64]")
    nbytes = C.c_size_t(0)
    _lib.check(_lib.lib().subspec_w4a16_packed_bytes(N, K, C.byref(nbytes)), "subspec_w4a16_packed_bytes")
    out = torch.empty(nbytes.value, dtype=torch.uint8, device=qweight.device)
    stream = torch.cuda.current_stream(qweight.device).cuda_stream
    _lib.check(_lib.lib().subspec_w4a16_pack(qweight.data_ptr(), scale.data_ptr(), zero.data_ptr(), out.data_ptr(), N, K,
                                            C.c_void_p(stream)), "subspec_w4a16_pack")
    return out


_scratch: Dict[int, torch.Tensor] = {}


@torch.no_grad()
def w4a16_matmul(x: torch.Tensor, packed: torch.Tensor, n: int, k: int, status: Optional[torch.Tensor] = None
                 ) -> torch.Tensor:
    """x bf16 [M, K] (M <= 256) times the packed 4-bit weight [N, K] -> bf16 [M, N]."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k or x.stride(1) != 1:
        raise ValueError("x must be a bf16 [M, K] matrix with contiguous rows")
    M = int(x.shape[0])
    dev = x.device
    need = C.c_size_t(0)
    _lib.check(_lib.lib().subspec_w4a16_scratch_bytes(M, n, k, C.byref(need)), "subspec_w4a16_scratch_bytes")
    buf = _scratch.get(dev.index or 0)
    if buf is None or buf.numel() < need.value + 256:
        buf = _scratch[dev.index or 0] = torch.empty(need.value + 256, dtype=torch.uint8, device=dev)
    y = torch.empty(M, n, dtype=torch.bfloat16, device=dev)
    a = _lib.W4A16Args()
    a.struct_size = C.sizeof(_lib.W4A16Args)
    a.m, a.n, a.k = M, n, k
    a.x, a.x_stride = x.data_ptr(), int(x.stride(0))
    a.packed, a.y, a.y_stride = packed.data_ptr(), y.data_ptr(), n
    a.scratch, a.scratch_bytes = (buf.data_ptr() + 255) // 256 * 256, need.value
    a.dev_status = 0 if status is None else status.data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().subspec_w4a16_gemm(C.byref(a), C.c_void_p(stream)), "subspec_w4a16_gemm")
    return y


@torch.no_grad()
def w4a16_matmul_grouped(x: torch.Tensor, packed, ns, k: int, status: Optional[torch.Tensor] = None):
    """x bf16 [M, K] (M <= 256) times several packed 4-bit weights [N_i, K] in ONE launch -> list of bf16 [M, N_i].

    The projections a decoder layer applies to the same activations (q/k/v; gate/up) cost one launch instead
    of one each; every result equals the separate call's within the GEMM's tolerance (bit for bit when both
    plans split K alike)."""
    if x.dtype != torch.bfloat16 or x.dim() != 2 or x.shape[1] != k or x.stride(1) != 1:
        raise ValueError("x must be a bf16 [M, K] matrix with contiguous rows")
    if not 1 <= len(packed) <= _lib.W4A16_MAX_GROUP or len(packed) != len(ns):
        raise ValueError(f"1 to {_lib.W4A16_MAX_GROUP} weight matrices per grouped call")
    M = int(x.shape[0])
    dev = x.device
    need = C.c_size_t(0)
    _lib.check(_lib.lib().subspec_w4a16_scratch_bytes(M, int(sum(ns)), k, C.byref(need)), "subspec_w4a16_scratch_bytes")
    buf = _scratch.get(dev.index or 0)
    if buf is None or buf.numel() < need.value + 256:
        buf = _scratch[dev.index or 0] = torch.empty(need.value + 256, dtype=torch.uint8, device=dev)
    ys = [torch.empty(M, int(n), dtype=torch.bfloat16, device=dev) for n in ns]
    a = _lib.W4A16GroupArgs()
    a.struct_size = C.sizeof(_lib.W4A16GroupArgs)
    a.m, a.k, a.count = M, k, len(ns)
    a.x, a.x_stride = x.data_ptr(), int(x.stride(0))
    for i, (w, n, y) in enumerate(zip(packed, ns, ys)):
        a.packed[i], a.n[i], a.y[i], a.y_stride[i] = w.data_ptr(), int(n), y.data_ptr(), int(n)
    a.scratch, a.scratch_bytes = (buf.data_ptr() + 255) // 256 * 256, need.value
    a.dev_status = 0 if status is None else status.data_ptr()
    stream = torch.cuda.current_stream(dev).cuda_stream
    _lib.check(_lib.lib().subspec_w4a16_gemm_grouped(C.byref(a), C.c_void_p(stream)), "subspec_w4a16_gemm_grouped")
    return ys


class W4A16Group:
    """The `W4A16Linear` children of one module that are applied to the same input (q/k/v; gate/up), evaluated
    in one launch.  `HqqQuantizer.quantize_model` installs one on the parent of every such set as
    `parent.w4a16_groups[name]`; module boundaries stay as they are, and a forward that wants the saving calls
    `parent.w4a16_groups["qkv"](x)` where it used to call the three projections."""

    def __init__(self, linears):
        linears = list(linears)
        if not linears or len({m.in_features for m in linears}) != 1:
            raise ValueError("a group needs W4A16Linear modules with one common in_features")
        self.linears = linears

    def __call__(self, x: torch.Tensor):
        k = self.linears[0].in_features
        lead = x.shape[:-1]
        x2 = x.reshape(-1, k).to(torch.bfloat16)
        if x2.shape[0] > 256:  # beyond one launch's token limit: the members' own forwards
            return [m(x) for m in self.linears]
        ys = w4a16_matmul_grouped(x2.contiguous(), [m.packed for m in self.linears],
                                  [m.out_features for m in self.linears], k)
        out = []
        for m, y in zip(self.linears, ys):
            if m.bias is not None:
                y = y + m.bias.to(y.dtype)
            out.append(y.reshape(*lead, m.out_features).to(x.dtype))
        return out


# names of sibling projections that a decoder layer applies to one input
_SIBLINGS = {"qkv": ("q_proj", "k_proj", "v_proj"), "gate_up": ("gate_proj", "up_proj")}


class W4A16Linear(nn.Module):
    """Drop-in for nn.Linear with 4-bit group-64 weights; forward(x[..., K]) -> [..., N] in x's dtype."""

    def __init__(self, in_features: int, out_features: int, packed: torch.Tensor, bias: Optional[torch.Tensor] = None):
        super().__init__()
        self.in_features, self.out_features = in_features, out_features
        self.register_buffer("packed", packed)
        self.bias = None if bias is None else nn.Parameter(bias, requires_grad=False)

    @classmethod
    @torch.no_grad()
    def from_linear(cls, linear: nn.Linear, device) -> "W4A16Linear":
        w = linear.weight.detach().to(device)
        qweight, scale, zero = quantize_weight(w)
        bias = None if linear.bias is None else linear.bias.detach().to(device)
        return cls(linear.in_features, linear.out_features, pack(qweight, scale, zero), bias)

    @classmethod
    def from_quantized(cls, qweight, scale, zero, bias=None) -> "W4A16Linear":
        return cls(int(qweight.shape[1]) * 8, int(qweight.shape[0]), pack(qweight, scale, zero), bias)

    def forward(self, x: torch.Tensor) -> torch.Tensor:
        lead = x.shape[:-1]
        x2 = x.reshape(-1, self.in_features).to(torch.bfloat16)
        outs = [w4a16_matmul(x2[i:i + 256].contiguous(), self.packed, self.out_features, self.in_features)
                for i in range(0, x2.shape[0], 256)]
        y = outs[0] if len(outs) == 1 else torch.cat(outs, dim=0)
        if self.bias is not None:
            y = y + self.bias.to(y.dtype)
        return y.reshape(*lead, self.out_features).to(x.dtype)


class HqqQuantizer:
    """Same hook as the reference's HqqQuantizer: swaps the tagged nn.Linear children of `model` in place."""

    @classmethod
    @torch.no_grad()
    def quantize_model(cls, model: nn.Module, quant_config: dict, compute_dtype=None, device="cuda"):
        for name, cfg in quant_config.items():
            _check_config(cfg)
            parent_name, _, child = name.rpartition(".")
            parent = model.get_submodule(parent_name) if parent_name else model
            lin = getattr(parent, child)
            if not isinstance(lin, nn.Linear):
                raise ValueError(f"{name} is not an nn.Linear")
            setattr(parent, child, W4A16Linear.from_linear(lin, device))
        # sibling projections of one input, where all of them were quantised: one launch per set on request
        for parent in model.modules():
            groups = {}
            for gname, members in _SIBLINGS.items():
                mods = [getattr(parent, m, None) for m in members]
                if all(isinstance(m, W4A16Linear) for m in mods):
                    groups[gname] = W4A16Group(mods)
            if groups:
                parent.w4a16_groups = groups
        return model
