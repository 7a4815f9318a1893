"""W4A16 dequant GEMM on tcgen05: against the fp32 restatement, max rel err 1e-2 (bf16 tolerance)."""
import pytest
import torch
import torch.nn as nn

from oracle import gemm_oracle as go
from subspec_b200 import quant

pytestmark = pytest.mark.gpu

TOL = 1e-2  # max |y - y_ref| / max |y_ref|, the stated bf16 tolerance


def _rel_err(y, ref):
    return float((y.float().cpu() - ref).abs().max() / ref.abs().max())


@pytest.mark.parametrize("n,k", [(512, 3584), (3584, 3584), (18944, 3584), (3584, 18944)])
@pytest.mark.parametrize("m", [16, 64, 256])
def test_config4_shapes(cuda_lib, n, k, m):
    qweight, scale, zero, x = go.config4_case(n, k, m, seed=n + k + m)
    packed = quant.pack(qweight.cuda(), scale.cuda(), zero.cuda())
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    y = quant.w4a16_matmul(x.cuda(), packed, n, k, status=status)
    assert int(status.item()) == 0
    ref = go.w4a16_matmul(x, qweight, scale, zero)
    assert y.shape == (m, n) and y.dtype == torch.bfloat16
    assert _rel_err(y, ref) < TOL
    # a second call on the same scratch gives the same bits (tickets reset, no stale partials)
    y2 = quant.w4a16_matmul(x.cuda(), packed, n, k, status=status)
    assert torch.equal(y, y2)


def test_small_and_ragged_m(cuda_lib):
    # every accumulator layout (8, 4, 2, 1 accumulators), 1-4 issuing warps, K ranges that end inside a
    # four-block chunk, one K block only, and rings that wrap many times (64 K blocks in one CTA)
    for m, n, k in [(1, 128, 64), (3, 256, 128), (17, 384, 640), (100, 128, 4096), (255, 640, 192),
                    (33, 256, 64 * 37), (48, 128, 64 * 5), (64, 18944, 4096), (96, 256, 64 * 9),
                    (130, 256, 1024), (200, 18944, 576), (16, 18944, 4096)]:
        qweight, scale, zero, x = go.config4_case(n, k, m, seed=m)
        y = quant.w4a16_matmul(x.cuda(), quant.pack(qweight.cuda(), scale.cuda(), zero.cuda()), n, k)
        assert _rel_err(y, go.w4a16_matmul(x, qweight, scale, zero)) < TOL, (m, n, k)
    # linearity in x: f(2x) = 2 f(x) exactly (powers of two commute with every rounding involved)
    qweight, scale, zero, x = go.config4_case(256, 512, 32, seed=9)
    packed = quant.pack(qweight.cuda(), scale.cuda(), zero.cuda())
    y1 = quant.w4a16_matmul(x.cuda(), packed, 256, 512)
    y2 = quant.w4a16_matmul((x * 2).cuda(), packed, 256, 512)
    assert torch.equal(y2.float(), y1.float() * 2)
    with pytest.raises(ValueError):
        quant.w4a16_matmul(x.cuda()[:, :100].contiguous(), packed, 256, 100)  # K not a multiple of 64


def test_quantizer_hook_replaces_linears(cuda_lib):
    """HqqQuantizer.quantize_model swaps tagged nn.Linear modules; the forward matches dequantised fp32 math."""
    torch.manual_seed(0)

    class Block(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = nn.Linear(256, 384, bias=True)
            self.o_proj = nn.Linear(384, 256, bias=False)
            self.norm = nn.LayerNorm(256)

    class Net(nn.Module):
        def __init__(self):
            super().__init__()
            self.layers = nn.ModuleList([Block(), Block()])

    net = Net().cuda()
    ref_w = net.layers[1].q_proj.weight.detach().clone()
    ref_b = net.layers[1].q_proj.bias.detach().clone()
    cfg = {f"layers.{i}.{p}": quant.BaseQuantizeConfig(nbits=4, group_size=64, axis=1)
           for i in range(2) for p in ("q_proj", "o_proj")}
    quant.HqqQuantizer.quantize_model(net, cfg, compute_dtype=torch.bfloat16, device="cuda")
    assert isinstance(net.layers[1].q_proj, quant.W4A16Linear) and isinstance(net.layers[0].norm, nn.LayerNorm)
    x = torch.randn(2, 5, 256, device="cuda", dtype=torch.bfloat16)
    y = net.layers[1].q_proj(x)
    assert y.shape == (2, 5, 384) and y.dtype == torch.bfloat16
    qweight, scale, zero = quant.quantize_weight(ref_w)
    ref = go.w4a16_matmul(x.reshape(-1, 256).cpu(), qweight.cpu(), scale.cpu(), zero.cpu()) + ref_b.float().cpu()
    assert _rel_err(y.reshape(-1, 384), ref) < TOL
    # 4-bit round-to-nearest keeps the layer close to the original weights
    full = x.reshape(-1, 256).float() @ ref_w.float().t() + ref_b.float()
    assert _rel_err(y.reshape(-1, 384), full.cpu()) < 0.15
    with pytest.raises(ValueError):
        quant.HqqQuantizer.quantize_model(Net().cuda(), {"layers.0.q_proj": quant.BaseQuantizeConfig(nbits=8)}, None,
                                          "cuda")


@pytest.mark.parametrize("m", [16, 64, 256])
@pytest.mark.parametrize("ns,k", [((3584, 512, 512), 3584), ((18944, 18944), 3584), ((128, 256, 128, 384), 640)])
def test_grouped_projections_equal_separate_calls(cuda_lib, ns, k, m):
    """q/k/v and gate/up as one launch each: every projection's result against the oracle, and against its own
    separate call -- bit for bit where both launches cut K into the same pieces (the partial sums are then
    added in the same order), within the stated tolerance otherwise."""
    from subspec_b200 import _lib
    import ctypes as C

    mats = [go.config4_case(n, k, m, seed=17 + i + n) for i, n in enumerate(ns)]
    x = mats[0][3]
    packed = [quant.pack(q.cuda(), s.cuda(), z.cuda()) for q, s, z, _ in mats]
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ys = quant.w4a16_matmul_grouped(x.cuda(), packed, list(ns), k, status=status)
    assert int(status.item()) == 0
    for (q, s, z, _), n, w, y in zip(mats, ns, packed, ys):
        assert y.shape == (m, n)
        assert _rel_err(y, go.w4a16_matmul(x, q, s, z)) < TOL
        sep = quant.w4a16_matmul(x.cuda(), w, n, k)
        assert _rel_err(y, sep.float().cpu()) < 4e-3   # fp32 sums added in another order: one bf16 ulp at most
    again = quant.w4a16_matmul_grouped(x.cuda(), packed, list(ns), k)
    assert all(torch.equal(a, b) for a, b in zip(ys, again))
    # a group of one is the plain call
    one = quant.w4a16_matmul_grouped(x.cuda(), packed[:1], [ns[0]], k)[0]
    assert torch.equal(one, quant.w4a16_matmul(x.cuda(), packed[0], ns[0], k))
    a = _lib.W4A16GroupArgs()
    a.struct_size = C.sizeof(_lib.W4A16GroupArgs)
    a.m, a.k, a.count = m, k, 5
    assert cuda_lib.subspec_w4a16_gemm_grouped(C.byref(a), None) == _lib.EINVAL


def test_quantizer_installs_sibling_groups(cuda_lib):
    torch.manual_seed(1)

    class Attn(nn.Module):
        def __init__(self):
            super().__init__()
            self.q_proj = nn.Linear(256, 384, bias=True)
            self.k_proj = nn.Linear(256, 128, bias=True)
            self.v_proj = nn.Linear(256, 128, bias=True)
            self.o_proj = nn.Linear(384, 256, bias=False)

    net = nn.ModuleList([Attn()]).cuda()
    cfg = {f"0.{p}": quant.BaseQuantizeConfig(nbits=4, group_size=64, axis=1)
           for p in ("q_proj", "k_proj", "v_proj", "o_proj")}
    quant.HqqQuantizer.quantize_model(net, cfg, compute_dtype=torch.bfloat16, device="cuda")
    attn = net[0]
    assert set(attn.w4a16_groups) == {"qkv"}
    x = torch.randn(3, 7, 256, device="cuda", dtype=torch.bfloat16)
    q, k, v = attn.w4a16_groups["qkv"](x)
    for got, mod in ((q, attn.q_proj), (k, attn.k_proj), (v, attn.v_proj)):
        want = mod(x)
        assert got.shape == want.shape and got.dtype == want.dtype
        assert float((got.float() - want.float()).abs().max() / want.float().abs().max()) < 4e-3
