"""The steps either side of a quantized layer: fused add + layer norm, and the activation / residual
epilogues fused into the layer kernels, against the unfused torch sequence on the same device."""
import pytest
import torch
import torch.nn.functional as F

import asrq_b200
from oracle import linearq_oracle as O
from tests.gpu_util import DEV, make_layer

pytestmark = pytest.mark.gpu


@pytest.mark.parametrize("rows,dim", [(32, 1280), (1, 1280), (1500, 1280), (7, 1024), (33, 2048), (5, 256), (9, 384), (3, 100)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("with_delta", [False, True])
def test_add_layernorm(rows, dim, dtype, with_delta):
    gen = torch.Generator().manual_seed(rows + dim)
    x = (torch.randn(rows, dim, generator=gen) * 2).to(dtype).to(DEV)
    d = (torch.randn(rows, dim, generator=gen)).to(dtype).to(DEV) if with_delta else None
    w = (1 + 0.1 * torch.randn(dim, generator=gen)).to(dtype).to(DEV)
    b = (0.1 * torch.randn(dim, generator=gen)).to(dtype).to(DEV)
    xs, h = asrq_b200.add_layernorm(x, d, w, b, 1e-5)
    x_ref = x + d if with_delta else x
    assert torch.equal(xs, x_ref)                                   # the sum is the 16-bit sum torch makes
    h_ref = F.layer_norm(x_ref.float(), (dim,), w.float(), b.float(), 1e-5)
    err = (h.float() - h_ref).abs().max().item()
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert err <= 0.6 * ulp * max(1.0, h_ref.abs().max().item()), err  # one rounding of the fp32 result
    # against torch's own 16-bit layer_norm: equal up to one unit in the last place
    h_t = F.layer_norm(x_ref, (dim,), w, b, 1e-5)
    assert (h.float() - h_t.float()).abs().max().item() <= 1.01 * ulp * max(1.0, h_ref.abs().max().item())


@pytest.mark.parametrize("m,k,n", [(32, 1280, 1280), (1500, 1280, 5120), (8, 1280, 1280), (200, 1280, 1280), (32, 5120, 1280)])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_fused_epilogues_match_the_unfused_sequence(m, k, n, dtype):
    """gelu(layer(x)) and residual + layer(x) from the kernel epilogue (tcgen05 kernels) or the library's extra
    pass (other kernels) against LinearQ followed by torch: the residual form bit for bit, the activation to
    one unit in the last place (torch may order the erf form's products differently)."""
    gen = torch.Generator().manual_seed(m + n)
    w = torch.randn(n, k, generator=gen) * 0.05
    codes, scales, zeros, _ = O.rtn_codes(w, 4, 128, False)
    case = dict(x=torch.randn(m, k, generator=gen).to(dtype), weight=O.pack_codes(codes, 4), scales=scales.half(),
                zeros=zeros.half(), bias=(torch.randn(n, generator=gen) * 0.05).half(), bits=4, group_size=128)
    lq = make_layer(case)
    x = case["x"].to(DEV)
    res = torch.randn(m, n, generator=gen).to(dtype).to(DEV)
    y = lq(x)
    y_res = lq.forward_fused(x, residual=res)
    assert torch.equal(y_res, res + y)
    y_act = lq.forward_fused(x, gelu=True)
    ref = F.gelu(y)
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    tol = 1.01 * ulp * ref.float().abs().clamp_min(2.0 ** -14)
    assert bool(((y_act.float() - ref.float()).abs() <= tol).all())
    assert float((y_act != ref).float().mean()) < 0.02
    asrq_b200.check_status()
