"""Converted model blocks on the GPU: forward parity with the fp32 CPU result of the dequantised
weights, fused projections against the separate layers."""
import pytest
import torch
import torch.nn as nn

import asrq_b200
from asrq_b200 import convert as C
from oracle import linearq_oracle as O
from tests.gpu_util import DEV, assert_close_rows

pytestmark = pytest.mark.gpu


class Mlp(nn.Module):
    def __init__(self, d, ff):
        super().__init__()
        self.gate_proj = nn.Linear(d, ff, bias=False)
        self.up_proj = nn.Linear(d, ff, bias=False)
        self.down_proj = nn.Linear(ff, d, bias=False)

    def forward(self, x):
        return self.down_proj(torch.nn.functional.silu(self.gate_proj(x)) * self.up_proj(x))


def _ref_layer(lq, x32):
    w = lq.dequantize_weight(device="cpu", dtype=torch.float32)   # includes the fp16 rounding of scale and zero
    y = x32 @ w.t()
    return y if lq.bias is None else y + lq.bias.float().cpu()


@pytest.mark.parametrize("m_tokens", [1, 7, 200])
@pytest.mark.parametrize("bits", [4, 2])
def test_converted_layers_and_fused_gate_up(bits, m_tokens):
    torch.manual_seed(bits * 100 + m_tokens)
    d, ff = 512, 1536
    mlp = Mlp(d, ff)
    with torch.no_grad():
        for p in mlp.parameters():
            p.mul_(0.5)
    C.convert(mlp, bits=bits, group_size=128)
    mlp.to(DEV)
    x = torch.randn(m_tokens, d).half()
    xd = x.to(DEV)
    g, u = mlp.gate_proj(xd), mlp.up_proj(xd)
    assert_close_rows(g, _ref_layer(mlp.gate_proj, x.float()), what="gate")
    assert_close_rows(u, _ref_layer(mlp.up_proj, x.float()), what="up")
    fused = C.FusedLinearQ([mlp.gate_proj, mlp.up_proj])
    gf, uf = fused(xd)
    assert gf.shape == g.shape and uf.shape == u.shape
    assert_close_rows(gf, _ref_layer(mlp.gate_proj, x.float()), what="fused gate")
    assert_close_rows(uf, _ref_layer(mlp.up_proj, x.float()), what="fused up")
    # the whole block, fp16 between the layers as the reference's *Q models run it
    y = mlp(xd)
    h = (torch.nn.functional.silu(g.float()) * u.float()).half().cpu()
    assert_close_rows(y, _ref_layer(mlp.down_proj, h.float()), what="down")
    asrq_b200.check_status()


def test_fused_qkv_matches_whisper_shapes_with_leading_dims():
    torch.manual_seed(5)
    d = 1280
    q, k, v = nn.Linear(d, d), nn.Linear(d, d), nn.Linear(d, d)
    parts = [C.linearq_from_linear(l, 4, 128).to(DEV) for l in (q, k, v)]
    fused = C.FusedLinearQ(parts)
    x = torch.randn(2, 3, d).half()
    outs = fused(x.to(DEV))
    for o, p in zip(outs, parts):
        assert o.shape == (2, 3, d)
        assert_close_rows(o.reshape(6, d), _ref_layer(p, x.reshape(6, d).float()), what="qkv")
