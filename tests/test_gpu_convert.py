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


def test_fused_qkv_with_mixed_bias():
    """Whisper's attention: q and v have a bias, k has none (asrq/models/transformers/whisper.py:94-97)."""
    torch.manual_seed(6)
    d = 1280
    q, k, v = nn.Linear(d, d), nn.Linear(d, d, bias=False), nn.Linear(d, d)
    parts = [C.linearq_from_linear(l, 4, 128).to(DEV) for l in (q, k, v)]
    assert parts[1].bias is None
    fused = C.FusedLinearQ(parts)
    for m in (1, 32, 200):
        x = torch.randn(m, d).half()
        outs = fused(x.to(DEV))
        for o, p in zip(outs, parts):
            assert_close_rows(o, _ref_layer(p, x.float()), what=f"mixed-bias qkv m={m}")


@pytest.mark.gpu
@pytest.mark.parametrize("chunks", [1, 4, 7])
def test_forward_host_matches_one_call(chunks):
    """Host-to-host pipelined call against copying in, one forward, copying out: same bits when the chunks
    are served by the same kernel as the whole batch, within the accuracy bar otherwise."""
    import asrq_b200
    from oracle import linearq_oracle as O
    case = O.make_c1(seed=3, m=1000, k=1280, n=1280)
    lq = asrq_b200.LinearQ(1280, 1280, 4, 128, bias=True).to("cuda:0")
    lq.load_quantized_params(case["scales"], case["zeros"], case["weight"])
    lq.bias = case["bias"].to("cuda:0")
    xh = case["x"].pin_memory()
    ref = lq(xh.to("cuda:0")).cpu()
    out = torch.empty(1000, 1280, dtype=torch.float16).pin_memory()
    got = asrq_b200.forward_host(lq, xh, out, chunks=chunks)
    torch.cuda.synchronize()
    assert got is out
    ref32 = O.linearq_forward_fp32(case["x"], case["weight"], case["scales"], case["zeros"], case["bias"], 4, 128)
    assert_close_rows(out, ref32, what=f"forward_host chunks={chunks}")
    if chunks == 1:
        assert torch.equal(out, ref)
    x2, w2 = torch.randn(900, 4096).half(), torch.randn(256, 4096) * 0.02
    qq = asrq_b200.LinearQQ(4096, 256, 4, 4, 128, bias=False).to("cuda:0")
    pw, sw = asrq_b200.pack_w4a4(w2, 128, True)
    qq.load_quantized_params(sw, torch.zeros_like(sw), pw)
    ref2 = qq(x2.to("cuda:0")).cpu()
    got2 = asrq_b200.forward_host(qq, x2.pin_memory(), chunks=chunks)
    torch.cuda.synchronize()
    scale = ref2.float().abs().max(dim=-1, keepdim=True).values
    assert float(((got2.float() - ref2.float()).abs() / scale).max()) < 2e-3
    if chunks == 1:
        assert torch.equal(got2, ref2)
