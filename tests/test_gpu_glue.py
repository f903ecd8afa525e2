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


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,dim,with_delta", [(64, 2048, True), (32, 2048, False), (7, 1024, True), (5, 256, True),
                                                 (3, 96, True), (16, 128, False)])
def test_add_rmsnorm(rows, dim, with_delta, dtype):
    """Against the module sequence of the Qwen3 decoder block: residual add in the tensor's type, then the norm module
    (fp32 statistics, the normalised value cast to the tensor's type, then times the weight).  The sum is bit-exact;
    the normalised output may differ by one unit in the last place where the fp32 reduction order moves a rounding."""
    gen = torch.Generator().manual_seed(rows * dim + 3)
    x = torch.randn(rows, dim, generator=gen).to(dtype)
    delta = (torch.randn(rows, dim, generator=gen) * 0.5).to(dtype) if with_delta else None
    gamma = (1 + 0.1 * torch.randn(dim, generator=gen)).to(dtype)
    eps = 1e-6
    xd, dd, gd = x.to(DEV), None if delta is None else delta.to(DEV), gamma.to(DEV)
    xs, h = asrq_b200.add_rmsnorm(xd, dd, gd, eps)
    xs_ref = x if delta is None else (x + delta)
    f = xs_ref.float()
    n = (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)
    h_ref = gamma * n
    assert torch.equal(xs.cpu(), xs_ref)
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    err = (h.float().cpu() - h_ref.float()).abs()
    assert bool((err <= 2 * ulp * h_ref.float().abs().clamp_min(2.0 ** -14)).all()), float(err.max())
    assert float((err > 0).float().mean()) < 0.02
    _, h2 = asrq_b200.add_rmsnorm(xd, dd, gd, eps, write_sum=False)
    assert torch.equal(h2, h)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,inter", [(64, 6144), (1, 6144), (33, 512), (5, 8)])
def test_silu_mul(rows, inter, dtype):
    """act_fn(gate) * up with each factor rounded to the tensor's type, as the unfused module sequence rounds them."""
    gen = torch.Generator().manual_seed(rows + inter)
    gu = (torch.randn(rows, 2 * inter, generator=gen) * 2).to(dtype)
    out = asrq_b200.silu_mul(gu.to(DEV))
    ref = torch.nn.functional.silu(gu[:, :inter].float()).to(dtype) * gu[:, inter:]
    err = (out.float().cpu() - ref.float()).abs()
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    assert bool((err <= 2 * ulp * ref.float().abs().clamp_min(2.0 ** -14)).all()), float(err.max())
    assert float((err > 0).float().mean()) < 0.02   # expf against the library's exp: a last-place difference, rarely
    assert out.shape == (rows, inter)


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("m,k,n", [(32, 1280, 51866), (1, 1280, 51866), (20, 2048, 4099), (32, 2048, 16384), (7, 96, 50), (32, 3200, 1000)])
def test_dense_head(m, k, n, dtype):
    """The floating-point output head against fp32 on the same values (the reduction order differs from the library
    GEMM's, so the comparison is against fp32): within 2e-3 of the row maximum, plus half a unit in the last place of
    the value for bf16, whose rounding alone can cost 3.9e-3 of the row maximum."""
    gen = torch.Generator().manual_seed(m + k + n)
    x = torch.randn(m, k, generator=gen).to(dtype).to(DEV)
    w = (torch.randn(n, k, generator=gen) * 0.05).to(dtype).to(DEV)
    pad = torch.full((m * n + 64,), 7.0, dtype=dtype, device=DEV)
    out = pad[:m * n].view(m, n)
    y = asrq_b200.dense_head(x, w, out=out)
    assert y.data_ptr() == out.data_ptr()
    ref = x.float() @ w.float().t()
    tol = 2e-3 * ref.abs().amax(dim=1, keepdim=True)
    if dtype == torch.bfloat16:
        tol = tol + 2.0 ** -8 * ref.abs()
    assert bool(((y.float() - ref).abs() <= tol).all()), float((y.float() - ref).abs().max())
    assert bool((pad[m * n:] == 7.0).all())                      # nothing written past the result
    assert torch.equal(asrq_b200.dense_head(x, w), y)            # deterministic
    # more than 32 rows go to the library GEMM
    x2 = torch.randn(40, k, generator=gen).to(dtype).to(DEV)
    assert asrq_b200.dense_head(x2, w).shape == (40, n)
    asrq_b200.check_status()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,T,nq,nkv,hd,pos0,on_device", [(64, 1, 16, 8, 128, 37, True), (3, 9, 4, 2, 64, 0, False), (2, 5, 16, 8, 128, 11, False)])
def test_qk_norm_rope(B, T, nq, nkv, hd, pos0, on_device, dtype):
    """Against the module sequence (norm in fp32 then cast, times weight, q * cos + rotate_half(q) * sin, cache update) in
    torch on the same device: values pass untouched, queries and keys agree to two units in the last place (the norm's
    fp32 reduction order), nothing else in the caches is written."""
    gen = torch.Generator().manual_seed(B + T + hd)
    max_len, eps = 64, 1e-6
    heads = nq + 2 * nkv
    qkv = torch.randn(B * T, heads * hd, generator=gen).to(dtype).to(DEV)
    qw = (1 + 0.1 * torch.randn(hd, generator=gen)).to(dtype).to(DEV)
    kw = (1 + 0.1 * torch.randn(hd, generator=gen)).to(dtype).to(DEV)
    inv = 1.0 / (10000.0 ** (torch.arange(0, hd, 2).float() / hd))
    fr = torch.outer(torch.arange(max_len).float(), inv)
    emb = torch.cat((fr, fr), -1)
    cos, sin = emb.cos().to(dtype).to(DEV), emb.sin().to(dtype).to(DEV)
    kc = torch.full((B, nkv, max_len, hd), 3.0, dtype=dtype, device=DEV)
    vc = torch.full((B, nkv, max_len, hd), 3.0, dtype=dtype, device=DEV)
    pos = torch.tensor([pos0], dtype=torch.long, device=DEV) if on_device else pos0
    q = asrq_b200.qk_norm_rope(qkv, qw, kw, cos, sin, kc, vc, pos, B, T, nq, nkv, eps)

    def rms(x, w):
        f = x.float()
        return w * (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).to(dtype)

    def rope(x, c, s):
        h = hd // 2
        return x * c + torch.cat((-x[..., h:], x[..., :h]), -1) * s
    v4 = qkv.view(B, T, heads, hd)
    c, s = cos[pos0:pos0 + T], sin[pos0:pos0 + T]
    q_ref = rope(rms(v4[:, :, :nq], qw).transpose(1, 2), c, s)
    k_ref = rope(rms(v4[:, :, nq:nq + nkv], kw).transpose(1, 2), c, s)
    v_ref = v4[:, :, nq + nkv:].transpose(1, 2)
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)

    def close(a, r):
        return bool(((a.float() - r.float()).abs() <= 2 * ulp * r.float().abs().clamp_min(0.25)).all())
    assert q.shape == (B, nq, T, hd) and close(q, q_ref)
    assert close(kc[:, :, pos0:pos0 + T], k_ref)
    assert torch.equal(vc[:, :, pos0:pos0 + T], v_ref)
    untouched = torch.ones(max_len, dtype=torch.bool)
    untouched[pos0:pos0 + T] = False
    assert bool((kc[:, :, untouched.to(DEV)] == 3.0).all()) and bool((vc[:, :, untouched.to(DEV)] == 3.0).all())


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("B,H,hd,max_len,pos0,scale", [(32, 20, 64, 129, 0, 1.0), (32, 20, 64, 129, 77, 1.0), (3, 4, 128, 40, 39, 0.5),
                                                       (5, 6, 64, 448, 300, 0.125)])
def test_decode_self_attention(B, H, hd, max_len, pos0, scale, dtype):
    """Against the cache update plus scaled_dot_product_attention in fp32 on the same values: the new key and value land at
    the position (nothing else in the cache moves), the output is one rounding of the fp32 result."""
    gen = torch.Generator().manual_seed(B * H + pos0)
    d = H * hd
    qkv = torch.randn(B, 3 * d, generator=gen).to(dtype).to(DEV)
    kv = torch.randn(2, B, H, max_len, hd, generator=gen).to(dtype).to(DEV)
    before = kv.clone()
    pos = torch.tensor([pos0], dtype=torch.long, device=DEV)
    out = asrq_b200.decode_self_attention(qkv, kv, pos, scale)
    k_new = qkv[:, d:2 * d].view(B, H, hd)
    v_new = qkv[:, 2 * d:].view(B, H, hd)
    assert torch.equal(kv[0, :, :, pos0], k_new) and torch.equal(kv[1, :, :, pos0], v_new)
    keep = torch.ones(max_len, dtype=torch.bool, device=DEV)
    keep[pos0] = False
    assert torch.equal(kv[:, :, :, keep], before[:, :, :, keep])
    q = qkv[:, :d].view(B, H, 1, hd).float()
    ref = F.scaled_dot_product_attention(q, kv[0, :, :, :pos0 + 1].float(), kv[1, :, :, :pos0 + 1].float(), scale=scale)
    ref = ref.reshape(B, d)
    ulp = 2.0 ** (-10 if dtype == torch.float16 else -7)
    err = (out.float() - ref).abs()
    assert bool((err <= 0.6 * ulp * ref.abs().clamp_min(1.0) + 1e-6).all()), float(err.max())
