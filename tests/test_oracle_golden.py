"""The oracle restatement against fixtures produced by the reference's own code."""
import glob
import os

import numpy as np
import pytest
import torch

from oracle import linearq_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _f16(a):
    return torch.from_numpy(a.view(np.float16).copy())


def _names(prefix):
    return sorted(os.path.basename(p)[len(prefix):-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


@pytest.mark.parametrize("name", _names("rtn_"))
def test_rtn_matches_reference(name):
    d = np.load(os.path.join(GOLDEN, f"rtn_{name}.npz"))
    w = torch.from_numpy(d["w"])
    if bool(d["w_is_f16"]):
        w = w.half()
    bits, g, sym = int(d["bits"]), int(d["group_size"]), bool(d["symmetric"])
    codes, scales, zeros, fq = O.rtn_codes(w, bits, g, sym)
    assert np.array_equal(scales.float().numpy(), d["scales"])
    assert np.array_equal(zeros.float().numpy(), d["zeros"])
    assert np.array_equal(fq.float().numpy(), d["fake_quant"])
    lo, hi = O.quant_range(bits, sym)
    assert int(codes.min()) >= lo and int(codes.max()) <= hi


@pytest.mark.parametrize("name", _names("linearq_"))
def test_linearq_matches_reference(name):
    d = np.load(os.path.join(GOLDEN, f"linearq_{name}.npz"))
    bits, g, k = int(d["bits"]), int(d["group_size"]), int(d["in_features"])
    weight = torch.from_numpy(d["weight"])
    scales, zeros = _f16(d["scales"]), _f16(d["zeros"])
    bias = _f16(d["bias"]) if "bias" in d else None
    x = _f16(d["x"])
    w32 = O.dequantize_weight(weight, scales, zeros, bits, g, k, torch.float32)
    assert np.array_equal(w32.numpy(), d["w_deq_f32"])
    w16 = O.dequantize_weight(weight, scales, zeros, bits, g, k, torch.float16)
    assert np.array_equal(w16.numpy().view(np.uint16), d["w_deq_f16"])
    y32 = O.linearq_forward_fp32(x, weight, scales, zeros, bias, bits, g)
    np.testing.assert_allclose(y32.numpy(), d["y_f32"], rtol=0, atol=1e-5)
    y16 = O.linearq_forward(x, weight, scales, zeros, bias, bits, g)
    np.testing.assert_allclose(y16.float().numpy(), _f16(d["y_f16"]).float().numpy(), rtol=0, atol=2e-3)
    # pack/unpack are mutually inverse on the fixture's packed bytes
    assert torch.equal(O.pack_codes(O.unpack_codes(weight, bits, k), bits), weight)


@pytest.mark.parametrize("name", _names("rtn_"))
def test_pack_roundtrip_through_reference_dequant(name):
    """codes -> pack -> (reference-pinned) dequant reproduces the reference's fake-quant weight."""
    d = np.load(os.path.join(GOLDEN, f"rtn_{name}.npz"))
    w = torch.from_numpy(d["w"])
    if bool(d["w_is_f16"]):
        w = w.half()
    bits, g, sym = int(d["bits"]), int(d["group_size"]), bool(d["symmetric"])
    geff = w.shape[1] if g == -1 else g
    codes, scales, zeros, fq = O.rtn_codes(w, bits, g, sym)
    if sym:
        codes, scales, zeros = O.symmetric_to_unsigned(codes, scales, bits)
    packed = O.pack_codes(codes, bits)
    assert packed.shape == (w.shape[0], w.shape[1] * bits // 8)
    # with un-rounded scales/zeros in the weight dtype, dequant == reference fake quant
    wd = O.dequantize_weight(packed, scales, zeros, bits, geff, w.shape[1], w.dtype)
    if sym:
        np.testing.assert_allclose(wd.float().numpy(), d["fake_quant"], rtol=0, atol=2e-3 if w.dtype == torch.float16 else 1e-6)
    else:
        assert np.array_equal(wd.float().numpy(), d["fake_quant"])


@pytest.mark.parametrize("n", [64, 1024, 4096])
def test_hadamard_matches_reference(n):
    d = np.load(os.path.join(GOLDEN, f"hadamard_{n}.npz"))
    x = torch.from_numpy(d["x"])
    assert np.array_equal(O.hadamard_pow2(x).numpy(), d["y_f32"])
    assert np.array_equal(O.hadamard_pow2(x.half()).numpy().view(np.uint16), d["y_f16"])
    # involution (orthogonal, symmetric)
    np.testing.assert_allclose(O.hadamard_pow2(O.hadamard_pow2(x)).numpy(), d["x"], atol=1e-4)


def test_act_quant_matches_reference():
    d = np.load(os.path.join(GOLDEN, "actquant_4bit.npz"))
    x = torch.from_numpy(d["x"])
    assert np.array_equal(O.fake_act_quant(x, 4).numpy(), d["fake_quant"])
    q2, s2 = O.act_quant_sym(torch.from_numpy(d["x2"]), 4)
    assert np.array_equal(q2.float().numpy(), d["q2"])
    assert np.array_equal(s2.numpy(), d["s2"])
    # the all-zero token takes the 1e-3 guard and quantises to zeros
    q, s = O.act_quant_sym(x, 4)
    assert float(s[0, 3, 0]) == pytest.approx(1e-3) and int(q[0, 3].abs().max()) == 0


def test_signed_int4_pack_roundtrip():
    g = torch.Generator().manual_seed(1)
    c = torch.randint(-8, 8, (5, 64), generator=g)
    p = O.pack_signed_int4(c)
    assert torch.equal(O.unpack_signed_int4(p).to(torch.int64), c)
    # convention: even k in the low nibble
    assert int(p[0, 0]) == ((int(c[0, 0]) & 0xF) | ((int(c[0, 1]) & 0xF) << 4))


def test_w4a4_composite_consistency():
    """The composite equals the fake-quant float product it stands for, and the rotation cancels."""
    g = torch.Generator().manual_seed(2)
    m, k, n, gs = 7, 256, 16, 128
    x = torch.randn(m, k, generator=g).half()
    w = torch.randn(n, k, generator=g) * 0.02
    qa, sa, pa = O.hadamard_quant_int4(x, True)
    codes, sw, pw = O.prepare_w4a4_weight(w, gs, True)
    acc = O.int4_group_accumulators(qa, codes, gs)
    ref_acc = torch.einsum("mgk,ngk->mng", qa.long().reshape(m, -1, gs), codes.long().reshape(n, -1, gs))
    assert torch.equal(acc.long(), ref_acc)
    y = O.w4a4_forward_fp32(qa, sa, codes, sw, None, gs)
    xa = qa.float() * sa[:, None]
    wq = (codes.float().reshape(n, -1, gs) * sw.float()[:, :, None]).reshape(n, k)
    np.testing.assert_allclose(y.numpy(), (xa @ wq.t()).numpy(), rtol=1e-4, atol=1e-5)
    # 4-bit x 4-bit is coarse, but must track the unquantised product
    y_true = x.float() @ w.t()
    assert float((y - y_true).abs().max()) < 0.35 * float(y_true.abs().max())


@pytest.mark.parametrize("k", [1024, 4096])
def test_w4a4_composite_against_reference_functions(k):
    """The W4A4 layer assembled out of the reference's own functions (matmul_hadU in fp32 on both
    operands, RTNQuantizer symmetric int4 g128 on the rotated weight, the activation fake-quant patch
    around F.linear) against the integer composite of the oracle.

    Every intermediate is bit-equal: rotated activations, weight codes and (fp32) weight scales.  With
    fp32 weight scales the two results differ only by float summation order: bound 1e-5 of the row
    maximum (measured 6e-7).  With the scales rounded to fp16, as LinearQ stores them
    (asrq/core/linear.py:21-25), the bound is 0.5e-3 of the row maximum (measured 0.37e-3), a quarter
    of the 2e-3 output bar."""
    d = np.load(os.path.join(GOLDEN, f"w4a4_composite_k{k}.npz"))
    x = torch.from_numpy(d["x"].view(np.float16).copy())
    w, g = torch.from_numpy(d["w"]), int(d["group_size"])
    bias = torch.from_numpy(d["bias"].view(np.float16).copy())
    y_ref = torch.from_numpy(d["y"])
    assert np.array_equal(O.hadamard_pow2(x.float()).numpy(), d["v"])
    qa, sa, _ = O.hadamard_quant_int4(x, True)
    codes, sw16, _ = O.prepare_w4a4_weight(w, g, True)
    assert np.array_equal(codes.to(torch.int8).numpy(), d["w_codes"])
    sw32 = torch.from_numpy(d["w_scales"])
    assert torch.equal(sw16, sw32.half())
    rowmax = y_ref.abs().max(dim=-1, keepdim=True).values
    y32 = O.w4a4_forward_fp32(qa, sa, codes, sw32, bias, g)
    assert float(((y32 - y_ref).abs() / rowmax).max()) < 1e-5
    y16 = O.w4a4_forward_fp32(qa, sa, codes, sw16, bias, g)
    assert float(((y16 - y_ref).abs() / rowmax).max()) < 0.5e-3
