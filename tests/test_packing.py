"""Host-side packer (product code) against the oracle and the reference-generated fixtures."""
import glob
import os

import numpy as np
import pytest
import torch

from asrq_b200 import packing as P
from oracle import linearq_oracle as O

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _names(prefix):
    return sorted(os.path.basename(p)[len(prefix):-4] for p in glob.glob(os.path.join(GOLDEN, prefix + "*.npz")))


@pytest.mark.parametrize("name", _names("rtn_"))
def test_rtn_quantize_matches_reference_grid(name):
    d = np.load(os.path.join(GOLDEN, f"rtn_{name}.npz"))
    w = torch.from_numpy(d["w"])
    if bool(d["w_is_f16"]):
        w = w.half()
    bits, g, sym = int(d["bits"]), int(d["group_size"]), bool(d["symmetric"])
    codes, scales, zeros = P.rtn_quantize(w, bits, g, sym)
    assert np.array_equal(scales.float().numpy(), d["scales"])
    assert np.array_equal(zeros.float().numpy(), d["zeros"])
    ocodes, _, _, fq = O.rtn_codes(w, bits, g, sym)
    assert torch.equal(codes, ocodes)
    # the quantizer-output route gives the same codes
    rec = P.codes_from_fake_quant(torch.from_numpy(d["fake_quant"]).to(w.dtype), scales, zeros, bits, g, sym)
    assert torch.equal(rec, codes)


@pytest.mark.parametrize("bits", [2, 4])
def test_pack_codes_bit_exact(bits):
    g = torch.Generator().manual_seed(bits)
    codes = torch.randint(0, 2 ** bits, (33, 128), generator=g)
    packed = P.pack_codes(codes, bits)
    assert packed.dtype == torch.uint8 and packed.shape == (33, 128 * bits // 8)
    assert torch.equal(packed, O.pack_codes(codes, bits))
    assert torch.equal(O.unpack_codes(packed, bits, 128).long(), codes)
    with pytest.raises(ValueError):
        P.pack_codes(codes + 2 ** bits, bits)


@pytest.mark.parametrize("name", _names("linearq_"))
def test_packed_fixture_bytes(name):
    """Packing the codes held by the fixture reproduces the bytes the reference LinearQ consumed."""
    d = np.load(os.path.join(GOLDEN, f"linearq_{name}.npz"))
    bits, k = int(d["bits"]), int(d["in_features"])
    weight = torch.from_numpy(d["weight"])
    codes = O.unpack_codes(weight, bits, k)
    assert torch.equal(P.pack_codes(codes, bits), weight)


def test_pack_linearq_symmetric_shift():
    g = torch.Generator().manual_seed(5)
    w = torch.randn(16, 256, generator=g) * 0.02
    codes, scales, zeros = P.rtn_quantize(w, 4, 128, True)
    weight, s16, z16 = P.pack_linearq(codes, scales, zeros, 4, True)
    wd = O.dequantize_weight(weight, s16, z16, 4, 128, 256, torch.float32)
    fq = (codes.float().reshape(16, 2, 128) * s16.float()[:, :, None]).reshape(16, 256)
    np.testing.assert_allclose(wd.numpy(), fq.numpy(), atol=2e-4)


def test_pack_signed_and_w4a4_match_oracle():
    g = torch.Generator().manual_seed(6)
    c = torch.randint(-8, 8, (9, 64), generator=g)
    assert torch.equal(P.pack_signed_int4(c), O.pack_signed_int4(c))
    w = torch.randn(32, 256, generator=g) * 0.02
    for had in (True, False):
        pw, sw = P.pack_w4a4(w, 128, had)
        ocodes, osw, opw = O.prepare_w4a4_weight(w, 128, had)
        assert torch.equal(pw, opw) and torch.equal(sw, osw)
    x = torch.randn(3, 256, generator=g)
    assert torch.equal(P.hadamard_pow2(x), O.hadamard_pow2(x))
