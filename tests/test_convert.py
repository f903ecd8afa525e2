"""Model wiring on the CPU: layers are swapped, packed as the reference grid says, and serialise
with the reference's LinearQ key names (asrq/core/linear.py:16-25)."""
import torch
import torch.nn as nn

import asrq_b200
from asrq_b200 import convert as C
from asrq_b200 import packing
from oracle import linearq_oracle as O


class Block(nn.Module):
    def __init__(self, d=256, ff=512, vocab=96):
        super().__init__()
        self.q_proj = nn.Linear(d, d)
        self.k_proj = nn.Linear(d, d, bias=False)
        self.v_proj = nn.Linear(d, d)
        self.fc1 = nn.Linear(d, ff)
        self.fc2 = nn.Linear(ff, d)
        self.odd = nn.Linear(100, 8)          # in_features not a multiple of the group size: stays fp
        self.proj_out = nn.Linear(d, vocab, bias=False)


def test_convert_swaps_layers_and_matches_rtn():
    torch.manual_seed(0)
    m = Block()
    ref_w = {n: p.detach().clone() for n, p in m.named_parameters()}
    C.convert(m, bits=4, group_size=128, skip=("proj_out",))
    assert isinstance(m.q_proj, asrq_b200.LinearQ) and isinstance(m.fc2, asrq_b200.LinearQ)
    assert type(m.proj_out) is nn.Linear and type(m.odd) is nn.Linear
    sd = m.state_dict()
    assert {"q_proj.weight", "q_proj.scales", "q_proj.zeros", "q_proj.bias", "k_proj.weight", "k_proj.scales",
            "k_proj.zeros"} <= set(sd) and "k_proj.bias" not in sd
    assert sd["fc1.weight"].dtype == torch.uint8 and sd["fc1.weight"].shape == (512, 128)
    # the packed layer dequantises to the reference's fake-quantised weight (rtn.py:39-46)
    w = ref_w["fc1.weight"]
    codes, scales, zeros, fq = O.rtn_codes(w, 4, 128, False)
    assert torch.equal(O.unpack_codes(m.fc1.weight, 4, 256).to(torch.int32), codes.to(torch.int32))
    got = m.fc1.dequantize_weight(dtype=torch.float32)
    want = codes.float() * scales.half().float().repeat_interleave(128, 1) + zeros.half().float().repeat_interleave(128, 1)
    assert torch.equal(got, want)
    assert torch.equal(m.fc1.bias, ref_w["fc1.bias"].half())


def test_convert_from_reference_quantizer_output():
    """The ModelQ.quantize flow: weights already fake-quantised in place, (scales, zeros) per layer name."""
    torch.manual_seed(1)
    m = Block()
    qparams = {}
    direct = {}
    for name in ("q_proj", "fc2"):
        lin = getattr(m, name)
        codes, scales, zeros, fq = O.rtn_codes(lin.weight.detach(), 2, 64, False)
        direct[name] = codes
        lin.weight.data.copy_(fq)                         # what the quantizer leaves in the module
        qparams[name] = (scales.unsqueeze(-1), zeros.unsqueeze(-1))
    C.convert(m, bits=2, group_size=64, qparams=qparams, select=lambda n, l: n in qparams)
    for name in qparams:
        lq = getattr(m, name)
        assert lq.bits == 2 and lq.group_size == 64
        assert torch.equal(O.unpack_codes(lq.weight, 2, lq.in_features).to(torch.int32), direct[name].to(torch.int32))
    assert type(m.fc1) is nn.Linear


def test_fused_parts_keep_their_state_dict_entries():
    torch.manual_seed(2)
    m = Block()
    C.convert(m, bits=4, group_size=128, skip=("proj_out",))
    # k_proj has no bias (as in Whisper's attention): its rows of the fused bias are zeros
    qkv = C.FusedLinearQ([m.q_proj, m.k_proj, m.v_proj])._fuse()
    assert qkv.out_features == 768 and torch.equal(qkv.bias[:256], m.q_proj.bias)
    assert int(qkv.bias[256:512].abs().sum()) == 0 and torch.equal(qkv.bias[512:], m.v_proj.bias)
    f = C.FusedLinearQ([m.q_proj, m.v_proj])
    keys = set(f.state_dict())
    assert keys == {f"parts.{i}.{b}" for i in (0, 1) for b in ("weight", "scales", "zeros", "bias")}
    fused = f._fuse()
    assert fused.out_features == 512 and torch.equal(fused.weight[256:], m.v_proj.weight)
    assert set(f.state_dict()) == keys                     # the fused copy is not serialised
    m.v_proj.scales.mul_(2)                                # in-place edit of a part refreshes the copy
    assert torch.equal(f._fuse().scales[256:], m.v_proj.scales)
