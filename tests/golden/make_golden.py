"""Generate the golden fixtures in this folder from the reference's own Python code.

Run where the reference checkout is available (it is NOT needed to run the
tests; the fixtures are committed):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_golden.py /path/to/reference

Each fixture is a small ``.npz`` holding seeded inputs and the outputs the
reference code produced for them:

* ``rtn_*.npz``      RTNQuantizer.__call__ (asrq/quantizers/rtn.py:32-46): fake-quantised
                     weight, scales, zeros.
* ``linearq_*.npz``  LinearQ.dequantize_weight / forward (asrq/core/linear.py:33-66) in
                     fp32 and fp16, on packed weights built from the reference RTN output.
* ``hadamard_*.npz`` matmul_hadU (asrq/transforms/rotation/hadamard_utils.py:60-81).
* ``w4a4_composite_*.npz`` the reference's own functions composed into the W4A4 layer the reference
                     never assembles: matmul_hadU (fp32) on the activations and on the weight rows,
                     RTNQuantizer (symmetric int4, g128) on the rotated weight, then
                     activation_quantization_forward_patch around F.linear on the fake-quantised weight.
                     A float result; the integer composite of this repository must agree with it to
                     within float summation error (tests/test_oracle_golden.py states the bound).
* ``actquant_*.npz`` activation_quantization_forward_patch (asrq/quantizers/activation.py:10-33)
                     with an identity weight, i.e. round(x/s)*s; and LinearQQ.quantize_activation
                     (asrq/core/linear.py:77-82).

The packing step itself has no reference implementation (the reference never
materialises integer codes); the fixtures pin it indirectly: codes are
recovered from the reference's fake-quantised weight as round((fq-zeros)/scales),
packed, loaded into the reference LinearQ and its dequantised weight is stored.
"""
import importlib.util
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))


def load_reference(root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, root)
    om = types.ModuleType("omegaconf")
    om.DictConfig = dict
    sys.modules["omegaconf"] = om
    from asrq.core.linear import LinearQ, LinearQQ
    from asrq.quantizers.rtn import RTNQuantizer
    from asrq.quantizers.activation import activation_quantization_forward_patch
    spec = importlib.util.spec_from_file_location(
        "hadamard_utils", os.path.join(root, "asrq/transforms/rotation/hadamard_utils.py"))
    hu = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(hu)
    return LinearQ, LinearQQ, RTNQuantizer, activation_quantization_forward_patch, hu


class Cfg:
    def __init__(self, bits, group_size, symmetric):
        self.name = "rtn"
        self.bits = bits
        self.group_size = group_size
        self.symmetric = symmetric
        self.exclude_modules = []


def pack_unsigned(codes, bits):
    c = codes.to(torch.int32)
    if bits == 4:
        return (c[:, 0::2] | (c[:, 1::2] << 4)).to(torch.uint8)
    return (c[:, 0::4] | (c[:, 1::4] << 2) | (c[:, 2::4] << 4) | (c[:, 3::4] << 6)).to(torch.uint8)


@torch.no_grad()
def main(root):
    LinearQ, LinearQQ, RTNQuantizer, act_patch, hu = load_reference(root)

    # --- RTN + LinearQ ------------------------------------------------------
    cases = [
        # name, N, K, bits, g, symmetric, weight dtype, M, bias
        ("w4_g128_asym_f16", 16, 256, 4, 128, False, torch.float16, 5, True),
        ("w4_g64_asym_f32", 24, 192, 4, 64, False, torch.float32, 3, False),
        ("w2_g64_asym_f32", 16, 256, 2, 64, False, torch.float32, 4, True),
        ("w2_g128_asym_f16", 8, 384, 2, 128, False, torch.float16, 1, False),
        ("w4_g128_sym_f32", 16, 256, 4, 128, True, torch.float32, 2, True),
        ("w4_gfull_asym_f32", 8, 128, 4, -1, False, torch.float32, 2, False),
    ]
    for i, (name, n, k, bits, g, sym, wdt, m, has_bias) in enumerate(cases):
        gen = torch.Generator().manual_seed(100 + i)
        w = torch.randn(n, k, generator=gen) * 0.02
        mask = torch.rand(w.shape, generator=gen) < 0.01
        w[mask] *= 10
        w = w.to(wdt)
        lin = torch.nn.Linear(k, n, bias=False)
        lin.weight.data = w.clone()
        qz = RTNQuantizer(lin, "l", Cfg(bits, g, sym))
        scales, zeros = qz()
        fq = lin.weight.data.clone()
        np.savez(os.path.join(HERE, f"rtn_{name}.npz"),
                 w=w.float().numpy(), w_is_f16=np.array(wdt == torch.float16),
                 bits=bits, group_size=g, symmetric=sym,
                 fake_quant=fq.float().numpy(),
                 scales=scales.squeeze(-1).float().numpy(),
                 zeros=zeros.squeeze(-1).float().numpy())

        # codes recovered from the reference's own output, then through LinearQ
        geff = k if g == -1 else g
        fqg = fq.reshape(n, k // geff, geff)
        if sym:
            codes = torch.round(fqg / scales) + 2 ** (bits - 1)
            z_lq = (-(2 ** (bits - 1)) * scales).squeeze(-1)
        else:
            codes = torch.round((fqg - zeros) / scales)
            z_lq = zeros.squeeze(-1)
        codes = codes.reshape(n, k)
        packed = pack_unsigned(codes, bits)
        lq = LinearQ(k, n, bits, geff, bias=has_bias)
        lq.load_quantized_params(scales.squeeze(-1).half(), z_lq.half(), packed)
        if has_bias:
            lq.bias = (torch.randn(n, generator=gen) * 0.02).half()
        x = torch.randn(m, k, generator=gen)
        x16 = x.half()
        out = dict(
            bits=bits, group_size=geff, in_features=k, out_features=n,
            weight=packed.numpy(), scales=lq.scales.numpy().view(np.uint16),
            zeros=lq.zeros.numpy().view(np.uint16),
            x=x16.numpy().view(np.uint16),
            w_deq_f32=lq.dequantize_weight("cpu", torch.float32).numpy(),
            w_deq_f16=lq.dequantize_weight("cpu", torch.float16).numpy().view(np.uint16),
            y_f32=lq.forward(x16.float()).numpy() if not has_bias else None,
        )
        if has_bias:
            out["bias"] = lq.bias.numpy().view(np.uint16)
            # reference forward adds the fp16 bias buffer in place
            out["y_f32"] = lq.forward(x16.float()).numpy()
        out["y_f16"] = lq.forward(x16).numpy().view(np.uint16)
        out = {k_: v for k_, v in out.items() if v is not None}
        np.savez(os.path.join(HERE, f"linearq_{name}.npz"), **out)

    # --- Hadamard -----------------------------------------------------------
    for n in (64, 1024, 4096):
        gen = torch.Generator().manual_seed(200 + n)
        x = torch.randn(3, n, generator=gen)
        x[:, 5] *= 20
        np.savez(os.path.join(HERE, f"hadamard_{n}.npz"),
                 x=x.numpy(), y_f32=hu.matmul_hadU(x).numpy(),
                 y_f16=hu.matmul_hadU(x.half()).numpy().view(np.uint16))

    # --- activation quantisation --------------------------------------------
    gen = torch.Generator().manual_seed(300)
    k = 256
    x = torch.randn(2, 6, k, generator=gen)
    x[:, :, 7] *= 20
    x[0, 3] = 0.0  # all-zero token exercises the 1e-3 guard
    lin = torch.nn.Linear(k, k, bias=False)
    lin.weight.data = torch.eye(k)
    act_patch(lin, 4, "l")
    with torch.no_grad():
        y = lin(x)
    qq = LinearQQ(k, 8, 4, 4, 128, bias=False)
    x2 = x.reshape(-1, k)[[0, 1, 2, 4, 5]]  # quantize_activation has no zero guard
    q2, s2 = qq.quantize_activation(x2)
    np.savez(os.path.join(HERE, "actquant_4bit.npz"),
             x=x.numpy(), fake_quant=y.numpy(),
             x2=x2.numpy(), q2=q2.numpy(), s2=s2.numpy())
    # --- W4A4 composite out of the reference's own pieces --------------------
    for (m, k, n, g) in ((24, 1024, 128, 128), (9, 4096, 64, 128)):
        gen = torch.Generator().manual_seed(400 + k)
        # heavy-tailed activations with outlier channels, like the W4A4 benchmark configuration
        z = torch.randn(m, k, generator=gen)
        c = torch.zeros(m, k)
        for _ in range(4):
            c += torch.randn(m, k, generator=gen) ** 2
        x = z / torch.sqrt(c / 4)
        x[:, torch.randperm(k, generator=gen)[:8]] *= 20
        x = x.half()
        w = torch.randn(n, k, generator=gen) * 0.02
        bias = (torch.randn(n, generator=gen) * 0.02).half()
        lin = torch.nn.Linear(k, n, bias=True)
        lin.weight.data = hu.matmul_hadU(w.clone())           # offline fold of the rotation into the weight
        lin.bias.data = bias.float()
        qz = RTNQuantizer(lin, "l", Cfg(4, g, True))          # fake-quantises lin.weight in place
        scales, _ = qz()
        act_patch(lin, 4, "l")                                # forward = fake act-quant + F.linear
        with torch.no_grad():
            v = hu.matmul_hadU(x.float())                     # online rotation, fp32
            y = lin(v)
        # the reference's fake-quantised weight, stored as the integer codes it implies (codes * scales
        # reproduces it bit for bit, checked here) to keep the fixture small
        fq = lin.weight.data.reshape(n, k // g, g)
        w_codes = torch.round(fq / scales)
        assert torch.equal(w_codes * scales, fq) and float(w_codes.abs().max()) <= 7
        np.savez_compressed(os.path.join(HERE, f"w4a4_composite_k{k}.npz"),
                            x=x.numpy().view(np.uint16), w=w.numpy(), bias=bias.numpy().view(np.uint16), group_size=g,
                            w_codes=w_codes.reshape(n, k).to(torch.int8).numpy(), w_scales=scales.squeeze(-1).numpy(),
                            v=v.numpy(), y=y.numpy())
    print("fixtures written to", HERE)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_golden.py <path to a checkout of the reference (wakandaai/asrq)>")
    main(sys.argv[1])
