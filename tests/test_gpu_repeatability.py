"""Every kernel family, launched back to back in chains of dependent layers, gives the same bits every time.

The kernels hand shared-memory slots, tensor-memory buffers and split-K partial sums between warps, CTAs and
consecutive launches through barriers and counters; a hand-over that is wrong only in a narrow timing window shows up
as a result that differs between repetitions (the pair kernel's packed-weight ring did, once in some hundred chains).
Parity with the oracle is tested elsewhere; this file only asks for the same answer every time."""
import pytest
import torch

import asrq_b200
from asrq_b200 import packing
from asrq_b200.linear import LinearQ, LinearQQ
from tests.gpu_util import DEV

pytestmark = pytest.mark.gpu


def _gen():
    return torch.Generator(device=DEV).manual_seed(0)


def _lq(gen, n, k, bits=4, g=128, bias=True):
    w = torch.randn(n, k, generator=gen, device=DEV) * 0.02
    codes, scales, zeros = packing.rtn_quantize(w.half(), bits, g, False)
    weight, s16, z16 = packing.pack_linearq(codes, scales, zeros, bits, False)
    m = LinearQ(k, n, bits, g, bias=bias).to(DEV)
    m.load_quantized_params(s16, z16, weight)
    if bias:
        m.bias = (torch.randn(n, generator=gen, device=DEV) * 0.02).half()
    return m


def _qq(gen, n, k, g=128):
    w = torch.randn(n, k, generator=gen, device=DEV) * 0.02
    weight, scales = packing.pack_w4a4_cuda(w, g, True)
    m = LinearQQ(k, n, 4, 4, g, bias=False, hadamard=True).to(DEV)
    m.load_quantized_params(scales, torch.zeros_like(scales), weight)
    return m


def _repeat(layers, x, reps):
    def run():
        outs, h = [], x
        for layer in layers:
            h = layer(h)
            outs.append(h)
        return outs
    ref = [t.clone() for t in run()]
    bad = sum(not all(torch.equal(a, b) for a, b in zip(ref, run())) for _ in range(reps))
    torch.cuda.synchronize()
    asrq_b200.check_status()
    assert bad == 0, f"{bad} of {reps} repetitions differ from the first"


@pytest.mark.parametrize("m,widths,bits,reps", [
    (200, (1280, 1280, 5120, 1280), 4, 200),     # one-CTA prefill kernel with split K
    (1500, (1280, 1152, 1280), 4, 150),          # one-CTA prefill kernel, N % 256 != 0
    (6000, (1280, 3840, 1280, 5120, 1280), 4, 150),  # CTA pairs, encoder-sized
    (2560, (2048, 4096, 2048), 2, 100),          # CTA pairs, 2-bit
    (1, (1280, 3840, 1280, 5120, 1280), 4, 200),  # decode kernels
    (8, (1280, 3840, 1280, 5120, 1280), 4, 200),
    (16, (1280, 3840, 1280, 5120, 1280), 4, 200),
    (32, (1280, 3840, 1280, 5120, 1280), 4, 200),  # chain-oriented tensor-core kernel, split K through the workspace
    (64, (1280, 3840, 1280, 5120, 1280), 4, 200),
    (64, (6144, 2048, 12288), 4, 150),
])
def test_w4a16_chain_repeats(m, widths, bits, reps):
    gen = _gen()
    layers = [_lq(gen, widths[i + 1], widths[i], bits=bits) for i in range(len(widths) - 1)]
    x = torch.randn(m, widths[0], generator=gen, device=DEV).half()
    _repeat(layers, x, reps)


@pytest.mark.parametrize("m,widths,reps", [(6000, (4096, 1024, 4096), 100), (16000, (1024, 4096, 1024), 50)])
def test_w4a4_chain_repeats(m, widths, reps):
    gen = _gen()
    layers = [_qq(gen, widths[i + 1], widths[i]) for i in range(len(widths) - 1)]
    x = torch.randn(m, widths[0], generator=gen, device=DEV).half()
    _repeat(layers, x, reps)
