"""W4A4 parity on the GPU through the C ABI.

Bit-exact: packed activation codes, per-token scales, int32 group accumulators.
Within 2e-3 * ||row||_inf of the fp32 CPU composite: the fp16 output.
"""
import os

import numpy as np
import pytest
import torch

import asrq_b200
from asrq_b200 import _lib
from oracle import linearq_oracle as O
from tests.gpu_util import DEV, assert_close_rows, bf16_half_ulp, check_canary, lib_option, padded

pytestmark = pytest.mark.gpu
GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def _quant_gpu(x, hadamard, dtype=torch.float16):
    xd = x.to(dtype).to(DEV).contiguous()
    m, k = xd.shape
    qa = torch.empty(m, k // 2, dtype=torch.uint8, device=DEV)
    sa = torch.empty(m, dtype=torch.float32, device=DEV)
    _lib.call("asrq_hadamard_quant_int4", xd.data_ptr(), qa.data_ptr(), sa.data_ptr(), m, k, int(hadamard),
              _lib.F16 if dtype == torch.float16 else _lib.BF16, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    return qa.cpu(), sa.cpu()


@pytest.mark.parametrize("k", [256, 512, 1024, 2048, 4096])
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_hadamard_quant_bit_exact(k, dtype):
    gen = torch.Generator().manual_seed(k)
    x = torch.randn(37, k, generator=gen)
    x[:, 3] *= 20
    x[5] = 0.0                       # all-zero token -> scale 1e-3, codes 0
    x[6] = 65504.0 if dtype == torch.float16 else 1e30
    x = x.to(dtype)
    qa, sa = _quant_gpu(x, True, dtype)
    q_ref, s_ref, p_ref = O.hadamard_quant_int4(x, True)
    assert torch.equal(sa, s_ref), "per-token scales differ"
    assert torch.equal(qa, p_ref), "packed activation codes differ"
    assert float(sa[5]) == pytest.approx(1e-3) and int(qa[5].max()) == 0


@pytest.mark.parametrize("k", [8, 264, 1280, 5120])
def test_quant_without_rotation_bit_exact(k):
    gen = torch.Generator().manual_seed(k)
    x = (torch.randn(19, k, generator=gen) * 3).half()
    x[2] = 0.0
    qa, sa = _quant_gpu(x, False)
    q_ref, s_ref, p_ref = O.hadamard_quant_int4(x, False)
    assert torch.equal(sa, s_ref) and torch.equal(qa, p_ref)


def test_quant_matches_reference_fixture():
    """activation.py:26-28 evaluated by the reference itself (fp32 input fixture, fed as fp16-exact values)."""
    d = np.load(os.path.join(GOLDEN, "actquant_4bit.npz"))
    x = torch.from_numpy(d["x"]).reshape(-1, 256).half()   # fixture values rounded to fp16 ...
    qa, sa = _quant_gpu(x, False)
    q, s = O.act_quant_sym(x.float(), 4)                   # ... and the pinned formula on the same values
    assert torch.equal(O.unpack_signed_int4(qa), q) and torch.equal(sa, s.reshape(-1))


@pytest.mark.parametrize("k,had", [(4096, True), (1024, True), (1280, False)])
def test_int8_operand_output_matches_packed_codes(k, had):
    """asrq_hadamard_quant_int8 writes 16 * code per byte, the same codes as the packed entry point."""
    gen = torch.Generator().manual_seed(k + 1)
    x = (torch.randn(70, k, generator=gen) * 2).half()
    qa, sa = _quant_gpu(x, had)
    xd = x.to(DEV)
    a8 = torch.empty(70, k, dtype=torch.uint8, device=DEV)
    s8 = torch.empty(70, dtype=torch.float32, device=DEV)
    _lib.call("asrq_hadamard_quant_int8", xd.data_ptr(), a8.data_ptr(), s8.data_ptr(), 70, k, int(had), _lib.F16,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    codes = O.unpack_signed_int4(qa).to(torch.int32)
    assert torch.equal(a8.cpu().view(torch.int8).to(torch.int32), codes * 16)
    assert torch.equal(s8.cpu(), sa)
    # and the weight-side expansion
    w = torch.randint(-8, 8, (128, k), generator=gen)
    pw = O.pack_signed_int4(w).to(DEV)
    w8 = torch.empty(128, k, dtype=torch.uint8, device=DEV)
    _lib.call("asrq_w4a4_prepare_weight", pw.data_ptr(), w8.data_ptr(), 128, k, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(w8.cpu().view(torch.int8).to(torch.int64), w * 16)


@pytest.mark.parametrize("k,had", [(4096, True), (512, True), (1280, False)])
def test_f8_operand_output_matches_packed_codes(k, had):
    """asrq_hadamard_quant_f8 writes the code itself as an e4m3 byte, the same codes as the packed entry point."""
    gen = torch.Generator().manual_seed(k + 2)
    x = (torch.randn(70, k, generator=gen) * 2).half()
    qa, sa = _quant_gpu(x, had)
    xd = x.to(DEV)
    a8 = torch.empty(70, k, dtype=torch.uint8, device=DEV)
    s8 = torch.empty(70, dtype=torch.float32, device=DEV)
    _lib.call("asrq_hadamard_quant_f8", xd.data_ptr(), a8.data_ptr(), s8.data_ptr(), 70, k, int(had), _lib.F16,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    codes = O.unpack_signed_int4(qa).to(torch.float32)
    assert torch.equal(a8.cpu().view(torch.float8_e4m3fn).to(torch.float32), codes)
    assert torch.equal(s8.cpu(), sa)
    w = torch.randint(-8, 8, (128, k), generator=gen)   # every code including -8
    pw = O.pack_signed_int4(w).to(DEV)
    w8 = torch.empty(128, k, dtype=torch.uint8, device=DEV)
    _lib.call("asrq_w4a4_prepare_weight_f8", pw.data_ptr(), w8.data_ptr(), 128, k, torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    assert torch.equal(w8.cpu().view(torch.float8_e4m3fn).to(torch.float32), w.to(torch.float32))


def test_hadamard_rejects_bad_k():
    x = torch.zeros(4, 768, dtype=torch.float16, device=DEV)
    qa = torch.empty(4, 384, dtype=torch.uint8, device=DEV)
    sa = torch.empty(4, dtype=torch.float32, device=DEV)
    with pytest.raises(_lib.AsrqError) as e:
        _lib.call("asrq_hadamard_quant_int4", x.data_ptr(), qa.data_ptr(), sa.data_ptr(), 4, 768, 1, 0, None)
    assert e.value.code == -2


def _w4a4_case(m, k, n, g, seed, bias=True, outliers=True):
    gen = torch.Generator().manual_seed(seed)
    x = torch.randn(m, k, generator=gen)
    if outliers:
        x[:, torch.randperm(k, generator=gen)[:8]] *= 20
    x = x.half()
    w = torch.randn(n, k, generator=gen) * 0.02
    b = (torch.randn(n, generator=gen) * 0.02).half() if bias else None
    return x, w, b


@pytest.mark.parametrize("m,k,n,g,bias", [
    (1, 256, 128, 128, False),
    (64, 1024, 128, 128, True),
    (100, 512, 256, 128, True),      # ragged M
    (333, 4096, 1024, 128, True),    # config-2 widths
    (257, 2048, 384, 128, False),
    (48, 1024, 64, 256, True),       # wider group, narrow N: register-tile kernel
])
def test_w4a4_gemm_exact_accumulators_and_output(m, k, n, g, bias):
    x, w, b = _w4a4_case(m, k, n, g, seed=m + k, bias=bias)
    had = (k & (k - 1)) == 0
    qa_ref, sa_ref, pa_ref = O.hadamard_quant_int4(x, had)
    codes, sw, pw = O.prepare_w4a4_weight(w, g, had)
    acc_ref = O.int4_group_accumulators(qa_ref, codes, g)
    y_ref = O.w4a4_forward_fp32(qa_ref, sa_ref, codes, sw, b, g)

    lq = asrq_b200.LinearQQ(k, n, 4, 4, g, bias=bias, hadamard=had).to(DEV)
    pw2, sw2 = asrq_b200.pack_w4a4(w, g, had)
    assert torch.equal(pw2, pw) and torch.equal(sw2, sw)
    lq.load_quantized_params(sw2, torch.zeros_like(sw2), pw2)
    if bias:
        lq.bias = b.to(DEV)
    acc = torch.full((m, n, k // g), -12345, dtype=torch.int32, device=DEV)
    y = lq(x.to(DEV), acc_dump=acc)
    asrq_b200.check_status()
    assert torch.equal(acc.cpu(), acc_ref), "int32 group accumulators differ"
    assert_close_rows(y, y_ref, what=f"w4a4 m{m} k{k} n{n}")
    # without the dump, through the packed two-call sequence and through the one-call entry point:
    # the same codes and the same int32 sums give the same output bits
    y2 = lq(x.to(DEV))
    assert torch.equal(y2, y)
    y3 = lq(x.to(DEV), two_call=True)
    assert torch.equal(y3, y)
    # the other 8-bit operand family (int8 / kind::i8 when the default is f8 / kind::f8f6f4): same sums, same bits
    lq.operand = "int8" if lq.operand == "f8" else "f8"
    acc5 = torch.full_like(acc, -1)
    y5 = lq(x.to(DEV), acc_dump=acc5)
    torch.cuda.synchronize()
    assert torch.equal(acc5.cpu(), acc_ref) and torch.equal(y5, y)
    if n % 128 == 0 and g % 128 == 0:
        xd = x.to(DEV)
        y4 = torch.empty(m, n, dtype=torch.float16, device=DEV)
        ws = torch.zeros(_lib.workspace_bytes(_lib.WS_W4A4_GEMM, m, n, k), dtype=torch.uint8, device=DEV)
        _lib.call("asrq_w4a4_linear", xd.data_ptr(), lq.weight.data_ptr(), lq.scales.data_ptr(),
                  None if lq.bias is None else lq.bias.data_ptr(), y4.data_ptr(), m, n, k, g, int(had), _lib.F16,
                  ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
        _lib.call("asrq_check_status", ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
        assert torch.equal(y4, y)
    qf, sf = lq.quantize_activation(x.to(DEV))
    assert torch.equal(qf.cpu(), qa_ref.float()) and torch.equal(sf.cpu().reshape(-1), sa_ref)


@pytest.mark.parametrize("m,k,n", [(333, 4096, 1024), (100, 512, 256), (700, 1024, 512)])
def test_w4a4_cta_pair_variant(m, k, n):
    """The opt-in CTA-pair kernel (tcgen05 cta_group::2): the same integer group sums and output bits."""
    g = 128
    x, w, b = _w4a4_case(m, k, n, g, seed=m + k + 1, bias=True)
    qa_ref, sa_ref, _ = O.hadamard_quant_int4(x, True)
    codes, sw, _ = O.prepare_w4a4_weight(w, g, True)
    acc_ref = O.int4_group_accumulators(qa_ref, codes, g)
    lq = asrq_b200.LinearQQ(k, n, 4, 4, g, bias=True, hadamard=True).to(DEV)
    pw2, sw2 = asrq_b200.pack_w4a4(w, g, True)
    lq.load_quantized_params(sw2, torch.zeros_like(sw2), pw2)
    lq.bias = b.to(DEV)
    y_single = lq(x.to(DEV))
    with lib_option("w4a4_pair", 1):
        acc = torch.full((m, n, k // g), -12345, dtype=torch.int32, device=DEV)
        y_pair = lq(x.to(DEV), acc_dump=acc)
        asrq_b200.check_status()
        assert torch.equal(acc.cpu(), acc_ref), "int32 group accumulators differ (pair kernel)"
        assert torch.equal(y_pair, y_single)
        lq.operand = "int8" if lq.operand == "f8" else "f8"
        assert torch.equal(lq(x.to(DEV)), y_single)


def test_w4a4_tracks_unquantised_product():
    """End-to-end sanity at config-2 widths: the rotation cancels and 4x4-bit error stays moderate."""
    x, w, b = _w4a4_case(128, 4096, 1024, 128, seed=9, bias=False)
    lq = asrq_b200.LinearQQ(4096, 1024, 4, 4, 128, bias=False).to(DEV)
    pw, sw = asrq_b200.pack_w4a4(w, 128, True)
    lq.load_quantized_params(sw, torch.zeros_like(sw), pw)
    y = lq(x.to(DEV)).float().cpu()
    y_true = x.float() @ w.t()
    rel = float((y - y_true).norm() / y_true.norm())
    assert rel < 0.25, rel


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_config2_full_size(dtype):
    """The W4A4 benchmark configuration at its own size: M=6000 tokens, K=4096, N=1024, g128, Student-t(4)
    activations with 8 outlier channels x20.  Heavy tails are where the division-free quantiser takes its
    exact-division branch.  Codes and scales bit-exact for every token; int32 group sums bit-exact and
    output within the bar on a sample of 640 rows."""
    c = O.make_c2(seed=0)
    x = c["x"].to(dtype)
    m, k = x.shape
    n, g = c["w_fp"].shape[0], c["group_size"]
    qa_ref, sa_ref, pa_ref = O.hadamard_quant_int4(x, True)
    codes, sw, pw = O.prepare_w4a4_weight(c["w_fp"], g, True)
    lq = asrq_b200.LinearQQ(k, n, 4, 4, g, bias=True, hadamard=True).to(DEV)
    lq.load_quantized_params(sw, torch.zeros_like(sw), pw)
    lq.bias = c["bias"].to(DEV)
    xd = x.to(DEV)
    qa, sa = _quant_gpu(x, True, dtype)
    assert torch.equal(sa, sa_ref), "per-token scales differ"
    assert torch.equal(qa, pa_ref), "packed activation codes differ"
    gen = torch.Generator().manual_seed(1)
    rows = torch.unique(torch.cat([torch.arange(0, 64), torch.arange(m - 64, m),
                                   torch.randint(0, m, (512,), generator=gen)]))
    acc = padded((m, n, k // g), torch.int32)
    y = lq(xd, acc_dump=acc)
    asrq_b200.check_status()
    check_canary(acc, "acc_dump")
    acc_ref = O.int4_group_accumulators(qa_ref[rows], codes, g)
    assert torch.equal(acc[rows.to(DEV)].cpu(), acc_ref), "int32 group accumulators differ"
    y_ref = O.w4a4_forward_fp32(qa_ref[rows], sa_ref[rows], codes, sw, c["bias"], g)
    extra = bf16_half_ulp(y_ref) if dtype == torch.bfloat16 else None
    assert_close_rows(y[rows.to(DEV)], y_ref, extra=extra, what=f"W4A4 M=6000 {dtype}")
    assert torch.equal(lq(xd), y)   # the timed path (no dump) gives the same bits


@pytest.mark.parametrize("g", [256, 512, 1024])
@pytest.mark.parametrize("family", ["f8", "int8"])
def test_tensor_core_group_sums_exact_for_wide_groups(g, family):
    """Wide weight groups on the tcgen05 kernel with the largest possible sums: all codes -8 x -8
    (sum 64 * g) and alternating +7 / -8.  The f8 family relies on the tensor core accumulating
    kind::f8f6f4 products exactly in fp32 up to 2^16; both families must dump the exact integers."""
    m, n, k = 128, 128, 2048
    gen = torch.Generator().manual_seed(g)
    qa = torch.full((m, k), -8, dtype=torch.int64)
    qw = torch.full((n, k), -8, dtype=torch.int64)
    qa[1::2] = torch.where(torch.arange(k) % 2 == 0, 7, -8)
    qw[1::2] = 7
    qa[m // 2:] = torch.randint(-8, 8, (m - m // 2, k), generator=gen)
    qw[n // 2:] = torch.randint(-8, 8, (n - n // 2, k), generator=gen)
    acc_ref = torch.einsum("mgk,ngk->mng", qa.reshape(m, -1, g), qw.reshape(n, -1, g)).to(torch.int32)
    sw = torch.ones(n, k // g, dtype=torch.float16)
    sa = torch.ones(m, dtype=torch.float32)
    pa, pw = O.pack_signed_int4(qa).to(DEV), O.pack_signed_int4(qw).to(DEV)
    a8 = torch.empty(m, k, dtype=torch.uint8, device=DEV)
    w8 = torch.empty(n, k, dtype=torch.uint8, device=DEV)
    st = torch.cuda.current_stream().cuda_stream
    prep = "asrq_w4a4_prepare_weight_f8" if family == "f8" else "asrq_w4a4_prepare_weight"
    _lib.call(prep, pw.data_ptr(), w8.data_ptr(), n, k, st)     # the same nibble -> operand expansion serves both sides
    _lib.call(prep, pa.data_ptr(), a8.data_ptr(), m, k, st)
    y = torch.empty(m, n, dtype=torch.float16, device=DEV)
    acc = padded((m, n, k // g), torch.int32)
    ws = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    _lib.call(f"asrq_w4a4_gemm_{family}", a8.data_ptr(), sa.to(DEV).data_ptr(), w8.data_ptr(), sw.to(DEV).data_ptr(),
              None, y.data_ptr(), acc.data_ptr(), m, n, k, g, _lib.F16, ws.data_ptr(), ws.numel(), st)
    _lib.call("asrq_check_status", ws.data_ptr(), st)
    check_canary(acc, "acc_dump")
    assert torch.equal(acc.cpu(), acc_ref), f"group sums differ for g={g} ({family})"


@pytest.mark.parametrize("k", [1024, 4096])
def test_w4a4_against_reference_composed_fixture(k):
    """The layer assembled from the reference's own functions (tests/golden/make_golden.py: matmul_hadU,
    RTNQuantizer, the activation fake-quant patch, F.linear): output within 2e-3 of the row maximum."""
    d = np.load(os.path.join(GOLDEN, f"w4a4_composite_k{k}.npz"))
    x = torch.from_numpy(d["x"].view(np.float16).copy())
    w, g = torch.from_numpy(d["w"]), int(d["group_size"])
    bias = torch.from_numpy(d["bias"].view(np.float16).copy())
    n = w.shape[0]
    pw, sw = asrq_b200.pack_w4a4(w, g, True)
    assert np.array_equal(O.unpack_signed_int4(pw).numpy(), d["w_codes"])
    lq = asrq_b200.LinearQQ(k, n, 4, 4, g, bias=True, hadamard=True).to(DEV)
    lq.load_quantized_params(sw, torch.zeros_like(sw), pw)
    lq.bias = bias.to(DEV)
    y = lq(x.to(DEV))
    assert_close_rows(y, torch.from_numpy(d["y"]), what=f"reference-composed W4A4 K={k}")
    xr = x.repeat(8, 1)   # 72 / 192 tokens: the tensor-core kernel instead of the register-tile one
    y2 = lq(xr.to(DEV))
    assert_close_rows(y2, torch.from_numpy(d["y"]).repeat(8, 1), what=f"reference-composed W4A4 K={k}, tcgen05 path")


def test_w4a4_gemm_rejects_bad_group_size():
    p = torch.zeros(4096, dtype=torch.uint8, device=DEV)
    for gs in (0, -128):
        with pytest.raises(_lib.AsrqError) as e:
            _lib.call("asrq_w4a4_gemm", p.data_ptr(), p.data_ptr(), p.data_ptr(), p.data_ptr(), None, p.data_ptr(), None,
                      8, 64, 128, gs, _lib.F16, p.data_ptr(), p.numel(), None)
        assert e.value.code == -2
