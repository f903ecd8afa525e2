"""Helpers shared by the GPU parity tests."""
import numpy as np
import torch

import asrq_b200
from asrq_b200 import _lib
from oracle import linearq_oracle as O

DEV = "cuda:0"


class lib_option:
    """``with lib_option("tc_pair", 1): ...`` sets a switch of the library (asrq_set_option) and puts
    the previous value back afterwards."""

    def __init__(self, name, value):
        self.name, self.value = name, value

    def __enter__(self):
        self.old = _lib.get_option(self.name)
        _lib.set_option(self.name, self.value)
        return self

    def __exit__(self, *exc):
        _lib.set_option(self.name, self.old)
        return False


CANARY = 0xA5


def padded(shape, dtype, device=DEV, pad_bytes=4096, fill=None):
    """A tensor of ``shape`` carved out of a larger allocation whose leading and trailing ``pad_bytes``
    hold a canary pattern; :func:`check_canary` verifies that a kernel wrote neither (the stand-in
    for a memory checker on machines where none may run)."""
    n = 1
    for s in shape:
        n *= s
    nbytes = n * torch.empty(0, dtype=dtype).element_size()
    raw = torch.full((pad_bytes + nbytes + pad_bytes,), CANARY, dtype=torch.uint8, device=device)
    t = raw[pad_bytes:pad_bytes + nbytes].view(dtype).reshape(shape)
    if fill is not None:
        t.fill_(fill)
    t._canary_raw = raw  # keeps the allocation alive and findable
    t._canary_pad = pad_bytes
    return t


def check_canary(t, what=""):
    raw, pad = t._canary_raw, t._canary_pad
    head, tail = raw[:pad], raw[raw.numel() - pad:]
    assert bool((head == CANARY).all()), f"{what}: bytes BEFORE the buffer were overwritten"
    assert bool((tail == CANARY).all()), f"{what}: bytes AFTER the buffer were overwritten"


def f16(a):
    return torch.from_numpy(a.view(np.float16).copy())


def make_layer(case, device=DEV):
    """oracle-case dict (x, weight, scales, zeros, bias, bits, group_size) -> LinearQ on the GPU."""
    n, k = case["weight"].shape[0], case["x"].shape[-1]
    lq = asrq_b200.LinearQ(k, n, case["bits"], case["group_size"], bias=case["bias"] is not None).to(device)
    lq.load_quantized_params(case["scales"], case["zeros"], case["weight"])
    if case["bias"] is not None:
        lq.bias = case["bias"].to(device)
    return lq


def assert_close_rows(y, y_ref32, rel=2e-3, extra=None, what=""):
    """max|err| <= rel * ||row||_inf of the fp32 CPU result (plus, for bf16 outputs, half an output ulp)."""
    err = (y.float().cpu() - y_ref32).abs()
    tol = O.row_tolerance(y_ref32, rel)
    if extra is not None:
        tol = tol + extra
    bad = err > tol
    if bool(bad.any()):
        idx = torch.nonzero(bad)[0].tolist()
        raise AssertionError(
            f"{what}: {int(bad.sum())} of {bad.numel()} outputs outside tolerance; first at {idx}: "
            f"got {float(y.float().cpu()[tuple(idx)])}, want {float(y_ref32[tuple(idx)])}, "
            f"tol {float(tol.expand_as(err)[tuple(idx)])}, max err {float(err.max())}")
    return float((err / tol.expand_as(err).clamp_min(1e-30)).max())


def bf16_half_ulp(y_ref32):
    """Half a bf16 ulp at each reference value: what rounding the output to bf16 alone may cost."""
    return y_ref32.abs() * 2.0 ** -8


def run_a16_abi(fn, case, dtype=torch.float16, device=DEV):
    """Calls one of the asrq_w{2,4}a16_{gemv,gemm} entry points directly."""
    x = case["x"].to(dtype).to(device).contiguous()
    m, k = x.shape
    n = case["weight"].shape[0]
    w = case["weight"].to(device)
    s, z = case["scales"].to(device), case["zeros"].to(device)
    b = None if case["bias"] is None else case["bias"].to(device)
    # output and workspace sit between canary bytes: a kernel that writes outside either fails the test
    y = padded((m, n), dtype, device)
    kind = _lib.WS_A16_GEMM if fn.endswith("gemm") else _lib.WS_LINEARQ
    ws = padded((max(_lib.workspace_bytes(kind, m, n, k), _lib.workspace_bytes(_lib.WS_LINEARQ, m, n, k)),),
                torch.uint8, device, fill=0)
    _lib.call(fn, x.data_ptr(), w.data_ptr(), s.data_ptr(), z.data_ptr(), None if b is None else b.data_ptr(),
              y.data_ptr(), m, n, k, case["group_size"], _lib.F16 if dtype == torch.float16 else _lib.BF16,
              ws.data_ptr(), ws.numel(), torch.cuda.current_stream().cuda_stream)
    _lib.call("asrq_check_status", ws.data_ptr(), torch.cuda.current_stream().cuda_stream)
    check_canary(y, f"{fn} output")
    check_canary(ws, f"{fn} workspace")
    assert int(ws[:16640].view(torch.int32).abs().sum()) == 0, f"{fn}: status block or tile counters not clean"
    return y
