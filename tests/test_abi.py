"""The C-ABI library: loads, exports every symbol the header declares, rejects bad arguments
on the host before touching a device.  No compute calls here (no GPU needed)."""
import ctypes
import os
import re

import pytest
import torch

import asrq_b200
from asrq_b200 import _lib

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _header_functions():
    text = open(os.path.join(ROOT, "include", "asrq_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(asrq_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    lib = _lib.load()
    names = _header_functions()
    assert len(names) >= 12
    for n in names:
        assert hasattr(lib, n), f"{n} is declared in include/asrq_b200.h but not exported"
    assert set(names) == set(_lib.SIGNATURES), "ctypes prototypes and header disagree"
    assert lib.asrq_version() >= 100


def test_workspace_bytes():
    assert _lib.workspace_bytes(_lib.WS_A16_GEMV, 1, 6144, 2048) >= 256 + 16 * 6144 * 4
    assert _lib.workspace_bytes(_lib.WS_LINEARQ, 1, 6144, 2048) == _lib.workspace_bytes(_lib.WS_A16_GEMV, 1, 6144, 2048)
    assert _lib.workspace_bytes(_lib.WS_A16_GEMM, 1500, 5120, 1280) >= 256
    assert _lib.workspace_bytes(99, 1, 1, 1) == 0


def test_null_and_dtype_rejected_before_launch():
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096 + 16)
    p = (ctypes.addressof(buf) + 15) & ~15
    rc = lib.asrq_w4a16_gemv(None, p, p, p, None, p, 1, 128, 128, 128, 0, p, 4096, None)
    assert rc == -1 and "NULL" in _lib.last_error()
    rc = lib.asrq_w4a16_gemv(p, p, p, p, None, p, 1, 128, 128, 128, 7, p, 4096, None)
    assert rc == -5
    rc = lib.asrq_w4a16_gemm(p, p, p, p, None, p + 2, 64, 128, 128, 128, 0, p, 4096, None)
    assert rc == -3 and "aligned" in _lib.last_error()
    rc = lib.asrq_w4a16_gemv(p, p, p, p, None, p, 1, 128, 128, 128, 0, None, 0, None)
    assert rc == -4
    rc = lib.asrq_linearq_a16(3, p, p, p, p, None, p, 1, 128, 128, 128, 0, p, 4096, None)
    assert rc == -2 and "bits" in _lib.last_error()
    rc = lib.asrq_hadamard_quant_int4(None, p, p, 1, 256, 1, 0, None)
    assert rc == -1
    rc = lib.asrq_w4a4_gemm(p, p, p, p, None, p, None, 1, 128, 128, 128, 0, None, 0, None)
    assert rc == -4
    with pytest.raises(_lib.AsrqError) as e:
        _lib.call("asrq_check_status", None, None)
    assert e.value.code == -1


def test_module_contract_matches_reference():
    """Constructor, buffers and state_dict keys of asrq/core/linear.py:10-25."""
    m = asrq_b200.LinearQ(1280, 5120, 4)  # bits is the third positional, as canary_qwen.py:83 passes it
    sd = m.state_dict()
    assert list(sd.keys()) == ["weight", "bias", "scales", "zeros"]
    assert sd["weight"].shape == (5120, 640) and sd["weight"].dtype == torch.uint8
    assert sd["scales"].shape == (5120, 10) and sd["scales"].dtype == torch.float16
    assert sd["zeros"].shape == (5120, 10) and sd["bias"].shape == (5120,) and sd["bias"].dtype == torch.float16
    assert (m.in_features, m.out_features, m.group_size, m.bits) == (1280, 5120, 128, 4)
    m2 = asrq_b200.LinearQ(256, 64, 2, group_size=64, bias=False)
    assert m2.bias is None and m2.weight.shape == (64, 64) and m2.scales.shape == (64, 4)
    assert list(m2.state_dict().keys()) == ["weight", "scales", "zeros"]
    q = asrq_b200.LinearQQ(256, 64, 4, 4, 128, bias=False)
    assert q.amax == 7 and q.abits == 4 and q.act_scales.shape == (256,)
    # load_quantized_params rebinding (linear.py:27-31)
    m2.load_quantized_params(torch.ones(64, 4).half(), torch.zeros(64, 4).half(), torch.ones(64, 64, dtype=torch.uint8))
    assert float(m2.scales[0, 0]) == 1.0 and int(m2.weight[0, 0]) == 1


def test_dequantize_weight_matches_golden(golden_dir):
    import numpy as np
    d = np.load(os.path.join(golden_dir, "linearq_w4_g128_asym_f16.npz"))
    m = asrq_b200.LinearQ(int(d["in_features"]), int(d["out_features"]), 4, int(d["group_size"]))
    m.load_quantized_params(torch.from_numpy(d["scales"].view(np.float16).copy()),
                            torch.from_numpy(d["zeros"].view(np.float16).copy()), torch.from_numpy(d["weight"]))
    assert np.array_equal(m.dequantize_weight("cpu", torch.float32).numpy(), d["w_deq_f32"])
    assert np.array_equal(m.dequantize_weight("cpu", torch.float16).numpy().view(np.uint16), d["w_deq_f16"])


def test_no_cpu_fallback():
    m = asrq_b200.LinearQ(256, 128, 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        m(torch.zeros(2, 256, dtype=torch.float16))
    q = asrq_b200.LinearQQ(256, 128, 4, 4)
    with pytest.raises(RuntimeError, match="no CPU path"):
        q(torch.zeros(2, 256, dtype=torch.float16))


def test_w4a4_gemm_rejects_nonpositive_group_size_on_the_host():
    """group_size 0 used to reach a modulus (division by zero killed the process); it is an argument
    error like any other, found before a device is touched."""
    lib = _lib.load()
    buf = ctypes.create_string_buffer(4096 + 16)
    p = (ctypes.addressof(buf) + 15) & ~15
    for gs in (0, -128):
        rc = lib.asrq_w4a4_gemm(p, p, p, p, None, p, None, 8, 64, 128, gs, 0, p, 4096, None)
        assert rc == -2 and "group_size" in _lib.last_error()


def test_options_are_set_and_read_back():
    assert _lib.get_option("tc_pair") == -1
    _lib.set_option("tc_pair", 1)
    assert _lib.get_option("tc_pair") == 1
    _lib.set_option("tc_pair", -1)
    with pytest.raises(_lib.AsrqError) as e:
        _lib.set_option("no_such_switch", 1)
    assert e.value.code == -2
