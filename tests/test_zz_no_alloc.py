"""asrq_w4a16_gemv_static: the decode kernel for callers that cannot allocate device memory.

Such callers (a server plugin that only receives input and output buffers, a real-time callback)
cannot pass a workspace, so the library keeps the scratch in a static device array.  The test
calls the entry point through the C ABI twice in a row -- the second call finds the array as the
first one left it -- and compares each result with the workspace-taking entry point, within the
tolerance the other decode tests use (2e-3 of the row maximum of the fp32 CPU result).
"""
import pytest
import torch

from asrq_b200 import _lib
from oracle import linearq_oracle as O
from tests.gpu_util import DEV, assert_close_rows, run_a16_abi

pytestmark = pytest.mark.gpu


def _static_call(case, expect_no_allocation=False):
    x = case["x"].to(DEV).contiguous()
    m, k = x.shape
    n = case["weight"].shape[0]
    w, s, z = case["weight"].to(DEV), case["scales"].to(DEV), case["zeros"].to(DEV)
    b = None if case["bias"] is None else case["bias"].to(DEV)
    y = torch.full((m, n), float("nan"), dtype=torch.float16, device=DEV)
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(DEV)[0]      # device-wide free bytes (cudaMemGetInfo)
    _lib.call("asrq_w4a16_gemv_static", x.data_ptr(), w.data_ptr(), s.data_ptr(), z.data_ptr(),
              None if b is None else b.data_ptr(), y.data_ptr(), m, n, k, case["group_size"], _lib.F16,
              torch.cuda.current_stream().cuda_stream)
    torch.cuda.synchronize()
    if expect_no_allocation:
        # nothing between the two readings goes through torch's allocator, so any difference would be
        # device memory taken by the entry point itself
        assert torch.cuda.mem_get_info(DEV)[0] == free_before, "the static-scratch entry point allocated device memory"
    return y


def test_static_scratch_entry_matches_workspace_entry_twice():
    # 6144 -> 2048 splits K across blocks, so the scratch (partials + counters) is really used
    cases = [O.make_c3(seed=21, m=4, k=6144, n=2048, bits=4, group_size=64),
             O.make_c3(seed=22, m=16, k=2048, n=4096, bits=4, group_size=64)]
    for rnd in range(2):
        for case in cases:
            ref32 = O.linearq_forward_fp32(case["x"], case["weight"], case["scales"], case["zeros"], None, 4, 64)
            y_ws = run_a16_abi("asrq_w4a16_gemv", case)
            y_st = _static_call(case)
            assert_close_rows(y_st, ref32, what=f"static entry, round {rnd}")
            scale = ref32.abs().max(dim=-1, keepdim=True).values
            assert float(((y_st.float().cpu() - y_ws.float().cpu()).abs() / scale).max()) < 2e-3


def test_static_scratch_entry_allocates_nothing_and_takes_bias_and_row_blocks():
    """After a first call (which looks the array's address up), a call leaves the device's free memory
    exactly as it found it.  With a bias, and with 20 tokens: two launches of 16 and 4 rows that share
    the scratch array one after the other."""
    gen = torch.Generator().manual_seed(23)
    case = O.make_c3(seed=23, m=20, k=6144, n=2048, bits=4, group_size=64)
    case["bias"] = (torch.randn(2048, generator=gen) * 0.02).half()
    ref32 = O.linearq_forward_fp32(case["x"], case["weight"], case["scales"], case["zeros"], case["bias"], 4, 64)
    _static_call(case)                                       # first call on this device: set-up
    for _ in range(2):
        y = _static_call(case, expect_no_allocation=True)
        assert_close_rows(y, ref32, what="static entry, bias, 20 tokens")
    y_ws = run_a16_abi("asrq_w4a16_gemv", case)
    scale = ref32.abs().max(dim=-1, keepdim=True).values
    assert float(((y.float().cpu() - y_ws.float().cpu()).abs() / scale).max()) < 2e-3


def test_static_scratch_entry_rejects_large_n():
    x = torch.zeros(1, 128, dtype=torch.float16, device=DEV)
    w = torch.zeros(8192 + 16, 64, dtype=torch.uint8, device=DEV)
    s = torch.zeros(8192 + 16, 1, dtype=torch.float16, device=DEV)
    y = torch.zeros(1, 8192 + 16, dtype=torch.float16, device=DEV)
    with pytest.raises(_lib.AsrqError) as e:
        _lib.call("asrq_w4a16_gemv_static", x.data_ptr(), w.data_ptr(), s.data_ptr(), s.data_ptr(), None, y.data_ptr(),
                  1, 8192 + 16, 128, 128, _lib.F16, None)
    assert e.value.code == -8 and "8192" in str(e.value)
