"""Turns quantizer output into the buffers ``LinearQ`` / ``LinearQQ`` hold.

The reference stops one step short of this: its quantizers write fake-quantised
floats back into ``nn.Linear`` and return ``(scales, zeros)``
(asrq/quantizers/rtn.py:44-46, asrq/quantizers/gptq.py:119-122); nothing produces the
packed ``uint8`` buffer that ``LinearQ.dequantize_weight`` reads
(asrq/core/linear.py:33-54).  These functions are that step.  They are offline
host-side torch code and run on whatever device the tensors live on.
"""
from __future__ import annotations

import torch


def quant_range(bits: int, symmetric: bool):
    """(minq, maxq) of the grid, as asrq/quantizers/base.py:58-59."""
    maxq = 2 ** (bits - 1) - 1 if symmetric else 2 ** bits - 1
    return (-maxq if symmetric else 0), maxq


def find_quant_params(w: torch.Tensor, bits: int, group_size: int, symmetric: bool):
    """Per-(row, group) ``scales`` and ``zeros`` of shape (N, K/g, 1), in ``w.dtype``.

    Same arithmetic as LinearQuantizer.find_quant_params (asrq/quantizers/base.py:61-77).
    """
    if w.ndim != 2:
        raise ValueError("only 2-D weights are supported")
    g = w.shape[1] if group_size == -1 else group_size
    if w.shape[1] % g:
        raise ValueError(f"in_features {w.shape[1]} is not divisible by group size {g}")
    wg = w.reshape(w.shape[0], w.shape[1] // g, g)
    if symmetric:
        scales = wg.abs().amax(dim=2, keepdim=True) / (2 ** (bits - 1) - 1)
        zeros = torch.zeros_like(scales)
    else:
        mx, mn = wg.amax(dim=2, keepdim=True), wg.amin(dim=2, keepdim=True)
        scales = (mx - mn) / (2 ** bits - 1)
        zeros = mn
    return scales, zeros


def rtn_quantize(w: torch.Tensor, bits: int, group_size: int = 128, symmetric: bool = False):
    """Round-to-nearest integer codes on the reference grid.

    ``round((W-zeros)/scales).clamp(minq,maxq)`` (asymmetric) or
    ``round(W/scales).clamp(minq,maxq)`` (symmetric), asrq/quantizers/rtn.py:39-42, in
    ``w.dtype``.  Returns ``(codes int16 (N,K), scales (N,K/g), zeros (N,K/g))``.
    GPTQ produces codes on the same grid (asrq/quantizers/gptq.py:104-107), so its
    output packs the same way through :func:`pack_codes`.
    """
    scales, zeros = find_quant_params(w, bits, group_size, symmetric)
    g = w.shape[1] if group_size == -1 else group_size
    minq, maxq = quant_range(bits, symmetric)
    wg = w.reshape(w.shape[0], w.shape[1] // g, g)
    q = torch.round(wg / scales) if symmetric else torch.round((wg - zeros) / scales)
    codes = q.clamp(minq, maxq).reshape(w.shape).to(torch.int16)
    return codes, scales.squeeze(-1), zeros.squeeze(-1)


def codes_from_fake_quant(fq: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, bits: int,
                          group_size: int, symmetric: bool):
    """Recovers the integer codes from a reference quantizer's output.

    ``fq`` is the fake-quantised weight the quantizer wrote into the module and
    ``scales``/``zeros`` what it returned, shape (N, K/g, 1) or (N, K/g).
    """
    g = fq.shape[1] if group_size == -1 else group_size
    s = scales.reshape(fq.shape[0], -1, 1)
    z = zeros.reshape(fq.shape[0], -1, 1)
    fg = fq.reshape(fq.shape[0], fq.shape[1] // g, g)
    q = torch.round(fg / s) if symmetric else torch.round((fg - z) / s)
    minq, maxq = quant_range(bits, symmetric)
    return q.clamp(minq, maxq).reshape(fq.shape).to(torch.int16)


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Unsigned codes (N,K) -> ``uint8`` (N, K*bits/8) in LinearQ's layout.

    4-bit: byte j = code[2j] | code[2j+1] << 4; 2-bit: byte j holds code[4j+e] at bits
    [2e, 2e+1] -- the inverse of the unpacking at asrq/core/linear.py:43-52.
    """
    c = codes.to(torch.int32)
    if int(c.min()) < 0 or int(c.max()) >= 2 ** bits:
        raise ValueError("codes outside [0, 2^bits)")
    if bits == 4:
        out = c[:, 0::2] | (c[:, 1::2] << 4)
    elif bits == 2:
        out = c[:, 0::4] | (c[:, 1::4] << 2) | (c[:, 2::4] << 4) | (c[:, 3::4] << 6)
    else:
        raise ValueError("bits must be 2 or 4")
    return out.to(torch.uint8).contiguous()


def pack_signed_int4(codes: torch.Tensor) -> torch.Tensor:
    """Signed codes in [-8,7] (R,K) -> ``uint8`` (R,K/2): ``(lo & 0xF) | (hi & 0xF) << 4``.

    The convention of the reference's int4 GEMM experiment (asrq/matmulq/test.py:141-142).
    """
    c = codes.to(torch.int32)
    if int(c.min()) < -8 or int(c.max()) > 7:
        raise ValueError("codes outside [-8, 7]")
    return ((c[:, 0::2] & 0xF) | ((c[:, 1::2] & 0xF) << 4)).to(torch.uint8).contiguous()


def pack_linearq(codes: torch.Tensor, scales: torch.Tensor, zeros: torch.Tensor, bits: int, symmetric: bool):
    """Codes + grid -> ``(weight uint8, scales fp16, zeros fp16)`` for ``LinearQ.load_quantized_params``.

    LinearQ dequantises ``q*scale+zero`` with unsigned ``q`` (asrq/core/linear.py:43-46), so
    a symmetric (signed) grid is shifted: ``q_u = q_s + 2^(b-1)``, ``zero = -2^(b-1)*scale``.
    """
    if symmetric:
        off = 2 ** (bits - 1)
        codes = codes + off
        zeros = -off * scales
    return pack_codes(codes, bits), scales.to(torch.float16).contiguous(), zeros.to(torch.float16).contiguous()


def hadamard_pow2(x: torch.Tensor) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform over the last dim (power-of-two length).

    Butterfly order of matmul_hadU (asrq/transforms/rotation/hadamard_utils.py:64-81).  Used
    offline to fold the rotation into W4A4 weights.
    """
    n = x.shape[-1]
    if n & (n - 1):
        raise ValueError("length must be a power of two")
    y = x.reshape(-1, n)
    h = 1
    while h < n:
        v = y.reshape(-1, n // (2 * h), 2, h)
        y = torch.stack((v[:, :, 0, :] + v[:, :, 1, :], v[:, :, 0, :] - v[:, :, 1, :]), dim=2).reshape(-1, n)
        h *= 2
    return (y / torch.tensor(n).sqrt()).reshape(x.shape)


def pack_w4a4(w: torch.Tensor, group_size: int = 128, hadamard: bool = True):
    """Float weight (N,K) -> ``(weight uint8 (N,K/2) signed nibbles, scales fp16 (N,K/g))`` for ``LinearQQ``.

    With ``hadamard`` the rotation the layer applies online to its input is folded into
    the weight first (hadU is orthogonal and symmetric: x.W^T == hadU(x).hadU(W)^T), in the
    spirit of the reference's offline fusion (asrq/transforms/rotation/utils.py:398-401);
    then symmetric int4 round-to-nearest per group on the reference grid.
    """
    wf = w.float()
    if hadamard:
        wf = hadamard_pow2(wf)
    codes, scales, _ = rtn_quantize(wf, 4, group_size, True)
    return pack_signed_int4(codes), scales.to(torch.float16).contiguous()


# --------------------------------------------------------------------------------------------------
# the same steps as kernels (weights already on a CUDA device: no host round trip, no (N, K) temporaries)
# --------------------------------------------------------------------------------------------------

_W_DTYPES = {torch.float16: 0, torch.bfloat16: 1, torch.float32: 2}


def _cuda_weight(w: torch.Tensor, who: str) -> int:
    if not w.is_cuda:
        raise RuntimeError(f"{who}: the weight is on {w.device}; this is the device version (use the host functions of this module otherwise)")
    if w.ndim != 2 or w.dtype not in _W_DTYPES:
        raise ValueError(f"{who}: a 2-D fp16, bf16 or fp32 weight is expected, got {tuple(w.shape)} {w.dtype}")
    return _W_DTYPES[w.dtype]


def rtn_pack_cuda(w: torch.Tensor, bits: int, group_size: int = 128, symmetric: bool = False):
    """:func:`rtn_quantize` + :func:`pack_linearq` in one kernel: ``(weight uint8, scales fp16, zeros fp16)`` with the same
    bits as the host path (every operation rounded to ``w.dtype``)."""
    from . import _lib
    dt = _cuda_weight(w, "rtn_pack_cuda")
    n, k = w.shape
    g = k if group_size == -1 else group_size
    w = w.contiguous()
    weight = torch.empty((n, k * bits // 8), dtype=torch.uint8, device=w.device)
    scales = torch.empty((n, k // g), dtype=torch.float16, device=w.device)
    zeros = torch.empty((n, k // g), dtype=torch.float16, device=w.device)
    with torch.cuda.device(w.device):
        _lib.call("asrq_rtn_pack", w.data_ptr(), dt, bits, g, int(symmetric), 0, weight.data_ptr(), scales.data_ptr(),
                  zeros.data_ptr(), n, k, torch.cuda.current_stream(w.device).cuda_stream)
    return weight, scales, zeros


def hadamard_fold_cuda(w: torch.Tensor) -> torch.Tensor:
    """:func:`hadamard_pow2` of ``w.float()`` along the last dimension as a kernel (fp32 result, same bits)."""
    from . import _lib
    dt = _cuda_weight(w, "hadamard_fold_cuda")
    w = w.contiguous()
    out = torch.empty(w.shape, dtype=torch.float32, device=w.device)
    with torch.cuda.device(w.device):
        _lib.call("asrq_hadamard_fold", w.data_ptr(), dt, out.data_ptr(), w.shape[0], w.shape[1],
                  torch.cuda.current_stream(w.device).cuda_stream)
    return out


def pack_w4a4_cuda(w: torch.Tensor, group_size: int = 128, hadamard: bool = True):
    """:func:`pack_w4a4` on the device: Hadamard fold (optional), then symmetric int4 codes as signed nibbles."""
    from . import _lib
    _cuda_weight(w, "pack_w4a4_cuda")
    wf = hadamard_fold_cuda(w) if hadamard else w.float().contiguous()
    n, k = wf.shape
    weight = torch.empty((n, k // 2), dtype=torch.uint8, device=w.device)
    scales = torch.empty((n, k // group_size), dtype=torch.float16, device=w.device)
    with torch.cuda.device(w.device):
        _lib.call("asrq_rtn_pack", wf.data_ptr(), 2, 4, group_size, 1, 1, weight.data_ptr(), scales.data_ptr(), None, n, k,
                  torch.cuda.current_stream(w.device).cuda_stream)
    return weight, scales
