"""CPU oracle for the quantized-linear path (TEST INFRASTRUCTURE ONLY).

This file restates, in plain torch-on-CPU / numpy arithmetic, the reference
algorithm of ASRQ's quantized linear layer.  It is the checker that the parity
tests, ``__graft_entry__.smoke()`` and the ``cpu_baseline`` / ``--impl
reference`` legs of ``bench.py`` use.  Nothing in the shipped package imports
it: the product path is the CUDA library and fails loudly without it.

Parity status: the reference holds no golden vectors or known-answer tests for
this path.  The oracle is pinned instead against outputs of the reference's own
Python code run on seeded inputs (``tests/golden/make_golden.py`` generates the
fixtures, ``tests/test_oracle_golden.py`` checks them).  The W4A4 composite
(online Hadamard + int4 activations + grouped int4 weights) has no executable
counterpart in the reference; only its pieces (FWHT, activation quantisation
formula, signed-nibble packing) are pinned, the composition is "parity
unpinned".

Every function cites the reference file:line it follows (paths relative to the
reference project root).
"""
from __future__ import annotations

import math

import numpy as np
import torch

# ----------------------------------------------------------------------------
# Weight grid (offline) -- asrq/quantizers/base.py:53-77, asrq/quantizers/rtn.py:32-46
# ----------------------------------------------------------------------------


def quant_range(bits: int, symmetric: bool):
    """(minq, maxq) of the integer grid.  asrq/quantizers/base.py:58-59."""
    maxq = 2 ** (bits - 1) - 1 if symmetric else 2 ** bits - 1
    minq = -maxq if symmetric else 0
    return minq, maxq


def find_quant_params(w: torch.Tensor, bits: int, group_size: int, symmetric: bool):
    """Per-(row, group) scales and zeros, shape (N, K/g, 1), in the dtype of ``w``.

    asrq/quantizers/base.py:61-77: asymmetric ``scales=(max-min)/(2^b-1)``,
    ``zeros=min``; symmetric ``scales=max|w|/(2^(b-1)-1)``, ``zeros=0``.
    """
    assert w.ndim == 2
    g = w.shape[1] if group_size == -1 else group_size
    assert w.shape[1] % g == 0
    wg = w.reshape(w.shape[0], w.shape[1] // g, g)
    if symmetric:
        maxq = 2 ** (bits - 1) - 1
        scales = torch.max(torch.abs(wg), dim=2, keepdim=True).values / maxq
        zeros = torch.zeros_like(scales)
    else:
        maxq = 2 ** bits - 1
        mx = torch.max(wg, dim=2, keepdim=True).values
        mn = torch.min(wg, dim=2, keepdim=True).values
        scales = (mx - mn) / maxq
        zeros = mn
    return scales, zeros


def rtn_codes(w: torch.Tensor, bits: int, group_size: int, symmetric: bool):
    """Integer codes of round-to-nearest quantisation plus the grid.

    asrq/quantizers/rtn.py:32-46 computes the fake-quantised weight
    ``round((W-zeros)/scales).clamp(minq,maxq)*scales+zeros`` (asymmetric) or
    ``round(W/scales).clamp(minq,maxq)*scales`` (symmetric) and never
    materialises the integer; this returns that integer (``torch.round`` is
    round-half-to-even), computed in the dtype of ``w`` like the reference.
    Returns (codes int16 (N,K), scales (N,K/g), zeros (N,K/g), fake_quant (N,K)).
    """
    scales, zeros = find_quant_params(w, bits, group_size, symmetric)
    g = w.shape[1] if group_size == -1 else group_size
    minq, maxq = quant_range(bits, symmetric)
    wg = w.reshape(w.shape[0], w.shape[1] // g, g)
    if symmetric:
        q = torch.round(wg / scales).clamp(minq, maxq)
        fq = q * scales
    else:
        q = torch.round((wg - zeros) / scales).clamp(minq, maxq)
        fq = q * scales + zeros
    codes = q.reshape(w.shape).to(torch.int16)
    return codes, scales.squeeze(-1), zeros.squeeze(-1), fq.reshape(w.shape)


# ----------------------------------------------------------------------------
# Packed layout -- defined implicitly by asrq/core/linear.py:33-54
# ----------------------------------------------------------------------------


def pack_codes(codes: torch.Tensor, bits: int) -> torch.Tensor:
    """Unsigned codes (N,K) -> uint8 (N, K*bits/8).

    Inverse of the unpack in asrq/core/linear.py:43-53: 4-bit byte j holds
    k=2j in its low nibble and k=2j+1 in its high nibble; 2-bit byte j holds
    k=4j+e at bits [2e, 2e+1].
    """
    c = codes.to(torch.int32)
    assert int(c.min()) >= 0 and int(c.max()) < 2 ** bits
    if bits == 4:
        out = c[:, 0::2] | (c[:, 1::2] << 4)
    elif bits == 2:
        out = c[:, 0::4] | (c[:, 1::4] << 2) | (c[:, 2::4] << 4) | (c[:, 3::4] << 6)
    elif bits == 8:
        out = c
    else:
        raise ValueError("bits must be 2, 4 or 8")
    return out.to(torch.uint8)


def pack_signed_int4(codes: torch.Tensor) -> torch.Tensor:
    """Signed int4 codes (R,K) -> uint8 (R,K/2), ``(lo & 0xF) | ((hi & 0xF) << 4)``.

    Pack convention of asrq/matmulq/test.py:141-142 (even k in the low nibble,
    two's-complement nibbles).
    """
    c = codes.to(torch.int32)
    assert int(c.min()) >= -8 and int(c.max()) <= 7
    return ((c[:, 0::2] & 0xF) | ((c[:, 1::2] & 0xF) << 4)).to(torch.uint8)


def unpack_signed_int4(packed: torch.Tensor) -> torch.Tensor:
    """uint8 (R,K/2) -> sign-extended int8 (R,K).  asrq/matmulq/csrc/bindings.cpp:373-384."""
    p = packed.to(torch.int32)
    lo = p & 0xF
    hi = (p >> 4) & 0xF
    lo = torch.where(lo >= 8, lo - 16, lo)
    hi = torch.where(hi >= 8, hi - 16, hi)
    out = torch.empty((p.shape[0], p.shape[1] * 2), dtype=torch.int8)
    out[:, 0::2] = lo.to(torch.int8)
    out[:, 1::2] = hi.to(torch.int8)
    return out


def symmetric_to_unsigned(codes: torch.Tensor, scales: torch.Tensor, bits: int):
    """Re-express a signed symmetric grid in LinearQ's unsigned-code format.

    LinearQ dequantises ``q_u*scale+zero`` with unsigned ``q_u``
    (asrq/core/linear.py:43-46); a symmetric grid ``q_s*scale`` becomes
    ``q_u=q_s+2^(b-1)``, ``zero=-2^(b-1)*scale``.
    """
    off = 2 ** (bits - 1)
    return codes + off, scales, -off * scales


# ----------------------------------------------------------------------------
# LinearQ -- asrq/core/linear.py:33-66
# ----------------------------------------------------------------------------


def unpack_codes(weight: torch.Tensor, bits: int, in_features: int) -> torch.Tensor:
    """uint8 packed (N, K*bits/8) -> unsigned codes uint8 (N,K).  asrq/core/linear.py:43-52."""
    n = weight.shape[0]
    q = torch.zeros((n, in_features), dtype=torch.uint8)
    if bits == 4:
        q[:, 0::2] = weight & 0x0F
        q[:, 1::2] = weight >> 4
    elif bits == 2:
        q[:, 0::4] = weight & 0x03
        q[:, 1::4] = (weight >> 2) & 0x03
        q[:, 2::4] = (weight >> 4) & 0x03
        q[:, 3::4] = (weight >> 6) & 0x03
    elif bits == 8:
        q = weight.clone()
    else:
        raise ValueError("bits must be 2, 4 or 8")
    return q


def dequantize_weight(weight, scales, zeros, bits, group_size, in_features, dtype=torch.float32):
    """W[n,k] = q[n,k]*scales[n,k//g] + zeros[n,k//g] in ``dtype``.

    asrq/core/linear.py:33-54: the multiply and the add are two separately
    rounded operations in the activation dtype; ``zeros`` is an additive float
    offset, not an integer zero-point.
    """
    scale = scales.repeat_interleave(group_size, dim=1).to(dtype)[:, :in_features]
    zero = zeros.repeat_interleave(group_size, dim=1).to(dtype)[:, :in_features]
    q = unpack_codes(weight, bits, in_features).to(dtype)
    return q * scale + zero


def linearq_forward(x, weight, scales, zeros, bias, bits, group_size):
    """y = x @ dequant(W)^T (+ bias) in the dtype of ``x``.  asrq/core/linear.py:56-66."""
    k = x.shape[-1]
    w = dequantize_weight(weight, scales, zeros, bits, group_size, k, x.dtype)
    out = torch.matmul(x, w.t())
    if bias is not None:
        out += bias
    return out


def linearq_forward_fp32(x, weight, scales, zeros, bias, bits, group_size):
    """The accuracy target: the same path evaluated entirely in fp32 on the CPU."""
    b = None if bias is None else bias.float()
    return linearq_forward(x.float(), weight, scales, zeros, b, bits, group_size)


# ----------------------------------------------------------------------------
# Hadamard -- asrq/transforms/rotation/hadamard_utils.py:60-81 (power-of-two n, K=1 branch)
# ----------------------------------------------------------------------------


def hadamard_pow2(x: torch.Tensor) -> torch.Tensor:
    """Normalised Walsh-Hadamard transform over the last dim (n a power of two).

    asrq/transforms/rotation/hadamard_utils.py:64-81: butterflies with strides
    1, 2, 4, ... n/2, each ``(a, b) -> (a+b, a-b)``, then division by sqrt(n).
    Runs in the dtype of ``x`` (every stage rounds to it), as the reference does.
    """
    n = x.shape[-1]
    assert n & (n - 1) == 0 and n > 0
    y = x.clone().reshape(-1, n)
    h = 1
    while h < n:
        v = y.reshape(-1, n // (2 * h), 2, h)
        a = v[:, :, 0, :] + v[:, :, 1, :]
        b = v[:, :, 0, :] - v[:, :, 1, :]
        y = torch.stack((a, b), dim=2).reshape(-1, n)
        h *= 2
    return (y / torch.tensor(n).sqrt()).reshape(x.shape)


# ----------------------------------------------------------------------------
# Activation quantisation -- asrq/quantizers/activation.py:26-28, asrq/core/linear.py:77-82
# ----------------------------------------------------------------------------


def act_quant_sym(x: torch.Tensor, bits: int = 4):
    """Per-token symmetric codes and scales, evaluated in the dtype of ``x``.

    asrq/quantizers/activation.py:26-28: ``s = absmax/(2^(b-1)-1)``, zero scale
    replaced by 1e-3, ``q = round(x/s)`` (round-half-even; |q| <= 2^(b-1)-1 by
    construction so the clamp of asrq/core/linear.py:81 never binds).
    Returns (codes int8 (...,K), scales (...,1)).
    """
    amax = 2 ** (bits - 1) - 1
    s = x.abs().max(dim=-1, keepdim=True).values / amax
    s = s.where(s != 0, torch.tensor(1e-3, dtype=s.dtype))
    q = torch.round(x / s).clamp(-amax, amax)
    return q.to(torch.int8), s


def fake_act_quant(x: torch.Tensor, bits: int = 4) -> torch.Tensor:
    """``round(x/s)*s`` -- the fake quantisation of asrq/quantizers/activation.py:28."""
    q, s = act_quant_sym(x, bits)
    return q.to(x.dtype) * s


def hadamard_quant_int4(x: torch.Tensor, hadamard: bool = True):
    """The W4A4 prologue as this build defines it (fp32 throughout).

    ``y = hadU(x.float())`` (hadamard_utils.py:60-81), then per-token symmetric
    int4 (activation.py:26-28) in fp32 with IEEE division.
    Returns (codes int8 (M,K), scales fp32 (M,), packed uint8 (M,K/2)).
    """
    y = x.float()
    if hadamard:
        y = hadamard_pow2(y)
    q, s = act_quant_sym(y, 4)
    return q, s.reshape(-1), pack_signed_int4(q)


# ----------------------------------------------------------------------------
# W4A4 composite (no executable counterpart in the reference)
# ----------------------------------------------------------------------------


def int4_group_accumulators(qa: torch.Tensor, qw: torch.Tensor, group_size: int) -> torch.Tensor:
    """Exact int32 sums per K-group: acc[m,n,g] = sum_{k in g} qa[m,k]*qw[n,k].

    Integer contraction of asrq/matmulq/test.py:28-92 restricted to one weight
    group.  Evaluated as fp32 matmuls, which are exact here: |product| <= 64
    and a group sum is at most 64*group_size < 2^24.
    """
    m, k = qa.shape
    n = qw.shape[0]
    ng = k // group_size
    assert group_size * 64 < 2 ** 24
    a = qa.float().reshape(m, ng, group_size)
    w = qw.float().reshape(n, ng, group_size)
    acc = torch.einsum("mgk,ngk->mng", a, w)
    return acc.round().to(torch.int32)


def w4a4_forward_fp32(qa, sa, qw, sw, bias, group_size):
    """y[m,n] = sA[m] * sum_g float(acc[m,n,g]) * sW[n,g]  (+ bias), fp32.

    Fused-dequant epilogue described at asrq/matmulq/csrc/bindings.cpp:552-560
    (per-(channel, group) weight scales, per-token activation scale).
    Groups are summed in ascending order in fp32.
    """
    acc = int4_group_accumulators(qa, qw, group_size).float()
    y = torch.zeros(acc.shape[0], acc.shape[1], dtype=torch.float32)
    swf = sw.float()
    for g in range(acc.shape[2]):
        y = y + acc[:, :, g] * swf[:, g][None, :]
    y = y * sa.float().reshape(-1, 1)
    if bias is not None:
        y = y + bias.float()
    return y


def prepare_w4a4_weight(w: torch.Tensor, group_size: int, hadamard: bool = True):
    """Offline weight side of the W4A4 layer.

    Folds the same normalised Hadamard along K that the prologue applies to the
    activations (hadU is orthogonal and symmetric, so x.W^T == hadU(x).hadU(W)^T;
    the offline-fusion idea of asrq/transforms/rotation/utils.py:398-401), then
    symmetric int4 round-to-nearest on the reference grid (rtn.py:39-40).
    Returns (codes int16 (N,K) in [-7,7], scales fp16 (N,K/g), packed uint8 (N,K/2)).
    """
    wf = w.float()
    if hadamard:
        wf = hadamard_pow2(wf)
    codes, scales, _, _ = rtn_codes(wf, 4, group_size, True)
    sw16 = scales.to(torch.float16)
    return codes, sw16, pack_signed_int4(codes)


# ----------------------------------------------------------------------------
# Seeded synthetic workloads (shapes and value distributions of the benchmark configs)
# ----------------------------------------------------------------------------


def make_c1(seed=0, m=1500, k=1280, n=5120, bits=4, group_size=128):
    """Single W4A16 layer: fp16 weights N(0,0.02) with 0.1% outliers x10, RTN asymmetric."""
    g = torch.Generator().manual_seed(seed)
    w = torch.randn(n, k, generator=g) * 0.02
    mask = torch.rand(w.shape, generator=g) < 1e-3
    w[mask] *= 10
    w = w.half()
    codes, scales, zeros, _ = rtn_codes(w, bits, group_size, False)
    x = torch.randn(m, k, generator=g).half()
    bias = (torch.randn(n, generator=g) * 0.02).half()
    return dict(x=x, weight=pack_codes(codes, bits), scales=scales.half(), zeros=zeros.half(),
                bias=bias, bits=bits, group_size=group_size, w_fp=w)


def make_c2(seed=0, m=6000, k=4096, n=1024, group_size=128):
    """W4A4 layer: Student-t(nu=4) activations with 8 outlier channels x20, N(0,0.02) weights."""
    g = torch.Generator().manual_seed(seed)
    z = torch.randn(m, k, generator=g)
    c = torch.zeros(m, k)
    for _ in range(4):
        c += torch.randn(m, k, generator=g) ** 2
    x = z / torch.sqrt(c / 4)
    idx = torch.randperm(k, generator=g)[:8]
    x[:, idx] *= 20
    x = x.half()
    w = torch.randn(n, k, generator=g) * 0.02
    bias = (torch.randn(n, generator=g) * 0.02).half()
    return dict(x=x, w_fp=w, bias=bias, group_size=group_size)


def make_c3(seed, m, k, n, bits, group_size=64, dtype=torch.float16):
    """Decode-shape layer: bf16-rounded N(0,0.02) weights, RTN asymmetric g64."""
    g = torch.Generator().manual_seed(seed)
    w = (torch.randn(n, k, generator=g) * 0.02).bfloat16().float()
    codes, scales, zeros, _ = rtn_codes(w, bits, group_size, False)
    x = torch.randn(m, k, generator=g).to(dtype)
    return dict(x=x, weight=pack_codes(codes, bits), scales=scales.half(), zeros=zeros.half(),
                bias=None, bits=bits, group_size=group_size, w_fp=w)


def row_tolerance(y_ref_fp32: torch.Tensor, rel: float = 2e-3) -> torch.Tensor:
    """Per-row absolute tolerance rel*||row||_inf of the fp32 CPU result, shape (M,1)."""
    return rel * y_ref_fp32.abs().max(dim=-1, keepdim=True).values


# ----------------------------------------------------------------------------
# Module form of the restatement (whole-model CPU baseline when the reference's files are not staged)
# ----------------------------------------------------------------------------


class PortLinearQ(torch.nn.Module):
    """``LinearQ`` as the reference runs it on the CPU: dequantize the whole weight on every call, then
    ``torch.matmul`` (asrq/core/linear.py:10-66), on top of the functions above."""

    def __init__(self, in_features, out_features, bits, group_size=128, bias=True):
        super().__init__()
        self.in_features, self.out_features, self.bits, self.group_size = in_features, out_features, bits, group_size
        self.register_buffer("weight", torch.zeros((out_features, in_features // (8 // bits)), dtype=torch.uint8))
        self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16) if bias else None)
        ng = (in_features + group_size - 1) // group_size
        self.register_buffer("scales", torch.zeros((out_features, ng), dtype=torch.float16))
        self.register_buffer("zeros", torch.zeros((out_features, ng), dtype=torch.float16))

    def forward(self, x):
        shape = x.shape
        y = linearq_forward(x.reshape(-1, shape[-1]), self.weight, self.scales, self.zeros, self.bias, self.bits,
                            self.group_size)
        return y.reshape(*shape[:-1], self.out_features)


def swap_in_port_linearq(model, bits, group_size, skip=()):
    """Replaces every ``nn.Linear`` of ``model`` (except names ending in ``skip``) by an empty PortLinearQ."""
    for name, mod in list(model.named_modules()):
        for cname, child in list(mod.named_children()):
            full = f"{name}.{cname}" if name else cname
            if type(child) is torch.nn.Linear and not any(full == s or full.endswith("." + s) for s in skip):
                setattr(mod, cname, PortLinearQ(child.in_features, child.out_features, bits, group_size,
                                                bias=child.bias is not None))
    return model
