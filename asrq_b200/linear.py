"""Drop-in ``LinearQ`` / ``LinearQQ`` modules backed by the B200 kernels.

Same constructor, buffer names, shapes and dtypes, ``state_dict`` keys and
``forward(input)`` contract as the reference module (asrq/core/linear.py:8-86), so the
``Whisper*Q`` / ``Qwen3*Q`` / ``Conformer*Q`` classes can import it unchanged.  The
forward pass calls the C ABI (``include/asrq_b200.h``); there is no CPU or PyTorch
fallback -- a CPU tensor, or a missing library, raises.
"""
from __future__ import annotations

import os

import torch
import torch.nn as nn

from . import _lib

_DTYPES = {torch.float16: _lib.F16, torch.bfloat16: _lib.BF16}
_CHECK = os.environ.get("ASRQ_B200_CHECK_STATUS", "0") == "1"

# one scratch buffer per (device, stream): kernels on one stream run in order, so they can share it
_workspaces: dict = {}


def _workspace(device: torch.device, nbytes: int) -> torch.Tensor:
    key = (device.index, torch.cuda.current_stream(device).cuda_stream)
    ws = _workspaces.get(key)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[key] = ws
    return ws


def check_status(device=None) -> None:
    """Synchronises the device and raises if a kernel on any of its streams reported a bounded wait that gave up."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    idx = device.index if device.index is not None else torch.cuda.current_device()
    torch.cuda.synchronize(idx)
    for (dev, stream), ws in list(_workspaces.items()):
        if dev == idx:
            with _on_device(torch.device("cuda", idx)):
                _lib.call("asrq_check_status", ws.data_ptr(), stream)


class _on_device:
    """Makes the tensor's device current around C-ABI calls (the library works on the current device:
    per-device facts, occupancy queries, launches).  Free when it already is."""

    def __init__(self, device: torch.device):
        self.idx = device.index if device.index is not None else torch.cuda.current_device()
        self.prev = None

    def __enter__(self):
        cur = torch.cuda.current_device()
        if cur != self.idx:
            self.prev = cur
            torch.cuda.set_device(self.idx)
        return self

    def __exit__(self, *exc):
        if self.prev is not None:
            torch.cuda.set_device(self.prev)
        return False


def add_layernorm(x: torch.Tensor, delta, weight: torch.Tensor, bias: torch.Tensor, eps: float = 1e-5, write_sum: bool = True):
    """``(x + delta, layer_norm(x + delta) * weight + bias)`` in one kernel (``delta`` may be None: then the
    first result is ``x`` itself).  16-bit tensors on a CUDA device; the last dimension is normalised."""
    dt = _require_cuda_16bit(x, "add_layernorm")
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    d2 = None
    if delta is not None:
        d2 = delta.reshape(-1, dim)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
    h = torch.empty_like(x2)
    xo = torch.empty_like(x2) if (delta is not None and write_sum) else None
    with _on_device(x.device):
        _lib.call("asrq_add_layernorm", x2.data_ptr(), None if d2 is None else d2.data_ptr(), weight.data_ptr(),
                  bias.data_ptr(), float(eps), None if xo is None else xo.data_ptr(), h.data_ptr(), x2.shape[0], dim, dt,
                  torch.cuda.current_stream(x.device).cuda_stream)
    return (x if xo is None else xo.reshape(x.shape)), h.reshape(x.shape)


def add_rmsnorm(x: torch.Tensor, delta, weight: torch.Tensor, eps: float = 1e-6, write_sum: bool = True):
    """``(x + delta, rms_norm(x + delta) * weight)`` in one kernel, with the rounding of the Qwen3 norm module (the
    normalised value is rounded to the tensor's type before the weight multiplies it).  ``delta`` may be None."""
    dt = _require_cuda_16bit(x, "add_rmsnorm")
    dim = x.shape[-1]
    x2 = x.reshape(-1, dim)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    d2 = None
    if delta is not None:
        d2 = delta.reshape(-1, dim)
        d2 = d2 if d2.is_contiguous() else d2.contiguous()
    h = torch.empty_like(x2)
    xo = torch.empty_like(x2) if (delta is not None and write_sum) else None
    with _on_device(x.device):
        _lib.call("asrq_add_rmsnorm", x2.data_ptr(), None if d2 is None else d2.data_ptr(), weight.data_ptr(), float(eps),
                  None if xo is None else xo.data_ptr(), h.data_ptr(), x2.shape[0], dim, dt,
                  torch.cuda.current_stream(x.device).cuda_stream)
    return (x if xo is None else xo.reshape(x.shape)), h.reshape(x.shape)


def silu_mul(gate_up: torch.Tensor) -> torch.Tensor:
    """``silu(gate) * up`` for the output of a fused gate/up projection: ``gate_up`` is ``(..., 2 * I)`` with the
    gate features first; returns ``(..., I)``."""
    dt = _require_cuda_16bit(gate_up, "silu_mul")
    inter = gate_up.shape[-1] // 2
    g2 = gate_up.reshape(-1, 2 * inter)
    g2 = g2 if g2.is_contiguous() else g2.contiguous()
    out = torch.empty((g2.shape[0], inter), dtype=gate_up.dtype, device=gate_up.device)
    with _on_device(gate_up.device):
        _lib.call("asrq_silu_mul", g2.data_ptr(), out.data_ptr(), g2.shape[0], inter, dt,
                  torch.cuda.current_stream(gate_up.device).cuda_stream)
    return out.reshape(*gate_up.shape[:-1], inter)


def qk_norm_rope(qkv: torch.Tensor, q_weight: torch.Tensor, k_weight: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                 k_cache: torch.Tensor, v_cache: torch.Tensor, pos, B: int, T: int, n_q: int, n_kv: int, eps: float) -> torch.Tensor:
    """Per-head RMS norm of queries and keys, rotary embedding, and the cache write for ``T`` new positions of ``B``
    sequences, in one kernel.  ``qkv``: (B*T, (n_q + 2 n_kv) * head_dim) from a fused projection; ``cos``/``sin``:
    (max_len, head_dim) tables; caches (B, n_kv, max_len, head_dim); ``pos``: first position, an int or a one-element int64
    CUDA tensor (read on the device).  Returns the queries (B, n_q, T, head_dim)."""
    dt = _require_cuda_16bit(qkv, "qk_norm_rope")
    hd = k_cache.shape[-1]
    q = torch.empty((B, n_q, T, hd), dtype=qkv.dtype, device=qkv.device)
    on_dev = isinstance(pos, torch.Tensor)
    with _on_device(qkv.device):
        _lib.call("asrq_qk_norm_rope", qkv.data_ptr(), q_weight.data_ptr(), k_weight.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                  pos.data_ptr() if on_dev else None, 0 if on_dev else int(pos), q.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
                  B, T, n_q, n_kv, hd, k_cache.shape[2], float(eps), dt, torch.cuda.current_stream(qkv.device).cuda_stream)
    return q


def decode_self_attention(qkv: torch.Tensor, kv_cache: torch.Tensor, pos: torch.Tensor, scale: float = 1.0) -> torch.Tensor:
    """Self-attention of one decoding step with the cache write: ``qkv`` (B, 3 * d) from a fused projection, ``kv_cache``
    (2, B, heads, max_len, head_dim), ``pos`` a one-element int64 CUDA tensor (the new token's position).  Returns (B, d)."""
    dt = _require_cuda_16bit(qkv, "decode_self_attention")
    _, B, H, max_len, hd = kv_cache.shape
    q2 = qkv.reshape(B, 3 * H * hd)
    q2 = q2 if q2.is_contiguous() else q2.contiguous()
    out = torch.empty((B, H * hd), dtype=qkv.dtype, device=qkv.device)
    with _on_device(qkv.device):
        _lib.call("asrq_decode_self_attention", q2.data_ptr(), kv_cache.data_ptr(), pos.data_ptr(), out.data_ptr(), B, H, hd, max_len,
                  float(scale), dt, torch.cuda.current_stream(qkv.device).cuda_stream)
    return out


def dense_head(x: torch.Tensor, weight: torch.Tensor, out: torch.Tensor = None) -> torch.Tensor:
    """``x @ weight.T`` for the floating-point output head of a decoding step (``weight`` is (vocabulary, K) in the
    activations' 16-bit type): this library's kernel for up to 32 rows of ``x`` and K a multiple of 32 up to 3200,
    ``torch.matmul`` otherwise."""
    dt = _require_cuda_16bit(x, "dense_head")
    k = x.shape[-1]
    x2 = x.reshape(-1, k)
    m, n = x2.shape[0], weight.shape[0]
    if out is None:
        out = torch.empty((m, n), dtype=x.dtype, device=x.device)
    if m > 32 or k % 32 or k > 3200 or weight.dtype != x.dtype or not weight.is_contiguous():
        torch.matmul(x2, weight.t(), out=out)
        return out.reshape(*x.shape[:-1], n)
    x2 = x2 if x2.is_contiguous() else x2.contiguous()
    with _on_device(x.device):
        _lib.call("asrq_dense_head", x2.data_ptr(), weight.data_ptr(), out.data_ptr(), m, n, k, dt,
                  torch.cuda.current_stream(x.device).cuda_stream)
    return out.reshape(*x.shape[:-1], n)


def _as_2d(x: torch.Tensor, k: int) -> torch.Tensor:
    if x.shape[-1] != k:
        raise ValueError(f"last dimension of the input is {x.shape[-1]}, expected in_features={k}")
    x2 = x.reshape(-1, k)
    return x2 if x2.is_contiguous() else x2.contiguous()


def _require_cuda_16bit(x: torch.Tensor, who: str) -> int:
    if not x.is_cuda:
        raise RuntimeError(f"{who}: input is on {x.device}; asrq_b200 runs on CUDA (sm_100a) only and has no CPU path")
    try:
        return _DTYPES[x.dtype]
    except KeyError:
        raise TypeError(f"{who}: input dtype {x.dtype} is not supported (float16 or bfloat16)") from None


class LinearQ(nn.Module):
    """Linear layer with packed 2-/4-bit weights and per-group fp16 scales and zeros.

    Mirrors asrq/core/linear.py:8-66: ``weight`` uint8 (out, in*bits/8), ``scales`` and
    ``zeros`` fp16 (out, ceil(in/group_size)), ``bias`` fp16 (out) or None;
    ``W[n,k] = q[n,k]*scales[n,k//g] + zeros[n,k//g]``; ``forward`` returns
    ``input @ W.T (+ bias)`` in the input dtype with the input's leading dimensions.
    """

    def __init__(self, in_features, out_features, bits, group_size=128, bias=True):
        super().__init__()
        self.in_features = in_features
        self.out_features = out_features
        self.group_size = group_size
        self.bits = bits
        self.register_buffer("weight", torch.zeros((out_features, in_features // (8 // bits)), dtype=torch.uint8))
        if bias:
            self.register_buffer("bias", torch.zeros(out_features, dtype=torch.float16))
        else:
            self.bias = None
        ngroups = (in_features + group_size - 1) // group_size
        self.register_buffer("scales", torch.zeros((out_features, ngroups), dtype=torch.float16))
        self.register_buffer("zeros", torch.zeros((out_features, ngroups), dtype=torch.float16))

    def load_quantized_params(self, scales, zeros, quantized_weight):
        """Binds already-packed parameters, moving them to the module's device (linear.py:27-31)."""
        self.scales = scales.to(self.scales.device)
        self.zeros = zeros.to(self.zeros.device)
        self.weight = quantized_weight.to(self.weight.device)

    def dequantize_weight(self, device="cpu", dtype=torch.float32):
        """Full (out, in) weight in ``dtype`` with the reference's two-step rounding
        (linear.py:33-54).  A debugging aid; ``forward`` never calls it."""
        g, k = self.group_size, self.in_features
        scale = self.scales.repeat_interleave(g, dim=1).to(device).to(dtype)[:, :k]
        zero = self.zeros.repeat_interleave(g, dim=1).to(device).to(dtype)[:, :k]
        wq = self.weight.to(device)
        q = torch.zeros((self.out_features, k), device=device, dtype=dtype)
        if self.bits == 4:
            q[:, 0::2] = (wq & 0x0F).to(dtype)
            q[:, 1::2] = (wq >> 4).to(dtype)
        elif self.bits == 2:
            for e in range(4):
                q[:, e::4] = ((wq >> (2 * e)) & 0x03).to(dtype)
        else:
            raise NotImplementedError("bits must be 2 or 4")
        return q * scale + zero

    def _check_buffers(self, x: torch.Tensor) -> None:
        for name in ("weight", "scales", "zeros"):
            t = getattr(self, name)
            if t.device != x.device:
                raise RuntimeError(f"LinearQ.{name} is on {t.device} but the input is on {x.device}")
            if not t.is_contiguous():
                setattr(self, name, t.contiguous())
        if self.scales.dtype != torch.float16 or self.zeros.dtype != torch.float16:
            raise TypeError("LinearQ.scales and LinearQ.zeros must be float16")
        if self.weight.dtype != torch.uint8:
            raise TypeError("LinearQ.weight must be uint8")
        if self.bias is not None and (self.bias.dtype != torch.float16 or self.bias.device != x.device):
            raise TypeError("LinearQ.bias must be float16 on the input's device")

    def forward(self, input):
        return self.forward_fused(input)

    def forward_fused(self, input, residual=None, gelu=False):
        """``forward`` with the step that follows the layer in a transformer block done in the kernel's
        epilogue: ``gelu(layer(input))`` or ``residual + layer(input)`` (``residual``: the output's shape and
        dtype).  Same bits as the unfused module sequence."""
        # fp16 / bf16 only (the reference computes in whatever dtype the input has, asrq/core/linear.py:58-59;
        # an fp32 input raises here rather than silently running a slower path)
        dt = _require_cuda_16bit(input, "LinearQ.forward")
        if self.bits not in (2, 4):
            raise NotImplementedError("LinearQ.forward: bits must be 2 or 4")
        self._check_buffers(input)
        n, k = self.out_features, self.in_features
        x2 = _as_2d(input, k)
        m = x2.shape[0]
        y = torch.empty((m, n), dtype=input.dtype, device=input.device)
        if m == 0:
            return y.reshape(*input.shape[:-1], n)
        ws = _workspace(input.device, _lib.workspace_bytes(_lib.WS_LINEARQ, m, n, k))
        stream = torch.cuda.current_stream(input.device).cuda_stream
        bias = None if self.bias is None else self.bias.data_ptr()
        with _on_device(input.device):
            if residual is None and not gelu:
                _lib.call("asrq_linearq_a16", self.bits, x2.data_ptr(), self.weight.data_ptr(), self.scales.data_ptr(),
                          self.zeros.data_ptr(), bias, y.data_ptr(), m, n, k, self.group_size, dt, ws.data_ptr(),
                          ws.numel(), stream)
            else:
                r2 = None
                if residual is not None:
                    if residual.dtype != input.dtype or residual.numel() != m * n or residual.device != input.device:
                        raise ValueError("forward_fused: residual must have the output's shape, dtype and device")
                    r2 = residual.reshape(m, n)
                    r2 = r2 if r2.is_contiguous() else r2.contiguous()
                _lib.call("asrq_linearq_a16_fused", self.bits, x2.data_ptr(), self.weight.data_ptr(),
                          self.scales.data_ptr(), self.zeros.data_ptr(), bias, None if r2 is None else r2.data_ptr(),
                          y.data_ptr(), m, n, k, self.group_size, dt, _lib.ACT_GELU if gelu else _lib.ACT_NONE,
                          ws.data_ptr(), ws.numel(), stream)
        if _CHECK:
            check_status(input.device)
        return y.reshape(*input.shape[:-1], n)

    def extra_repr(self):
        return (f"in_features={self.in_features}, out_features={self.out_features}, bits={self.bits}, "
                f"group_size={self.group_size}, bias={self.bias is not None}")


class LinearQQ(LinearQ):
    """W4A4 linear: online Hadamard rotation + per-token int4 activations, grouped int4 weights.

    Constructor signature of the reference stub (asrq/core/linear.py:69-75), whose
    ``forward`` returns None.  ``weight`` holds two's-complement signed nibbles
    (asrq/matmulq/test.py:141-142), ``scales`` the per-(row, group) weight scales;
    ``zeros`` is unused and stays zero.  ``forward`` computes

        v = hadU(x) (if ``hadamard``);  s = absmax(v)/7 per token;  q = rint(v/s)
        y[m,n] = s[m] * sum_g (sum_{k in g} q[m,k]*qw[n,k]) * scales[n,g]  (+ bias[n])

    which equals ``x @ W.T`` up to quantisation error when ``weight`` was produced by
    :func:`asrq_b200.packing.pack_w4a4` with the same ``hadamard`` flag.
    """

    def __init__(self, in_features, out_features, wbits, abits, group_size=128, bias=True, hadamard=True):
        if wbits != 4 or abits != 4:
            raise NotImplementedError("LinearQQ supports wbits=4, abits=4")
        super().__init__(in_features, out_features, wbits, group_size, bias)
        self.register_buffer("act_scales", torch.ones(in_features))
        self.amax = 2 ** (abits - 1) - 1
        self.abits = abits
        self.hadamard = hadamard

    def _quantize(self, input):
        dt = _require_cuda_16bit(input, "LinearQQ")
        x2 = _as_2d(input, self.in_features)
        m, k = x2.shape
        qa = torch.empty((m, k // 2), dtype=torch.uint8, device=input.device)
        sa = torch.empty((m,), dtype=torch.float32, device=input.device)
        stream = torch.cuda.current_stream(input.device).cuda_stream
        _lib.call("asrq_hadamard_quant_int4", x2.data_ptr(), qa.data_ptr(), sa.data_ptr(), m, k,
                  1 if self.hadamard else 0, dt, stream)
        return qa, sa, dt, stream

    def quantize_activation(self, input):
        """(codes, scales): integer-valued float codes (M,K) and per-token scales (M,1), the
        return convention of the reference method (linear.py:77-82), computed by the CUDA prologue."""
        _require_cuda_16bit(input, "LinearQQ")
        with _on_device(input.device):
            qa, sa, _, _ = self._quantize(input)
        p = qa.to(torch.int32)
        lo, hi = p & 0xF, (p >> 4) & 0xF
        lo = torch.where(lo >= 8, lo - 16, lo)
        hi = torch.where(hi >= 8, hi - 16, hi)
        q = torch.stack((lo, hi), dim=-1).reshape(qa.shape[0], -1).to(torch.float32)
        return q, sa.reshape(-1, 1)

    # 8-bit operand family of the tensor-core path: "f8" (e4m3 bytes holding the code, tcgen05 kind::f8f6f4,
    # fp32 group sums) or "int8" (16x the code, kind::i8, int32 group sums).  Same bits out; f8 is faster.
    operand = os.environ.get("ASRQ_B200_W4A4_OPERAND", "f8")

    def _entry(self, stem: str) -> str:
        if self.operand not in ("f8", "int8"):
            raise ValueError(f"LinearQQ.operand must be 'f8' or 'int8', got {self.operand!r}")
        if stem == "prepare":
            return "asrq_w4a4_prepare_weight_f8" if self.operand == "f8" else "asrq_w4a4_prepare_weight"
        return f"asrq_{stem}_{self.operand}"

    def _prepared_weight(self) -> torch.Tensor:
        """8-bit operand form of ``weight`` (natural k order), derived on first use and whenever the
        packed buffer is replaced or modified; not part of ``state_dict``."""
        key = (self.weight.data_ptr(), self.weight._version, self.weight.device, self.operand)
        if getattr(self, "_w8_key", None) != key:
            n, k = self.out_features, self.in_features
            w8 = torch.empty((n, k), dtype=torch.uint8, device=self.weight.device)
            _lib.call(self._entry("prepare"), self.weight.data_ptr(), w8.data_ptr(), n, k,
                      torch.cuda.current_stream(self.weight.device).cuda_stream)
            self._w8, self._w8_key = w8, key
        return self._w8

    def _tensor_core_ok(self, m: int) -> bool:
        n, k, g = self.out_features, self.in_features, self.group_size
        return m >= 64 and n % 128 == 0 and k % 128 == 0 and g % 128 == 0 and k % g == 0

    def forward(self, input, acc_dump=None, two_call=False):
        _require_cuda_16bit(input, "LinearQQ")
        with _on_device(input.device):
            return self._forward(input, acc_dump, two_call)

    def _forward(self, input, acc_dump=None, two_call=False):
        """``two_call=True`` forces the packed-activation sequence (asrq_hadamard_quant_int4 then
        asrq_w4a4_gemm); the default for large M is the prologue writing 8-bit operands directly.
        Both produce the same bits."""
        self._check_buffers(input)
        if input.numel() == 0:
            _require_cuda_16bit(input, "LinearQQ")
            return input.new_empty(*input.shape[:-1], self.out_features)
        n, k = self.out_features, self.in_features
        bias = None if self.bias is None else self.bias.data_ptr()
        dump = None if acc_dump is None else acc_dump.data_ptr()
        if two_call or not self._tensor_core_ok(input.numel() // k):
            qa, sa, dt, stream = self._quantize(input)
            m = qa.shape[0]
            y = torch.empty((m, n), dtype=input.dtype, device=input.device)
            ws = _workspace(input.device, _lib.workspace_bytes(_lib.WS_W4A4_GEMM, m, n, k))
            _lib.call("asrq_w4a4_gemm", qa.data_ptr(), sa.data_ptr(), self.weight.data_ptr(), self.scales.data_ptr(),
                      bias, y.data_ptr(), dump, m, n, k, self.group_size, dt, ws.data_ptr(), ws.numel(), stream)
        else:
            dt = _require_cuda_16bit(input, "LinearQQ")
            x2 = _as_2d(input, k)
            m = x2.shape[0]
            w8 = self._prepared_weight()
            a8 = torch.empty((m, k), dtype=torch.uint8, device=input.device)
            sa = torch.empty((m,), dtype=torch.float32, device=input.device)
            y = torch.empty((m, n), dtype=input.dtype, device=input.device)
            ws = _workspace(input.device, _lib.STATUS_BYTES)
            stream = torch.cuda.current_stream(input.device).cuda_stream
            _lib.call(self._entry("hadamard_quant"), x2.data_ptr(), a8.data_ptr(), sa.data_ptr(), m, k,
                      1 if self.hadamard else 0, dt, stream)
            _lib.call(self._entry("w4a4_gemm"), a8.data_ptr(), sa.data_ptr(), w8.data_ptr(), self.scales.data_ptr(),
                      bias, y.data_ptr(), dump, m, n, k, self.group_size, dt, ws.data_ptr(), ws.numel(), stream)
        if _CHECK:
            check_status(input.device)
        return y.reshape(*input.shape[:-1], n)
