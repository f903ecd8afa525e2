"""Running a quantized layer on activations that live in host memory.

The reference has no counterpart: its ``LinearQ.forward`` takes whatever device its input is on
(asrq/core/linear.py:56-66).  A caller whose activations arrive in (pinned) host memory and whose
results go back there pays for two PCIe transfers that dwarf the kernels; :func:`forward_host` hides
what can be hidden by cutting the token dimension into chunks and running three streams: chunk i+1 is
copied in while chunk i is computed and chunk i-1 is copied out (the two copy directions use
different DMA engines).  Rows are independent; a chunk may be served by a different kernel than the whole
batch would be (the dispatch depends on the token count), so results agree with one call to within
the kernels' common accuracy bound, and bit for bit when the dispatch is the same.
"""
from __future__ import annotations

import torch

_streams = {}


def _side_streams(device: torch.device):
    key = device.index if device.index is not None else torch.cuda.current_device()
    if key not in _streams:
        _streams[key] = (torch.cuda.Stream(device), torch.cuda.Stream(device))
    return _streams[key]


def forward_host(layer, x_host: torch.Tensor, out_host: torch.Tensor = None, chunks: int = 4) -> torch.Tensor:
    """``layer(x)`` for a 2-D ``x_host`` in host memory; returns (and fills) ``out_host``.

    Both host tensors should be pinned, otherwise the copies are synchronous.  Work is ordered after the
    current stream of the layer's device and the current stream waits for the last copy out, so the
    usual stream semantics hold for the caller; ``out_host`` is valid after a synchronisation of that
    stream.  ``chunks`` <= 1 runs the plain sequence copy in, compute, copy out.
    """
    if x_host.dim() != 2:
        raise ValueError("forward_host takes a 2-D activation matrix (tokens, in_features)")
    if x_host.is_cuda:
        raise TypeError("forward_host: x_host must be a host tensor")
    dev = layer.weight.device
    if dev.type != "cuda":
        raise RuntimeError("forward_host: the layer is not on a CUDA device (there is no CPU path)")
    m = x_host.shape[0]
    n = layer.out_features
    if out_host is None:
        out_host = torch.empty((m, n), dtype=x_host.dtype).pin_memory()
    if out_host.shape != (m, n) or out_host.dtype != x_host.dtype:
        raise ValueError("forward_host: out_host must have shape (tokens, out_features) and the input's dtype")
    if m == 0:
        return out_host
    cur = torch.cuda.current_stream(dev)
    if chunks <= 1 or m < 128 * chunks:
        y = layer(x_host.to(dev, non_blocking=True))
        out_host.copy_(y, non_blocking=True)
        return out_host
    s_in, s_out = _side_streams(dev)
    s_in.wait_stream(cur)
    s_out.wait_stream(cur)
    step = -(-m // chunks)
    step = (step + 63) // 64 * 64  # whole token tiles per chunk
    for a in range(0, m, step):
        b = min(a + step, m)
        with torch.cuda.stream(s_in):
            xd = x_host[a:b].to(dev, non_blocking=True)
        xd.record_stream(cur)
        cur.wait_stream(s_in)
        y = layer(xd)
        y.record_stream(s_out)
        s_out.wait_stream(cur)
        with torch.cuda.stream(s_out):
            out_host[a:b].copy_(y, non_blocking=True)
    cur.wait_stream(s_out)
    return out_host
