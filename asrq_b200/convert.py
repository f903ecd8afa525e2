"""Model wiring: turn the ``nn.Linear`` layers of a model into packed ``LinearQ`` layers.

The reference quantises a model in place (``ModelQ.quantize``, asrq/core/model.py:122-133: every
quantizer writes fake-quantised floats back into ``linear.weight`` and returns ``(scales, zeros)``)
and, separately, builds model classes out of ``LinearQ`` (``Whisper*Q``, asrq/models/transformers/
whisper.py:38-271; ``load_modelQ``, whisper.py:314-327), but has no step that goes from the first to
the second.  This module is that step:

* :func:`linearq_from_linear` packs one layer, either with round-to-nearest on the reference grid or
  from the ``(scales, zeros)`` a reference quantizer returned for a layer it already fake-quantised;
* :func:`convert` walks a module tree and swaps the layers in place (same attribute names, so
  ``state_dict`` keys become ``<name>.weight`` / ``.scales`` / ``.zeros`` / ``.bias`` as in the
  reference's ``*Q`` classes);
* :class:`FusedLinearQ` runs several ``LinearQ`` layers that share their input (q/k/v, gate/up) as
  one kernel call over their concatenated rows, while the layers stay separate modules with separate
  ``state_dict`` entries.
"""
from __future__ import annotations

from typing import Callable, Dict, Iterable, Optional, Sequence, Tuple

import torch
import torch.nn as nn

from . import packing
from .linear import LinearQ


def linearq_from_linear(linear: nn.Linear, bits: int, group_size: int = 128, symmetric: bool = False,
                        qparams: Optional[Tuple[torch.Tensor, torch.Tensor]] = None) -> LinearQ:
    """Packs one ``nn.Linear`` into a ``LinearQ`` on the same device.

    ``qparams = (scales, zeros)`` as a reference quantizer returned them, shape (N, K/g, 1) or
    (N, K/g), for a layer whose weight that quantizer has already fake-quantised; without it the
    weight is quantised here with round-to-nearest (asrq/quantizers/rtn.py:32-46).
    """
    w = linear.weight.detach().float().cpu()
    n, k = w.shape
    g = k if group_size == -1 else group_size
    if k % g or (k * bits) % 8:
        raise ValueError(f"in_features={k} is not a multiple of group_size={g}")
    if qparams is None:
        codes, scales, zeros = packing.rtn_quantize(w, bits, g, symmetric)
    else:
        scales, zeros = (t.detach().float().cpu().reshape(n, -1) for t in qparams)
        codes = packing.codes_from_fake_quant(w, scales, zeros, bits, g, symmetric)
    weight, s16, z16 = packing.pack_linearq(codes, scales, zeros, bits, symmetric)
    lq = LinearQ(k, n, bits, g, bias=linear.bias is not None).to(linear.weight.device)
    lq.load_quantized_params(s16, z16, weight)
    if linear.bias is not None:
        lq.bias = linear.bias.detach().to(torch.float16).to(linear.weight.device)
    return lq


def convert(model: nn.Module, bits: int = 4, group_size: int = 128, symmetric: bool = False,
            skip: Iterable[str] = (), qparams: Optional[Dict[str, Tuple[torch.Tensor, torch.Tensor]]] = None,
            select: Optional[Callable[[str, nn.Linear], bool]] = None) -> nn.Module:
    """Replaces the ``nn.Linear`` layers of ``model`` by ``LinearQ`` in place and returns ``model``.

    ``skip``: qualified names (or name suffixes) left untouched -- the reference keeps the output head
    in fp16 (``proj_out``, whisper.py:268; ``lm_head``, canary_qwen.py:179).  ``qparams``: name ->
    ``(scales, zeros)`` from the reference's quantization flow; layers not in it are quantised with
    round-to-nearest.  ``select(name, layer)`` may veto individual layers.
    """
    skip = tuple(skip)
    todo = []
    for name, mod in model.named_modules():
        if isinstance(mod, nn.Linear) and not isinstance(mod, LinearQ):
            if any(name == s or name.endswith("." + s) for s in skip):
                continue
            if select is not None and not select(name, mod):
                continue
            g = mod.in_features if group_size == -1 else group_size
            if mod.in_features % g or (mod.in_features * bits) % 8:
                continue  # shapes the packed layout cannot hold stay in floating point
            todo.append((name, mod))
    for name, mod in todo:
        parent = model
        *path, leaf = name.split(".")
        for p in path:
            parent = getattr(parent, p)
        setattr(parent, leaf, linearq_from_linear(mod, bits, group_size, symmetric,
                                                  None if qparams is None else qparams.get(name)))
    return model


class FusedLinearQ(nn.Module):
    """Several ``LinearQ`` layers with the same input as ONE kernel call.

    The parts stay ordinary submodules (``parts.0.weight`` ... in ``state_dict``); their packed rows,
    scales, zeros and biases are concatenated into one set of buffers the first time ``forward`` runs
    and again whenever a part's buffers are replaced or modified in place.  ``forward`` returns one
    tensor per part (views of one output).  All parts must agree on ``in_features``, ``bits`` and
    ``group_size``; either all or none have a bias.
    """

    def __init__(self, parts: Sequence[LinearQ]):
        super().__init__()
        if len(parts) == 0:
            raise ValueError("FusedLinearQ needs at least one part")
        p0 = parts[0]
        for p in parts:
            if (p.in_features, p.bits, p.group_size) != (p0.in_features, p0.bits, p0.group_size):
                raise ValueError("FusedLinearQ: parts differ in in_features, bits or group_size")
        self.parts = nn.ModuleList(parts)
        self._fused: Optional[LinearQ] = None
        self._key = None

    def _fuse(self) -> LinearQ:
        key = tuple((t.data_ptr(), t._version) for p in self.parts
                    for t in (p.weight, p.scales, p.zeros) + (() if p.bias is None else (p.bias,)))
        if self._fused is None or key != self._key:
            p0 = self.parts[0]
            n = sum(p.out_features for p in self.parts)
            any_bias = any(p.bias is not None for p in self.parts)
            f = LinearQ(p0.in_features, n, p0.bits, p0.group_size, bias=any_bias)
            f.weight = torch.cat([p.weight for p in self.parts], dim=0).contiguous()
            f.scales = torch.cat([p.scales for p in self.parts], dim=0).contiguous()
            f.zeros = torch.cat([p.zeros for p in self.parts], dim=0).contiguous()
            if any_bias:
                f.bias = torch.cat([p.bias if p.bias is not None else
                                    torch.zeros(p.out_features, dtype=torch.float16, device=p.weight.device)
                                    for p in self.parts], dim=0).contiguous()
            if f.weight.is_cuda:
                # The decode kernels fetch weights ahead of their stream dependency (programmatic dependent
                # launch): the concatenated buffers must be complete before the first call is enqueued.
                torch.cuda.current_stream(f.weight.device).synchronize()
            # not registered as a submodule: the fused copy must not show up in state_dict
            object.__setattr__(self, "_fused", f)
            self._key = key
        return self._fused

    def forward(self, input):
        y = self._fuse()(input)
        return y.split([p.out_features for p in self.parts], dim=-1)
