"""A FastConformer-shaped encoder whose linear layers are ``LinearQQ`` (W4A4 with the online Hadamard rotation),
and the speech-to-text pipeline that feeds its output to a :class:`asrq_b200.qwen3.Qwen3Engine`.

The reference's Canary-Qwen model takes its encoder body from NeMo (asrq/models/nemo/conformerq.py imports the
NeMo ConformerEncoder and only replaces its linear layers: feed-forward ``linear1``/``linear2`` at
conformerq.py:73-76, attention ``linear_q/k/v/out/pos`` at conformerq.py:259-262); NeMo is neither installed nor part
of the reference's tree, so this is a **stand-in of the same shape**, not that encoder: the layer structure of a
Conformer block (half-step feed-forward, self-attention, convolution module, half-step feed-forward, layer norm),
its widths (d_model 1024, feed-forward 4096, 8 heads, convolution kernel 9, 8x time subsampling), and exactly the
quantized call sites of the reference -- seven ``LinearQQ`` per block -- with plain torch operations for the rest.
Two simplifications are stated rather than hidden: the subsampling is three strided 1-D convolutions, and the
relative-position term of the attention is reduced to the projected positional embedding added to the keys
(``linear_pos`` keeps its call site and shape).  It exists to run the quantized layers at the call-site shapes of
the whole model (M = batch x 250 tokens) inside a realistic launch sequence; parity is judged per ``LinearQQ`` call
and against this same model evaluated with the CPU oracle's layers.
"""
from __future__ import annotations

import math
from typing import List, Optional

import torch
import torch.nn.functional as F

from . import packing
from .linear import LinearQQ


class FastConformerStandIn:
    """log-mel (B, mel, frames) -> encoder states (B, frames / 8, d_model).  Weights are seeded N(0, 0.02), generated
    and packed on the device (Hadamard fold + symmetric int4 round-to-nearest, g128)."""

    def __init__(self, device, n_layers: int = 32, d_model: int = 1024, ffn: int = 4096, heads: int = 8, mel: int = 80,
                 conv_kernel: int = 9, sub_channels: int = 256, seed: int = 0, dtype=torch.float16, group_size: int = 128):
        self.device = torch.device(device)
        self.dtype, self.d, self.ffn, self.heads, self.mel = dtype, d_model, ffn, heads, mel
        gen = torch.Generator(device=self.device).manual_seed(seed)
        dev = self.device

        def rnd(*shape, std=0.02):
            return (torch.randn(*shape, generator=gen, device=dev) * std).to(dtype)

        def qq(n, k, bias=True):
            w = torch.randn(n, k, generator=gen, device=dev) * 0.02
            weight, scales = packing.pack_w4a4_cuda(w, group_size, True)
            m = LinearQQ(k, n, 4, 4, group_size, bias=bias, hadamard=True).to(dev)
            m.load_quantized_params(scales, torch.zeros_like(scales), weight)
            if bias:
                m.bias = rnd(n).to(torch.float16)
            return m

        def ln():
            return (torch.ones(d_model, device=dev, dtype=dtype), torch.zeros(d_model, device=dev, dtype=dtype))

        c = sub_channels
        self.sub = [(rnd(c, mel, 3, std=0.05), rnd(c)), (rnd(c, c, 3, std=0.05), rnd(c)), (rnd(c, c, 3, std=0.05), rnd(c))]
        self.sub_out = (rnd(d_model, c, std=0.05), rnd(d_model))
        self.layers: List[dict] = []
        for _ in range(n_layers):
            self.layers.append(dict(
                ln_ff1=ln(), ff1_a=qq(ffn, d_model), ff1_b=qq(d_model, ffn),
                ln_att=ln(), q=qq(d_model, d_model), k=qq(d_model, d_model), v=qq(d_model, d_model), out=qq(d_model, d_model),
                pos=qq(d_model, d_model, bias=False),
                ln_conv=ln(), pw1=(rnd(2 * d_model, d_model, 1), rnd(2 * d_model)), dw=(rnd(d_model, 1, conv_kernel, std=0.1), rnd(d_model)),
                bn=(torch.ones(d_model, device=dev, dtype=dtype), torch.zeros(d_model, device=dev, dtype=dtype)),
                pw2=(rnd(d_model, d_model, 1), rnd(d_model)),
                ln_ff2=ln(), ff2_a=qq(ffn, d_model), ff2_b=qq(d_model, ffn), ln_out=ln()))
        self.conv_kernel = conv_kernel
        torch.cuda.current_stream(self.device).synchronize()

    def linear_layers(self) -> List[LinearQQ]:
        return [L[k] for L in self.layers for k in ("ff1_a", "ff1_b", "q", "k", "v", "out", "pos", "ff2_a", "ff2_b")]

    def _pos_emb(self, t: int) -> torch.Tensor:
        pos = torch.arange(t, device=self.device, dtype=torch.float32).unsqueeze(1)
        div = torch.exp(torch.arange(0, self.d, 2, device=self.device, dtype=torch.float32) * (-math.log(10000.0) / self.d))
        pe = torch.zeros(t, self.d, device=self.device, dtype=torch.float32)
        pe[:, 0::2] = torch.sin(pos * div)
        pe[:, 1::2] = torch.cos(pos * div)
        return pe.to(self.dtype)

    def subsample(self, feats: torch.Tensor) -> torch.Tensor:
        x = feats.to(device=self.device, dtype=self.dtype)
        for w, b in self.sub:
            x = F.relu(F.conv1d(x, w, b, stride=2, padding=1))
        return F.linear(x.transpose(1, 2), *self.sub_out)          # (B, T/8, d)

    def block(self, L: dict, x: torch.Tensor, pe: torch.Tensor, hook=None) -> torch.Tensor:
        """One Conformer block.  ``hook(name, layer, input, output)`` sees every quantized call (parity checks)."""
        def lin(name, inp):
            out = L[name](inp)
            if hook is not None:
                hook(name, L[name], inp, out)
            return out
        b, t, d = x.shape
        h = F.layer_norm(x, (d,), *L["ln_ff1"])
        x = x + 0.5 * lin("ff1_b", F.silu(lin("ff1_a", h)))
        h = F.layer_norm(x, (d,), *L["ln_att"])
        q, k, v = lin("q", h), lin("k", h), lin("v", h)
        k = k + lin("pos", pe).unsqueeze(0)
        hd = d // self.heads
        sp = lambda z: z.view(b, t, self.heads, hd).transpose(1, 2)  # noqa: E731
        a = F.scaled_dot_product_attention(sp(q), sp(k), sp(v)).transpose(1, 2).reshape(b, t, d)
        x = x + lin("out", a)
        h = F.layer_norm(x, (d,), *L["ln_conv"]).transpose(1, 2)
        h = F.glu(F.conv1d(h, *L["pw1"]), dim=1)
        h = F.conv1d(h, *L["dw"], padding=self.conv_kernel // 2, groups=d)
        h = F.silu(h * L["bn"][0].view(1, -1, 1) + L["bn"][1].view(1, -1, 1))
        x = x + F.conv1d(h, *L["pw2"]).transpose(1, 2)
        h = F.layer_norm(x, (d,), *L["ln_ff2"])
        x = x + 0.5 * lin("ff2_b", F.silu(lin("ff2_a", h)))
        return F.layer_norm(x, (d,), *L["ln_out"])

    @torch.no_grad()
    def encode(self, feats: torch.Tensor, hook=None) -> torch.Tensor:
        with torch.cuda.device(self.device):
            x = self.subsample(feats)
            pe = self._pos_emb(x.shape[1])
            for L in self.layers:
                x = self.block(L, x, pe, hook)
            return x


class SpeechLM:
    """Encoder stand-in -> projection to the decoder's width -> ``Qwen3Engine`` greedy decoding: the data flow of the
    reference's Canary-Qwen model (audio frames become the first embeddings of the decoder's prompt,
    asrq/models/nemo/canary_qwen.py:185-330) at its shapes."""

    def __init__(self, encoder: FastConformerStandIn, decoder, prompt_tokens: int = 8, seed: int = 0):
        self.enc, self.dec = encoder, decoder
        dev, dt = encoder.device, encoder.dtype
        gen = torch.Generator(device=dev).manual_seed(seed + 17)
        self.proj_w = (torch.randn(decoder.hidden, encoder.d, generator=gen, device=dev) * 0.02).to(dt)
        self.proj_b = torch.zeros(decoder.hidden, device=dev, dtype=dt)
        self.prompt_ids = torch.randint(0, decoder.embed.shape[0], (prompt_tokens,), generator=gen, device=dev)

    @torch.no_grad()
    def prompt_embeddings(self, feats: torch.Tensor) -> torch.Tensor:
        e = self.enc.encode(feats)
        a = F.linear(e, self.proj_w, self.proj_b)
        p = self.dec.embed[self.prompt_ids].unsqueeze(0).expand(a.shape[0], -1, -1)
        return torch.cat([a, p], dim=1).contiguous()

    @torch.no_grad()
    def generate(self, feats: torch.Tensor, steps: int = 200, use_graph: bool = True) -> torch.Tensor:
        with torch.cuda.device(self.enc.device):
            return self.dec.generate(self.prompt_embeddings(feats), steps, use_graph=use_graph)


def audio_seconds(batch: int, frames: int) -> float:
    """Seconds of audio in a batch of log-mel windows at 100 frames per second."""
    return batch * frames / 100.0
