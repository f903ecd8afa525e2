"""Whisper with ``LinearQ`` layers: the ``Whisper*Q`` model classes and a CUDA-graph engine.

Two things live here.

* ``WhisperAttentionQ`` ... ``WhisperForConditionalGenerationQ``: the model classes of the reference
  (asrq/models/transformers/whisper.py:38-271) -- stock Hugging Face Whisper modules whose ``nn.Linear``
  layers are ``LinearQ`` (every projection and feed-forward layer; the output head ``proj_out`` stays in
  floating point, whisper.py:268).  Same class names, same ``state_dict`` keys, so a packed checkpoint
  loads into either implementation.  The reference spells every constructor out; here a constructor
  runs the stock one and swaps the linear layers it made, which keeps the classes independent of the
  installed transformers version.  :func:`quantize_whisper` is the step the reference lacks between
  "a float model" and "a ``*Q`` model": round-to-nearest packing of every linear layer.

* :class:`WhisperEngine`: greedy transcription for a batch of utterances with the same arithmetic
  as those classes (checked against them), organised for one B200: q/k/v (and cross-attention k/v)
  run as one ``LinearQ`` call over concatenated rows, the keys and values of both attentions live in
  static caches, and one decoder step -- about 600 kernel launches -- is captured once as a CUDA
  graph and replayed per token with the position read from device memory.  Utterances are
  independent, so several GPUs run one engine each on their share of the batch (``asrq_b200.dp``).
"""
from __future__ import annotations

import math
import os
from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import packing
from .convert import linearq_from_linear
from .linear import LinearQ, add_layernorm, decode_self_attention, dense_head

try:  # the model classes need transformers; the engine does not
    from transformers.models.whisper.modeling_whisper import (WhisperAttention, WhisperConfig, WhisperDecoder,
                                                              WhisperDecoderLayer, WhisperEncoder,
                                                              WhisperEncoderLayer, WhisperForConditionalGeneration,
                                                              WhisperModel)
    _HAVE_HF = True
except Exception:  # pragma: no cover
    _HAVE_HF = False
    WhisperAttention = WhisperDecoder = WhisperDecoderLayer = WhisperEncoder = WhisperEncoderLayer = object
    WhisperForConditionalGeneration = WhisperModel = object
    WhisperConfig = None


# --------------------------------------------------------------------------------------------------
# model classes
# --------------------------------------------------------------------------------------------------

def _swap_direct_linears(module: nn.Module, bits: int, group_size: int) -> None:
    """Replaces the ``nn.Linear`` children of ``module`` (not of its submodules) by empty ``LinearQ``
    layers of the same shape; their buffers are filled by ``load_state_dict`` / ``load_quantized_params``."""
    for name, child in list(module.named_children()):
        if type(child) is nn.Linear:
            setattr(module, name, LinearQ(child.in_features, child.out_features, bits, group_size,
                                          bias=child.bias is not None))


class WhisperAttentionQ(WhisperAttention):
    """asrq/models/transformers/whisper.py:38-97: q/k/v/out projections are ``LinearQ`` (k without bias)."""

    def __init__(self, *args, bits: int = 4, group_size: int = 128, **kwargs):
        super().__init__(*args, **kwargs)
        _swap_direct_linears(self, bits, group_size)


def _swap_attention(layer: nn.Module, names, bits, group_size):
    for name in names:
        a = getattr(layer, name)
        q = WhisperAttentionQ(a.embed_dim, a.num_heads, dropout=a.dropout, is_decoder=a.is_decoder,
                              bias=a.q_proj.bias is not None, is_causal=a.is_causal, layer_idx=a.layer_idx,
                              config=a.config, bits=bits, group_size=group_size)
        setattr(layer, name, q)


class WhisperEncoderLayerQ(WhisperEncoderLayer):
    """whisper.py:100-125: quantized attention, ``fc1`` and ``fc2``; layer norms stay."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        _swap_attention(self, ("self_attn",), bits, group_size)
        _swap_direct_linears(self, bits, group_size)


class WhisperDecoderLayerQ(WhisperDecoderLayer):
    """whisper.py:163-203: quantized self- and cross-attention, ``fc1`` and ``fc2``."""

    def __init__(self, config, layer_idx: Optional[int] = None, bits: int = 4, group_size: int = 128):
        super().__init__(config, layer_idx)
        _swap_attention(self, ("self_attn", "encoder_attn"), bits, group_size)
        _swap_direct_linears(self, bits, group_size)


class WhisperEncoderQ(WhisperEncoder):
    """whisper.py:128-160."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        self.layers = nn.ModuleList([WhisperEncoderLayerQ(config, bits, group_size) for _ in range(config.encoder_layers)])


class WhisperDecoderQ(WhisperDecoder):
    """whisper.py:206-236."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        self.layers = nn.ModuleList([WhisperDecoderLayerQ(config, i, bits, group_size)
                                     for i in range(config.decoder_layers)])


class WhisperModelQ(WhisperModel):
    """whisper.py:239-253."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        self.encoder = WhisperEncoderQ(config, bits, group_size)
        self.decoder = WhisperDecoderQ(config, bits, group_size)


class WhisperForConditionalGenerationQ(WhisperForConditionalGeneration):
    """whisper.py:256-271: quantized backbone, floating-point ``proj_out`` tied to the token embedding."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        self.model = WhisperModelQ(config, bits, group_size)
        self.bits, self.group_size = bits, group_size
        self.tie_weights()


def quantize_whisper(model: nn.Module, bits: int = 4, group_size: int = 128, symmetric: bool = False,
                     qparams: Optional[Dict[str, tuple]] = None) -> "WhisperForConditionalGenerationQ":
    """A float ``WhisperForConditionalGeneration`` -> ``WhisperForConditionalGenerationQ`` with every linear
    layer except ``proj_out`` packed (round-to-nearest on the reference grid, or from the
    ``(scales, zeros)`` a reference quantizer returned for layers it already fake-quantised)."""
    q = WhisperForConditionalGenerationQ(model.config, bits, group_size)
    src = dict(model.named_modules())
    sd = {k: v for k, v in model.state_dict().items()}
    for name, mod in q.named_modules():
        if isinstance(mod, LinearQ):
            packed = linearq_from_linear(src[name], bits, group_size, symmetric,
                                         None if qparams is None else qparams.get(name))
            mod.load_quantized_params(packed.scales, packed.zeros, packed.weight)
            if packed.bias is not None:
                mod.bias = packed.bias
            for suffix in ("weight", "bias"):
                sd.pop(f"{name}.{suffix}", None)
    q.load_state_dict(sd, strict=False)  # everything that is not a quantized layer: convs, norms, embeddings
    q.tie_weights()
    if getattr(model, "generation_config", None) is not None:
        q.generation_config = model.generation_config
    return q.eval()


# --------------------------------------------------------------------------------------------------
# engine
# --------------------------------------------------------------------------------------------------

def _cat_linearq(parts: List[LinearQ]) -> LinearQ:
    """One ``LinearQ`` over the concatenated output rows of ``parts`` (same input, bits and group size);
    parts without a bias contribute zeros."""
    p0 = parts[0]
    dev = p0.weight.device
    any_bias = any(p.bias is not None for p in parts)
    f = LinearQ(p0.in_features, sum(p.out_features for p in parts), p0.bits, p0.group_size, bias=any_bias)
    f.weight = torch.cat([p.weight for p in parts], 0).contiguous()
    f.scales = torch.cat([p.scales for p in parts], 0).contiguous()
    f.zeros = torch.cat([p.zeros for p in parts], 0).contiguous()
    if any_bias:
        f.bias = torch.cat([p.bias if p.bias is not None else torch.zeros(p.out_features, dtype=torch.float16, device=dev)
                            for p in parts], 0).contiguous()
    return f


class _Norm:
    """Layer norm through the library's kernel (one launch; fp32 statistics, 16-bit in and out)."""
    __slots__ = ("w", "b", "eps")

    def __init__(self, w, b, eps=1e-5):
        self.w, self.b, self.eps = w, b, eps

    def __call__(self, x):
        return add_layernorm(x, None, self.w, self.b, self.eps)[1]


def _fold_query_scale(lq: LinearQ, rows: int, s: float) -> bool:
    """Folds the attention's query scaling (head_dim ** -0.5) into the first ``rows`` output rows of a layer:
    (x W^T + b) * s == x (s W)^T + s b, with s W expressed by scaling the group scales and zeros.  Done only
    when ``s`` is a power of two and every scaled scale and zero stays exactly representable (then the layer's
    fp32 sums are scaled exactly); bias values whose product falls below the fp16 normal range are rounded
    (absolute error <= 2^-25).  Returns whether the scaling was folded; otherwise the caller multiplies."""
    if s <= 0 or math.frexp(s)[0] != 0.5:
        return False
    sc, ze = lq.scales[:rows].float() * s, lq.zeros[:rows].float() * s
    if not (torch.equal(sc.half().float(), sc) and torch.equal(ze.half().float(), ze)):
        return False
    lq.scales[:rows] = sc.half()
    lq.zeros[:rows] = ze.half()
    if lq.bias is not None:
        lq.bias[:rows] = (lq.bias[:rows].float() * s).half()
    return True


class WhisperEngine:
    """Greedy decoding of a batch of 30-second windows on one GPU.

    ``input_features`` (batch, mel bins, 2 * max_source_positions) -> token ids (batch, steps).  The
    arithmetic follows the model classes above layer by layer (pre-norm blocks, query scaled before the
    attention, fp16 clamp after each encoder layer, tied output head); what differs is the schedule:
    fused projections, static key/value caches, and a decoder step captured as one CUDA graph.
    End-of-sequence is not interpreted: every utterance runs ``steps`` tokens (callers cut at the first
    end-of-sequence id), which is also how the throughput benchmark wants it.
    """

    fused_self_attention = os.environ.get("ASRQ_B200_WHISPER_FUSED_SELF_ATTENTION", "1") == "1"
    cross_kv_views = os.environ.get("ASRQ_B200_WHISPER_CROSS_KV_VIEWS", "1") == "1"

    def __init__(self, config, device, dtype=torch.float16):
        self.cfg = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.d = config.d_model
        self.heads_e, self.heads_d = config.encoder_attention_heads, config.decoder_attention_heads
        self.enc_layers: List[dict] = []
        self.dec_layers: List[dict] = []
        self._graph = None
        self._graph_key = None

    # ---- construction -------------------------------------------------------------------------
    @classmethod
    def from_model(cls, model, device=None, dtype=torch.float16) -> "WhisperEngine":
        """From a ``WhisperForConditionalGenerationQ`` (these classes' or a packed checkpoint loaded into them)."""
        device = torch.device(device) if device is not None else next(model.parameters()).device
        eng = cls(model.config, device, dtype)
        enc, dec = model.model.encoder, model.model.decoder

        def t(x):
            return x.detach().to(device=device, dtype=dtype).contiguous()

        def lq(m):
            return m.to(device)

        def norm(m):
            return _Norm(t(m.weight), t(m.bias), m.eps)

        eng.conv1_w, eng.conv1_b = t(enc.conv1.weight), t(enc.conv1.bias)
        eng.conv2_w, eng.conv2_b = t(enc.conv2.weight), t(enc.conv2.bias)
        eng.enc_pos = t(enc.embed_positions.weight)
        for L in enc.layers:
            a = L.self_attn
            eng.enc_layers.append(dict(ln1=norm(L.self_attn_layer_norm), qkv=_cat_linearq([lq(a.q_proj), lq(a.k_proj), lq(a.v_proj)]),
                                       out=lq(a.out_proj), ln2=norm(L.final_layer_norm), fc1=lq(L.fc1), fc2=lq(L.fc2)))
        eng.enc_ln = norm(enc.layer_norm)
        eng.embed = t(dec.embed_tokens.weight)
        eng.dec_pos = t(dec.embed_positions.weight)
        for L in dec.layers:
            a, c = L.self_attn, L.encoder_attn
            eng.dec_layers.append(dict(
                ln1=norm(L.self_attn_layer_norm), qkv=_cat_linearq([lq(a.q_proj), lq(a.k_proj), lq(a.v_proj)]), out=lq(a.out_proj),
                lnx=norm(L.encoder_attn_layer_norm), xq=_cat_linearq([lq(c.q_proj)]), xkv=_cat_linearq([lq(c.k_proj), lq(c.v_proj)]), xout=lq(c.out_proj),
                ln2=norm(L.final_layer_norm), fc1=lq(L.fc1), fc2=lq(L.fc2)))
        eng.dec_ln = norm(dec.layer_norm)
        eng.head = t(model.proj_out.weight)
        eng._finalize()
        return eng

    @classmethod
    def random_init(cls, config, device, seed: int = 0, bits: int = 4, group_size: int = 128,
                    dtype=torch.float16) -> "WhisperEngine":
        """A model of ``config``'s architecture with seeded N(0, 0.02) weights, generated and packed on
        the device (round-to-nearest, asymmetric): the stand-in for a checkpoint that cannot be
        downloaded.  Layer norms start at (1, 0), the token embedding doubles as the output head."""
        device = torch.device(device)
        eng = cls(config, device, dtype)
        gen = torch.Generator(device=device).manual_seed(seed)
        d, ffe, ffd = config.d_model, config.encoder_ffn_dim, config.decoder_ffn_dim

        def rnd(*shape, std=0.02):
            return (torch.randn(*shape, generator=gen, device=device) * std).to(dtype)

        def qlin(n, k, bias_mask=None):
            w = torch.randn(n, k, generator=gen, device=device) * 0.02
            codes, scales, zeros = packing.rtn_quantize(w.to(dtype), bits, group_size, False)
            weight, s16, z16 = packing.pack_linearq(codes, scales, zeros, bits, False)
            m = LinearQ(k, n, bits, group_size, bias=True).to(device)
            m.load_quantized_params(s16, z16, weight)
            b = rnd(n)
            if bias_mask is not None:
                b = b * bias_mask
            m.bias = b.to(torch.float16)
            return m

        def norm():
            return _Norm(torch.ones(d, device=device, dtype=dtype), torch.zeros(d, device=device, dtype=dtype))

        def qkv_mask():  # k has no bias
            m = torch.ones(3 * d, device=device, dtype=dtype)
            m[d:2 * d] = 0
            return m

        eng.conv1_w, eng.conv1_b = rnd(d, config.num_mel_bins, 3), rnd(d)
        eng.conv2_w, eng.conv2_b = rnd(d, d, 3), rnd(d)
        eng.enc_pos = rnd(config.max_source_positions, d)
        for _ in range(config.encoder_layers):
            eng.enc_layers.append(dict(ln1=norm(), qkv=qlin(3 * d, d, qkv_mask()), out=qlin(d, d), ln2=norm(),
                                       fc1=qlin(ffe, d), fc2=qlin(d, ffe)))
        eng.enc_ln = norm()
        eng.embed = rnd(config.vocab_size, d)
        eng.dec_pos = rnd(config.max_target_positions, d)
        kv_mask = torch.ones(2 * d, device=device, dtype=dtype)
        kv_mask[:d] = 0
        for _ in range(config.decoder_layers):
            eng.dec_layers.append(dict(ln1=norm(), qkv=qlin(3 * d, d, qkv_mask()), out=qlin(d, d), lnx=norm(),
                                       xq=qlin(d, d), xkv=qlin(2 * d, d, kv_mask), xout=qlin(d, d), ln2=norm(),
                                       fc1=qlin(ffd, d), fc2=qlin(d, ffd)))
        eng.dec_ln = norm()
        eng.head = eng.embed
        eng._finalize()
        return eng

    def _finalize(self):
        """After the layers exist: fold the query scaling into the projections where that is exact."""
        se, sd = (self.d // self.heads_e) ** -0.5, (self.d // self.heads_d) ** -0.5
        for L in self.enc_layers:
            L["q_folded"] = _fold_query_scale(L["qkv"], self.d, se)
        for L in self.dec_layers:
            L["q_folded"] = _fold_query_scale(L["qkv"], self.d, sd)
            L["xq_folded"] = _fold_query_scale(L["xq"], self.d, sd)
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()  # weights complete before any launch prefetches them

    def linear_layers(self) -> List[LinearQ]:
        out = []
        for L in self.enc_layers + self.dec_layers:
            out += [v for v in L.values() if isinstance(v, LinearQ)]
        return out

    # ---- encoder ------------------------------------------------------------------------------
    def _attend(self, q, k, v, heads, mask=None):
        """q (B, Tq, d) already scaled; k, v (B, H, Tk, hd).  Returns (B, Tq, d)."""
        b, tq, _ = q.shape
        qh = q.view(b, tq, heads, -1).transpose(1, 2)
        o = F.scaled_dot_product_attention(qh, k, v, attn_mask=mask, scale=1.0)
        return o.transpose(1, 2).reshape(b, tq, -1)

    def _split_heads(self, x, heads):
        b, t, _ = x.shape
        return x.view(b, t, heads, -1).transpose(1, 2)

    @torch.no_grad()
    def encode(self, input_features: torch.Tensor) -> torch.Tensor:
        """(B, mel, frames) -> encoder states (B, frames / 2, d)."""
        x = input_features.to(device=self.device, dtype=self.dtype)
        x = F.gelu(F.conv1d(x, self.conv1_w, self.conv1_b, padding=1))
        x = F.gelu(F.conv1d(x, self.conv2_w, self.conv2_b, stride=2, padding=1))
        x = (x.permute(0, 2, 1) + self.enc_pos).contiguous()
        scaling = (self.d // self.heads_e) ** -0.5
        clamp = torch.finfo(torch.float16).max - 1000 if self.dtype == torch.float16 else None
        for L in self.enc_layers:
            h = L["ln1"](x)
            q, k, v = L["qkv"](h).split(self.d, dim=-1)
            if not L["q_folded"]:
                q = q * scaling
            a = self._attend(q, self._split_heads(k, self.heads_e), self._split_heads(v, self.heads_e), self.heads_e)
            x = L["out"].forward_fused(a, residual=x)              # x + out_proj(a) in the kernel's epilogue
            h = L["ln2"](x)
            x = L["fc2"].forward_fused(L["fc1"].forward_fused(h, gelu=True), residual=x)
            if clamp is not None:
                x = torch.clamp(x, min=-clamp, max=clamp)
        return self.enc_ln(x)

    # ---- decoder ------------------------------------------------------------------------------
    def _alloc(self, batch: int, src_len: int, max_len: int):
        key = (batch, src_len, max_len)
        if getattr(self, "_alloc_key", None) == key:
            return
        dev, dt, nl = self.device, self.dtype, len(self.dec_layers)
        hd = self.d // self.heads_d
        self.kv_self = torch.zeros(nl, 2, batch, self.heads_d, max_len, hd, device=dev, dtype=dt)  # keys, values
        if self.cross_kv_views:
            # the cross-attention keys and values stay where the fused projection wrote them, (B, T, [k | v]); the attention
            # reads them through head-major views (128-byte runs per head and position)
            self.xkv = torch.empty(nl, batch, src_len, 2 * self.d, device=dev, dtype=dt)
            kv = self.xkv.view(nl, batch, src_len, 2, self.heads_d, hd)
            self.k_cross = kv[:, :, :, 0].permute(0, 1, 3, 2, 4)   # (layer, B, H, T, hd) views
            self.v_cross = kv[:, :, :, 1].permute(0, 1, 3, 2, 4)
        else:
            self.k_cross = torch.empty(nl, batch, self.heads_d, src_len, hd, device=dev, dtype=dt)
            self.v_cross = torch.empty_like(self.k_cross)
        self.tok = torch.zeros(batch, dtype=torch.long, device=dev)      # token fed to the next step
        self.pos = torch.zeros(1, dtype=torch.long, device=dev)          # its position
        self.mask = torch.full((1, 1, 1, max_len), float("-inf"), device=dev, dtype=dt)  # 0 where a key exists
        self.out_ids = torch.zeros(max_len, batch, dtype=torch.long, device=dev)
        self.logits = torch.empty(batch, self.head.shape[0], device=dev, dtype=dt)
        self._alloc_key = key
        self._graph = None

    @torch.no_grad()
    def _cross_kv(self, enc: torch.Tensor):
        """Keys and values of every decoder layer's cross-attention, once per batch."""
        b, t, _ = enc.shape
        hd = self.d // self.heads_d
        for i, L in enumerate(self.dec_layers):
            if self.cross_kv_views:
                self.xkv[i].copy_(L["xkv"](enc))
                continue
            k, v = L["xkv"](enc).split(self.d, dim=-1)
            self.k_cross[i].copy_(k.view(b, t, self.heads_d, hd).transpose(1, 2))
            self.v_cross[i].copy_(v.view(b, t, self.heads_d, hd).transpose(1, 2))

    def _step(self):
        """One decoder step on the static buffers: reads ``tok`` and ``pos``, writes the key and value of
        that position, the logits, the next token into ``tok`` and ``out_ids[pos]``, and advances
        ``pos``.  Every shape is fixed and every index comes from device memory, so the sequence of
        launches is the same for every token."""
        b = self.tok.shape[0]
        hd = self.d // self.heads_d
        scaling = hd ** -0.5
        if not self.fused_self_attention:
            self.mask.index_fill_(3, self.pos, 0.0)
        x = (self.embed[self.tok] + self.dec_pos[self.pos]).unsqueeze(1)  # (B, 1, d)
        for i, L in enumerate(self.dec_layers):
            h = L["ln1"](x)
            qkv = L["qkv"](h)
            if self.fused_self_attention:
                # this position's key and value into the cache and the attention over the cache: one kernel
                a = decode_self_attention(qkv, self.kv_self[i], self.pos, 1.0 if L["q_folded"] else scaling).unsqueeze(1)
            else:
                q = qkv[..., :self.d]
                if not L["q_folded"]:
                    q = q * scaling
                self.kv_self[i].index_copy_(3, self.pos, qkv[..., self.d:].view(b, 1, 2, self.heads_d, hd).permute(2, 0, 3, 1, 4))
                a = self._attend(q, self.kv_self[i, 0], self.kv_self[i, 1], self.heads_d, self.mask)
            x = L["out"].forward_fused(a, residual=x)
            h = L["lnx"](x)
            q = L["xq"](h)
            if not L["xq_folded"]:
                q = q * scaling
            a = self._attend(q, self.k_cross[i], self.v_cross[i], self.heads_d)
            x = L["xout"].forward_fused(a, residual=x)
            h = L["ln2"](x)
            x = L["fc2"].forward_fused(L["fc1"].forward_fused(h, gelu=True), residual=x)
        x = self.dec_ln(x).squeeze(1)
        dense_head(x, self.head, out=self.logits)
        nxt = torch.argmax(self.logits, dim=-1)
        self.out_ids.index_copy_(0, self.pos, nxt.unsqueeze(0))
        self.tok.copy_(nxt)
        self.pos.add_(1)

    def _ensure_graph(self):
        if self._graph is not None:
            return
        # warm-up on a side stream (lazy initialisation inside libraries must not happen under capture),
        # then capture; the buffers are reset by generate() before every use
        side = torch.cuda.Stream(self.device)
        side.wait_stream(torch.cuda.current_stream(self.device))
        with torch.cuda.stream(side):
            for _ in range(2):
                self.pos.zero_()
                self._step()
            side.synchronize()
            g = torch.cuda.CUDAGraph()
            self.pos.zero_()
            with torch.cuda.graph(g, stream=side):
                self._step()
        torch.cuda.current_stream(self.device).wait_stream(side)
        self._graph = g

    @torch.no_grad()
    def decode(self, enc: torch.Tensor, steps: int, start_token: Optional[int] = None, use_graph: bool = True,
               forced_ids: Optional[torch.Tensor] = None, keep_logits: bool = False):
        """Greedy decoding from ``start_token`` for ``steps`` tokens.  ``forced_ids`` (steps, B) feeds a given
        token sequence instead of the argmax (teacher forcing, for parity checks); ``keep_logits`` returns
        the per-step logits as well (steps, B, vocab)."""
        b, t, _ = enc.shape
        max_len = steps + 1
        if max_len > self.dec_pos.shape[0]:
            raise ValueError(f"{steps} steps exceed the model's {self.dec_pos.shape[0]} target positions")
        with torch.cuda.device(self.device):
            self._alloc(b, t, max_len)
            self._cross_kv(enc)
            start = self.cfg.decoder_start_token_id if start_token is None else start_token
            self.tok.fill_(start)
            self.pos.zero_()
            self.mask.fill_(float("-inf"))
            graph = use_graph and forced_ids is None and not keep_logits
            if graph:
                self._ensure_graph()
                self.tok.fill_(start)
                self.pos.zero_()
                self.mask.fill_(float("-inf"))
            all_logits = []
            for s in range(steps):
                if graph:
                    self._graph.replay()
                else:
                    self._step()
                    if keep_logits:
                        all_logits.append(self.logits.clone())
                    if forced_ids is not None:
                        self.tok.copy_(forced_ids[s].to(self.device))
            ids = self.out_ids[:steps].t().contiguous()
        return (ids, torch.stack(all_logits)) if keep_logits else ids

    @torch.no_grad()
    def generate(self, input_features: torch.Tensor, steps: int = 128, use_graph: bool = True) -> torch.Tensor:
        """Token ids (B, steps) for a batch of log-mel windows (host or device tensor)."""
        with torch.cuda.device(self.device):
            enc = self.encode(input_features)
            return self.decode(enc, steps, use_graph=use_graph)


def audio_seconds(config, batch: int) -> float:
    """Seconds of audio in a batch of full windows: 2 frames per source position, 100 frames per second."""
    return batch * config.max_source_positions * 2 / 100.0


def rtfx(config, batch: int, wall_seconds: float) -> float:
    """Inverse real-time factor as the reference's evaluation defines it: total audio seconds divided by
    the seconds spent transcribing them (asrq/evaluation/openasr.py:481-483)."""
    return audio_seconds(config, batch) / wall_seconds
