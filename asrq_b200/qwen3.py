"""Qwen3 with ``LinearQ`` layers: the ``Qwen3*Q`` model classes and a CUDA-graph decoding engine.

* ``Qwen3MLPQ`` ... ``Qwen3ForCausalLMQ``: the decoder classes of the reference's Canary-Qwen model
  (asrq/models/nemo/canary_qwen.py:70-182) -- stock Hugging Face Qwen3 modules whose q/k/v/o and
  gate/up/down projections are ``LinearQ``; norms, rotary embedding, token embedding and ``lm_head`` stay in
  floating point (canary_qwen.py:179).  Same class names and ``state_dict`` keys.  As in
  ``asrq_b200.whisper`` a constructor runs the stock one and swaps the linear layers it made.
  :func:`quantize_qwen3` packs a float model into these classes (round-to-nearest on the reference grid).

* :class:`Qwen3Engine`: greedy decoding for a batch of sequences that start from given input embeddings
  (in the speech model: projected encoder frames followed by the prompt's token embeddings).  The
  arithmetic follows the classes above; the schedule is this library's: q/k/v and gate/up as one
  ``LinearQ`` call each, residual add + RMS norm and the gated activation as one kernel each, static
  key/value caches, one CUDA graph per decoding step.
"""
from __future__ import annotations

from typing import Dict, List, Optional

import torch
import torch.nn as nn
import torch.nn.functional as F

from . import packing
from .convert import linearq_from_linear
from .linear import LinearQ, add_rmsnorm, dense_head, qk_norm_rope, silu_mul
from .whisper import _cat_linearq

try:
    from transformers.models.qwen3.modeling_qwen3 import (Qwen3Attention, Qwen3Config, Qwen3DecoderLayer,
                                                          Qwen3ForCausalLM, Qwen3MLP, Qwen3Model)
    _HAVE_HF = True
except Exception:  # pragma: no cover
    _HAVE_HF = False
    Qwen3Attention = Qwen3DecoderLayer = Qwen3ForCausalLM = Qwen3MLP = Qwen3Model = object
    Qwen3Config = None


def _swap_direct_linears(module: nn.Module, bits: int, group_size: int) -> None:
    for name, child in list(module.named_children()):
        if type(child) is nn.Linear:
            setattr(module, name, LinearQ(child.in_features, child.out_features, bits, group_size,
                                          bias=child.bias is not None))


class Qwen3MLPQ(Qwen3MLP):
    """canary_qwen.py:70-86: gate, up and down projections are ``LinearQ`` (no bias)."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        _swap_direct_linears(self, bits, group_size)


class Qwen3AttentionQ(Qwen3Attention):
    """canary_qwen.py:89-120: q/k/v/o projections are ``LinearQ``; the per-head q and k norms stay."""

    def __init__(self, config, layer_idx: int, bits: int = 4, group_size: int = 128):
        super().__init__(config, layer_idx)
        _swap_direct_linears(self, bits, group_size)


class Qwen3DecoderLayerQ(Qwen3DecoderLayer):
    """canary_qwen.py:123-139."""

    def __init__(self, config, layer_idx: int, bits: int = 4, group_size: int = 128):
        super().__init__(config, layer_idx)
        self.self_attn = Qwen3AttentionQ(config, layer_idx, bits, group_size)
        self.mlp = Qwen3MLPQ(config, bits, group_size)


class Qwen3ModelQ(Qwen3Model):
    """canary_qwen.py:142-164."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        self.layers = nn.ModuleList([Qwen3DecoderLayerQ(config, i, bits, group_size)
                                     for i in range(config.num_hidden_layers)])


class Qwen3ForCausalLMQ(Qwen3ForCausalLM):
    """canary_qwen.py:167-182: quantized backbone, floating-point ``lm_head``."""

    def __init__(self, config, bits: int = 4, group_size: int = 128):
        super().__init__(config)
        self.model = Qwen3ModelQ(config, bits, group_size)
        self.bits, self.group_size = bits, group_size


def quantize_qwen3(model: nn.Module, bits: int = 4, group_size: int = 128, symmetric: bool = False,
                   qparams: Optional[Dict[str, tuple]] = None) -> "Qwen3ForCausalLMQ":
    """A float ``Qwen3ForCausalLM`` -> ``Qwen3ForCausalLMQ`` with every projection packed (``lm_head`` excepted)."""
    q = Qwen3ForCausalLMQ(model.config, bits, group_size)
    src = dict(model.named_modules())
    sd = dict(model.state_dict())
    for name, mod in q.named_modules():
        if isinstance(mod, LinearQ):
            packed = linearq_from_linear(src[name], bits, group_size, symmetric,
                                         None if qparams is None else qparams.get(name))
            mod.load_quantized_params(packed.scales, packed.zeros, packed.weight)
            if packed.bias is not None:
                mod.bias = packed.bias
            for suffix in ("weight", "bias"):
                sd.pop(f"{name}.{suffix}", None)
    q.load_state_dict(sd, strict=False)
    if getattr(model, "generation_config", None) is not None:
        q.generation_config = model.generation_config
    return q.eval()


# --------------------------------------------------------------------------------------------------
# engine
# --------------------------------------------------------------------------------------------------

def _rms(x: torch.Tensor, w: torch.Tensor, eps: float) -> torch.Tensor:
    """The norm module's arithmetic on the last dimension (used for the per-head q and k norms)."""
    f = x.float()
    return w * (f * torch.rsqrt(f.pow(2).mean(-1, keepdim=True) + eps)).to(x.dtype)


def _rope(x: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor) -> torch.Tensor:
    """x: (batch, heads, T, head_dim); cos, sin: (T, head_dim) or (batch, 1, T, head_dim)."""
    h = x.shape[-1] // 2
    rot = torch.cat((-x[..., h:], x[..., :h]), dim=-1)
    return x * cos + rot * sin


class Qwen3Engine:
    """Greedy decoding of a batch on one GPU: ``prefill(inputs_embeds)`` then ``decode(steps)``.

    All sequences of a batch have the same prompt length (the speech model's prompts do: a fixed number of
    encoder frames plus a fixed text prompt).  End-of-sequence is not interpreted; callers cut the ids.
    """

    def __init__(self, config, device, dtype=torch.float16):
        self.cfg = config
        self.device = torch.device(device)
        self.dtype = dtype
        self.hidden = config.hidden_size
        self.nq, self.nkv = config.num_attention_heads, config.num_key_value_heads
        self.hd = getattr(config, "head_dim", None) or config.hidden_size // config.num_attention_heads
        self.eps = config.rms_norm_eps
        self.layers: List[dict] = []
        self._graph = None
        self._graph_key = None

    # ---- construction -------------------------------------------------------------------------
    def _rotary_table(self, max_len: int):
        theta = getattr(self.cfg, "rope_theta", None)
        if theta is None:
            rp = getattr(self.cfg, "rope_parameters", None) or {}
            theta = rp.get("rope_theta", 1000000.0)
        inv = 1.0 / (theta ** (torch.arange(0, self.hd, 2, dtype=torch.float32, device=self.device) / self.hd))
        fr = torch.outer(torch.arange(max_len, dtype=torch.float32, device=self.device), inv)
        emb = torch.cat((fr, fr), dim=-1)
        self.cos, self.sin = emb.cos().to(self.dtype), emb.sin().to(self.dtype)

    @classmethod
    def from_model(cls, model, device=None, dtype=torch.float16) -> "Qwen3Engine":
        """From a ``Qwen3ForCausalLMQ``."""
        device = torch.device(device) if device is not None else next(model.parameters()).device
        eng = cls(model.config, device, dtype)

        def t(x):
            return x.detach().to(device=device, dtype=dtype).contiguous()

        for L in model.model.layers:
            a, m = L.self_attn, L.mlp
            eng.layers.append(dict(
                ln1=t(L.input_layernorm.weight), qkv=_cat_linearq([a.q_proj.to(device), a.k_proj.to(device), a.v_proj.to(device)]),
                qn=t(a.q_norm.weight), kn=t(a.k_norm.weight), o=a.o_proj.to(device), ln2=t(L.post_attention_layernorm.weight),
                gu=_cat_linearq([m.gate_proj.to(device), m.up_proj.to(device)]), down=m.down_proj.to(device)))
        eng.norm = t(model.model.norm.weight)
        eng.embed = t(model.model.embed_tokens.weight)
        eng.head = t(model.lm_head.weight)
        eng._finalize()
        return eng

    @classmethod
    def random_init(cls, config, device, seed: int = 0, bits: int = 4, group_size: int = 128, dtype=torch.float16) -> "Qwen3Engine":
        """Seeded N(0, 0.02) weights generated and packed on the device (round-to-nearest, asymmetric): the stand-in
        for a checkpoint that cannot be downloaded.  Norm weights start at one; the head is tied to the embedding
        when the configuration says so."""
        device = torch.device(device)
        eng = cls(config, device, dtype)
        gen = torch.Generator(device=device).manual_seed(seed)
        H, I = config.hidden_size, config.intermediate_size

        def qlin(n, k):
            w = torch.randn(n, k, generator=gen, device=device) * 0.02
            codes, scales, zeros = packing.rtn_quantize(w.to(dtype), bits, group_size, False)
            weight, s16, z16 = packing.pack_linearq(codes, scales, zeros, bits, False)
            m = LinearQ(k, n, bits, group_size, bias=False).to(device)
            m.load_quantized_params(s16, z16, weight)
            return m

        ones = lambda n: torch.ones(n, device=device, dtype=dtype)  # noqa: E731
        for _ in range(config.num_hidden_layers):
            eng.layers.append(dict(ln1=ones(H), qkv=qlin((eng.nq + 2 * eng.nkv) * eng.hd, H), qn=ones(eng.hd), kn=ones(eng.hd),
                                   o=qlin(H, eng.nq * eng.hd), ln2=ones(H), gu=qlin(2 * I, H), down=qlin(H, I)))
        eng.norm = ones(H)
        eng.embed = (torch.randn(config.vocab_size, H, generator=gen, device=device) * 0.02).to(dtype)
        eng.head = eng.embed if getattr(config, "tie_word_embeddings", False) else \
            (torch.randn(config.vocab_size, H, generator=gen, device=device) * 0.02).to(dtype)
        eng._finalize()
        return eng

    def _finalize(self):
        if self.device.type == "cuda":
            torch.cuda.current_stream(self.device).synchronize()

    def linear_layers(self) -> List[LinearQ]:
        return [L[k] for L in self.layers for k in ("qkv", "o", "gu", "down")]

    # ---- one block ------------------------------------------------------------------------------
    def _block(self, L, x, delta, kc, vc, pos0: int, pos_t, T: int, mask):
        """x: (B*T, H) residual stream, delta: pending residual contribution or None.  Writes keys and values of the
        T new positions into the caches (at pos0.., or at the device-side position pos_t when decoding under a
        graph) and returns (x', delta') with delta' = the block's MLP output, still to be added."""
        B = x.shape[0] // T
        x, h = add_rmsnorm(x, delta, L["ln1"], self.eps)
        # per-head q/k norms, rotary embedding and the cache write of the new positions: one kernel
        q = qk_norm_rope(L["qkv"](h), L["qn"], L["kn"], self.cos, self.sin, kc, vc, pos0 if pos_t is None else pos_t, B, T,
                         self.nq, self.nkv, self.eps)
        if pos_t is None:
            keys, vals = kc[:, :, :pos0 + T], vc[:, :, :pos0 + T]
        else:  # one new position whose index lives on the device: attend over the whole cache under a mask
            keys, vals = kc, vc
        a = F.scaled_dot_product_attention(q, keys, vals, attn_mask=mask, is_causal=(mask is None and T > 1),
                                           enable_gqa=self.nq != self.nkv)
        a = a.transpose(1, 2).reshape(B * T, self.nq * self.hd)
        att = L["o"](a)
        x, h = add_rmsnorm(x, att, L["ln2"], self.eps)
        return x, L["down"](silu_mul(L["gu"](h)))

    def _final(self, x, delta):
        return add_rmsnorm(x, delta, self.norm, self.eps)[1]

    # ---- prefill / decode -------------------------------------------------------------------------
    def _alloc(self, B: int, max_len: int):
        """Static state for a batch size and a maximal length; kept (with the captured graph) across calls."""
        key = (B, max_len)
        if getattr(self, "_alloc_key", None) == key:
            return
        dev, dt = self.device, self.dtype
        self.B, self.max_len = B, max_len
        self._rotary_table(max_len)
        self.kc = [torch.zeros(B, self.nkv, max_len, self.hd, device=dev, dtype=dt) for _ in self.layers]
        self.vc = [torch.zeros(B, self.nkv, max_len, self.hd, device=dev, dtype=dt) for _ in self.layers]
        self.pos = torch.zeros(1, device=dev, dtype=torch.long)
        self.tok = torch.zeros(B, device=dev, dtype=torch.long)
        self.last_logits = torch.zeros(B, self.head.shape[0], device=dev, dtype=dt)
        self._alloc_key = key
        self._graph = None

    def prefill(self, inputs_embeds: torch.Tensor, max_new: int) -> torch.Tensor:
        """inputs_embeds: (B, T, H).  Runs the prompt into caches sized for T + max_new positions and returns the first
        generated token ids (B,)."""
        B, T, H = inputs_embeds.shape
        self._alloc(B, T + max_new)
        self.T0 = T
        dev, dt = self.device, self.dtype
        x = inputs_embeds.to(device=dev, dtype=dt).reshape(B * T, H).contiguous()
        delta = None
        for i, L in enumerate(self.layers):
            x, delta = self._block(L, x, delta, self.kc[i], self.vc[i], 0, None, T, None)
        h = self._final(x, delta).view(B, T, H)[:, -1]
        logits = dense_head(h.contiguous(), self.head)
        self.pos.fill_(T)
        self.tok.copy_(logits.argmax(-1))
        self.last_logits.copy_(logits)
        return self.tok.clone()

    def _step(self):
        """One token for every sequence: reads self.tok and self.pos (device), writes self.tok, self.last_logits
        and advances self.pos."""
        B = self.B
        x = self.embed[self.tok]
        mask = (torch.arange(self.max_len, device=self.device) <= self.pos).view(1, 1, 1, self.max_len)
        delta = None
        for i, L in enumerate(self.layers):
            x, delta = self._block(L, x, delta, self.kc[i], self.vc[i], 0, self.pos, 1, mask)
        h = self._final(x, delta)
        logits = dense_head(h, self.head)
        self.last_logits.copy_(logits)
        self.tok.copy_(logits.argmax(-1))
        self.pos.add_(1)

    def decode(self, steps: int, use_graph: bool = True, keep_logits: bool = False):
        """Runs ``steps`` further tokens after :meth:`prefill`; returns ids (B, steps) [and logits (steps, B, V)]."""
        ids = torch.empty(steps, self.B, dtype=torch.long, device=self.device)
        lg = torch.empty(steps, self.B, self.head.shape[0], dtype=self.dtype, device=self.device) if keep_logits else None
        if use_graph and self._graph is None:
            st = torch.cuda.Stream(self.device)
            st.wait_stream(torch.cuda.current_stream(self.device))
            tok0, pos0 = self.tok.clone(), self.pos.clone()
            with torch.cuda.stream(st):
                self._step()  # warm-up outside capture (allocations, kernel selection)
                st.synchronize()
                self.tok.copy_(tok0)
                self.pos.copy_(pos0)
                g = torch.cuda.CUDAGraph()
                with torch.cuda.graph(g, stream=st):
                    self._step()
            torch.cuda.current_stream(self.device).wait_stream(st)
            self.tok.copy_(tok0)
            self.pos.copy_(pos0)
            self._graph = g
        for s in range(steps):
            if use_graph:
                self._graph.replay()
            else:
                self._step()
            ids[s] = self.tok
            if keep_logits:
                lg[s] = self.last_logits
        out = ids.t().contiguous()
        return (out, lg) if keep_logits else out

    def generate(self, inputs_embeds: torch.Tensor, steps: int, use_graph: bool = True) -> torch.Tensor:
        """Greedy ids (B, steps): the first from the prompt, the rest one decoding step each."""
        first = self.prefill(inputs_embeds, steps)
        if steps == 1:
            return first.view(-1, 1)
        rest = self.decode(steps - 1, use_graph=use_graph)
        return torch.cat([first.view(-1, 1), rest], dim=1)
