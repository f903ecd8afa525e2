"""Qwen3*Q model classes on the CPU: structure, state_dict layout (the reference's, asrq/models/nemo/canary_qwen.py:70-182)
and packing of a float model."""
import pytest
import torch

import asrq_b200
from asrq_b200 import qwen3 as Q
from oracle import linearq_oracle as O
from tests.qwen3_util import TOY, toy_models

transformers = pytest.importorskip("transformers")


def test_class_structure_and_state_dict_layout():
    cfg = transformers.Qwen3Config(**TOY)
    m = Q.Qwen3ForCausalLMQ(cfg, bits=4)
    layer = m.model.layers[1]
    assert isinstance(layer, Q.Qwen3DecoderLayerQ) and isinstance(layer.self_attn, Q.Qwen3AttentionQ) and isinstance(layer.mlp, Q.Qwen3MLPQ)
    for name in ("q_proj", "k_proj", "v_proj", "o_proj"):
        assert isinstance(getattr(layer.self_attn, name), asrq_b200.LinearQ) and getattr(layer.self_attn, name).bias is None
    for name in ("gate_proj", "up_proj", "down_proj"):
        assert isinstance(getattr(layer.mlp, name), asrq_b200.LinearQ)
    assert type(m.lm_head) is torch.nn.Linear                            # canary_qwen.py:179: the head stays in floating point
    assert layer.self_attn.k_proj.out_features == TOY["num_key_value_heads"] * TOY["head_dim"]
    sd = m.state_dict()
    # a packed layer contributes weight (uint8), scales and zeros (fp16) -- the reference LinearQ's buffers (linear.py:16-25)
    pre = "model.layers.0.mlp.down_proj."
    assert sd[pre + "weight"].dtype == torch.uint8 and sd[pre + "weight"].shape == (TOY["hidden_size"], TOY["intermediate_size"] // 2)
    assert sd[pre + "scales"].dtype == torch.float16 and sd[pre + "scales"].shape == (TOY["hidden_size"], TOY["intermediate_size"] // 128)
    assert pre + "bias" not in sd
    assert sum(isinstance(x, asrq_b200.LinearQ) for x in m.modules()) == 7 * TOY["num_hidden_layers"]
    # the float model's keys, with each projection's "weight" re-typed and "scales"/"zeros" added
    fkeys = set(transformers.Qwen3ForCausalLM(cfg).state_dict())
    extra = {k for k in sd if k.endswith(".scales") or k.endswith(".zeros")}
    assert set(sd) - extra == fkeys and len(extra) == 2 * 7 * TOY["num_hidden_layers"]


def test_quantize_qwen3_packs_every_projection_but_the_head():
    torch.manual_seed(5)
    cfg = transformers.Qwen3Config(**TOY)
    fm = transformers.Qwen3ForCausalLM(cfg).eval()
    q = Q.quantize_qwen3(fm, bits=4, group_size=128)
    lin, lq = fm.model.layers[0].mlp.up_proj, q.model.layers[0].mlp.up_proj
    codes, scales, zeros, _ = O.rtn_codes(lin.weight.detach().float(), 4, 128, False)
    assert torch.equal(lq.weight, O.pack_codes(codes, 4)) and torch.equal(lq.scales, scales.half()) and torch.equal(lq.zeros, zeros.half())
    assert torch.equal(q.lm_head.weight, fm.lm_head.weight) and torch.equal(q.model.norm.weight, fm.model.norm.weight)
    assert not any(type(x) is torch.nn.Linear for n, x in q.named_modules() if n != "lm_head")
    # round trip of the packed checkpoint through a fresh instance
    fresh = Q.Qwen3ForCausalLMQ(cfg, 4, 128)
    missing, unexpected = fresh.load_state_dict(q.state_dict(), strict=True)
    assert not missing and not unexpected


def test_toy_float_model_holds_the_decoded_weights():
    cfg, fm, q = toy_models()
    lq = q.model.layers[1].self_attn.q_proj
    w = O.dequantize_weight(lq.weight, lq.scales, lq.zeros, 4, 128, lq.in_features, torch.float32)
    assert torch.equal(fm.model.layers[1].self_attn.q_proj.weight, w)
