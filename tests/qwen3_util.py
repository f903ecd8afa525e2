"""Shared by the Qwen3 tests: a toy configuration and a float model whose projections hold exactly the values
the packed layers decode to, so that the stock Hugging Face model in fp32 on the CPU is the oracle of the
``Qwen3*Q`` classes (the reference's own classes import NeMo, which is not installed: asrq/models/nemo/canary_qwen.py:37-48)."""
import torch

TOY = dict(vocab_size=512, hidden_size=256, intermediate_size=512, num_hidden_layers=2, num_attention_heads=4,
           num_key_value_heads=2, head_dim=64, max_position_embeddings=128, rms_norm_eps=1e-6, tie_word_embeddings=False,
           attention_bias=False)


def toy_models(seed: int = 0, bits: int = 4, group_size: int = 128):
    """(float model with fake-quantised projections in fp32, packed Qwen3ForCausalLMQ) from the same seeded weights."""
    import transformers
    from asrq_b200 import qwen3 as Q
    from oracle import linearq_oracle as O
    torch.manual_seed(seed)
    cfg = transformers.Qwen3Config(**TOY)
    fm = transformers.Qwen3ForCausalLM(cfg).eval()
    with torch.no_grad():
        for name, p in fm.named_parameters():
            if "norm" in name:
                p.copy_(1 + 0.1 * torch.randn_like(p))
            elif "embed_tokens" in name or "lm_head" in name:
                p.copy_((torch.randn_like(p) * 0.5).half().float())     # large enough for distinct greedy choices
            else:
                p.copy_(torch.randn_like(p) * 0.08)
    q = Q.quantize_qwen3(fm, bits=bits, group_size=group_size)
    with torch.no_grad():  # the float model's projections := what the packed layers decode to (fp32, from fp16 scales)
        src = dict(fm.named_modules())
        for name, mod in q.named_modules():
            if isinstance(mod, Q.LinearQ):
                w = O.dequantize_weight(mod.weight, mod.scales, mod.zeros, bits, group_size, mod.in_features, torch.float32)
                src[name].weight.copy_(w)
        for name, p in fm.named_parameters():
            if "norm" in name:
                p.copy_(p.half().float())
    return cfg, fm, q
