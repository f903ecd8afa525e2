"""Generate ``whisper_tiny_q.npz`` from the reference's own Whisper*Q classes.

Run where the reference checkout is available (the fixture is committed, the tests do not need the
checkout):

    PYTHONDONTWRITEBYTECODE=1 python tests/golden/make_whisper_golden.py /path/to/reference

A Whisper-shaped model of toy size (2 + 2 layers, d_model 128, 2 heads, FFN 512, 128 mel bins, 64
source positions, vocabulary 256) is built from the reference's ``WhisperForConditionalGenerationQ``
(asrq/models/transformers/whisper.py:256-271), every ``LinearQ`` in it is filled from seeded random
weights through the reference's ``RTNQuantizer`` (4 bits, group 128, asymmetric), and the reference
model -- ``LinearQ.forward`` = dequantize + matmul, in fp32 on the CPU -- transcribes a seeded batch
greedily.  Stored: the configuration, the packed ``state_dict``, the input, the greedy token ids and the
logits of a teacher-forced pass over those ids.
"""
import os
import sys
import types

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))

CONFIG = dict(vocab_size=256, num_mel_bins=128, encoder_layers=2, decoder_layers=2, encoder_attention_heads=2,
              decoder_attention_heads=2, d_model=128, encoder_ffn_dim=512, decoder_ffn_dim=512,
              max_source_positions=64, max_target_positions=32, pad_token_id=0, bos_token_id=1, eos_token_id=2,
              decoder_start_token_id=1, suppress_tokens=None, begin_suppress_tokens=None)
STEPS, BATCH = 12, 3


class Cfg:
    name, bits, group_size, symmetric, exclude_modules = "rtn", 4, 128, False, []


def load_reference(root):
    sys.dont_write_bytecode = True
    sys.path.insert(0, root)
    for name, attrs in (("omegaconf", dict(DictConfig=dict)), ("asrq.transforms", {}),
                        ("asrq.transforms.base", dict(TransformConfig=object)), ("asrq.calibration", {}),
                        ("asrq.calibration.base", dict(CalibConfig=object)), ("asrq.evaluation", {}),
                        ("asrq.evaluation.english_text_normalizer", dict(normalizer=None))):
        if name not in sys.modules:
            m = types.ModuleType(name)
            m.__dict__.update(attrs)
            m.__path__ = []
            sys.modules[name] = m
    try:
        import datasets  # noqa: F401
    except Exception:
        m = types.ModuleType("datasets")
        m.load_dataset = None
        sys.modules["datasets"] = m
    from asrq.models.transformers.whisper import WhisperForConditionalGenerationQ
    from asrq.core.linear import LinearQ
    from asrq.quantizers.rtn import RTNQuantizer
    return WhisperForConditionalGenerationQ, LinearQ, RTNQuantizer


@torch.no_grad()
def main(root):
    import transformers
    ModelQ, LinearQ, RTNQuantizer = load_reference(root)
    torch.manual_seed(0)
    cfg = transformers.WhisperConfig(**CONFIG)
    model = ModelQ(cfg).eval()
    gen = torch.Generator().manual_seed(1)
    # floating-point parts: larger than the library's 0.02 init so that logits have clear maxima
    for name, p in model.named_parameters():
        if p.dim() > 1:
            # (token embeddings small against position embeddings: with the tied output head a dominant
            # token embedding would make every step repeat its input token)
            std = 0.1 if "embed_tokens" in name else (0.6 if "decoder.embed_positions" in name else 0.05)
            p.copy_(torch.randn(p.shape, generator=gen) * std)
        elif "layer_norm" in name and name.endswith("weight"):
            p.copy_(1.0 + 0.1 * torch.randn(p.shape, generator=gen))
        else:
            p.copy_(0.05 * torch.randn(p.shape, generator=gen))
    model.tie_weights()
    for name, mod in model.named_modules():
        if isinstance(mod, LinearQ):
            n, k = mod.out_features, mod.in_features
            lin = torch.nn.Linear(k, n, bias=False)
            lin.weight.data = torch.randn(n, k, generator=gen) * 0.08
            qz = RTNQuantizer(lin, name, Cfg())
            scales, zeros = qz()                                   # fake-quantises lin.weight in place
            fq = lin.weight.data.reshape(n, k // 128, 128)
            codes = torch.round((fq - zeros) / scales).clamp(0, 15).reshape(n, k).to(torch.int32)
            packed = (codes[:, 0::2] | (codes[:, 1::2] << 4)).to(torch.uint8)
            mod.load_quantized_params(scales.squeeze(-1).half(), zeros.squeeze(-1).half(), packed)
            if mod.bias is not None:
                mod.bias = (torch.randn(n, generator=gen) * 0.05).half()
    x = torch.randn(BATCH, CONFIG["num_mel_bins"], 2 * CONFIG["max_source_positions"], generator=gen)
    out = model.generate(x, max_new_tokens=STEPS, do_sample=False)
    ids = out[:, -STEPS:] if out.shape[1] >= STEPS else out
    start = torch.full((BATCH, 1), CONFIG["decoder_start_token_id"], dtype=torch.long)
    dec_in = torch.cat([start, ids[:, :-1]], dim=1)
    res = model(input_features=x, decoder_input_ids=dec_in)
    logits = res.logits                                            # (B, STEPS, V): teacher-forced on the greedy ids
    assert torch.equal(logits.argmax(-1), ids), "greedy ids and teacher-forced argmax disagree"
    enc = model.model.encoder(x).last_hidden_state
    sd = {k: v.numpy() for k, v in model.state_dict().items()}
    np.savez_compressed(os.path.join(HERE, "whisper_tiny_q.npz"), config=np.array(repr(CONFIG)), x=x.numpy(),
                        ids=ids.numpy(), logits=logits.numpy(), encoder_out=enc.numpy(),
                        **{"sd/" + k: (v.view(np.uint16) if v.dtype == np.float16 else v) for k, v in sd.items()},
                        **{"f16/" + k: np.array(v.dtype == np.float16) for k, v in sd.items()})
    print("keys:", len(sd), "ids[0]:", ids[0].tolist())


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python tests/golden/make_whisper_golden.py <path to a checkout of the reference>")
    main(sys.argv[1])
