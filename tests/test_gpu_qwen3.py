"""Qwen3*Q on the GPU against the stock Hugging Face model in fp32 on the CPU holding the decoded weights, and
the CUDA-graph engine against the model classes."""
import pytest
import torch

import asrq_b200
from asrq_b200 import qwen3 as Q
from tests.gpu_util import DEV
from tests.qwen3_util import toy_models

transformers = pytest.importorskip("transformers")
pytestmark = pytest.mark.gpu


def _inputs(cfg, batch=3, T=9, seed=1):
    gen = torch.Generator().manual_seed(seed)
    return torch.randint(0, cfg.vocab_size, (batch, T), generator=gen)


def test_model_classes_match_float_model():
    """fp16 through the CUDA kernels against fp32 on the CPU: logits within 1e-2 of the largest magnitude."""
    cfg, fm, q = toy_models()
    ids = _inputs(cfg)
    with torch.no_grad():
        ref = fm(input_ids=ids).logits
        out = q.half().to(DEV)(input_ids=ids.to(DEV)).logits
    err = float((out.float().cpu() - ref).abs().max())
    assert err <= 1e-2 * float(ref.abs().max()), err
    asrq_b200.check_status()


def test_engine_matches_float_model_and_graph_replay():
    cfg, fm, q = toy_models()
    ids = _inputs(cfg, batch=4, T=7)
    steps = 6
    with torch.no_grad():
        emb = fm.model.embed_tokens(ids)
        ref_ids = fm.generate(input_ids=ids, max_new_tokens=steps, do_sample=False, min_new_tokens=steps,
                              pad_token_id=0, eos_token_id=None)[:, ids.shape[1]:]
        full = torch.cat([ids, ref_ids], 1)
        ref_logits = fm(input_ids=full).logits[:, ids.shape[1] - 1:-1]          # (B, steps, V): the logits each id was chosen from
    eng = Q.Qwen3Engine.from_model(q.half().to(DEV))
    a = eng.generate(emb.half().to(DEV), steps, use_graph=False).clone()
    first = eng.prefill(emb.half().to(DEV), steps)
    rel = float((eng.last_logits.float().cpu() - ref_logits[:, 0]).abs().max()) / float(ref_logits.abs().max())
    assert rel <= 1e-2, rel
    rest, lg = eng.decode(steps - 1, use_graph=True, keep_logits=True)
    b = torch.cat([first.view(-1, 1), rest], 1)
    c = eng.generate(emb.half().to(DEV), steps, use_graph=True).clone()
    assert torch.equal(a, b) and torch.equal(b, c)                            # eager step, captured step, second capture
    # against the float model: equal ids up to the first position where its top-2 margin is within the error
    top2 = ref_logits.topk(2, dim=-1).values
    clear = (top2[..., 0] - top2[..., 1]) > 4 * max(rel, 2e-3) * float(ref_logits.abs().max())
    for r in range(ids.shape[0]):
        n_clear = int((~clear[r]).nonzero()[0]) if bool((~clear[r]).any()) else steps
        assert torch.equal(a[r, :n_clear].cpu(), ref_ids[r, :n_clear]), (r, n_clear)
    assert int(clear.sum()) >= clear.numel() // 2
    asrq_b200.check_status()


def test_engine_random_init_qwen3_1p7b_widths():
    """Qwen3-1.7B widths (hidden 2048, 16 query / 8 key-value heads of 128, FFN 6144) at reduced depth and vocabulary,
    batch 64 as the speech model decodes: runs through the graph and is deterministic."""
    cfg = transformers.Qwen3Config(vocab_size=4096, hidden_size=2048, intermediate_size=6144, num_hidden_layers=2,
                                   num_attention_heads=16, num_key_value_heads=8, head_dim=128, max_position_embeddings=512,
                                   tie_word_embeddings=True)
    eng = Q.Qwen3Engine.random_init(cfg, DEV, seed=0)
    gen = torch.Generator().manual_seed(0)
    emb = (torch.randn(64, 40, 2048, generator=gen) * 0.02).half().to(DEV)
    a = eng.generate(emb, 5).clone()
    b = eng.generate(emb, 5).clone()
    assert a.shape == (64, 5) and torch.equal(a, b)
    asrq_b200.check_status()
