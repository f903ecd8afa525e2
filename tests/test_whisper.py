"""Whisper*Q model classes on the CPU: structure, state_dict compatibility with the reference's
classes, packing of a float model, and the on-disk round trip through the reference's own LinearQ."""
import io

import pytest
import torch

import asrq_b200
from asrq_b200 import whisper as W
from oracle import linearq_oracle as O
from tests.whisper_util import load_fixture, staged_reference

transformers = pytest.importorskip("transformers")


def _config(cfg):
    return transformers.WhisperConfig(**cfg)


def test_state_dict_layout_equals_the_reference_classes():
    """Keys, shapes and dtypes of WhisperForConditionalGenerationQ equal those of the state_dict the
    reference's class produced (the fixture), so packed checkpoints move between the two."""
    cfg, sd_ref, *_ = load_fixture()
    m = W.WhisperForConditionalGenerationQ(_config(cfg))
    sd = m.state_dict()
    assert set(sd) == set(sd_ref)
    for k, v in sd.items():
        assert v.shape == sd_ref[k].shape and v.dtype == sd_ref[k].dtype, k
    n_q = sum(isinstance(x, asrq_b200.LinearQ) for x in m.modules())
    assert n_q == 2 * 6 + 2 * 10           # 6 per encoder layer, 10 per decoder layer (whisper.py:94-97,124-125,202-203)
    assert type(m.proj_out) is torch.nn.Linear and m.proj_out.weight.data_ptr() == m.model.decoder.embed_tokens.weight.data_ptr()
    assert m.model.encoder.layers[0].self_attn.k_proj.bias is None
    missing, unexpected = m.load_state_dict(sd_ref, strict=True)
    assert not missing and not unexpected


def test_quantize_whisper_packs_every_linear_but_the_head():
    cfg, *_ = load_fixture()
    torch.manual_seed(3)
    fm = transformers.WhisperForConditionalGeneration(_config(cfg)).eval()
    q = W.quantize_whisper(fm, bits=4, group_size=128)
    lin = fm.model.decoder.layers[1].encoder_attn.v_proj
    lq = q.model.decoder.layers[1].encoder_attn.v_proj
    codes, scales, zeros, _ = O.rtn_codes(lin.weight.detach().float(), 4, 128, False)
    assert torch.equal(lq.weight, O.pack_codes(codes, 4)) and torch.equal(lq.scales, scales.half())
    assert torch.equal(lq.bias, lin.bias.detach().half())
    assert torch.equal(q.model.encoder.conv1.weight, fm.model.encoder.conv1.weight)
    assert torch.equal(q.proj_out.weight, fm.proj_out.weight)
    assert not any(type(x) is torch.nn.Linear for n, x in q.named_modules() if n != "proj_out")


def test_checkpoint_round_trip_through_the_reference_classes():
    """torch.save of this repository's state_dict -> the reference's own WhisperForConditionalGenerationQ
    and LinearQ (staged under oracle/_ref) -> equal bytes back, and the reference's CPU forward on the
    loaded checkpoint reproduces the fixture's logits."""
    R = staged_reference()
    if R is None:
        pytest.skip("the reference's files are not staged under oracle/_ref")
    cfg, sd_ref, x, ids, logits, _ = load_fixture()
    mine = W.WhisperForConditionalGenerationQ(_config(cfg))
    mine.load_state_dict(sd_ref)
    buf = io.BytesIO()
    torch.save(mine.state_dict(), buf)
    buf.seek(0)
    ref_model = R.whisper().WhisperForConditionalGenerationQ(_config(cfg)).eval()
    ref_model.load_state_dict(torch.load(buf), strict=True)
    back = ref_model.state_dict()
    for k, v in mine.state_dict().items():
        assert torch.equal(back[k], v), k
    start = torch.full((ids.shape[0], 1), cfg["decoder_start_token_id"], dtype=torch.long)
    with torch.no_grad():
        out = ref_model(input_features=x, decoder_input_ids=torch.cat([start, ids[:, :-1]], 1)).logits
    assert torch.allclose(out, logits, atol=1e-5)
    # a single layer: this repository's LinearQ -> file -> the reference's LinearQ
    case = O.make_c3(seed=9, m=3, k=256, n=64, bits=2, group_size=64)
    lq = asrq_b200.LinearQ(256, 64, 2, 64, bias=False)
    lq.load_quantized_params(case["scales"], case["zeros"], case["weight"])
    buf = io.BytesIO()
    torch.save(lq.state_dict(), buf)
    buf.seek(0)
    rq = R.linear().LinearQ(256, 64, 2, 64, bias=False)
    rq.load_state_dict(torch.load(buf))
    assert torch.equal(rq.dequantize_weight("cpu", torch.float32), lq.dequantize_weight("cpu", torch.float32))
    y_ref = rq.forward(case["x"].float())
    assert torch.allclose(y_ref, O.linearq_forward_fp32(case["x"], case["weight"], case["scales"], case["zeros"], None, 2, 64))


def test_rtfx_definition():
    cfg, *_ = load_fixture()
    c = _config(dict(cfg, max_source_positions=1500))
    assert W.audio_seconds(c, 32) == 960.0 and W.rtfx(c, 32, 2.0) == 480.0
