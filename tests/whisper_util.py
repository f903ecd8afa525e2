"""Shared by the Whisper tests: the toy model fixture generated from the reference's classes."""
import ast
import os

import numpy as np
import torch

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")


def load_fixture():
    d = np.load(os.path.join(GOLDEN, "whisper_tiny_q.npz"))
    cfg = ast.literal_eval(str(d["config"]))
    sd = {}
    for k in d.files:
        if k.startswith("sd/"):
            name = k[3:]
            a = d[k]
            if bool(d["f16/" + name]):
                a = a.view(np.float16)
            sd[name] = torch.from_numpy(a.copy())
    return cfg, sd, torch.from_numpy(d["x"]), torch.from_numpy(d["ids"]), torch.from_numpy(d["logits"]), \
        torch.from_numpy(d["encoder_out"])


def staged_reference():
    """oracle.ref_loader if the reference's files are staged under oracle/_ref (staging them first when a
    checkout sits next to this repository or ASRQ_REFERENCE_ROOT names one), else None."""
    from oracle import ref_loader, stage_ref
    if not ref_loader.available("asrq/models/transformers/whisper.py"):
        root = os.environ.get("ASRQ_REFERENCE_ROOT") or os.path.join(
            os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference")
        if os.path.isdir(os.path.join(root, "asrq")):
            stage_ref.stage(root)
    return ref_loader if ref_loader.available("asrq/models/transformers/whisper.py") else None
