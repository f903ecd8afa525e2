"""Stages the reference's own Python sources for the quantized-linear path under ``oracle/_ref/``.

TEST INFRASTRUCTURE ONLY.  The reference (wakandaai/asrq) is pure Python on top of torch, so there is
nothing to compile; what the checker and the CPU baseline need is the reference's files themselves.
This script copies the few files of the path from a checkout of the reference into ``oracle/_ref/``
(git-ignored: the sources never enter this repository's history) so that machines without the
checkout -- the GPU box -- can still run the reference's own ``LinearQ.forward`` and
``WhisperForConditionalGenerationQ.generate`` as the CPU baseline.  ``__graft_entry__.build()`` runs
it whenever the checkout is present.

    python oracle/stage_ref.py /path/to/reference

Nothing in the shipped package imports ``oracle/``.
"""
import os
import shutil
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
DEST = os.path.join(HERE, "_ref")

# path within the reference project -> what it is used for
FILES = {
    "asrq/core/linear.py": "LinearQ / LinearQQ: dequantize + torch.matmul (the CPU baseline of the single-layer workloads)",
    "asrq/core/types.py": "type aliases imported by the model file",
    "asrq/core/registry.py": "decorator registries imported by the model file",
    "asrq/core/model.py": "ModelQ base class imported by the model file",
    "asrq/core/utils.py": "cuda_synchronize / cuda_empty_cache helpers imported by the model file",
    "asrq/quantizers/base.py": "uniform grid (find_quant_params)",
    "asrq/quantizers/rtn.py": "round-to-nearest quantizer",
    "asrq/quantizers/activation.py": "activation fake-quantisation patch",
    "asrq/transforms/rotation/hadamard_utils.py": "matmul_hadU",
    "asrq/models/transformers/whisper.py": "Whisper*Q model classes (the whole-model CPU baseline and parity check)",
}


def stage(reference_root: str, dest: str = DEST) -> str:
    if not os.path.isdir(os.path.join(reference_root, "asrq")):
        raise SystemExit(f"{reference_root} does not look like a checkout of the reference (no asrq/ package)")
    for rel in FILES:
        src = os.path.join(reference_root, rel)
        dst = os.path.join(dest, rel)
        os.makedirs(os.path.dirname(dst), exist_ok=True)
        shutil.copyfile(src, dst)
    with open(os.path.join(dest, "STAGED_FROM"), "w") as f:
        f.write(os.path.abspath(reference_root) + "\n")
    return dest


if __name__ == "__main__":
    if len(sys.argv) != 2:
        raise SystemExit("usage: python oracle/stage_ref.py <path to a checkout of the reference (wakandaai/asrq)>")
    print(stage(sys.argv[1]))
