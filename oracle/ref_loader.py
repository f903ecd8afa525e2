"""Imports the reference's own modules from ``oracle/_ref`` (TEST INFRASTRUCTURE ONLY).

``oracle/stage_ref.py`` puts the reference's files for the quantized-linear path there.  The files are
loaded one by one under their own package names with the few third-party modules they import only for
type annotations or for parts of the project outside this path (omegaconf, the transforms and
calibration packages, datasets) replaced by empty stand-ins, so that importing them has no side
effects and needs nothing that is not installed.  Only ``tests/``, ``__graft_entry__.smoke()`` and
``bench.py``'s CPU-baseline legs use this module.
"""
import importlib.util
import os
import sys
import types

HERE = os.path.dirname(os.path.abspath(__file__))
REF = os.path.join(HERE, "_ref")


def available(rel: str = "asrq/core/linear.py") -> bool:
    return os.path.exists(os.path.join(REF, rel))


def _stub(name: str, **attrs):
    if name not in sys.modules:
        m = types.ModuleType(name)
        m.__dict__.update(attrs)
        m.__path__ = []  # behaves as a package for "import a.b"
        sys.modules[name] = m
    return sys.modules[name]


def _load(modname: str, rel: str):
    if modname in sys.modules and getattr(sys.modules[modname], "__file__", "").startswith(REF):
        return sys.modules[modname]
    spec = importlib.util.spec_from_file_location(modname, os.path.join(REF, rel))
    mod = importlib.util.module_from_spec(spec)
    sys.modules[modname] = mod
    sys.dont_write_bytecode = True
    spec.loader.exec_module(mod)
    return mod


def _packages():
    for name in ("asrq", "asrq.core", "asrq.quantizers", "asrq.models", "asrq.models.transformers"):
        _stub(name)
    _stub("omegaconf", DictConfig=dict)


def linear():
    """The reference's asrq/core/linear.py module (LinearQ, LinearQQ)."""
    _packages()
    return _load("asrq.core.linear", "asrq/core/linear.py")


def rtn():
    _packages()
    _load("asrq.quantizers.base", "asrq/quantizers/base.py")
    return _load("asrq.quantizers.rtn", "asrq/quantizers/rtn.py")


def hadamard_utils():
    return _load("asrq_ref_hadamard_utils", "asrq/transforms/rotation/hadamard_utils.py")


def whisper():
    """The reference's asrq/models/transformers/whisper.py module (Whisper*Q classes)."""
    _packages()
    _stub("asrq.transforms")
    _stub("asrq.transforms.base", TransformConfig=type("TransformConfig", (), {}))
    _stub("asrq.calibration")
    _stub("asrq.calibration.base", CalibConfig=type("CalibConfig", (), {}))
    if "datasets" not in sys.modules:
        try:
            import datasets  # noqa: F401  (installed on some machines; only named by the calibration code)
        except Exception:
            _stub("datasets", load_dataset=None, Dataset=object, Audio=object)
    _stub("asrq.evaluation")
    _stub("asrq.evaluation.english_text_normalizer", normalizer=None)  # WER text normaliser: outside this path
    linear()
    for name, rel in (("asrq.core.types", "asrq/core/types.py"), ("asrq.core.registry", "asrq/core/registry.py"),
                      ("asrq.core.utils", "asrq/core/utils.py"), ("asrq.quantizers.base", "asrq/quantizers/base.py"),
                      ("asrq.core.model", "asrq/core/model.py")):
        _load(name, rel)
    return _load("asrq.models.transformers.whisper", "asrq/models/transformers/whisper.py")
