"""asrq_b200: B200 (sm_100a) kernels behind ASRQ's ``LinearQ`` quantized-linear API."""
from . import _lib, convert, host_io, packing
from .convert import FusedLinearQ, linearq_from_linear
from .host_io import forward_host
from .linear import LinearQ, LinearQQ, add_layernorm, add_rmsnorm, check_status, decode_self_attention, dense_head, qk_norm_rope, silu_mul
from .packing import pack_codes, pack_linearq, pack_signed_int4, pack_w4a4, rtn_quantize

__all__ = ["LinearQ", "LinearQQ", "FusedLinearQ", "linearq_from_linear", "convert", "check_status", "add_layernorm", "add_rmsnorm", "silu_mul", "dense_head", "qk_norm_rope", "decode_self_attention", "forward_host", "packing", "pack_codes", "pack_linearq", "pack_signed_int4",
           "pack_w4a4", "rtn_quantize", "_lib"]
__version__ = "0.1.0"
