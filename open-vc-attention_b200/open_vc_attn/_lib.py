"""ctypes binding of libovc.so (declared in include/ovc.h).

The library is the product: when it is missing or a call fails this module raises; there is no
PyTorch or CPU fallback.
"""

import ctypes
import os

_HERE = os.path.dirname(os.path.abspath(__file__))
LIBRARY_PATH = os.path.join(os.path.dirname(_HERE), "lib", "libovc.so")

OVC_F16, OVC_BF16 = 0, 1
OVC_ATTN_CAUSAL, OVC_ATTN_V_UNPACKED = 1, 2  # flags of ovc_attention_ex
STATUS_WAIT_EXPIRED = 1

_p, _i, _l, _f = ctypes.c_void_p, ctypes.c_int, ctypes.c_int64, ctypes.c_float

SIGNATURES = {
    "ovc_version": (_i, []),
    "ovc_error_string": (ctypes.c_char_p, [_i]),
    "ovc_last_cuda_error": (_i, []),
    "ovc_quantize_per_block": (_i, [_p, _i, _l, _l, _l, _p, _p, _l, _p]),
    "ovc_head_amax": (_i, [_p, _i, _l, _l, _l, _p, _p]),
    "ovc_quantize_per_head": (_i, [_p, _i, _l, _l, _l, _p, _p, _p, _p]),
    "ovc_prepare_fused": (_i, [_p, _p, _p, _i, _l, _l, _p, _p, _p, _p, _p, _p, _p, _p]),
    "ovc_prepare_fused_static": (_i, [_p, _p, _p, _i, _l, _l, _p, _p, _p, _p, _p, _p, _p]),
    "ovc_pack_v": (_i, [_p, _l, _l, _l, _p, _p]),
    "ovc_div_full": (_i, [_p, _p, _p, _l, _p]),
    "ovc_repair_score": (_i, [_p, _i, _l, _l, _p, _p, _p, _p]),
    "ovc_repair_rows": (_i, [_p, _p, _p, _i, _p, _p, _p, _p, _l, _l, _l, _l, _l, _p]),
    "ovc_attention": (_i, [_p, _p, _p, _p, _l, _p, _p, _p, _l, _p, _l, _l, _l, _l, _f, _i, _p, _p]),
    "ovc_bench_conversion": (_i, [_p, _l, _l, _p]),
    "ovc_selftest_wait": (_i, [_p, _l, _p, _p]),
    "ovc_copy_head_slice": (_i, [_p, _l, _l, _p, _l, _l, _l, _l, _l, _i, _p]),
    "ovc_attention_ex": (_i, [_p, _p, _p, _p, _l, _p, _p, _p, _l, _p, _p, _i, _l, _l, _l, _l, _f, _i, _p, _p]),
    "ovc_vs_assign": (_i, [_p, _p, _p, _l, _l, _l, _p]),
    "ovc_vs_accumulate": (_i, [_p, _p, _p, _p, _l, _l, _l, _p]),
    "ovc_vs_update_centers": (_i, [_p, _p, _p, _l, _l, _p]),
    "ovc_vs_block_stats": (_i, [_p, _p, _p, _p, _l, _l, _p]),
    "ovc_vs_block_write": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _p, _l, _l, _p]),
    "ovc_cast_e4m3": (_i, [_p, _i, _p, _l, _p]),
    "ovc_attention_vsmooth_workspace": (_l, [_l, _l]),
    "ovc_attention_vsmooth": (_i, [_p, _p, _p, _p, _p, _p, _p, _p, _l, _l, _l, _f, _i, _p, _p]),
}

_lib = None


def load():
    """Load libovc.so once and declare every entry point's signature."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIBRARY_PATH):
            raise RuntimeError(
                f"{LIBRARY_PATH} is missing: build it with `python open-vc-attention_b200/build.py` "
                "(needs nvcc); open_vc_attn has no fallback path"
            )
        lib = ctypes.CDLL(LIBRARY_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype, fn.argtypes = restype, argtypes
        _lib = lib
    return _lib


def check(code, what):
    if code != 0:
        lib = load()
        text = lib.ovc_error_string(code).decode()
        raise RuntimeError(f"{what} failed: {text} (code {code}, cuda error {lib.ovc_last_cuda_error()})")


def dtype_code(dtype):
    import torch

    if dtype == torch.float16:
        return OVC_F16
    if dtype == torch.bfloat16:
        return OVC_BF16
    raise ValueError(f"Expected float16 or bfloat16, got {dtype}")


def stream_pointer(device):
    import torch

    return torch.cuda.current_stream(device).cuda_stream
