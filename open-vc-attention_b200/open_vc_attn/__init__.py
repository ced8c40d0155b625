"""FP8 ExpCast forward attention for NVIDIA B200, drop-in for the ``open_vc_attn`` API.

Importing the package loads neither torch nor CUDA; every public name resolves lazily
(as src/open_vc_attn/__init__.py of the reference does).
"""

__version__ = "0.3.0+b200"


def attention(*args, **kwargs):
    from .api import attention as implementation

    return implementation(*args, **kwargs)


def prepare_fp8(*args, **kwargs):
    from .api import prepare_fp8 as implementation

    return implementation(*args, **kwargs)


def attention_fp8(*args, **kwargs):
    from .api import attention_fp8 as implementation

    return implementation(*args, **kwargs)


def prepare_fp8_fused(*args, **kwargs):
    from .api import prepare_fp8_fused as implementation

    return implementation(*args, **kwargs)


def prepare_v_repair(*args, **kwargs):
    from .v_repair import prepare_v_repair as implementation

    return implementation(*args, **kwargs)


def attention_v_repair(*args, **kwargs):
    from .v_repair import attention_v_repair as implementation

    return implementation(*args, **kwargs)


def raw_forward(*args, **kwargs):
    from .api import raw_forward as implementation

    return implementation(*args, **kwargs)


__all__ = [
    "attention",
    "attention_fp8",
    "prepare_fp8",
    "prepare_fp8_fused",
    "prepare_v_repair",
    "attention_v_repair",
    "raw_forward",
]
