"""Backends that the paired benchmark can time (src/open_vc_attn/benchmarking/backends.py of the reference).

Same three names.  `bf16` is the accuracy reference and default baseline; the reference times the
FlashAttention-4 BF16 kernel there, which is a third-party package that this engine does not ship, so
here it is PyTorch's scaled_dot_product_attention on the same BF16 inputs (a library kernel, used only
as the yardstick).
"""

from collections import namedtuple

Backend = namedtuple("Backend", ["version", "mode", "description"])

BACKENDS = {
    "bf16": Backend("reference", "bf16", "BF16 attention: torch.nn.functional.scaled_dot_product_attention"),
    "vc": Backend("open-vc", "vsmooth", "VC-Attention: ExpCast + V-Smooth, original scan, no Open-VC optimizations"),
    "open-vc": Backend("open-vc", "expcast", "Open-VC Attn: ExpCast with Open-VC optimizations (B200 CUDA engine)"),
}
DEFAULT_BACKENDS = tuple(BACKENDS)
DEFAULT_BASELINE = "bf16"
CANDIDATE = "open-vc"


def get_backend(name):
    try:
        return BACKENDS[name]
    except KeyError:
        raise ValueError(f"Unknown backend {name!r}; choose from {tuple(BACKENDS)}") from None
