"""Dense and packed diffusion attention on top of ``open_vc_attn.attention``, with the constructor and the two
forward methods a serving framework's attention layer expects (src/open_vc_attn/integrations/diffusion.py:13-57 of
the reference).  A packed batch is attended one sequence at a time, so that no 128-token scale block of the FP8
preparation covers tokens of two sequences."""

import os

import torch

from open_vc_attn._dispatch import DEFAULT_VERSION, VERSIONS
from open_vc_attn.api import attention

from .packed import segments

_MODE_OF_VERSION = {"reference": "bf16", "open-vc": "expcast"}


def _backend_from_environment():
    """(version, mode) from OPEN_VC_ATTN_IMPLEMENTATION / OPEN_VC_ATTN_MODE; each version has exactly one mode."""
    version = os.environ.get("OPEN_VC_ATTN_IMPLEMENTATION", DEFAULT_VERSION)
    mode = os.environ.get("OPEN_VC_ATTN_MODE", "expcast")
    if version not in VERSIONS or mode not in _MODE_OF_VERSION.values():
        raise ValueError("Invalid OPEN_VC_ATTN_IMPLEMENTATION or OPEN_VC_ATTN_MODE")
    if _MODE_OF_VERSION.get(version, "expcast") != mode:
        raise ValueError("Use reference with bf16, or open-vc with expcast")
    return version, mode


class DenseDiffusionAdapter:
    """Non-causal multi-head inference attention with head size 128, dense (``forward``) or packed
    (``forward_varlen``)."""

    def __init__(self, num_heads, head_size, softmax_scale, causal=False, num_kv_heads=None, prefix="",
                 **extra_impl_args):
        grouped = num_kv_heads is not None and num_kv_heads != num_heads
        if head_size != 128 or grouped:
            raise ValueError("Open-VC diffusion adapter requires MHA with head_size=128")
        if causal or extra_impl_args.get("dropout_p", 0):
            raise ValueError("Open-VC diffusion adapter supports dense noncausal inference only")
        self.version, self.mode = _backend_from_environment()
        self.scale = softmax_scale
        self.trailing_padding = bool(extra_impl_args.get("packed_trailing_padding", False))

    def forward(self, query, key, value, attn_metadata=None):
        return attention(query, key, value, version=self.version, mode=self.mode, softmax_scale=self.scale)

    def forward_varlen(self, query, key, value, *, cu_seqlens, max_seqlen, cu_seqlens_host=None):
        same = query.ndim == 3 and query.shape == key.shape and query.shape == value.shape
        if not same:
            raise ValueError("Packed Open-VC adapter expects matching [T,H,128] self-attention")
        pieces = segments(cu_seqlens_host, query.shape[0], max_seqlen, trailing_padding=self.trailing_padding)
        if cu_seqlens.dtype != torch.int32 or cu_seqlens.numel() != len(pieces) + 1:
            raise ValueError("Device and host sequence metadata must describe the same bounds")
        if cu_seqlens.device != query.device:
            raise ValueError("Device sequence metadata must reside with Q/K/V")
        if len(pieces) == 1:
            return self.forward(query, key, value)
        out = torch.empty_like(query)
        for start, stop, padding in pieces:
            if padding:
                out[start:stop].zero_()
            else:
                out[start:stop] = self.forward(query[start:stop], key[start:stop], value[start:stop])
        return out
