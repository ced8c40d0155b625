"""FP8 E4M3 quantisers on the GPU (host side of libovc.so's preparation kernels).

Same groups, scales and bytes as the reference's Triton quantisers
(src/open_vc_attn/quantization.py): Q/K get one scale per (batch, head, 128-token block),
V one per (batch, head); descale = max(amax, 1e-12) / 448.
"""

import torch

from . import _lib

BLOCK = 128


def _as_batched(x):
    if x.dim() == 3:
        x = x[None]
    if x.dim() != 4 or x.shape[-1] != 128:
        raise ValueError("Expected [S,H,128] or [B,S,H,128]")
    return x.contiguous()


def fp8_quantize_per_block(x, block_l=BLOCK, *, descale_blocks=None):
    """(B,S,H,128) f16/bf16 -> (codes e4m3 same shape, descale f32 [B,H,blocks]).

    ``descale_blocks`` > blocks allocates a wider descale row; the first padding entry is set
    to 1.0 (what the fused preparation needs for an odd block count).
    """
    if block_l != BLOCK:
        raise ValueError("Only 128-token quantisation blocks are supported")
    x = _as_batched(x)
    b, s, h, _ = x.shape
    blocks = (s + BLOCK - 1) // BLOCK
    width = blocks if descale_blocks is None else descale_blocks
    lib = _lib.load()
    with torch.cuda.device(x.device):
        codes = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        descale = torch.empty((b, h, width), dtype=torch.float32, device=x.device)
        _lib.check(
            lib.ovc_quantize_per_block(
                x.data_ptr(), _lib.dtype_code(x.dtype), b, s, h, codes.data_ptr(), descale.data_ptr(), width,
                _lib.stream_pointer(x.device),
            ),
            "ovc_quantize_per_block",
        )
    return codes, descale


def fp8_quantize_per_head(x):
    """(B,S,H,128) f16/bf16 -> (codes e4m3 same shape, descale f32 [B,H])."""
    x = _as_batched(x)
    b, s, h, _ = x.shape
    lib = _lib.load()
    with torch.cuda.device(x.device):
        codes = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
        amax = torch.empty((b, h), dtype=torch.float32, device=x.device)
        descale = torch.empty((b, h), dtype=torch.float32, device=x.device)
        stream = _lib.stream_pointer(x.device)
        code = _lib.dtype_code(x.dtype)
        _lib.check(lib.ovc_head_amax(x.data_ptr(), code, b, s, h, amax.data_ptr(), stream), "ovc_head_amax")
        _lib.check(
            lib.ovc_quantize_per_head(x.data_ptr(), code, b, s, h, amax.data_ptr(), codes.data_ptr(),
                                      descale.data_ptr(), stream),
            "ovc_quantize_per_head",
        )
    return codes, descale


def pack_v(value):
    """FP8 [S,H,128] or [B,S,H,128] -> the padded key-contiguous layout, returned as the logical view.

    The buffer is [B,H,128,S_pad] with a zero tail; the result is ``buffer[..., :S].movedim(-1, -3)``
    (src/open_vc_attn/_kernels/blackwell/flash_attn/cute/v_layout.py:36-49 of the reference).
    """
    if value.dtype != torch.float8_e4m3fn:
        raise ValueError("pack_v expects float8_e4m3fn")
    batched = value.dim() == 4
    x = _as_batched(value)
    b, s, h, d = x.shape
    padded = (s + BLOCK - 1) // BLOCK * BLOCK
    lib = _lib.load()
    with torch.cuda.device(x.device):
        buffer = torch.empty((b, h, d, padded), dtype=value.dtype, device=x.device)
        _lib.check(
            lib.ovc_pack_v(x.data_ptr(), b, s, h, buffer.data_ptr(), _lib.stream_pointer(x.device)), "ovc_pack_v"
        )
    result = buffer[..., :s].movedim(-1, -3)
    return result if batched else result.squeeze(0)


# The reference's names for the same operations.
fp8_quantize_per_block_triton = fp8_quantize_per_block
fp8_quantize_per_head_triton = fp8_quantize_per_head
