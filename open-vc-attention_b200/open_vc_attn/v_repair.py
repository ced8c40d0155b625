"""V residual repair on the packed ExpCast path.

For the tokens whose V rounds worst in FP8 (largest squared residual per head) a repair entry is
added: a copy of the token's FP8 key and its V residual, again in FP8.  The repairs form a K/V
prefix that the kernel visits after the original tokens; they add to the output but are left out
of the softmax denominator.  Same contract as src/open_vc_attn/v_repair.py of the reference.
"""

import math
from dataclasses import dataclass

import torch

from . import _lib
from ._dispatch import DEFAULT_MID_WINDOW_BLOCKS, DEFAULT_VERSION
from .api import _layout, raw_forward, validate_qkv


@dataclass(frozen=True)
class PreparedVRepair:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    q_descale: torch.Tensor
    k_descale: torch.Tensor
    v_descale: torch.Tensor
    repair_k_descale: torch.Tensor | None
    layout: dict
    output_shape: tuple
    repair_tokens: int
    selected_tokens: int = 0
    v_prepacked: bool = False


MIN_LENGTH = 32768


@torch.no_grad()
def prepare_v_repair(q, k, v, *, budget):
    """Prepare BF16/FP16 [S,H,128] or [1,S,H,128] with a V repair budget.

    ``budget`` is the fraction of tokens repaired per head (0.02 = worst 2 %).  One sequence with
    S >= 32768 on B200.  A budget that selects no token is the plain fused preparation.
    """
    validate_qkv(q, k, v)
    if q.shape != k.shape or q.shape != v.shape or q.shape[-1] != 128:
        raise ValueError("V repair expects equal self-attention shapes ending in D=128")
    if not 0.0 <= budget < 1.0:
        raise ValueError("budget must be in [0, 1)")
    if q.shape[-3] < MIN_LENGTH or (q.ndim == 4 and q.shape[0] != 1):
        raise ValueError("V repair requires one sequence with S >= 32768")
    if torch.cuda.get_device_capability(q.device) != (10, 0):
        raise ValueError("V repair currently requires B200")
    return _prepare(q, k, v, budget)


def _prepare(q, k, v, budget):
    """prepare_v_repair without the length/device policy checks (any S >= 1)."""
    from .preparation import _prepare_packed
    from .quantization import fp8_quantize_per_block, pack_v

    lib = _lib.load()
    with torch.cuda.device(q.device):
        q, k, v, layout, shape = _layout(q, k, v)
        if q.ndim != 3:
            raise ValueError("V repair supports one sequence")
        s, h, d = v.shape
        selected = round(budget * s)
        rows = math.ceil(selected / 128) * 128
        if selected == 0:
            plain = _prepare_packed(q, k, v, shape)
            return PreparedVRepair(
                plain.q, plain.k, plain.v, plain.q_descale, plain.k_descale, plain.v_descale, None,
                plain.layout, shape, 0, 0, plain.v_prepacked,
            )
        total = rows + s
        blocks = math.ceil(s / 128)
        device = q.device
        stream = _lib.stream_pointer(device)
        code = _lib.dtype_code(q.dtype)

        q8, q_descale = fp8_quantize_per_block(q)
        k_all = torch.empty((total, h, d), device=device, dtype=torch.float8_e4m3fn)
        v_all = torch.empty((total, h, d), device=device, dtype=torch.float8_e4m3fn)
        k_descale = torch.empty((1, h, blocks), device=device, dtype=torch.float32)
        _lib.check(
            lib.ovc_quantize_per_block(k.data_ptr(), code, 1, s, h, k_all[rows:].data_ptr(), k_descale.data_ptr(),
                                       blocks, stream),
            "ovc_quantize_per_block",
        )
        amax = torch.empty((1, h), device=device, dtype=torch.float32)
        _lib.check(lib.ovc_head_amax(v.data_ptr(), code, 1, s, h, amax.data_ptr(), stream), "ovc_head_amax")
        score = torch.empty((h, s), device=device, dtype=torch.float32)
        _lib.check(
            lib.ovc_repair_score(v.data_ptr(), code, s, h, amax.data_ptr(), v_all[rows:].data_ptr(),
                                 score.data_ptr(), stream),
            "ovc_repair_score",
        )
        # As in the reference (v_repair.py:190): torch divides by a scalar by multiplying with its float32
        # reciprocal, which is also what the kernels' division gives for 448.
        v_descale = amax.clamp(min=1e-12) / 448.0

        layout = dict(layout)
        index = torch.topk(score, selected, dim=1, sorted=False).indices.to(torch.int32).contiguous()
        repair_kd = torch.empty((1, h, rows), device=device, dtype=torch.float32)
        _lib.check(
            lib.ovc_repair_rows(
                k_all.data_ptr(), v_all.data_ptr(), v.data_ptr(), code, k_descale.data_ptr(), v_descale.data_ptr(),
                index.data_ptr(), repair_kd.data_ptr(), selected, rows, s, h, blocks, stream,
            ),
            "ovc_repair_rows",
        )
        ones = torch.ones((1, h, rows // 128), device=device, dtype=torch.float32)
        k_descale_all = torch.cat((ones, k_descale), dim=2)
        layout["cu_seqlens_k"] = torch.arange(2, device=device, dtype=torch.int32) * total
        layout["max_seqlen_k"] = total
        return PreparedVRepair(
            q8[0], k_all, pack_v(v_all), q_descale, k_descale_all, v_descale, repair_kd, layout, shape,
            rows, selected, v_prepacked=True,
        )


def attention_v_repair(prepared, *, mid_window_blocks=DEFAULT_MID_WINDOW_BLOCKS, softmax_scale=None):
    """Dense ExpCast attention plus optional V repair tokens.

    ``mid_window_blocks=4`` is the default scan; None selects the plain right-to-left scan.
    """
    out, _ = raw_forward(
        prepared.q,
        prepared.k,
        prepared.v,
        version=DEFAULT_VERSION,
        q_descale=prepared.q_descale,
        k_descale=prepared.k_descale,
        v_descale=prepared.v_descale,
        **prepared.layout,
        expcast=True,
        softmax_scale=softmax_scale,
        mid_window_blocks=mid_window_blocks,
        return_lse=False,
        repair_k_descale=prepared.repair_k_descale,
        v_prepacked=prepared.v_prepacked,
    )
    return out.reshape(prepared.output_shape)
