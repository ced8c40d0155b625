"""Host interface of the attention kernel (ovc_attention in libovc.so).

Takes the argument contract that the reference's public functions hand to its kernel interface
``_flash_attn_fwd(q, k, v, **kwargs) -> (out, lse)``
(src/open_vc_attn/_kernels/blackwell/flash_attn/cute/interface.py:110-179), restricted to what
those functions use: FP8 E4M3 Q/K/V with FP32 descales, ExpCast, optional causal mask, optional LSE,
optional prepacked V and optional repair prefix.  Anything else raises instead of degrading.
"""

import math

import torch

from . import _lib

_status_words = {}


def status_word(device):
    """Two uint32 per device for the kernel: [0] the current launch's word (cleared by the library before each
    launch), [1] sticky, OR-ed by any launch whose bounded wait expired."""
    return _status(device)[0]


def _status(device):
    key = torch.device(device).index
    if key is None:
        key = torch.cuda.current_device()
    if key not in _status_words:
        words = torch.zeros(2, dtype=torch.int32, device=torch.device("cuda", key))
        mirror = torch.zeros(1, dtype=torch.int32).pin_memory()  # host copy of words[1], refreshed after every launch
        _status_words[key] = (words, mirror)
    return _status_words[key]


def _failure(value):
    return RuntimeError(
        f"open_vc_attn attention kernel reported status {value:#x} (a bounded wait expired); "
        "the output of that call holds NaN"
    )


def _raise_if_flagged(device):
    """No synchronisation: looks at the host copy of the sticky word, which reflects every launch whose
    trailing 4-byte copy has completed.  Called at the start of each public attention call."""
    words, mirror = _status(device)
    value = int(mirror[0])
    if value != 0:
        mirror.zero_()
        words[1:].zero_()
        raise _failure(value)


def _publish_status(device):
    """Stream-ordered 4-byte copy of the sticky word to pinned host memory (capturable in a CUDA graph)."""
    words, mirror = _status(device)
    mirror.copy_(words[1:], non_blocking=True)


def check_status(device):
    """Synchronise and raise if any attention launch on ``device`` gave up on a barrier wait since the last check."""
    words, mirror = _status(device)
    value = int(words[1].item())
    if value != 0:
        words[1:].zero_()
        mirror.zero_()
        raise _failure(value)


def _validate_packed_view(v):
    # src/open_vc_attn/_kernels/blackwell/flash_attn/cute/interface.py:206-217
    if v.ndim != 3:
        raise ValueError("v_prepacked requires a single-sequence [S,H,128] view")
    length, heads, dim = v.shape
    padded = (length + 127) // 128 * 128
    if (
        dim != 128
        or v.dtype != torch.float8_e4m3fn
        or tuple(v.stride()) != (1, dim * padded, padded)
        or v.storage_offset() != 0
        or v.untyped_storage().nbytes() < heads * dim * padded
    ):
        raise ValueError("v_prepacked must use the padded sequence-contiguous FP8 layout")


def flash_attn_fwd(
    q,
    k,
    v,
    *,
    q_descale=None,
    k_descale=None,
    v_descale=None,
    cu_seqlens_q=None,
    cu_seqlens_k=None,
    max_seqlen_q=None,
    max_seqlen_k=None,
    expcast=False,
    v_prepacked=False,
    causal=False,
    softmax_scale=None,
    mid_window_blocks=None,
    return_lse=False,
    repair_k_descale=None,
    v_smooth=False,
    v_smooth_means=None,
    v_smooth_scale=None,
    **unsupported,
):
    """FP8 ExpCast attention.  Returns (out bf16 in Q's shape, lse or None).

    With ``return_lse`` the second value is the float32 log-sum-exp of the scaled scores, [B,H,Sq] for 4-D and
    [H,Sq] for 3-D inputs (the shapes of cute/interface.py:410 of the reference).

    q [Sq,H,128] or [B,Sq,H,128] e4m3; k the same with Sk; v like k, or (v_prepacked) the logical
    [Sk,H,128] view of a [H,128,Sk_pad] buffer.  q_descale [B,H,>=ceil(Sq/128)], k_descale
    [B,H,ceil(Sk/128)], v_descale [B,H], all float32.  A 3-D call is one sequence spanning the whole tensor:
    cu_seqlens_* may be passed only in the single-sequence form the reference's public functions build
    (int32 [2] = [0, S], api.py:52-55; its values are the caller's contract and are not read), max_seqlen_*
    only equal to the tensor's length; packed multi-sequence input raises instead of attending across
    sequences.
    v_smooth: V holds residual codes of one sequence, ``v_smooth_means`` [1,ceil(Sk/128),H,128] (float32 or
    bfloat16) the block means in code units and ``v_smooth_scale`` [1,H,128] float32 the channel scales; no
    descales are taken on that path.

    A launch whose bounded waits expire leaves NaN in its output; that is reported by the next call on the
    device (without synchronising) or by ``check_status`` (which synchronises).
    """
    if unsupported:
        raise NotImplementedError(f"Unsupported kernel options in this build: {sorted(unsupported)}")
    if not expcast:
        raise NotImplementedError("Only the ExpCast FP8 path (expcast=True) is built")
    if causal and (mid_window_blocks is not None or repair_k_descale is not None or v_smooth):
        raise ValueError("causal attention uses the plain key scan (mid_window_blocks=None) and takes no repair prefix or V-Smooth")
    if any(t.dtype != torch.float8_e4m3fn for t in (q, k, v)):
        raise ValueError("ExpCast attention expects float8_e4m3fn Q/K/V")
    for name, cu, t, given_max in (("q", cu_seqlens_q, q, max_seqlen_q), ("k", cu_seqlens_k, k, max_seqlen_k)):
        if cu is not None:
            if t.ndim != 3:
                raise ValueError(f"cu_seqlens_{name} goes with packed [S,H,128] input, not with a batched tensor")
            if tuple(cu.shape) != (2,):
                raise NotImplementedError(
                    f"cu_seqlens_{name} with {cu.numel() - 1} sequences: packed multi-sequence (varlen) input is not "
                    "built; call once per sequence"
                )
        if given_max is not None and t.ndim >= 3 and int(given_max) != t.shape[-3]:
            raise ValueError(f"max_seqlen_{name}={given_max} does not match the sequence length {t.shape[-3]}")
    if v_smooth:
        return _v_smooth_forward(q, k, v, v_smooth_means, v_smooth_scale, softmax_scale, mid_window_blocks,
                                 (q_descale, k_descale, v_descale, repair_k_descale), v_prepacked), None
    if v_smooth_means is not None or v_smooth_scale is not None:
        raise ValueError("v_smooth_means / v_smooth_scale need v_smooth=True")
    if q_descale is None or k_descale is None or v_descale is None:
        raise ValueError("ExpCast attention expects q_descale, k_descale and v_descale")
    if v_prepacked:
        _validate_packed_view(v)
    if q.ndim not in (3, 4) or k.ndim != q.ndim or q.shape[-1] != 128 or k.shape[-1] != 128:
        raise ValueError("Expected [S,H,128] or [B,S,H,128] Q/K")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(128)
    if not math.isfinite(softmax_scale) or softmax_scale <= 0.0:
        raise ValueError("ExpCast requires a positive finite softmax_scale")

    q, k = q.contiguous(), k.contiguous()
    batch = q.shape[0] if q.ndim == 4 else 1
    sq, heads = q.shape[-3], q.shape[-2]
    sk = k.shape[-3]
    if k.shape[-2] != heads or (q.ndim == 4 and k.shape[0] != batch):
        raise ValueError("Q and K must agree on batch and heads (MHA)")
    if v_prepacked and batch != 1:
        raise ValueError("v_prepacked requires a single-sequence [S,H,128] view")
    if tuple(v.shape[-3:]) != (sk, heads, 128):
        raise ValueError("K and V shapes must match")
    device = q.device
    for t, name, shape in (
        (q_descale, "q_descale", (batch, heads)),
        (k_descale, "k_descale", (batch, heads)),
    ):
        if t.dtype != torch.float32 or t.device != device or t.dim() != 3 or tuple(t.shape[:2]) != shape:
            raise ValueError(f"{name} must be float32 [batch, heads, blocks] on the input device")
    k_blocks = (sk + 127) // 128
    if q_descale.shape[2] < (sq + 127) // 128 or k_descale.shape[2] != k_blocks:
        raise ValueError("descale block counts do not match the sequence lengths")
    if v_descale.dtype != torch.float32 or v_descale.device != device or tuple(v_descale.shape) != (batch, heads):
        raise ValueError("v_descale must be float32 [batch, heads] on the input device")
    repair_rows = 0
    if repair_k_descale is not None:
        # src/open_vc_attn/_kernels/blackwell/flash_attn/cute/interface.py:538-558
        rows = repair_k_descale.shape[-1] if repair_k_descale.dim() == 3 else 0
        if (
            repair_k_descale.dim() != 3
            or tuple(repair_k_descale.shape[:2]) != (batch, heads)
            or rows == 0
            or rows % 128 != 0
            or rows >= sk
            or repair_k_descale.dtype != torch.float32
            or repair_k_descale.device != device
            or not repair_k_descale.is_contiguous()
            or batch != 1
        ):
            raise ValueError(
                "repair_k_descale must be contiguous float32 [batch, kv_heads, R] on the "
                f"input device with 0 < R < {sk} and R a multiple of 128"
            )
        repair_rows = rows
    window = -1 if mid_window_blocks is None else int(mid_window_blocks)
    if window < -1:
        raise ValueError("mid_window_blocks must be None or >= 0")

    lib = _lib.load()
    _raise_if_flagged(device)
    with torch.cuda.device(device):
        flags = _lib.OVC_ATTN_CAUSAL if causal else 0
        if v_prepacked:
            packed_ptr = v.data_ptr()
            keep = v
        elif repair_rows == 0:
            # V codes as the quantiser wrote them, [.., S, H, 128]: the kernel reads them as the MN-major operand
            # of P V (what the reference's general path does, cute/flash_fwd_sm100.py:726-729), no packing pass.
            keep = v.contiguous()
            packed_ptr = keep.data_ptr()
            flags |= _lib.OVC_ATTN_V_UNPACKED
        else:
            from .quantization import pack_v

            keep = pack_v(v.contiguous())
            packed_ptr = keep.data_ptr()
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=device)
        q_descale, k_descale, v_descale = q_descale.contiguous(), k_descale.contiguous(), v_descale.contiguous()
        repair_ptr = None if repair_k_descale is None else repair_k_descale.data_ptr()
        tail = (batch, sq, sk, heads, float(softmax_scale), window, status_word(device).data_ptr(), _lib.stream_pointer(device))
        lse = None
        if return_lse or flags:
            if return_lse:
                lse = torch.empty((batch, heads, sq) if q.ndim == 4 else (heads, sq), dtype=torch.float32, device=device)
            _lib.check(
                lib.ovc_attention_ex(
                    q.data_ptr(), k.data_ptr(), packed_ptr, q_descale.data_ptr(), q_descale.shape[2], k_descale.data_ptr(),
                    v_descale.data_ptr(), repair_ptr, repair_rows, out.data_ptr(), None if lse is None else lse.data_ptr(),
                    flags, *tail,
                ),
                "ovc_attention_ex",
            )
        else:
            _lib.check(
                lib.ovc_attention(
                    q.data_ptr(), k.data_ptr(), packed_ptr, q_descale.data_ptr(), q_descale.shape[2], k_descale.data_ptr(),
                    v_descale.data_ptr(), repair_ptr, repair_rows, out.data_ptr(), *tail,
                ),
                "ovc_attention",
            )
        _publish_status(device)
        del keep
    return out, lse


_unit_descales = {}


def _unit_descale(device, count):
    """A device buffer of at least ``count`` ones (the V-Smooth path has no Q/K/V descales)."""
    key = torch.device(device).index
    have = _unit_descales.get(key)
    if have is None or have.numel() < count:
        have = torch.ones(max(count, 1 << 16), dtype=torch.float32, device=device)
        _unit_descales[key] = have
    return have


def _v_smooth_forward(q, k, v, means, scale, softmax_scale, mid_window_blocks, descales, v_prepacked):
    # Argument rules of src/open_vc_attn/_kernels/blackwell/flash_attn/cute/interface.py:560-600 for v_smooth.
    if any(d is not None for d in descales):
        raise NotImplementedError("V-Smooth attention takes no descales or repair prefix in this build")
    if v_prepacked:
        raise NotImplementedError("V-Smooth attention takes sequence-major V codes")
    if q.ndim == 4:
        if q.shape[0] != 1:
            raise ValueError("V-Smooth attention supports one sequence")
        q, k, v = q[0], k[0], v[0]
    if q.ndim != 3 or k.ndim != 3 or q.shape[-1] != 128 or tuple(v.shape) != tuple(k.shape) or k.shape[1] != q.shape[1]:
        raise ValueError("Expected [S,H,128] Q/K/V with matching heads")
    sq, heads, _ = q.shape
    sk = k.shape[0]
    blocks = (sk + 127) // 128
    device = q.device
    if means is None or scale is None:
        raise ValueError("v_smooth=True needs v_smooth_means and v_smooth_scale")
    if (
        means.numel() != blocks * heads * 128
        or tuple(means.shape[-3:]) != (blocks, heads, 128)
        or means.device != device
        or means.dtype not in (torch.float32, torch.bfloat16)
    ):
        raise ValueError("v_smooth_means must be [1, key blocks, heads, 128] float32 or bfloat16 on the input device")
    if scale.numel() != heads * 128 or tuple(scale.shape[-2:]) != (heads, 128) or scale.device != device or scale.dtype != torch.float32:
        raise ValueError("v_smooth_scale must be float32 [1, heads, 128] on the input device")
    if softmax_scale is None:
        softmax_scale = 1.0 / math.sqrt(128)
    if not math.isfinite(softmax_scale) or softmax_scale <= 0.0:
        raise ValueError("ExpCast requires a positive finite softmax_scale")
    window = -1 if mid_window_blocks is None else int(mid_window_blocks)
    if window < -1:
        raise ValueError("mid_window_blocks must be None or >= 0")
    lib = _lib.load()
    _raise_if_flagged(device)
    with torch.cuda.device(device):
        from .quantization import pack_v

        q, k = q.contiguous(), k.contiguous()
        packed = pack_v(v.contiguous())
        means = means.float().contiguous()
        scale = scale.contiguous()
        ones = _unit_descale(device, heads * ((max(sq, sk) + 127) // 128))
        out = torch.empty(q.shape, dtype=torch.bfloat16, device=device)
        workspace = torch.empty(lib.ovc_attention_vsmooth_workspace(sk, heads), dtype=torch.uint8, device=device)
        _lib.check(
            lib.ovc_attention_vsmooth(
                q.data_ptr(), k.data_ptr(), packed.data_ptr(), ones.data_ptr(), means.data_ptr(), scale.data_ptr(),
                workspace.data_ptr(), out.data_ptr(), sq, sk, heads, float(softmax_scale), window, status_word(device).data_ptr(),
                _lib.stream_pointer(device),
            ),
            "ovc_attention_vsmooth",
        )
        _publish_status(device)
        del packed, workspace
    return out


_flash_attn_fwd = flash_attn_fwd
