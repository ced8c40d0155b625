"""Helpers shared by the GPU parity tests."""

import numpy as np
import torch

from oracle import attention as oatt
from oracle import prep as oprep

DEV = "cuda:0"


def u8(t):
    return t.contiguous().view(torch.uint8).cpu().numpy()


def f32(t):
    return t.float().cpu().numpy()


def packed_buffer(view):
    """The [H,128,S_pad] buffer behind a prepacked [S,H,128] view."""
    s, h, d = view.shape
    padded = (s + 127) // 128 * 128
    flat = torch.empty(0, dtype=torch.uint8, device=view.device).set_(view.untyped_storage(), 0, (h, d, padded))
    return flat.cpu().numpy()


def structured_qkv(s, h, seed, dtype=torch.bfloat16, device=DEV):
    """Synthetic stand-in for the video-DiT captures (see open_vc_attn/synthetic.py)."""
    from open_vc_attn.synthetic import video_dit_qkv

    return video_dit_qkv(s, h, seed=seed, dtype=dtype, device=device)


def oracle_rows(prepared, m_blocks, heads, window=4, repair_kd=None):
    """Oracle output for the query rows of the given 256-row blocks and heads, from prepared FP8
    tensors (packed or row-major V).  Returns (rows index array, float32 [len(rows), len(heads), 128])."""
    q8, k8 = u8(prepared.q), u8(prepared.k)
    s_k = k8.shape[0]
    if getattr(prepared, "v_prepacked", False):
        v8 = packed_buffer(prepared.v)[:, :, :s_k].transpose(2, 0, 1)
    else:
        v8 = u8(prepared.v)
    heads = list(heads)
    out = oatt.expcast_attention(
        q8[:, heads], k8[:, heads], np.ascontiguousarray(v8[:, heads]),
        f32(prepared.q_descale)[0][heads], f32(prepared.k_descale)[0][heads], f32(prepared.v_descale)[0][heads],
        mid_window_blocks=window, rows=list(m_blocks),
        repair_k_descale=None if repair_kd is None else f32(repair_kd)[0][heads],
    )
    rows = np.concatenate([np.arange(256 * m, min(256 * m + 256, q8.shape[0])) for m in m_blocks])
    return rows, out[rows]


def hw_div(a, b):
    """a / b evaluated by the GPU with the preparation kernels' division (ovc_div_full); float32 numpy arrays."""
    from open_vc_attn import _lib

    lib = _lib.load()
    a = np.ascontiguousarray(a, dtype=np.float32)
    b = np.ascontiguousarray(np.broadcast_to(np.asarray(b, dtype=np.float32), a.shape))
    ta, tb = torch.from_numpy(a.reshape(-1).copy()).to(DEV), torch.from_numpy(b.reshape(-1).copy()).to(DEV)
    tq = torch.empty_like(ta)
    _lib.check(lib.ovc_div_full(ta.data_ptr(), tb.data_ptr(), tq.data_ptr(), ta.numel(), _lib.stream_pointer(DEV)), "ovc_div_full")
    return tq.cpu().numpy().reshape(a.shape)


def hw_arith():
    """The oracle's arithmetic with the hardware's own reciprocals (see oracle/prep.py)."""
    def recip(b):
        b = np.asarray(b, dtype=np.float32)
        return hw_div(np.ones_like(b), b)

    return oprep.Arithmetic(recip=recip, contract=True)
