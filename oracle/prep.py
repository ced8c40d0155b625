"""CPU restatement of the reference's FP8 input preparation.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

All arithmetic is IEEE float32 in numpy, in the operation order of the
reference kernels: one division ``448 / amax``, one multiply, clamp, then the
round-to-nearest-even E4M3 cast.  Inputs are float16/bfloat16 values already
widened (exactly) to float32 arrays.
"""

import math

import numpy as np

from .fp8 import e4m3_decode, e4m3_encode

F32 = np.float32
QMAX = F32(448.0)
FLOOR = F32(1e-12)
BLOCK = 128


def _blocks(length):
    return (length + BLOCK - 1) // BLOCK


def quantize_per_block(x):
    """Q/K quantiser: one scale per (batch, head, 128-token block).

    Follows _per_block_quant_kernel, src/open_vc_attn/quantization.py:154-188
    (rows past S read as 0; amax floored at 1e-12; descale = amax/448;
    codes = cast(clamp(x * (448/amax)))).

    x: float32 [B,S,H,128].  Returns (codes uint8 [B,S,H,128], descale f32 [B,H,blocks]).
    """
    x = np.asarray(x, dtype=F32)
    b, s, h, d = x.shape
    nb = _blocks(s)
    padded = np.zeros((b, nb * BLOCK, h, d), dtype=F32)
    padded[:, :s] = x
    tiles = padded.reshape(b, nb, BLOCK, h, d)
    amax = np.maximum(np.abs(tiles).max(axis=(2, 4)), FLOOR)  # [B,nb,H]
    descale = (amax / QMAX).astype(F32)
    scale = (QMAX / amax).astype(F32)
    scaled = np.clip(tiles * scale[:, :, None, :, None], -QMAX, QMAX).astype(F32)
    codes = e4m3_encode(scaled).reshape(b, nb * BLOCK, h, d)[:, :s]
    return np.ascontiguousarray(codes), np.ascontiguousarray(descale.transpose(0, 2, 1))


def head_amax(v):
    """Per-(batch, head) max |v| (order independent).

    Follows _per_head_amax_kernel, src/open_vc_attn/quantization.py:23-53.
    v: float32 [B,S,H,128] -> f32 [B,H].
    """
    v = np.asarray(v, dtype=F32)
    return np.abs(v).max(axis=(1, 3)).astype(F32)


def quantize_per_head(v):
    """V quantiser: one scale per (batch, head).

    Follows _per_head_scale_cast_kernel and the host division,
    src/open_vc_attn/quantization.py:57-93,144.
    Returns (codes uint8 [B,S,H,128], descale f32 [B,H]).
    """
    v = np.asarray(v, dtype=F32)
    amax = np.maximum(head_amax(v), FLOOR)
    scale = (QMAX / amax).astype(F32)
    scaled = np.clip(v * scale[:, None, :, None], -QMAX, QMAX).astype(F32)
    return e4m3_encode(scaled), (amax / QMAX).astype(F32)


def pack_v(codes):
    """FP8 bytes [S,H,128] (or [B,S,H,128]) -> [H,128,S_pad] ([B,H,128,S_pad]), zero tail.

    Follows transpose_v / pack_v, src/open_vc_attn/_kernels/blackwell/flash_attn/cute/v_layout.py:8-49.
    """
    codes = np.asarray(codes, dtype=np.uint8)
    squeeze = codes.ndim == 3
    if squeeze:
        codes = codes[None]
    b, s, h, d = codes.shape
    padded = _blocks(s) * BLOCK
    out = np.zeros((b, h, d, padded), dtype=np.uint8)
    out[..., :s] = codes.transpose(0, 2, 3, 1)
    return out[0] if squeeze else out


def prepare_general(q, k, v):
    """prepare_fp8, src/open_vc_attn/api.py:102-118 (Q/K per block, V per head).

    Inputs float32 [B,S,H,128]; returns a dict of numpy arrays.
    """
    q8, qs = quantize_per_block(q)
    k8, ks = quantize_per_block(k)
    v8, vs = quantize_per_head(v)
    return dict(q=q8, k=k8, v=v8, q_descale=qs, k_descale=ks, v_descale=vs)


def prepare_fused(q, k, v):
    """prepare_fp8_fused, src/open_vc_attn/preparation.py:83-162.

    Same groups and scales as prepare_general for one sequence, plus: the Q
    descale row is padded to an even block count with 1.0 (:47-49,116) and V is
    returned in the packed layout [H,128,S_pad] with a zero tail (:73-78).
    Inputs float32 [S,H,128].
    """
    general = prepare_general(q[None], k[None], v[None])
    s, h, _ = q.shape
    nb = _blocks(s)
    q_blocks = (nb + 1) // 2 * 2
    qs = np.ones((1, h, q_blocks), dtype=F32)
    qs[..., :nb] = general["q_descale"]
    return dict(
        q=general["q"][0],
        k=general["k"][0],
        v_packed=pack_v(general["v"][0]),
        q_descale=qs,
        k_descale=general["k_descale"],
        v_descale=general["v_descale"],
    )


def repair_counts(budget, length):
    """selected = round(budget*S) (banker's rounding), rows padded to 128.

    src/open_vc_attn/v_repair.py:139-140.
    """
    selected = round(budget * length)
    return selected, math.ceil(selected / BLOCK) * BLOCK


def v_residual_score(v, codes, descale):
    """Per-token squared FP8 rounding residual of V, summed over channels.

    Follows _v_quant_score_kernel, src/open_vc_attn/v_repair.py:53-76.
    v f32 [S,H,128], codes uint8 [S,H,128], descale f32 [H] -> f32 [H,S].
    The float32 summation order over the 128 channels is not specified by the
    reference (a Triton reduction); pairwise numpy summation is used here.
    """
    residual = (v - e4m3_decode(codes) * descale[None, :, None]).astype(F32)
    return np.ascontiguousarray((residual * residual).sum(axis=2, dtype=F32).T)


def prepare_repair(q, k, v, budget, index=None):
    """prepare_v_repair, src/open_vc_attn/v_repair.py:117-233, for one sequence.

    Inputs float32 [S,H,128].  ``index`` (int [H,selected]) overrides the top-k
    choice so that a device-side selection can be replayed exactly (the tie
    order of an unsorted top-k is unspecified, :193).
    """
    s, h, d = v.shape
    selected, rows = repair_counts(budget, s)
    if selected == 0:
        out = prepare_fused(q, k, v)
        out.update(repair_k_descale=None, repair_tokens=0, selected_tokens=0, total=s)
        return out
    q8, qs = quantize_per_block(q[None])
    k8, ks = quantize_per_block(k[None])
    v8, vs = quantize_per_head(v[None])
    score = v_residual_score(v, v8[0], vs[0])
    if index is None:
        index = np.argsort(-score, axis=1, kind="stable")[:, :selected]
    index = np.asarray(index, dtype=np.int64)
    total = rows + s
    k_all = np.zeros((total, h, d), dtype=np.uint8)
    v_all = np.zeros((total, h, d), dtype=np.uint8)
    k_all[rows:] = k8[0]
    v_all[rows:] = v8[0]
    repair_kd = np.zeros((1, h, rows), dtype=F32)
    for head in range(h):
        for row in range(rows):
            # _repair_rows_kernel, src/open_vc_attn/v_repair.py:80-113: pad rows
            # (row >= selected) reuse index[head, 0] for K and carry a zero V.
            source = int(index[head, row if row < selected else 0])
            k_all[row, head] = k8[0, source, head]
            repair_kd[0, head, row] = ks[0, head, source // BLOCK]
            if row < selected:
                descale = vs[0, head]
                rounded = (e4m3_decode(v8[0, source, head]) * descale).astype(F32)
                residual = (v[source, head] - rounded).astype(F32)
                scaled = np.clip((residual / descale).astype(F32), -QMAX, QMAX)
                v_all[row, head] = e4m3_encode(scaled)
    ks_all = np.concatenate([np.ones((1, h, rows // BLOCK), dtype=F32), ks], axis=2)
    return dict(
        q=q8[0],
        k=k_all,
        v_packed=pack_v(v_all),
        q_descale=qs,
        k_descale=ks_all,
        v_descale=vs,
        repair_k_descale=repair_kd,
        repair_tokens=rows,
        selected_tokens=selected,
        total=total,
        score=score,
        index=index,
    )
