"""CPU restatement of the reference's FP8 ExpCast forward attention.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Parity status: the reference stores no golden outputs for its attention kernel
and the kernel cannot run without a Blackwell GPU and its pinned CuTe-DSL
version, so this restatement is pinned only by the worked examples in the
reference's technical report (ExpCast codes for given scores) and by the
tolerance against exact attention that the reference's own tests use.

Execution order follows the packed kernel of
src/open_vc_attn/_kernels/blackwell/flash_attn/cute/flash_fwd_sm100.py
(abbreviated ``fwd`` below) and ``cute/softmax.py`` / ``cute/utils.py``:

* scale folding                  fwd:3093-3107
* key-tile traversal             fwd:3350-3460
* running max / rescale factor   softmax.py:203-248
* ExpCast encoder (packed)       fwd:3749-3764, utils.py:704-795
* ExpCast encoder (general)      softmax.py:360-372,393-394, utils.py:798-821
* denominator = sum of decoded codes   fwd:903-905 (tensor core, N extension)
* repair tiles                   fwd:4597-4655, 3844-3848, 3478-3480
* final normalisation            fwd:4298-4303
* sequence-tail mask             cute/mask.py:126-136
"""

import math

import numpy as np

from .fp8 import E4M3_DECODE_F32, e4m3_decode

F32 = np.float32
F64 = np.float64
LOG2_E = math.log2(math.e)
TILE = 128
# 119.65 * 2^-24 as the float32 constant the reference embeds (bits 0x36EF4CCD).
PEAK_SUBNORMAL = np.array([0x36EF4CCD], dtype=np.uint32).view(np.float32)[0]


def _fma_rn(a, b, c):
    """Single-rounding float32 fused multiply-add (products of two float32 are exact in float64)."""
    return (a.astype(F64) * F64(b) + F64(c)).astype(F32)


def _fma_rd(a, b, c):
    """float32 FMA rounded toward minus infinity (fma.rm.f32)."""
    exact = a.astype(F64) * F64(b) + F64(c)
    near = exact.astype(F32)
    too_high = near.astype(F64) > exact
    return np.where(too_high, np.nextafter(near, F32(-np.inf)), near).astype(F32)


def tile_order(n_tiles, first_tile, m_block, mid_window_blocks, q_stages=2):
    """Key tiles in visiting order; repair tiles [0, first_tile) come last, descending.

    fwd:3350-3460.  ``first_tile`` is R/128 (0 without repair).
    """
    if mid_window_blocks is None:
        order = list(range(n_tiles - 1, first_tile - 1, -1))
    else:
        diag = q_stages * m_block + first_tile
        j0 = min(diag + mid_window_blocks, n_tiles - 1)
        order = list(range(j0, first_tile - 1, -1)) + list(range(n_tiles - 1, j0, -1))
    return order + list(range(first_tile - 1, -1, -1))


def encode_packed(scores, row_max, sigma, k_descale):
    """Encoder of the packed path: FP16-subnormal rounding trick.

    fwd:3749-3764 with utils.py:704-720 (bias, rounded down) and :746-795 (affine,
    cvt.rn.relu.f16x2.f32, low byte).  scores f32 [rows,128]; row_max f32 [rows].
    """
    code_scale0 = F32(sigma * F32(8.0 * 2.0**-24))
    bias = _fma_rd(-row_max, code_scale0, PEAK_SUBNORMAL)
    code_scale = F32(code_scale0 * F32(k_descale))
    y = (scores.astype(F64) * F64(code_scale) + bias.astype(F64)[:, None]).astype(F32)
    # FP16 subnormals step by 2^-24, so RN to FP16 of y in [0, 2^-14) is RNE of y*2^24.
    code = np.rint(np.maximum(y.astype(F64), 0.0) * 2.0**24)
    code = np.where(np.isnan(code), 0, code)
    return np.minimum(code, 255).astype(np.uint8)


def encode_general(scores, row_max, sigma, k_descale):
    """Encoder of the general path: saturating FMA to [0,1], then 120*y rounded to integer.

    softmax.py:360-372,393-394 and utils.py:798-821.
    """
    eff = F32(F32(sigma) * F32(k_descale))
    code_scale = F32(F32(eff * F32(8.0)) * F32(1.0 / 120.0))
    bias = (F32(119.65) - row_max * F32(F32(sigma) * F32(8.0))).astype(F32)
    bias = (bias * F32(1.0 / 120.0)).astype(F32)
    y = (scores.astype(F64) * F64(code_scale) + bias.astype(F64)[:, None]).astype(F32)
    y = np.clip(np.where(np.isnan(y), 0, y), 0.0, 1.0).astype(F32)
    return np.rint(y.astype(F64) * 120.0).astype(np.uint8)


def expcast_attention(
    q8,
    k8,
    v8,
    q_descale,
    k_descale,
    v_descale,
    *,
    softmax_scale=None,
    mid_window_blocks=4,
    repair_k_descale=None,
    encoder="packed",
    rows=None,
    v_smooth_means=None,
    v_channel_scale=None,
    return_lse=False,
    causal=False,
):
    """ExpCast attention for one (batch item, head set) on FP8 codes.

    q8 uint8 [Sq,H,128]; k8, v8 uint8 [Sk,H,128] (Sk includes any repair prefix);
    q_descale f32 [H,>=ceil(Sq/128)]; k_descale f32 [H,ceil(Sk/128)]; v_descale f32 [H];
    repair_k_descale f32 [H,R] or None.  ``rows`` optionally restricts the query rows
    computed to a list of 256-row CTA blocks (m_block indices); other rows stay zero.
    V-Smooth (fwd:4857-4863): v8 holds residual codes, ``v_smooth_means`` f32 [tiles,H,128] the block
    means in code units and ``v_channel_scale`` f32 [H,128]; each tile adds (sum of its decoded
    probabilities) x (its block mean) to the accumulator and the result is scaled per channel.
    Returns float32 [Sq,H,128] already rounded to bfloat16 precision; with ``return_lse`` also the float32
    log-sum-exp [H,Sq] = (m*sigma + log2(l) - 8) ln 2, -inf where l is 0 or NaN (fwd:4437-4475).
    ``causal``: key column c is visible to query row r iff c < r + 1 + Sk - Sq (cute/mask.py:186-199); a 256-row
    block visits only the tiles that one of its rows can see (at least one), in the plain descending order.
    """
    sq, h, d = q8.shape
    sk = k8.shape[0]
    assert d == TILE
    tau = 1.0 / math.sqrt(d) if softmax_scale is None else float(softmax_scale)
    scale_log2 = F32(tau * LOG2_E)
    n_tiles = (sk + TILE - 1) // TILE
    repair_rows = 0 if repair_k_descale is None else repair_k_descale.shape[-1]
    first_tile = repair_rows // TILE
    encode = encode_packed if encoder == "packed" else encode_general

    qf = e4m3_decode(q8)
    kf = np.zeros((n_tiles * TILE, h, d), dtype=F32)
    kf[:sk] = e4m3_decode(k8)
    vf = np.zeros((n_tiles * TILE, h, d), dtype=F32)
    vf[:sk] = e4m3_decode(v8)
    out = np.zeros((sq, h, d), dtype=F32)
    lse = np.zeros((h, sq), dtype=F32)
    m_blocks = (sq + 2 * TILE - 1) // (2 * TILE)
    todo = range(m_blocks) if rows is None else rows
    q_blocks = q_descale.shape[-1]

    for head in range(h):
        for m_block in todo:
            if causal:
                assert mid_window_blocks is None and first_tile == 0
                limit = min((m_block + 1) * 2 * TILE, sq) + sk - sq  # columns below this are visible to the block's last row
                visible = max(1, min(n_tiles, (limit + TILE - 1) // TILE))
                order = list(range(visible - 1, -1, -1))
            else:
                order = tile_order(n_tiles, first_tile, m_block, mid_window_blocks)
            for stage in range(2):
                q_tile = 2 * m_block + stage
                r0 = q_tile * TILE
                if r0 >= sq:
                    continue
                r1 = min(r0 + TILE, sq)
                q_rows = qf[r0:r1, head]
                qd = q_descale[head, q_tile] if q_tile < q_blocks else F32(1.0)
                sigma = F32(scale_log2 * F32(qd))
                run_max = None
                acc = np.zeros((r1 - r0, d), dtype=F32)
                denom = np.zeros(r1 - r0, dtype=F32)
                saved = None
                for tile in order:
                    c0 = tile * TILE
                    s_raw = (q_rows @ kf[c0 : c0 + TILE, head].T).astype(F32)
                    if tile == n_tiles - 1 and sk - c0 < TILE:
                        s_raw[:, sk - c0 :] = -np.inf
                    if causal:
                        columns = c0 + np.arange(TILE)[None, :]
                        rows_here = np.arange(r0, r1)[:, None]
                        s_raw = np.where(columns < rows_here + 1 + sk - sq, s_raw, F32(-np.inf)).astype(F32)
                    if tile < first_tile:
                        s_raw = (s_raw * repair_k_descale[head, c0 : c0 + TILE][None, :]).astype(F32)
                        kd = F32(1.0)
                    else:
                        kd = F32(k_descale[head, tile])
                    tile_max = (s_raw.max(axis=1) * kd).astype(F32)
                    if run_max is None:
                        new_max = tile_max
                        alpha = np.zeros_like(tile_max)
                    else:
                        new_max = np.maximum(run_max, tile_max)
                        safe = np.where(np.isneginf(new_max), F32(0), new_max)
                        alpha = np.exp2(((run_max - safe) * sigma).astype(F32)).astype(F32)
                    safe = np.where(np.isneginf(new_max), F32(0), new_max).astype(F32)
                    codes = encode(s_raw, safe, sigma, kd)
                    if tile == first_tile - 1 and repair_rows:
                        saved = denom.copy()  # denominator of the original tokens only
                    if run_max is not None:
                        acc = (acc * alpha[:, None]).astype(F32)
                        denom = (denom * alpha).astype(F32)
                    run_max = new_max
                    p = E4M3_DECODE_F32[codes]
                    acc = (acc + p @ vf[c0 : c0 + TILE, head]).astype(F32)
                    tile_sum = p.sum(axis=1, dtype=F32)
                    if v_smooth_means is not None:
                        acc = (acc + tile_sum[:, None] * v_smooth_means[tile, head][None, :]).astype(F32)
                    denom = (denom + tile_sum).astype(F32)
                if saved is not None:
                    denom = saved
                bad = (denom == 0) | np.isnan(denom)
                factor = (F32(1.0) / np.where(bad, F32(1.0), denom)).astype(F32) * F32(v_descale[head])
                if v_channel_scale is not None:
                    acc = (acc * v_channel_scale[head][None, :]).astype(F32)
                out[r0:r1, head] = acc * factor[:, None]
                with np.errstate(divide="ignore", invalid="ignore"):
                    value = ((run_max * sigma + np.log2(np.where(bad, F32(1.0), denom)).astype(F32)).astype(F32) - F32(8.0)) * F32(math.log(2.0))
                lse[head, r0:r1] = np.where(bad, F32(-np.inf), value)
    if return_lse:
        return _round_bf16(out), lse
    return _round_bf16(out)


def _round_bf16(x):
    """float32 -> nearest-even bfloat16, returned as float32."""
    bits = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    rounded = (bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000
    return rounded.astype(np.uint32).view(F32)


def exact_attention(q, k, v, softmax_scale=None, rows=None, causal=False):
    """Exact softmax attention in float64 (tests/gpu/test_attention.py:18-24 in the reference).

    q [Sq,H,128], k/v [Sk,H,128] float arrays.  ``rows``: optional index array of query rows.
    Returns float64 [len(rows) or Sq, H, 128].
    """
    q = np.asarray(q, dtype=F64)
    k = np.asarray(k, dtype=F64)
    v = np.asarray(v, dtype=F64)
    full_rows = q.shape[0]
    if rows is not None:
        q = q[rows]
    tau = 1.0 / math.sqrt(q.shape[-1]) if softmax_scale is None else float(softmax_scale)
    out = np.empty(q.shape, dtype=F64)
    for head in range(q.shape[1]):
        s = (q[:, head] @ k[:, head].T) * tau
        if causal:
            row_index = (np.arange(q.shape[0]) if rows is None else np.asarray(rows))[:, None]
            s = np.where(np.arange(k.shape[0])[None, :] < row_index + 1 + k.shape[0] - full_rows, s, -np.inf)
        top = s.max(axis=1, keepdims=True)
        p = np.exp(s - np.where(np.isneginf(top), 0.0, top))
        total = p.sum(axis=1, keepdims=True)
        out[:, head] = (p @ v[:, head]) / np.where(total == 0, 1.0, total)
    return out


def relative_l2(a, b):
    a = np.asarray(a, dtype=F64)
    b = np.asarray(b, dtype=F64)
    return float(np.linalg.norm(a - b) / max(np.linalg.norm(b), 1e-300))
