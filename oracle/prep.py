"""CPU restatement of the reference's FP8 input preparation.

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

All arithmetic is float32 in numpy, in the operation order of the reference
kernels: one division ``448 / amax``, one multiply, clamp, then the
round-to-nearest-even E4M3 cast.  Inputs are float16/bfloat16 values already
widened (exactly) to float32 arrays.

Two details of the reference are decided by its compiler, not by its source, and
they change results (16-bit inputs put many scaled values exactly on E4M3 rounding
ties, where the last bit of the scale picks the code):

* ``a / b``.  On a GPU Triton lowers it to ``div.full.f32``: the dividend times the
  hardware's approximate reciprocal of ``b``, rounded once.  That reciprocal is within
  one ulp of 1/b but is not reproducible on a CPU, so an ``Arithmetic`` carries a
  ``recip`` function: tests feed it the hardware's values (a table stored with the
  fixtures made on a B200, or the library's ``ovc_div_full`` on the GPU); the default
  ``RN(1/b)`` is exact for b = 448 and for most other b.
* ``x - c * d``.  Contracted into one FMA on the GPU.

``GPU`` is what the reference computes on the hardware and what the CUDA kernels
follow.  ``IEEE`` (true division, separate roundings) is what Triton's CPU interpreter
computes; it pins this file to the interpreter-made fixtures.
"""

import math

import numpy as np

from .fp8 import e4m3_decode, e4m3_encode

F32 = np.float32
QMAX = F32(448.0)
FLOOR = F32(1e-12)
BLOCK = 128


def recip_model(b):
    """RN(1/b): the stand-in for the hardware's approximate reciprocal (differs from it by one ulp for some b)."""
    return (F32(1.0) / np.asarray(b, dtype=F32)).astype(F32)


class RecipTable:
    """Hardware reciprocals recorded on a GPU: ``b`` values (float32) and ``r`` = div.full.f32(1, b)."""

    def __init__(self, b, r):
        self._map = dict(zip(np.asarray(b, dtype=F32).view(np.uint32).tolist(), np.asarray(r, dtype=F32).tolist()))

    def __call__(self, b):
        b = np.asarray(b, dtype=F32)
        flat = [self._map[bits] for bits in b.reshape(-1).view(np.uint32).tolist()]  # KeyError: value not recorded
        return np.asarray(flat, dtype=F32).reshape(b.shape)


class Arithmetic:
    """How `/` and `x - c*d` are evaluated (see the module docstring)."""

    def __init__(self, recip=None, contract=True):
        self.recip, self.contract = recip, contract

    def div(self, a, b):
        a, b = np.asarray(a, dtype=F32), np.asarray(b, dtype=F32)
        if self.recip is None:
            return (a / b).astype(F32)
        return (a * self.recip(b)).astype(F32)

    def sub_mul(self, x, c, d):
        """x - c*d: one rounding when contracted (extended precision holds the product exactly)."""
        if not self.contract:
            return (x - (c * d).astype(F32)).astype(F32)
        wide = np.longdouble
        return (np.asarray(x, dtype=wide) - np.asarray(c, dtype=wide) * np.asarray(d, dtype=wide)).astype(F32)


IEEE = Arithmetic(recip=None, contract=False)
GPU = Arithmetic(recip=recip_model, contract=True)


def _blocks(length):
    return (length + BLOCK - 1) // BLOCK


def quantize_per_block(x, arith=GPU):
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
    descale = arith.div(amax, QMAX)
    scale = arith.div(QMAX, amax)
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


def quantize_per_head(v, arith=GPU):
    """V quantiser: one scale per (batch, head).

    Follows _per_head_scale_cast_kernel and the host division,
    src/open_vc_attn/quantization.py:57-93,144.  On a GPU that host division is torch's, which
    multiplies by the float32 reciprocal of the scalar 448: the same value as div.full.f32 gives.
    Returns (codes uint8 [B,S,H,128], descale f32 [B,H]).
    """
    v = np.asarray(v, dtype=F32)
    amax = np.maximum(head_amax(v), FLOOR)
    scale = arith.div(QMAX, amax)
    scaled = np.clip(v * scale[:, None, :, None], -QMAX, QMAX).astype(F32)
    return e4m3_encode(scaled), arith.div(amax, QMAX)


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


def prepare_general(q, k, v, arith=GPU):
    """prepare_fp8, src/open_vc_attn/api.py:102-118 (Q/K per block, V per head).

    Inputs float32 [B,S,H,128]; returns a dict of numpy arrays.
    """
    q8, qs = quantize_per_block(q, arith)
    k8, ks = quantize_per_block(k, arith)
    v8, vs = quantize_per_head(v, arith)
    return dict(q=q8, k=k8, v=v8, q_descale=qs, k_descale=ks, v_descale=vs)


def prepare_fused(q, k, v, arith=GPU):
    """prepare_fp8_fused, src/open_vc_attn/preparation.py:83-162.

    Same groups and scales as prepare_general for one sequence, plus: the Q
    descale row is padded to an even block count with 1.0 (:47-49,116) and V is
    returned in the packed layout [H,128,S_pad] with a zero tail (:73-78).
    Inputs float32 [S,H,128].
    """
    general = prepare_general(q[None], k[None], v[None], arith)
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


def v_residual_score(v, codes, descale, arith=GPU):
    """Per-token squared FP8 rounding residual of V, summed over channels.

    Follows _v_quant_score_kernel, src/open_vc_attn/v_repair.py:53-76.
    v f32 [S,H,128], codes uint8 [S,H,128], descale f32 [H] -> f32 [H,S].
    The float32 summation order over the 128 channels is not specified by the
    reference (a Triton reduction); pairwise numpy summation is used here.
    """
    residual = arith.sub_mul(v, e4m3_decode(codes), descale[None, :, None])
    return np.ascontiguousarray((residual * residual).sum(axis=2, dtype=F32).T)


def prepare_repair(q, k, v, budget, index=None, arith=GPU):
    """prepare_v_repair, src/open_vc_attn/v_repair.py:117-233, for one sequence.

    Inputs float32 [S,H,128].  ``index`` (int [H,selected]) overrides the top-k
    choice so that a device-side selection can be replayed exactly (the tie
    order of an unsorted top-k is unspecified, :193).
    """
    s, h, d = v.shape
    selected, rows = repair_counts(budget, s)
    if selected == 0:
        out = prepare_fused(q, k, v, arith)
        out.update(repair_k_descale=None, repair_tokens=0, selected_tokens=0, total=s)
        return out
    q8, qs = quantize_per_block(q[None], arith)
    k8, ks = quantize_per_block(k[None], arith)
    v8, vs = quantize_per_head(v[None], arith)
    score = v_residual_score(v, v8[0], vs[0], arith)
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
                residual = arith.sub_mul(v[source, head], e4m3_decode(v8[0, source, head]), descale)
                scaled = np.clip(arith.div(residual, np.full_like(residual, descale)), -QMAX, QMAX)
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
