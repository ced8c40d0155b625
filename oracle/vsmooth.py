"""CPU restatement of the reference's V-Smooth preparation (the VC-Attention baseline).

TEST INFRASTRUCTURE ONLY (see oracle/__init__.py).

Follows src/open_vc_attn/_kernels/blackwell/v_smooth.py of the reference:
  * k-means grouping of V tokens per head       prepare_v_smooth :245-313, _assign_values :10-39,
                                                 _accumulate_centers :42-73
  * block means, channel scales, residual codes  _block_stats :76-94, _block_write :97-134
Parity status: unpinned.  The reference's grouping uses BF16 tensor-core products whose accumulation
order is not specified, so labels of near-tied tokens (and with them the permutation) can differ between
implementations; tests therefore replay a given permutation and compare everything downstream of it.
Block sums are taken in float32 in the fixed two-level order of the CUDA kernel (see block_sum); the
reference's Triton reduction order is unspecified (on a B200 its means differ from these by at most a few ulp,
tests/test_gpu_prep_hw.py).  Everything computed from given block means is pinned bit for bit by the fixture the
reference's kernels produced on a B200 (tests/golden/prep_golden_gpu.npz, test_oracle_golden.py).
"""

import numpy as np

from .fp8 import e4m3_encode
from .prep import GPU

F32 = np.float32
BLOCK = 128


def _bf16(x):
    """Round float32 to bfloat16 (nearest even), returned as float32."""
    bits = np.ascontiguousarray(x, dtype=F32).view(np.uint32)
    return ((bits + 0x7FFF + ((bits >> 16) & 1)) & 0xFFFF0000).astype(np.uint32).view(F32)


def assign(values, centers):
    """labels[h, s] = argmin_k (|c_k|^2 - 2 v.c_k); first index wins ties.  values [H,S,128], centers [H,K,128]
    (both already BF16-representable float32)."""
    labels = np.empty(values.shape[:2], dtype=np.int32)
    for h in range(values.shape[0]):
        dist = -2.0 * (values[h] @ centers[h].T).astype(F32) + (centers[h] * centers[h]).sum(axis=1, dtype=F32)[None, :]
        labels[h] = dist.argmin(axis=1)
    return labels


def kmeans_permutation(v, clusters=64, iterations=4):
    """v float32 [S,H,128] (BF16 values) -> (permutation int64 [H,S], centers f32 [H,K,128], labels)."""
    s, h, d = v.shape
    vh = np.ascontiguousarray(v.transpose(1, 0, 2))
    idx = np.linspace(0, s - 1, clusters).astype(np.int64)  # torch.linspace(...).long() truncates
    centers = vh[:, idx].copy()
    for _ in range(iterations):
        labels = assign(vh, centers)
        new = centers.copy()
        for head in range(h):
            sums = np.zeros((clusters, d), dtype=F32)
            np.add.at(sums, labels[head], vh[head])
            counts = np.bincount(labels[head], minlength=clusters).astype(F32)
            filled = counts > 0
            new[head][filled] = _bf16(sums[filled] / counts[filled, None])
        centers = new
    labels = assign(vh, centers)
    permutation = np.argsort(labels, axis=1, kind="stable").astype(np.int64)
    return permutation, centers, labels


def block_sum(rows):
    """Float32 sum over the rows of one block in the fixed order of the CUDA kernel: rows g + 16 i are added in
    ascending i into sixteen partial sums, which are then added in ascending g (missing rows count as 0)."""
    padded = np.zeros((BLOCK, rows.shape[1]), dtype=F32)
    padded[: rows.shape[0]] = rows
    lanes = padded.reshape(8, 16, -1)
    partial = lanes[0].copy()
    for i in range(1, 8):
        partial = (partial + lanes[i]).astype(F32)
    total = partial[0].copy()
    for g in range(1, 16):
        total = (total + partial[g]).astype(F32)
    return total


def apply_v_smooth(q, k, v, permutation, arith=GPU, block_means=None):
    """Permute K/V by group, demean V per 128-token block, quantise.  q,k,v float32 [S,H,128] (BF16 values),
    permutation int [H,S].  Returns dict(q, k, v codes uint8 [S,H,128], means f32 [blocks,H,128] (BF16-rounded,
    in code units), scale f32 [H,128], block_means f32 [H,blocks,128], amax f32 [H,128]).  ``arith`` evaluates the
    divisions as the reference's GPU code does (oracle/prep.py); ``block_means`` (f32 [H,blocks,128]) replaces the
    block means computed here, whose float32 summation order the reference leaves to its compiler."""
    s, h, d = v.shape
    blocks = (s + BLOCK - 1) // BLOCK
    k8 = np.zeros((s, h, d), dtype=np.uint8)
    v8 = np.zeros((s, h, d), dtype=np.uint8)
    means_out = np.zeros((blocks, h, d), dtype=F32)
    scale_out = np.zeros((h, d), dtype=F32)
    all_means = np.zeros((h, blocks, d), dtype=F32)
    all_amax = np.zeros((h, d), dtype=F32)
    for head in range(h):
        vp = v[permutation[head], head]  # [S,128] in group order
        kp = k[permutation[head], head]
        means = np.zeros((blocks, d), dtype=F32)
        amax = np.zeros(d, dtype=F32)
        for b in range(blocks):
            rows = vp[b * BLOCK : (b + 1) * BLOCK]
            if block_means is not None:
                means[b] = block_means[head, b]
            else:
                total = block_sum(rows)
                means[b] = arith.div(total, np.full_like(total, F32(rows.shape[0])))
            amax = np.maximum(amax, np.abs((rows - means[b][None, :]).astype(F32)).max(axis=0))
        positive = np.where(amax > 0, amax, F32(448.0)).astype(F32)
        scale = np.where(amax > 0, arith.div(positive, np.full_like(positive, F32(448.0))), F32(1.0)).astype(F32)
        all_means[head], all_amax[head] = means, amax
        for b in range(blocks):
            rows = vp[b * BLOCK : (b + 1) * BLOCK]
            residual = (rows - means[b][None, :]).astype(F32)
            codes = np.clip(arith.div(residual, np.broadcast_to(scale[None, :], residual.shape)), -448.0, 448.0)
            v8[b * BLOCK : b * BLOCK + rows.shape[0], head] = e4m3_encode(codes)
            means_out[b, head] = _bf16(arith.div(means[b], scale))
        k8[:, head] = e4m3_encode(np.clip(kp, -448.0, 448.0))
        scale_out[head] = scale
    q8 = e4m3_encode(np.clip(q, -448.0, 448.0))
    return dict(q=q8, k=k8, v=v8, means=means_out, scale=scale_out, block_means=all_means, amax=all_amax)
