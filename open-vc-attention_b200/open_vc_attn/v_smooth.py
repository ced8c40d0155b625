"""V-Smooth preparation for the VC-Attention baseline.

Host-side mirror of src/open_vc_attn/_kernels/blackwell/v_smooth.py of the reference: the same
functions, arguments, dataclass fields and error messages; the device work is done by the
ovc_vs_* entry points of libovc.so instead of Triton kernels and torch expressions.

Built: one sequence ([S,H,128] or [1,S,H,128]), sequence-major K/V.  ``head_major_kv=True`` and
batches of several sequences raise NotImplementedError.
"""

from dataclasses import dataclass

import torch

from . import _lib


@dataclass(frozen=True)
class PreparedVSmooth:
    q: torch.Tensor
    k: torch.Tensor
    v: torch.Tensor
    means: torch.Tensor
    scale: torch.Tensor
    permutation: torch.Tensor
    centroids: torch.Tensor | None

    def forward_kwargs(self):
        return dict(v_smooth=True, v_smooth_means=self.means, v_smooth_scale=self.scale)


def prefer_head_major_v_smooth(q, *, expcast=False, mid_window_blocks=4):
    """The head-major K/V layout of the reference (v_smooth.py:182-196) is not built: never preferred."""
    return False


def _cast_fp8(x):
    out = torch.empty(x.shape, dtype=torch.float8_e4m3fn, device=x.device)
    _lib.check(
        _lib.load().ovc_cast_e4m3(x.data_ptr(), _lib.dtype_code(x.dtype), out.data_ptr(), x.numel(),
                                  _lib.stream_pointer(x.device)),
        "ovc_cast_e4m3",
    )
    return out


@torch.no_grad()
def apply_v_smooth(q, k, v, permutation):
    """Permute K/V by an existing grouping, demean V per 128-token block and quantise (two passes).

    q, k, v: BF16 [S,H,128]; permutation: int64 [1,H,S].  Returns a PreparedVSmooth with float32 means
    (v_smooth.py:136-164 of the reference).
    """
    length, heads, dim = v.shape
    if dim != 128 or q.shape != v.shape or k.shape != v.shape:
        raise ValueError("Fused V-Smooth expects matching [S,H,128] self-attention inputs")
    q, k, v = q.contiguous(), k.contiguous(), v.contiguous()
    blocks = (length + 127) // 128
    perm = permutation.reshape(heads, length).contiguous()
    lib = _lib.load()
    device = v.device
    with torch.cuda.device(device):
        stream = _lib.stream_pointer(device)
        means = torch.empty((heads, blocks, dim), device=device, dtype=torch.float32)
        amax = torch.empty((heads, dim), device=device, dtype=torch.float32)
        _lib.check(
            lib.ovc_vs_block_stats(v.data_ptr(), perm.data_ptr(), means.data_ptr(), amax.data_ptr(), length, heads, stream),
            "ovc_vs_block_stats",
        )
        k_out = torch.empty(k.shape, device=device, dtype=torch.float8_e4m3fn)
        codes = torch.empty(v.shape, device=device, dtype=torch.float8_e4m3fn)
        means_out = torch.empty((1, blocks, heads, dim), device=device, dtype=torch.float32)
        scale = torch.empty((1, heads, dim), device=device, dtype=torch.float32)
        _lib.check(
            lib.ovc_vs_block_write(k.data_ptr(), v.data_ptr(), perm.data_ptr(), means.data_ptr(), amax.data_ptr(),
                                   k_out.data_ptr(), codes.data_ptr(), means_out.data_ptr(), scale.data_ptr(),
                                   length, heads, stream),
            "ovc_vs_block_write",
        )
        q8 = _cast_fp8(q)
    return PreparedVSmooth(q8, k_out, codes, means_out, scale, permutation, None)


@torch.no_grad()
def group_values(v, *, clusters=64, iterations=4, centroids=None):
    """Lloyd iterations on the V tokens of each head; returns (permutation int64 [1,H,S], centres bf16 [1,H,K,128]).

    v BF16 [S,H,128], read in place.  v_smooth.py:245-313 of the reference.
    """
    length, heads, dim = v.shape
    device = v.device
    lib = _lib.load()
    with torch.cuda.device(device):
        stream = _lib.stream_pointer(device)
        if centroids is None:
            indices = torch.linspace(0, length - 1, clusters, device=device).long()
            centers = v[indices].permute(1, 0, 2).contiguous()
        else:
            centers = centroids.reshape(heads, clusters, dim).contiguous().clone()
        labels = torch.empty((heads, length), device=device, dtype=torch.int32)
        sums = torch.empty((heads, clusters, dim), device=device, dtype=torch.float32)
        counts = torch.empty((heads, clusters), device=device, dtype=torch.float32)

        def assign():
            _lib.check(
                lib.ovc_vs_assign(v.data_ptr(), centers.data_ptr(), labels.data_ptr(), length, heads, clusters, stream),
                "ovc_vs_assign",
            )

        for _ in range(iterations):
            assign()
            _lib.check(
                lib.ovc_vs_accumulate(v.data_ptr(), labels.data_ptr(), sums.data_ptr(), counts.data_ptr(), length,
                                      heads, clusters, stream),
                "ovc_vs_accumulate",
            )
            _lib.check(
                lib.ovc_vs_update_centers(sums.data_ptr(), counts.data_ptr(), centers.data_ptr(), heads, clusters, stream),
                "ovc_vs_update_centers",
            )
        assign()
        permutation = torch.argsort(labels, dim=-1, stable=True).reshape(1, heads, length)
    return permutation, centers.reshape(1, heads, clusters, dim)


@torch.no_grad()
def prepare_v_smooth(
    q,
    k,
    v,
    *,
    clusters=64,
    iterations=4,
    permutation=None,
    centroids=None,
    expand_means=False,
    head_major_kv=False,
    check_permutation=True,
):
    """Group V tokens (or reuse a grouping), permute K/V, demean V per block and quantise.

    Same contract as prepare_v_smooth of the reference (v_smooth.py:199-381) for one sequence:
    means are BF16 in residual-code units (float32 copies of the same values with expand_means),
    scales FP32 per head and channel; K/V share the per-head permutation, Q keeps its order.
    """
    if q.ndim not in (3, 4) or q.shape != k.shape or q.shape != v.shape or q.shape[-1] != 128:
        raise ValueError("V-Smooth expects equal self-attention Q/K/V shapes ending in D=128")
    if any(x.dtype != torch.bfloat16 or x.device != q.device or not x.is_cuda for x in (q, k, v)):
        raise ValueError("V-Smooth preprocessing requires BF16 Q/K/V on one CUDA device")
    squeeze = q.ndim == 3
    qb, kb, vb = (x.unsqueeze(0) if squeeze else x for x in (q, k, v))
    batch, length, heads, dim = qb.shape
    if length == 0 or not 1 <= clusters <= min(128, length) or iterations < 1:
        raise ValueError("Require nonempty tokens, 1 <= clusters <= min(128,S), iterations >= 1")
    if batch != 1:
        raise NotImplementedError("V-Smooth preparation is built for one sequence per call")
    if head_major_kv:
        raise NotImplementedError("The head-major K/V layout is not built")
    centers = None
    if permutation is None:
        if centroids is not None and (
            centroids.shape != (batch, heads, clusters, dim)
            or centroids.dtype != torch.bfloat16
            or centroids.device != q.device
        ):
            raise ValueError("centroids must be BF16 [B,H,clusters,128] on the input device")
        permutation, centers = group_values(vb[0].contiguous(), clusters=clusters, iterations=iterations, centroids=centroids)
    else:
        if centroids is not None:
            raise ValueError("Pass a permutation or centroids, not both")
        if (
            permutation.shape != (batch, heads, length)
            or permutation.dtype != torch.int64
            or permutation.device != q.device
        ):
            raise ValueError("permutation must be int64 [B,H,S] on the input device")
        expected = torch.arange(length, device=q.device).expand(batch, heads, length)
        if check_permutation and not torch.equal(permutation.sort(dim=-1).values, expected):
            raise ValueError("Each head permutation must contain every token exactly once")
    fused = apply_v_smooth(qb[0], kb[0], vb[0], permutation)
    means = fused.means if expand_means else fused.means.to(torch.bfloat16)
    if squeeze:
        return PreparedVSmooth(fused.q, fused.k, fused.v, means, fused.scale, permutation, centers)
    return PreparedVSmooth(fused.q[None], fused.k[None], fused.v[None], means, fused.scale, permutation, centers)
