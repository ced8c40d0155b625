"""VC-Attention baseline on the GPU: V-Smooth preparation bit-exact against the CPU oracle for a replayed
grouping, the grouping kernels against their restatement, and the mean-restoring attention kernel within
0.5 % rel-L2 of the oracle and 10 % of exact attention (the bound of tests/gpu/test_attention.py:110-126 of
the reference, whose shapes and seeds the first test reuses)."""

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from oracle import vsmooth as ovs

pytestmark = pytest.mark.gpu

from gpu_util import DEV, f32, hw_arith, structured_qkv, u8  # noqa: E402

ORACLE_TOL = 5e-3


def _modules():
    from open_vc_attn import _lib, baselines, forward, v_smooth

    return _lib, baselines, forward, v_smooth


def _oracle_vc(prepared, rows=None):
    """Oracle attention from the device's prepared tensors (so only the attention kernel is compared)."""
    q8, k8, v8 = u8(prepared.q), u8(prepared.k), u8(prepared.v)
    s, h, _ = q8.shape
    blocks = (s + 127) // 128
    ones = np.ones((h, blocks), dtype=np.float32)
    return oatt.expcast_attention(
        q8, k8, v8, ones, ones, np.ones(h, dtype=np.float32), mid_window_blocks=None, rows=rows,
        v_smooth_means=f32(prepared.means).reshape(blocks, h, 128), v_channel_scale=f32(prepared.scale).reshape(h, 128),
    )


@pytest.mark.parametrize("s", [129, 1024])
def test_vc_baseline_against_exact_attention_and_oracle(s):
    _, baselines, forward, _ = _modules()
    torch.manual_seed(900 + s)
    q, k, v = [torch.randn(s, 2, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    out = baselines.vc_attention(q, k, v)
    forward.check_status(q.device)
    assert out.shape == q.shape and out.dtype == torch.bfloat16 and torch.isfinite(out).all()
    assert oatt.relative_l2(f32(out), oatt.exact_attention(f32(q), f32(k), f32(v))) < 0.10
    grouped = baselines.prepare_vc(q, k, v)
    reused = baselines.prepare_vc(q, k, v, permutation=grouped.permutation, check_permutation=False)
    first = baselines.attention_vc(grouped, output_shape=q.shape)
    assert torch.equal(first, baselines.attention_vc(reused, output_shape=q.shape))
    assert oatt.relative_l2(f32(first), _oracle_vc(grouped)) < ORACLE_TOL


@pytest.mark.parametrize("s,h,clusters", [(1, 1, 1), (127, 2, 8), (300, 3, 64), (2048, 2, 64), (1500, 2, 128)])
def test_preparation_is_bit_exact_for_a_replayed_grouping(s, h, clusters):
    _, baselines, _, v_smooth = _modules()
    q, k, v = structured_qkv(s, h, seed=31 + s)
    prepared = baselines.prepare_vc(q, k, v, clusters=clusters, iterations=3)
    perm = prepared.permutation.cpu().numpy().reshape(h, s)
    assert all(np.array_equal(np.sort(perm[i]), np.arange(s)) for i in range(h))
    want = ovs.apply_v_smooth(f32(q), f32(k), f32(v), perm, arith=hw_arith())
    assert np.array_equal(u8(prepared.q), want["q"])
    assert np.array_equal(u8(prepared.k), want["k"])
    assert np.array_equal(u8(prepared.v), want["v"])
    assert prepared.means.dtype == torch.float32 and tuple(prepared.means.shape) == (1, (s + 127) // 128, h, 128)
    assert np.array_equal(f32(prepared.means)[0], want["means"])
    assert np.array_equal(f32(prepared.scale)[0], want["scale"])
    # BF16 means (expand_means=False) hold the same values.
    plain = v_smooth.prepare_v_smooth(q, k, v, clusters=clusters, permutation=prepared.permutation)
    assert plain.means.dtype == torch.bfloat16 and torch.equal(plain.means.float(), prepared.means)
    assert torch.equal(plain.v.view(torch.uint8), prepared.v.view(torch.uint8))


def test_grouping_kernels_match_their_restatement():
    lib_mod, _, _, v_smooth = _modules()
    s, h, clusters = 3000, 3, 64
    _, _, v = structured_qkv(s, h, seed=5)
    lib = lib_mod.load()
    stream = lib_mod.stream_pointer(v.device)
    index = torch.linspace(0, s - 1, clusters, device=DEV).long()
    centers = v[index].permute(1, 0, 2).contiguous()
    labels = torch.empty((h, s), dtype=torch.int32, device=DEV)
    lib_mod.check(lib.ovc_vs_assign(v.data_ptr(), centers.data_ptr(), labels.data_ptr(), s, h, clusters, stream), "assign")
    vh = np.ascontiguousarray(f32(v).transpose(1, 0, 2))
    want = ovs.assign(vh, f32(centers))
    got = labels.cpu().numpy()
    differ = got != want
    assert differ.mean() < 1e-3
    # Where the labels differ the two centres are (nearly) equidistant.
    for head, token in zip(*np.nonzero(differ)):
        c = f32(centers)[head].astype(np.float64)
        d = ((vh[head, token].astype(np.float64)[None, :] - c) ** 2).sum(axis=1)
        assert abs(d[got[head, token]] - d[want[head, token]]) <= 1e-4 * max(d[want[head, token]], 1e-6)

    sums = torch.full((h, clusters, 128), 7.0, device=DEV)  # the entry point clears its outputs
    counts = torch.full((h, clusters), 7.0, device=DEV)
    lib_mod.check(
        lib.ovc_vs_accumulate(v.data_ptr(), labels.data_ptr(), sums.data_ptr(), counts.data_ptr(), s, h, clusters, stream),
        "accumulate",
    )
    want_sums = np.zeros((h, clusters, 128), dtype=np.float64)
    want_counts = np.zeros((h, clusters), dtype=np.float32)
    for head in range(h):
        np.add.at(want_sums[head], got[head], vh[head].astype(np.float64))
        want_counts[head] = np.bincount(got[head], minlength=clusters)
    assert np.array_equal(f32(counts), want_counts)
    assert np.allclose(f32(sums), want_sums, rtol=1e-5, atol=1e-4)

    before = centers.clone()
    lib_mod.check(lib.ovc_vs_update_centers(sums.data_ptr(), counts.data_ptr(), centers.data_ptr(), h, clusters, stream), "update")
    filled = want_counts > 0
    quotient = (f32(sums) / np.maximum(f32(counts), 1)[..., None]).astype(np.float32)
    want_centers = np.where(filled[..., None], ovs._bf16(quotient), f32(before))
    assert np.array_equal(f32(centers), want_centers)

    # The whole grouping: a valid permutation that sorts the final labels, deterministic when replayed.
    permutation, final = v_smooth.group_values(v, clusters=clusters, iterations=4)
    perm = permutation.cpu().numpy().reshape(h, s)
    assert all(np.array_equal(np.sort(perm[i]), np.arange(s)) for i in range(h))
    lib_mod.check(lib.ovc_vs_assign(v.data_ptr(), final.data_ptr(), labels.data_ptr(), s, h, clusters, stream), "assign")
    sorted_labels = np.take_along_axis(labels.cpu().numpy(), perm, axis=1)
    assert (np.diff(sorted_labels, axis=1) >= 0).all()


def test_demeaning_helps_on_values_with_block_structure():
    """On inputs whose V has a strong per-token-group offset the baseline is closer to exact attention than
    its 10 % bound by a wide margin, and the attention kernel tracks the oracle on sampled query blocks."""
    _, baselines, forward, _ = _modules()
    s, h = 4096, 2
    q, k, v = structured_qkv(s, h, seed=77)
    prepared = baselines.prepare_vc(q, k, v)
    out = baselines.attention_vc(prepared, output_shape=q.shape)
    forward.check_status(q.device)
    exact = oatt.exact_attention(f32(q), f32(k), f32(v))
    assert oatt.relative_l2(f32(out), exact) < 0.035
    m_blocks = [0, 7, 15]
    want = _oracle_vc(prepared, rows=m_blocks)
    rows = np.concatenate([np.arange(256 * m, 256 * m + 256) for m in m_blocks])
    assert oatt.relative_l2(f32(out)[rows], want[rows]) < ORACLE_TOL


@pytest.mark.parametrize("s,h,window", [(255, 1, None), (257, 2, 4), (1500, 2, 0), (1500, 3, None)])
def test_tails_and_scan_orders(s, h, window):
    _, baselines, forward, _ = _modules()
    from open_vc_attn.api import raw_forward

    q, k, v = structured_qkv(s, h, seed=s + h)
    prepared = baselines.prepare_vc(q, k, v, clusters=16, iterations=2)
    out, _ = raw_forward(prepared.q, prepared.k, prepared.v, expcast=True, mid_window_blocks=window,
                         **prepared.forward_kwargs())
    forward.check_status(q.device)
    q8, k8, v8 = u8(prepared.q), u8(prepared.k), u8(prepared.v)
    blocks = (s + 127) // 128
    ones = np.ones((h, blocks), dtype=np.float32)
    want = oatt.expcast_attention(
        q8, k8, v8, ones, ones, np.ones(h, dtype=np.float32), mid_window_blocks=window,
        v_smooth_means=f32(prepared.means).reshape(blocks, h, 128), v_channel_scale=f32(prepared.scale).reshape(h, 128),
    )
    assert oatt.relative_l2(f32(out), want) < ORACLE_TOL


@pytest.mark.parametrize("s,h,window,exact_bf16_means", [(9000, 1, None, True), (9000, 2, 4, True), (4500, 1, 20, False),
                                                         (6200, 1, None, False)])
def test_long_scans_restore_means_on_the_tensor_core(s, h, window, exact_bf16_means):
    """More than 16 key blocks: the masses of complete slices of sixteen blocks meet their means in BF16 tensor-core
    products (several tiles of means, both scan orders); means that are not BF16 values keep 16 bits."""
    _, baselines, forward, _ = _modules()
    from open_vc_attn.api import raw_forward

    q, k, v = structured_qkv(s, h, seed=3 * s + h)
    prepared = baselines.prepare_vc(q, k, v, clusters=32, iterations=2)
    kwargs = prepared.forward_kwargs()
    means = prepared.means
    if not exact_bf16_means:
        means = means * 1.00173
        kwargs = {key: (means if value is prepared.means else value) for key, value in kwargs.items()}
        assert any(value is means for value in kwargs.values())
    out, _ = raw_forward(prepared.q, prepared.k, prepared.v, expcast=True, mid_window_blocks=window, **kwargs)
    forward.check_status(q.device)
    blocks = (s + 127) // 128
    m_blocks = [0, (blocks // 2) // 2, (blocks - 1) // 2]
    ones = np.ones((h, blocks), dtype=np.float32)
    want = oatt.expcast_attention(
        u8(prepared.q), u8(prepared.k), u8(prepared.v), ones, ones, np.ones(h, dtype=np.float32), mid_window_blocks=window,
        rows=m_blocks, v_smooth_means=f32(means).reshape(blocks, h, 128), v_channel_scale=f32(prepared.scale).reshape(h, 128),
    )
    rows = np.concatenate([np.arange(256 * m, min(256 * m + 256, s)) for m in m_blocks])
    error = oatt.relative_l2(f32(out)[rows], want[rows])
    print(f"S={s} H={h} window={window}: rel-L2 vs oracle {error:.2e}")
    assert error < ORACLE_TOL


@pytest.mark.parametrize("blocks", [17, 32, 33, 34, 49, 64, 65, 66, 97, 129])
def test_every_scan_order_completes(blocks):
    """The means tiles (32 key blocks each) are loaded, read and released through barriers of their own; which
    group follows which depends on the length and on the window (a group of a single block at the turn of the
    mid-window order once made the loader wait for a step that needed the loader).  Every combination must finish
    without an expired wait, and the cases that used to stall must match the oracle."""
    _, baselines, forward, _ = _modules()
    from open_vc_attn.api import raw_forward

    s = 128 * (blocks - 1) + 113
    q, k, v = structured_qkv(s, 1, seed=blocks)
    prepared = baselines.prepare_vc(q, k, v, clusters=16, iterations=1)
    for window in (None, 0, 1, 4, 17, 40):
        out, _ = raw_forward(prepared.q, prepared.k, prepared.v, expcast=True, mid_window_blocks=window,
                             **prepared.forward_kwargs())
        forward.check_status(q.device)
        assert torch.isfinite(out).all(), (blocks, window)


@pytest.mark.parametrize("s,h,window", [(4209, 2, 4), (12379, 1, 17)])
def test_single_block_group_at_the_turn_of_the_scan(s, h, window):
    _, baselines, forward, _ = _modules()
    from open_vc_attn.api import raw_forward

    q, k, v = structured_qkv(s, h, seed=s)
    prepared = baselines.prepare_vc(q, k, v, clusters=32, iterations=1)
    out, _ = raw_forward(prepared.q, prepared.k, prepared.v, expcast=True, mid_window_blocks=window,
                         **prepared.forward_kwargs())
    forward.check_status(q.device)
    blocks = (s + 127) // 128
    m_blocks = [0, 3, (blocks - 1) // 2]
    ones = np.ones((h, blocks), dtype=np.float32)
    want = oatt.expcast_attention(
        u8(prepared.q), u8(prepared.k), u8(prepared.v), ones, ones, np.ones(h, dtype=np.float32), mid_window_blocks=window,
        rows=m_blocks, v_smooth_means=f32(prepared.means).reshape(blocks, h, 128),
        v_channel_scale=f32(prepared.scale).reshape(h, 128),
    )
    rows = np.concatenate([np.arange(256 * m, min(256 * m + 256, s)) for m in m_blocks])
    assert oatt.relative_l2(f32(out)[rows], want[rows]) < ORACLE_TOL


def test_headline_length_against_the_oracle():
    """S = 73397 (574 key blocks, 18 tiles of means through the two buffers), both scan orders, sampled query blocks."""
    _, baselines, forward, _ = _modules()
    from open_vc_attn.api import raw_forward

    s, h = 73397, 2
    q, k, v = structured_qkv(s, h, seed=99)
    prepared = baselines.prepare_vc(q, k, v, clusters=64, iterations=1)
    blocks = (s + 127) // 128
    ones = np.ones((h, blocks), dtype=np.float32)
    for window, m_blocks in ((None, [0, 286]), (4, [143])):
        out, _ = raw_forward(prepared.q, prepared.k, prepared.v, expcast=True, mid_window_blocks=window,
                             **prepared.forward_kwargs())
        forward.check_status(q.device)
        want = oatt.expcast_attention(
            u8(prepared.q), u8(prepared.k), u8(prepared.v), ones, ones, np.ones(h, dtype=np.float32),
            mid_window_blocks=window, rows=m_blocks, v_smooth_means=f32(prepared.means).reshape(blocks, h, 128),
            v_channel_scale=f32(prepared.scale).reshape(h, 128),
        )
        rows = np.concatenate([np.arange(256 * m, min(256 * m + 256, s)) for m in m_blocks])
        error = oatt.relative_l2(f32(out)[rows], want[rows])
        print(f"window={window}: rel-L2 vs oracle {error:.2e}")
        assert error < ORACLE_TOL


def test_reuse_path_is_graph_capturable():
    # tests/gpu/test_attention.py:128-150 of the reference
    _, baselines, _, _ = _modules()
    torch.manual_seed(77)
    q, k, v = [torch.randn(1024, 2, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    grouped = baselines.prepare_vc(q, k, v)

    def call():
        prepared = baselines.prepare_vc(q, k, v, permutation=grouped.permutation, check_permutation=False)
        return baselines.attention_vc(prepared, output_shape=q.shape)

    eager = call().clone()
    stream = torch.cuda.Stream()
    stream.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(stream):
        call()
    torch.cuda.current_stream().wait_stream(stream)
    graph = torch.cuda.CUDAGraph()
    with torch.cuda.graph(graph):
        out = call()
    graph.replay()
    torch.cuda.synchronize()
    assert torch.equal(out, eager)


def test_argument_errors():
    _, baselines, _, v_smooth = _modules()
    q = torch.randn(256, 2, 128, device=DEV, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="matching BF16"):
        baselines.prepare_vc(q.half(), q.half(), q.half())
    with pytest.raises(ValueError, match="one sequence"):
        baselines.prepare_vc(q[None].repeat(2, 1, 1, 1), q[None].repeat(2, 1, 1, 1), q[None].repeat(2, 1, 1, 1))
    with pytest.raises(ValueError, match="clusters"):
        v_smooth.prepare_v_smooth(q, q, q, clusters=129)
    with pytest.raises(ValueError, match="every token exactly once"):
        v_smooth.prepare_v_smooth(q, q, q, permutation=torch.zeros((1, 2, 256), dtype=torch.int64, device=DEV))
    with pytest.raises(ValueError, match="not both"):
        v_smooth.prepare_v_smooth(
            q, q, q, permutation=torch.arange(256, device=DEV).expand(1, 2, 256).contiguous(),
            centroids=torch.zeros((1, 2, 64, 128), dtype=torch.bfloat16, device=DEV),
        )
