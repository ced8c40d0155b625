"""The V-Smooth restatement on the CPU: the prepared tensors reconstruct V, and ExpCast attention with
mean restoration stays within the reference's 10 % bound of exact attention."""

import numpy as np

from oracle import attention as oatt
from oracle import vsmooth as ovs
from oracle.fp8 import e4m3_decode


def _inputs(s, h, seed):
    rng = np.random.default_rng(seed)
    group = rng.integers(0, 6, size=s)
    offsets = rng.normal(0, 2.0, size=(6, h, 128)).astype(np.float32)
    q = ovs._bf16(rng.normal(0, 1, (s, h, 128)).astype(np.float32))
    k = ovs._bf16(rng.normal(0, 1, (s, h, 128)).astype(np.float32))
    v = ovs._bf16((rng.normal(0, 0.3, (s, h, 128)) + offsets[group]).astype(np.float32))
    return q, k, v


def test_grouping_is_a_permutation_sorted_by_label():
    _, _, v = _inputs(700, 2, 1)
    permutation, centers, labels = ovs.kmeans_permutation(v, clusters=8, iterations=3)
    assert centers.shape == (2, 8, 128)
    for head in range(2):
        assert np.array_equal(np.sort(permutation[head]), np.arange(700))
        assert (np.diff(labels[head][permutation[head]]) >= 0).all()


def test_prepared_tensors_reconstruct_v_and_attention_stays_close():
    s, h = 300, 2
    q, k, v = _inputs(s, h, 2)
    permutation, _, _ = ovs.kmeans_permutation(v, clusters=8, iterations=3)
    prepared = ovs.apply_v_smooth(q, k, v, permutation)
    blocks = (s + 127) // 128
    assert prepared["means"].shape == (blocks, h, 128) and prepared["scale"].shape == (h, 128)
    for head in range(h):
        block_of_row = np.arange(s) // 128
        rebuilt = (e4m3_decode(prepared["v"][:, head]) + prepared["means"][block_of_row, head]) * prepared["scale"][head]
        want = v[permutation[head], head]
        assert np.abs(rebuilt - want).max() <= 0.07 * np.abs(want).max()
        assert np.array_equal(e4m3_decode(prepared["k"][:, head]), e4m3_decode(ovs.e4m3_encode(k[permutation[head], head])))
    ones = np.ones((h, blocks), dtype=np.float32)
    out = oatt.expcast_attention(
        prepared["q"], prepared["k"], prepared["v"], ones, ones, np.ones(h, dtype=np.float32), mid_window_blocks=None,
        v_smooth_means=prepared["means"], v_channel_scale=prepared["scale"],
    )
    assert oatt.relative_l2(out, oatt.exact_attention(q, k, v)) < 0.10


def test_log_sum_exp_of_the_restatement_tracks_the_exact_value():
    from oracle import prep as oprep

    rng = np.random.default_rng(3)
    q, k, v = [rng.normal(size=(200, 2, 128)).astype(np.float32) for _ in range(3)]
    pq, pk, pv = oprep.quantize_per_block(q[None]), oprep.quantize_per_block(k[None]), oprep.quantize_per_head(v[None])
    out, lse = oatt.expcast_attention(pq[0][0], pk[0][0], pv[0][0], pq[1][0], pk[1][0], pv[1][0], return_lse=True)
    assert lse.shape == (2, 200) and lse.dtype == np.float32
    scores = np.einsum("qhd,khd->hqk", q.astype(np.float64), k.astype(np.float64)) / np.sqrt(128.0)
    exact = np.log(np.exp(scores - scores.max(axis=-1, keepdims=True)).sum(axis=-1)) + scores.max(axis=-1)
    assert np.abs(lse - exact).max() < 0.1
