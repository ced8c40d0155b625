"""V residual repair on the GPU (tests/gpu/test_v_repair.py of the reference, plus the oracle)."""

import dataclasses

import numpy as np
import pytest
import torch

from oracle import attention as oatt
from oracle import prep as oprep

pytestmark = pytest.mark.gpu

from gpu_util import DEV, f32, hw_arith, oracle_rows, packed_buffer, u8  # noqa: E402


def _mods():
    import open_vc_attn
    from open_vc_attn import api, forward, v_repair

    return open_vc_attn, api, forward, v_repair


def student_t_v(s, h, seed):
    g = torch.Generator(device="cpu").manual_seed(seed)
    normal = torch.randn(s, h, 128, generator=g)
    chi2 = torch.randn(3, s, h, 128, generator=g).pow(2).sum(0)
    return (normal / torch.sqrt(chi2 / 3)).to(DEV).to(torch.bfloat16)


def test_budget_zero_is_plain_attention():
    ovc, api, forward, v_repair = _mods()
    torch.manual_seed(1)
    q, k, v = [torch.randn(32768, 2, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    prepared = ovc.prepare_v_repair(q, k, v, budget=0.0)
    assert prepared.repair_tokens == 0 and prepared.selected_tokens == 0 and prepared.repair_k_descale is None
    assert torch.equal(ovc.attention_v_repair(prepared), ovc.attention(q, k, v))


@pytest.mark.parametrize("window", [None, 4])
def test_zeroed_repair_rows_equal_the_base_output(window):
    """Repair rows with zero V add nothing to the numerator and are left out of the denominator."""
    ovc, api, forward, v_repair = _mods()
    torch.manual_seed(2)
    s, h = 32769, 2
    q, k = [torch.randn(s, h, 128, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    v = student_t_v(s, h, 5)
    prepared = ovc.prepare_v_repair(q, k, v, budget=0.005)
    assert (prepared.selected_tokens, prepared.repair_tokens) == (164, 256)
    assert prepared.k.shape[0] == s + 256 and prepared.k_descale.shape[-1] == (s + 127) // 128 + 2
    base = ovc.attention(q, k, v, mid_window_blocks=window)
    padded = (s + 256 + 127) // 128 * 128
    buffer = torch.empty(0, dtype=torch.uint8, device=DEV).set_(prepared.v.untyped_storage(), 0, (h, 128, padded))
    buffer[:, :, :256] = 0
    out = ovc.attention_v_repair(prepared, mid_window_blocks=window)
    forward.check_status(q.device)
    assert torch.equal(out, base)


def test_repair_matches_oracle_and_reduces_the_error():
    ovc, api, forward, v_repair = _mods()
    torch.manual_seed(3)
    s, h = 32769, 2
    q, k = [torch.randn(s, h, 128, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    v = student_t_v(s, h, 7)
    prepared = ovc.prepare_v_repair(q, k, v, budget=0.02)
    out = ovc.attention_v_repair(prepared)
    forward.check_status(q.device)
    plain = ovc.attention(q, k, v)
    rows, selected = prepared.repair_tokens, prepared.selected_tokens
    assert selected == round(0.02 * s) and rows == -(-selected // 128) * 128
    vf = f32(v)
    # the oracle consumes the device-prepared tensors, so the device's own top-k choice is replayed
    m_blocks = (s + 255) // 256
    o_rows, expect = oracle_rows(prepared, [0, m_blocks // 2], [1], repair_kd=prepared.repair_k_descale)
    assert oatt.relative_l2(f32(out[:, 1])[o_rows], expect[:, 0]) < 5e-3
    pick = o_rows[::16]
    exact = oatt.exact_attention(f32(q[pick][:, 1:2]), f32(k[:, 1:2]), vf[:, 1:2])
    err_repair = oatt.relative_l2(f32(out[pick][:, 1:2]), exact)
    err_plain = oatt.relative_l2(f32(plain[pick][:, 1:2]), exact)
    assert err_repair < err_plain
    assert torch.equal(ovc.attention_v_repair(ovc.prepare_v_repair(q[None], k[None], v[None], budget=0.02))[0], out)


def test_repair_prefix_contents_against_the_oracle():
    """Replay the device's token selection (read back from the prefix keys' descales and codes) in the
    oracle and compare every prepared tensor byte for byte."""
    ovc, api, forward, v_repair = _mods()
    torch.manual_seed(11)
    s, h = 1000, 2
    q, k = [torch.randn(s, h, 128, device=DEV, dtype=torch.bfloat16) for _ in range(2)]
    v = student_t_v(s, h, 13)
    prepared = v_repair._prepare(q, k, v, 0.03)
    selected, rows = prepared.selected_tokens, prepared.repair_tokens
    assert (selected, rows) == (30, 128)
    vf, kf, qf = f32(v), f32(k), f32(q)
    arith = hw_arith()
    oc, od = oprep.quantize_per_head(vf[None], arith)
    score = oprep.v_residual_score(vf, oc[0], od[0], arith)
    k8 = u8(prepared.k)
    index = np.zeros((h, selected), dtype=np.int64)
    for head in range(h):
        top = set(np.argsort(-score[head], kind="stable")[:selected].tolist())
        for r in range(selected):
            matches = [t for t in top if np.array_equal(k8[rows + t, head], k8[r, head])]
            assert matches, "repair key is not one of the top-scoring tokens"
            index[head, r] = matches[0]
        assert len(set(index[head].tolist())) == selected
    o = oprep.prepare_repair(qf, kf, vf, budget=0.03, index=index, arith=arith)
    assert np.array_equal(u8(prepared.q), o["q"])
    assert np.array_equal(k8, o["k"])
    assert np.array_equal(packed_buffer(prepared.v), o["v_packed"])
    assert np.array_equal(f32(prepared.q_descale), o["q_descale"])
    assert np.array_equal(f32(prepared.k_descale), o["k_descale"])
    assert np.array_equal(f32(prepared.v_descale), o["v_descale"])
    assert np.array_equal(f32(prepared.repair_k_descale), o["repair_k_descale"])
    out = ovc.attention_v_repair(prepared)
    forward.check_status(q.device)
    v_all = o["v_packed"][:, :, : o["total"]].transpose(2, 0, 1)
    expect = oatt.expcast_attention(o["q"], o["k"], np.ascontiguousarray(v_all), o["q_descale"][0], o["k_descale"][0],
                                    o["v_descale"][0], repair_k_descale=o["repair_k_descale"][0])
    assert oatt.relative_l2(f32(out), expect) < 5e-3


def test_repair_validation():
    ovc, api, forward, v_repair = _mods()
    q = torch.randn(32768, 1, 128, device=DEV, dtype=torch.bfloat16)
    for bad in (-0.01, 1.0, float("nan")):
        with pytest.raises(ValueError, match="budget"):
            ovc.prepare_v_repair(q, q, q, budget=bad)
    with pytest.raises(ValueError, match="S >= 32768"):
        ovc.prepare_v_repair(q[:5000], q[:5000], q[:5000], budget=0.01)
    prepared = ovc.prepare_v_repair(q, q, q, budget=0.01)
    wrong = dataclasses.replace(prepared, repair_k_descale=prepared.repair_k_descale[..., :100].contiguous())
    with pytest.raises(ValueError, match="repair_k_descale"):
        ovc.attention_v_repair(wrong)


def test_repair_at_the_benchmark_size():
    """[73397,14,128], Student-t V, budget 0.005: 367 tokens in 384 rows per head; zeroed repair rows give
    the plain output bit for bit; with the residuals in place the error against exact attention drops."""
    ovc, api, forward, v_repair = _mods()
    from open_vc_attn.synthetic import student_t_values

    s, h = 73397, 14
    g = torch.Generator(device=DEV).manual_seed(73)
    q, k = [torch.randn(s, h, 128, generator=g, device=DEV).to(torch.bfloat16) for _ in range(2)]
    v = student_t_values(s, h, seed=74, device=DEV)
    prepared = ovc.prepare_v_repair(q, k, v, budget=0.005)
    assert (prepared.selected_tokens, prepared.repair_tokens) == (367, 384)
    assert prepared.k.shape[0] == s + 384 and prepared.repair_k_descale.shape == (1, h, 384)
    repaired = ovc.attention_v_repair(prepared)
    plain = ovc.attention(q, k, v)
    forward.check_status(q.device)
    head, rows = 5, torch.arange(0, s, 997, device=DEV)
    exact = oatt.exact_attention(f32(q[rows][:, head : head + 1]), f32(k[:, head : head + 1]), f32(v[:, head : head + 1]))
    assert oatt.relative_l2(f32(repaired[rows][:, head : head + 1]), exact) < oatt.relative_l2(
        f32(plain[rows][:, head : head + 1]), exact)
    padded = (s + 384 + 127) // 128 * 128
    buffer = torch.empty(0, dtype=torch.uint8, device=DEV).set_(prepared.v.untyped_storage(), 0, (h, 128, padded))
    buffer[:, :, :384] = 0
    assert torch.equal(ovc.attention_v_repair(prepared), plain)
