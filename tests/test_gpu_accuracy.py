"""Accuracy of the attention kernel at the benchmark shapes: sampled rows against the oracle at every head
count of the headline configuration and for the repair configuration, the reference's own sharper statistic
(kernel output against exact attention on the same dequantised FP8 inputs, docs/performance.md:73 of the
reference: 0.71 %), and the error against exact attention on the original BF16 inputs split into its two
parts, quantisation and ExpCast."""

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_util import DEV, f32, oracle_rows, structured_qkv  # noqa: E402
from oracle import attention as oatt  # noqa: E402

ORACLE_TOL = 5e-3  # rel-L2 bound against the oracle (the reference's ExpCast output stands behind it)


def _api():
    import open_vc_attn
    from open_vc_attn import api, forward

    return open_vc_attn, api, forward


def exact_rows(q, k, v, rows, head, scale=None):
    """Float64 softmax attention for the given query rows of one head, on the GPU.  q, k, v float tensors
    [S, 128] (already the values to attend over)."""
    tau = 1.0 / np.sqrt(128.0) if scale is None else scale
    s = (q[rows].double() @ k.double().T) * tau
    p = torch.softmax(s, dim=1)
    return (p @ v.double()).cpu().numpy()


def dequantised(prepared, head):
    """The FP8 inputs of one head as the values they stand for: codes times descales."""
    s = prepared.q.shape[0]
    blocks = (s + 127) // 128
    qd = prepared.q_descale[0, head, :blocks].repeat_interleave(128)[:s, None]
    kd = prepared.k_descale[0, head, :blocks].repeat_interleave(128)[:s, None]
    q = prepared.q[:, head].float() * qd
    k = prepared.k[:, head].float() * kd
    v = prepared.v[:, head].float() * prepared.v_descale[0, head]
    return q, k, v


def rel_l2(a, b):
    return float(np.linalg.norm(np.asarray(a, dtype=np.float64) - b) / np.linalg.norm(b))


@pytest.mark.parametrize("h", [14, 56])
def test_headline_shape_rows_against_the_oracle(h):
    """[73397, H, 128] for the head counts the packed-path test does not cover (it runs H = 7)."""
    ovc, api, forward = _api()
    s = 73397
    q, k, v = structured_qkv(s, h, seed=s + h)
    fused = api.prepare_fp8_fused(q, k, v)
    del q, k, v
    out = api.attention_fp8(fused)
    forward.check_status(out.device)
    m_blocks = (s + 255) // 256
    for head, m in ((0, 0), (h - 1, m_blocks - 1), (h // 2, m_blocks // 3)):
        rows, expect = oracle_rows(fused, [m], [head])
        assert oatt.relative_l2(f32(out[:, head])[rows], expect[:, 0]) < ORACLE_TOL, (head, m)
    assert torch.isfinite(out.float()).all()


def test_repair_configuration_rows_against_the_oracle():
    """[73397, 14, 128], Student-t V, budget 0.005: rows of attention_v_repair against the oracle with the
    device's own repair prefix (selection, key copies, residual codes) as input."""
    ovc, api, forward = _api()
    from open_vc_attn.synthetic import student_t_values

    s, h = 73397, 14
    g = torch.Generator(device=DEV).manual_seed(73)
    q, k = [torch.randn(s, h, 128, generator=g, device=DEV).to(torch.bfloat16) for _ in range(2)]
    v = student_t_values(s, h, seed=74, device=DEV)
    prepared = ovc.prepare_v_repair(q, k, v, budget=0.005)
    out = ovc.attention_v_repair(prepared)
    forward.check_status(out.device)
    m_blocks = (s + 255) // 256
    for head, m in ((0, 0), (h - 1, m_blocks - 1), (6, 100)):
        rows, expect = oracle_rows(prepared, [m], [head], repair_kd=prepared.repair_k_descale)
        assert oatt.relative_l2(f32(out[:, head])[rows], expect[:, 0]) < ORACLE_TOL, (head, m)


@pytest.mark.parametrize("case", ["c2", "c3"])
def test_error_against_exact_attention_and_its_two_parts(case):
    """64 evenly spaced query rows of two heads.  kernel vs exact attention on the dequantised FP8 inputs is
    the ExpCast part; exact-on-dequantised vs exact-on-original is what FP8 quantisation of Q, K, V costs;
    together they are the error against exact BF16-input attention.

    Structured inputs (c3: outlier channels, token-norm spread, so that a row's softmax has a few large terms):
    ExpCast part below 1.2 % (measured 0.45-0.6 %; the reference reports 0.71 % on its captures), total below
    4.5 % (measured 3.4-3.9 %, almost all of it quantisation; the reference's 3.0-3.2 % are for its captures).
    I.i.d. N(0,1) inputs (c2) give flat rows: most probabilities land in the lowest ExpCast codes, whose decoded
    values are furthest from the exponential, and the ExpCast part rises to about 3 % - a property of the
    encoding (the oracle agrees with the kernel to 1e-4 on the same rows), inside the reference's own 10 %
    bound for random data (tests/gpu/test_attention.py:36)."""
    ovc, api, forward = _api()
    if case == "c2":
        s, h = 32768, 8
        g = torch.Generator(device=DEV).manual_seed(s)
        q, k, v = [torch.randn(s, h, 128, device=DEV, generator=g).to(torch.bfloat16) for _ in range(3)]
    else:
        s, h = 73397, 7
        q, k, v = structured_qkv(s, h, seed=s + h)
    fused = api.prepare_fp8_fused(q, k, v)
    out = api.attention_fp8(fused)
    forward.check_status(out.device)
    rows = torch.linspace(0, s - 1, 64, device=DEV).long()
    for head in (0, h - 1):
        got = f32(out[rows][:, head])
        dq, dk, dv = dequantised(fused, head)
        on_fp8 = exact_rows(dq, dk, dv, rows, head)
        on_bf16 = exact_rows(q[:, head].float(), k[:, head].float(), v[:, head].float(), rows, head)
        expcast, quantisation, total = rel_l2(got, on_fp8), rel_l2(on_fp8, on_bf16), rel_l2(got, on_bf16)
        print(f"{case} head {head}: kernel vs exact on dequantised FP8 {expcast:.4f}; quantisation alone {quantisation:.4f}; "
              f"kernel vs exact on BF16 inputs {total:.4f}")
        assert expcast < (0.012 if case == "c3" else 0.04)
        assert total < (0.045 if case == "c3" else 0.10)
