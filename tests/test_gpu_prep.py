"""FP8 preparation on the GPU against the CPU oracle: bit-exact.  The oracle is given the GPU's own
reciprocals (gpu_util.hw_arith), the one piece of the reference's arithmetic a CPU cannot reproduce; the
comparison with the reference's kernels themselves is in test_gpu_prep_hw.py."""

import numpy as np
import pytest
import torch

from oracle import prep as oprep

pytestmark = pytest.mark.gpu


def _imports():
    from open_vc_attn import api, preparation, quantization, v_repair

    return api, preparation, quantization, v_repair


from gpu_util import DEV, f32, hw_arith, packed_buffer, u8  # noqa: E402


def as_dev(bits, dtype):
    raw = torch.from_numpy(bits.view(np.int16).copy()).to(DEV)
    return raw.view(dtype)


def test_pack_v_reproduces_the_reference_fixture(golden):
    _, _, quantization, _ = _imports()
    codes = torch.from_numpy(golden["pack_in"]).to(DEV).view(torch.float8_e4m3fn)
    view = quantization.pack_v(codes)
    assert tuple(view.shape) == tuple(codes.shape)
    assert np.array_equal(u8(view), golden["pack_in"])
    b, s, h, d = codes.shape
    buffer = torch.empty(0, dtype=torch.uint8, device=DEV).set_(view.untyped_storage(), 0, (b, h, d, 256))
    assert np.array_equal(buffer.cpu().numpy(), golden["pack_out"])


@pytest.mark.parametrize(
    "b,s,h,dtype",
    [(1, 1, 1, torch.float16), (1, 127, 2, torch.bfloat16), (1, 128, 1, torch.bfloat16), (2, 129, 3, torch.float16),
     (1, 255, 2, torch.bfloat16), (1, 257, 1, torch.float16), (3, 1000, 5, torch.bfloat16), (4, 8191, 24, torch.float16)],
)
def test_general_preparation_matches_the_oracle(b, s, h, dtype):
    api, _, quantization, _ = _imports()
    g = torch.Generator(device=DEV).manual_seed(1000 + s)
    x = (torch.randn(b, s, h, 128, generator=g, device=DEV) * 2).to(dtype)
    x[0, : min(s, 128), 0] *= 16
    if h > 1:
        x[-1, :, 1] = 0  # an all-zero (batch, head)
    xf = f32(x)
    codes, descale = quantization.fp8_quantize_per_block(x)
    arith = hw_arith()
    oc, od = oprep.quantize_per_block(xf, arith)
    assert np.array_equal(u8(codes), oc) and np.array_equal(f32(descale), od)
    codes, descale = quantization.fp8_quantize_per_head(x)
    oc, od = oprep.quantize_per_head(xf, arith)
    assert np.array_equal(u8(codes), oc) and np.array_equal(f32(descale), od)
    packed = quantization.pack_v(codes)
    padded = (s + 127) // 128 * 128
    buffer = torch.empty(0, dtype=torch.uint8, device=DEV).set_(packed.untyped_storage(), 0, (b, h, 128, padded))
    assert np.array_equal(buffer.cpu().numpy(), oprep.pack_v(oc))


@pytest.mark.parametrize("s,h,dtype", [(32768, 2, torch.float16), (32769, 2, torch.bfloat16), (73397, 7, torch.bfloat16)])
def test_fused_equals_general_bytes_and_the_oracle(s, h, dtype):
    """The reference's own large test (tests/gpu/test_preparation.py:24-58): fused and general
    preparation agree byte for byte, with scaled blocks and an all-zero V head."""
    api, _, _, _ = _imports()
    torch.manual_seed(414)
    q, k, v = [torch.randn(s, h, 128, device=DEV, dtype=dtype) for _ in range(3)]
    q[:128] *= 16
    k[-129:] *= 0.125
    v[:, 0] = 0
    plain = api.prepare_fp8(q, k, v)
    cu = torch.arange(2, device=DEV, dtype=torch.int32) * s
    fused = api.prepare_fp8_fused(q, k, v, cu_seqlens=cu)
    for name in ("q", "k", "v"):
        assert torch.equal(getattr(plain, name).contiguous().view(torch.uint8),
                           getattr(fused, name).contiguous().view(torch.uint8)), name
    blocks = (s + 127) // 128
    assert torch.equal(plain.q_descale, fused.q_descale[..., :blocks])
    assert fused.q_descale.shape[-1] % 2 == 0
    if blocks % 2:
        assert float(fused.q_descale[0, 0, blocks]) == 1.0
    assert torch.equal(plain.k_descale, fused.k_descale)
    assert torch.equal(plain.v_descale, fused.v_descale)
    assert fused.layout["cu_seqlens_q"] is cu and fused.layout["cu_seqlens_k"] is cu
    assert fused.v_prepacked and fused.v.stride(0) == 1
    buffer = packed_buffer(fused.v)
    assert not buffer[:, :, s:].any()  # zero tail
    # oracle on a slice of heads (full tensors would take the CPU minutes)
    head = h - 1
    o = oprep.prepare_fused(*[f32(t[:, head : head + 1]) for t in (q, k, v)], arith=hw_arith())
    assert np.array_equal(u8(fused.q[:, head : head + 1]), o["q"])
    assert np.array_equal(u8(fused.k[:, head : head + 1]), o["k"])
    assert np.array_equal(buffer[head : head + 1], o["v_packed"])
    assert np.array_equal(f32(fused.q_descale)[:, head : head + 1], o["q_descale"])
    assert np.array_equal(f32(fused.k_descale)[:, head : head + 1], o["k_descale"])
    assert np.array_equal(f32(fused.v_descale)[:, head : head + 1], o["v_descale"])


def test_fused_preparation_argument_errors():
    api, _, _, _ = _imports()
    q = torch.randn(32768, 1, 128, device=DEV, dtype=torch.bfloat16)
    short = q[:1000]
    with pytest.raises(ValueError, match="S >= 32768"):
        api.prepare_fp8_fused(short, short, short)
    with pytest.raises(ValueError, match="single-sequence"):
        api.prepare_fp8_fused(q, q[:-1], q[:-1])
    with pytest.raises(ValueError, match="cu_seqlens"):
        api.prepare_fp8_fused(q, q, q, cu_seqlens=torch.zeros(2, dtype=torch.int64, device=DEV))
    with pytest.raises(ValueError, match="Fused preparation requires"):
        api.attention(short, short, short, preparation="fused")


def test_repair_pieces_match_the_oracle(golden):
    """Key copies, per-row K descales and V residual codes for a given token selection."""
    from open_vc_attn import _lib

    lib = _lib.load()
    arith = hw_arith()
    v = as_dev(golden["repair_v_bf16"], torch.bfloat16)
    k = as_dev(golden["repair_k_bf16"], torch.bfloat16)
    vf, kf = f32(v), f32(k)
    s, h, rows, selected = 260, 2, 128, 5
    o = oprep.prepare_repair(np.zeros_like(vf), kf, vf, budget=5 / 260, index=golden["repair_index"], arith=arith)
    k_all = torch.from_numpy(o["k"].copy()).to(DEV)
    k_all[:rows] = 0
    index = torch.from_numpy(golden["repair_index"]).to(DEV)
    amax = torch.from_numpy(oprep.head_amax(vf[None])).to(DEV)
    v_all = torch.zeros(rows + s, h, 128, dtype=torch.uint8, device=DEV)
    score = torch.empty(h, s, dtype=torch.float32, device=DEV)
    stream = _lib.stream_pointer(torch.device(DEV))
    _lib.check(lib.ovc_repair_score(v.data_ptr(), 1, s, h, amax.data_ptr(), v_all[rows:].data_ptr(), score.data_ptr(),
                                    stream), "score")
    oc, od = oprep.quantize_per_head(vf[None], arith)
    assert np.array_equal(v_all[rows:].cpu().numpy(), oc[0])
    assert np.allclose(f32(score), o["score"], rtol=1e-5, atol=0)
    k_descale = torch.from_numpy(oprep.quantize_per_block(kf[None], arith)[1]).to(DEV)
    v_descale = torch.from_numpy(od).to(DEV)
    repair_kd = torch.empty(1, h, rows, dtype=torch.float32, device=DEV)
    _lib.check(lib.ovc_repair_rows(k_all.data_ptr(), v_all.data_ptr(), v.data_ptr(), 1, k_descale.data_ptr(),
                                   v_descale.data_ptr(), index.data_ptr(), repair_kd.data_ptr(), selected, rows, s, h,
                                   3, stream), "rows")
    assert np.array_equal(k_all.cpu().numpy(), o["k"])
    assert np.array_equal(f32(repair_kd), o["repair_k_descale"])
    expect_v = o["v_packed"][:, :, : rows + s].transpose(2, 0, 1)
    assert np.array_equal(v_all.cpu().numpy(), expect_v)
