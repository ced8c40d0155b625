"""FP8 preparation on the GPU against what the reference's own Triton kernels produced on a B200
(tests/golden/prep_golden_gpu.npz, made by tests/golden/make_golden_gpu.py): byte for byte."""

import hashlib
import os

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_util import DEV, f32, hw_div, packed_buffer, u8  # noqa: E402

HERE = os.path.dirname(os.path.abspath(__file__))


@pytest.fixture(scope="module")
def hw():
    return np.load(os.path.join(HERE, "golden", "prep_golden_gpu.npz"))


def as_dev(bits, dtype):
    return torch.from_numpy(bits.view(np.int16).copy()).to(DEV).view(dtype)


def same(mine, theirs, what):
    mine, theirs = np.asarray(mine), np.asarray(theirs)
    assert mine.shape == theirs.shape, (what, mine.shape, theirs.shape)
    wrong = int((mine != theirs).sum())
    assert wrong == 0, f"{what}: {wrong} of {mine.size} elements differ from the reference's GPU result"


def digest(array):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(array).tobytes()).digest(), dtype=np.uint8)


def big_inputs(s, h):
    """The large cases' inputs, rebuilt exactly as make_golden_gpu.big_inputs builds them."""
    gen = torch.Generator().manual_seed(414000 + s + h)
    q, k, v = [torch.randn(s, h, 128, generator=gen).to(torch.bfloat16) for _ in range(3)]
    q[:128] *= 16
    k[-129:] *= 0.125
    v[:, 0] = 0
    return q, k, v


def test_division_is_the_reference_gpu_division(hw):
    same(hw_div(hw["div_a"], hw["div_b"]), hw["div_q"], "a / b")
    same(hw_div(np.ones_like(hw["rcp_b"]), hw["rcp_b"]), hw["rcp_r"], "1 / b")
    assert int(hw["div_model_violations"]) == 0  # a / b == RN(a * (1 / b)) held for every recorded pair


def test_general_quantisers_reproduce_the_hardware_fixture(golden, hw):
    from open_vc_attn import quantization

    x = as_dev(golden["general_x_f16"], torch.float16)
    codes, descale = quantization.fp8_quantize_per_block(x)
    same(u8(codes), hw["hw_general_block_codes"], "per-block codes")
    same(f32(descale), hw["hw_general_block_descale"], "per-block descale")
    codes, descale = quantization.fp8_quantize_per_head(x)
    same(u8(codes), hw["hw_general_head_codes"], "per-head codes")
    same(f32(descale), hw["hw_general_head_descale"], "per-head descale")


def test_fused_preparation_reproduces_the_hardware_fixture(golden, hw):
    from open_vc_attn import preparation

    q, k, v = (as_dev(golden[f"fused_{n}_bf16"], torch.bfloat16) for n in "qkv")
    p = preparation._prepare_packed(q, k, v, tuple(q.shape))
    same(u8(p.q), hw["hw_fused_q_codes"], "q codes")
    same(u8(p.k), hw["hw_fused_k_codes"], "k codes")
    same(packed_buffer(p.v), hw["hw_fused_v_packed"], "packed v")
    same(f32(p.q_descale), hw["hw_fused_q_descale"], "q descale")
    same(f32(p.k_descale), hw["hw_fused_k_descale"], "k descale")
    same(f32(p.v_descale), hw["hw_fused_v_descale"], "v descale")


def test_config_c1_reproduces_the_hardware_fixture(hw):
    """Q, K, V [1024, 2, 128] BF16, N(0,1), seed 0: general and fused preparation."""
    from open_vc_attn import preparation, quantization

    torch.manual_seed(0)
    q, k, v = [torch.randn(1024, 2, 128).to(torch.bfloat16).to(DEV) for _ in range(3)]
    for name, x in (("q", q), ("k", k)):
        codes, descale = quantization.fp8_quantize_per_block(x[None])
        same(u8(codes[0]), hw[f"c1_{name}_codes"], name + " codes")
        same(f32(descale), hw[f"c1_{name}_descale"], name + " descale")
    codes, descale = quantization.fp8_quantize_per_head(v[None])
    same(u8(codes[0]), hw["c1_v_codes"], "v codes")
    same(f32(descale), hw["c1_v_descale"], "v descale")
    p = preparation._prepare_packed(q, k, v, tuple(q.shape))
    same(u8(p.q), hw["c1_fused_q_codes"], "fused q codes")
    same(u8(p.k), hw["c1_fused_k_codes"], "fused k codes")
    same(packed_buffer(p.v), hw["c1_fused_v_packed"], "fused packed v")
    same(f32(p.q_descale), hw["c1_fused_q_descale"], "fused q descale")
    same(f32(p.k_descale), hw["c1_fused_k_descale"], "fused k descale")
    same(f32(p.v_descale), hw["c1_fused_v_descale"], "fused v descale")


@pytest.mark.parametrize("s,h", [(32769, 2), (73397, 7)])
def test_large_preparation_digests_match_the_hardware_fixture(hw, s, h):
    from open_vc_attn import api

    q, k, v = [t.to(DEV) for t in big_inputs(s, h)]
    tag = f"big_{s}_{h}_"
    fused = api.prepare_fp8_fused(q, k, v)
    for name, value in (("q_codes", u8(fused.q)), ("k_codes", u8(fused.k)), ("v_packed", packed_buffer(fused.v)),
                        ("q_descale", f32(fused.q_descale)), ("k_descale", f32(fused.k_descale)),
                        ("v_descale", f32(fused.v_descale))):
        assert np.array_equal(digest(value), hw[tag + "fused_" + name]), "fused " + name
    plain = api.prepare_fp8(q, k, v)
    for name, value in (("q_codes", u8(plain.q)), ("k_codes", u8(plain.k)), ("v_codes", u8(plain.v)),
                        ("q_descale", f32(plain.q_descale)), ("k_descale", f32(plain.k_descale)),
                        ("v_descale", f32(plain.v_descale))):
        assert np.array_equal(digest(value), hw[tag + "general_" + name]), "general " + name


def test_repair_pieces_reproduce_the_hardware_fixture(golden, hw):
    from open_vc_attn import _lib
    from open_vc_attn.quantization import fp8_quantize_per_block

    lib = _lib.load()
    v = as_dev(golden["repair_v_bf16"], torch.bfloat16)
    k = as_dev(golden["repair_k_bf16"], torch.bfloat16)
    s, h, d = v.shape
    selected, rows = 5, 128
    amax = torch.empty(1, h, dtype=torch.float32, device=DEV)
    stream = _lib.stream_pointer(DEV)
    _lib.check(lib.ovc_head_amax(v.data_ptr(), _lib.OVC_BF16, 1, s, h, amax.data_ptr(), stream), "amax")
    same(f32(amax), hw["hw_repair_amax"], "amax")
    v_all = torch.zeros(rows + s, h, d, dtype=torch.uint8, device=DEV)
    k_all = torch.zeros(rows + s, h, d, dtype=torch.uint8, device=DEV)
    score = torch.empty(h, s, dtype=torch.float32, device=DEV)
    _lib.check(lib.ovc_repair_score(v.data_ptr(), _lib.OVC_BF16, s, h, amax.data_ptr(), v_all[rows:].data_ptr(),
                                    score.data_ptr(), stream), "score")
    same(u8(v_all[rows:]), hw["hw_repair_v_codes"], "v codes")
    # the residual energies are float32 sums over 128 channels whose order the reference leaves to Triton
    assert np.allclose(f32(score), hw["hw_repair_score"], rtol=2e-6, atol=0)
    k8, k_descale = fp8_quantize_per_block(k[None])
    k_all[rows:] = k8[0].view(torch.uint8)
    v_descale = torch.from_numpy(hw["hw_repair_v_descale"]).to(DEV)
    index = torch.from_numpy(golden["repair_index"]).to(DEV)
    repair_kd = torch.empty(1, h, rows, dtype=torch.float32, device=DEV)
    _lib.check(lib.ovc_repair_rows(k_all.data_ptr(), v_all.data_ptr(), v.data_ptr(), _lib.OVC_BF16,
                                   k_descale.data_ptr(), v_descale.data_ptr(), index.data_ptr(), repair_kd.data_ptr(),
                                   selected, rows, s, h, k_descale.shape[2], stream), "rows")
    same(u8(k_all), hw["hw_repair_k_all"], "k rows")
    same(f32(repair_kd), hw["hw_repair_kd"], "repair k descale")
    same(u8(v_all[:rows]), hw["hw_repair_v_prefix"], "v residual rows")


def test_v_smooth_block_kernels_against_the_hardware_fixture(hw):
    """Block means are float32 sums whose order the reference leaves to Triton: means within 2 ulp, and
    everything computed from them compared where the means agree exactly."""
    from open_vc_attn import _lib

    lib = _lib.load()
    k = as_dev(hw["vs_k_bf16"], torch.bfloat16)
    v = as_dev(hw["vs_v_bf16"], torch.bfloat16)
    perm = torch.from_numpy(hw["vs_perm"]).to(DEV)
    s, h, d = v.shape
    blocks = (s + 127) // 128
    stream = _lib.stream_pointer(DEV)
    means = torch.empty(h, blocks, d, dtype=torch.float32, device=DEV)
    amax = torch.zeros(h, d, dtype=torch.float32, device=DEV)
    _lib.check(lib.ovc_vs_block_stats(v.data_ptr(), perm.data_ptr(), means.data_ptr(), amax.data_ptr(), s, h, stream), "stats")
    theirs = hw["vs_block_means"]
    mine = f32(means)
    ulp = np.abs(mine.view(np.int32).astype(np.int64) - theirs.view(np.int32).astype(np.int64))
    print("block means: exact", float((ulp == 0).mean()), "max ulp", int(ulp.max()))
    assert ulp.max() <= 4
    k_out = torch.empty(s, h, d, dtype=torch.uint8, device=DEV)
    codes = torch.empty(s, h, d, dtype=torch.uint8, device=DEV)
    means_out = torch.empty(1, blocks, h, d, dtype=torch.float32, device=DEV)
    scale = torch.empty(1, h, d, dtype=torch.float32, device=DEV)
    # downstream of the reference's own statistics, everything is defined bit for bit
    ref_means = torch.from_numpy(theirs).to(DEV)
    ref_amax = torch.from_numpy(hw["vs_amax"]).to(DEV)
    _lib.check(lib.ovc_vs_block_write(k.data_ptr(), v.data_ptr(), perm.data_ptr(), ref_means.data_ptr(), ref_amax.data_ptr(),
                                      k_out.data_ptr(), codes.data_ptr(), means_out.data_ptr(), scale.data_ptr(), s, h,
                                      stream), "write")
    same(u8(k_out), hw["vs_k_out"], "permuted k")
    same(f32(scale), hw["vs_scale"], "channel scales")
    same(f32(means_out), hw["vs_means_out"], "scaled means")
    same(u8(codes), hw["vs_codes"], "residual codes")
