"""The CPU oracle against fixtures produced by the reference's own Triton kernels and against the worked
examples of its report.  Two fixture files pin the preparation: prep_golden.npz (tests/golden/make_golden.py,
Triton's CPU interpreter: IEEE division) and prep_golden_gpu.npz (tests/golden/make_golden_gpu.py, the same
kernels on a B200: the GPU's division, whose reciprocals are stored with the fixture)."""

import os

import numpy as np
import pytest

from oracle import attention as oatt
from oracle import fp8, prep


def f16(bits):
    return bits.view(np.float16).astype(np.float32)


def bf16(bits):
    return (bits.astype(np.uint32) << 16).view(np.float32)


def test_e4m3_roundtrip_and_ties():
    codes = np.arange(256, dtype=np.uint8)
    values = fp8.e4m3_decode(codes)
    finite = ~np.isnan(values)
    assert (fp8.e4m3_encode(values[finite]) == codes[finite]).all()
    # ties go to the even mantissa; 2^-10 is half of the smallest subnormal
    assert fp8.e4m3_encode(np.float32([2.0**-10, 3 * 2.0**-10, 17.0, 19.0, 1000.0])).tolist() == [
        0, 2, 0x58, 0x5A, 126]


def test_e4m3_matches_torch_cast():
    torch = pytest.importorskip("torch")
    gen = torch.Generator().manual_seed(3)
    x = (torch.randn(200000, generator=gen) * torch.exp(3 * torch.randn(200000, generator=gen))).clamp(-448, 448)
    assert (fp8.e4m3_encode(x.numpy()) == x.to(torch.float8_e4m3fn).view(torch.uint8).numpy()).all()


def test_general_quantisers_match_reference(golden):
    x = f16(golden["general_x_f16"])
    codes, descale = prep.quantize_per_block(x, prep.IEEE)
    assert np.array_equal(codes, golden["general_block_codes"])
    assert np.array_equal(descale, golden["general_block_descale"])
    assert np.array_equal(prep.head_amax(x), golden["general_head_amax"])
    codes, descale = prep.quantize_per_head(x, prep.IEEE)
    assert np.array_equal(codes, golden["general_head_codes"])
    assert np.array_equal(descale, golden["general_head_descale"])
    # the all-zero (batch, head): codes 0 and the floored scale
    assert not codes[1, :, 2].any() and descale[1, 2] == np.float32(1e-12) / np.float32(448)


def test_fused_preparation_matches_reference(golden):
    q, k, v = (bf16(golden[f"fused_{n}_bf16"]) for n in "qkv")
    out = prep.prepare_fused(q, k, v, prep.IEEE)
    assert not golden["fused_amax_after_init"].any()
    assert np.array_equal(out["q"], golden["fused_q_codes"])
    assert np.array_equal(out["k"], golden["fused_k_codes"])
    assert np.array_equal(out["q_descale"], golden["fused_q_descale"])
    assert out["q_descale"][0, 0, 3] == 1.0  # odd block count padded with 1.0
    assert np.array_equal(out["k_descale"], golden["fused_k_descale"])
    assert np.array_equal(out["v_packed"], golden["fused_v_packed"])
    assert not out["v_packed"][:, :, 333:].any()
    assert np.array_equal(out["v_descale"], golden["fused_v_descale"])


def test_pack_v_matches_reference(golden):
    assert np.array_equal(prep.pack_v(golden["pack_in"]), golden["pack_out"])


def test_repair_pieces_match_reference(golden):
    v, k = bf16(golden["repair_v_bf16"]), bf16(golden["repair_k_bf16"])
    index = golden["repair_index"]
    out = prep.prepare_repair(np.zeros_like(k), k, v, budget=5 / 260, index=index, arith=prep.IEEE)
    assert (out["selected_tokens"], out["repair_tokens"], out["total"]) == (5, 128, 388)
    assert np.array_equal(out["k"], golden["repair_k_all"])
    assert np.array_equal(out["repair_k_descale"], golden["repair_kd"])
    assert np.array_equal(out["v_descale"], golden["repair_v_descale"])
    assert (out["k_descale"][0, :, 0] == 1.0).all()
    ok = golden["repair_score_row_ok"].T  # [h, s]
    assert ok.sum() >= 5  # rows on which the interpreter's cast fault did not strike
    assert np.allclose(out["score"][ok], golden["repair_score"][ok], rtol=2e-6, atol=0)
    # V residual rows: the interpreter's cast is only wrong at mantissa carries, so
    # demand agreement on almost every byte and exact zero pad rows.
    mine = out["v_packed"][:, :, :128].transpose(2, 0, 1)
    theirs = golden["repair_v_prefix_interp"]
    assert not mine[5:].any() and not theirs[5:].any()
    assert (mine[:5] == theirs[:5]).mean() > 0.9


@pytest.fixture(scope="module")
def hw():
    return np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "prep_golden_gpu.npz"))


def hw_arith(hw):
    return prep.Arithmetic(recip=prep.RecipTable(hw["rcp_b"], hw["rcp_r"]), contract=True)


def test_gpu_division_model(hw):
    """a / b on the GPU is the dividend times the recorded reciprocal, rounded once; the reciprocal of 448
    is the correctly rounded one, other reciprocals differ from RN(1/b) in the last bit now and then."""
    assert int(hw["div_model_violations"]) == 0
    table = prep.RecipTable(hw["rcp_b"], hw["rcp_r"])
    assert table(np.float32([448.0]))[0] == np.float32(1.0) / np.float32(448.0)
    off = (prep.recip_model(hw["rcp_b"]) != hw["rcp_r"]).mean()
    assert 0.0 < off < 0.5


def test_general_quantisers_match_the_reference_on_hardware(golden, hw):
    x = f16(golden["general_x_f16"])
    arith = hw_arith(hw)
    codes, descale = prep.quantize_per_block(x, arith)
    assert np.array_equal(codes, hw["hw_general_block_codes"])
    assert np.array_equal(descale, hw["hw_general_block_descale"])
    codes, descale = prep.quantize_per_head(x, arith)
    assert np.array_equal(codes, hw["hw_general_head_codes"])
    assert np.array_equal(descale, hw["hw_general_head_descale"])


def test_fused_preparation_matches_the_reference_on_hardware(golden, hw):
    q, k, v = (bf16(golden[f"fused_{n}_bf16"]) for n in "qkv")
    out = prep.prepare_fused(q, k, v, hw_arith(hw))
    for name in ("q", "k"):
        assert np.array_equal(out[name], hw[f"hw_fused_{name}_codes"]), name
        assert np.array_equal(out[name + "_descale"], hw[f"hw_fused_{name}_descale"]), name
    assert np.array_equal(out["v_packed"], hw["hw_fused_v_packed"])
    assert np.array_equal(out["v_descale"], hw["hw_fused_v_descale"])


def test_config_c1_matches_the_reference_on_hardware(hw):
    """BASELINE configuration 1: Q, K, V [1024, 2, 128] BF16, N(0,1), seed 0."""
    torch = pytest.importorskip("torch")
    torch.manual_seed(0)
    q, k, v = [torch.randn(1024, 2, 128).to(torch.bfloat16).float().numpy() for _ in range(3)]
    out = prep.prepare_fused(q, k, v, hw_arith(hw))
    assert np.array_equal(out["q"], hw["c1_fused_q_codes"]) and np.array_equal(out["q"], hw["c1_q_codes"])
    assert np.array_equal(out["k"], hw["c1_fused_k_codes"]) and np.array_equal(out["k"], hw["c1_k_codes"])
    assert np.array_equal(out["v_packed"], hw["c1_fused_v_packed"])
    assert np.array_equal(out["q_descale"], hw["c1_fused_q_descale"])
    assert np.array_equal(out["k_descale"], hw["c1_fused_k_descale"]) and np.array_equal(out["k_descale"], hw["c1_k_descale"])
    assert np.array_equal(out["v_descale"], hw["c1_fused_v_descale"]) and np.array_equal(out["v_descale"], hw["c1_v_descale"])


def test_repair_pieces_match_the_reference_on_hardware(golden, hw):
    v, k = bf16(golden["repair_v_bf16"]), bf16(golden["repair_k_bf16"])
    out = prep.prepare_repair(np.zeros_like(k), k, v, budget=5 / 260, index=golden["repair_index"], arith=hw_arith(hw))
    assert np.array_equal(out["k"], hw["hw_repair_k_all"])
    assert np.array_equal(out["repair_k_descale"], hw["hw_repair_kd"])
    assert np.array_equal(out["v_descale"], hw["hw_repair_v_descale"])
    v_all = out["v_packed"][:, :, : out["total"]].transpose(2, 0, 1)
    assert np.array_equal(v_all[128:], hw["hw_repair_v_codes"])
    assert np.array_equal(v_all[:128], hw["hw_repair_v_prefix"])
    assert np.allclose(out["score"], hw["hw_repair_score"], rtol=2e-6, atol=0)


def test_v_smooth_block_kernels_match_the_reference_on_hardware(hw):
    """Downstream of the reference's own block means (a Triton reduction), codes, scales and scaled means are
    reproduced bit for bit; the oracle's own means are within a few ulp of the reference's."""
    from oracle import vsmooth

    k, v = bf16(hw["vs_k_bf16"]), bf16(hw["vs_v_bf16"])
    arith = hw_arith(hw)
    out = vsmooth.apply_v_smooth(np.zeros_like(k), k, v, hw["vs_perm"], arith=arith, block_means=hw["vs_block_means"])
    assert np.array_equal(out["amax"], hw["vs_amax"])
    assert np.array_equal(out["scale"], hw["vs_scale"][0])
    assert np.array_equal(out["k"], hw["vs_k_out"])
    assert np.array_equal(out["v"], hw["vs_codes"])
    assert np.array_equal(out["means"], hw["vs_means_out"][0])
    own = vsmooth.apply_v_smooth(np.zeros_like(k), k, v, hw["vs_perm"], arith=arith)
    ulp = np.abs(own["block_means"].view(np.int32).astype(np.int64) - hw["vs_block_means"].view(np.int32).astype(np.int64))
    assert ulp.max() <= 4


def test_repair_counts_follow_the_reference_examples():
    # docs/api.md:72 and tests/gpu/test_repair_cli.py:69-70 of the reference
    assert prep.repair_counts(0.005, 73397) == (367, 384)
    assert prep.repair_counts(0.005, 32769) == (164, 256)
    assert prep.repair_counts(0.0, 40000) == (0, 0)


@pytest.mark.parametrize("encoder", [oatt.encode_packed, oatt.encode_general])
def test_expcast_worked_examples(encoder):
    # docs/technical-report/report.en.md:171 -- u=-1 -> code 108 (value 96), u=-0.17 -> 118 (224)
    sigma = np.float32(oatt.LOG2_E)
    zero = np.zeros(1, np.float32)
    for u, code in ((-1.0, 108), (-0.17, 118), (0.0, 120), (-10.4, 0), (-np.inf, 0)):
        got = encoder(np.float32([[u]]), zero, sigma, 1.0)
        assert got[0, 0] == code, (u, got)
    assert fp8.e4m3_decode(np.uint8([108, 118, 120])).tolist() == [96.0, 224.0, 256.0]


def test_tile_order_examples():
    # docs/technical-report/report.en.md:230: 10 tiles, diagonal 3, window 4
    assert oatt.tile_order(10, 0, 0, 4, q_stages=1)[:1] == [4]
    assert oatt.tile_order(10, 0, 3, 4, q_stages=1) == [7, 6, 5, 4, 3, 2, 1, 0, 9, 8]
    assert oatt.tile_order(5, 0, 1, None) == [4, 3, 2, 1, 0]
    assert oatt.tile_order(6, 2, 0, 4) == [5, 4, 3, 2, 1, 0]
    assert oatt.tile_order(12, 2, 1, 4) == [8, 7, 6, 5, 4, 3, 2, 11, 10, 9, 1, 0]


def test_cpu_plumbing_config_against_exact_attention():
    """[1024,2,128] BF16 N(0,1) seed 0: ExpCast output within the reference's smoke
    tolerance (rel-L2 < 0.10, src/open_vc_attn/cli/check.py:64-72) of exact attention."""
    torch = pytest.importorskip("torch")
    torch.manual_seed(0)
    q, k, v = [torch.randn(1024, 2, 128).to(torch.bfloat16).float().numpy() for _ in range(3)]
    p = prep.prepare_fused(q, k, v)
    v8 = p["v_packed"][:, :, :1024].transpose(2, 0, 1)
    args = (p["q"], p["k"], v8, p["q_descale"][0], p["k_descale"][0], p["v_descale"][0])
    exact = oatt.exact_attention(q, k, v)
    packed = oatt.expcast_attention(*args)
    general = oatt.expcast_attention(*args, encoder="general")
    assert oatt.relative_l2(packed, exact) < 0.10
    assert oatt.relative_l2(general, packed) < 0.005


def test_zeroed_repair_rows_leave_the_output_unchanged():
    """tests/gpu/test_v_repair.py:31-39 of the reference: repair rows with zero V add nothing and
    are dropped from the denominator, so the output equals the plain one bit for bit."""
    rng = np.random.default_rng(5)
    s, h = 300, 1
    q, k, v = [bf16((rng.standard_normal((s, h, 128)).astype(np.float32).view(np.uint32) >> 16).astype(np.uint16))
               for _ in range(3)]
    base = prep.prepare_fused(q, k, v)
    v8 = base["v_packed"][:, :, :s].transpose(2, 0, 1)
    plain = oatt.expcast_attention(base["q"], base["k"], v8, base["q_descale"][0], base["k_descale"][0],
                                   base["v_descale"][0])
    rep = prep.prepare_repair(q, k, v, budget=0.02)
    v_all = rep["v_packed"][:, :, : rep["total"]].transpose(2, 0, 1).copy()
    v_all[: rep["repair_tokens"]] = 0
    repaired = oatt.expcast_attention(rep["q"], rep["k"], v_all, rep["q_descale"][0], rep["k_descale"][0],
                                      rep["v_descale"][0], repair_k_descale=rep["repair_k_descale"][0])
    assert np.array_equal(plain, repaired)
