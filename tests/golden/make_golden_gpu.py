"""Generate tests/golden/prep_golden_gpu.npz from the reference's Triton kernels running on a B200.

    REFERENCE_SRC=<reference>/src python tests/golden/make_golden_gpu.py [output.npz]

Unlike make_golden.py (Triton's CPU interpreter, final E4M3 cast substituted), this script launches the
reference's preparation kernels on the GPU itself, so the fixture holds what the reference really
produces on the hardware: Triton's lowering of `/`, `tl.max`, `tl.sum`, FMA contraction and the
hardware float32 -> float8e4nv conversion.

Contents
  hw_*            the cases of prep_golden.npz again (same inputs, read from that file), outputs from the GPU
  c1_*            Q, K, V [1024, 2, 128] BF16, N(0,1) from torch.manual_seed(0) on the CPU: general and
                  fused-kernel preparation and the byte transpose
  big_<S>_<H>_*   SHA-256 digests of codes and scales at (32769, 2) and (73397, 7), inputs from
                  `big_inputs(S, H)` below (CPU generator, so a test can rebuild them anywhere)
  vs_*            V-Smooth block statistics and write kernels for a fixed grouping permutation
  rcp_b, rcp_r    r = 1 / b as the GPU evaluates Triton's `/` (div.full.f32), for every divisor the small cases use
  div_a/b/q       random (a, b) pairs and q = a / b from the same instruction; div_model_violations counts pairs
                  where q != RN(a * (1 / b)) with that hardware reciprocal
  interp_diff_*   number of elements where the interpreter-made fixture differs from the hardware result
"""

import hashlib
import os
import sys

if "REFERENCE_SRC" not in os.environ:
    raise SystemExit("set REFERENCE_SRC to the src/ directory of an open-vc-attention 0.3.0 checkout")
sys.path.insert(0, os.environ["REFERENCE_SRC"])

import numpy as np  # noqa: E402
import torch  # noqa: E402
import triton  # noqa: E402
import triton.language as tl  # noqa: E402

from open_vc_attn.quantization import (  # noqa: E402
    _per_block_quant_kernel,
    _per_head_amax_kernel,
    _per_head_scale_cast_kernel,
)
from open_vc_attn.preparation import _cast_pack_v, _quantize_qk  # noqa: E402
from open_vc_attn.v_repair import _repair_rows_kernel, _v_quant_score_kernel  # noqa: E402
from open_vc_attn._kernels.blackwell.flash_attn.cute.v_layout import transpose_v  # noqa: E402
from open_vc_attn._kernels.blackwell.v_smooth import _block_stats, _block_write  # noqa: E402

E4M3 = torch.float8_e4m3fn
HERE = os.path.dirname(os.path.abspath(__file__))
DEV = "cuda:0"


def u8(t):
    return t.contiguous().view(torch.uint8).cpu().numpy()


def f32(t):
    return t.float().cpu().numpy()


def from_bits(bits, dtype):
    return torch.from_numpy(bits.view(np.int16).copy()).to(DEV).view(dtype)


def digest(array):
    return np.frombuffer(hashlib.sha256(np.ascontiguousarray(array).tobytes()).digest(), dtype=np.uint8).copy()


@triton.jit
def _div_kernel(A, B, Q, n, BLOCK: tl.constexpr):
    offs = tl.program_id(0) * BLOCK + tl.arange(0, BLOCK)
    mask = offs < n
    tl.store(Q + offs, tl.load(A + offs, mask, 1.0) / tl.load(B + offs, mask, 1.0), mask)


def hw_div(a, b):
    """a / b (float32 numpy arrays) as Triton's GPU code computes it."""
    a = torch.from_numpy(np.ascontiguousarray(a, dtype=np.float32)).to(DEV)
    b = torch.from_numpy(np.ascontiguousarray(b, dtype=np.float32)).to(DEV)
    q = torch.empty_like(a)
    n = a.numel()
    _div_kernel[((n + 1023) // 1024,)](a, b, q, n, BLOCK=1024)
    return q.cpu().numpy()


def block_amax(x):
    """max |x| per (batch, head, 128-token block), floored at 1e-12, as a flat float32 numpy array."""
    if x.dim() == 3:
        x = x[None]
    b, s, h, d = x.shape
    nb = (s + 127) // 128
    padded = torch.zeros(b, nb * 128, h, d, dtype=torch.float32, device=x.device)
    padded[:, :s] = x.float()
    return padded.view(b, nb, 128, h, d).abs().amax(dim=(2, 4)).clamp_min(1e-12).flatten().cpu().numpy()


def big_inputs(s, h):
    """Inputs of the large cases: CPU generator, BF16, a loud Q block, a quiet K tail, an all-zero V head."""
    gen = torch.Generator().manual_seed(414000 + s + h)
    q, k, v = [torch.randn(s, h, 128, generator=gen).to(torch.bfloat16) for _ in range(3)]
    q[:128] *= 16
    k[-129:] *= 0.125
    v[:, 0] = 0
    return q, k, v


def per_block(x):
    b, s, h, d = x.shape
    nb = (s + 127) // 128
    out = torch.empty_like(x, dtype=E4M3)
    scales = torch.empty(b, h, nb, dtype=torch.float32, device=DEV)
    _per_block_quant_kernel[(b, nb, h)](
        x, out, scales, s, h, d, nb, IS_INT8=False, QMAX=448.0, BLOCK_L=128, BLOCK_D=128, num_warps=4
    )
    return out, scales


def per_head(x):
    b, s, h, d = x.shape
    nb = (s + 127) // 128
    amax = torch.zeros(b, h, dtype=torch.float32, device=DEV)
    _per_head_amax_kernel[(b, nb, h)](x, amax, s, h, d, BLOCK_L=128, BLOCK_D=128, num_warps=4)
    out = torch.empty_like(x, dtype=E4M3)
    _per_head_scale_cast_kernel[(b, nb, h)](
        x, out, amax, s, h, d, IS_INT8=False, QMAX=448.0, BLOCK_L=128, BLOCK_D=128, num_warps=4
    )
    raw_amax = amax.clone()
    descale = torch.empty(b, h, dtype=torch.float32, device=DEV)
    torch.div(amax.clamp_(min=1e-12), 448.0, out=descale)
    return out, descale, raw_amax


def fused(q, k, v):
    s, h, d = q.shape
    blocks = (s + 127) // 128
    q_blocks = (blocks + 1) // 2 * 2
    padded = blocks * 128
    q8, k8 = [torch.empty_like(q, dtype=E4M3) for _ in range(2)]
    qs = torch.full((1, h, q_blocks), -7.0, dtype=torch.float32, device=DEV)
    ks = torch.full((1, h, blocks), -7.0, dtype=torch.float32, device=DEV)
    amax = torch.full((1, h), 123.0, dtype=torch.float32, device=DEV)
    _quantize_qk[(blocks, h, 2)](q, k, q8, k8, qs, ks, amax, s, h, blocks, q_blocks, num_warps=4)
    _per_head_amax_kernel[(1, blocks, h)](v, amax, s, h, d, BLOCK_L=128, BLOCK_D=128, num_warps=4)
    packed = torch.full((h, d, padded), 0.5, dtype=torch.float32, device=DEV).to(E4M3)
    vs = torch.empty(1, h, dtype=torch.float32, device=DEV)
    _cast_pack_v[(padded // 64, h)](v, packed, amax, vs, s, h, padded, num_warps=4)
    return q8, k8, packed, qs, ks, vs


def main():
    assert torch.cuda.is_available(), "this generator runs the reference kernels on a GPU"
    old = np.load(os.path.join(HERE, "prep_golden.npz"))
    out = {}
    diff = {}
    divisors = [np.float32([448.0, 1e-12])]

    def keep(name, value, old_name=None):
        out[name] = value
        if old_name is not None:
            diff["interp_diff_" + old_name] = np.int64((value != old[old_name]).sum())

    # ---- the interpreter fixture's cases on the hardware ------------------------------------
    x = from_bits(old["general_x_f16"], torch.float16)
    divisors += [block_amax(x), x.float().abs().amax(dim=(1, 3)).clamp_min(1e-12).flatten().cpu().numpy()]
    codes, scales = per_block(x)
    keep("hw_general_block_codes", u8(codes), "general_block_codes")
    keep("hw_general_block_descale", f32(scales), "general_block_descale")
    codes, descale, amax = per_head(x)
    keep("hw_general_head_amax", f32(amax), "general_head_amax")
    keep("hw_general_head_codes", u8(codes), "general_head_codes")
    keep("hw_general_head_descale", f32(descale), "general_head_descale")

    q, k, v = (from_bits(old[f"fused_{n}_bf16"], torch.bfloat16) for n in "qkv")
    divisors += [block_amax(q), block_amax(k), v.float().abs().amax(dim=(0, 2)).clamp_min(1e-12).cpu().numpy()]
    q8, k8, packed, qs, ks, vs = fused(q, k, v)
    keep("hw_fused_q_codes", u8(q8), "fused_q_codes")
    keep("hw_fused_k_codes", u8(k8), "fused_k_codes")
    keep("hw_fused_q_descale", f32(qs), "fused_q_descale")
    keep("hw_fused_k_descale", f32(ks), "fused_k_descale")
    keep("hw_fused_v_packed", u8(packed), "fused_v_packed")
    keep("hw_fused_v_descale", f32(vs), "fused_v_descale")

    src = torch.from_numpy(old["pack_in"]).to(DEV)
    buf = torch.full((2, 2, 128, 256), 0xAB, dtype=torch.uint8, device=DEV)
    transpose_v[(256 // 64, 2, 2)](src, buf, 200, 2 * 128, 256, 64, 128, num_warps=4)
    keep("hw_pack_out", buf.cpu().numpy(), "pack_out")

    # repair pieces (same inputs and selection as the interpreter fixture)
    v = from_bits(old["repair_v_bf16"], torch.bfloat16)
    k = from_bits(old["repair_k_bf16"], torch.bfloat16)
    s, h, d = v.shape
    blocks = (s + 127) // 128
    amax = torch.zeros(1, h, dtype=torch.float32, device=DEV)
    _per_head_amax_kernel[(1, blocks, h)](v, amax, s, h, d, BLOCK_L=128, BLOCK_D=128, num_warps=4)
    selected, rows = 5, 128
    total = rows + s
    v_all = torch.zeros(total, h, d, dtype=torch.float32, device=DEV).to(E4M3)
    score = torch.empty(h, s, dtype=torch.float32, device=DEV)
    _v_quant_score_kernel[(blocks, h)](v, v_all[rows:], amax, score, s, h, QMAX=448.0, BLOCK_L=128, D=d, num_warps=4)
    k_all = torch.zeros(total, h, d, dtype=torch.float32, device=DEV).to(E4M3)
    k8, k_descale = per_block(k[None])
    k_all[rows:] = k8[0]
    v_descale = amax.clamp(min=1e-12) / 448.0
    divisors += [block_amax(k), amax.clamp(min=1e-12).flatten().cpu().numpy(), v_descale.flatten().cpu().numpy()]
    index = torch.from_numpy(old["repair_index"]).to(DEV)
    repair_kd = torch.empty(1, h, rows, dtype=torch.float32, device=DEV)
    _repair_rows_kernel[(rows, h)](
        k_all, v_all, v, k_descale, v_descale, index, repair_kd, selected, rows, s, h, blocks,
        QMAX=448.0, D=d, num_warps=1,
    )
    keep("hw_repair_amax", f32(amax), "repair_amax")
    keep("hw_repair_score", f32(score))
    keep("hw_repair_v_codes", u8(v_all[rows:]))
    keep("hw_repair_k_all", u8(k_all), "repair_k_all")
    keep("hw_repair_kd", f32(repair_kd), "repair_kd")
    keep("hw_repair_v_prefix", u8(v_all[:rows]))
    keep("hw_repair_v_descale", f32(v_descale), "repair_v_descale")
    # residual scores are float sums: how far the interpreter's are, on rows where its codes were right
    ok = old["repair_score_row_ok"].T
    rel = np.abs(out["hw_repair_score"] - old["repair_score"]) / np.maximum(np.abs(old["repair_score"]), 1e-30)
    diff["interp_diff_repair_score_max_rel"] = np.float64(rel[ok].max())

    # ---- C1: [1024, 2, 128] BF16, N(0,1), seed 0 --------------------------------------------
    torch.manual_seed(0)
    q, k, v = [torch.randn(1024, 2, 128).to(torch.bfloat16) for _ in range(3)]
    qd, kd, vd = q.to(DEV), k.to(DEV), v.to(DEV)
    divisors += [block_amax(qd), block_amax(kd), vd.float().abs().amax(dim=(0, 2)).clamp_min(1e-12).cpu().numpy()]
    codes, scales = per_block(qd[None])
    keep("c1_q_codes", u8(codes[0]))
    keep("c1_q_descale", f32(scales))
    codes, scales = per_block(kd[None])
    keep("c1_k_codes", u8(codes[0]))
    keep("c1_k_descale", f32(scales))
    codes, descale, _ = per_head(vd[None])
    keep("c1_v_codes", u8(codes[0]))
    keep("c1_v_descale", f32(descale))
    q8, k8, packed, qs, ks, vs = fused(qd, kd, vd)
    keep("c1_fused_q_codes", u8(q8))
    keep("c1_fused_k_codes", u8(k8))
    keep("c1_fused_v_packed", u8(packed))
    keep("c1_fused_q_descale", f32(qs))
    keep("c1_fused_k_descale", f32(ks))
    keep("c1_fused_v_descale", f32(vs))

    # ---- large cases: digests ----------------------------------------------------------------
    for s, h in ((32769, 2), (73397, 7)):
        q, k, v = [t.to(DEV) for t in big_inputs(s, h)]
        tag = f"big_{s}_{h}_"
        q8, k8, packed, qs, ks, vs = fused(q, k, v)
        for name, value in (("q_codes", u8(q8)), ("k_codes", u8(k8)), ("v_packed", u8(packed)),
                            ("q_descale", f32(qs)), ("k_descale", f32(ks)), ("v_descale", f32(vs))):
            keep(tag + "fused_" + name, digest(value))
        gq, gqs = per_block(q[None])
        gk, gks = per_block(k[None])
        gv, gvs, _ = per_head(v[None])
        for name, value in (("q_codes", u8(gq[0])), ("k_codes", u8(gk[0])), ("v_codes", u8(gv[0])),
                            ("q_descale", f32(gqs)), ("k_descale", f32(gks)), ("v_descale", f32(gvs))):
            keep(tag + "general_" + name, digest(value))
        diff[f"fused_vs_general_{s}_{h}"] = np.int64(
            (u8(q8) != u8(gq[0])).sum() + (u8(k8) != u8(gk[0])).sum()
            + (f32(qs)[..., : gqs.shape[-1]] != f32(gqs)).sum() + (f32(ks) != f32(gks)).sum() + (f32(vs) != f32(gvs)).sum()
        )
        del q, k, v, q8, k8, packed, gq, gk, gv
        torch.cuda.empty_cache()

    # ---- V-Smooth block kernels for a fixed grouping -----------------------------------------
    s, h = 1000, 2
    gen = torch.Generator().manual_seed(515)
    k = torch.randn(s, h, 128, generator=gen).to(torch.bfloat16).to(DEV)
    v = (torch.randn(s, h, 128, generator=gen) + torch.randn(1, h, 128, generator=gen) * 2).to(torch.bfloat16).to(DEV)
    perm = torch.stack([torch.randperm(s, generator=gen) for _ in range(h)]).to(DEV)  # int64 [H,S]
    blocks = (s + 127) // 128
    means = torch.empty(h, blocks, 128, dtype=torch.float32, device=DEV)
    amax = torch.zeros(h, 128, dtype=torch.float32, device=DEV)
    _block_stats[(h, blocks)](v, perm, means, amax, s, h, 128, 128)
    k_out = torch.empty_like(k, dtype=E4M3)
    codes = torch.empty_like(v, dtype=E4M3)
    means_out = torch.empty(1, blocks, h, 128, dtype=torch.float32, device=DEV)
    scale = torch.empty(1, h, 128, dtype=torch.float32, device=DEV)
    _block_write[(h, blocks)](k, v, perm, means, amax, k_out, codes, means_out, scale, s, h, 128, 128)
    keep("vs_k_bf16", k.cpu().view(torch.int16).numpy().view(np.uint16))
    keep("vs_v_bf16", v.cpu().view(torch.int16).numpy().view(np.uint16))
    keep("vs_perm", perm.cpu().numpy())
    keep("vs_block_means", f32(means))
    keep("vs_amax", f32(amax))
    keep("vs_k_out", u8(k_out))
    keep("vs_codes", u8(codes))
    keep("vs_means_out", f32(means_out))
    keep("vs_scale", f32(scale))
    divisors += [np.float32([128.0, s - (blocks - 1) * 128]), f32(amax).reshape(-1), f32(scale).reshape(-1)]

    # ---- the division itself --------------------------------------------------------------------
    rcp_b = np.unique(np.concatenate([np.asarray(d, dtype=np.float32).reshape(-1) for d in divisors]))
    keep("rcp_b", rcp_b)
    keep("rcp_r", hw_div(np.ones_like(rcp_b), rcp_b))
    rng = np.random.default_rng(7)
    div_a = (rng.standard_normal(65536) * np.exp(4 * rng.standard_normal(65536))).astype(np.float32)
    div_b = np.abs(rng.standard_normal(65536) * np.exp(4 * rng.standard_normal(65536))).astype(np.float32) + np.float32(1e-20)
    div_q = hw_div(div_a, div_b)
    keep("div_a", div_a)
    keep("div_b", div_b)
    keep("div_q", div_q)
    modelled = (div_a * hw_div(np.ones_like(div_b), div_b)).astype(np.float32)
    diff["div_model_violations"] = np.int64((modelled != div_q).sum())
    diff["div_differs_from_ieee"] = np.int64(((div_a / div_b).astype(np.float32) != div_q).sum())
    diff["rcp_differs_from_ieee"] = np.int64(((np.float32(1) / rcp_b).astype(np.float32) != out["rcp_r"]).sum())

    out.update(diff)
    path = sys.argv[1] if len(sys.argv) > 1 else os.path.join(HERE, "prep_golden_gpu.npz")
    np.savez_compressed(path, **out)
    print("wrote", path)
    for name, value in diff.items():
        print(f"  {name}: {value}")
    print("  device:", torch.cuda.get_device_name(0), "torch", torch.__version__)
    print("  triton", triton.__version__)


if __name__ == "__main__":
    main()
