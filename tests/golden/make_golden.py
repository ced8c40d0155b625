"""Generate tests/golden/prep_golden.npz from the reference's own Triton kernels.

Run once where the reference checkout is available:

    REFERENCE_SRC=<reference>/src python tests/golden/make_golden.py

The reference's preparation kernels are executed on CPU tensors through Triton's
interpreter (TRITON_INTERPRET=1).  That interpreter's float32 -> float8e4nv cast
is faulty at mantissa carries (e.g. 124.09 -> 64), so wherever a kernel ends in
that cast it is given a float32 output buffer: the stored value is then the
reference's own scaled-and-clamped float32 number, and the final
round-to-nearest-even E4M3 cast (what the GPU's hardware conversion does) is
applied here with torch's CPU cast.  Scales, amax values, layouts, padding and
byte moves come straight from the reference kernels.

Kernels that read FP8 codes back (_v_quant_score_kernel, _repair_rows_kernel)
cannot avoid the faulty cast; for those the fixture records, per row, whether
the interpreter's codes agree with the correct cast, and tests use agreeing
rows only.
"""

import os
import sys

os.environ["TRITON_INTERPRET"] = "1"
if "REFERENCE_SRC" not in os.environ:
    raise SystemExit("set REFERENCE_SRC to the src/ directory of an open-vc-attention 0.3.0 checkout")
sys.path.insert(0, os.environ["REFERENCE_SRC"])

import numpy as np  # noqa: E402
import torch  # noqa: E402

from open_vc_attn.quantization import (  # noqa: E402
    _per_block_quant_kernel,
    _per_head_amax_kernel,
    _per_head_scale_cast_kernel,
)
from open_vc_attn.preparation import _cast_pack_v, _quantize_qk  # noqa: E402
from open_vc_attn.v_repair import _repair_rows_kernel, _v_quant_score_kernel  # noqa: E402
from open_vc_attn._kernels.blackwell.flash_attn.cute.v_layout import transpose_v  # noqa: E402

E4M3 = torch.float8_e4m3fn


def rne(x):
    return x.to(E4M3).view(torch.uint8).numpy()


def bits16(x):
    return x.view(torch.int16).numpy().view(np.uint16)


def main():
    out = {}
    gen = torch.Generator().manual_seed(20260101)

    # ---- general quantisers, batched, ragged tail, fp16 -------------------
    b, s, h, d = 2, 300, 3, 128
    nb = (s + 127) // 128
    x = (torch.randn(b, s, h, d, generator=gen) * 3).to(torch.float16)
    x[0, :128, 1] *= 16  # a loud block
    x[1, :, 2] = 0  # an all-zero (batch, head)
    pre = torch.empty(b, s, h, d, dtype=torch.float32)
    scales = torch.empty(b, h, nb, dtype=torch.float32)
    _per_block_quant_kernel[(b, nb, h)](
        x, pre, scales, s, h, d, nb, IS_INT8=False, QMAX=448.0, BLOCK_L=128, BLOCK_D=128, num_warps=4
    )
    out["general_x_f16"] = bits16(x)
    out["general_block_codes"] = rne(pre)
    out["general_block_descale"] = scales.numpy()
    amax = torch.zeros(b, h, dtype=torch.float32)
    _per_head_amax_kernel[(b, nb, h)](x, amax, s, h, d, BLOCK_L=128, BLOCK_D=128, num_warps=4)
    pre = torch.empty(b, s, h, d, dtype=torch.float32)
    _per_head_scale_cast_kernel[(b, nb, h)](
        x, pre, amax, s, h, d, IS_INT8=False, QMAX=448.0, BLOCK_L=128, BLOCK_D=128, num_warps=4
    )
    out["general_head_amax"] = amax.numpy().copy()
    out["general_head_codes"] = rne(pre)
    descale = torch.empty(b, h, dtype=torch.float32)
    torch.div(amax.clamp_(min=1e-12), 448.0, out=descale)
    out["general_head_descale"] = descale.numpy()

    # ---- fused three-kernel preparation, odd block count, bf16 ------------
    s, h = 333, 2
    blocks = (s + 127) // 128
    q_blocks = (blocks + 1) // 2 * 2
    padded = blocks * 128
    q, k, v = [torch.randn(s, h, d, generator=gen).to(torch.bfloat16) for _ in range(3)]
    k[-129:] *= 0.125
    v[:, 1] += 2.5
    q_pre, k_pre = [torch.empty(s, h, d, dtype=torch.float32) for _ in range(2)]
    qs = torch.full((1, h, q_blocks), -7.0, dtype=torch.float32)
    ks = torch.full((1, h, blocks), -7.0, dtype=torch.float32)
    amax = torch.full((1, h), 123.0, dtype=torch.float32)  # must be reset by the kernel
    _quantize_qk[(blocks, h, 2)](q, k, q_pre, k_pre, qs, ks, amax, s, h, blocks, q_blocks, num_warps=4)
    out["fused_amax_after_init"] = amax.numpy().copy()
    _per_head_amax_kernel[(1, blocks, h)](v, amax, s, h, d, BLOCK_L=128, BLOCK_D=128, num_warps=4)
    packed_pre = torch.full((h, d, padded), 9.0, dtype=torch.float32)
    vs = torch.empty(1, h, dtype=torch.float32)
    _cast_pack_v[(padded // 64, h)](v, packed_pre, amax, vs, s, h, padded, num_warps=4)
    out["fused_q_bf16"], out["fused_k_bf16"], out["fused_v_bf16"] = bits16(q), bits16(k), bits16(v)
    out["fused_q_codes"], out["fused_k_codes"] = rne(q_pre), rne(k_pre)
    out["fused_q_descale"], out["fused_k_descale"] = qs.numpy(), ks.numpy()
    out["fused_v_packed"] = rne(packed_pre)
    out["fused_v_descale"] = vs.numpy()

    # ---- byte transpose (no cast involved) ---------------------------------
    codes = torch.randint(0, 256, (2, 200, 2, d), generator=gen, dtype=torch.uint8)
    pad = 256
    buf = torch.full((2, 2, d, pad), 0xAB, dtype=torch.uint8)
    transpose_v[(pad // 64, 2, 2)](codes, buf, 200, 2 * d, pad, 64, 128, num_warps=4)
    out["pack_in"], out["pack_out"] = codes.numpy(), buf.numpy()

    # ---- repair preparation pieces -----------------------------------------
    s, h = 260, 2
    blocks = (s + 127) // 128
    v = torch.distributions.StudentT(3.0).sample((s, h, d)).to(torch.bfloat16)
    k = torch.randn(s, h, d, generator=gen).to(torch.bfloat16)
    amax = torch.zeros(1, h, dtype=torch.float32)
    _per_head_amax_kernel[(1, blocks, h)](v, amax, s, h, d, BLOCK_L=128, BLOCK_D=128, num_warps=4)
    selected, rows = 5, 128
    total = rows + s
    v_all = torch.zeros(total, h, d, dtype=E4M3)
    score = torch.empty(h, s, dtype=torch.float32)
    _v_quant_score_kernel[(blocks, h)](
        v, v_all[rows:], amax, score, s, h, QMAX=448.0, BLOCK_L=128, D=d, num_warps=4
    )
    # Correct codes for the same scaled values, to flag rows hit by the interpreter's cast fault.
    scale = 448.0 / amax.clamp(min=1e-12).double()
    good = (v.double() * scale[0][None, :, None]).float().clamp(-448, 448).to(E4M3)
    row_ok = (good.view(torch.uint8) == v_all[rows:].view(torch.uint8)).all(dim=2)  # [s,h]
    v_all[rows:] = good
    k_all = torch.zeros(total, h, d, dtype=E4M3)
    k_pre = torch.empty(s, h, d, dtype=torch.float32)
    k_descale = torch.empty(1, h, blocks, dtype=torch.float32)
    _per_block_quant_kernel[(1, blocks, h)](
        k, k_pre, k_descale, s, h, d, blocks, IS_INT8=False, QMAX=448.0, BLOCK_L=128, BLOCK_D=128, num_warps=4
    )
    k_all[rows:] = k_pre.to(E4M3)
    v_descale = amax.clamp(min=1e-12) / 448.0
    index = torch.tensor([[3, 259, 128, 127, 40], [0, 1, 2, 200, 131]], dtype=torch.int32)
    repair_kd = torch.empty(1, h, rows, dtype=torch.float32)
    v_res = v_all.clone()
    _repair_rows_kernel[(rows, h)](
        k_all, v_res, v, k_descale, v_descale, index, repair_kd, selected, rows, s, h, blocks,
        QMAX=448.0, D=d, num_warps=1,
    )
    out["repair_v_bf16"], out["repair_k_bf16"] = bits16(v), bits16(k)
    out["repair_amax"] = amax.numpy()
    out["repair_score"] = score.numpy()
    out["repair_score_row_ok"] = row_ok.numpy()
    out["repair_index"] = index.numpy()
    out["repair_k_all"] = k_all.view(torch.uint8).numpy()
    out["repair_kd"] = repair_kd.numpy()
    out["repair_v_prefix_interp"] = v_res[:rows].view(torch.uint8).numpy()
    out["repair_v_descale"] = v_descale.numpy()

    path = os.path.join(os.path.dirname(os.path.abspath(__file__)), "prep_golden.npz")
    np.savez_compressed(path, **out)
    print("wrote", path, {k: v.shape for k, v in out.items()})


if __name__ == "__main__":
    main()
