"""ovc_prepare_fused_static: the fused preparation for callers that cannot give the library any scratch
memory (a server whose pool already owns the GPU, a plugin that only receives inputs and outputs).

Collected last on purpose.  Called straight through the C ABI, twice in a row with different inputs, and
compared bit for bit with ovc_prepare_fused, which takes the scratch buffer from the caller: the second
call shows that what the first one left in the library's built-in array does not leak into the next result.
"""

import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _prepare(lib, name, q, k, v, with_scratch):
    from open_vc_attn import _lib

    s, h, d = q.shape
    blocks = (s + 127) // 128
    q_blocks = (blocks + 1) // 2 * 2
    out = dict(
        q8=torch.empty(s, h, d, dtype=torch.uint8, device=DEV),
        k8=torch.empty(s, h, d, dtype=torch.uint8, device=DEV),
        packed=torch.full((h, d, blocks * 128), 0xAB, dtype=torch.uint8, device=DEV),
        qs=torch.empty(h, q_blocks, dtype=torch.float32, device=DEV),
        ks=torch.empty(h, blocks, dtype=torch.float32, device=DEV),
        vs=torch.empty(h, dtype=torch.float32, device=DEV),
    )
    args = [q.data_ptr(), k.data_ptr(), v.data_ptr(), _lib.dtype_code(q.dtype), s, h, out["q8"].data_ptr(),
            out["k8"].data_ptr(), out["packed"].data_ptr(), out["qs"].data_ptr(), out["ks"].data_ptr(),
            out["vs"].data_ptr()]
    if with_scratch:
        scratch = torch.full((h,), 7.0, dtype=torch.float32, device=DEV)
        args.append(scratch.data_ptr())
    args.append(_lib.stream_pointer(torch.device(DEV)))
    _lib.check(getattr(lib, name)(*args), name)
    torch.cuda.synchronize()
    return out


def test_static_scratch_variant_matches_the_caller_scratch_variant_twice():
    from open_vc_attn import _lib

    lib = _lib.load()
    g = torch.Generator(device=DEV).manual_seed(77)
    for call, (s, h, dtype, gain) in enumerate([(1000, 5, torch.bfloat16, 8.0), (333, 3, torch.float16, 0.25)]):
        q, k, v = [(torch.randn(s, h, 128, generator=g, device=DEV) * gain).to(dtype) for _ in range(3)]
        if call == 1:
            v[:, 0] = 0  # a head whose max is 0: a stale, larger max from the first call would show here
        expect = _prepare(lib, "ovc_prepare_fused", q, k, v, with_scratch=True)
        got = _prepare(lib, "ovc_prepare_fused_static", q, k, v, with_scratch=False)
        for name in expect:
            assert torch.equal(expect[name], got[name]), (call, name)


def test_static_scratch_variant_refuses_too_many_heads():
    from open_vc_attn import _lib

    lib = _lib.load()
    x = torch.zeros(16, dtype=torch.uint8, device=DEV)
    p = x.data_ptr()
    code = lib.ovc_prepare_fused_static(p, p, p, 1, 128, 4097, p, p, p, p, p, p, None)
    assert code == -5
    assert b"scratch" in lib.ovc_error_string(code)
