"""The bounded-wait failure path, exercised without hanging or faulting anything: a self-test kernel whose wait
cannot complete runs into its (short) limit and reports it; the attention kernels share that wait."""

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_util import DEV, f32  # noqa: E402
from oracle import attention as oatt  # noqa: E402


def _mods():
    import open_vc_attn
    from open_vc_attn import _lib, forward

    return open_vc_attn, _lib, forward


def test_expired_wait_is_reported_and_the_next_calls_are_unaffected():
    ovc, _lib, forward = _mods()
    lib = _lib.load()
    device = torch.device(DEV)
    forward.check_status(device)  # start clean
    words = forward.status_word(device)
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    with torch.cuda.device(device):
        _lib.check(lib.ovc_selftest_wait(words.data_ptr(), 200_000, gave_up.data_ptr(), _lib.stream_pointer(device)),
                   "ovc_selftest_wait")
    torch.cuda.synchronize()
    assert int(gave_up.item()) == 64  # every thread of the CTA ran into the limit and returned
    assert words.tolist() == [_lib.STATUS_WAIT_EXPIRED, _lib.STATUS_WAIT_EXPIRED]
    with pytest.raises(RuntimeError, match="bounded wait expired"):
        forward.check_status(device)
    forward.check_status(device)  # reading it cleared the sticky word

    # The context is intact and a normal call right after is correct.  The per-launch word the self-test
    # left set does not stop it: the library clears that word before every launch.
    assert int(words[0].item()) == _lib.STATUS_WAIT_EXPIRED
    torch.manual_seed(5)
    q, k, v = [torch.randn(300, 2, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    out = ovc.attention(q, k, v)
    forward.check_status(device)
    assert torch.isfinite(out.float()).all()
    assert oatt.relative_l2(f32(out), oatt.exact_attention(f32(q), f32(k), f32(v))) < 0.10


def test_a_failure_surfaces_at_the_next_public_call_without_a_sync():
    ovc, _lib, forward = _mods()
    lib = _lib.load()
    device = torch.device(DEV)
    forward.check_status(device)
    words = forward.status_word(device)
    gave_up = torch.zeros(1, dtype=torch.int32, device=DEV)
    torch.manual_seed(6)
    q, k, v = [torch.randn(200, 1, 128, device=DEV, dtype=torch.bfloat16) for _ in range(3)]
    with torch.cuda.device(device):
        _lib.check(lib.ovc_selftest_wait(words.data_ptr(), 100_000, gave_up.data_ptr(), _lib.stream_pointer(device)),
                   "ovc_selftest_wait")
    first = ovc.attention(q, k, v)  # computes normally and publishes the sticky word behind it
    torch.cuda.synchronize()
    with pytest.raises(RuntimeError, match="bounded wait expired"):
        ovc.attention(q, k, v)  # raised from host memory, before anything is launched
    again = ovc.attention(q, k, v)
    forward.check_status(device)
    assert torch.equal(first, again)
