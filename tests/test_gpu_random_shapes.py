"""Randomised sweep over the public calls: every combination of length, head count, window, layout and option must
finish without an expired wait, give finite output and give the same bits when repeated (the barrier protocols of
the kernel depend on the length and on the scan order, and a stall shows up as an error status, not as a hang)."""

import random

import pytest
import torch

pytestmark = pytest.mark.gpu

from gpu_util import DEV  # noqa: E402


def _run(tag, call):
    from open_vc_attn import forward

    outs = [call() for _ in range(2)]
    forward.check_status(torch.device(DEV))
    first, second = (o[0] if isinstance(o, tuple) else o for o in outs)
    assert torch.isfinite(first.float()).all(), tag
    assert torch.equal(first, second), tag


def test_random_shapes_complete_and_repeat():
    import open_vc_attn as ovc

    rng = random.Random(5)
    lengths = [1, 127, 128, 129, 255, 256, 257, 511, 1000, 2049, 4097, 8191, 16384]
    for trial in range(36):
        s = rng.choice(lengths + [9000 + rng.randint(0, 3000), 20000 + rng.randint(0, 9999)])
        h = rng.choice([1, 2, 3, 7])
        window = rng.choice([None, 0, 1, 4, 9, 64, 1000])
        kind = rng.choice(["plain", "plain", "batched", "repair", "causal", "lse", "fp16", "vc"])
        dtype = torch.float16 if kind == "fp16" else torch.bfloat16
        torch.manual_seed(trial)
        tag = (trial, kind, s, h, window)
        if kind == "batched":
            batch = rng.choice([2, 3])
            q, k, v = [torch.randn(batch, min(s, 6000), h, 128, device=DEV, dtype=dtype) for _ in range(3)]
            _run(tag, lambda: ovc.attention(q, k, v, mid_window_blocks=window))
        elif kind == "repair":
            s, h = 32768 + rng.randint(0, 9000), min(h, 2)
            q, k, v = [torch.randn(s, h, 128, device=DEV, dtype=dtype) for _ in range(3)]
            prepared = ovc.prepare_v_repair(q, k, v, budget=rng.choice([0.001, 0.005, 0.02]))
            _run(tag, lambda: ovc.attention_v_repair(prepared))
        elif kind == "vc":
            from open_vc_attn import baselines
            from open_vc_attn.api import raw_forward

            s = max(s, 129)
            q, k, v = [torch.randn(s, h, 128, device=DEV, dtype=dtype) for _ in range(3)]
            prepared = baselines.prepare_vc(q, k, v, clusters=16, iterations=1)
            _run(tag, lambda: raw_forward(prepared.q, prepared.k, prepared.v, expcast=True, mid_window_blocks=window,
                                          **prepared.forward_kwargs()))
        else:
            q, k, v = [torch.randn(s, h, 128, device=DEV, dtype=dtype) for _ in range(3)]
            options = dict(causal=True) if kind == "causal" else dict(mid_window_blocks=window)
            if kind == "lse":
                options["return_lse"] = True
            _run(tag, lambda: ovc.attention(q, k, v, **options))
