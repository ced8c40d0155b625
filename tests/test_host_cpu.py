"""Host-side mirror of the reference API: lazy import, argument policy, sharding arithmetic."""

import os
import subprocess
import sys

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
PACKAGE_ROOT = os.path.join(ROOT, "open-vc-attention_b200")


def test_import_needs_neither_torch_nor_cuda():
    # tests/cpu/test_contracts.py:85-96 of the reference
    code = (
        "import sys; sys.path.insert(0, %r); import open_vc_attn; "
        "assert 'torch' not in sys.modules and 'ctypes' not in sys.modules; "
        "print(sorted(open_vc_attn.__all__))" % PACKAGE_ROOT
    )
    out = subprocess.run([sys.executable, "-c", code], capture_output=True, text=True, check=True).stdout
    for name in ("attention", "attention_fp8", "prepare_fp8", "prepare_fp8_fused", "prepare_v_repair",
                 "attention_v_repair", "raw_forward"):
        assert name in out


def test_defaults_match_the_reference():
    from open_vc_attn import _dispatch

    assert _dispatch.DEFAULT_VERSION == "open-vc"
    assert _dispatch.DEFAULT_MID_WINDOW_BLOCKS == 4
    with pytest.raises(ValueError, match="not available"):
        _dispatch.require_version("reference")
    with pytest.raises(ValueError, match="Unknown implementation"):
        _dispatch.require_version("other")


def test_cpu_tensors_are_refused_with_the_reference_messages():
    torch = pytest.importorskip("torch")
    import open_vc_attn
    from open_vc_attn import api

    q = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="same CUDA device"):
        open_vc_attn.attention(q, q, q)
    with pytest.raises(ValueError, match=r"\[S,H,128\] or \[B,S,H,128\]"):
        api.validate_qkv(q[0], q[0], q[0])
    with pytest.raises(ValueError, match="D=128"):
        api.validate_qkv(q[..., :64], q[..., :64], q[..., :64])
    with pytest.raises(ValueError, match="matching K/V shapes"):
        api.validate_qkv(q, q, q[:2])


def test_argument_policy_of_attention(monkeypatch):
    """Mode/version/preparation checks come before any device work (src/open_vc_attn/api.py:198-211)."""
    torch = pytest.importorskip("torch")
    from open_vc_attn import api

    monkeypatch.setattr(api, "validate_qkv", lambda *a, **k: None)
    monkeypatch.setattr(api, "_fused_preparation_eligible", lambda *a, **k: False)
    q = torch.zeros(4, 2, 128, dtype=torch.bfloat16)
    with pytest.raises(ValueError, match="mode must be bf16 or expcast"):
        api.attention(q, q, q, mode="fp4")
    with pytest.raises(ValueError, match='requires version="reference"'):
        api.attention(q, q, q, mode="bf16")
    with pytest.raises(ValueError, match="not available"):
        api.attention(q, q, q, mode="bf16", version="reference")
    with pytest.raises(ValueError, match="preparation must be"):
        api.attention(q, q, q, preparation="maybe")
    with pytest.raises(ValueError, match="Fused preparation requires"):
        api.attention(q, q, q, preparation="fused")
    with pytest.raises(ValueError, match="requires version"):
        api.attention_fp8(object(), version="reference")


def test_unbuilt_options_raise_instead_of_degrading():
    torch = pytest.importorskip("torch")
    from open_vc_attn import baselines, forward

    q = torch.zeros(4, 2, 128, dtype=torch.float8_e4m3fn)
    d3 = torch.ones(1, 2, 1)
    d2 = torch.ones(1, 2)
    common = dict(q_descale=d3, k_descale=d3, v_descale=d2, expcast=True)
    with pytest.raises(ValueError, match="plain key scan"):
        forward.flash_attn_fwd(q, q, q, causal=True, mid_window_blocks=4, **common)
    with pytest.raises(NotImplementedError, match="Unsupported kernel options"):
        forward.flash_attn_fwd(q, q, q, v_smooth_head_major=True, **common)
    with pytest.raises(NotImplementedError, match="takes no descales"):
        forward.flash_attn_fwd(q, q, q, v_smooth=True, **common)
    with pytest.raises(ValueError, match="needs v_smooth_means"):
        forward.flash_attn_fwd(q, q, q, v_smooth=True, expcast=True)
    with pytest.raises(ValueError, match="need v_smooth=True"):
        forward.flash_attn_fwd(q, q, q, v_smooth_means=d3, **common)
    with pytest.raises(ValueError, match="v_prepacked must use"):
        forward.flash_attn_fwd(q, q, q, v_prepacked=True, **common)
    with pytest.raises(ValueError, match="positive finite softmax_scale"):
        forward.flash_attn_fwd(q, q, q, softmax_scale=0.0, **common)
    with pytest.raises(ValueError, match="same CUDA device"):
        baselines.vc_attention(q, q, q)  # CPU tensors: the reference's validation message


def test_repair_budget_validation(monkeypatch):
    # tests/gpu/test_v_repair.py:84-88 of the reference
    torch = pytest.importorskip("torch")
    from open_vc_attn import v_repair

    monkeypatch.setattr(v_repair, "validate_qkv", lambda *a, **k: None)
    q = torch.zeros(40000, 1, 128, dtype=torch.bfloat16)
    for bad in (-0.1, 1.0, float("nan"), float("inf")):
        with pytest.raises(ValueError, match="budget"):
            v_repair.prepare_v_repair(q, q, q, budget=bad)
    with pytest.raises(ValueError, match="S >= 32768"):
        v_repair.prepare_v_repair(q[:100], q[:100], q[:100], budget=0.1)


def test_head_ranges_cover_all_heads_once():
    from open_vc_attn.sharding import head_range

    for heads, world in ((56, 8), (56, 4), (14, 4), (14, 8), (7, 8), (1, 2), (5, 3)):
        ranges = [head_range(heads, world, r) for r in range(world)]
        assert ranges[0][0] == 0 and ranges[-1][1] == heads
        assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
        sizes = [b - a for a, b in ranges]
        assert max(sizes) - min(sizes) <= 1
    assert head_range(56, 8, 3) == (21, 28)
    assert head_range(7, 8, 7) == (7, 7)  # one idle rank
    with pytest.raises(ValueError):
        head_range(8, 2, 2)


def _gather_worker(rank, world, port, heads, result):
    import torch
    import torch.distributed as dist

    from open_vc_attn.sharding import gather_heads, head_range

    dist.init_process_group("gloo", init_method=f"tcp://127.0.0.1:{port}", rank=rank, world_size=world)
    try:
        h0, h1 = head_range(heads, world, rank)
        full = torch.arange(3 * heads * 128, dtype=torch.float32).reshape(3, heads, 128).to(torch.bfloat16)
        merged = gather_heads(full[:, h0:h1].contiguous(), heads)
        result[rank] = bool(torch.equal(merged, full))
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("heads", [4, 5])
def test_gather_heads_with_two_gloo_ranks(heads):
    """World size 2 on CPU: uneven head counts are padded for the all-gather and trimmed after it."""
    pytest.importorskip("torch")
    import torch.multiprocessing as mp

    sys.path.insert(0, PACKAGE_ROOT)
    port = 29500 + (os.getpid() % 2000) + heads
    manager = mp.Manager()
    result = manager.dict()
    ctx = mp.get_context("spawn")
    procs = [ctx.Process(target=_gather_worker, args=(r, 2, port, heads, result)) for r in range(2)]
    for p in procs:
        p.start()
    for p in procs:
        p.join(120)
        assert p.exitcode == 0
    assert result[0] and result[1]


def test_packed_bounds():
    # tests/cpu/test_contracts.py:75-83 of the reference, and every fault segments() reports
    from open_vc_attn.integrations import segments

    assert segments((0, 129, 258), 258, 129) == [(0, 129, False), (129, 258, False)]
    assert segments([0, 7], 7, 7) == [(0, 7, False)]
    # one sequence and trailing padding: only with the option, only for two pieces, only if the first fills max_seqlen
    assert segments((0, 129, 200), 200, 129, trailing_padding=True) == [(0, 129, False), (129, 200, True)]
    assert segments((0, 129, 200), 200, 129) == [(0, 129, False), (129, 200, False)]
    assert segments((0, 100, 200), 200, 129, trailing_padding=True) == [(0, 100, False), (100, 200, False)]
    # padding may be longer than max_seqlen, a sequence may not
    assert segments((0, 4, 20), 20, 4, trailing_padding=True)[1] == (4, 20, True)
    for bounds, total, longest, text in [
        (None, 9, 9, "cu_seqlens_host is required"),
        ((0,), 0, 1, "start at zero"),
        ((1, 9), 9, 9, "start at zero"),
        ((0, 5, 8), 9, 9, "end at the tensor length"),
        ((0, 5, 5, 9), 9, 9, "strictly increasing"),
        ((0, 5.0, 9), 9, 9, "strictly increasing integers"),
        ((0, 5, 9), 9, 4, "max_seqlen is inconsistent"),
        ((0, 9), 9, 0, "max_seqlen is inconsistent"),
    ]:
        with pytest.raises(ValueError, match=text):
            segments(bounds, total, longest)


def test_diffusion_adapter_dispatches_per_sequence(monkeypatch):
    """tests/gpu/test_attention.py:69-87 of the reference is the acceptance test on a GPU; here the host logic:
    construction, environment selection, metadata checks, one attention() call per packed sequence."""
    torch = pytest.importorskip("torch")
    from open_vc_attn.integrations import DenseDiffusionAdapter, diffusion

    monkeypatch.delenv("OPEN_VC_ATTN_IMPLEMENTATION", raising=False)
    monkeypatch.delenv("OPEN_VC_ATTN_MODE", raising=False)
    adapter = DenseDiffusionAdapter(2, 128, 0.1)
    assert (adapter.version, adapter.mode, adapter.scale, adapter.trailing_padding) == ("open-vc", "expcast", 0.1, False)
    assert DenseDiffusionAdapter(2, 128, 0.1, num_kv_heads=2, prefix="blocks.0.attn").version == "open-vc"
    with pytest.raises(ValueError, match="head_size=128"):
        DenseDiffusionAdapter(2, 64, 0.1)
    with pytest.raises(ValueError, match="MHA"):
        DenseDiffusionAdapter(8, 128, 0.1, num_kv_heads=2)
    with pytest.raises(ValueError, match="noncausal"):
        DenseDiffusionAdapter(2, 128, 0.1, causal=True)
    with pytest.raises(ValueError, match="noncausal"):
        DenseDiffusionAdapter(2, 128, 0.1, dropout_p=0.1)
    monkeypatch.setenv("OPEN_VC_ATTN_MODE", "bf16")
    with pytest.raises(ValueError, match="reference with bf16"):
        DenseDiffusionAdapter(2, 128, 0.1)
    # the reference's BF16 backend (a third-party package) is not part of this build: not a valid choice here
    for version in ("reference", "fastest"):
        monkeypatch.setenv("OPEN_VC_ATTN_IMPLEMENTATION", version)
        with pytest.raises(ValueError, match="Invalid OPEN_VC_ATTN"):
            DenseDiffusionAdapter(2, 128, 0.1)
    monkeypatch.delenv("OPEN_VC_ATTN_IMPLEMENTATION")
    monkeypatch.delenv("OPEN_VC_ATTN_MODE")

    calls = []

    def fake_attention(q, k, v, **options):
        calls.append((tuple(q.shape), options["version"], options["mode"], options["softmax_scale"]))
        return q + 1

    monkeypatch.setattr(diffusion, "attention", fake_attention)
    q = torch.zeros(258, 2, 128, dtype=torch.bfloat16)
    cu = torch.tensor([0, 129, 258], dtype=torch.int32)
    out = adapter.forward_varlen(q, q, q, cu_seqlens=cu, max_seqlen=129, cu_seqlens_host=(0, 129, 258))
    assert out.shape == q.shape and bool((out == 1).all())
    assert calls == [((129, 2, 128), "open-vc", "expcast", 0.1)] * 2
    # one sequence: the call's own result, no copy; dense forward the same
    del calls[:]
    one = adapter.forward_varlen(q, q, q, cu_seqlens=cu[[0, 2]], max_seqlen=258, cu_seqlens_host=(0, 258))
    assert one.shape == q.shape and calls == [((258, 2, 128), "open-vc", "expcast", 0.1)]
    assert adapter.forward(q, q, q).shape == q.shape
    # trailing padding rows are zero and never attended
    del calls[:]
    padded = DenseDiffusionAdapter(2, 128, 0.1, packed_trailing_padding=True)
    out = padded.forward_varlen(q, q, q, cu_seqlens=cu, max_seqlen=129, cu_seqlens_host=(0, 129, 258))
    assert len(calls) == 1 and bool((out[:129] == 1).all()) and bool((out[129:] == 0).all())
    # metadata faults
    with pytest.raises(ValueError, match="matching"):
        adapter.forward_varlen(q, q[:100], q, cu_seqlens=cu, max_seqlen=129, cu_seqlens_host=(0, 129, 258))
    with pytest.raises(ValueError, match="same bounds"):
        adapter.forward_varlen(q, q, q, cu_seqlens=cu.long(), max_seqlen=129, cu_seqlens_host=(0, 129, 258))
    with pytest.raises(ValueError, match="same bounds"):
        adapter.forward_varlen(q, q, q, cu_seqlens=cu[:2], max_seqlen=129, cu_seqlens_host=(0, 129, 258))
    with pytest.raises(ValueError, match="cu_seqlens_host is required"):
        adapter.forward_varlen(q, q, q, cu_seqlens=cu, max_seqlen=129)


def test_sglang_registration_needs_sglang():
    try:
        import sglang  # noqa: F401
    except ImportError:
        with pytest.raises(ImportError, match="sglang"):
            import open_vc_attn.integrations.sglang  # noqa: F401
    else:
        from open_vc_attn.integrations import DenseDiffusionAdapter
        from open_vc_attn.integrations.sglang import OpenVCAttentionBackend

        assert OpenVCAttentionBackend.get_supported_head_sizes() == [128]
        assert issubclass(OpenVCAttentionBackend.get_impl_cls(), DenseDiffusionAdapter)


# a checkout of the reference beside this repository (or wherever REFERENCE_SRC points)
REFERENCE_PACKED = os.path.join(
    os.environ.get("REFERENCE_SRC") or os.path.join(os.path.dirname(os.path.dirname(os.path.dirname(os.path.abspath(__file__)))), "reference", "src"),
    "open_vc_attn", "integrations", "packed.py",
)


@pytest.mark.skipif(not os.path.isfile(REFERENCE_PACKED), reason="needs a checkout of the reference beside this repository")
def test_packed_bounds_agree_with_the_reference_on_random_metadata():
    """The reference's own segments(), read where it lies, against this package's on 3000 random cases (valid and
    faulty): same pieces or a ValueError with the same text."""
    import importlib.util
    import random

    from open_vc_attn.integrations import segments

    spec = importlib.util.spec_from_file_location("reference_packed", REFERENCE_PACKED)
    theirs = importlib.util.module_from_spec(spec)
    spec.loader.exec_module(theirs)
    rng = random.Random(7)
    for _ in range(3000):
        count = rng.randint(1, 4)
        edges = sorted(rng.sample(range(1, 40), count))
        bounds = [0] + edges
        mutation = rng.randint(0, 9)
        if mutation == 0:
            bounds[0] = 1
        elif mutation == 1:
            bounds[rng.randrange(len(bounds))] = float(bounds[-1])
        elif mutation == 2 and len(bounds) > 2:
            bounds[1] = bounds[2]
        elif mutation == 3:
            bounds = None
        total = edges[-1] + (1 if mutation == 4 else 0)
        longest = rng.choice([0, 1, 5, 20, 40] + edges)
        padding = rng.random() < 0.5

        def run(fn):
            try:
                return [tuple(piece) for piece in fn(None if bounds is None else tuple(bounds), total, longest, trailing_padding=padding)]
            except ValueError as error:
                return str(error)

        assert run(segments) == run(theirs.segments), (bounds, total, longest, padding)


def test_benchmark_statistics_and_shapes():
    # tests/cpu/test_records.py of the reference checks the same helpers through its record validator
    from open_vc_attn.benchmarking import measurement

    summary = measurement.summarize([2.0, 1.0, 3.0])
    assert summary["median_ms"] == 2.0 and summary["min_ms"] == 1.0 and summary["max_ms"] == 3.0
    assert summary["samples_ms"] == [2.0, 1.0, 3.0] and abs(summary["cv_percent"] - 40.8248) < 1e-3
    paired = measurement.speedup([4.0, 2.0, 6.0], [2.0, 2.0, 2.0])
    assert paired["ratio_of_medians"] == 2.0 and paired["median_paired_ratio"] == 2.0
    assert paired["paired_ratios"] == [2.0, 1.0, 3.0] and paired["latency_reduction_percent"] == 50.0
    for bad in ([], [1.0, float("nan")], [0.0], [-1.0]):
        with pytest.raises(ValueError, match="finite and positive"):
            measurement.summarize(bad)
    with pytest.raises(ValueError, match="equal nonzero length"):
        measurement.speedup([1.0], [1.0, 2.0])
    assert measurement.parse_shape("73397x56x128") == (73397, 56, 128)
    assert measurement.parse_shape("1024,7,128") == (1024, 7, 128)
    for bad in ("1024x7", "1024x7x64", "0x7x128", "axbx128"):
        with pytest.raises(ValueError, match="SxHx128"):
            measurement.parse_shape(bad)


def _record(rounds=2, isolated=True):
    timing = lambda values: {"samples_ms": values}  # noqa: E731
    return {
        "schema_version": 1, "status": "complete", "baseline": "bf16", "scope": "attention", "timing": "events",
        "gpu": "B200", "isolation_checked": isolated, "settings": {"rounds": rounds, "repair_budget": 0.0, "preparation": "auto"},
        "shapes": [{
            "shape": [1024, 7, 128],
            "timings": {"bf16": timing([2.0, 2.0]), "vc": timing([1.5, 1.5]), "open-vc": timing([1.0, 1.0])},
            "accuracy": {"open-vc": {"finite": True, "relative_l2": 0.03}, "vc": {"finite": True, "relative_l2": 0.031}},
        }],
    }


def test_benchmark_report_rendering():
    from open_vc_attn.benchmarking import report

    text = report.render(_record())
    assert "| 1024 x 7 x 128 | 2.000 | 1.500 | 1.000 | 2.000x | 3.000% |" in text
    assert "Shared-GPU" not in text and "Shared-GPU result" in report.render(_record(isolated=False))
    assert "| 1.333x |" in report.render(_record(), candidate="vc")
    with pytest.raises(ValueError, match="complete standalone benchmark report"):
        report.render({**_record(), "status": "running"})
    with pytest.raises(ValueError, match="Incomplete sample count"):
        report.render(_record(rounds=3))
    broken = _record()
    broken["shapes"][0]["accuracy"]["open-vc"]["finite"] = False
    with pytest.raises(ValueError, match="finite output"):
        report.render(broken)
    with pytest.raises(ValueError, match="must be measured backends"):
        report.render(_record(), baseline="fa3")


def test_benchmark_command_line_rules(capsys):
    from open_vc_attn.benchmarking import runner

    parser = runner.build_parser()
    assert runner.validated_shapes(parser.parse_args(["--preset", "smoke"]), parser) == [(129, 2, 128), (1024, 7, 128)]
    assert len(runner.validated_shapes(parser.parse_args(["--preset", "video"]), parser)) == 6
    for argv, message in (
        (["--rounds", "0"], "Rounds/repeats must be positive"),
        (["--backends", "bf16", "bf16"], "Duplicate backend names"),
        (["--backends", "vc", "open-vc"], "baseline must be included"),
        (["--repair-budget", "1.0"], "in \\[0, 1\\)"),
        (["--repair-budget", "0.01", "--backends", "bf16", "vc"], "requires the open-vc backend"),
        (["--preparation", "fused"], "requires quantize-attention scope"),
        (["--repair-budget", "0.01", "--shapes", "4096x7x128"], "sequence lengths >= 32768"),
        (["--shapes", "64x2x128"], "vc backend requires sequence lengths >= 128"),
        (["--shapes", "64x2x64"], "SxHx128"),
    ):
        with pytest.raises(SystemExit):
            runner.validated_shapes(parser.parse_args(argv), parser)
        import re

        assert re.search(message, capsys.readouterr().err)


def test_kernel_interface_rejects_packed_multi_sequence_metadata():
    """cu_seqlens with more than one sequence, metadata on batched input and a wrong max_seqlen raise before
    anything touches a GPU (the reference's kernel would treat the first as varlen input)."""
    import torch

    from open_vc_attn import forward

    q = torch.zeros(256, 2, 128).to(torch.float8_e4m3fn)
    args = dict(q_descale=torch.ones(1, 2, 2), k_descale=torch.ones(1, 2, 2), v_descale=torch.ones(1, 2), expcast=True)
    three = torch.tensor([0, 100, 256], dtype=torch.int32)
    with pytest.raises(NotImplementedError, match="varlen"):
        forward.flash_attn_fwd(q, q, q, cu_seqlens_q=three, **args)
    with pytest.raises(NotImplementedError, match="varlen"):
        forward.flash_attn_fwd(q, q, q, cu_seqlens_k=three, **args)
    with pytest.raises(ValueError, match="max_seqlen_q"):
        forward.flash_attn_fwd(q, q, q, max_seqlen_q=100, **args)
    with pytest.raises(ValueError, match="max_seqlen_k"):
        forward.flash_attn_fwd(q, q, q, max_seqlen_k=255, **args)
    q4 = q[None]
    with pytest.raises(ValueError, match="batched"):
        forward.flash_attn_fwd(q4, q4, q4, cu_seqlens_q=torch.tensor([0, 256], dtype=torch.int32), **args)
