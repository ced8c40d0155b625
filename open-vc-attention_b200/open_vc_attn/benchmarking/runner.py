"""Paired benchmark of BF16 attention, the VC-Attention baseline and the Open-VC path on one GPU.

Command line, record layout (schema version 1) and measurement protocol of `open-vc-attn-bench` of the
reference (src/open_vc_attn/benchmarking/runner.py): per shape, every backend is prepared and warmed
up, then timed in `rounds` rounds of `repeats` back-to-back calls in a freshly shuffled order per
round, with CUDA events or as CUDA-graph replays; accuracy is the relative L2 error against the BF16
output.  The record is rewritten after every round, so an interrupted run leaves a file whose
status is not "complete".

    python -m open_vc_attn.benchmarking.runner --preset smoke --allow-shared-gpu --output results/smoke.json
"""

import argparse
import datetime
import gc
import hashlib
import importlib.metadata
import json
import math
import os
import pathlib
import random
import subprocess
import time

from .backends import BACKENDS, CANDIDATE, DEFAULT_BACKENDS, DEFAULT_BASELINE, get_backend
from .measurement import parse_shape, speedup, summarize

PACKAGE_ROOT = pathlib.Path(__file__).resolve().parents[1]
VIDEO_SHAPES = [f"{s}x{h}x128" for s in (32768, 73426, 188214) for h in (7, 56)]
SMOKE_SHAPES = ["129x2x128", "1024x7x128"]


def _utc_now():
    return datetime.datetime.now(datetime.timezone.utc).isoformat()


def _file_digest(path):
    return hashlib.sha256(pathlib.Path(path).read_bytes()).hexdigest()


class GpuGuard:
    """Rejects the run when another process has a compute context on the benchmarked GPU."""

    def __init__(self, device, enabled):
        import torch

        uuid = str(torch.cuda.get_device_properties(device).uuid)
        self.uuid = uuid if uuid.startswith(("GPU-", "MIG-")) else "GPU-" + uuid
        self.enabled = enabled
        self.samples = 0

    def check(self):
        if not self.enabled:
            return
        listing = subprocess.run(
            ["nvidia-smi", "-i", self.uuid, "--query-compute-apps=pid", "--format=csv,noheader,nounits"],
            capture_output=True, text=True, check=True,
        ).stdout
        others = {int(line) for line in listing.split() if line.strip()} - {os.getpid()}
        if others:
            raise RuntimeError(f"Other CUDA processes detected: {sorted(others)}; reject this run")
        self.samples += 1

    def device_state(self):
        fields = ["driver_version", "pstate", "clocks.sm", "clocks.mem", "power.limit"]
        try:
            text = subprocess.run(
                ["nvidia-smi", "-i", self.uuid, "--query-gpu=" + ",".join(fields), "--format=csv,noheader,nounits"],
                capture_output=True, text=True, check=True, timeout=10,
            ).stdout
            values = [item.strip() for item in text.strip().split(",")]
            if len(values) != len(fields):
                raise ValueError("Unexpected GPU metadata columns")
            return dict(zip(fields, values))
        except (OSError, ValueError, subprocess.SubprocessError) as exc:
            return {"unavailable": type(exc).__name__}


def provenance(root=PACKAGE_ROOT):
    """Hashes of every Python source of the package and of the native library it loads."""
    from .. import _lib

    sources = {
        path.relative_to(root).as_posix(): _file_digest(path)
        for path in sorted(root.rglob("*.py")) if "__pycache__" not in path.parts
    }
    digest = hashlib.sha256()
    for name, value in sources.items():
        digest.update(f"{name}\0{value}\n".encode())
    revision = None
    try:
        top, commit = subprocess.run(["git", "-C", str(root), "rev-parse", "--show-toplevel", "HEAD"],
                                     capture_output=True, text=True, check=True, timeout=10).stdout.split()
        dirty = subprocess.run(["git", "-C", top, "status", "--porcelain", "--untracked-files=no"],
                               capture_output=True, text=True, check=True, timeout=10).stdout.strip()
        revision = {"commit": commit, "dirty": bool(dirty)}
    except (OSError, ValueError, subprocess.SubprocessError):
        pass
    native = _file_digest(_lib.LIBRARY_PATH) if os.path.exists(_lib.LIBRARY_PATH) else None
    return {"package_sha256": digest.hexdigest(), "source_sha256": sources, "source_revision": revision,
            "native_library_sha256": native}


def bf16_attention(q, k, v):
    """The BF16 yardstick: softmax(QK^T / sqrt(D)) V by PyTorch's fused attention, [S,H,D] in and out."""
    import torch

    out = torch.nn.functional.scaled_dot_product_attention(
        q.transpose(0, 1).unsqueeze(0), k.transpose(0, 1).unsqueeze(0), v.transpose(0, 1).unsqueeze(0))
    return out.squeeze(0).transpose(0, 1).contiguous()


def accuracy(out, ref):
    import torch

    if not bool(torch.isfinite(out).all()):
        raise RuntimeError("Non-finite attention output")
    diff = out.float() - ref.float()
    return {
        "finite": True,
        "relative_l2": (diff.norm() / ref.float().norm().clamp_min(1e-12)).item(),
        "max_abs": diff.abs().max().item(),
        "rmse": diff.square().mean().sqrt().item(),
    }


def make_call(name, q, k, v, *, scope, repair_budget=0.0, preparation="auto"):
    """A zero-argument callable for one backend, and its metadata.

    Scope "attention" prepares FP8 inputs (and a V grouping, a repair prefix) before timing, so that a
    timed call is one attention launch; scope "quantize-attention" times the complete BF16-in call.  The
    VC baseline always reuses one grouping per shape, as VC-Attention does after its first denoising steps.
    """
    from .. import api, baselines, v_repair

    description = get_backend(name).description
    if name == "bf16":
        return (lambda: bf16_attention(q, k, v)), {"implementation": description}
    if name == "vc":
        grouped = baselines.prepare_vc(q, k, v)
        metadata = {"implementation": description, "mid_window_blocks": None}
        if scope == "attention":
            return (lambda: baselines.attention_vc(grouped, output_shape=q.shape)), metadata
        return (lambda: baselines.attention_vc(
            baselines.prepare_vc(q, k, v, permutation=grouped.permutation, check_permutation=False),
            output_shape=q.shape)), metadata
    metadata = {"implementation": description, "mid_window_blocks": 4}
    if repair_budget > 0:
        selected = round(repair_budget * q.shape[-3])
        metadata.update(repair_budget=repair_budget, selected_tokens_per_head=selected,
                        repair_tokens_per_head=(selected + 127) // 128 * 128)
        if selected:
            if scope == "attention":
                repaired = v_repair.prepare_v_repair(q, k, v, budget=repair_budget)
                return (lambda: v_repair.attention_v_repair(repaired)), metadata
            return (lambda: v_repair.attention_v_repair(v_repair.prepare_v_repair(q, k, v, budget=repair_budget))), metadata
    if scope == "quantize-attention":
        return (lambda: api.attention(q, k, v, preparation=preparation)), metadata
    # V goes into the kernel's packed layout before timing, so that a timed call is one attention launch:
    # by the fused preparation where the public call would take it, else by packing the generic result.
    if api._fused_preparation_eligible(q, k, v, version=api.DEFAULT_VERSION, mode="expcast", causal=False, return_lse=False):
        prepared = api.prepare_fp8_fused(q, k, v)
    else:
        import dataclasses

        from ..quantization import pack_v

        prepared = api.prepare_fp8(q, k, v)
        if prepared.v.ndim == 3:
            prepared = dataclasses.replace(prepared, v=pack_v(prepared.v), v_prepacked=True)
    return (lambda: api.attention_fp8(prepared)), metadata


def time_calls(fn, repeats):
    """Milliseconds per call over `repeats` back-to-back calls, CUDA events on the current stream."""
    import torch

    first, last = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    first.record()
    for _ in range(repeats):
        fn()
    last.record()
    last.synchronize()
    return first.elapsed_time(last) / repeats


def vc_grouping_times(q, k, v, samples=5):
    """Complete VC calls with a fresh and with a reused grouping, interleaved; their difference is the
    k-means cost that a caller amortises over the steps that reuse a grouping."""
    from .. import baselines

    grouping = baselines.prepare_vc(q, k, v).permutation
    variants = {
        "fresh_grouping": lambda: baselines.attention_vc(baselines.prepare_vc(q, k, v), output_shape=q.shape),
        "reused_grouping": lambda: baselines.attention_vc(
            baselines.prepare_vc(q, k, v, permutation=grouping, check_permutation=False), output_shape=q.shape),
    }
    times = {name: [] for name in variants}
    for _ in range(samples):
        for name, call in variants.items():
            times[name].append(time_calls(call, 1))
    return times


def build_parser():
    parser = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    parser.add_argument("--shapes", nargs="+", default=["4096x7x128"])
    parser.add_argument("--preset", choices=["video", "smoke"])
    parser.add_argument("--backends", nargs="+", choices=list(BACKENDS), default=list(DEFAULT_BACKENDS))
    parser.add_argument("--baseline", choices=list(BACKENDS), default=DEFAULT_BASELINE)
    parser.add_argument("--scope", choices=["attention", "quantize-attention"], default="attention")
    parser.add_argument("--repair-budget", type=float, default=0.0,
                        help="Optional Open-VC V repair fraction per head; long single sequence only")
    parser.add_argument("--preparation", choices=["auto", "unfused", "fused"], default="auto",
                        help="Open-VC preparation for quantize-attention scope without V repair")
    parser.add_argument("--timing", choices=["events", "graph"], default="events")
    parser.add_argument("--rounds", type=int, default=12)
    parser.add_argument("--repeats", type=int, default=10)
    parser.add_argument("--warm-calls", type=int, default=6)
    parser.add_argument("--warm-seconds", type=float, default=3.0)
    parser.add_argument("--seed", type=int, default=20260928)
    parser.add_argument("--device", type=int, default=0)
    parser.add_argument("--input", type=pathlib.Path, help="Optional tensor-only .pt mapping with q/k/v; never uploaded")
    parser.add_argument("--allow-shared-gpu", action="store_true", help="Disable PID guard; marks results non-isolated")
    parser.add_argument("--output", type=pathlib.Path, default=pathlib.Path("results/benchmark.json"))
    return parser


def validated_shapes(args, parser):
    """Argument rules of the reference's command line; returns the list of (S, H, 128)."""
    if min(args.rounds, args.repeats) < 1 or args.warm_calls < 0 or args.warm_seconds < 0 or not math.isfinite(args.warm_seconds):
        parser.error("Rounds/repeats must be positive; warmup must be nonnegative")
    if len(set(args.backends)) != len(args.backends):
        parser.error("Duplicate backend names")
    if args.baseline not in args.backends:
        parser.error("The named baseline must be included in --backends")
    if not 0.0 <= args.repair_budget < 1.0:
        parser.error("--repair-budget must be finite and in [0, 1)")
    if args.repair_budget and CANDIDATE not in args.backends:
        parser.error(f"--repair-budget requires the {CANDIDATE} backend")
    if args.preparation != "auto" and (args.scope != "quantize-attention" or args.repair_budget or CANDIDATE not in args.backends):
        parser.error(f"--preparation requires quantize-attention scope with {CANDIDATE} and no repair")
    if args.device < 0:
        parser.error("--device must be a nonnegative visible CUDA device index")
    texts = {"video": VIDEO_SHAPES, "smoke": SMOKE_SHAPES}.get(args.preset, args.shapes)
    try:
        shapes = [parse_shape(text) for text in texts]
    except ValueError as exc:
        parser.error(str(exc))
    if args.repair_budget and any(s < 32768 for s, _, _ in shapes):
        parser.error("--repair-budget requires sequence lengths >= 32768")
    if "vc" in args.backends and any(s < 128 for s, _, _ in shapes):
        parser.error("The vc backend requires sequence lengths >= 128")
    return shapes


def _installed_versions():
    versions = {}
    for package in ("open-vc-attn", "torch", "triton", "nvidia-cutlass-dsl", "quack-kernels", "flash-attn-4", "cuda-python"):
        try:
            versions[package] = importlib.metadata.version(package)
        except importlib.metadata.PackageNotFoundError:
            versions[package] = "not installed as a distribution"
    return versions


def _inputs_for(shape, args, captured):
    import torch

    s, h, d = shape
    torch.manual_seed(args.seed + s + h)
    if captured is None:
        return [torch.randn(s, h, d, device="cuda", dtype=torch.bfloat16) for _ in range(3)]
    if any(tuple(captured[x].shape) != shape for x in "qkv"):
        raise ValueError("Capture must match the exact requested shape; no implicit slicing")
    return [captured[x].to(device="cuda", dtype=torch.bfloat16).contiguous() for x in "qkv"]


def _measure_shape(shape, args, guard, captured, save):
    """One entry of report["shapes"]; `save` is called after every round."""
    import torch

    s, h, d = shape
    q, k, v = _inputs_for(shape, args, captured)
    ref = bf16_attention(q, k, v).clone()
    row = {"shape": [s, h, d], "accuracy_reference": "bf16", "accuracy": {}, "backend_metadata": {}, "orders": [],
           "timings": {}, "speedups": {}}
    yield row
    calls = {}
    for name in args.backends:
        guard.check()
        call, row["backend_metadata"][name] = make_call(name, q, k, v, scope=args.scope, repair_budget=args.repair_budget,
                                                        preparation=args.preparation)
        row["accuracy"][name] = accuracy(call(), ref)
        if name == "vc":
            row["vc_complete_call_events_ms"] = vc_grouping_times(q, k, v)
        torch.cuda.synchronize()
        deadline = time.monotonic() + args.warm_seconds
        while time.monotonic() < deadline:
            call()
            torch.cuda.synchronize()
        calls[name] = call
        print(f"READY {s}x{h}x{d} {name}", flush=True)
    del ref
    graphs, keep = {}, {}
    timed = calls
    if args.timing == "graph":
        for name, fn in calls.items():
            side = torch.cuda.Stream()
            side.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(side):
                for _ in range(3):
                    fn()
            torch.cuda.current_stream().wait_stream(side)
            graphs[name] = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graphs[name]):
                keep[name] = fn()
        timed = {name: graph.replay for name, graph in graphs.items()}
    samples = {name: [] for name in timed}
    shuffle = random.Random(args.seed + s + h)
    for index in range(args.rounds):
        order = list(timed)
        shuffle.shuffle(order)
        row["orders"].append(order)
        for name in order:
            guard.check()
            for _ in range(args.warm_calls):
                timed[name]()
            samples[name].append(time_calls(timed[name], args.repeats))
            guard.check()
        row["timings"] = {name: summarize(values) for name, values in samples.items()}
        row["speedups"] = {name: speedup(samples[args.baseline], values) for name, values in samples.items()}
        print(f"ROUND {s}x{h} {index + 1}/{args.rounds}", flush=True)
        save()
    torch.cuda.synchronize()
    del timed, graphs, keep, calls, q, k, v
    gc.collect()
    torch.cuda.empty_cache()


def main(argv=None):
    parser = build_parser()
    args = parser.parse_args(argv)
    shapes = validated_shapes(args, parser)
    import torch

    if not torch.cuda.is_available():
        parser.error("CUDA unavailable; install CUDA-enabled PyTorch and build libovc.so")
    torch.cuda.set_device(args.device)
    torch.set_grad_enabled(False)
    guard = GpuGuard(args.device, enabled=not args.allow_shared_gpu)
    report = {
        "schema_version": 1,
        "started_at_utc": _utc_now(),
        "source_provenance": provenance(),
        "device_configuration_start": guard.device_state(),
        "status": "running",
        "baseline": args.baseline,
        "scope": args.scope,
        "timing": args.timing,
        "fp8_default_quantization": "Q/K per-block128; V per-head; E4M3 absmax/448",
        "backends": {name: BACKENDS[name].description for name in args.backends},
        "v_packing_included": args.scope == "quantize-attention",
        "input_kind": "local_capture" if args.input else "synthetic",
        "seed": args.seed,
        "versions": _installed_versions(),
        "gpu": torch.cuda.get_device_name(),
        "capability": list(torch.cuda.get_device_capability()),
        "cuda_runtime": torch.version.cuda,
        "isolation_checked": guard.enabled,
        "settings": {key: value for key, value in vars(args).items() if key not in ("input", "output")},
        "shapes": [],
    }

    def save():
        args.output.parent.mkdir(parents=True, exist_ok=True)
        scratch = args.output.with_suffix(".tmp")
        scratch.write_text(json.dumps(report, indent=2) + "\n")
        scratch.replace(args.output)

    try:
        guard.check()
        captured = None
        if args.input:
            captured = torch.load(args.input, map_location="cpu", weights_only=True)
            if not isinstance(captured, dict) or any(not isinstance(captured.get(x), torch.Tensor) for x in "qkv"):
                raise ValueError("--input requires a tensor-only q/k/v mapping")
            report["input_sha256"] = _file_digest(args.input)
        for shape in shapes:
            steps = _measure_shape(shape, args, guard, captured, save)
            report["shapes"].append(next(steps))  # the row exists in the record before it is filled
            for _ in steps:
                pass
        report["device_configuration_end"] = guard.device_state()
        report["completed_at_utc"] = _utc_now()
        report["status"] = "complete"
        report["ownership_checks"] = guard.samples
    except BaseException as exc:
        report["status"] = "invalid"
        report["failure_type"] = type(exc).__name__  # no message: it could carry local paths
        raise
    finally:
        save()
    from .report import render

    print(render(report))
    print(f"Saved {args.output}", flush=True)


if __name__ == "__main__":
    main()
