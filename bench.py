"""Benchmark of the hot path: open_vc_attn.attention(q, k, v) at S=73397, H=56, D=128, BF16 input.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--config c3|c2|c4|c5]

A step is one complete call (FP8 preparation + ExpCast attention) over the rank's heads.  With N GPUs the
heads are split by head (7 per GPU at N=8 for the default workload) and every rank works on inputs resident
in its own HBM; there is no collective on the timed path.  Rank 0 prints one JSON line.

Workloads (`--config`; the default c3 is the one the headline metric is quoted on):
  c3  Q, K, V [73397, 56, 128] BF16, video-DiT-like structure           attention(q, k, v), packed path
  c2  Q, K, V [32768, 8, 128] BF16, i.i.d. N(0,1)                        attention(q, k, v), packed path
  c4  Q, K, V [4, 8191, 24, 128] FP16, i.i.d. N(0,1)                     attention(q, k, v), general batched path
  c5  Q, K [73397, 14, 128] BF16 N(0,1), V Student-t(3), budget 0.005    prepare_v_repair + attention_v_repair

`--impl reference` times the CPU restatement of the reference's arithmetic (oracle/) on the host cores over a
bounded sample of the same workload; the reference's own kernels cannot run without its pinned JIT toolchain
and are not part of this repository.

`--small SEQ HEADS` replaces the workload's sizes (for short profiler captures of the same call).
"""

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)
sys.path.insert(0, os.path.join(ROOT, "open-vc-attention_b200"))

D = 128
SEED = 20260928
METRIC = "attention throughput, 4*S^2*H*D FLOP model, complete call (FP8 prep + ExpCast attention)"

CONFIGS = {
    # name: batch, tokens, heads, dtype, value structure, call, our kernels launched per step
    "c3": dict(B=1, S=73397, H=56, dtype="bf16", values="video-DiT-like (4 outlier channels x8, LogNormal(0,0.3) token norms, V ~ N(mu_h,1))",
               call="attention", launches=4),
    "c2": dict(B=1, S=32768, H=8, dtype="bf16", values="i.i.d. N(0,1)", call="attention", launches=4),
    "c4": dict(B=4, S=8191, H=24, dtype="fp16", values="i.i.d. N(0,1)", call="attention", launches=5),
    "c5": dict(B=1, S=73397, H=14, dtype="bf16", values="Q,K i.i.d. N(0,1), V Student-t(3)", call="v_repair budget 0.005",
               launches=7),
}


def workload_label(name, cfg):
    shape = f"[{cfg['S']},{cfg['H']},{D}]" if cfg["B"] == 1 else f"[{cfg['B']},{cfg['S']},{cfg['H']},{D}]"
    return f"{name}: Q,K,V {shape} {cfg['dtype'].upper()} in, non-causal, {cfg['values']}, {cfg['call']}, heads sharded over the GPUs"


def config_entry(name, cfg, gpus):
    """The `config` object of the JSON line: identical for both arms of a comparison."""
    return {"workload": workload_label(name, cfg), "seed": SEED, "parallelism": f"heads{gpus}",
            "l2": "inputs (3 x S x H x 128 x 2 B per rank) exceed the 126 MB L2; nothing is flushed between steps"}


def flops(cfg, heads):
    return 4.0 * cfg["B"] * cfg["S"] * cfg["S"] * heads * D


def measured_peaks():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return json.load(f), "measured"
    return {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0, "bf16_tflops_sustained": 1400.0}, "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while the timed region runs."""

    FIELDS = ("clocks.sm,clocks.max.sm,power.draw,clocks_event_reasons.hw_slowdown,"
              "clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,"
              "clocks_event_reasons.sw_power_cap")

    def __init__(self, index):
        self.rows = []
        self.proc = None
        try:
            self.proc = subprocess.Popen(
                ["nvidia-smi", f"--query-gpu={self.FIELDS}", "--format=csv,noheader,nounits", "-lms", "200", "-i",
                 str(index)], stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
            self.thread = threading.Thread(target=self._read, daemon=True)
            self.thread.start()
        except OSError:
            self.proc = None

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 7:
                self.rows.append(parts)

    def stop(self):
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, peak, power = [], set(), None, []
        names = ("hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap")
        for row in self.rows:
            try:
                clocks.append(float(row[0]))
                peak = float(row[1])
                power.append(float(row[2]))
            except ValueError:
                continue
            for name, flag in zip(names, row[3:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": statistics.median(clocks) if clocks else None, "sm_max_mhz": peak,
                "power_w_max": max(power) if power else None, "samples": len(clocks), "reasons": sorted(reasons)}


def auto_group(heads):
    """Heads per streamed group.  What the stream cannot hide is the first group's copy in and the last group's
    copy out, so small groups win (measured at 56 heads on one GPU: 80 ms per call with groups of 2, 86 ms with
    groups of 8); below two heads a group no longer fills the GPU (287 CTAs per head on 148 SMs)."""
    return 2 if heads >= 2 else 1


def make_inputs(name, cfg, heads, first_head, device):
    """The workload's Q, K, V for heads [first_head, first_head + heads), generated on `device`."""
    import torch

    from open_vc_attn.synthetic import student_t_values, video_dit_qkv

    dtype = torch.bfloat16 if cfg["dtype"] == "bf16" else torch.float16
    s, b = cfg["S"], cfg["B"]
    if name == "c3":
        return video_dit_qkv(s, heads, seed=SEED, dtype=dtype, device=device, first_head=first_head)
    g = torch.Generator(device=device).manual_seed(SEED + 1000 * first_head + heads)
    shape = (s, heads, D) if b == 1 else (b, s, heads, D)
    q, k = [torch.randn(*shape, generator=g, device=device).to(dtype) for _ in range(2)]
    if name == "c5":
        v = student_t_values(s, heads, seed=SEED + 77 + first_head, dtype=dtype, device=device)
    else:
        v = torch.randn(*shape, generator=g, device=device).to(dtype)
    return q, k, v


def cpu_sample(name, cfg, m_blocks=None, threads=None):
    """Times the oracle on a bounded sample of the workload: one (batch, head), full FP8 preparation, a few
    256-row query blocks x all keys; extrapolated linearly to every query row."""
    import numpy as np
    import torch

    from oracle import attention as oatt
    from oracle import prep as oprep

    cores = threads or os.cpu_count() or 1
    torch.set_num_threads(cores)
    s = cfg["S"]
    all_blocks = (s + 255) // 256
    if m_blocks is None:
        m_blocks = tuple(range(0, all_blocks, max(1, all_blocks // 32)))[:32]
    q, k, v = [t.float().numpy() for t in make_inputs(name, dict(cfg, B=1), 1, 0, "cpu")]
    t0 = time.perf_counter()
    if name == "c5":
        prepared = oprep.prepare_repair(q, k, v, budget=0.005)
    else:
        prepared = oprep.prepare_fused(q, k, v)
    t_prep = time.perf_counter() - t0
    total = prepared.get("total", s)
    v8 = np.ascontiguousarray(prepared["v_packed"][:, :, :total].transpose(2, 0, 1))
    t0 = time.perf_counter()
    oatt.expcast_attention(prepared["q"], prepared["k"], v8, prepared["q_descale"][0], prepared["k_descale"][0],
                           prepared["v_descale"][0], rows=list(m_blocks),
                           repair_k_descale=None if prepared.get("repair_k_descale") is None else prepared["repair_k_descale"][0])
    t_attn = time.perf_counter() - t0
    rows = min(s, 256 * len(m_blocks))
    seconds_per_head = t_prep + t_attn * (s / rows)  # preparation covers the whole head, attention only `rows` rows
    value = flops(dict(cfg, B=1), 1) / seconds_per_head / 1e15
    sample = (f"oracle (numpy/BLAS) on 1 of {cfg['B'] * cfg['H']} (batch, head) pairs: full FP8 preparation ({t_prep:.2f} s) + "
              f"{rows} of {s} query rows x all keys ({t_attn:.2f} s), extrapolated linearly to S rows")
    return value, cores, sample


def run_reference(args, name, cfg, rank):
    if rank != 0:
        return
    values, cores, sample = [], 1, ""
    for step in range(args.warmup + args.steps):
        blocks = None if step >= args.warmup else (0,)
        value, cores, sample = cpu_sample(name, cfg, m_blocks=blocks)
        if step >= args.warmup:
            values.append(value)
    value = statistics.median(values)
    ms = flops(cfg, cfg["H"]) / (value * 1e15) * 1e3
    print(json.dumps({
        "impl": "reference", "metric": METRIC, "value": value, "unit": "PFLOP/s", "n_gpus": args.gpus,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True, "scaling": "strong",
        "vs_baseline": None, "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": config_entry(name, cfg, args.gpus),
        "cpu_baseline": {"value": value, "unit": "PFLOP/s", "cores": cores, "kind": "port", "sample": sample},
        "e2e": {"value": value, "unit": "PFLOP/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
        "gpu_launches": 0,
    }))


def conversion_rate(device, repeats=3):
    """Scores per second that the attention kernel's score conversion sustains on its own on this GPU right
    now (ovc_bench_conversion: every SM, eight conversion warps, scores in tensor memory, no exp instruction)."""
    import torch

    from open_vc_attn import _lib

    lib = _lib.load()
    sms = torch.cuda.get_device_properties(device).multi_processor_count
    tiles = 4096
    sink = torch.zeros(1, dtype=torch.int32, device=device)
    best = None
    for _ in range(repeats + 1):
        a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        a.record()
        _lib.check(lib.ovc_bench_conversion(sink.data_ptr(), sms, tiles, _lib.stream_pointer(device)), "ovc_bench_conversion")
        b.record()
        torch.cuda.synchronize()
        ms = a.elapsed_time(b)
        best = ms if best is None else min(best, ms)
    return sms * 256 * 128 * tiles / (best * 1e-3)


def main():
    parser = argparse.ArgumentParser()
    parser.add_argument("--gpus", type=int, default=1)
    parser.add_argument("--steps", type=int, default=10)
    parser.add_argument("--warmup", type=int, default=3)
    parser.add_argument("--impl", default="ours", choices=["ours", "reference"])
    parser.add_argument("--config", default="c3", choices=sorted(CONFIGS))
    parser.add_argument("--small", type=int, nargs=2, metavar=("SEQ", "HEADS"), default=None)
    parser.add_argument("--no-cpu-baseline", action="store_true")
    parser.add_argument("--no-e2e", action="store_true")
    parser.add_argument("--e2e-group", type=int, default=0,
                        help="heads per streamed group in the end-to-end leg (0: chosen from the head count)")
    args = parser.parse_args()
    rank = int(os.environ.get("RANK", "0"))
    local_rank = int(os.environ.get("LOCAL_RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    name, cfg = args.config, dict(CONFIGS[args.config])
    if args.small:
        cfg["S"], cfg["H"] = args.small
    if args.impl == "reference":
        run_reference(args, name, cfg, rank)
        return

    import torch
    import torch.distributed as dist

    import open_vc_attn
    from open_vc_attn import api, forward
    from open_vc_attn.sharding import head_range

    if not torch.cuda.is_available():
        raise SystemExit("bench.py needs a CUDA device: the product path has no CPU fallback")
    torch.cuda.set_device(local_rank)
    device = torch.device("cuda", local_rank)
    if world > 1:
        dist.init_process_group("nccl", device_id=device)
    s, h_total = cfg["S"], cfg["H"]
    h0, h1 = head_range(h_total, world, rank)
    heads = h1 - h0
    q, k, v = make_inputs(name, cfg, heads, h0, device)
    warmup = max(args.warmup, 3)
    packed = cfg["B"] == 1 and s >= 32768

    if name == "c5":
        def prepare():
            return open_vc_attn.prepare_v_repair(q, k, v, budget=0.005)

        attend = open_vc_attn.attention_v_repair
    else:
        def prepare():
            return api.prepare_fp8_fused(q, k, v) if packed else api.prepare_fp8(q, k, v)

        attend = api.attention_fp8

    def barrier():
        torch.cuda.synchronize()
        if world > 1:
            dist.barrier()
        torch.cuda.synchronize()

    def max_over_ranks(x):
        t = torch.tensor([x], dtype=torch.float64, device=device)
        if world > 1:
            dist.all_reduce(t, op=dist.ReduceOp.MAX)
        return float(t.item())

    # ---- resident inputs: complete call, and the attention kernel on its own ----
    for _ in range(warmup):
        out = attend(prepare())
    forward.check_status(device)
    sampler = ClockSampler(local_rank) if rank == 0 else None
    barrier()
    start, stop = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    marks = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(args.steps)]
    start.record()
    for a, b in marks:
        prepared = prepare()
        a.record()
        out = attend(prepared)
        b.record()
    stop.record()
    barrier()
    total_ms = max_over_ranks(start.elapsed_time(stop))
    kernel_ms = max_over_ranks(statistics.mean(a.elapsed_time(b) for a, b in marks))
    clocks = sampler.stop() if sampler else None
    forward.check_status(device)
    ms_per_step = total_ms / args.steps
    value = flops(cfg, h_total) / (ms_per_step * 1e-3) / 1e15
    expcast_rate = conversion_rate(device) if rank == 0 else None

    # ---- end to end: pinned host buffers in, result read back, every step ----
    e2e = None
    if not args.no_e2e:
        host_in = [torch.empty(t.shape, dtype=t.dtype, pin_memory=True).copy_(t) for t in (q, k, v)]
        host_out = torch.empty(out.shape, dtype=out.dtype, pin_memory=True)
        nbytes = q.numel() * q.element_size()
        del q, k, v, out, prepared
        torch.cuda.empty_cache()
        extra = {}
        if name in ("c2", "c3"):
            from open_vc_attn.streaming import HostAttention

            # The public call for host-resident tensors: head groups are copied in, computed and copied out
            # on three streams, so the PCIe transfers overlap the kernels of the neighbouring groups.
            group = args.e2e_group if args.e2e_group > 0 else auto_group(heads)
            streamed = HostAttention(s, heads, host_in[0].dtype, device, heads_per_group=group)
            extra["heads_per_group"] = group

            def e2e_step():
                streamed(*host_in, out=host_out)
        else:
            dev_in = [torch.empty(t.shape, dtype=t.dtype, device=device) for t in host_in]

            def e2e_step():
                nonlocal q, k, v
                for d, hbuf in zip(dev_in, host_in):
                    d.copy_(hbuf, non_blocking=True)
                q, k, v = dev_in
                host_out.copy_(attend(prepare()), non_blocking=True)

        e2e_step()
        barrier()
        t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        t0.record()
        for _ in range(args.steps):
            e2e_step()
        t1.record()
        barrier()
        e2e_ms = max_over_ranks(t0.elapsed_time(t1)) / args.steps
        forward.check_status(device)
        # The floor the host link puts under that number: the same bytes as plain contiguous pinned copies
        # (three tensors in on one stream, one out on another), all ranks at once, nothing computed.
        streamed = None
        torch.cuda.empty_cache()
        dev_in = [torch.empty(t.shape, dtype=t.dtype, device=device) for t in host_in]
        dev_out = torch.empty(host_out.shape, dtype=host_out.dtype, device=device)
        s_in, s_out = torch.cuda.Stream(), torch.cuda.Stream()

        def copy_step():
            with torch.cuda.stream(s_in):
                for d, hbuf in zip(dev_in, host_in):
                    d.copy_(hbuf, non_blocking=True)
            with torch.cuda.stream(s_out):
                host_out.copy_(dev_out, non_blocking=True)

        copy_step()
        barrier()
        c0, c1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        c0.record()
        s_in.wait_event(c0)
        s_out.wait_event(c0)
        for _ in range(args.steps):
            copy_step()
        torch.cuda.current_stream().wait_stream(s_in)
        torch.cuda.current_stream().wait_stream(s_out)
        c1.record()
        barrier()
        copy_ms = max_over_ranks(c0.elapsed_time(c1)) / args.steps
        e2e = {"value": flops(cfg, h_total) / (e2e_ms * 1e-3) / 1e15, "unit": "PFLOP/s", "ms_per_step": e2e_ms,
               "h2d_bytes_per_step": 3 * nbytes, "d2h_bytes_per_step": nbytes,
               "copy_only_ms_per_step": copy_ms, "copy_only_gbs_per_rank": 4 * nbytes / (copy_ms * 1e-3) / 1e9,
               "note": "copy_only: the step's bytes as contiguous pinned cudaMemcpyAsync copies, every rank at once, "
                       "nothing computed - the floor the host link sets for ms_per_step", **extra}

    if rank != 0:
        if world > 1:
            dist.destroy_process_group()
        return

    peaks, peak_kind = measured_peaks()
    fp8_peak = 2.0 * peaks["bf16_tflops_sustained"]
    achieved = flops(cfg, heads) / (kernel_ms * 1e-3) / 1e12
    scores_per_s = cfg["B"] * float(s) * s * heads / (kernel_ms * 1e-3)
    line = {
        "metric": METRIC, "value": value, "unit": "PFLOP/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
        "ms_per_step": ms_per_step, "higher_is_better": True, "scaling": "strong", "vs_baseline": None,
        "dtype": "fp8_e4m3 x fp8_e4m3 -> f32", "data": "synthetic",
        "config": config_entry(name, cfg, world), "heads_on_rank0": heads,
        "attention_kernel_ms": kernel_ms,
        "roofline": {"bound": "tensor", "achieved": achieved, "peak": fp8_peak, "unit": "TFLOP/s",
                     "frac": achieved / fp8_peak,
                     "traffic": None,
                     "traffic_note": "not measured in this run; an ncu capture at [73397,7,128] read + wrote 333.4 MB per "
                                     "launch against 328.8 MB algorithmic (profiles/)",
                     "peak_source": f"2 x bf16_tflops_sustained of {peak_kind} peaks (FP8 runs at twice the BF16 rate)",
                     "frac_of_nominal_4500": achieved / 4500.0,
                     "expcast": {"bound": "MUFU-free score conversion on the CUDA cores (ovc_bench_conversion, measured "
                                          "in this run at the clock of the moment)",
                                 "achieved": scores_per_s, "peak": expcast_rate, "unit": "scores/s",
                                 "frac": scores_per_s / expcast_rate}},
        "gpu_launches": cfg["launches"] * args.steps,
        "clocks": clocks,
    }
    if e2e is not None:
        line["e2e"] = e2e
    if world == 1 and not args.no_cpu_baseline:
        cpu_value, cores, sample = cpu_sample(name, cfg)
        line["cpu_baseline"] = {"value": cpu_value, "unit": "PFLOP/s", "cores": cores, "kind": "port", "sample": sample}
    print(json.dumps(line))
    if world > 1:
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
