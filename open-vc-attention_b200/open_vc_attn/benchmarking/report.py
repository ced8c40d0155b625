"""Markdown table from a completed benchmark record (schema version 1); imports nothing from CUDA.

Entry point, checks and table layout of `open-vc-attn-report` of the reference
(src/open_vc_attn/benchmarking/report.py), so that records of either engine render side by side.
"""

import argparse
import json
import pathlib

from .backends import CANDIDATE
from .measurement import summarize


def _require(condition, message):
    if not condition:
        raise ValueError(message)


def _medians(row, names, rounds):
    timings = row.get("timings", {})
    _require(set(timings) == set(names), "Measured backend sets differ between shapes")
    result = {}
    for name in names:
        samples = timings[name].get("samples_ms", [])
        _require(rounds is None or len(samples) == rounds, "Incomplete sample count in a completed report")
        result[name] = summarize(samples)["median_ms"]
    return result


def _table_row(row, names, medians, baseline, candidate):
    accuracy = row.get("accuracy", {}).get(candidate, {})
    _require(accuracy.get("finite") is True, "Candidate did not record finite output")
    error = accuracy.get("relative_l2")
    cells = [" x ".join(map(str, row["shape"]))]
    cells += [f"{medians[name]:.3f}" for name in names]
    cells.append(f"{medians[baseline] / medians[candidate]:.3f}x")
    cells.append(f"{100 * error:.3f}%" if isinstance(error, (int, float)) else "unavailable")
    return "| " + " | ".join(cells) + " |"


def render(report, *, baseline=None, candidate=None):
    _require(report.get("schema_version") == 1 and report.get("status") == "complete",
             "Expected a complete standalone benchmark report (schema_version=1)")
    shapes = report.get("shapes") or []
    _require(shapes, "Report contains no measured shapes")
    names = list(shapes[0].get("timings", {}))
    _require(names, "Report contains no measured backends")
    baseline = baseline or report.get("baseline")
    if candidate is None:
        candidate = CANDIDATE if CANDIDATE in names else names[-1]
    _require(baseline in names and candidate in names, f"Both {baseline!r} and {candidate!r} must be measured backends")
    settings = report.get("settings", {})
    head = "| S x H x D | " + " | ".join(f"{name} ms" for name in names)
    lines = [
        f"GPU: {report.get('gpu', 'unknown')}; scope: {report.get('scope')}; timer: {report.get('timing')}; "
        f"isolation checked: {report.get('isolation_checked')}",
        f"Speedup = {baseline} median / {candidate} median. Approximate attention; errors are relative to the BF16 reference.",
        f"Open-VC repair budget: {settings.get('repair_budget', 0.0)}; preparation policy: {settings.get('preparation', 'auto')}",
        "",
        head + f" | {candidate} speedup | {candidate} rel L2 |",
        "|---|" + "---:|" * (len(names) + 2),
    ]
    for row in shapes:
        lines.append(_table_row(row, names, _medians(row, names, settings.get("rounds")), baseline, candidate))
    if report.get("isolation_checked") is not True:
        lines += ["", "Shared-GPU result: do not use as an isolated performance claim."]
    return "\n".join(lines)


def main(argv=None):
    parser = argparse.ArgumentParser(description=__doc__)
    parser.add_argument("result", type=pathlib.Path)
    parser.add_argument("--baseline", help="Choose any backend measured in this same run")
    parser.add_argument("--candidate", help=f"Defaults to {CANDIDATE} when present")
    args = parser.parse_args(argv)
    try:
        print(render(json.loads(args.result.read_text()), baseline=args.baseline, candidate=args.candidate))
    except (OSError, ValueError, KeyError, TypeError) as exc:
        parser.error(str(exc))


if __name__ == "__main__":
    main()
