"""The paired benchmark harness end to end on a GPU: record layout (schema version 1), accuracy fields, both
timers, both scopes and the repair option, then the report rendered from the written file."""

import json

import pytest

pytestmark = pytest.mark.gpu

TOP_LEVEL = {
    "schema_version", "started_at_utc", "completed_at_utc", "source_provenance", "device_configuration_start",
    "device_configuration_end", "status", "baseline", "scope", "timing", "fp8_default_quantization", "backends",
    "v_packing_included", "input_kind", "seed", "versions", "gpu", "capability", "cuda_runtime", "isolation_checked",
    "settings", "shapes", "ownership_checks",
}


def _run(tmp_path, *extra):
    from open_vc_attn.benchmarking import runner

    out = tmp_path / "record.json"
    runner.main(["--rounds", "2", "--repeats", "2", "--warm-calls", "1", "--warm-seconds", "0", "--allow-shared-gpu",
                 "--output", str(out), *extra])
    return json.loads(out.read_text()), out


def test_smoke_preset_writes_a_complete_record(tmp_path, capsys):
    from open_vc_attn.benchmarking import report

    record, path = _run(tmp_path, "--preset", "smoke")
    assert TOP_LEVEL <= set(record) and record["schema_version"] == 1 and record["status"] == "complete"
    assert record["isolation_checked"] is False and record["scope"] == "attention" and record["timing"] == "events"
    assert record["v_packing_included"] is False and record["input_kind"] == "synthetic"
    assert set(record["backends"]) == {"bf16", "vc", "open-vc"}
    assert record["source_provenance"]["native_library_sha256"] and "api.py" in record["source_provenance"]["source_sha256"]
    assert [row["shape"] for row in record["shapes"]] == [[129, 2, 128], [1024, 7, 128]]
    for row in record["shapes"]:
        assert len(row["orders"]) == 2 and all(sorted(order) == ["bf16", "open-vc", "vc"] for order in row["orders"])
        for name in ("bf16", "vc", "open-vc"):
            assert len(row["timings"][name]["samples_ms"]) == 2 and row["timings"][name]["median_ms"] > 0
            assert len(row["speedups"][name]["paired_ratios"]) == 2
            assert row["accuracy"][name]["finite"] is True
        assert row["accuracy"]["bf16"]["relative_l2"] == 0.0
        assert row["accuracy"]["open-vc"]["relative_l2"] < 0.10 and row["accuracy"]["vc"]["relative_l2"] < 0.10
        assert row["backend_metadata"]["open-vc"]["mid_window_blocks"] == 4
        assert row["backend_metadata"]["vc"]["mid_window_blocks"] is None
        assert set(row["vc_complete_call_events_ms"]) == {"fresh_grouping", "reused_grouping"}
    text = report.render(record)
    assert "| 1024 x 7 x 128 |" in text and "Shared-GPU result" in text
    report.main([str(path), "--candidate", "vc"])
    assert "vc speedup" in capsys.readouterr().out


def test_graph_timer_complete_call_scope_and_repair(tmp_path):
    record, _ = _run(tmp_path, "--shapes", "32768x1x128", "--backends", "bf16", "open-vc", "--timing", "graph",
                     "--scope", "quantize-attention", "--repair-budget", "0.005")
    assert record["status"] == "complete" and record["timing"] == "graph" and record["v_packing_included"] is True
    row = record["shapes"][0]
    meta = row["backend_metadata"]["open-vc"]
    assert meta["selected_tokens_per_head"] == 164 and meta["repair_tokens_per_head"] == 256
    assert row["accuracy"]["open-vc"]["relative_l2"] < 0.10
    assert len(row["timings"]["open-vc"]["samples_ms"]) == 2
