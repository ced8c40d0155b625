"""Paired benchmark harness with the record format of the reference's `open-vc-attn-bench` (schema version 1)."""
