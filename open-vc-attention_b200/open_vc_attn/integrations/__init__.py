"""Callers that sit on top of ``open_vc_attn.attention`` (framework adapters)."""
