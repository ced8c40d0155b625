"""The C-ABI library: it loads, exports everything include/ovc.h declares, and rejects bad
arguments before touching a GPU."""

import ctypes
import os
import re

import pytest

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


@pytest.fixture(scope="module")
def lib():
    import __graft_entry__

    __graft_entry__.build()
    from open_vc_attn import _lib

    return _lib.load()


def declared_functions():
    text = open(os.path.join(ROOT, "include", "ovc.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(ovc_[a-z0-9_]+)\s*\(", text)))


def test_header_declares_the_path():
    names = declared_functions()
    for needed in ("ovc_prepare_fused", "ovc_quantize_per_block", "ovc_quantize_per_head", "ovc_head_amax",
                   "ovc_pack_v", "ovc_repair_score", "ovc_repair_rows", "ovc_attention"):
        assert needed in names


def test_every_declared_symbol_is_exported_and_bound(lib):
    from open_vc_attn import _lib

    for name in declared_functions():
        assert hasattr(lib, name), name
        assert name in _lib.SIGNATURES, f"{name} has no ctypes signature"
    assert lib.ovc_version() >= 1
    assert lib.ovc_error_string(0) == b"ok"
    assert b"argument" in lib.ovc_error_string(-1)


def test_null_and_bad_arguments_are_rejected_without_a_gpu(lib):
    null = None
    bad = -1
    assert lib.ovc_quantize_per_block(null, 1, 1, 128, 1, null, null, 1, null) == bad
    assert lib.ovc_head_amax(null, 1, 1, 128, 1, null, null) == bad
    assert lib.ovc_quantize_per_head(null, 1, 1, 128, 1, null, null, null, null) == bad
    assert lib.ovc_prepare_fused(null, null, null, 1, 128, 1, null, null, null, null, null, null, null, null) == bad
    assert lib.ovc_pack_v(null, 1, 128, 1, null, null) == bad
    assert lib.ovc_repair_score(null, 1, 128, 1, null, null, null, null) == bad
    assert lib.ovc_repair_rows(null, null, null, 1, null, null, null, null, 1, 128, 128, 1, 1, null) == bad
    assert lib.ovc_attention(null, null, null, null, 1, null, null, null, 0, null, 1, 128, 128, 1, 0.1, 4, null, null) == bad
    # non-null but otherwise invalid: sizes, dtype, alignment, scale
    buf = ctypes.create_string_buffer(4096)
    p = ctypes.addressof(buf) // 16 * 16 + 16
    assert lib.ovc_quantize_per_block(p, 7, 1, 128, 1, p, p, 1, null) == bad          # dtype
    assert lib.ovc_quantize_per_block(p, 1, 1, 0, 1, p, p, 1, null) == bad            # S = 0
    assert lib.ovc_quantize_per_block(p, 1, 1, 300, 1, p, p, 2, null) == bad          # descale row too short
    assert lib.ovc_quantize_per_block(p + 2, 1, 1, 128, 1, p, p, 1, null) == bad      # misaligned input
    assert lib.ovc_attention(p, p, p, p, 1, p, p, null, 0, p, 1, 128, 128, 1, 0.0, 4, null, null) == bad   # scale
    assert lib.ovc_attention(p, p, p, p, 1, p, p, null, 0, p, 1, 128, 128, 1, float("nan"), 4, null, null) == bad
    assert lib.ovc_attention(p, p, p, p, 1, p, p, null, 128, p, 1, 128, 256, 1, 0.1, 4, null, null) == bad  # repair w/o kd
    assert lib.ovc_attention(p, p, p, p, 1, p, p, p, 100, p, 1, 128, 256, 1, 0.1, 4, null, null) == bad     # R % 128
    assert lib.ovc_attention(p, p, p, p, 0, p, p, null, 0, p, 1, 128, 128, 1, 0.1, 4, null, null) == bad    # q_blocks
    assert lib.ovc_attention(p, p, p, p, 1, p, p, null, 0, p, 1, 128, 128, 1, 0.1, -2, null, null) == bad   # window
    # extended attention entry, V-Smooth attention and preparation entries
    assert lib.ovc_attention_ex(null, null, null, null, 1, null, null, null, 0, null, null, 0, 1, 128, 128, 1, 0.1, -1, null, null) == bad
    assert lib.ovc_attention_ex(p, p, p, p, 1, p, p, null, 0, p, null, 1, 1, 128, 128, 1, 0.1, 4, null, null) == bad   # causal + window
    assert lib.ovc_attention_ex(p, p, p, p, 1, p, p, p, 128, p, null, 1, 1, 128, 256, 1, 0.1, -1, null, null) == bad   # causal + repair
    assert lib.ovc_attention_ex(p, p, p, p, 1, p, p, p, 128, p, null, 2, 1, 128, 256, 1, 0.1, -1, null, null) == bad   # unpacked V + repair
    assert lib.ovc_attention_ex(p, p, p, p, 1, p, p, null, 0, p, null, 4, 1, 128, 128, 1, 0.1, -1, null, null) == bad   # unknown flag
    assert lib.ovc_attention_vsmooth(p, p, p, p, null, p, p, p, 128, 128, 1, 0.1, -1, null, null) == bad                # no means
    assert lib.ovc_attention_vsmooth(p, p, p, p, p + 4, p, p, p, 128, 128, 1, 0.1, -1, null, null) == bad               # misaligned means
    assert lib.ovc_attention_vsmooth(p, p, p, p, p, p, null, p, 128, 128, 1, 0.1, -1, null, null) == bad                # no workspace
    assert lib.ovc_attention_vsmooth(p, p, p, p, p, p, p + 4, p, 128, 128, 1, 0.1, -1, null, null) == bad               # misaligned workspace
    # one 128-byte row per (head, channel) and group of 32 key blocks
    assert lib.ovc_attention_vsmooth_workspace(73397, 7) == 18 * 128 * 128 * 7
    assert lib.ovc_attention_vsmooth_workspace(128, 1) == 128 * 128
    assert lib.ovc_attention_vsmooth_workspace(0, 1) == 0
    assert lib.ovc_vs_assign(null, null, null, 128, 1, 8, null) == bad
    assert lib.ovc_vs_assign(p, p, p, 128, 1, 129, null) == bad            # more than 128 clusters
    assert lib.ovc_vs_assign(p, p, p, 4, 1, 8, null) == bad                # more clusters than tokens
    assert lib.ovc_vs_accumulate(p, p, null, p, 128, 1, 8, null) == bad
    assert lib.ovc_vs_update_centers(null, p, p, 1, 8, null) == bad
    assert lib.ovc_vs_block_stats(p, null, p, p, 128, 1, null) == bad
    assert lib.ovc_vs_block_write(p, p, p, p, p, p, null, p, p, 128, 1, null) == bad
    assert lib.ovc_vs_block_stats(p + 2, p, p, p, 128, 1, null) == bad           # misaligned V
    assert lib.ovc_vs_block_stats(p, p + 4, p, p, 128, 1, null) == bad           # misaligned permutation
    assert lib.ovc_vs_block_write(p, p + 8, p, p, p, p, p, p, p, 128, 1, null) == bad   # misaligned V
    assert lib.ovc_vs_block_write(p, p, p, p, p, p + 4, p, p, p, 128, 1, null) == bad   # misaligned K codes
    assert lib.ovc_vs_block_write(p, p, p, p, p, p, p + 2, p, p, 128, 1, null) == bad   # misaligned V codes
    assert lib.ovc_div_full(null, p, p, 4, null) == bad
    assert lib.ovc_div_full(p, p, p, 0, null) == bad
    assert lib.ovc_selftest_wait(null, 1000, p, null) == bad
    assert lib.ovc_selftest_wait(p, 0, p, null) == bad
    assert lib.ovc_cast_e4m3(p, 1, p, 12, null) == bad                     # not a multiple of 8
    assert lib.ovc_cast_e4m3(p, 9, p, 16, null) == bad                     # dtype
