"""CPU-only checks of the C-ABI boundary: the library loads, exports every symbol the header
declares, and rejects bad arguments with an error code before touching CUDA."""
from __future__ import annotations

import ctypes as C
import re
from pathlib import Path

import pytest

REPO = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def lib(pkg):
    pkg.build_lib.build()
    return pkg.load_library()


def declared_symbols():
    text = (REPO / "include" / "q35_engine.h").read_text()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(q35_[a-z0-9_]+)\s*\(", text)))


def test_header_symbols_exported(lib, pkg):
    names = declared_symbols()
    assert len(names) >= 25
    for n in names:
        assert hasattr(lib, n), f"{n} declared in include/q35_engine.h but not exported"
    assert set(pkg.engine.EXPORTS) == set(names)


def test_abi_version_and_error_string(lib):
    assert lib.q35_abi_version() == 1
    assert isinstance(lib.q35_last_error(), bytes)


def test_state_sizes_match_reference_arithmetic(pkg):
    # engine/state.h:83-120 / specification 08: 18,874,368 B of GDN state and 12,288 B per position
    s = pkg.LaneState.sizes(lanes=3, max_ctx=640)
    assert s["gdn_state_bytes"] == 18 * 16 * 128 * 128 * 4 == 18874368
    assert s["per_token_bytes"] == 12288
    assert s["kv_bytes"] == 12288 * 640
    assert s["conv_window_bytes"] == 18 * 3 * 6144 * 2
    assert s["total_bytes"] == 3 * (s["gdn_state_bytes"] + s["kv_bytes"] + s["conv_window_bytes"])


def test_bad_arguments_are_refused_without_cuda(lib):
    null = C.c_void_p(0)
    one = C.c_void_p(16)
    assert lib.q35_op_linear(null, null, null, 1, 8, 1024, null) == 1
    assert b"q35_op_linear" in lib.q35_last_error()
    assert lib.q35_op_linear(one, one, one, 1, 12, 1024, null) == 1      # N not a multiple of 8
    assert lib.q35_op_linear(one, one, one, 1, 8, 1000, null) == 1       # unsupported K
    assert lib.q35_op_linear(C.c_void_p(18), one, one, 1, 8, 1024, null) == 1   # misaligned
    assert lib.q35_engine_create(null, null, null, null) == 1
    assert lib.q35_decode_step(null, null, null, null, null, null, null) == 1
    assert lib.q35_prefill(null, null, null, 4, null, null, null) == 1
    assert lib.q35_mtp_verify(null, null, null, null, null, null, null, null, null) == 1
    assert lib.q35_state_sizes_of(0, 10, null) == 1
    assert lib.q35_op_gdn_step(one, one, one, one, one, one, one, one, 70000, 1, null) == 1
    assert lib.q35_state_export_lane(null, 0, null, null, null, null, 0, null) == 1
    # the entry points of depth-k rounds and of the bound resynchronisation
    assert lib.q35_mtp_state_reserve_depth(null, 2) == 1
    assert lib.q35_mtp_draft_k(null, null, null, null, null, 2, null, null) == 1
    assert lib.q35_mtp_verify_k(null, null, null, null, null, 2, null, null, null, null) == 1
    assert b"q35_mtp_verify_k" in lib.q35_last_error()
    assert lib.q35_state_sync_bound(null, null) == 1
    assert lib.q35_mtp_state_sync_bound(null, null) == 1
    assert lib.q35_state_note_advance(null, 1) == 1
    assert lib.q35_mtp_state_note_advance(null, 1) == 1
    assert lib.q35_lm_head_argmax_static(null, null, 248320, 1, null, null) == 1


def test_engine_requires_gpu(pkg):
    import torch
    if torch.cuda.is_available():
        pytest.skip("GPU present")
    with pytest.raises(RuntimeError, match="no CPU path"):
        pkg.Engine({}, max_rows=1)
