"""The allocation-free head entry point, q35_lm_head_argmax_static.

It exists for hosts that are not allowed to allocate device memory (a plugin inside a runtime
that owns the device heap; a serving loop with a frozen pool), so it takes no engine and keeps
its scratch in a fixed device array of the library.  The test calls it through the C-ABI twice in
a row, with different inputs, and requires the same tokens as the engine-backed entry point
(q35_op_lm_head); tokens are integers, so the comparison is exact.  The second call also shows
that whatever the first call left in the shared scratch does not leak into the result.
This file sorts last on purpose: a run that stops at the first failure has then already run
every other test.
"""
from __future__ import annotations

import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu


def test_static_head_matches_engine_head_twice(pkg, weights):
    pkg.build_lib.build()
    lib = pkg.load_library()
    E = weights["model.language_model.embed_tokens.weight"].cuda()
    eng = pkg.Engine(weights, max_rows=32)
    gen = torch.Generator().manual_seed(123)
    for call, rows in enumerate((16, 3)):
        x = (torch.randn((rows, 1024), generator=gen) * 2).to(torch.bfloat16).cuda()
        want, _ = eng.op_lm_head(x)
        got = torch.full((rows,), -7, dtype=torch.int32, device="cuda")
        rc = lib.q35_lm_head_argmax_static(C.c_void_p(x.data_ptr()), C.c_void_p(E.data_ptr()), E.shape[0],
                                           rows, C.c_void_p(got.data_ptr()),
                                           C.c_void_p(torch.cuda.current_stream().cuda_stream))
        assert rc == 0, lib.q35_last_error()
        torch.cuda.synchronize()
        assert torch.equal(got, want), f"call {call}"
    # all-zero rows: every logit ties at 0 and the lowest id must win, also after the calls above
    z = torch.zeros((2, 1024), dtype=torch.bfloat16, device="cuda")
    assert pkg.engine.lm_head_argmax_static(z, E).tolist() == [0, 0]
    eng.close()


def test_static_head_refuses_sizes_beyond_its_scratch(pkg):
    pkg.build_lib.build()
    lib = pkg.load_library()
    x = torch.zeros((17, 1024), dtype=torch.bfloat16, device="cuda")
    E = torch.zeros((64, 1024), dtype=torch.bfloat16, device="cuda")
    out = torch.zeros(17, dtype=torch.int32, device="cuda")
    args = (C.c_void_p(x.data_ptr()), C.c_void_p(E.data_ptr()))
    assert lib.q35_lm_head_argmax_static(*args, 64, 17, C.c_void_p(out.data_ptr()), None) == 3
    assert b"at most 16" in lib.q35_last_error()
    assert lib.q35_lm_head_argmax_static(*args, 262152, 1, C.c_void_p(out.data_ptr()), None) == 3
    assert lib.q35_lm_head_argmax_static(*args, 60, 1, C.c_void_p(out.data_ptr()), None) == 3
