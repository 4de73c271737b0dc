"""The allocation-free head entry point, q35_lm_head_argmax_static.

It exists for hosts that are not allowed to allocate device memory (a plugin inside a runtime
that owns the device heap; a serving loop with a frozen pool), so it takes no engine and keeps
its scratch in a fixed device array of the library.  The test calls it through the C-ABI twice in
a row, with different inputs, against the engine-backed entry point (q35_op_lm_head) under the
tolerance every head test here uses: the two entries sum their dot products in different orders
(weight-streaming kernel vs tensor-core tiles), so they must agree wherever the f32 top-2 margin of
the row exceeds 1e-2, and below that each must pick a token whose logit is within 1e-2 of the best.
The second call also shows that whatever the first call left in the shared scratch does not leak
into the result; small ragged vocabularies right after the full-size calls change the stride over
the shared array and exercise the clamped last CTA.
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
        ref = x.float() @ E.float().t()                       # f32 logits of the same bf16 operands
        top2 = ref.topk(2, dim=-1)
        margin = top2.values[:, 0] - top2.values[:, 1]
        for r in range(rows):
            best = int(top2.indices[r, 0])
            for name, tok in (("static", int(got[r])), ("engine", int(want[r]))):
                if margin[r] > 1e-2:
                    assert tok == best, f"call {call} row {r}: {name} entry picked {tok}, f32 argmax {best} at margin {float(margin[r])}"
                else:
                    assert float(top2.values[r, 0] - ref[r, tok]) <= 1e-2, f"call {call} row {r}: {name} entry far from the top"
    # all-zero rows: every logit ties at 0 and the lowest id must win, also after the calls above
    z = torch.zeros((2, 1024), dtype=torch.bfloat16, device="cuda")
    assert pkg.engine.lm_head_argmax_static(z, E).tolist() == [0, 0]
    eng.close()


@pytest.mark.parametrize("vocab", [8, 40, 72])
def test_static_head_small_ragged_vocabularies(pkg, weights, vocab):
    """Vocabularies that are not a multiple of the 32 rows a CTA owns (last CTA clamped, tail filtered out
    of the argmax) and row counts between 1 and 16, called right after a full-size call so that the stride
    of the partials over the shared array changes; an all-equal row must give id 0 and a row whose maximum
    sits in the ragged tail must find it."""
    pkg.build_lib.build()
    E_full = weights["model.language_model.embed_tokens.weight"].cuda()
    gen = torch.Generator().manual_seed(vocab)
    pkg.engine.lm_head_argmax_static((torch.randn((16, 1024), generator=gen)).to(torch.bfloat16).cuda(), E_full)
    E = (torch.randn((vocab, 1024), generator=gen) * 0.05).to(torch.bfloat16).cuda()
    for rows in (1, 8, 16):
        x = torch.randn((rows, 1024), generator=gen).to(torch.bfloat16).cuda()
        x[0] = 0                                               # all logits equal: the lowest id wins
        if rows > 1:
            x[1] = E[vocab - 1] * 40                           # the maximum sits in the last (ragged) rows
        got = pkg.engine.lm_head_argmax_static(x, E)
        ref = x.float() @ E.float().t()
        top2 = ref.topk(2, dim=-1)
        assert int(got[0]) == 0
        if rows > 1:
            assert int(got[1]) == vocab - 1
        for r in range(rows):
            if float(top2.values[r, 0] - top2.values[r, 1]) > 1e-2:
                assert int(got[r]) == int(top2.indices[r, 0]), (vocab, rows, r)


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
