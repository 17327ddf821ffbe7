"""The allocation-free paged-attention entry point against the regular one.

Some callers of the library are not allowed to allocate device memory once the model is loaded
(a runtime that plans all buffers up front, a loop with a fixed memory budget, code inside a
stream capture), so they cannot supply the workspace the regular entry point needs.
`nncb_paged_attention_decode_noalloc` keeps that scratch in a fixed array inside the library.
This test calls it through the C ABI twice in a row -- the second call with shorter, ragged
contexts, so stale partials of the first call would show -- and compares each result with the
regular entry point within the tolerance of the attention tests. It lives in a file that pytest
collects last; it passes alone in a fresh process and after the other tests.
"""
import ctypes as C

import numpy as np
import pytest
import torch

from nncase_b200 import lib as L

pytestmark = pytest.mark.gpu
TOL = 1e-3  # of the output range, as in tests/test_attention_gpu.py


def _inputs(seed, b, hq, hkv, lens, d=64, page=16):
    g = torch.Generator(device="cuda").manual_seed(seed)
    max_pages = (max(lens) + page - 1) // page
    total = b * max_pages + 3
    k = torch.randn((total, hkv, page, d), device="cuda", generator=g, dtype=torch.float16)
    v = torch.randn((total, hkv, page, d), device="cuda", generator=g, dtype=torch.float16)
    q = torch.randn((b, hq, d), device="cuda", generator=g, dtype=torch.float16)
    table = torch.randperm(total, device="cuda", generator=g)[: b * max_pages].to(torch.int32).reshape(b, max_pages)
    return q, k, v, table.contiguous(), torch.tensor(lens, dtype=torch.int32, device="cuda")


def _noalloc(ctx, q, k, v, table, lens):
    b, hq, d = q.shape
    out = torch.empty_like(q)
    L.check(ctx._lib.nncb_paged_attention_decode_noalloc(
        ctx._h, q.data_ptr(), k.data_ptr(), v.data_ptr(), table.data_ptr(), lens.data_ptr(), out.data_ptr(), b, hq,
        k.shape[1], d, k.shape[2], table.shape[1], k.shape[0], C.c_float(1.0 / np.sqrt(d))))
    return out


def test_noalloc_matches_regular_entry_point_twice(ctx):
    ctx.use_current_stream()
    cases = [_inputs(11, 16, 14, 2, [2048] * 16),
             _inputs(12, 16, 14, 2, [1, 40, 700, 16, 333, 2047, 0, 512, 90, 1500, 33, 64, 1000, 7, 250, 1800])]
    for q, k, v, table, lens in cases:
        want = ctx.paged_attention_decode(q, k, v, table, lens).float()
        got = _noalloc(ctx, q, k, v, table, lens).float()
        torch.cuda.synchronize()
        rng = max(float(want.max() - want.min()), 1e-6)
        assert float((got - want).abs().max()) <= TOL * rng


def test_noalloc_rejects_problems_beyond_the_built_in_scratch(ctx):
    # The one-wave split policy never asks for more than about 625 KiB on a 148-SM part, so the limit is
    # reached through the library's split-count override: 64 x 16 heads x 8 splits x 264 bytes = 2112 KiB.
    ctx.set_option("attention.splits", 8)
    try:
        b, hq, hkv, pages = 64, 16, 2, 128
        q = torch.zeros((b, hq, 64), dtype=torch.float16, device="cuda")
        k = torch.zeros((4, hkv, 16, 64), dtype=torch.float16, device="cuda")
        table = torch.zeros((b, pages), dtype=torch.int32, device="cuda")
        lens = torch.ones(b, dtype=torch.int32, device="cuda")
        need = C.c_size_t()
        L.check(ctx._lib.nncb_paged_attention_workspace_size(ctx._h, b, hq, hkv, 64, 16, pages, C.byref(need)))
        assert need.value > (768 << 10), "the split policy changed: pick a shape that exceeds the built-in scratch"
        with pytest.raises(L.NncbError) as e:
            _noalloc(ctx, q, k, k, table, lens)
        assert e.value.code == -7 and "786432" in str(e.value)
        # the regular entry point takes the same problem with a caller-provided workspace
        out = ctx.paged_attention_decode(q, k, k, table, lens)
        assert out.shape == q.shape
    finally:
        ctx.set_option("attention.splits", 0)
