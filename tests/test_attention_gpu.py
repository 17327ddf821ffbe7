"""Paged-attention decode on the GPU against the numpy restatement: f32 math on f16 data,
max-abs error <= 1e-3 of the output range."""
import numpy as np
import pytest
import torch

from oracle import attention as OA

pytestmark = pytest.mark.gpu
TOL = 1e-3  # relative to the output range


def make_cache(seed, b, hq, hkv, ctx_lens, d=64, page=16, extra_pages=5):
    rng = np.random.default_rng(seed)
    max_pages = max(1, (max(ctx_lens) + page - 1) // page)
    total = b * max_pages + extra_pages
    k_pool = rng.normal(0, 1, (total, hkv, page, d)).astype(np.float16)
    v_pool = rng.normal(0, 1, (total, hkv, page, d)).astype(np.float16)
    perm = rng.permutation(total)[: b * max_pages].astype(np.int32)  # random block-table permutation
    table = perm.reshape(b, max_pages)
    q = rng.normal(0, 1, (b, hq, d)).astype(np.float16)
    return q, k_pool, v_pool, table, np.asarray(ctx_lens, np.int32)


def check(ctx, case):
    q, k, v, table, lens = case
    want = OA.paged_attention_decode(q, k, v, table, lens).astype(np.float32)
    got = ctx.paged_attention_decode(torch.from_numpy(q), torch.from_numpy(k), torch.from_numpy(v),
                                     torch.from_numpy(table), torch.from_numpy(lens)).cpu().numpy().astype(np.float32)
    rng_ = max(float(want.max() - want.min()), 1e-6)
    err = float(np.abs(got - want).max())
    assert err <= TOL * rng_, f"max abs err {err} vs range {rng_}"


@pytest.mark.parametrize("hq,hkv", [(14, 2), (8, 8), (8, 1), (4, 2)])
def test_ragged_contexts(ctx, hq, hkv):
    lens = [1, 15, 16, 17, 33, 100, 511, 512, 513, 700, 0, 2048]
    check(ctx, make_cache(5, len(lens), hq, hkv, lens))


@pytest.mark.parametrize("warps", [4, 8])
def test_both_cta_widths(ctx, warps):
    """The four-warp (context splits, merge kernel) and the eight-warp (one CTA per sequence and kv head)
    forms of the kernel on the same ragged batch."""
    ctx.set_option("attention.warps", warps)
    try:
        lens = [1, 15, 16, 17, 33, 100, 511, 512, 513, 700, 0, 2048, 31, 32, 1000, 255]
        check(ctx, make_cache(15, len(lens), 14, 2, lens))
    finally:
        ctx.set_option("attention.warps", 0)


def test_many_sequences_take_the_wide_form(ctx):
    """80 sequences x 2 kv heads fill the SMs without context splits (eight-warp CTAs, no merge)."""
    rng = np.random.default_rng(16)
    lens = [int(v) for v in rng.integers(0, 400, 80)]
    check(ctx, make_cache(16, len(lens), 14, 2, lens))


def test_single_token_and_empty(ctx):
    check(ctx, make_cache(6, 3, 14, 2, [0, 1, 1]))


def test_qwen2_shape_small_batch(ctx):
    """Qwen2-0.5B shape (14 query / 2 kv heads, head_dim 64, 16-token pages) at context 2048."""
    check(ctx, make_cache(7, 8, 14, 2, [2048] * 8))


def test_large_scores_are_stable(ctx):
    q, k, v, table, lens = make_cache(8, 2, 14, 2, [300, 64])
    q = (q.astype(np.float32) * 6).astype(np.float16)  # sharp softmax
    check(ctx, (q, k, v, table, lens))


def test_softmax_rows_sum_to_one_full_size(ctx):
    """Config size (batch 64, context 2048): with V = 1 everywhere every output must be 1 -- a
    property of softmax that needs no oracle."""
    b, hq, hkv, n = 64, 14, 2, 2048
    g = torch.Generator(device="cuda").manual_seed(1)
    pages = b * n // 16
    k = torch.randn((pages, hkv, 16, 64), device="cuda", generator=g, dtype=torch.float16)
    v = torch.ones((pages, hkv, 16, 64), device="cuda", dtype=torch.float16)
    q = torch.randn((b, hq, 64), device="cuda", generator=g, dtype=torch.float16)
    table = torch.randperm(pages, device="cuda", generator=g).to(torch.int32).reshape(b, n // 16)
    lens = torch.full((b,), n, dtype=torch.int32, device="cuda")
    out = ctx.paged_attention_decode(q, k, v, table, lens)
    assert float((out.float() - 1.0).abs().max()) <= 1e-3


def test_unsupported_shapes_are_rejected(ctx):
    from nncase_b200.lib import NncbError
    q = torch.zeros((1, 4, 128), dtype=torch.float16)
    k = torch.zeros((2, 4, 16, 128), dtype=torch.float16)
    with pytest.raises(NncbError) as e:
        ctx.paged_attention_decode(q, k, k, torch.zeros((1, 2), dtype=torch.int32), torch.ones(1, dtype=torch.int32))
    assert e.value.code == -38


@pytest.mark.parametrize("positions", [
    [0, 14, 15, 16, 17, 100, 511, 512, 2047],                 # few sequences: context splits and the merge kernel
    None,                                                     # 80 sequences: one CTA per sequence and kv head
])
def test_rope_and_append_inside_the_attention_launch(ctx, positions):
    """nncb_paged_attention_decode_rope against nncb_rope_kv_append_f16 followed by nncb_paged_attention_decode on
    the same inputs: the output and both pools must come out bit-identical (first token, page boundaries, last
    position of the block table)."""
    import ctypes as C

    from nncase_b200 import lib as L
    rng = np.random.default_rng(23)
    if positions is None:
        positions = [int(v) for v in rng.integers(0, 400, 80)]
    hq, hkv, d = 14, 2, 64
    b = len(positions)
    lens = [p + 1 for p in positions]
    _, k_pool, v_pool, table, lens_np = make_cache(23, b, hq, hkv, lens)
    max_pos = 2048
    qkv = rng.normal(0, 1, (b, (hq + 2 * hkv) * d)).astype(np.float16)
    inv = 1.0 / (10000.0 ** (np.arange(32, dtype=np.float64) / 32.0))
    ang = np.arange(max_pos, dtype=np.float64)[:, None] * inv[None, :]
    cos, sin = np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)
    t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
    qkv_d, cos_d, sin_d, pos_d, tab_d, len_d = t(qkv), t(cos), t(sin), t(np.asarray(positions, np.int32)), t(table), t(lens_np)
    lib, h = ctx._lib, ctx._h
    need = C.c_size_t()
    L.check(lib.nncb_paged_attention_workspace_size(h, b, hq, hkv, d, 16, table.shape[1], C.byref(need)))
    ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device="cuda")
    scale = C.c_float(0.125)
    # two launches
    k1, v1 = t(k_pool), t(v_pool)
    q1 = torch.empty((b, hq, d), dtype=torch.float16, device="cuda")
    out1 = torch.empty_like(q1)
    L.check(lib.nncb_rope_kv_append_f16(h, qkv_d.data_ptr(), q1.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), pos_d.data_ptr(),
                                        tab_d.data_ptr(), k1.data_ptr(), v1.data_ptr(), b, hq, hkv, d, 16, table.shape[1], max_pos,
                                        k1.shape[0]))
    L.check(lib.nncb_paged_attention_decode(h, q1.data_ptr(), k1.data_ptr(), v1.data_ptr(), tab_d.data_ptr(), len_d.data_ptr(),
                                            out1.data_ptr(), b, hq, hkv, d, 16, table.shape[1], k1.shape[0], scale, ws.data_ptr(),
                                            ws.numel()))
    # one launch
    k2, v2 = t(k_pool), t(v_pool)
    out2 = torch.empty_like(q1)
    L.check(lib.nncb_paged_attention_decode_rope(h, qkv_d.data_ptr(), cos_d.data_ptr(), sin_d.data_ptr(), pos_d.data_ptr(),
                                                 k2.data_ptr(), v2.data_ptr(), tab_d.data_ptr(), len_d.data_ptr(), out2.data_ptr(),
                                                 b, hq, hkv, d, 16, table.shape[1], max_pos, k2.shape[0], scale, ws.data_ptr(),
                                                 ws.numel()))
    ctx.synchronize()
    assert torch.equal(k1, k2) and torch.equal(v1, v2)
    assert not torch.equal(k1, t(k_pool))  # the append happened
    assert torch.equal(out1, out2)
    ctx.check_status()


def test_rope_inside_attention_flags_a_position_outside_the_context(ctx):
    """A position the context length does not cover, or outside the rotary table, appends nothing and sets the
    status word; the launch itself completes."""
    import ctypes as C

    from nncase_b200 import lib as L
    from nncase_b200.lib import NncbError
    hq, hkv, d = 14, 2, 64
    for positions, lens in (([40, 5], [41, 3]), ([5000, 3], [17, 4])):
        b = 2
        _, k_pool, v_pool, table, lens_np = make_cache(29, b, hq, hkv, [64, 64])
        lens_np = np.asarray(lens, np.int32)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).cuda()
        qkv = t(np.ones((b, (hq + 2 * hkv) * d), np.float16))
        cos, sin = t(np.ones((64, 32), np.float32)), t(np.zeros((64, 32), np.float32))
        k2, v2, out = t(k_pool), t(v_pool), torch.empty((b, hq, d), dtype=torch.float16, device="cuda")
        lib, h = ctx._lib, ctx._h
        need = C.c_size_t()
        L.check(lib.nncb_paged_attention_workspace_size(h, b, hq, hkv, d, 16, table.shape[1], C.byref(need)))
        ws = torch.empty(max(need.value, 16), dtype=torch.uint8, device="cuda")
        L.check(lib.nncb_paged_attention_decode_rope(h, qkv.data_ptr(), cos.data_ptr(), sin.data_ptr(),
                                                     t(np.asarray(positions, np.int32)).data_ptr(), k2.data_ptr(), v2.data_ptr(),
                                                     t(table).data_ptr(), t(lens_np).data_ptr(), out.data_ptr(), b, hq, hkv, d, 16,
                                                     table.shape[1], 64, k2.shape[0], C.c_float(0.125), ws.data_ptr(), ws.numel()))
        ctx.synchronize()
        with pytest.raises(NncbError):
            ctx.check_status()
