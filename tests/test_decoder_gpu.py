"""Decode-step operators and the whole decode step against the numpy restatement (f16 storage, f32
math; tolerance relative to each output's range)."""
import ctypes as C

import numpy as np
import pytest
import torch

from nncase_b200 import decoder as D
from nncase_b200 import lib as L
from oracle import decoder as OD

pytestmark = pytest.mark.gpu


def close(got, want, tol=1e-3):
    got, want = np.asarray(got, np.float32), np.asarray(want, np.float32)
    rng = max(float(want.max() - want.min()), 1e-6)
    err = float(np.abs(got - want).max())
    assert err <= tol * rng, f"max abs err {err} vs range {rng}"


@pytest.fixture(params=[0, 2], ids=["mma_sync", "tcgen05"])
def matmul_form(ctx, request):
    """Both forms of the w8a16 MatMul: CUDA-core-fed mma.sync, and tcgen05 with the accumulator in TMEM (forced for
    every shape that fits; by default it takes more than 32 tokens on matrices of 128 K weights or more). The
    shapes below cover both launch forms, K split over clusters of 2, 4 and 8 CTAs, a cluster rank without K blocks,
    ragged token and channel counts."""
    ctx.set_option("matmul.tensor_core", request.param)
    yield request.param
    ctx.set_option("matmul.tensor_core", 1)


@pytest.mark.parametrize("m,n,k", [(64, 1152, 896), (64, 896, 4864), (5, 1000, 128), (1, 16, 64), (33, 9728, 896), (64, 4224, 896),
                                   (64, 19208, 128), (37, 19204, 192)])
def test_gemv_w8a16(ctx, matmul_form, m, n, k):
    rng = np.random.default_rng(m + n)
    x = rng.normal(0, 1, (m, k)).astype(np.float16)
    wq, s = D.quantize_per_channel_i8(rng.normal(0, 0.02, (n, k)).astype(np.float32))
    bias = rng.normal(0, 0.1, n).astype(np.float16)
    res = rng.normal(0, 1, (m, n)).astype(np.float16)
    t = lambda a: torch.from_numpy(a).cuda()
    xd, wd, sd, bd, rd = t(x), t(wq), t(s), t(bias), t(res)
    y = torch.empty((m, n), dtype=torch.float16, device="cuda")
    L.check(ctx._lib.nncb_gemv_w8a16(ctx._h, xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), bd.data_ptr(), rd.data_ptr(),
                                     y.data_ptr(), m, n, k))
    close(y.cpu().numpy(), OD.gemv_w8a16(x, wq, s, bias, res))
    L.check(ctx._lib.nncb_gemv_w8a16(ctx._h, xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), None, None, y.data_ptr(), m, n, k))
    close(y.cpu().numpy(), OD.gemv_w8a16(x, wq, s))


@pytest.mark.parametrize("m,inter,k", [(64, 4864, 896), (64, 2432, 896), (5, 24, 128), (33, 1024, 1280), (64, 64, 4864)])
def test_gemv_with_swiglu_epilogue(ctx, matmul_form, m, inter, k):
    """The gate/up MatMul with SwiGLU in its epilogue, on interleaved gate/up rows: bit-identical to the
    MatMul followed by swiglu (the same f16 gate/up values meet the same f32 formula)."""
    rng = np.random.default_rng(m + inter + k)
    x = rng.normal(0, 1, (m, k)).astype(np.float16)
    wq, s = D.quantize_per_channel_i8(rng.normal(0, 0.02, (2 * inter, k)).astype(np.float32))
    wi, si = D.interleave_gate_up(wq, s)
    t = lambda a: torch.from_numpy(a).cuda()
    xd, wid, sid, wd, sd = t(x), t(wi), t(si), t(wq), t(s)
    y = torch.empty((m, inter), dtype=torch.float16, device="cuda")
    L.check(ctx._lib.nncb_gemv_w8a16_swiglu(ctx._h, xd.data_ptr(), wid.data_ptr(), sid.data_ptr(), None, y.data_ptr(), m,
                                            2 * inter, k))
    gu = torch.empty((m, 2 * inter), dtype=torch.float16, device="cuda")
    L.check(ctx._lib.nncb_gemv_w8a16(ctx._h, xd.data_ptr(), wd.data_ptr(), sd.data_ptr(), None, None, gu.data_ptr(), m, 2 * inter, k))
    act = torch.empty_like(y)
    L.check(ctx._lib.nncb_swiglu_f16(ctx._h, gu.data_ptr(), act.data_ptr(), m, inter))
    assert torch.equal(y, act)
    close(y.cpu().numpy(), OD.swiglu(OD.gemv_w8a16(x, wq, s), inter))
    # a second call gives the same bits (k = 4864 is split over a cluster)
    y2 = torch.empty_like(y)
    L.check(ctx._lib.nncb_gemv_w8a16_swiglu(ctx._h, xd.data_ptr(), wid.data_ptr(), sid.data_ptr(), None, y2.data_ptr(), m,
                                            2 * inter, k))
    assert torch.equal(y, y2)


def test_matmul_chain_with_and_without_launch_overlap(ctx):
    """RMSNorm -> gate/up MatMul with SwiGLU -> down MatMul with residual, 64 tokens: the tensor-core MatMuls are
    launched as programmatic dependents of the kernel before them (their set-up and first weight loads run beside
    it); the chain gives the same bits with plain launches."""
    rng = np.random.default_rng(11)
    m, d, inter = 64, 896, 4864
    x = rng.normal(0, 1, (m, d)).astype(np.float16)
    g = rng.normal(1, 0.1, d).astype(np.float16)
    wgu0, sgu0 = D.quantize_per_channel_i8(rng.normal(0, 0.02, (2 * inter, d)).astype(np.float32))
    wgu, sgu = D.interleave_gate_up(wgu0, sgu0)
    wdn, sdn = D.quantize_per_channel_i8(rng.normal(0, 0.02, (d, inter)).astype(np.float32))
    t = lambda a: torch.from_numpy(a).cuda()
    gd, wgud, sgud, wdnd, sdnd = t(g), t(wgu), t(sgu), t(wdn), t(sdn)
    outs = []
    for overlap in (1, 0, 1):
        ctx.set_option("launch.overlap", overlap)
        xd = t(x)
        h = torch.empty_like(xd)
        act = torch.empty((m, inter), dtype=torch.float16, device="cuda")
        y = torch.empty_like(xd)
        for _ in range(3):  # back to back: each launch finds the one before still running
            L.check(ctx._lib.nncb_add_rmsnorm_f16(ctx._h, xd.data_ptr(), None, gd.data_ptr(), h.data_ptr(), m, d, 1e-6))
            L.check(ctx._lib.nncb_gemv_w8a16_swiglu(ctx._h, h.data_ptr(), wgud.data_ptr(), sgud.data_ptr(), None, act.data_ptr(),
                                                    m, 2 * inter, d))
            L.check(ctx._lib.nncb_gemv_w8a16(ctx._h, act.data_ptr(), wdnd.data_ptr(), sdnd.data_ptr(), None, xd.data_ptr(),
                                             y.data_ptr(), m, d, inter))
        ctx.synchronize()
        outs.append(y.cpu())
    ctx.set_option("launch.overlap", 1)
    assert torch.equal(outs[0], outs[1]) and torch.equal(outs[0], outs[2])
    _, hh = OD.add_rmsnorm(x, None, g, 1e-6)
    close(outs[0].numpy(), OD.gemv_w8a16(OD.swiglu(OD.gemv_w8a16(hh, wgu0, sgu0), inter), wdn, sdn, None, x))


def _peer_case(ctx, world, rank, rows, cols, seed):
    """Buffers of a fake tensor-parallel group inside one process: every 'rank' is a local buffer."""
    rng = np.random.default_rng(seed)
    parts = [rng.normal(0, 1, (rows, cols)).astype(np.float16) for _ in range(world)]
    x = rng.normal(0, 1, (rows, cols)).astype(np.float16)
    g = rng.normal(1, 0.1, cols).astype(np.float16)
    t = lambda a: torch.from_numpy(a).cuda()
    parts_d = [t(p) for p in parts]
    flags_d = [torch.zeros(32, dtype=torch.int32, device="cuda") for _ in range(world)]
    arr = C.c_void_p * world
    return dict(parts=parts, x=x, g=g, parts_d=parts_d, flags_d=flags_d, xd=t(x), gd=t(g), h=torch.empty((rows, cols), dtype=torch.float16, device="cuda"),
                parts_arr=arr(*[p.data_ptr() for p in parts_d]), flags_arr=arr(*[f.data_ptr() for f in flags_d]), world=world, rank=rank)


def _peer_call(ctx, c, slot):
    return ctx._lib.nncb_peer_allreduce_add_rmsnorm_f16(ctx._h, c["xd"].data_ptr(), c["parts_arr"], c["flags_arr"], c["world"], c["rank"],
                                                        slot, c["gd"].data_ptr(), c["h"].data_ptr(), c["x"].shape[0], c["x"].shape[1],
                                                        1e-6)


@pytest.mark.parametrize("world,rank", [(2, 0), (4, 2), (8, 7)])
def test_peer_allreduce_add_rmsnorm_with_flags_already_set(ctx, world, rank):
    """The exchange kernel of tensor-parallel decode on one GPU: the other ranks' partials are local buffers and their
    'ready' flags for the first two sequence numbers are set by the host beforehand, so nothing waits. The result is
    the rank-ordered f32 sum rounded to f16, added to x, then RMSNorm; the second launch on the slot uses sequence
    number 2 and the kernel has told every peer (flag blocks of the other ranks) about both."""
    c = _peer_case(ctx, world, rank, 7, 896, 40 + world)
    own_flags = np.zeros(32, np.int32)
    own_flags[8 * 1:8 * 1 + world] = 2  # slot 1: every peer is already at sequence number 2
    c["flags_d"][rank].copy_(torch.from_numpy(own_flags))
    x = c["x"]
    for launch in (1, 2):
        L.check(_peer_call(ctx, c, 1))
        ctx.synchronize()
        delta = sum(p.astype(np.float32) for p in c["parts"]).astype(np.float16)
        x, want_h = OD.add_rmsnorm(x, delta, c["g"], 1e-6)
        assert np.array_equal(c["xd"].cpu().numpy(), x)
        close(c["h"].cpu().numpy(), want_h)
        for p in range(world):
            f = c["flags_d"][p].cpu().numpy()
            if p != rank:
                assert f[8 * 1 + rank] == launch  # told by this rank
        mine = c["flags_d"][rank].cpu().numpy()
        assert mine[16 + 1] == launch and mine[18 + 1] == 0
    ctx.check_status()


def test_peer_allreduce_wait_runs_out(ctx):
    """A peer that never reports: the wait gives up after the limit, the launch returns, the status word says so once,
    later launches on the context do not wait again until the status has been read, and the context still works."""
    c = _peer_case(ctx, 2, 0, 4, 896, 77)
    ctx.set_option("peer_wait_limit_us", 2000)
    try:
        L.check(_peer_call(ctx, c, 0))
        L.check(_peer_call(ctx, c, 0))
        ctx.synchronize()
        with pytest.raises(L.NncbError) as e:
            ctx.check_status()
        assert e.value.code == -110  # -ETIMEDOUT
        ctx.check_status()
    finally:
        ctx.set_option("peer_wait_limit_us", 30000000)
    y = torch.empty((4, 896), dtype=torch.float16, device="cuda")
    L.check(ctx._lib.nncb_add_rmsnorm_f16(ctx._h, c["xd"].data_ptr(), None, c["gd"].data_ptr(), y.data_ptr(), 4, 896, 1e-6))
    ctx.check_status()


def test_gemv_rejects_unsupported(ctx):
    z = torch.zeros(1 << 16, dtype=torch.float16, device="cuda")
    w = torch.zeros(1 << 16, dtype=torch.int8, device="cuda")
    assert ctx._lib.nncb_gemv_w8a16(ctx._h, z.data_ptr(), w.data_ptr(), z.data_ptr(), None, None, z.data_ptr(), 65, 16, 64) == -38
    assert ctx._lib.nncb_gemv_w8a16(ctx._h, z.data_ptr(), w.data_ptr(), z.data_ptr(), None, None, z.data_ptr(), 4, 16, 70) == -38


def test_add_rmsnorm_swiglu_embedding(ctx):
    rng = np.random.default_rng(9)
    x = rng.normal(0, 1, (7, 896)).astype(np.float16)
    dl = rng.normal(0, 1, (7, 896)).astype(np.float16)
    w = (1 + rng.normal(0, 0.02, 896)).astype(np.float16)
    xd, dd, wd = torch.from_numpy(x).cuda(), torch.from_numpy(dl).cuda(), torch.from_numpy(w).cuda()
    h = torch.empty_like(xd)
    L.check(ctx._lib.nncb_add_rmsnorm_f16(ctx._h, xd.data_ptr(), dd.data_ptr(), wd.data_ptr(), h.data_ptr(), 7, 896, 1e-6))
    xn, hn = OD.add_rmsnorm(x, dl, w, 1e-6)
    assert np.array_equal(xd.cpu().numpy(), xn)  # the residual add itself is exact in f16
    close(h.cpu().numpy(), hn)
    gu = rng.normal(0, 2, (7, 2 * 608)).astype(np.float16)
    gd = torch.from_numpy(gu).cuda()
    out = torch.empty((7, 608), dtype=torch.float16, device="cuda")
    L.check(ctx._lib.nncb_swiglu_f16(ctx._h, gd.data_ptr(), out.data_ptr(), 7, 608))
    close(out.cpu().numpy(), OD.swiglu(gu, 608))
    table = rng.normal(0, 1, (50, 896)).astype(np.float16)
    ids = np.array([3, 49, 0, 17], np.int32)
    td, idd = torch.from_numpy(table).cuda(), torch.from_numpy(ids).cuda()
    e = torch.empty((4, 896), dtype=torch.float16, device="cuda")
    L.check(ctx._lib.nncb_embedding_f16(ctx._h, td.data_ptr(), idd.data_ptr(), e.data_ptr(), 4, 896, 50))
    assert np.array_equal(e.cpu().numpy(), table[ids])


def _run_steps(ctx, cfg, weights, B, start_lens, steps, seed):
    """Prefill the caches with random K/V, then decode `steps` tokens on both sides."""
    rng = np.random.default_rng(seed)
    max_pages = (max(start_lens) + steps + cfg.page - 1) // cfg.page
    num_pages = B * max_pages + 2
    table = rng.permutation(num_pages)[: B * max_pages].astype(np.int32).reshape(B, max_pages)
    cos, sin = D.rope_tables(cfg)
    ref = OD.Decoder(cfg, weights, cos, sin, num_pages)
    dec = D.Decoder(cfg, weights, B, num_pages, ctx=ctx)
    for li in range(cfg.layers):
        k = rng.normal(0, 1, ref.k_pools[li].shape).astype(np.float16)
        v = rng.normal(0, 1, ref.v_pools[li].shape).astype(np.float16)
        ref.k_pools[li][...], ref.v_pools[li][...] = k, v
        dec.layers[li]["k_pool"].copy_(torch.from_numpy(k))
        dec.layers[li]["v_pool"].copy_(torch.from_numpy(v))
    pos = np.asarray(start_lens, np.int32)
    td = torch.from_numpy(table).cuda()
    outs = []
    for s in range(steps):
        ids = rng.integers(0, cfg.vocab, B).astype(np.int32)
        want = ref.step(ids, pos, table)
        got = dec.step(torch.from_numpy(ids).cuda(), torch.from_numpy(pos).cuda(), td)
        ctx.check_status()
        outs.append((got.cpu().numpy(), want))
        pos = pos + 1
    return outs, dec, ref


def test_decode_steps_small_model(ctx):
    cfg = D.DecoderConfig(layers=3, hidden=256, q_heads=4, kv_heads=2, inter=512, vocab=1000, max_pos=256)
    weights = D.make_weights(cfg, 7)
    outs, dec, ref = _run_steps(ctx, cfg, weights, 5, [0, 1, 15, 16, 40], 3, 1)
    for got, want in outs:
        close(got, want, 5e-3)
    # the appended K/V pages agree bit for bit up to f16 rounding of the rope
    for li in range(cfg.layers):
        close(dec.layers[li]["k_pool"].cpu().numpy(), ref.k_pools[li], 2e-3)


def test_decode_step_qwen2_shape_two_layers(ctx):
    """Full widths of the Qwen2-0.5B shape (hidden 896, 14/2 heads, inter 4864), two layers, a small
    vocabulary, batch 64."""
    cfg = D.DecoderConfig(layers=2, vocab=2048, max_pos=512)
    weights = D.make_weights(cfg, 8)
    outs, _, _ = _run_steps(ctx, cfg, weights, 64, list(np.random.default_rng(2).integers(1, 300, 64)), 1, 2)
    close(outs[0][0], outs[0][1], 5e-3)
