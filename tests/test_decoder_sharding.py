"""Tensor-parallel sharding of the decoder weights (host logic), checked on the CPU: the sharded
model with the all-reduce emulated as a sum gives the unsharded model's logits."""
import numpy as np
import pytest

from nncase_b200 import decoder as D
from nncase_b200.lib import NncbError
from oracle import decoder as OD


def test_two_way_sharding_reproduces_the_unsharded_step():
    cfg = D.DecoderConfig(layers=2, hidden=256, q_heads=4, kv_heads=2, inter=512, vocab=1000, max_pos=128)
    w = D.make_weights(cfg, 11)
    cos, sin = D.rope_tables(cfg)
    rng = np.random.default_rng(5)
    B, pages = 4, 16
    table = rng.permutation(pages)[: B * 3].astype(np.int32).reshape(B, 3)
    pos = np.array([0, 5, 16, 33], np.int32)
    ids = rng.integers(0, cfg.vocab, B).astype(np.int32)
    full = OD.Decoder(cfg, w, cos, sin, pages)
    k0 = [rng.normal(0, 1, p.shape).astype(np.float16) for p in full.k_pools]
    v0 = [rng.normal(0, 1, p.shape).astype(np.float16) for p in full.v_pools]
    for li in range(cfg.layers):
        full.k_pools[li][...], full.v_pools[li][...] = k0[li], v0[li]
    want = full.step(ids, pos, table).astype(np.float32)
    world = 2
    sh = [D.shard_weights(cfg, w, world, r) for r in range(world)]
    kp = [[k0[li][:, r:r + 1].copy() for li in range(cfg.layers)] for r in range(world)]  # one kv head per rank
    vp = [[v0[li][:, r:r + 1].copy() for li in range(cfg.layers)] for r in range(world)]
    got = OD.tp_step(cfg, sh, cos, sin, kp, vp, ids, pos, table).astype(np.float32)
    rng_ = float(want.max() - want.min())
    assert np.abs(got - want).max() <= 5e-3 * rng_
    # every weight element lands on exactly one rank
    for name in ("qkv", "gate_up", "lm_head"):
        rows = sum((s["layers"][0][name][0].shape[0] if name != "lm_head" else s["lm_head"][0].shape[0]) for s in sh)
        ref_rows = w["layers"][0][name][0].shape[0] if name != "lm_head" else w["lm_head"][0].shape[0]
        assert rows == ref_rows
    assert sum(s["layers"][0]["o"][0].shape[1] for s in sh) == w["layers"][0]["o"][0].shape[1]


@pytest.mark.parametrize("world", [4, 8])
def test_sharding_beyond_the_kv_heads(world):
    """More ranks than kv heads: kv heads are shared by several ranks, the query-head groups are padded with zero
    heads (3 -> 4 per group here) and the MLP width per rank is rounded up to the MatMul's K granule with zero
    channels; the summed partials still reproduce the unsharded step."""
    cfg = D.DecoderConfig(layers=2, hidden=256, q_heads=6, kv_heads=2, inter=320, vocab=1000, max_pos=128)
    w = D.make_weights(cfg, 12)
    cos, sin = D.rope_tables(cfg)
    rng = np.random.default_rng(6)
    B, pages = 3, 12
    table = rng.permutation(pages)[: B * 3].astype(np.int32).reshape(B, 3)
    pos = np.array([0, 17, 40], np.int32)
    ids = rng.integers(0, cfg.vocab, B).astype(np.int32)
    full = OD.Decoder(cfg, w, cos, sin, pages)
    k0 = [rng.normal(0, 1, p.shape).astype(np.float16) for p in full.k_pools]
    v0 = [rng.normal(0, 1, p.shape).astype(np.float16) for p in full.v_pools]
    for li in range(cfg.layers):
        full.k_pools[li][...], full.v_pools[li][...] = k0[li], v0[li]
    want = full.step(ids, pos, table).astype(np.float32)
    plan = D.shard_plan(cfg, world)
    assert plan["hkv"] == 1 and plan["rep"] == world // 2 and plan["hq"] * plan["rep"] == plan["gpad"] >= 3
    assert plan["inter_pad"] % 64 == 0 and plan["inter_pad"] * world >= cfg.inter
    sh = [D.shard_weights(cfg, w, world, r) for r in range(world)]
    heads = [D.rank_kv_heads(cfg, world, r) for r in range(world)]
    assert sorted(set(h for hs in heads for h in hs)) == [0, 1] and all(len(hs) == 1 for hs in heads)
    kp = [[k0[li][:, heads[r]].copy() for li in range(cfg.layers)] for r in range(world)]
    vp = [[v0[li][:, heads[r]].copy() for li in range(cfg.layers)] for r in range(world)]
    got = OD.tp_step(cfg, sh, cos, sin, kp, vp, ids, pos, table).astype(np.float32)
    assert np.abs(got - want).max() <= 5e-3 * float(want.max() - want.min())
    # every real q head appears on exactly one rank: the o-projection columns that are not padding add up
    nonzero_cols = sum(int((s_["layers"][0]["o"][0] != 0).any(axis=0).sum()) for s_ in sh)
    assert nonzero_cols <= cfg.q_heads * cfg.head_dim
    assert sum(s_["lm_head"][0].shape[0] for s_ in sh) == cfg.vocab


def test_qwen2_shape_plans():
    cfg = D.DecoderConfig()
    assert {k: D.shard_plan(cfg, 2)[k] for k in ("hq", "hkv", "rep", "inter_pad")} == dict(hq=7, hkv=1, rep=1, inter_pad=2432)
    assert {k: D.shard_plan(cfg, 4)[k] for k in ("hq", "hkv", "rep", "inter_pad")} == dict(hq=4, hkv=1, rep=2, inter_pad=1216)
    assert {k: D.shard_plan(cfg, 8)[k] for k in ("hq", "hkv", "rep", "inter_pad")} == dict(hq=2, hkv=1, rep=4, inter_pad=640)


def test_indivisible_degree_is_rejected():
    cfg = D.DecoderConfig(layers=1, hidden=256, q_heads=4, kv_heads=2, inter=512, vocab=1000)
    w = D.make_weights(cfg, 1)
    with pytest.raises(NncbError):
        D.shard_weights(cfg, w, 3, 0)  # 3 neither divides nor is a multiple of the 2 kv heads


def _gloo_rank(rank, world, port, out_q):
    """One CPU rank of a world-4 decode step: numpy kernels, torch.distributed (gloo) all-reduce and all-gather."""
    import os

    import torch
    import torch.distributed as dist
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        cfg = D.DecoderConfig(layers=2, hidden=256, q_heads=6, kv_heads=2, inter=320, vocab=1000, max_pos=128)
        w = D.make_weights(cfg, 12)
        cos, sin = D.rope_tables(cfg)
        rng = np.random.default_rng(6)
        B, pages = 3, 12
        table = rng.permutation(pages)[: B * 3].astype(np.int32).reshape(B, 3)
        pos = np.array([0, 17, 40], np.int32)
        ids = rng.integers(0, cfg.vocab, B).astype(np.int32)
        shape = (pages, cfg.kv_heads, cfg.page, cfg.head_dim)
        k0 = [rng.normal(0, 1, shape).astype(np.float16) for _ in range(cfg.layers)]
        v0 = [rng.normal(0, 1, shape).astype(np.float16) for _ in range(cfg.layers)]
        heads = D.rank_kv_heads(cfg, world, rank)
        kp = [k[:, heads].copy() for k in k0]
        vp = [v[:, heads].copy() for v in v0]

        def all_reduce(a):
            t = torch.from_numpy(np.ascontiguousarray(a))
            dist.all_reduce(t)
            return t.numpy()

        local = OD.rank_step(cfg, D.shard_weights(cfg, w, world, rank), cos, sin, kp, vp, ids, pos, table, all_reduce)
        parts = [torch.empty(local.shape, dtype=torch.float16) for _ in range(world)]
        dist.all_gather(parts, torch.from_numpy(np.ascontiguousarray(local)))
        if rank == 0:
            full = OD.Decoder(cfg, w, cos, sin, pages)
            for li in range(cfg.layers):
                full.k_pools[li][...], full.v_pools[li][...] = k0[li], v0[li]
            want = full.step(ids, pos, table).astype(np.float32)
            got = torch.cat(parts, 1).float().numpy()
            out_q.put(float(np.abs(got - want).max() / (want.max() - want.min())))
        dist.barrier()
    finally:
        dist.destroy_process_group()


def test_world_four_over_gloo():
    """Four CPU processes, real collectives: the sharded step with shared kv heads and padded groups."""
    import socket

    import torch.multiprocessing as mp
    with socket.socket() as s_:
        s_.bind(("127.0.0.1", 0))
        port = s_.getsockname()[1]
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    procs = [ctx.Process(target=_gloo_rank, args=(r, 4, port, q)) for r in range(4)]
    for p in procs:
        p.start()
    err = q.get(timeout=240)
    for p in procs:
        p.join(timeout=60)
        assert p.exitcode == 0
    assert err <= 5e-3
