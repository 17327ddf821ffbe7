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


def test_indivisible_degree_is_rejected():
    cfg = D.DecoderConfig(layers=1, hidden=256, q_heads=4, kv_heads=2, inter=512, vocab=1000)
    w = D.make_weights(cfg, 1)
    with pytest.raises(NncbError):
        D.shard_weights(cfg, w, 4, 0)  # 2 kv heads do not split four ways
