"""Decode step of the Qwen2-shaped transformer on the CPU, in numpy. TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the reference has no transformer operators (no RMSNorm, rotary embedding, SwiGLU,
weight-only-quantized MatMul, attention or KV cache; op list
src/Native/include/nncase/kernels/stackvm/tensor_ops.h:29-479). The operators are defined by
include/nncase_b200.h; this file restates them with f32 arithmetic (the reference's mat_mul
convention, reference/matmul.cpp:28-51) and f16 rounding wherever the CUDA path stores f16.
"""
import numpy as np

from . import attention as A

f16, f32 = np.float16, np.float32


def gemv_w8a16(x, wq, scale, bias=None, residual=None):
    y = (x.astype(f32) @ wq.astype(f32).T) * scale.astype(f32)[None, :]
    if bias is not None:
        y = y + bias.astype(f32)[None, :]
    if residual is not None:
        y = y + residual.astype(f32)
    return y.astype(f16)


def add_rmsnorm(x, delta, w, eps):
    """Returns (x_new f16, h f16)."""
    xf = x.astype(f32)
    if delta is not None:
        xf = (xf + delta.astype(f32)).astype(f16).astype(f32)
    ms = (xf * xf).sum(axis=1, dtype=f32) / f32(x.shape[1])
    h = xf * (f32(1.0) / np.sqrt(ms + f32(eps)))[:, None] * w.astype(f32)[None, :]
    return xf.astype(f16), h.astype(f16)


def rope(v, cos, sin, pos):
    """v [B, heads, 64] f16 -> rotated f16 ("rotate half")."""
    x = v.astype(f32)
    c, s = cos[pos][:, None, :], sin[pos][:, None, :]
    lo, hi = x[..., :32], x[..., 32:]
    return np.concatenate([lo * c - hi * s, hi * c + lo * s], axis=-1).astype(f16)


def swiglu(gu, inter):
    g, u = gu[:, :inter].astype(f32), gu[:, inter:].astype(f32)
    return (g / (f32(1.0) + np.exp(-g, dtype=f32)) * u).astype(f16)


class Decoder:
    def __init__(self, cfg, weights, cos, sin, num_pages):
        self.cfg, self.w, self.cos, self.sin = cfg, weights, cos, sin
        shape = (num_pages, cfg.kv_heads, cfg.page, cfg.head_dim)
        self.k_pools = [np.zeros(shape, f16) for _ in range(cfg.layers)]
        self.v_pools = [np.zeros(shape, f16) for _ in range(cfg.layers)]

    def step(self, token_ids, positions, block_table, trace=None):
        cfg = self.cfg
        B, D, Hq, Hkv = len(token_ids), cfg.head_dim, cfg.q_heads, cfg.kv_heads
        x = self.w["embed"][np.clip(token_ids, 0, cfg.vocab - 1)].copy()
        delta = None
        for li, lw in enumerate(self.w["layers"]):
            x, h = add_rmsnorm(x, delta, lw["ln1"], cfg.eps)
            qkv = gemv_w8a16(h, lw["qkv"][0], lw["qkv"][1], lw["qkv_bias"])
            q = rope(qkv[:, :Hq * D].reshape(B, Hq, D), self.cos, self.sin, positions)
            k = rope(qkv[:, Hq * D:(Hq + Hkv) * D].reshape(B, Hkv, D), self.cos, self.sin, positions)
            v = qkv[:, (Hq + Hkv) * D:].reshape(B, Hkv, D)
            for b in range(B):
                page = block_table[b, positions[b] // cfg.page]
                self.k_pools[li][page, :, positions[b] % cfg.page] = k[b]
                self.v_pools[li][page, :, positions[b] % cfg.page] = v[b]
            attn = A.paged_attention_decode(q, self.k_pools[li], self.v_pools[li], block_table, positions + 1)
            proj = gemv_w8a16(attn.reshape(B, Hq * D), lw["o"][0], lw["o"][1])
            x, h = add_rmsnorm(x, proj, lw["ln2"], cfg.eps)
            gu = gemv_w8a16(h, lw["gate_up"][0], lw["gate_up"][1])
            act = swiglu(gu, cfg.inter)
            delta = gemv_w8a16(act, lw["down"][0], lw["down"][1])
            if trace is not None:
                trace.append(dict(qkv=qkv, q=q, attn=attn, proj=proj, gu=gu, act=act, down=delta, x=x.copy()))
        x, h = add_rmsnorm(x, delta, self.w["ln_f"], cfg.eps)
        return gemv_w8a16(h, self.w["lm_head"][0], self.w["lm_head"][1])


def tp_step(cfg, sharded, cos, sin, k_pools, v_pools, token_ids, positions, block_table):
    """Tensor-parallel decode step emulated in one process: `sharded[r]` are rank r's weights
    (nncase_b200.decoder.shard_weights), k_pools[r][layer] / v_pools[r][layer] its local KV pages.
    The all-reduce after the o and down projections is a sum of the ranks' f16 partials in f32,
    rounded to f16 (what an f16 all-reduce delivers up to summation order). Returns the full logits
    (ranks' vocabulary slices concatenated)."""
    world = len(sharded)
    B, D = len(token_ids), cfg.head_dim
    # per-rank sizes from the sharded weights themselves (ranks may carry zero heads / channels as padding)
    hkv = k_pools[0][0].shape[1]
    hq = sharded[0]["layers"][0]["qkv"][0].shape[0] // D - 2 * hkv
    inter = sharded[0]["layers"][0]["gate_up"][0].shape[0] // 2
    x = sharded[0]["embed"][np.clip(token_ids, 0, cfg.vocab - 1)].copy()
    delta = None
    for li in range(cfg.layers):
        x, h = add_rmsnorm(x, delta, sharded[0]["layers"][li]["ln1"], cfg.eps)
        parts = []
        for r in range(world):
            lw = sharded[r]["layers"][li]
            qkv = gemv_w8a16(h, lw["qkv"][0], lw["qkv"][1], lw["qkv_bias"])
            q = rope(qkv[:, :hq * D].reshape(B, hq, D), cos, sin, positions)
            k = rope(qkv[:, hq * D:(hq + hkv) * D].reshape(B, hkv, D), cos, sin, positions)
            v = qkv[:, (hq + hkv) * D:].reshape(B, hkv, D)
            for b in range(B):
                page = block_table[b, positions[b] // cfg.page]
                k_pools[r][li][page, :, positions[b] % cfg.page] = k[b]
                v_pools[r][li][page, :, positions[b] % cfg.page] = v[b]
            attn = A.paged_attention_decode(q, k_pools[r][li], v_pools[r][li], block_table, positions + 1)
            parts.append(gemv_w8a16(attn.reshape(B, hq * D), lw["o"][0], lw["o"][1]))
        proj = sum(p.astype(f32) for p in parts).astype(f16)
        x, h = add_rmsnorm(x, proj, sharded[0]["layers"][li]["ln2"], cfg.eps)
        parts = []
        for r in range(world):
            lw = sharded[r]["layers"][li]
            act = swiglu(gemv_w8a16(h, lw["gate_up"][0], lw["gate_up"][1]), inter)
            parts.append(gemv_w8a16(act, lw["down"][0], lw["down"][1]))
        delta = sum(p.astype(f32) for p in parts).astype(f16)
    x, h = add_rmsnorm(x, delta, sharded[0]["ln_f"], cfg.eps)
    return np.concatenate([gemv_w8a16(h, s["lm_head"][0], s["lm_head"][1]) for s in sharded], axis=1)


def rank_step(cfg, shard, cos, sin, k_pools, v_pools, token_ids, positions, block_table, all_reduce):
    """One tensor-parallel rank's decode step: `shard` = this rank's weights, k_pools / v_pools [layer] its local
    KV pages, `all_reduce(f32 array) -> f32 array` the sum over ranks (a real collective in the multi-process
    tests). Returns this rank's slice of the logits."""
    B, D = len(token_ids), cfg.head_dim
    hkv = k_pools[0].shape[1]
    hq = shard["layers"][0]["qkv"][0].shape[0] // D - 2 * hkv
    inter = shard["layers"][0]["gate_up"][0].shape[0] // 2
    x = shard["embed"][np.clip(token_ids, 0, cfg.vocab - 1)].copy()
    delta = None
    for li, lw in enumerate(shard["layers"]):
        x, h = add_rmsnorm(x, delta, lw["ln1"], cfg.eps)
        qkv = gemv_w8a16(h, lw["qkv"][0], lw["qkv"][1], lw["qkv_bias"])
        q = rope(qkv[:, :hq * D].reshape(B, hq, D), cos, sin, positions)
        k = rope(qkv[:, hq * D:(hq + hkv) * D].reshape(B, hkv, D), cos, sin, positions)
        v = qkv[:, (hq + hkv) * D:].reshape(B, hkv, D)
        for b in range(B):
            page = block_table[b, positions[b] // cfg.page]
            k_pools[li][page, :, positions[b] % cfg.page] = k[b]
            v_pools[li][page, :, positions[b] % cfg.page] = v[b]
        attn = A.paged_attention_decode(q, k_pools[li], v_pools[li], block_table, positions + 1)
        proj = all_reduce(gemv_w8a16(attn.reshape(B, hq * D), lw["o"][0], lw["o"][1]).astype(f32)).astype(f16)
        x, h = add_rmsnorm(x, proj, lw["ln2"], cfg.eps)
        act = swiglu(gemv_w8a16(h, lw["gate_up"][0], lw["gate_up"][1]), inter)
        delta = all_reduce(gemv_w8a16(act, lw["down"][0], lw["down"][1]).astype(f32)).astype(f16)
    x, h = add_rmsnorm(x, delta, shard["ln_f"], cfg.eps)
    return gemv_w8a16(h, shard["lm_head"][0], shard["lm_head"][1])
