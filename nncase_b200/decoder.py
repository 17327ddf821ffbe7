"""Decode step of a Qwen2-shaped transformer on the `cuda` module's kernels.

i8 weights (per output channel, symmetric, f16 scales), f16 activations, paged f16 KV cache with
16-token pages. One call = one new token for every sequence of the batch. Tensor parallel over the
GPUs of one node: qkv / gate-up projections split by output channel (whole heads), o / down
projections split by input channel, so each rank produces a partial [batch, hidden] sum that is
all-reduced with NCCL (torch.distributed) after the attention-output and the down projection; KV
pages are rank-local. The reference has no transformer operators and no multi-device runtime; the
operator semantics are those of include/nncase_b200.h.
"""
import ctypes as C
from dataclasses import dataclass

import numpy as np
import torch
import torch.distributed as dist

from . import lib as L
from .kernels import Context, NncbError, check


@dataclass(frozen=True)
class DecoderConfig:
    layers: int = 24
    hidden: int = 896
    q_heads: int = 14
    kv_heads: int = 2
    head_dim: int = 64
    inter: int = 4864
    vocab: int = 151936
    eps: float = 1e-6
    rope_theta: float = 1e6
    max_pos: int = 4096
    page: int = 16


def quantize_per_channel_i8(w):
    """[N, K] f32 -> (i8 [N, K], f16 scales [N]): symmetric, scale = max|w| / 127 rounded to f16."""
    amax = np.abs(w).max(axis=1)
    scale = np.maximum(amax / 127.0, 1e-8).astype(np.float16)
    q = np.clip(np.rint(w / scale.astype(np.float32)[:, None]), -127, 127).astype(np.int8)
    return q, scale


def make_weights(cfg, seed=1005):
    """Seeded N(0, 0.02) weights of the given shape, quantized; norm weights 1 + N(0, 0.02)."""
    rng = np.random.default_rng(seed)
    H, D = cfg.hidden, cfg.head_dim
    nq, nkv = cfg.q_heads * D, cfg.kv_heads * D

    def lin(n, k):
        return quantize_per_channel_i8(rng.normal(0, 0.02, (n, k)).astype(np.float32))

    layers = []
    for _ in range(cfg.layers):
        layers.append(dict(
            ln1=(1 + rng.normal(0, 0.02, H)).astype(np.float16), ln2=(1 + rng.normal(0, 0.02, H)).astype(np.float16),
            qkv=lin(nq + 2 * nkv, H), qkv_bias=rng.normal(0, 0.02, nq + 2 * nkv).astype(np.float16),
            o=lin(H, nq), gate_up=lin(2 * cfg.inter, H), down=lin(H, cfg.inter)))
    return dict(embed=rng.normal(0, 0.02, (cfg.vocab, H)).astype(np.float16), layers=layers,
                ln_f=(1 + rng.normal(0, 0.02, H)).astype(np.float16), lm_head=lin(cfg.vocab, H))


def rope_tables(cfg):
    """cos/sin [max_pos][head_dim/2] f32, angles computed in double."""
    half = cfg.head_dim // 2
    inv = cfg.rope_theta ** (-np.arange(half, dtype=np.float64) * 2.0 / cfg.head_dim)
    ang = np.arange(cfg.max_pos, dtype=np.float64)[:, None] * inv[None, :]
    return np.cos(ang).astype(np.float32), np.sin(ang).astype(np.float32)


def shard_plan(cfg, world):
    """How the model splits over `world` tensor-parallel ranks (Megatron-style: qkv / gate-up by output channel,
    o / down by input channel, LM head by vocabulary).

    KV heads split when there are enough of them; otherwise several ranks share one KV head (each keeps its
    own copy of that head's pages) and the query heads of the head's group are dealt to those ranks, the group
    padded with zero heads to a multiple of the sharing degree -- a zero head has zero q rows and zero o
    columns, so it adds nothing. The MLP width per rank is rounded up to the MatMul's K granule (64) with zero
    channels. Qwen2-0.5B (14 q / 2 kv heads, 4864): world 2 -> 7 q + 1 kv per rank; world 4 -> 4 q (one
    padded per group) + 1 shared kv; world 8 -> 2 q + 1 shared kv, MLP 608 -> 640 per rank."""
    if world < 1 or cfg.q_heads % cfg.kv_heads:
        raise NncbError(-22, "bad tensor parallel degree or head counts")
    group = cfg.q_heads // cfg.kv_heads
    if cfg.kv_heads % world == 0:
        rep, hkv, gpad = 1, cfg.kv_heads // world, group
        hq = hkv * group
    elif world % cfg.kv_heads == 0:
        rep, hkv = world // cfg.kv_heads, 1
        gpad = -(-group // rep) * rep
        hq = gpad // rep
    else:
        raise NncbError(-38, f"tensor parallel degree {world} neither divides nor is a multiple of the {cfg.kv_heads} kv heads")
    if cfg.vocab % world:
        raise NncbError(-38, f"tensor parallel degree {world} does not divide the vocabulary")
    if hq // hkv > 8:
        raise NncbError(-38, "more than 8 query heads per kv head on a rank")
    inter = -(-cfg.inter // world)
    inter_pad = -(-inter // 64) * 64
    return dict(world=world, group=group, rep=rep, hq=hq, hkv=hkv, gpad=gpad, inter=inter, inter_pad=inter_pad,
                vocab=cfg.vocab // world)


def rank_kv_heads(cfg, world, rank):
    """Indices of the model's kv heads whose pages rank `rank` keeps."""
    p = shard_plan(cfg, world)
    if p["rep"] == 1:
        return list(range(rank * p["hkv"], (rank + 1) * p["hkv"]))
    return [rank // p["rep"]]


def shard_weights(cfg, w, world, rank):
    """The slice of every projection that tensor-parallel rank `rank` of `world` owns (see shard_plan)."""
    if world == 1:
        return w
    p = shard_plan(cfg, world)
    D = cfg.head_dim
    nq, nkv = cfg.q_heads * D, cfg.kv_heads * D
    kv_heads = rank_kv_heads(cfg, world, rank)
    # query heads of this rank, as indices into the model's heads; None = a zero head that pads the group
    if p["rep"] == 1:
        q_heads = list(range(rank * p["hq"], (rank + 1) * p["hq"]))
    else:
        j = rank % p["rep"]
        q_heads = [kv_heads[0] * p["group"] + i if i < p["group"] else None for i in range(j * p["hq"], (j + 1) * p["hq"])]
    ii, ipad = p["inter"], p["inter_pad"]
    g0, g1 = rank * ii, min((rank + 1) * ii, cfg.inter)
    vv = p["vocab"]

    def take_rows(t, idx_blocks, bias=None):
        """Rows of a quantized [N, K] matrix (and of its scales / bias) by blocks of row indices; a None block of
        length L gives L zero rows."""
        wq, sc = t
        ws, ss, bs = [], [], []
        for blk in idx_blocks:
            if isinstance(blk, int):
                ws.append(np.zeros((blk, wq.shape[1]), wq.dtype)), ss.append(np.zeros(blk, sc.dtype))
                bs.append(np.zeros(blk, np.float16))
            else:
                ws.append(wq[blk]), ss.append(sc[blk])
                if bias is not None:
                    bs.append(bias[blk])
        out = (np.ascontiguousarray(np.concatenate(ws)), np.concatenate(ss))
        return out if bias is None else (out, np.concatenate(bs))

    def take_cols(t, idx_blocks):
        wq, sc = t
        cols = [np.zeros((wq.shape[0], blk), wq.dtype) if isinstance(blk, int) else wq[:, blk] for blk in idx_blocks]
        return np.ascontiguousarray(np.concatenate(cols, axis=1)), sc

    def head_rows(h, base=0):
        return D if h is None else slice(base + h * D, base + (h + 1) * D)

    q_blocks = [head_rows(h) for h in q_heads]
    k_blocks = [head_rows(h, nq) for h in kv_heads]
    v_blocks = [head_rows(h, nq + nkv) for h in kv_heads]
    pad = ipad - (g1 - g0)
    gate_blocks = [slice(g0, g1)] + ([pad] if pad else [])
    up_blocks = [slice(cfg.inter + g0, cfg.inter + g1)] + ([pad] if pad else [])
    layers = []
    for lw in w["layers"]:
        qkv, qkv_bias = take_rows(lw["qkv"], q_blocks + k_blocks + v_blocks, lw["qkv_bias"])
        layers.append(dict(ln1=lw["ln1"], ln2=lw["ln2"], qkv=qkv, qkv_bias=qkv_bias,
                           o=take_cols(lw["o"], q_blocks), gate_up=take_rows(lw["gate_up"], gate_blocks + up_blocks),
                           down=take_cols(lw["down"], gate_blocks)))
    return dict(embed=w["embed"], layers=layers, ln_f=w["ln_f"],
                lm_head=take_rows(w["lm_head"], [slice(rank * vv, (rank + 1) * vv)]))


def interleave_gate_up(wq, scale):
    """[gate rows (inter) | up rows (inter)] -> blocks of 16 rows: the gate rows of 8 outputs, then their up
    rows -- the order nncb_gemv_w8a16_swiglu expects. inter must be a multiple of 8."""
    inter = wq.shape[0] // 2
    assert inter % 8 == 0
    idx = np.arange(inter).reshape(-1, 8)
    order = np.concatenate([idx, idx + inter], axis=1).reshape(-1)
    return np.ascontiguousarray(wq[order]), np.ascontiguousarray(scale[order])


class Decoder:
    """One tensor-parallel rank of the decoder (world 1 = the whole model)."""

    def __init__(self, cfg, weights, max_batch, num_pages, ctx=None, device=0, world=1, rank=0, group=None, fused_rope=True,
                 peer_reduce=True):
        self.cfg, self.world, self.rank, self.group = cfg, world, rank, group
        self.fused_rope = fused_rope  # rotary embedding and KV append inside the attention launch (one launch fewer per layer)
        self.ctx = ctx or Context(device)
        dev = self.ctx.device
        w = shard_weights(cfg, weights, world, rank)
        t = lambda a: torch.from_numpy(np.ascontiguousarray(a)).to(dev)
        self.embed, self.ln_f = t(w["embed"]), t(w["ln_f"])
        self.lm_w, self.lm_s = t(w["lm_head"][0]), t(w["lm_head"][1])
        self.layers = []
        plan = shard_plan(cfg, world)
        self.hq, self.hkv = plan["hq"], plan["hkv"]
        self.inter = plan["inter_pad"] if world > 1 else cfg.inter
        self.parallelism = (f"tp{world}: {self.hq} q + {self.hkv} kv heads, MLP {self.inter} per rank" +
                            (f", each kv head on {plan['rep']} ranks" if plan["rep"] > 1 else "")) if world > 1 else "tp1"
        for lw in w["layers"]:
            lw = dict(lw, gate_up=interleave_gate_up(*lw["gate_up"]))  # SwiGLU runs in the gate/up MatMul's epilogue
            self.layers.append(dict(
                ln1=t(lw["ln1"]), ln2=t(lw["ln2"]), qkv_w=t(lw["qkv"][0]), qkv_s=t(lw["qkv"][1]), qkv_b=t(lw["qkv_bias"]),
                o_w=t(lw["o"][0]), o_s=t(lw["o"][1]), gu_w=t(lw["gate_up"][0]), gu_s=t(lw["gate_up"][1]),
                d_w=t(lw["down"][0]), d_s=t(lw["down"][1]),
                k_pool=torch.zeros((num_pages, self.hkv, cfg.page, cfg.head_dim), dtype=torch.float16, device=dev),
                v_pool=torch.zeros((num_pages, self.hkv, cfg.page, cfg.head_dim), dtype=torch.float16, device=dev)))
        cos, sin = rope_tables(cfg)
        self.cos, self.sin = t(cos), t(sin)
        B, H, D = max_batch, cfg.hidden, cfg.head_dim
        f16 = dict(dtype=torch.float16, device=dev)
        self.x, self.h = torch.empty((B, H), **f16), torch.empty((B, H), **f16)
        self.qkv = torch.empty((B, (self.hq + 2 * self.hkv) * D), **f16)
        self.q = torch.empty((B, self.hq * D), **f16)
        self.attn = torch.empty((B, self.hq * D), **f16)
        self.proj = torch.empty((B, H), **f16)
        self.act = torch.empty((B, self.inter), **f16)
        self.logits = torch.empty((B, cfg.vocab // world), **f16)
        self.ws = torch.empty(4 << 20, dtype=torch.uint8, device=dev)
        self.max_batch = B
        # the all-reduce after the o and down projections: one kernel over peer memory (with the residual add and the
        # RMSNorm that follow it), or NCCL followed by the norm kernel
        self.peer = None
        if world > 1 and peer_reduce:
            self._setup_peer()
        if world > 1:
            self.parallelism += (", all-reduce as one kernel over peer memory with the residual add and RMSNorm" if self.peer
                                 else ", NCCL all-reduce")

    def _setup_peer(self):
        """Allocates this rank's two partial buffers ([max_batch, hidden] f16 each: o projection, down projection) and
        its flag block, exchanges their CUDA IPC handles with the other ranks and maps theirs."""
        lib, h = self.ctx._lib, self.ctx._h
        part_bytes = self.max_batch * self.cfg.hidden * 2
        part_bytes = (part_bytes + 255) // 256 * 256
        total = 2 * part_bytes + 256
        base = C.c_void_p()
        check(lib.nncb_malloc(h, total, C.byref(base)))
        check(lib.nncb_memset(h, base, 0, total))
        self.ctx.synchronize()
        handle = C.create_string_buffer(64)
        check(lib.nncb_ipc_export(h, base, handle, 64))
        handles = [None] * self.world
        dist.all_gather_object(handles, handle.raw, group=self.group)
        bases, failed = [], None
        for r in range(self.world):
            if r == self.rank:
                bases.append(base.value)
                continue
            p = C.c_void_p()
            try:
                check(lib.nncb_ipc_import(h, handles[r], 64, C.byref(p)))
            except NncbError as e:  # no peer access between these two GPUs, or IPC closed to this process
                failed = e
                p = C.c_void_p(0)
            bases.append(p.value or 0)
        # every rank takes the same path: if one mapping failed anywhere, all fall back to NCCL's all-reduce
        okay = torch.tensor([0 if failed else 1], dtype=torch.int32, device=self.ctx.device)
        dist.all_reduce(okay, op=dist.ReduceOp.MIN, group=self.group)
        if int(okay.item()) == 0:
            for r, b in enumerate(bases):
                if r != self.rank and b:
                    lib.nncb_ipc_close(h, C.c_void_p(b))
            dist.barrier(group=self.group)
            check(lib.nncb_free(h, base))
            import warnings
            warnings.warn(f"tensor-parallel decode: peer memory could not be mapped ({failed}); using NCCL all-reduce")
            return
        dist.barrier(group=self.group)  # every block of flags is zeroed and mapped before the first step
        arr = C.c_void_p * self.world
        self.peer = dict(
            base=base, bases=bases, part_bytes=part_bytes,
            parts=[arr(*[b + s * part_bytes for b in bases]) for s in (0, 1)],
            flags=arr(*[b + 2 * part_bytes for b in bases]),
            own=[base.value + s * part_bytes for s in (0, 1)])

    def close(self):
        """Unmaps the other ranks' buffers and frees this rank's (after a barrier: nobody reads them any more)."""
        if self.peer is not None:
            lib, h = self.ctx._lib, self.ctx._h
            self.ctx.synchronize()
            dist.barrier(group=self.group)
            for r, b in enumerate(self.peer["bases"]):
                if r != self.rank:
                    check(lib.nncb_ipc_close(h, C.c_void_p(b)))
            dist.barrier(group=self.group)
            check(lib.nncb_free(h, self.peer["base"]))
            self.peer = None

    # thin wrappers over the C ABI (device pointers of preallocated tensors)
    def _gemv(self, x, w, s, b, y):
        """y: a tensor, or the device address of this rank's partial buffer."""
        lib, h = self.ctx._lib, self.ctx._h
        check(lib.nncb_gemv_w8a16(h, x.data_ptr(), w.data_ptr(), s.data_ptr(), b.data_ptr() if b is not None else None,
                                  None, y if isinstance(y, int) else y.data_ptr(), x.shape[0], w.shape[0], w.shape[1]))

    def _gemv_swiglu(self, x, w, s, y):
        """y = swiglu(gemv(x)) over interleaved gate/up rows (SwiGLU in the MatMul's epilogue)."""
        check(self.ctx._lib.nncb_gemv_w8a16_swiglu(self.ctx._h, x.data_ptr(), w.data_ptr(), s.data_ptr(), None, y.data_ptr(),
                                                   x.shape[0], w.shape[0], w.shape[1]))

    def _norm(self, x, delta, w, out):
        check(self.ctx._lib.nncb_add_rmsnorm_f16(self.ctx._h, x.data_ptr(), delta.data_ptr() if delta is not None else None,
                                                 w.data_ptr(), out.data_ptr(), x.shape[0], x.shape[1], self.cfg.eps))

    def _all_reduce(self, t):
        if self.world > 1:
            dist.all_reduce(t, group=self.group)

    def _reduce_norm(self, x, slot, w, out):
        """x += all-reduce of the ranks' partials of `slot`; out = RMSNorm(x): one launch over peer memory."""
        pr = self.peer
        check(self.ctx._lib.nncb_peer_allreduce_add_rmsnorm_f16(self.ctx._h, x.data_ptr(), pr["parts"][slot], pr["flags"], self.world,
                                                                self.rank, slot, w.data_ptr(), out.data_ptr(), x.shape[0],
                                                                x.shape[1], self.cfg.eps))

    def step(self, token_ids, positions, block_table):
        """token_ids, positions [B] int32 (position = number of tokens already cached), block_table
        [B, max_pages] int32 (device tensors). Appends this token's K/V and returns this rank's slice of
        the logits [B, vocab / world] f16."""
        cfg, lib, h = self.cfg, self.ctx._lib, self.ctx._h
        B = token_ids.shape[0]
        if B > self.max_batch:
            raise NncbError(-22, "batch larger than planned")
        x, hh, qkv, q, attn, proj, act = (self.x[:B], self.h[:B], self.qkv[:B], self.q[:B], self.attn[:B], self.proj[:B],
                                          self.act[:B])
        ctx_lens = positions + 1
        check(lib.nncb_embedding_f16(h, self.embed.data_ptr(), token_ids.data_ptr(), x.data_ptr(), B, cfg.hidden, cfg.vocab))
        delta = None
        peer = self.peer is not None
        for lw in self.layers:
            if peer and delta is not None:
                self._reduce_norm(x, 1, lw["ln1"], hh)  # the down projection's partials of the layer before
            else:
                self._norm(x, delta, lw["ln1"], hh)
            self._gemv(hh, lw["qkv_w"], lw["qkv_s"], lw["qkv_b"], qkv)
            if self.fused_rope:
                # rotary embedding and KV append inside the attention launch
                check(lib.nncb_paged_attention_decode_rope(h, qkv.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                                                           positions.data_ptr(), lw["k_pool"].data_ptr(), lw["v_pool"].data_ptr(),
                                                           block_table.data_ptr(), ctx_lens.data_ptr(), attn.data_ptr(), B,
                                                           self.hq, self.hkv, cfg.head_dim, cfg.page, block_table.shape[1],
                                                           self.cos.shape[0], lw["k_pool"].shape[0],
                                                           C.c_float(1.0 / np.sqrt(cfg.head_dim)), self.ws.data_ptr(),
                                                           self.ws.numel()))
            else:
                check(lib.nncb_rope_kv_append_f16(h, qkv.data_ptr(), q.data_ptr(), self.cos.data_ptr(), self.sin.data_ptr(),
                                                  positions.data_ptr(), block_table.data_ptr(), lw["k_pool"].data_ptr(),
                                                  lw["v_pool"].data_ptr(), B, self.hq, self.hkv, cfg.head_dim, cfg.page,
                                                  block_table.shape[1], self.cos.shape[0], lw["k_pool"].shape[0]))
                check(lib.nncb_paged_attention_decode(h, q.data_ptr(), lw["k_pool"].data_ptr(), lw["v_pool"].data_ptr(),
                                                      block_table.data_ptr(), ctx_lens.data_ptr(), attn.data_ptr(), B,
                                                      self.hq, self.hkv, cfg.head_dim, cfg.page, block_table.shape[1],
                                                      lw["k_pool"].shape[0],
                                                      C.c_float(1.0 / np.sqrt(cfg.head_dim)), self.ws.data_ptr(),
                                                      self.ws.numel()))
            if peer:
                self._gemv(attn, lw["o_w"], lw["o_s"], None, self.peer["own"][0])
                self._reduce_norm(x, 0, lw["ln2"], hh)
            else:
                self._gemv(attn, lw["o_w"], lw["o_s"], None, proj)
                self._all_reduce(proj)
                self._norm(x, proj, lw["ln2"], hh)
            self._gemv_swiglu(hh, lw["gu_w"], lw["gu_s"], act)
            if peer:
                self._gemv(act, lw["d_w"], lw["d_s"], None, self.peer["own"][1])
            else:
                self._gemv(act, lw["d_w"], lw["d_s"], None, proj)
                self._all_reduce(proj)
            delta = proj
        if peer and delta is not None:
            self._reduce_norm(x, 1, self.ln_f, hh)
        else:
            self._norm(x, delta, self.ln_f, hh)
        self._gemv(hh, self.lm_w, self.lm_s, None, self.logits[:B])
        return self.logits[:B]
