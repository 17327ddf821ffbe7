"""Tensor-parallel decode on two and four GPUs against the single-GPU decode of the same model, with both forms of
the all-reduce after the o and down projections: the kernel over peer memory that also does the residual add and the
RMSNorm (plain peer loads, bounded flag waits; eager and replayed as a CUDA graph), and NCCL followed by the norm
kernel. Four ranks share the two kv heads pairwise and pad the query-head
groups (see nncase_b200.decoder.shard_plan). Skipped when too few GPUs are visible."""
import os
import socket

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu


def _free_port():
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, q, peer_reduce):
    import torch.distributed as dist
    from nncase_b200 import decoder as D
    from nncase_b200.kernels import Context
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port), NCCL_NVLS_ENABLE="0")
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        cfg = D.DecoderConfig(layers=2, vocab=2048, max_pos=512)
        w = D.make_weights(cfg, 21)
        rng = np.random.default_rng(3)
        B, max_pages = 16, 8
        num_pages = B * max_pages + 1
        table = torch.from_numpy(rng.permutation(num_pages)[: B * max_pages].astype(np.int32).reshape(B, max_pages)).cuda()
        pos = torch.from_numpy(rng.integers(0, 100, B).astype(np.int32)).cuda()
        ids = torch.from_numpy(rng.integers(0, cfg.vocab, B).astype(np.int32)).cuda()
        kv = [(rng.normal(0, 1, (num_pages, cfg.kv_heads, 16, 64)).astype(np.float16),
               rng.normal(0, 1, (num_pages, cfg.kv_heads, 16, 64)).astype(np.float16)) for _ in range(cfg.layers)]
        ctx = Context(rank)
        tp = D.Decoder(cfg, w, B, num_pages, ctx=ctx, world=world, rank=rank, peer_reduce=peer_reduce)
        heads = D.rank_kv_heads(cfg, world, rank)
        for li in range(cfg.layers):
            tp.layers[li]["k_pool"].copy_(torch.from_numpy(np.ascontiguousarray(kv[li][0][:, heads])))
            tp.layers[li]["v_pool"].copy_(torch.from_numpy(np.ascontiguousarray(kv[li][1][:, heads])))
        local = tp.step(ids, pos, table).clone()
        if peer_reduce:
            # the same step again (it rewrites the same KV slots), replayed from a CUDA graph: the sequence numbers of
            # the exchange live in device memory, so a replay needs no new arguments
            ctx.synchronize()
            dist.barrier()
            side = torch.cuda.Stream(rank)
            side.wait_stream(torch.cuda.current_stream(rank))
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.stream(side):
                with torch.cuda.graph(graph, capture_error_mode="thread_local"):
                    ctx.use_current_stream()
                    out = tp.step(ids, pos, table)
            ctx.use_current_stream()
            for _ in range(3):
                graph.replay()
            torch.cuda.synchronize(rank)
            assert torch.equal(out, local)
        parts = [torch.empty_like(local) for _ in range(world)]
        dist.all_gather(parts, local.contiguous())
        got = torch.cat(parts, 1).float().cpu().numpy()
        ctx.check_status()
        if rank == 0:
            single = D.Decoder(cfg, w, B, num_pages, ctx=ctx)
            for li in range(cfg.layers):
                single.layers[li]["k_pool"].copy_(torch.from_numpy(kv[li][0]))
                single.layers[li]["v_pool"].copy_(torch.from_numpy(kv[li][1]))
            want = single.step(ids, pos, table).float().cpu().numpy()
            q.put((got, want))
        dist.barrier()
        tp.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("peer_reduce", [True, False])
@pytest.mark.parametrize("world", [2, 4])
def test_tp_matches_single_gpu(world, peer_reduce):
    if torch.cuda.device_count() < world:
        pytest.skip(f"needs {world} GPUs")
    import torch.multiprocessing as mp
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = _free_port()
    procs = [ctx.Process(target=_worker, args=(r, world, port, q, peer_reduce)) for r in range(world)]
    for p in procs:
        p.start()
    got, want = q.get(timeout=300)
    for p in procs:
        p.join(timeout=120)
        assert p.exitcode == 0
    rng = float(want.max() - want.min())
    assert np.abs(got - want).max() <= 5e-3 * rng
