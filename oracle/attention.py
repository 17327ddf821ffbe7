"""Paged-attention decode on the CPU, in numpy. TEST INFRASTRUCTURE ONLY.

PARITY UNPINNED: the reference has no attention operator, KV cache or paged layout (its complete
native op list is src/Native/include/nncase/kernels/stackvm/tensor_ops.h:29-479), so there is no
reference output or test to pin this against. The math is composed from the reference's own
kernels: scores and value sums as its mat_mul (f32 accumulate, reference/matmul.cpp:28-51), the
softmax as reference/softmax.cpp:30-80 (subtract the row maximum, expf, sum, multiply by 1/sum).
Inputs are f16 (q, K, V), all arithmetic is f32, the result is rounded to f16.
"""
import numpy as np


def paged_attention_decode(q, k_pool, v_pool, block_table, context_lens, scale=None):
    """q [B,Hq,D] f16; k_pool/v_pool [pages,Hkv,page,D] f16; block_table [B,max_pages] i32;
    context_lens [B] -> [B,Hq,D] f16. An empty context gives zeros."""
    q = np.asarray(q, np.float16)
    b, hq, d = q.shape
    _, hkv, page, _ = k_pool.shape
    group = hq // hkv
    scale = np.float32(scale if scale is not None else 1.0 / np.sqrt(d))
    out = np.zeros((b, hq, d), np.float16)
    for i in range(b):
        n = int(context_lens[i])
        if n == 0:
            continue
        pages = block_table[i, :(n + page - 1) // page]
        for h in range(hq):
            kv = h // group
            k = k_pool[pages, kv].reshape(-1, d)[:n].astype(np.float32)
            v = v_pool[pages, kv].reshape(-1, d)[:n].astype(np.float32)
            s = (k @ q[i, h].astype(np.float32)) * scale
            e = np.exp(s - s.max(), dtype=np.float32)
            p = e * (np.float32(1.0) / e.sum(dtype=np.float32))
            out[i, h] = (p @ v).astype(np.float16)
    return out
