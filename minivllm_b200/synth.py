"""Seeded synthetic inputs with the shapes and value distributions of the
benchmark configurations of this path.  No dataset, tokenizer or checkpoint is
involved: everything is drawn from `torch.Generator(seed)` on the CPU, in a
fixed order, so the tests, the benchmark and the CPU baseline see the same
tensors.  Callers move the tensors to the GPU and cast them.
"""
import math

import torch


def decode_inputs(seed=0, batch=16, ctx_lo=64, ctx_hi=1024, num_heads=16, num_kv_heads=8, head_dim=128,
                  block_size=256, spare_blocks=0):
    """Paged decode: context lengths uniform in [ctx_lo, ctx_hi], physical
    blocks = sum(ceil(len / block_size)) (+ spare) handed out through a seeded
    permutation, -1 padded tables, q/k/v ~ N(0,1) in fp32, scale 1/sqrt(head_dim).
    Draw order: context_lens, permutation, q, k_cache, v_cache.
    """
    g = torch.Generator().manual_seed(seed)
    context_lens = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g, dtype=torch.int64)
    nblk = [(int(n) + block_size - 1) // block_size for n in context_lens]
    total = sum(nblk) + spare_blocks
    perm = torch.randperm(total, generator=g)
    max_blocks = max(nblk)
    block_tables = torch.full((batch, max_blocks), -1, dtype=torch.int32)
    at = 0
    for b, n in enumerate(nblk):
        block_tables[b, :n] = perm[at:at + n].to(torch.int32)
        at += n
    q = torch.randn(batch, num_heads, head_dim, generator=g)
    k_cache = torch.randn(total, block_size, num_kv_heads, head_dim, generator=g)
    v_cache = torch.randn(total, block_size, num_kv_heads, head_dim, generator=g)
    return dict(q=q, k_cache=k_cache, v_cache=v_cache, block_tables=block_tables, context_lens=context_lens,
                scale=1.0 / math.sqrt(head_dim), num_heads=num_heads, num_kv_heads=num_kv_heads,
                head_dim=head_dim, block_size=block_size)


def prefill_inputs(seed=1, num_seqs=32, len_lo=128, len_hi=2048, num_heads=32, num_kv_heads=8, head_dim=128):
    """Varlen prefill: lengths uniform in [len_lo, len_hi], cu_seqlens prefix
    sum (int32), packed q/k/v ~ N(0,1) in fp32.  Draw order: lens, q, k, v.
    """
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(len_lo, len_hi + 1, (num_seqs,), generator=g, dtype=torch.int64)
    cu = torch.zeros(num_seqs + 1, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0).to(torch.int32)
    total = int(cu[-1])
    q = torch.randn(total, num_heads, head_dim, generator=g)
    k = torch.randn(total, num_kv_heads, head_dim, generator=g)
    v = torch.randn(total, num_kv_heads, head_dim, generator=g)
    return dict(q=q, k=k, v=v, cu_seqlens=cu, lens=lens, max_seqlen=int(lens.max()), scale=1.0 / math.sqrt(head_dim),
                num_heads=num_heads, num_kv_heads=num_kv_heads, head_dim=head_dim)


def store_inputs(seed=2, num_tokens=65536, num_blocks=4096, block_size=256, num_kv_heads=8, head_dim=128,
                 pad_frac=0.03, std=2.0):
    """store_kvcache: slots = first num_tokens entries of a seeded permutation
    of all cache slots, a pad_frac share set to -1, k/v ~ N(0, std) in fp32.
    Draw order: permutation, pad mask, k, v.
    """
    g = torch.Generator().manual_seed(seed)
    slots = torch.randperm(num_blocks * block_size, generator=g)[:num_tokens].to(torch.int64)
    pad = torch.rand(num_tokens, generator=g) < pad_frac
    slots[pad] = -1
    k = torch.randn(num_tokens, num_kv_heads, head_dim, generator=g) * std
    v = torch.randn(num_tokens, num_kv_heads, head_dim, generator=g) * std
    return dict(k=k, v=v, slot_mapping=slots, num_blocks=num_blocks, block_size=block_size,
                num_kv_heads=num_kv_heads, head_dim=head_dim)


def prefill_flops(lens, num_heads, head_dim):
    """Causal attention FLOPs: QK^T and PV, 2 per multiply-add, lower triangle only."""
    return float(sum(4 * num_heads * head_dim * (int(n) * (int(n) + 1) // 2) for n in lens))


def decode_bytes(context_lens, batch, num_heads, num_kv_heads, head_dim, elem_bytes, max_blocks, int8=False):
    """Algorithmic HBM bytes of one decode call: KV read once per KV head, q
    and out once, the block tables once."""
    tokens = int(sum(int(n) for n in context_lens))
    if int8:
        kv = tokens * num_kv_heads * (head_dim + 2) * 2
    else:
        kv = tokens * num_kv_heads * head_dim * 2 * elem_bytes
    return kv + 2 * batch * num_heads * head_dim * elem_bytes + batch * max_blocks * 4
