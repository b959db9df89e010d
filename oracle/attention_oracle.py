"""CPU oracle for the ragged-batch attention path.  TEST INFRASTRUCTURE ONLY.

This file restates, on the CPU, what the reference engine (Wenyueh/MinivLLM)
computes on this path.  It exists to check the CUDA kernels and to be timed as
the CPU baseline; nothing in the `minivllm_b200` package imports it and it is
never a fallback.  Only the tests, the smoke check and the benchmark's CPU
baseline may call it.

Parity status, per function:
  * store_kvcache, paged_attention_decode, flash_attention_prefill,
    prepare_prefill, prepare_decode: pinned.  The reference holds no tests or
    golden vectors, so the pins are outputs of the reference's own code run on
    CPU (its PyTorch paths and its Triton kernels under the Triton
    interpreter), recorded in tests/golden/ by tests/golden/make_golden.py.
  * quantize_kv_int8 / dequantize_kv_int8: PARITY UNPINNED BY THE REFERENCE —
    the reference has no quantisation code.  The definition here is the
    specification; it is cross-checked against an exact-rational evaluation.

Arithmetic: fp32 on inputs already rounded to the GPU dtype (fp16 / bf16).
"""
import math

import numpy as np
import torch


# --------------------------------------------------------------------------
# store_kvcache
# --------------------------------------------------------------------------
def store_kvcache(key, value, k_cache, v_cache, slot_mapping):
    """In-place scatter; follows src/myvllm/layers/attention.py:25-34,48-64:
    program (t, head) returns early when slot == -1, else copies head_dim
    elements of key[t, head] to cache.flat[slot, head].  Restated as a masked
    row assignment on the cache viewed as (slots, kv_heads, head_dim).
    """
    kv_heads, head_dim = key.shape[1], key.shape[2]
    live = slot_mapping >= 0
    slots = slot_mapping[live]
    k_cache.view(-1, kv_heads, head_dim)[slots] = key[live].to(k_cache.dtype)
    v_cache.view(-1, kv_heads, head_dim)[slots] = value[live].to(v_cache.dtype)


# --------------------------------------------------------------------------
# int8 KV quantisation (no counterpart in the reference)
# --------------------------------------------------------------------------
def quantize_kv_int8(x):
    """Per-token-per-head symmetric int8.  x: (tokens, kv_heads, head_dim) torch
    tensor (fp16/bf16/fp32).  Returns (codes int8, scales fp16) as torch tensors.

      amax = max|x| over head_dim, in fp32
      scale16 = fp16(amax / 127)          (IEEE division, round to nearest even)
      s = fp32(scale16)
      code = clamp(rint(x / s), -127, 127), 0 where s == 0   (rint = half to even)
    """
    xf = x.detach().to(torch.float32).cpu().numpy()
    amax = np.abs(xf).max(axis=-1, keepdims=True).astype(np.float32)
    with np.errstate(over="ignore"):
        scale16 = (amax / np.float32(127.0)).astype(np.float16)
    s = scale16.astype(np.float32)
    with np.errstate(divide="ignore", invalid="ignore"):
        r = np.rint(xf / s)
    r = np.where(s == 0, np.float32(0), r)
    codes = np.clip(r, -127, 127).astype(np.int8)
    return torch.from_numpy(codes), torch.from_numpy(scale16.squeeze(-1))


def dequantize_kv_int8(codes, scales):
    """float(code) * float(scale) in fp32; codes (..., head_dim), scales (...)."""
    return codes.to(torch.float32) * scales.to(torch.float32).unsqueeze(-1)


def store_kvcache_int8(key, value, k_codes, v_codes, k_scale, v_scale, slot_mapping):
    """Quantise, then scatter codes and scales by slot (-1 skipped)."""
    kv_heads, head_dim = key.shape[1], key.shape[2]
    live = slot_mapping >= 0
    slots = slot_mapping[live]
    kc, ks = quantize_kv_int8(key[live])
    vc, vs = quantize_kv_int8(value[live])
    k_codes.view(-1, kv_heads, head_dim)[slots] = kc
    v_codes.view(-1, kv_heads, head_dim)[slots] = vc
    k_scale.view(-1, kv_heads)[slots] = ks
    v_scale.view(-1, kv_heads)[slots] = vs


# --------------------------------------------------------------------------
# paged decode attention
# --------------------------------------------------------------------------
def paged_attention_decode(query, k_cache, v_cache, block_tables, context_lens, scale, num_heads, num_kv_heads,
                           head_dim, block_size):
    """fp32 restatement of src/myvllm/layers/attention.py:283-415 (the Triton
    kernel's semantics): token j of sequence b lives at
    cache[block_tables[b, j // block_size], j % block_size]; tokens whose table
    entry is -1 are skipped (:355, :394); GQA head h reads kv head
    h // (num_heads // num_kv_heads) (:307); softmax over the live tokens.
    Agrees with benchmark_decoding.py:136-189 `decode_torch_optimized` whenever
    the first ceil(len/block_size) table entries are all valid.
    A row with no live token yields zeros (the reference divides 0 by 0).
    """
    q = query.to(torch.float32)
    kc = k_cache.to(torch.float32)
    vc = v_cache.to(torch.float32)
    batch = q.shape[0]
    group = num_heads // num_kv_heads
    out = torch.zeros(batch, num_heads, head_dim, dtype=torch.float32)
    max_blocks = block_tables.shape[1]
    for b in range(batch):
        n = int(context_lens[b])
        n = max(0, min(n, max_blocks * block_size))
        if n == 0:
            continue
        tok = torch.arange(n)
        blk = block_tables[b, tok // block_size].to(torch.int64)
        live = blk >= 0
        if not bool(live.any()):
            continue
        rows = blk[live] * block_size + (tok % block_size)[live]
        k = kc.reshape(-1, num_kv_heads, head_dim)[rows]          # (n_live, KVH, D)
        v = vc.reshape(-1, num_kv_heads, head_dim)[rows]
        qb = q[b].reshape(num_kv_heads, group, head_dim)          # (KVH, G, D)
        scores = torch.einsum("kgd,nkd->kgn", qb, k) * scale
        probs = torch.softmax(scores, dim=-1)
        out[b] = torch.einsum("kgn,nkd->kgd", probs, v).reshape(num_heads, head_dim)
    return out


# --------------------------------------------------------------------------
# varlen causal prefill attention
# --------------------------------------------------------------------------
def flash_attention_prefill(q, k, v, cu_seqlens, scale, num_heads, num_kv_heads, head_dim):
    """fp32 restatement of src/myvllm/layers/attention.py:111-209: per sequence
    [cu[s], cu[s+1]) and head h, row i attends to rows <= i of the same
    sequence (:181), kv head h // group (:132), scores scaled after the dot
    (:177-178).  Same result as benchmark_prefilling.py:9-52
    `pytorch_standard_attention`.
    """
    qf, kf, vf = q.to(torch.float32), k.to(torch.float32), v.to(torch.float32)
    group = num_heads // num_kv_heads
    out = torch.zeros_like(qf)
    cu = [int(x) for x in cu_seqlens]
    for s in range(len(cu) - 1):
        a, e = cu[s], cu[s + 1]
        n = e - a
        if n <= 0:
            continue
        qs = qf[a:e].reshape(n, num_kv_heads, group, head_dim)
        scores = torch.einsum("ikgd,jkd->kgij", qs, kf[a:e]) * scale
        mask = torch.ones(n, n, dtype=torch.bool).tril_()
        scores = scores.masked_fill(~mask, float("-inf"))
        probs = torch.softmax(scores, dim=-1)
        o = torch.einsum("kgij,jkd->ikgd", probs, vf[a:e])
        out[a:e] = o.reshape(n, num_heads, head_dim)
    return out


# --------------------------------------------------------------------------
# q/k RMSNorm + rotary embedding (the step right before the attention operators)
# --------------------------------------------------------------------------
def qk_norm_rope(x, positions, cos_table, sin_table, gamma, eps, dtype):
    """x (tokens, heads, head_dim) already rounded to `dtype`; fp32 restatement of
    src/myvllm/layers/layernorm.py:10-17 (x / sqrt(mean(x^2) + eps) * gamma) followed by
    src/myvllm/layers/rotary_embedding.py:4-23 (rotate-half with cos/sin[positions]), with the result of
    each of the two steps rounded to the model dtype, as two separate kernels in that dtype would."""
    xf = x.to(torch.float32)
    n = xf / torch.sqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.to(torch.float32)
    n = n.to(dtype).to(torch.float32)
    cos, sin = cos_table[positions][:, None, :], sin_table[positions][:, None, :]
    x1, x2 = n.chunk(2, dim=-1)
    return torch.cat([x1 * cos - x2 * sin, x1 * sin + x2 * cos], dim=-1).to(dtype)


# --------------------------------------------------------------------------
# prefill with a cached prefix (keys and values read from the paged cache)
# --------------------------------------------------------------------------
def flash_attention_prefill_paged(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables, scale, num_heads,
                                  num_kv_heads, head_dim):
    """Sequence s: q rows [cu_q[s], cu_q[s+1]) are its LAST queries; it has cu_k[s+1]-cu_k[s] keys at cache rows
    block_tables[s, j // bs] * bs + j % bs.  Query i sits at position keys - queries + i and attends to keys at
    positions <= its own: the rows that the full-sequence causal attention (flash_attention_prefill above,
    src/myvllm/layers/attention.py:111-209) would produce for those positions.  The reference never computes
    this case (its kernel ignores cu_seqlens_k), so the pin is that equivalence, checked in the tests."""
    qf = q.to(torch.float32)
    kc, vc = k_cache.to(torch.float32), v_cache.to(torch.float32)
    bs = k_cache.shape[1]
    group = num_heads // num_kv_heads
    out = torch.zeros_like(qf)
    cq, ck = [int(x) for x in cu_seqlens_q], [int(x) for x in cu_seqlens_k]
    for s in range(len(cq) - 1):
        nq, nk = cq[s + 1] - cq[s], ck[s + 1] - ck[s]
        if nq <= 0:
            continue
        pos = torch.arange(nk)
        rows = block_tables[s, pos // bs].to(torch.int64) * bs + pos % bs
        k = kc.reshape(-1, num_kv_heads, head_dim)[rows]
        v = vc.reshape(-1, num_kv_heads, head_dim)[rows]
        qs = qf[cq[s]:cq[s + 1]].reshape(nq, num_kv_heads, group, head_dim)
        scores = torch.einsum("ikgd,jkd->kgij", qs, k) * scale
        qpos = (nk - nq) + torch.arange(nq)
        mask = pos[None, :] <= qpos[:, None]
        scores = scores.masked_fill(~mask, float("-inf"))
        o = torch.einsum("kgij,jkd->ikgd", torch.softmax(scores, dim=-1), v)
        out[cq[s]:cq[s + 1]] = o.reshape(nq, num_heads, head_dim)
    return out
