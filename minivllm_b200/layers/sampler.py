"""Sampling tail on the GPU: vocabulary-sharded logits reduced to token ids, greedy or with a temperature.

The reference computes each rank's vocabulary shard of the logits, gathers the
full matrix on rank 0 (src/myvllm/layers/embedding_head.py:56-77) and samples
there (src/myvllm/layers/sampler.py:15-19).  Greedy decoding needs none of the
gather: every rank reduces its shard to one 64-bit key per row
(`argmax_rows`), the keys are merged by an integer MAX over the ranks and
decoded to token ids (`decode_keys`); every rank ends with the same tokens.
Temperature sampling works the same way (`sample_rows`, `sampled_tokens`): the
reference's exponential race argmax(softmax(logits/T) / E) equals
argmax(logits/T - log E), a per-column score, and E comes from a counter-based
generator keyed by (seed, step, row, global column) so that every rank draws
the same noise for the same column.
"""
import torch
import torch.distributed as dist

from .. import _cabi


def argmax_rows(logits, index_offset=0, want_keys=True, want_tokens=False):
    """logits (rows, cols) fp16/bf16, last dim contiguous.  Returns (keys, tokens): int64 (rows,) each or None.

    A key orders first by logit (NaN highest, as torch.argmax), then by lower index `index_offset + column`.
    `tokens` are the indices of this shard's maxima."""
    _cabi.require_cuda(logits)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be (rows, cols) with a contiguous last dimension")
    rows, cols = logits.shape
    keys = torch.empty(rows, dtype=torch.int64, device=logits.device) if want_keys else None
    tokens = torch.empty(rows, dtype=torch.int64, device=logits.device) if want_tokens else None
    if rows:
        _cabi.check(_cabi.lib().mv_argmax_rows(
            logits.data_ptr(), logits.stride(0), rows, cols, int(index_offset),
            keys.data_ptr() if want_keys else None, tokens.data_ptr() if want_tokens else None,
            _cabi.dtype_code(logits.dtype), _cabi.stream_ptr()))
    return keys, tokens


def decode_keys(keys):
    """keys (shards, rows) or (rows,) int64 -> token ids (rows,) int64: the largest key of each row, decoded."""
    _cabi.require_cuda(keys)
    if keys.dtype != torch.int64 or not keys.is_contiguous():
        raise ValueError("keys must be a contiguous int64 tensor")
    shards, rows = (1, keys.shape[0]) if keys.dim() == 1 else keys.shape
    tokens = torch.empty(rows, dtype=torch.int64, device=keys.device)
    if rows:
        _cabi.check(_cabi.lib().mv_argmax_decode(keys.data_ptr(), shards, rows, tokens.data_ptr(), _cabi.stream_ptr()))
    return tokens


def greedy_tokens(shard_logits, index_offset=0, group=None, world_size=1):
    """Token ids (rows,) from this rank's vocabulary shard of the logits; with world_size > 1 the ranks'
    keys are merged by an all-reduce(MAX) of 8 bytes per row, so every rank returns the same ids."""
    if world_size <= 1:
        return argmax_rows(shard_logits, index_offset, want_keys=False, want_tokens=True)[1]
    keys, _ = argmax_rows(shard_logits, index_offset)
    dist.all_reduce(keys, op=dist.ReduceOp.MAX, group=group)
    return decode_keys(keys)


def sample_rows(logits, temperatures, seed, step, index_offset=0, want_keys=True, want_tokens=False):
    """Exponential-race scores of this vocabulary shard reduced to one key per row.

    logits (rows, cols) fp16/bf16; temperatures (rows,) fp32 on the device (0 = greedy row); seed: Python int
    (64 bits); step: int64 device tensor with one element, read by the kernel (advance it between calls, e.g.
    `step.add_(1)` inside a captured graph).  Returns (keys, tokens) like `argmax_rows`."""
    _cabi.require_cuda(logits, temperatures, step)
    if logits.dim() != 2 or logits.stride(1) != 1:
        raise ValueError("logits must be (rows, cols) with a contiguous last dimension")
    rows, cols = logits.shape
    if temperatures.dtype != torch.float32 or temperatures.numel() != rows or not temperatures.is_contiguous():
        raise ValueError("temperatures must be a contiguous fp32 vector with one entry per row")
    if step.dtype != torch.int64 or step.numel() != 1:
        raise ValueError("step must be an int64 tensor with one element")
    keys = torch.empty(rows, dtype=torch.int64, device=logits.device) if want_keys else None
    tokens = torch.empty(rows, dtype=torch.int64, device=logits.device) if want_tokens else None
    if rows:
        _cabi.check(_cabi.lib().mv_sample_rows(
            logits.data_ptr(), logits.stride(0), rows, cols, int(index_offset), temperatures.data_ptr(),
            int(seed) & 0xffffffffffffffff, step.data_ptr(), keys.data_ptr() if want_keys else None,
            tokens.data_ptr() if want_tokens else None, _cabi.dtype_code(logits.dtype), _cabi.stream_ptr()))
    return keys, tokens


def sampled_tokens(shard_logits, temperatures, seed, step, index_offset=0, group=None, world_size=1):
    """Token ids (rows,) drawn from softmax(logits / T) per row; with world_size > 1 each rank passes its
    vocabulary shard and the ranks merge 8 bytes per row, ending with identical ids."""
    if world_size <= 1:
        return sample_rows(shard_logits, temperatures, seed, step, index_offset, want_keys=False, want_tokens=True)[1]
    keys, _ = sample_rows(shard_logits, temperatures, seed, step, index_offset)
    dist.all_reduce(keys, op=dist.ReduceOp.MAX, group=group)
    return decode_keys(keys)
