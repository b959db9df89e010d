"""CPU oracle for the greedy sampling tail.  TEST INFRASTRUCTURE ONLY (see
attention_oracle.py for the rules on who may import this).

Greedy decoding in the reference is the argmax of the full-vocabulary logits
that `ParallelLMHead.forward` gathers on rank 0
(src/myvllm/layers/embedding_head.py:56-77); its sampler
(src/myvllm/layers/sampler.py:15-19) draws `argmax(softmax(logits / T) / Exp(1))`,
whose T -> 0 limit is that argmax.  Restated with plain loops so that the rule
for equal logits (lowest index) and for NaN (a NaN is the maximum; the first
one wins) is explicit.  Pinned against `torch.argmax` on CPU, which follows
the same rules (tests/test_sampler.py).
"""
import math

import numpy as np


def argmax_rows(logits):
    """logits: (rows, cols) array of floats -> (rows,) int64, lowest index among equal maxima, NaN as maximum."""
    a = np.asarray(logits, dtype=np.float64)
    out = np.zeros(a.shape[0], dtype=np.int64)
    for r in range(a.shape[0]):
        best, best_i, best_nan = -math.inf, -1, False
        for i, v in enumerate(a[r]):
            if best_nan:
                break
            if math.isnan(v) or best_i < 0 or v > best:
                best, best_i, best_nan = v, i, math.isnan(v)
        out[r] = best_i
    return out


def argmax_sharded(logits, num_shards):
    """The same token ids computed the tensor-parallel way: each shard's (max, global index), merged by
    (larger value, then lower index)."""
    a = np.asarray(logits, dtype=np.float64)
    rows, cols = a.shape
    assert cols % num_shards == 0
    w = cols // num_shards
    out = np.zeros(rows, dtype=np.int64)
    for r in range(rows):
        cands = []
        for s in range(num_shards):
            i = int(argmax_rows(a[r:r + 1, s * w:(s + 1) * w])[0])
            cands.append((a[r, s * w + i], s * w + i))
        best = cands[0]
        for v, i in cands[1:]:
            bv = best[0]
            if (math.isnan(v) and not math.isnan(bv)) or (not math.isnan(bv) and v > bv):
                best = (v, i)
        out[r] = best[1]
    return out


def make_key(value, index):
    """The 64-bit key of (logit, global index) as a Python int in the signed 64-bit range: high word = the
    float32 bits mapped so that integer order is float order (NaN above +inf), low word = 2^32-1 - index."""
    v = np.float32(value)
    if np.isnan(v):
        hi = 0x7fffffff
    else:
        b = int(np.array(v, dtype=np.float32).view(np.int32))
        hi = (b ^ 0x7fffffff) if b < 0 else b
    key = ((hi & 0xffffffff) << 32) | (0xffffffff - int(index))
    return key - (1 << 64) if key >= (1 << 63) else key


def token_of_key(key):
    return 0xffffffff - (int(key) & 0xffffffff)


def shard_keys(logits, index_offset=0):
    """(rows, cols) -> list of keys of each row's maximum within this shard (what one rank contributes)."""
    a = np.asarray(logits, dtype=np.float32)
    idx = argmax_rows(a)
    return [make_key(a[r, i], index_offset + int(i)) for r, i in enumerate(idx)]
