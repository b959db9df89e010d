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
    float32 bits mapped so that integer order is float order (NaN above +inf, -0.0 as +0.0), low word = 2^32-1 - index."""
    v = np.float32(value)
    if np.isnan(v):
        hi = 0x7fffffff
    else:
        b = int(np.array(v, dtype=np.float32).view(np.int32))
        if v == 0:
            b = 0                      # -0.0 and +0.0 are equal logits: one key, the lower index wins
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


# ---- temperature sampling: the exponential race of src/myvllm/layers/sampler.py:15-19 ---------------------
# argmax_i softmax(logits/T)_i / E_i  ==  argmax_i (logits_i / T - log E_i).  The CUDA kernel draws E_i from
# Philox4x32-10 (Salmon et al., "Parallel random numbers: as easy as 1, 2, 3", SC'11) with key = seed and
# counter = (global column // 4, row, step); this is that generator restated with Python integers.
_M0, _M1, _W0, _W1 = 0xD2511F53, 0xCD9E8D57, 0x9E3779B9, 0xBB67AE85


def philox4x32_10(counter, key):
    """counter: 4 uint32, key: 2 uint32 -> 4 uint32."""
    c0, c1, c2, c3 = (int(x) & 0xffffffff for x in counter)
    k0, k1 = (int(x) & 0xffffffff for x in key)
    for _ in range(10):
        p0, p1 = _M0 * c0, _M1 * c2
        c0, c1, c2, c3 = ((p1 >> 32) ^ c1 ^ k0) & 0xffffffff, p1 & 0xffffffff, ((p0 >> 32) ^ c3 ^ k1) & 0xffffffff, \
            p0 & 0xffffffff
        k0, k1 = (k0 + _W0) & 0xffffffff, (k1 + _W1) & 0xffffffff
    return c0, c1, c2, c3


def race_bits(seed, step, row, column):
    """The 32 random bits of (row, global column) at `step`."""
    words = philox4x32_10((column >> 2, row, step & 0xffffffff, (step >> 32) & 0xffffffff),
                          (seed & 0xffffffff, (seed >> 32) & 0xffffffff))
    return words[column & 3]


def race_scores(logits, temperatures, seed, step, index_offset=0):
    """(rows, cols) float32 scores logit / T - log E with E = -log(u), u = (top 24 bits + 0.5) / 2^24;
    a row with temperature 0 keeps its logits (greedy)."""
    a = np.asarray(logits, dtype=np.float32)
    out = np.empty_like(a)
    for r in range(a.shape[0]):
        t = float(temperatures[r])
        if not t > 0:
            out[r] = a[r]
            continue
        bits = np.array([race_bits(seed, step, r, index_offset + c) for c in range(a.shape[1])], dtype=np.uint64)
        u = ((bits >> np.uint64(8)).astype(np.float32) + np.float32(0.5)) * np.float32(1.0 / 16777216.0)
        noise = -np.log(-np.log(u.astype(np.float64)))
        out[r] = (a[r].astype(np.float32) * np.float32(1.0 / t)).astype(np.float64) + noise
    return out


def sample_rows(logits, temperatures, seed, step, index_offset=0):
    """Token ids the race selects (lowest index among equal scores), and the scores."""
    sc = race_scores(logits, temperatures, seed, step, index_offset)
    return argmax_rows(sc) + index_offset, sc
