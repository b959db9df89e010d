"""The paged-decode work plan, restated on the CPU from minivllm_b200/csrc/paged_decode.cuh (build_plan,
seq_items, piece_of, walk_*) and checked for the properties the kernels rely on: every KV token of the batch is
covered by exactly one work item, item ids are unique, contiguous per sequence and below the bound the scratch
is sized with, units are equal in length, and the walk of a CTA visits exactly the items of its units."""
import random

K_CTA_TOK = 64          # kTileTok * kDecWarps
NUM_SMS, CTAS_PER_SM, WAVES = 148, 2, 1


def target_items(num_kv_heads, mtiles):
    return max((NUM_SMS * CTAS_PER_SM * WAVES) // (num_kv_heads * mtiles), 1)


def items_max(batch, num_kv_heads, mtiles):
    return target_items(num_kv_heads, mtiles) + batch


def build_plan(ctx, target):
    s_tok = [0]
    for c in ctx:
        s_tok.append(s_tok[-1] + c)
    total = s_tok[-1]
    seg = (total + target - 1) // target
    seg = max(((seg + K_CTA_TOK - 1) // K_CTA_TOK) * K_CTA_TOK, K_CTA_TOK)
    return s_tok, seg, (total + seg - 1) // seg


def seq_items(s_tok, seg_len, b):
    t0, t1 = s_tok[b], s_tok[b + 1]
    if t1 <= t0:
        return (0, 0)
    s0, s1 = t0 // seg_len, (t1 - 1) // seg_len
    return (b + s0, s1 - s0 + 1)


def seq_at(s_tok, batch, pos):
    lo, hi = 0, batch - 1
    while lo < hi:
        mid = (lo + hi + 1) >> 1
        if s_tok[mid] <= pos:
            lo = mid
        else:
            hi = mid - 1
    return lo


def piece_of(s_tok, seg_len, b, seg):
    t0, t1 = s_tok[b], s_tok[b + 1]
    g0, g1 = seg * seg_len, (seg + 1) * seg_len
    return dict(b=b, item=b + seg, tok_begin=max(g0 - t0, 0), tok_end=min(g1, t1) - t0,
                nsplit=(t1 - 1) // seg_len - t0 // seg_len + 1)


def walk(s_tok, batch, seg_len, n_seg, ydim, first, stride):
    """Items (seg, y, piece) of the units first, first + stride, ... in the order a CTA visits them."""
    out, unit, n_units = [], first, n_seg * ydim
    while unit < n_units:
        seg, y = divmod(unit, ydim)
        b = seq_at(s_tok, batch, seg * seg_len)
        while True:
            out.append((seg, y, piece_of(s_tok, seg_len, b, seg)))
            b += 1
            while b < batch and s_tok[b + 1] == s_tok[b]:
                b += 1
            if not (b < batch and s_tok[b] < (seg + 1) * seg_len):
                break
        unit += stride
    return out


def _check(ctx, num_kv_heads, mtiles, grid):
    batch, ydim = len(ctx), num_kv_heads * mtiles
    target = target_items(num_kv_heads, mtiles)
    s_tok, seg_len, n_seg = build_plan(ctx, target)
    assert n_seg <= target and seg_len % K_CTA_TOK == 0
    covered = {}                       # (y, b) -> token intervals
    ids = {}                           # y -> item ids seen
    for cta in range(grid):
        for seg, y, p in walk(s_tok, batch, seg_len, n_seg, ydim, cta, grid):
            assert 0 <= p["tok_begin"] < p["tok_end"] <= ctx[p["b"]]
            assert p["tok_end"] - p["tok_begin"] <= seg_len
            first, count = seq_items(s_tok, seg_len, p["b"])
            assert count == p["nsplit"] and first <= p["item"] < first + count
            assert p["item"] < items_max(batch, num_kv_heads, mtiles)
            assert p["item"] not in ids.setdefault(y, set())
            ids[y].add(p["item"])
            covered.setdefault((y, p["b"]), []).append((p["tok_begin"], p["tok_end"]))
    for y in range(ydim):
        for b, c in enumerate(ctx):
            iv = sorted(covered.get((y, b), []))
            if c == 0:
                assert not iv and seq_items(s_tok, seg_len, b) == (0, 0)
                continue
            assert iv[0][0] == 0 and iv[-1][1] == c
            assert all(a[1] == b_[0] for a, b_ in zip(iv, iv[1:]))      # no gap, no overlap
            assert len(iv) == seq_items(s_tok, seg_len, b)[1]
    if sum(ctx) == 0:
        assert n_seg == 0


def test_plan_covers_every_token_once_on_random_batches():
    rng = random.Random(0)
    for _ in range(60):
        batch = rng.choice([1, 2, 7, 37, 130, 300])
        hi = rng.choice([1, 60, 128, 700, 5000])
        ctx = [rng.choice([0, rng.randint(1, hi)]) if rng.random() < 0.2 else rng.randint(1, hi) for _ in range(batch)]
        kvh, mt = rng.choice([(1, 1), (2, 1), (8, 1), (1, 2), (4, 1)])
        _check(ctx, kvh, mt, grid=rng.choice([1, 5, 296]))


def test_plan_edge_cases():
    _check([0, 0, 0], 2, 1, 296)                     # nothing to do at all
    _check([128] * 37, 8, 1, 296)                    # every cut on a sequence boundary
    _check([64] * 592, 1, 1, 296)                    # one segment per sequence
    _check([1], 8, 1, 296)
    _check([100000], 1, 1, 296)                      # one sequence over all segments
    _check([0, 5, 0, 0, 70000, 0, 3, 0], 1, 1, 296)
