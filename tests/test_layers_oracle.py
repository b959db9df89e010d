"""The CPU oracle of the fused layer steps (oracle/layers_oracle.py) against outputs of the reference's own
LayerNorm and SiluAndMul modules (tests/golden/layers_small.npz), the row partition of the all-reduce, and the
all-reduce oracle's equivalence with all_reduce + add + norm in fp32."""
import os

import numpy as np
import torch

from minivllm_b200.layers.allreduce import shard_rows
from oracle import layers_oracle as oracle

HERE = os.path.dirname(os.path.abspath(__file__))


def _inputs():
    g = torch.Generator().manual_seed(50)
    x = torch.randn(11, 96, generator=g)
    residual = torch.randn(11, 96, generator=g) * 2
    gamma = torch.rand(96, generator=g) + 0.5
    gu = torch.randn(7, 2 * 40, generator=g) * 2
    return x, residual, gamma, gu


def test_oracle_matches_reference_layernorm_and_activation():
    z = np.load(os.path.join(HERE, "golden", "layers_small.npz"))
    x, residual, gamma, gu = _inputs()
    h, r = oracle.add_rms_norm(x, residual, gamma, 1e-5)
    assert np.abs(h.numpy() - z["normed"]).max() <= 2e-6
    assert np.array_equal(r.numpy(), z["new_residual"])
    assert np.abs(oracle.rms_norm(x, gamma, 1e-5).numpy() - z["plain"]).max() <= 2e-6
    assert np.abs(oracle.silu_and_mul(gu).numpy() - z["act"]).max() <= 2e-6


def test_row_partition_covers_every_row_once():
    for world in (1, 2, 3, 4, 8):
        for rows in (0, 1, 5, 8, 63, 64, 65, 512, 16384):
            spans = [shard_rows(rows, r, world) for r in range(world)]
            assert spans == [oracle.shard_rows(rows, r, world) for r in range(world)]
            covered = [i for lo, hi in spans for i in range(lo, hi)]
            assert covered == list(range(rows))
            per = (rows + world - 1) // world
            assert all(hi - lo <= per for lo, hi in spans)


def test_allreduce_oracle_is_allreduce_then_add_then_norm():
    g = torch.Generator().manual_seed(1)
    parts = [torch.randn(6, 64, generator=g) for _ in range(4)]
    residual = torch.randn(6, 64, generator=g)
    gamma = torch.rand(64, generator=g) + 0.5
    h, r = oracle.allreduce_residual_rmsnorm(parts, residual, gamma, 1e-5)
    summed = parts[0] + parts[1] + parts[2] + parts[3]
    want_h, want_r = oracle.add_rms_norm(summed, residual, gamma, 1e-5)
    assert torch.equal(r, want_r) and torch.equal(h, want_h)
    # in bf16 the sum is rounded once before the residual add (what an all-reduce leaves in the model dtype)
    pb = [p.bfloat16() for p in parts]
    hb, rb = oracle.allreduce_residual_rmsnorm(pb, residual.bfloat16(), gamma.bfloat16(), 1e-5)
    o = sum(p.float() for p in pb).bfloat16()
    assert torch.equal(rb, (o.float() + residual.bfloat16().float()).bfloat16())
