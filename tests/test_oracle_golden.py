"""The CPU oracle against outputs of the reference's own code (tests/golden,
made by tests/golden/make_golden.py).  Inputs are regenerated from seeds."""
import ast
import os

import numpy as np
import pytest
import torch

from minivllm_b200 import synth
from oracle import attention_oracle as oracle


def _load(golden_dir, name):
    z = np.load(os.path.join(golden_dir, name + ".npz"))
    return z, ast.literal_eval(str(z["kwargs"]))


def _r(x, dt):
    return x.to(dt).to(torch.float32)


@pytest.mark.parametrize("name", ["decode_small_bs16", "decode_gqa4_bs256", "decode_cfg0_like"])
def test_decode_oracle_matches_reference(golden_dir, name):
    z, kw = _load(golden_dir, name)
    d = synth.decode_inputs(**kw)
    out = oracle.paged_attention_decode(_r(d["q"], torch.float16), _r(d["k_cache"], torch.float16),
                                        _r(d["v_cache"], torch.float16), d["block_tables"], d["context_lens"],
                                        d["scale"], d["num_heads"], d["num_kv_heads"], d["head_dim"],
                                        d["block_size"]).numpy()
    for key in ("torch_optimized", "naive", "triton"):
        if key in z.files:
            # fp32 vs fp32, different summation orders only
            assert np.abs(out - z[key]).max() < 2e-5, key


@pytest.mark.parametrize("name", ["prefill_small", "prefill_gqa4"])
def test_prefill_oracle_matches_reference(golden_dir, name):
    z, kw = _load(golden_dir, name)
    d = synth.prefill_inputs(**kw)
    out = oracle.flash_attention_prefill(_r(d["q"], torch.bfloat16), _r(d["k"], torch.bfloat16),
                                         _r(d["v"], torch.bfloat16), d["cu_seqlens"], d["scale"], d["num_heads"],
                                         d["num_kv_heads"], d["head_dim"]).numpy()
    for key in ("torch_standard", "triton"):
        if key in z.files:
            assert np.abs(out - z[key]).max() < 2e-5, key


def test_store_oracle_matches_reference(golden_dir):
    z, kw = _load(golden_dir, "store_small")
    d = synth.store_inputs(**kw)
    shape = (d["num_blocks"], d["block_size"], d["num_kv_heads"], d["head_dim"])
    kc, vc = torch.full(shape, -7.0), torch.full(shape, -7.0)
    oracle.store_kvcache(_r(d["k"], torch.bfloat16), _r(d["v"], torch.bfloat16), kc, vc, d["slot_mapping"])
    assert np.array_equal(kc.numpy(), z["k_cache"])
    assert np.array_equal(vc.numpy(), z["v_cache"])
    assert (d["slot_mapping"] < 0).any(), "the fixture must exercise the -1 skip"


def test_decode_skips_negative_table_entries():
    """Triton-kernel semantics (reference attention.py:355,394): tokens of a -1 block get no weight."""
    d = synth.decode_inputs(seed=5, batch=2, ctx_lo=40, ctx_hi=48, num_heads=2, num_kv_heads=1, head_dim=64,
                            block_size=16)
    bt = d["block_tables"].clone()
    bt[0, 1] = -1
    full = oracle.paged_attention_decode(d["q"], d["k_cache"], d["v_cache"], bt, d["context_lens"], d["scale"], 2, 1,
                                         64, 16)
    # same as attending to the tokens outside [16, 32) only
    n = int(d["context_lens"][0])
    keep = [j for j in range(n) if not (16 <= j < 32)]
    rows = torch.tensor([int(d["block_tables"][0, j // 16]) * 16 + j % 16 for j in keep])
    k = d["k_cache"].reshape(-1, 1, 64)[rows, 0]
    v = d["v_cache"].reshape(-1, 1, 64)[rows, 0]
    p = torch.softmax(d["q"][0] @ k.T * d["scale"], -1)
    assert torch.allclose(full[0], p @ v, atol=1e-5)


def test_decode_empty_rows_are_zero():
    d = synth.decode_inputs(seed=6, batch=2, ctx_lo=8, ctx_hi=8, num_heads=2, num_kv_heads=1, head_dim=64,
                            block_size=16)
    cl = d["context_lens"].clone()
    cl[1] = 0
    out = oracle.paged_attention_decode(d["q"], d["k_cache"], d["v_cache"], d["block_tables"], cl, d["scale"], 2, 1,
                                        64, 16)
    assert torch.count_nonzero(out[1]) == 0 and torch.count_nonzero(out[0]) > 0
