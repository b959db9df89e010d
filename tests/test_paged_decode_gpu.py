"""paged_attention_decode on the GPU (through the C ABI) against the CPU oracle
and the reference's recorded outputs.  Tolerance: 2e-3 max-abs on fp16/bf16
outputs of N(0,1) data (fp32 accumulation on both sides)."""
import numpy as np
import pytest
import torch

from minivllm_b200 import synth
from minivllm_b200.layers import attention as A
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3


def _close(got, want, dtype):
    """2e-3 max-abs, plus one rounding step of the output dtype where |out| is large
    (a bf16 output of magnitude 1..2 is itself rounded by up to 3.9e-3)."""
    rel = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    excess = (got - want).abs() - (TOL + rel * want.abs())
    assert float(excess.max()) <= 0, f"max-abs error {float((got - want).abs().max())}"


def _gpu_decode(d, dtype, ctx_dtype=torch.int64, block_tables=None, context_lens=None):
    bt = d["block_tables"] if block_tables is None else block_tables
    cl = d["context_lens"] if context_lens is None else context_lens
    out = A.paged_attention_decode(d["q"].to(dtype).to(DEV), d["k_cache"].to(dtype).to(DEV),
                                   d["v_cache"].to(dtype).to(DEV), bt.to(DEV), cl.to(ctx_dtype).to(DEV), d["scale"],
                                   d["num_heads"], d["num_kv_heads"], d["head_dim"], d["block_size"])
    torch.cuda.synchronize()
    assert out.dtype == dtype and tuple(out.shape) == tuple(d["q"].shape)
    return out.float().cpu()


def _oracle_decode(d, dtype, block_tables=None, context_lens=None):
    bt = d["block_tables"] if block_tables is None else block_tables
    cl = d["context_lens"] if context_lens is None else context_lens
    r = lambda x: x.to(dtype).float()
    return oracle.paged_attention_decode(r(d["q"]), r(d["k_cache"]), r(d["v_cache"]), bt, cl, d["scale"],
                                         d["num_heads"], d["num_kv_heads"], d["head_dim"], d["block_size"])


@pytest.mark.parametrize("name,kw", [
    ("decode_small_bs16", dict(seed=10, batch=3, ctx_lo=5, ctx_hi=70, num_heads=4, num_kv_heads=2, head_dim=64,
                               block_size=16)),
    ("decode_gqa4_bs256", dict(seed=11, batch=4, ctx_lo=64, ctx_hi=600, num_heads=8, num_kv_heads=2, head_dim=128,
                               block_size=256)),
    ("decode_cfg0_like", dict(seed=0, batch=16, ctx_lo=64, ctx_hi=1024, num_heads=16, num_kv_heads=8, head_dim=128,
                              block_size=256)),
])
def test_decode_matches_reference_outputs(golden_dir, name, kw):
    z = np.load(f"{golden_dir}/{name}.npz")
    d = synth.decode_inputs(**kw)
    out = _gpu_decode(d, torch.float16).numpy()
    for key in z.files:
        if key != "kwargs":
            assert np.abs(out - z[key]).max() < TOL, key


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("kw", [
    dict(batch=1, ctx_lo=1, ctx_hi=1, num_heads=1, num_kv_heads=1, head_dim=64, block_size=16),
    dict(batch=2, ctx_lo=15, ctx_hi=17, num_heads=8, num_kv_heads=8, head_dim=128, block_size=16),     # MHA
    dict(batch=5, ctx_lo=1, ctx_hi=300, num_heads=8, num_kv_heads=2, head_dim=128, block_size=4),      # tiny blocks
    dict(batch=7, ctx_lo=100, ctx_hi=3000, num_heads=32, num_kv_heads=8, head_dim=128, block_size=256),
    dict(batch=3, ctx_lo=10, ctx_hi=500, num_heads=32, num_kv_heads=1, head_dim=64, block_size=48),     # G=32 -> two row tiles
    dict(batch=64, ctx_lo=1, ctx_hi=700, num_heads=4, num_kv_heads=1, head_dim=128, block_size=256),   # TP=8 shard shape
    dict(batch=300, ctx_lo=1, ctx_hi=90, num_heads=4, num_kv_heads=2, head_dim=64, block_size=32),     # batch > CTA threads
])
def test_decode_shape_sweep(dtype, kw):
    d = synth.decode_inputs(seed=40, **kw)
    got = _gpu_decode(d, dtype)
    want = _oracle_decode(d, dtype)
    _close(got, want, dtype)


def test_decode_int32_and_int64_context_lens_agree():
    d = synth.decode_inputs(seed=42, batch=6, ctx_lo=30, ctx_hi=900)
    a = _gpu_decode(d, torch.float16, ctx_dtype=torch.int64)
    b = _gpu_decode(d, torch.float16, ctx_dtype=torch.int32)
    assert torch.equal(a, b)


def test_decode_is_deterministic():
    d = synth.decode_inputs(seed=43, batch=16, ctx_lo=64, ctx_hi=1024)
    assert torch.equal(_gpu_decode(d, torch.float16), _gpu_decode(d, torch.float16))


def test_decode_negative_table_entries_and_empty_rows():
    d = synth.decode_inputs(seed=44, batch=4, ctx_lo=40, ctx_hi=64, num_heads=4, num_kv_heads=2, head_dim=128,
                            block_size=16)
    bt = d["block_tables"].clone()
    bt[0, 1] = -1                      # a hole in the middle: those 16 tokens get no weight
    cl = d["context_lens"].clone()
    cl[2] = 0                          # padded row of a captured graph: zeros out
    got = _gpu_decode(d, torch.float16, block_tables=bt, context_lens=cl)
    want = _oracle_decode(d, torch.float16, block_tables=bt, context_lens=cl)
    assert float((got - want).abs().max()) < TOL
    assert torch.count_nonzero(got[2]) == 0
    bt[3, :] = -1                      # no live token at all
    got = _gpu_decode(d, torch.float16, block_tables=bt, context_lens=cl)
    assert torch.count_nonzero(got[3]) == 0 and not torch.isnan(got).any()


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_decode_segment_cuts_on_and_off_sequence_boundaries(dtype):
    """The kernel cuts the concatenated tokens of the batch into equal segments.  37 sequences of 128 tokens with
    8 KV heads put every cut exactly on a sequence boundary; then some sequences are emptied (they own no token,
    their rows are zeros) and one is shortened, which moves every cut into the middle of a sequence."""
    d = synth.decode_inputs(seed=46, batch=37, ctx_lo=128, ctx_hi=128, num_heads=16, num_kv_heads=8, head_dim=128,
                            block_size=64)
    got, want = _gpu_decode(d, dtype), _oracle_decode(d, dtype)
    assert float((got - want).abs().max()) < TOL + (2.0 ** -8 if dtype == torch.bfloat16 else 0) * float(want.abs().max())
    cl = d["context_lens"].clone()
    cl[0] = 0
    cl[5:9] = 0
    cl[36] = 0
    cl[20] = 77
    got, want = _gpu_decode(d, dtype, context_lens=cl), _oracle_decode(d, dtype, context_lens=cl)
    assert float((got - want).abs().max()) < TOL + (2.0 ** -8 if dtype == torch.bfloat16 else 0) * float(want.abs().max())
    for b in (0, 5, 8, 36):
        assert torch.count_nonzero(got[b]) == 0


def test_decode_long_context_is_split():
    """One sequence far longer than a chunk: exercises the partial-result path and the combine kernel."""
    d = synth.decode_inputs(seed=45, batch=2, ctx_lo=9000, ctx_hi=12000, num_heads=8, num_kv_heads=2, head_dim=128,
                            block_size=256)
    got = _gpu_decode(d, torch.float16)
    want = _oracle_decode(d, torch.float16)
    assert float((got - want).abs().max()) < TOL


def test_decode_wide_table_narrow_use():
    """Graph-style call: the table is much wider than any sequence needs."""
    d = synth.decode_inputs(seed=46, batch=5, ctx_lo=20, ctx_hi=400)
    wide = torch.full((5, 64), -1, dtype=torch.int32)
    wide[:, :d["block_tables"].shape[1]] = d["block_tables"]
    got = _gpu_decode(d, torch.float16, block_tables=wide)
    want = _oracle_decode(d, torch.float16)
    assert float((got - want).abs().max()) < TOL


def test_decode_rejects_bad_arguments():
    d = synth.decode_inputs(seed=47, batch=2, ctx_lo=20, ctx_hi=40)
    q = d["q"].half().to(DEV)
    kc = d["k_cache"].half().to(DEV)
    with pytest.raises(ValueError):
        A.paged_attention_decode(q, kc, kc, d["block_tables"].to(DEV), d["context_lens"].to(DEV), 0.1, 16, 8, 128, 16)
    with pytest.raises(ValueError):
        A.paged_attention_decode(q, kc, kc, d["block_tables"].long().to(DEV), d["context_lens"].to(DEV), 0.1, 16, 8,
                                 128, 256)
