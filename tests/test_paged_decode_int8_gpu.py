"""Paged decode over an int8 KV cache: the cache is filled by the quantising
store_kvcache (bit-exact against the oracle, see test_store_kvcache_gpu.py) and
the attention output must be within 2e-3 max-abs of the fp32 oracle run on the
DEQUANTISED cache (float(code) * float(scale))."""
import pytest
import torch

from minivllm_b200 import synth
from minivllm_b200.layers import attention as A
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3


def _build_int8_cache(d, dtype, std=1.0):
    """Writes every slot of the synthetic cache through store_kvcache(int8) in one call."""
    nb, bs, kvh, hd = d["k_cache"].shape
    slots = torch.arange(nb * bs, dtype=torch.int64)
    k = (d["k_cache"] * std).reshape(-1, kvh, hd).to(dtype)
    v = (d["v_cache"] * std).reshape(-1, kvh, hd).to(dtype)
    kq = torch.zeros(nb, bs, kvh, hd, dtype=torch.int8, device=DEV)
    vq = torch.zeros_like(kq)
    ks = torch.zeros(nb, bs, kvh, dtype=torch.float16, device=DEV)
    vs = torch.zeros_like(ks)
    A.store_kvcache(k.to(DEV), v.to(DEV), kq, vq, slots.to(DEV), bs, k_scale=ks, v_scale=vs)
    torch.cuda.synchronize()
    kdq = oracle.dequantize_kv_int8(kq.cpu(), ks.cpu())
    vdq = oracle.dequantize_kv_int8(vq.cpu(), vs.cpu())
    return (kq, vq, ks, vs), (kdq, vdq)


def _check(d, dtype, std=1.0, block_tables=None, context_lens=None):
    bt = d["block_tables"] if block_tables is None else block_tables
    cl = d["context_lens"] if context_lens is None else context_lens
    (kq, vq, ks, vs), (kdq, vdq) = _build_int8_cache(d, dtype, std)
    got = A.paged_attention_decode(d["q"].to(dtype).to(DEV), kq, vq, bt.to(DEV), cl.to(DEV), d["scale"],
                                   d["num_heads"], d["num_kv_heads"], d["head_dim"], d["block_size"], k_scale=ks,
                                   v_scale=vs)
    torch.cuda.synchronize()
    assert got.dtype == dtype
    want = oracle.paged_attention_decode(d["q"].to(dtype).float(), kdq, vdq, bt, cl, d["scale"], d["num_heads"],
                                         d["num_kv_heads"], d["head_dim"], d["block_size"])
    got = got.float().cpu()
    rel = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    excess = (got - want).abs() - (TOL + rel * want.abs())
    assert float(excess.max()) <= 0, f"max-abs error {float((got - want).abs().max())}"
    return got


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_int8_decode_config_shape(dtype):
    """Batch 16, ctx in [64,1024], 16 q / 8 kv heads, head_dim 128, 256-token blocks, N(0,2) values."""
    _check(synth.decode_inputs(seed=0), dtype, std=2.0)


@pytest.mark.parametrize("kw", [
    dict(batch=1, ctx_lo=1, ctx_hi=1, num_heads=1, num_kv_heads=1, block_size=16),
    dict(batch=5, ctx_lo=1, ctx_hi=300, num_heads=8, num_kv_heads=2, block_size=4),
    dict(batch=9, ctx_lo=100, ctx_hi=3000, num_heads=32, num_kv_heads=8, block_size=256),
    dict(batch=3, ctx_lo=10, ctx_hi=500, num_heads=32, num_kv_heads=1, block_size=48),   # two row tiles; odd scale indices
    dict(batch=40, ctx_lo=1, ctx_hi=700, num_heads=4, num_kv_heads=1, block_size=256),
    dict(batch=4, ctx_lo=200, ctx_hi=900, num_heads=9, num_kv_heads=3, block_size=32),   # odd kv head count
])
def test_int8_decode_shape_sweep(kw):
    _check(synth.decode_inputs(seed=50, head_dim=128, **kw), torch.float16)


def test_int8_decode_long_context_split_and_holes():
    d = synth.decode_inputs(seed=51, batch=2, ctx_lo=5000, ctx_hi=9000, num_heads=8, num_kv_heads=2, block_size=256)
    bt = d["block_tables"].clone()
    bt[0, 3] = -1
    cl = d["context_lens"].clone()
    got = _check(d, torch.float16, block_tables=bt, context_lens=cl)
    assert not torch.isnan(got).any()


def test_int8_decode_rejects_head_dim_64():
    d = synth.decode_inputs(seed=52, batch=2, ctx_lo=10, ctx_hi=20, num_heads=2, num_kv_heads=1, head_dim=64,
                            block_size=16)
    kq = torch.zeros(d["k_cache"].shape, dtype=torch.int8, device=DEV)
    ks = torch.zeros(d["k_cache"].shape[:3], dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        A.paged_attention_decode(d["q"].half().to(DEV), kq, kq, d["block_tables"].to(DEV), d["context_lens"].to(DEV),
                                 d["scale"], 2, 1, 64, 16, k_scale=ks, v_scale=ks)
