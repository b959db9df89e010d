"""store_kvcache on the GPU (through the C ABI) against the CPU oracle: bit-exact."""
import numpy as np
import pytest
import torch

from minivllm_b200 import synth
from minivllm_b200.layers import attention as A
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _run_copy(d, dtype, fill=-7.0, token_stride_pad=0):
    shape = (d["num_blocks"], d["block_size"], d["num_kv_heads"], d["head_dim"])
    k, v = d["k"].to(dtype), d["v"].to(dtype)
    kc_ref, vc_ref = torch.full(shape, fill, dtype=dtype), torch.full(shape, fill, dtype=dtype)
    oracle.store_kvcache(k, v, kc_ref, vc_ref, d["slot_mapping"])
    kc, vc = torch.full(shape, fill, dtype=dtype, device=DEV), torch.full(shape, fill, dtype=dtype, device=DEV)
    if token_stride_pad:
        # k and v as split views of one fused (tokens, (KVH*2 + pad) * D) buffer, like qkv.split()
        kvh, hd = d["num_kv_heads"], d["head_dim"]
        fused = torch.zeros(k.shape[0], (2 * kvh + token_stride_pad) * hd, dtype=dtype, device=DEV)
        fused[:, token_stride_pad * hd:(token_stride_pad + kvh) * hd] = k.reshape(k.shape[0], -1).to(DEV)
        fused[:, (token_stride_pad + kvh) * hd:] = v.reshape(v.shape[0], -1).to(DEV)
        _, kg, vg = fused.split([token_stride_pad * hd, kvh * hd, kvh * hd], dim=-1)
        kg, vg = kg.view(-1, kvh, hd), vg.view(-1, kvh, hd)
        assert not vg.is_contiguous()
    else:
        kg, vg = k.to(DEV), v.to(DEV)
    A.store_kvcache(kg, vg, kc, vc, d["slot_mapping"].to(DEV), d["block_size"])
    torch.cuda.synchronize()
    assert torch.equal(kc.cpu().view(torch.int16), kc_ref.view(torch.int16))
    assert torch.equal(vc.cpu().view(torch.int16), vc_ref.view(torch.int16))


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_store_matches_golden_case(golden_dir, dtype):
    d = synth.store_inputs(seed=30, num_tokens=40, num_blocks=8, block_size=16, num_kv_heads=2, head_dim=64,
                           pad_frac=0.2)
    _run_copy(d, dtype)
    if dtype == torch.bfloat16:
        z = np.load(f"{golden_dir}/store_small.npz")
        shape = (8, 16, 2, 64)
        kc = torch.full(shape, -7.0, dtype=dtype, device=DEV)
        vc = torch.full(shape, -7.0, dtype=dtype, device=DEV)
        A.store_kvcache(d["k"].to(dtype).to(DEV), d["v"].to(dtype).to(DEV), kc, vc, d["slot_mapping"].to(DEV), 16)
        assert np.array_equal(kc.float().cpu().numpy(), z["k_cache"])
        assert np.array_equal(vc.float().cpu().numpy(), z["v_cache"])


@pytest.mark.parametrize("kw", [
    dict(num_tokens=1, num_blocks=2, block_size=4, num_kv_heads=1, head_dim=64),
    dict(num_tokens=777, num_blocks=16, block_size=64, num_kv_heads=4, head_dim=128),
    dict(num_tokens=5000, num_blocks=40, block_size=256, num_kv_heads=8, head_dim=128),
    dict(num_tokens=300, num_blocks=3, block_size=128, num_kv_heads=3, head_dim=256),
])
def test_store_shapes(kw):
    _run_copy(synth.store_inputs(seed=31, pad_frac=0.1, **kw), torch.bfloat16)


def test_store_reads_split_views_in_place():
    d = synth.store_inputs(seed=32, num_tokens=513, num_blocks=8, block_size=128, num_kv_heads=2, head_dim=128)
    _run_copy(d, torch.bfloat16, token_stride_pad=4)


def test_store_full_config_bit_exact():
    """65,536 tokens into a 4,096 x 256-slot cache, ~3% padding slots."""
    d = synth.store_inputs()
    _run_copy(d, torch.bfloat16, fill=0.0)


def test_store_empty_and_all_padding():
    shape = (2, 16, 2, 64)
    kc = torch.full(shape, 3.0, dtype=torch.float16, device=DEV)
    vc = kc.clone()
    A.store_kvcache(torch.zeros(0, 2, 64, dtype=torch.float16, device=DEV),
                    torch.zeros(0, 2, 64, dtype=torch.float16, device=DEV), kc, vc,
                    torch.zeros(0, dtype=torch.int64, device=DEV), 16)
    k = torch.ones(5, 2, 64, dtype=torch.float16, device=DEV)
    A.store_kvcache(k, k, kc, vc, torch.full((5,), -1, dtype=torch.int64, device=DEV), 16)
    torch.cuda.synchronize()
    assert bool((kc == 3).all()) and bool((vc == 3).all())


def test_store_rejects_wrong_block_size_and_sizes():
    kc = torch.zeros(2, 16, 2, 64, dtype=torch.float16, device=DEV)
    k = torch.zeros(5, 2, 64, dtype=torch.float16, device=DEV)
    with pytest.raises(ValueError):
        A.store_kvcache(k, k, kc, kc.clone(), torch.zeros(5, dtype=torch.int64, device=DEV), 32)
    with pytest.raises(AssertionError):
        A.store_kvcache(k, k, kc, kc.clone(), torch.zeros(4, dtype=torch.int64, device=DEV), 16)


def _run_quant(d, dtype):
    nb, bs, kvh, hd = d["num_blocks"], d["block_size"], d["num_kv_heads"], d["head_dim"]
    k, v = d["k"].to(dtype), d["v"].to(dtype)
    ref = [torch.zeros(nb, bs, kvh, hd, dtype=torch.int8), torch.zeros(nb, bs, kvh, hd, dtype=torch.int8),
           torch.zeros(nb, bs, kvh, dtype=torch.float16), torch.zeros(nb, bs, kvh, dtype=torch.float16)]
    oracle.store_kvcache_int8(k, v, *ref, d["slot_mapping"])
    got = [torch.zeros_like(t, device=DEV) for t in ref]
    A.store_kvcache(k.to(DEV), v.to(DEV), got[0], got[1], d["slot_mapping"].to(DEV), bs, k_scale=got[2],
                    v_scale=got[3])
    torch.cuda.synchronize()
    for name, a, b in zip(("k_codes", "v_codes", "k_scale", "v_scale"), got, ref):
        if a.dtype == torch.float16:
            assert torch.equal(a.cpu().view(torch.int16), b.view(torch.int16)), name
        else:
            assert torch.equal(a.cpu(), b), name
    return got


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("hd", [64, 128, 256])
def test_store_int8_bit_exact_small(dtype, hd):
    d = synth.store_inputs(seed=33, num_tokens=1000, num_blocks=8, block_size=256, num_kv_heads=2, head_dim=hd,
                           pad_frac=0.1)
    d["k"][0] = 0            # zero row -> scale 0, codes 0
    d["k"][1] *= 1e-6        # subnormal fp16 scale
    d["v"][2] *= 1e-9        # scale underflows to 0
    # exact ties: amax 127 -> scale 1.0, then k + 1/2 values must round to even
    ties = torch.tensor([0.5, 1.5, 2.5, -0.5, -1.5, -2.5, 3.5, 12.5, 100.5, -100.5, 63.5, -64.5, 126.5, 127.0])
    d["k"][3, 0, :14] = ties
    d["k"][3, 0, 14:] = 0.25
    d["v"][4, 1, :14] = ties * 0.5   # scale 0.5, same ties
    d["v"][4, 1, 14:] = 0.125
    if dtype == torch.bfloat16:
        d["k"][5] *= 1e7             # amax/127 exceeds fp16 range: scale inf -> codes 0
    _run_quant(d, dtype)


def test_store_int8_full_config_bit_exact():
    d = synth.store_inputs()
    codes = _run_quant(d, torch.bfloat16)[0]
    assert int(codes.min()) == -127 and int(codes.max()) == 127
