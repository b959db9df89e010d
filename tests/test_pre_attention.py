"""q/k RMSNorm + rotary embedding (+ fused K/V store): the oracle against the reference's own LayerNorm and
RotaryEmbedding outputs (CPU), and the fused CUDA kernel against the oracle and the separate store (GPU)."""
import numpy as np
import pytest
import torch

from oracle import attention_oracle as oracle


def _inputs():
    g = torch.Generator().manual_seed(40)
    tokens, heads, kv_heads, d = 37, 4, 2, 128
    q = torch.randn(tokens, heads, d, generator=g)
    k = torch.randn(tokens, kv_heads, d, generator=g) * 3
    gamma = torch.rand(d, generator=g) + 0.5
    positions = torch.randint(0, 500, (tokens,), generator=g)
    inv = 1.0 / (1000000 ** (torch.arange(0, d, 2).float() / d))
    ang = torch.arange(512).float()[:, None] * inv[None, :]
    return q, k, gamma, positions, torch.cos(ang), torch.sin(ang)


def test_norm_rope_oracle_matches_reference_modules(golden_dir):
    z = np.load(f"{golden_dir}/prenorm_rope.npz")
    q, k, gamma, pos, cos, sin = _inputs()
    qo = oracle.qk_norm_rope(q, pos, cos, sin, gamma, 1e-5, torch.float32)
    ko = oracle.qk_norm_rope(k, pos, cos, sin, gamma, 1e-5, torch.float32)
    assert np.abs(qo.numpy() - z["q"]).max() < 1e-5
    assert np.abs(ko.numpy() - z["k"]).max() < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_norm_rope_store_on_gpu(dtype):
    from minivllm_b200.layers import attention as A
    dev = "cuda:0"
    g = torch.Generator().manual_seed(41)
    tokens, H, KVH, D, bs, nb = 300, 8, 2, 128, 16, 32
    qkv = (torch.randn(tokens, (H + 2 * KVH) * D, generator=g) * 2).to(dtype)
    gq = (torch.rand(D, generator=g) + 0.5).to(dtype)
    gk = (torch.rand(D, generator=g) + 0.5).to(dtype)
    pos = torch.randint(0, 2000, (tokens,), generator=g)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(2048).float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang), torch.sin(ang)
    slots = torch.randperm(nb * bs, generator=g)[:tokens]
    slots[torch.rand(tokens, generator=g) < 0.1] = -1
    q_in, k_in, v_in = qkv.split([H * D, KVH * D, KVH * D], dim=-1)
    want_q = oracle.qk_norm_rope(q_in.reshape(tokens, H, D), pos, cos, sin, gq, 1e-5, dtype)
    want_k = oracle.qk_norm_rope(k_in.reshape(tokens, KVH, D), pos, cos, sin, gk, 1e-5, dtype)
    kc = torch.full((nb, bs, KVH, D), 9.0, dtype=dtype, device=dev)
    vc = torch.full((nb, bs, KVH, D), 9.0, dtype=dtype, device=dev)
    # a padded leading column block makes the token stride larger than the row (like a wider fused buffer)
    wide = torch.zeros(tokens, qkv.shape[1] + 64, dtype=dtype, device=dev)
    wide[:, :qkv.shape[1]] = qkv.to(dev)
    q, k = A.qk_norm_rope_store(wide[:, :qkv.shape[1]], pos.to(dev), cos.to(dev), sin.to(dev), gq.to(dev),
                                gk.to(dev), 1e-5, H, KVH, D, kc, vc, slots.to(dev))
    torch.cuda.synchronize()
    # Almost every element is bit-equal.  Where rsqrt vs 1/sqrt or the reduction order moves the normalised
    # value across a rounding boundary (one step of the model dtype), the rotation mixes that step into both
    # outputs of the pair, so the bound is one step of the row's largest element, not of the element itself.
    ulp = 2.0 ** -7 if dtype == torch.bfloat16 else 2.0 ** -10
    for got, want in ((q.cpu(), want_q), (k.cpu(), want_k)):
        diff = (got.float() - want.float()).abs()
        row_max = want.float().abs().amax(-1, keepdim=True)
        assert float((diff - 1.5 * ulp * row_max).max()) <= 0
        assert float((diff > 0).float().mean()) < 0.02
    # the fused store equals store_kvcache of the kernel's own k and the raw v, bit for bit
    kc2 = torch.full_like(kc, 9.0)
    vc2 = torch.full_like(vc, 9.0)
    A.store_kvcache(k, v_in.reshape(tokens, KVH, D).to(dev), kc2, vc2, slots.to(dev), bs)
    torch.cuda.synchronize()
    assert torch.equal(kc, kc2) and torch.equal(vc, vc2)
    # without a slot mapping nothing is stored
    q3, k3 = A.qk_norm_rope_store(qkv.to(dev), pos.to(dev), cos.to(dev), sin.to(dev), gq.to(dev), gk.to(dev), 1e-5,
                                  H, KVH, D)
    assert torch.equal(q3, q) and torch.equal(k3, k)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_fused_norm_rope_store_into_an_int8_cache(dtype):
    """The int8 variant of the fusion: codes and fp16 scales in the cache equal, bit for bit, what the quantising
    store_kvcache writes for the kernel's own k output and the raw v (which is itself bit-exact against the
    CPU definition, tests/test_store_kvcache_gpu.py), and therefore equal the CPU quantiser applied to them."""
    from minivllm_b200.layers import attention as A
    dev = "cuda:0"
    g = torch.Generator().manual_seed(43)
    tokens, H, KVH, D, bs, nb = 257, 4, 2, 128, 16, 24
    qkv = (torch.randn(tokens, (H + 2 * KVH) * D, generator=g) * 2).to(dtype)
    qkv[5, H * D:(H + 1) * D] = 0                      # an all-zero k row: scale 0, codes 0
    qkv[7, (H + KVH) * D + 3] = 60000.0 if dtype == torch.float16 else 3e38   # a huge v element
    gam = (torch.rand(D, generator=g) + 0.5).to(dtype)
    pos = torch.randint(0, 2000, (tokens,), generator=g)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(2048).float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(dev), torch.sin(ang).to(dev)
    slots = torch.randperm(nb * bs, generator=g)[:tokens]
    slots[torch.rand(tokens, generator=g) < 0.1] = -1
    mk = lambda: (torch.full((nb, bs, KVH, D), 7, dtype=torch.int8, device=dev),
                  torch.full((nb, bs, KVH), 3.0, dtype=torch.float16, device=dev))
    (kq, ks), (vq, vs) = mk(), mk()
    q, k = A.qk_norm_rope_store(qkv.to(dev), pos.to(dev), cos, sin, gam.to(dev), gam.to(dev), 1e-5, H, KVH, D, kq, vq,
                                slots.to(dev), k_scale=ks, v_scale=vs)
    (kq2, ks2), (vq2, vs2) = mk(), mk()
    v_in = qkv[:, (H + KVH) * D:].reshape(tokens, KVH, D).to(dev)
    A.store_kvcache(k, v_in, kq2, vq2, slots.to(dev), bs, k_scale=ks2, v_scale=vs2)
    torch.cuda.synchronize()
    assert torch.equal(kq, kq2) and torch.equal(vq, vq2) and torch.equal(ks, ks2) and torch.equal(vs, vs2)
    live = slots >= 0
    codes, scales = oracle.quantize_kv_int8(k.cpu()[live])
    assert torch.equal(kq.cpu().view(-1, KVH, D)[slots[live]], codes)
    assert torch.equal(ks.cpu().view(-1, KVH)[slots[live]], scales)
    # the same q and k as the unquantised call
    kc, vc = (torch.zeros(nb, bs, KVH, D, dtype=dtype, device=dev) for _ in range(2))
    q2, k2 = A.qk_norm_rope_store(qkv.to(dev), pos.to(dev), cos, sin, gam.to(dev), gam.to(dev), 1e-5, H, KVH, D, kc, vc,
                                  slots.to(dev))
    assert torch.equal(q, q2) and torch.equal(k, k2)
