"""Small, self-contained runs of each kernel for profilers:

    python -m minivllm_b200.profile_cases {store|store_int8|decode_int8|prefill|pre_attention|argmax} [launches]

Each case holds well under 2 GB on the device, is larger than L2 where DRAM
figures matter, launches its kernel a handful of times and prints the CUDA
event time per launch.  Shapes follow the benchmark configurations.
"""
import sys

import torch

from . import synth
from .layers import attention as A

DEV = "cuda:0"


def _timed(fn, n):
    fn()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for _ in range(n):
        fn()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / n


def case_store(n, int8=False):
    s = synth.store_inputs()
    bf = torch.bfloat16
    k, v, slots = s["k"].to(bf).to(DEV), s["v"].to(bf).to(DEV), s["slot_mapping"].to(DEV)
    shape = (s["num_blocks"], s["block_size"], 8, 128)
    valid = int((s["slot_mapping"] >= 0).sum())
    if int8:
        kc, vc = torch.zeros(shape, dtype=torch.int8, device=DEV), torch.zeros(shape, dtype=torch.int8, device=DEV)
        ks = torch.zeros(shape[:3], dtype=torch.float16, device=DEV)
        vs = torch.zeros_like(ks)
        ms = _timed(lambda: A.store_kvcache(k, v, kc, vc, slots, 256, k_scale=ks, v_scale=vs), n)
        nbytes = valid * 8 * (128 * (2 * 2 + 2 * 1) + 2 * 2) + 65536 * 8
    else:
        kc, vc = torch.zeros(shape, dtype=bf, device=DEV), torch.zeros(shape, dtype=bf, device=DEV)
        ms = _timed(lambda: A.store_kvcache(k, v, kc, vc, slots, 256), n)
        nbytes = valid * 8 * 128 * (2 * 2 + 2 * 2) + 65536 * 8
    print(f"store_kvcache int8={int8}: {ms * 1e3:.1f} us/launch, algorithmic {nbytes / 1e6:.1f} MB, {nbytes / ms / 1e6:.0f} GB/s")


def case_decode_int8(n):
    d = synth.decode_inputs(seed=3, batch=64, ctx_lo=1024, ctx_hi=4096, num_heads=16, num_kv_heads=8)
    nb, bs, kvh, hd = d["k_cache"].shape
    dt = torch.float16
    kq, vq = torch.zeros(nb, bs, kvh, hd, dtype=torch.int8, device=DEV), torch.zeros(nb, bs, kvh, hd, dtype=torch.int8, device=DEV)
    ks, vs = torch.zeros(nb, bs, kvh, dtype=torch.float16, device=DEV), torch.zeros(nb, bs, kvh, dtype=torch.float16, device=DEV)
    slots = torch.arange(nb * bs, dtype=torch.int64, device=DEV)
    A.store_kvcache(d["k_cache"].reshape(-1, kvh, hd).to(dt).to(DEV), d["v_cache"].reshape(-1, kvh, hd).to(dt).to(DEV),
                    kq, vq, slots, bs, k_scale=ks, v_scale=vs)
    q, bt, cl = d["q"].to(dt).to(DEV), d["block_tables"].to(DEV), d["context_lens"].to(DEV)
    ms = _timed(lambda: A.paged_attention_decode(q, kq, vq, bt, cl, d["scale"], 16, 8, 128, 256, k_scale=ks, v_scale=vs), n)
    nbytes = synth.decode_bytes(d["context_lens"], 64, 16, 8, 128, 2, bt.shape[1], int8=True)
    print(f"paged decode int8: {ms * 1e3:.1f} us/launch, algorithmic {nbytes / 1e6:.1f} MB, {nbytes / ms / 1e6:.0f} GB/s")


def case_argmax(n):
    """Greedy tail on decode-sized logits: 512 rows x 151,936 columns bf16 (the full vocabulary of one rank at TP=1)."""
    from minivllm_b200.layers import sampler as S
    g = torch.Generator().manual_seed(5)
    x = torch.randn(512, 151936, generator=g).to(torch.bfloat16).to(DEV)
    ms = _timed(lambda: S.argmax_rows(x, want_keys=False, want_tokens=True), n)
    ref = _timed(lambda: x.argmax(dim=-1), n)
    same = bool((S.argmax_rows(x, want_keys=False, want_tokens=True)[1] == x.float().argmax(dim=-1)).all())
    nbytes = x.numel() * 2 + 512 * 8
    print(f"argmax_rows 512x151936 bf16: {ms * 1e3:.1f} us/launch, algorithmic {nbytes / 1e6:.1f} MB, "
          f"{nbytes / ms / 1e6:.0f} GB/s; torch.argmax {ref * 1e3:.1f} us; same tokens {same}")


def case_prefill(n):
    p = synth.prefill_inputs()
    bf = torch.bfloat16
    q, k, v, cu = p["q"].to(bf).to(DEV), p["k"].to(bf).to(DEV), p["v"].to(bf).to(DEV), p["cu_seqlens"].to(DEV)
    ms = _timed(lambda: A.flash_attention_prefill(q, k, v, cu, p["scale"], 32, 8, 128), n)
    fl = synth.prefill_flops(p["lens"], 32, 128)
    print(f"prefill varlen: {ms:.3f} ms/launch, {fl / 1e9:.1f} GFLOP, {fl / ms / 1e9:.0f} TFLOP/s, "
          f"error word {A.prefill_error_code(DEV)}")


def case_pre_attention(n):
    g = torch.Generator().manual_seed(5)
    tokens, H, KVH, D = 16384, 32, 8, 128
    bf = torch.bfloat16
    qkv = torch.randn(tokens, (H + 2 * KVH) * D, generator=g).to(bf).to(DEV)
    gam = torch.ones(D, dtype=bf, device=DEV)
    pos = torch.randint(0, 2048, (tokens,), generator=g).to(DEV)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(2048).float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(DEV), torch.sin(ang).to(DEV)
    kc = torch.zeros(128, 256, KVH, D, dtype=bf, device=DEV)
    vc = torch.zeros_like(kc)
    slots = torch.randperm(128 * 256, generator=g)[:tokens].to(DEV)
    ms = _timed(lambda: A.qk_norm_rope_store(qkv, pos, cos, sin, gam, gam, 1e-5, H, KVH, D, kc, vc, slots), n)
    nbytes = tokens * ((H + 2 * KVH) * D * 2 + (H + KVH) * D * 2 + 2 * KVH * D * 2 + 16)
    print(f"qk_norm_rope_store: {ms * 1e3:.1f} us/launch, algorithmic {nbytes / 1e6:.1f} MB, {nbytes / ms / 1e6:.0f} GB/s")


def main():
    case = sys.argv[1] if len(sys.argv) > 1 else "store"
    n = int(sys.argv[2]) if len(sys.argv) > 2 else 3
    {"store": lambda: case_store(n), "store_int8": lambda: case_store(n, True), "decode_int8": lambda: case_decode_int8(n),
     "prefill": lambda: case_prefill(n), "pre_attention": lambda: case_pre_attention(n),
     "argmax": lambda: case_argmax(n)}[case]()


if __name__ == "__main__":
    main()
