"""Prefill attention with a cached prefix.  The reference prepares this case but never computes it, so the pin
is an equivalence: the paged oracle must reproduce the rows that the (pinned) full-sequence causal oracle gives
for the uncached positions.  The GPU kernel is then checked against the paged oracle."""
import pytest
import torch

from oracle import attention_oracle as oracle


def make_case(seed, lens, cached, H, KVH, D, bs, extra_blocks=3):
    """Full sequences of `lens` tokens with the first `cached` tokens counted as cached; K/V of ALL tokens sit in
    a paged cache (shuffled blocks); q holds only the uncached tokens."""
    g = torch.Generator().manual_seed(seed)
    T = sum(lens)
    qf = torch.randn(T, H, D, generator=g)
    kf = torch.randn(T, KVH, D, generator=g)
    vf = torch.randn(T, KVH, D, generator=g)
    nblk = [(n + bs - 1) // bs for n in lens]
    total = sum(nblk) + extra_blocks
    perm = torch.randperm(total, generator=g)
    kc = torch.randn(total, bs, KVH, D, generator=g)   # stale contents where nothing is written
    vc = torch.randn(total, bs, KVH, D, generator=g)
    bt = torch.full((len(lens), max(nblk) + 1), -1, dtype=torch.int32)
    cu_full, at, q_rows = [0], 0, []
    for s, n in enumerate(lens):
        bt[s, :nblk[s]] = perm[at:at + nblk[s]].to(torch.int32)
        at += nblk[s]
        start = cu_full[-1]
        for j in range(n):
            row = int(bt[s, j // bs]) * bs + j % bs
            kc.view(-1, KVH, D)[row] = kf[start + j]
            vc.view(-1, KVH, D)[row] = vf[start + j]
        q_rows.extend(range(start + cached[s], start + n))
        cu_full.append(start + n)
    cu_q = torch.tensor([0] + list(torch.tensor([n - c for n, c in zip(lens, cached)]).cumsum(0)), dtype=torch.int32)
    cu_k = torch.tensor(cu_full, dtype=torch.int32)
    return dict(q=qf[q_rows], q_full=qf, k_full=kf, v_full=vf, k_cache=kc, v_cache=vc, block_tables=bt, cu_q=cu_q,
                cu_k=cu_k, q_rows=q_rows, scale=D ** -0.5, H=H, KVH=KVH, D=D, bs=bs)


CASES = [
    dict(seed=1, lens=[300, 77, 513], cached=[128, 0, 256], H=4, KVH=2, D=128, bs=16),     # block-aligned prefixes
    dict(seed=2, lens=[260, 140], cached=[100, 139], H=8, KVH=2, D=128, bs=256),            # unaligned: band crosses tiles
    dict(seed=3, lens=[700, 130, 65], cached=[512, 1, 64], H=2, KVH=1, D=128, bs=64),
    dict(seed=4, lens=[1000], cached=[999], H=4, KVH=4, D=128, bs=128),                       # a single uncached token
]


@pytest.mark.parametrize("case", CASES)
def test_paged_oracle_equals_rows_of_full_causal_attention(case):
    d = make_case(**case)
    full = oracle.flash_attention_prefill(d["q_full"], d["k_full"], d["v_full"], d["cu_k"], d["scale"], d["H"],
                                          d["KVH"], d["D"])
    paged = oracle.flash_attention_prefill_paged(d["q"], d["k_cache"], d["v_cache"], d["cu_q"], d["cu_k"],
                                                 d["block_tables"], d["scale"], d["H"], d["KVH"], d["D"])
    assert float((paged - full[d["q_rows"]]).abs().max()) < 1e-5


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("case", CASES)
def test_paged_prefill_on_gpu(case, dtype):
    from minivllm_b200.layers import attention as A
    dev = "cuda:0"
    d = make_case(**case)
    r = lambda x: x.to(dtype).float()
    want = oracle.flash_attention_prefill_paged(r(d["q"]), r(d["k_cache"]), r(d["v_cache"]), d["cu_q"], d["cu_k"],
                                                d["block_tables"], d["scale"], d["H"], d["KVH"], d["D"])
    got = A.flash_attention_prefill_paged(d["q"].to(dtype).to(dev), d["k_cache"].to(dtype).to(dev),
                                          d["v_cache"].to(dtype).to(dev), d["cu_q"].to(dev), d["cu_k"].to(dev),
                                          d["block_tables"].to(dev), d["scale"], d["H"], d["KVH"], d["D"])
    torch.cuda.synchronize()
    assert A.prefill_error_code(dev) == 0
    got = got.float().cpu()
    rel = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    excess = (got - want).abs() - (2e-3 + rel * want.abs())
    assert float(excess.max()) <= 0, f"max-abs error {float((got - want).abs().max())}"


@pytest.mark.gpu
def test_paged_prefill_without_prefix_equals_packed_prefill():
    """No cached tokens at all: the paged kernel path and the packed path must agree bit for bit."""
    from minivllm_b200.layers import attention as A
    dev = "cuda:0"
    d = make_case(seed=5, lens=[333, 128, 50], cached=[0, 0, 0], H=4, KVH=2, D=128, bs=64)
    dt = torch.bfloat16
    a = A.flash_attention_prefill_paged(d["q"].to(dt).to(dev), d["k_cache"].to(dt).to(dev), d["v_cache"].to(dt).to(dev),
                                        d["cu_q"].to(dev), d["cu_k"].to(dev), d["block_tables"].to(dev), d["scale"],
                                        4, 2, 128)
    b = A.flash_attention_prefill(d["q_full"].to(dt).to(dev), d["k_full"].to(dt).to(dev), d["v_full"].to(dt).to(dev),
                                  d["cu_k"].to(dev), d["scale"], 4, 2, 128)
    torch.cuda.synchronize()
    assert torch.equal(a, b)


@pytest.mark.gpu
def test_paged_prefill_rejects_odd_block_size():
    from minivllm_b200.layers import attention as A
    dev = "cuda:0"
    kc = torch.zeros(4, 48, 1, 128, dtype=torch.float16, device=dev)
    q = torch.zeros(5, 2, 128, dtype=torch.float16, device=dev)
    cu = torch.tensor([0, 5], dtype=torch.int32, device=dev)
    with pytest.raises(ValueError):
        A.flash_attention_prefill_paged(q, kc, kc, cu, cu, torch.zeros(1, 2, dtype=torch.int32, device=dev), 0.1, 2, 1, 128)
