"""flash_attention_prefill on the GPU (tcgen05 kernel, through the C ABI)
against the fp32 CPU oracle and the reference's recorded outputs.
Tolerance: 2e-3 max-abs plus one rounding step of the output dtype."""
import numpy as np
import pytest
import torch

import ctypes

from minivllm_b200 import _cabi, synth
from minivllm_b200.layers import attention as A
from oracle import attention_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
TOL = 2e-3


def _close(got, want, dtype):
    rel = 2.0 ** -8 if dtype == torch.bfloat16 else 2.0 ** -11
    excess = (got - want).abs() - (TOL + rel * want.abs())
    assert float(excess.max()) <= 0, f"max-abs error {float((got - want).abs().max())}"


def _gpu(d, dtype, q=None, k=None, v=None):
    q = d["q"].to(dtype).to(DEV) if q is None else q
    k = d["k"].to(dtype).to(DEV) if k is None else k
    v = d["v"].to(dtype).to(DEV) if v is None else v
    out = A.flash_attention_prefill(q, k, v, d["cu_seqlens"].to(DEV), d["scale"], d["num_heads"], d["num_kv_heads"],
                                    d["head_dim"])
    torch.cuda.synchronize()
    assert A.prefill_error_code(DEV) == 0, "a kernel wait ran out of time"
    assert out.dtype == dtype and tuple(out.shape) == tuple(d["q"].shape)
    return out.float().cpu()


def _oracle(d, dtype):
    r = lambda x: x.to(dtype).float()
    return oracle.flash_attention_prefill(r(d["q"]), r(d["k"]), r(d["v"]), d["cu_seqlens"], d["scale"],
                                          d["num_heads"], d["num_kv_heads"], d["head_dim"])


def test_prefill_matches_reference_outputs(golden_dir):
    z = np.load(f"{golden_dir}/prefill_gqa4.npz")
    d = synth.prefill_inputs(seed=21, num_seqs=3, len_lo=40, len_hi=200, num_heads=8, num_kv_heads=2, head_dim=128)
    got = _gpu(d, torch.bfloat16)
    for key in ("torch_standard", "triton"):
        _close(got, torch.from_numpy(z[key]), torch.bfloat16)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("kw", [
    dict(num_seqs=1, len_lo=1, len_hi=1, num_heads=2, num_kv_heads=1),          # a single token
    dict(num_seqs=1, len_lo=128, len_hi=128, num_heads=2, num_kv_heads=1),      # exactly one tile
    dict(num_seqs=1, len_lo=129, len_hi=129, num_heads=2, num_kv_heads=1),      # one row into the second tile
    dict(num_seqs=5, len_lo=1, len_hi=300, num_heads=4, num_kv_heads=2),        # ragged, shorter than a tile too
    dict(num_seqs=3, len_lo=200, len_hi=700, num_heads=8, num_kv_heads=8),      # MHA: one head per CTA
    dict(num_seqs=2, len_lo=300, len_hi=520, num_heads=6, num_kv_heads=2),      # odd group: a pair plus a single
    dict(num_seqs=4, len_lo=500, len_hi=1100, num_heads=8, num_kv_heads=1),     # MQA, four pairs
])
def test_prefill_shape_sweep(dtype, kw):
    d = synth.prefill_inputs(seed=60, head_dim=128, **kw)
    _close(_gpu(d, dtype), _oracle(d, dtype), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prefill_more_tiles_than_sms_with_odd_group(dtype):
    """Several hundred (tile, head pair) units with a group of three heads (a pair plus a single head): every
    SM works through many units, of different lengths and with and without a second head."""
    d = synth.prefill_inputs(seed=61, num_seqs=14, len_lo=250, len_hi=900, num_heads=6, num_kv_heads=2, head_dim=128)
    _close(_gpu(d, dtype), _oracle(d, dtype), dtype)


def test_prefill_batch_of_many_short_sequences():
    """More sequences than the kernel keeps a tile table for in shared memory, some of them empty."""
    g = torch.Generator().manual_seed(62)
    lens = torch.randint(0, 40, (1100,), generator=g)
    lens[::97] = 0
    lens[5] = 300
    cu = torch.zeros(1101, dtype=torch.int32)
    cu[1:] = torch.cumsum(lens, 0)
    total = int(cu[-1])
    d = dict(q=torch.randn(total, 2, 128, generator=g), k=torch.randn(total, 1, 128, generator=g),
             v=torch.randn(total, 1, 128, generator=g), cu_seqlens=cu, scale=128 ** -0.5, num_heads=2, num_kv_heads=1,
             head_dim=128)
    _close(_gpu(d, torch.float16), _oracle(d, torch.float16), torch.float16)


def test_prefill_long_sequence_and_large_logits():
    """2,048-token sequences (16 KV tiles), then a scale that makes the running maximum jump by far more
    than the lazy-rescale threshold, so O in tensor memory is rescaled."""
    d = synth.prefill_inputs(seed=61, num_seqs=2, len_lo=1500, len_hi=2048, num_heads=4, num_kv_heads=2)
    _close(_gpu(d, torch.bfloat16), _oracle(d, torch.bfloat16), torch.bfloat16)
    _close(_gpu(d, torch.float16), _oracle(d, torch.float16), torch.float16)
    d["scale"] = 1.0  # logits ~ N(0, 128): every row is dominated by one or two keys
    _close(_gpu(d, torch.float16), _oracle(d, torch.float16), torch.float16)
    # With such peaked rows the 8-bit rounding of the weights themselves (P is bf16 on the tensor cores, as
    # in the reference's `p.to(v.dtype)`) is visible: bound it by the reference's own bf16 error level.
    err = (_gpu(d, torch.bfloat16) - _oracle(d, torch.bfloat16)).abs().max()
    assert float(err) < 2.5e-2


def test_prefill_reads_split_views_in_place():
    d = synth.prefill_inputs(seed=62, num_seqs=3, len_lo=50, len_hi=400, num_heads=4, num_kv_heads=2)
    dt = torch.bfloat16
    T = d["q"].shape[0]
    fused = torch.cat([d["q"].reshape(T, -1), d["k"].reshape(T, -1), d["v"].reshape(T, -1)], dim=-1).to(dt).to(DEV)
    q, k, v = fused.split([4 * 128, 2 * 128, 2 * 128], dim=-1)
    q, k, v = q.view(T, 4, 128), k.view(T, 2, 128), v.view(T, 2, 128)
    assert not v.is_contiguous()
    _close(_gpu(d, dt, q=q, k=k, v=v), _oracle(d, dt), dt)


def test_prefill_is_deterministic_and_handles_empty():
    d = synth.prefill_inputs(seed=63, num_seqs=4, len_lo=100, len_hi=600, num_heads=4, num_kv_heads=2)
    assert torch.equal(_gpu(d, torch.bfloat16), _gpu(d, torch.bfloat16))
    out = A.flash_attention_prefill(torch.zeros(0, 4, 128, dtype=torch.bfloat16, device=DEV),
                                    torch.zeros(0, 2, 128, dtype=torch.bfloat16, device=DEV),
                                    torch.zeros(0, 2, 128, dtype=torch.bfloat16, device=DEV),
                                    torch.zeros(1, dtype=torch.int32, device=DEV), 0.1, 4, 2, 128)
    assert out.shape[0] == 0


def test_prefill_zero_length_sequences_in_batch():
    d = synth.prefill_inputs(seed=64, num_seqs=3, len_lo=60, len_hi=200, num_heads=2, num_kv_heads=1)
    cu = d["cu_seqlens"]
    d["cu_seqlens"] = torch.tensor([0, int(cu[1]), int(cu[1]), int(cu[2]), int(cu[3]), int(cu[3])], dtype=torch.int32)
    _close(_gpu(d, torch.float16), _oracle(d, torch.float16), torch.float16)


def test_prefill_rejects_head_dim_64():
    d = synth.prefill_inputs(seed=65, num_seqs=1, len_lo=10, len_hi=10, num_heads=2, num_kv_heads=1, head_dim=64)
    with pytest.raises(ValueError):
        A.flash_attention_prefill(d["q"].half().to(DEV), d["k"].half().to(DEV), d["v"].half().to(DEV),
                                  d["cu_seqlens"].to(DEV), 0.1, 2, 1, 64)


def _call_c_abi(d, dtype, out, error_word):
    q, k, v = (d[n].to(dtype).to(DEV) for n in ("q", "k", "v"))
    cu = d["cu_seqlens"].to(DEV)
    h, kvh, hd = d["num_heads"], d["num_kv_heads"], d["head_dim"]
    rc = _cabi.lib().mv_prefill_varlen(out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), h * hd, kvh * hd,
                                       kvh * hd, cu.data_ptr(), cu.numel() - 1, q.shape[0], h, kvh, hd,
                                       float(d["scale"]), error_word.data_ptr(), _cabi.dtype_code(dtype),
                                       _cabi.stream_ptr())
    torch.cuda.synchronize()
    return rc


def test_prefill_with_error_word_set_returns_at_once():
    """A wait that ran out leaves the error word set; until the caller clears it every launch is a no-op
    (its CTAs return before touching tensor memory or the output)."""
    d = synth.prefill_inputs(seed=64, num_seqs=2, len_lo=100, len_hi=300, num_heads=4, num_kv_heads=2, head_dim=128)
    dtype = torch.float16
    out = torch.full(tuple(d["q"].shape), 7.0, dtype=dtype, device=DEV)
    word = torch.full((1,), 0x105, dtype=torch.int32, device=DEV)
    assert _call_c_abi(d, dtype, out, word) == 0
    assert int(word.item()) == 0x105 and bool((out == 7.0).all())
    word.zero_()
    assert _call_c_abi(d, dtype, out, word) == 0
    assert int(word.item()) == 0
    _close(out.float().cpu(), _oracle(d, dtype), dtype)


def test_prefill_wait_that_runs_out_is_reported():
    """Failure detection without a fault: one arrival on an mbarrier is withheld (host-side injection for ONE
    launch), the MMA warp's bounded wait runs out after 200 ms, the kernel sets the error word, frees its tensor
    memory and returns; the context stays usable and the next launch is clean."""
    d = synth.prefill_inputs(seed=65, num_seqs=1, len_lo=128, len_hi=128, num_heads=2, num_kv_heads=1, head_dim=128)
    dtype = torch.float16
    out = torch.zeros(tuple(d["q"].shape), dtype=dtype, device=DEV)
    word = torch.zeros(1, dtype=torch.int32, device=DEV)
    assert _cabi.lib().mv_debug_prefill_inject(ctypes.c_int(1)) == 0
    assert _call_c_abi(d, dtype, out, word) == 0          # the launch itself succeeds
    code = int(word.item())
    assert code >> 8 == 1, f"error word {code:#x}"         # 0x100 + the number of the wait that gave up
    word.zero_()
    assert _call_c_abi(d, dtype, out, word) == 0          # the injection was for one launch only
    assert int(word.item()) == 0
    _close(out.float().cpu(), _oracle(d, dtype), dtype)


def test_prefill_benchmark_configuration_exactly():
    """The prefill configuration of the benchmark plan, as `bench.py` times it: 32 sequences, lengths uniform in
    [128, 2048] (34,277 tokens with this seed), 32 query / 8 KV heads, head_dim 128, bf16 -- every sequence, every
    head, every row against the fp32 oracle."""
    d = synth.prefill_inputs()                      # the defaults ARE that configuration (seed 1)
    assert d["q"].shape[0] == 34277 and d["num_heads"] == 32 and d["num_kv_heads"] == 8
    _close(_gpu(d, torch.bfloat16), _oracle(d, torch.bfloat16), torch.bfloat16)


@pytest.mark.parametrize("form", [1, 2])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_prefill_both_launch_forms(form, dtype):
    """One CTA per query tile (form 1) and persistent CTAs that stream through their tiles (form 2): the launch
    picks by the number of sequences; here each is forced in turn (measurement hook outside the public header)
    on ragged batches -- more units than SMs, odd and single-head groups, a one-tile batch -- and must match
    the oracle."""
    lib = _cabi.lib()
    try:
        assert lib.mv_debug_prefill_form(ctypes.c_int(form)) == 0
        for kw in (dict(num_seqs=9, len_lo=1, len_hi=900, num_heads=8, num_kv_heads=2),
                   dict(num_seqs=14, len_lo=250, len_hi=900, num_heads=6, num_kv_heads=2),
                   dict(num_seqs=2, len_lo=129, len_hi=400, num_heads=3, num_kv_heads=3),
                   dict(num_seqs=1, len_lo=17, len_hi=17, num_heads=2, num_kv_heads=1),
                   dict(num_seqs=300, len_lo=0, len_hi=90, num_heads=4, num_kv_heads=2)):
            d = synth.prefill_inputs(seed=66, head_dim=128, **kw)
            _close(_gpu(d, dtype), _oracle(d, dtype), dtype)
    finally:
        lib.mv_debug_prefill_form(ctypes.c_int(0))
