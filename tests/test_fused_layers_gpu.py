"""GPU parity of the fused layer steps around attention: residual add + RMSNorm, SwiGLU activation, and the
all-reduce + residual + RMSNorm kernel run as an EMULATED world (all ranks on one GPU, one cooperative
launch), against the CPU oracle.  The new residual is bit-exact; normalised rows are within one rounding
step of the model dtype (the kernel's rsqrt and summation order differ from the CPU's in the last fp32 bits).
"""
import ctypes

import pytest
import torch

from minivllm_b200 import _cabi
from minivllm_b200.layers.activation import silu_and_mul
from minivllm_b200.layers.allreduce import EmulatedCommunicator, shard_rows
from minivllm_b200.layers.layernorm import add_rms_norm
from oracle import layers_oracle as oracle

pytestmark = pytest.mark.gpu
DEV = "cuda:0"
EPS = 1e-5


def _ulp_close(got, want, dtype):
    """|got - want| <= one rounding step of `dtype` at the value's magnitude."""
    step = 2.0 ** (-7 if dtype == torch.bfloat16 else -10)
    g, w = got.float().cpu(), want.float()
    return bool(((g - w).abs() <= step * w.abs().clamp_min(1e-30) * 1.001 + 1e-30).all())


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
@pytest.mark.parametrize("rows,hidden", [(1, 1024), (7, 4096), (300, 4096), (3, 16384), (5, 200)])
def test_add_rms_norm_matches_oracle(dtype, rows, hidden):
    g = torch.Generator().manual_seed(rows * 31 + hidden)
    x = torch.randn(rows, hidden, generator=g).to(dtype)
    res = (torch.randn(rows, hidden, generator=g) * 3).to(dtype)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    want_h, want_r = oracle.add_rms_norm(x, res, gamma, EPS)
    r_dev = res.to(DEV)
    h = add_rms_norm(x.to(DEV), r_dev, gamma.to(DEV), EPS, residual_out=r_dev)     # in place
    assert torch.equal(r_dev.cpu(), want_r)
    assert _ulp_close(h, want_h, dtype)
    # no residual: plain RMSNorm; the sum is kept only for a row range
    lo, hi = rows // 3, rows
    keep = torch.zeros(hi - lo, hidden, dtype=dtype, device=DEV)
    h2 = add_rms_norm(x.to(DEV), None, gamma.to(DEV), EPS, residual_out=keep, residual_rows=(lo, hi))
    assert torch.equal(keep.cpu(), x[lo:hi])
    assert _ulp_close(h2, oracle.rms_norm(x, gamma, EPS), dtype)


@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_silu_and_mul_matches_oracle(dtype):
    g = torch.Generator().manual_seed(5)
    gu = (torch.randn(37, 2 * 1536, generator=g) * 2).to(dtype)
    got = silu_and_mul(gu.to(DEV))
    assert _ulp_close(got, oracle.silu_and_mul(gu), dtype)
    wide = torch.randn(9, 2 * 1536 + 64, generator=g).to(dtype).to(DEV)          # strided rows
    view = wide[:, :2 * 1536]
    assert _ulp_close(silu_and_mul(view), oracle.silu_and_mul(view.cpu()), dtype)


def _emulated_case(comm, rows, hidden, dtype, seed, staged=False):
    world = comm.world
    g = torch.Generator().manual_seed(seed)
    partials = [torch.randn(rows, hidden, generator=g).to(dtype) for _ in range(world)]
    residual = (torch.randn(rows, hidden, generator=g) * 2).to(dtype)
    gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
    per = (rows + world - 1) // world
    shards = torch.zeros(world, max(per, 1), hidden, dtype=dtype)
    for r in range(world):
        lo, hi = shard_rows(rows, r, world)
        shards[r, :hi - lo] = residual[lo:hi]
    shards = shards.to(DEV)
    for r in range(world):
        comm.inputs[r][:rows].copy_(partials[r])
        comm.outputs[r][:rows].fill_(float("nan"))
    outs = comm.allreduce_residual_rmsnorm(rows, shards, gamma.to(DEV), EPS, staged=staged)
    torch.cuda.synchronize()
    assert int(comm.error_word.item()) == 0
    want_h, want_r = oracle.allreduce_residual_rmsnorm(partials, residual, gamma, EPS)
    for r in range(world):
        lo, hi = shard_rows(rows, r, world)
        assert torch.equal(shards[r, :hi - lo].cpu(), want_r[lo:hi]), f"residual shard of rank {r}"
        assert _ulp_close(outs[r], want_h, dtype), f"gathered rows on rank {r}"
        assert torch.equal(outs[r], outs[0]), "every rank must hold identical rows"


@pytest.mark.parametrize("world", [2, 4, 8])
@pytest.mark.parametrize("dtype", [torch.bfloat16, torch.float16])
def test_emulated_allreduce_residual_rmsnorm(world, dtype):
    """Several calls in a row on one communicator (the generation counters advance), with row counts that
    divide evenly, leave a ragged tail, and leave some ranks without rows."""
    comm = EmulatedCommunicator(world, 640, 4096, dtype, DEV)
    try:
        for i, rows in enumerate([world * 4, 64, 5, 1, world + 1, 64, 640]):
            _emulated_case(comm, rows, 4096, dtype, seed=100 * world + i)
    finally:
        comm.close()


def test_emulated_allreduce_other_widths():
    for hidden, rows in [(1024, 16), (16384, 6), (200, 9)]:
        comm = EmulatedCommunicator(2, 16, hidden, torch.bfloat16, DEV)
        try:
            _emulated_case(comm, rows, hidden, torch.bfloat16, seed=hidden)
        finally:
            comm.close()


@pytest.mark.parametrize("world", [2, 4, 8])
def test_emulated_staged_form_matches_the_oracle(world):
    """The copy-engine form: every rank's pulls, local reduction and pushes (the barrier kernels between real
    ranks are covered by the multi-GPU test), alternating with the fused form on the same communicator."""
    comm = EmulatedCommunicator(world, 640, 4096, torch.bfloat16, DEV)
    try:
        for i, rows in enumerate([world * 4, 64, 5, 1, world + 1, 640]):
            _emulated_case(comm, rows, 4096, torch.bfloat16, seed=300 * world + i, staged=True)
            _emulated_case(comm, rows, 4096, torch.bfloat16, seed=300 * world + i + 50, staged=False)
    finally:
        comm.close()
    comm = EmulatedCommunicator(2, 16, 16384, torch.float16, DEV)       # two vectors per thread
    try:
        _emulated_case(comm, 6, 16384, torch.float16, seed=9, staged=True)
    finally:
        comm.close()


def test_a_capped_grid_gives_the_same_rows():
    """mv_comm_set_max_blocks: rows are strided over however many blocks there are; the barriers do not depend on
    the grid."""
    comm = EmulatedCommunicator(4, 64, 4096, torch.bfloat16, DEV)
    try:
        for cap in (1, 3, 0):
            comm.set_max_blocks(cap)
            _emulated_case(comm, 64, 4096, torch.bfloat16, seed=7 + cap)
            _emulated_case(comm, 13, 4096, torch.bfloat16, seed=70 + cap)
    finally:
        comm.close()


def test_withheld_signal_times_out_and_reports():
    """A rank that never signals: the others' waits run out (200 ms limit), the error word is set, the launch
    ends by itself and later launches return at once; after a reset the communicator works again."""
    world, rows, hidden = 2, 8, 1024
    comm = EmulatedCommunicator(world, 16, hidden, torch.bfloat16, DEV, timeout_ms=200)
    try:
        _emulated_case(comm, rows, hidden, torch.bfloat16, seed=1)
        assert _cabi.lib().mv_debug_comm_withhold_signal(comm._comm, ctypes.c_int(1)) == 0
        shards = torch.zeros(world, rows // world, hidden, dtype=torch.bfloat16, device=DEV)
        gamma = torch.ones(hidden, dtype=torch.bfloat16, device=DEV)
        comm.allreduce_residual_rmsnorm(rows, shards, gamma, EPS)
        torch.cuda.synchronize()                          # returns: every wait is bounded
        code = int(comm.error_word.item())
        assert code & 0x300, hex(code)
        comm.allreduce_residual_rmsnorm(rows, shards, gamma, EPS)   # no-op while the word is set
        torch.cuda.synchronize()
        comm.error_word.zero_()
        comm.reset()
        _emulated_case(comm, rows, hidden, torch.bfloat16, seed=2)
    finally:
        comm.close()


def test_argument_checks():
    comm = EmulatedCommunicator(2, 8, 1024, torch.bfloat16, DEV)
    try:
        shards = torch.zeros(2, 8, 1024, dtype=torch.bfloat16, device=DEV)
        gamma = torch.ones(1024, dtype=torch.bfloat16, device=DEV)
        with pytest.raises(ValueError):                    # more rows than the buffers hold
            comm.allreduce_residual_rmsnorm(9, shards, gamma, EPS)
    finally:
        comm.close()
    with pytest.raises(ValueError):
        add_rms_norm(torch.zeros(2, 12, dtype=torch.bfloat16, device=DEV), None,
                     torch.ones(12, dtype=torch.bfloat16, device=DEV), EPS)     # hidden not a multiple of 8
