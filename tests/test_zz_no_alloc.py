"""The allocation-free decode entry point (mv_paged_decode_static) against the
regular one (mv_paged_decode with a caller-owned workspace), both called
through the C ABI with raw pointers.

Who needs it: a server that has given all of its HBM to the KV-cache pool and
then forbids allocation, code that runs where the allocator must not be
touched, and bindings that can only hand over input and output pointers.  The
scratch is an 8 MiB array built into the library, shared by every call on the
device, so the test makes two calls in a row (the second sees what the first
left in the array) and checks both, then checks that an oversized problem is
refused instead of overrunning the array.

This file is named so that pytest collects it last.
"""
import pytest
import torch

from minivllm_b200 import _cabi, synth

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _args(d, dtype, out):
    q = d["q"].to(dtype).to(DEV)
    kc, vc = d["k_cache"].to(dtype).to(DEV), d["v_cache"].to(dtype).to(DEV)
    bt, cl = d["block_tables"].to(DEV), d["context_lens"].to(DEV)
    keep = (q, kc, vc, bt, cl)
    head = [out.data_ptr(), q.data_ptr(), kc.data_ptr(), vc.data_ptr(), None, None, bt.data_ptr(), bt.stride(0),
            bt.shape[1], cl.data_ptr(), 1, q.shape[0], d["num_heads"], d["num_kv_heads"], d["head_dim"],
            d["block_size"], kc.shape[0], d["scale"]]
    return keep, head


def _run_both(d, dtype):
    lib = _cabi.lib()
    stream = torch.cuda.current_stream().cuda_stream
    code = _cabi.dtype_code(dtype)
    shape = tuple(d["q"].shape)
    out_ref = torch.zeros(shape, dtype=dtype, device=DEV)
    out_new = torch.zeros(shape, dtype=dtype, device=DEV)
    keep, head = _args(d, dtype, out_ref)
    need = lib.mv_paged_decode_workspace_bytes(shape[0], d["num_heads"], d["num_kv_heads"], d["head_dim"],
                                               d["block_tables"].shape[1], d["block_size"])
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)   # the counters at its start must begin at zero
    assert lib.mv_paged_decode(*head, ws.data_ptr(), need, code, stream) == 0, lib.mv_last_error_string()
    head[0] = out_new.data_ptr()
    # warm-up call (the first call on a device resolves the array's address), then the checked one: the
    # driver's count of free device memory must not move, which would also show an allocation made inside
    # the library, invisible to torch's allocator statistics
    assert lib.mv_paged_decode_static(*head, code, stream) == 0, lib.mv_last_error_string()
    torch.cuda.synchronize()
    free_before = torch.cuda.mem_get_info(DEV)[0]
    assert lib.mv_paged_decode_static(*head, code, stream) == 0, lib.mv_last_error_string()
    torch.cuda.synchronize()
    assert torch.cuda.mem_get_info(DEV)[0] == free_before
    del keep
    return out_ref, out_new


def test_static_scratch_decode_matches_workspace_decode_twice():
    # first call: sequences long enough to be split, so the scratch array is really used
    d1 = synth.decode_inputs(seed=70, batch=3, ctx_lo=3000, ctx_hi=6000, num_heads=8, num_kv_heads=2, head_dim=128,
                             block_size=256)
    ref1, new1 = _run_both(d1, torch.float16)
    assert torch.equal(ref1, new1)
    assert float(ref1.float().abs().max()) > 0
    # second call, other shapes: the array still holds the first call's partial results
    d2 = synth.decode_inputs(seed=71, batch=16, ctx_lo=64, ctx_hi=1024, num_heads=16, num_kv_heads=8, head_dim=128,
                             block_size=256)
    ref2, new2 = _run_both(d2, torch.bfloat16)
    assert torch.equal(ref2, new2)
    # and the first problem again gives the first answer again
    ref3, new3 = _run_both(d1, torch.float16)
    assert torch.equal(new3, new1) and torch.equal(ref3, new3)


def test_static_scratch_decode_is_within_tolerance_of_the_oracle():
    from oracle import attention_oracle as oracle
    d = synth.decode_inputs(seed=72, batch=5, ctx_lo=2000, ctx_hi=5000, num_heads=8, num_kv_heads=4, head_dim=128,
                            block_size=256)
    _, new = _run_both(d, torch.float16)
    r = lambda x: x.to(torch.float16).float()
    want = oracle.paged_attention_decode(r(d["q"]), r(d["k_cache"]), r(d["v_cache"]), d["block_tables"],
                                         d["context_lens"], d["scale"], 8, 4, 128, 256)
    assert float((new.float().cpu() - want).abs().max()) < 2e-3


def test_static_scratch_decode_reads_an_int8_cache_too():
    """The k_scale / v_scale route through the allocation-free entry point, against the workspace entry point."""
    from minivllm_b200.layers import attention as A
    lib = _cabi.lib()
    d = synth.decode_inputs(seed=73, batch=4, ctx_lo=1500, ctx_hi=4000, num_heads=8, num_kv_heads=2, head_dim=128,
                            block_size=256)
    dt = torch.float16
    nb, bs, kvh, hd = d["k_cache"].shape
    kq, vq = (torch.zeros(nb, bs, kvh, hd, dtype=torch.int8, device=DEV) for _ in range(2))
    ks, vs = (torch.zeros(nb, bs, kvh, dtype=torch.float16, device=DEV) for _ in range(2))
    slots = torch.arange(nb * bs, dtype=torch.int64, device=DEV)
    A.store_kvcache(d["k_cache"].reshape(-1, kvh, hd).to(dt).to(DEV), d["v_cache"].reshape(-1, kvh, hd).to(dt).to(DEV),
                    kq, vq, slots, bs, k_scale=ks, v_scale=vs)
    q, bt, cl = d["q"].to(dt).to(DEV), d["block_tables"].to(DEV), d["context_lens"].to(DEV)
    stream = torch.cuda.current_stream().cuda_stream
    outs = [torch.zeros_like(q) for _ in range(2)]
    need = lib.mv_paged_decode_workspace_bytes(4, 8, 2, 128, bt.shape[1], 256)
    ws = torch.zeros(need, dtype=torch.uint8, device=DEV)   # the counters at its start must begin at zero
    head = lambda o: [o.data_ptr(), q.data_ptr(), kq.data_ptr(), vq.data_ptr(), ks.data_ptr(), vs.data_ptr(),
                      bt.data_ptr(), bt.stride(0), bt.shape[1], cl.data_ptr(), 1, 4, 8, 2, 128, 256, nb, d["scale"]]
    assert lib.mv_paged_decode(*head(outs[0]), ws.data_ptr(), need, 0, stream) == 0, lib.mv_last_error_string()
    assert lib.mv_paged_decode_static(*head(outs[1]), 0, stream) == 0, lib.mv_last_error_string()
    torch.cuda.synchronize()
    assert torch.equal(outs[0], outs[1]) and float(outs[0].float().abs().max()) > 0


def test_static_scratch_refuses_oversized_problems():
    lib = _cabi.lib()
    cap = lib.mv_paged_decode_static_capacity()
    assert cap == 8 << 20
    # batch 4096 x 32 heads needs far more than 8 MiB: rejected before any launch, pointers never touched
    assert lib.mv_paged_decode_workspace_bytes(4096, 32, 8, 128, 8, 256) > cap
    rc = lib.mv_paged_decode_static(16, 16, 16, 16, None, None, 16, 8, 8, 16, 1, 4096, 32, 8, 128, 256, 100, 0.1, 0,
                                    None)
    assert rc == 7 and b"scratch" in lib.mv_last_error_string()
