#!/usr/bin/env python
"""Benchmark of the ragged-batch attention hot path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload decode]

Prints ONE JSON line (rank 0).  A step is one paged-decode call over the whole
batch.  `value` is measured with the inputs resident in HBM; `e2e` is the same
call through the public Python operator with the per-step host tensors
(q, block tables, context lens) copied from pinned memory and the output
copied back, inside the timed region.  `--impl reference` times the CPU path
(the oracle's restatement of the reference's PyTorch decode) on a bounded
sample of the same workload.
"""
import argparse
import json
import os
import subprocess
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from minivllm_b200 import synth  # noqa: E402

L2_BYTES = 126 * 1024 * 1024
# dram__bytes_read+write / algorithmic bytes of paged_decode_kernel, from the ncu capture summarised in
# profiles/paged_decode_fp16_b64_ctx1024-4096.md (traffic grows in proportion to the KV tokens read)
NCU_TRAFFIC_RATIO = 652.4 / 652.1


def peaks():
    p = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(p):
        d = json.load(open(p))
        return dict(hbm_gbs=d["hbm_gbs"], bf16_tflops=d["bf16_tflops"], src="measured")
    return dict(hbm_gbs=6650.0, bf16_tflops=1590.0, src="fallback")


class ClockSampler:
    """Samples SM clocks and throttle reasons through NVML (read-only) while the timed region runs."""

    def __init__(self, index, period_s=0.005):
        self.index, self.period, self.rows, self.stop = index, period_s, [], threading.Event()
        self.thread = None

    def __enter__(self):
        try:
            import pynvml
            pynvml.nvmlInit()
            self.nv = pynvml
            self.h = pynvml.nvmlDeviceGetHandleByIndex(self._physical_index())
            self.max_mhz = pynvml.nvmlDeviceGetMaxClockInfo(self.h, pynvml.NVML_CLOCK_SM)
            self.thread = threading.Thread(target=self._loop, daemon=True)
            self.thread.start()
        except Exception:  # no NVML: the summary says "unsampled"
            self.thread = None
        return self

    def _physical_index(self):
        vis = os.environ.get("CUDA_VISIBLE_DEVICES")
        if vis:
            ids = [v for v in vis.split(",") if v.strip() != ""]
            if self.index < len(ids) and ids[self.index].strip().isdigit():
                return int(ids[self.index])
        return self.index

    def _loop(self):
        nv = self.nv
        while not self.stop.is_set():
            try:
                self.rows.append((nv.nvmlDeviceGetClockInfo(self.h, nv.NVML_CLOCK_SM),
                                  nv.nvmlDeviceGetCurrentClocksEventReasons(self.h)))
            except Exception:
                break
            time.sleep(self.period)

    def __exit__(self, *a):
        self.stop.set()
        if self.thread:
            self.thread.join(timeout=2)

    def summary(self):
        if not self.rows:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["unsampled"]}
        nv = self.nv
        sm = sorted(r[0] for r in self.rows)
        bits = 0
        for r in self.rows:
            bits |= r[1]
        names = {"hw_slowdown": nv.nvmlClocksEventReasonHwSlowdown,
                 "hw_thermal_slowdown": nv.nvmlClocksEventReasonHwThermalSlowdown,
                 "sw_thermal_slowdown": nv.nvmlClocksEventReasonSwThermalSlowdown,
                 "sw_power_cap": nv.nvmlClocksEventReasonSwPowerCap}
        reasons = [k for k, v in names.items() if bits & v]
        return {"sm_mhz": sm[len(sm) // 2], "sm_max_mhz": self.max_mhz, "reasons": reasons, "samples": len(sm)}


# ----------------------------------------------------------------------------
# workloads
# ----------------------------------------------------------------------------
class DecodeWorkload:
    """Paged decode attention with the distributions of the decode configuration
    (16 query / 8 KV heads, head_dim 128, fp16, 256-token blocks, seeded block
    permutation, q/k/v ~ N(0,1)) scaled to batch 256 and context lengths in
    [1024, 8192] so that the KV read of one step (about 4.8 GB) is far larger
    than L2 and the kernel, not the launch, is measured.
    """
    name = ("paged decode attention op: batch 256, ctx uniform[1024,8192], 16q/8kv heads, head_dim 128, fp16, "
            "block 256, shuffled block tables (decode config distributions scaled past L2)")

    def __init__(self, rank, device, batch=256, ctx_lo=1024, ctx_hi=8192):
        self.H, self.KVH, self.D, self.bs = 16, 8, 128, 256
        self.dtype = torch.float16
        self.device = device
        g = torch.Generator().manual_seed(100 + rank)
        self.context_lens = torch.randint(ctx_lo, ctx_hi + 1, (batch,), generator=g, dtype=torch.int64)
        nblk = (self.context_lens + self.bs - 1) // self.bs
        total = int(nblk.sum())
        perm = torch.randperm(total, generator=g)
        self.max_blocks = int(nblk.max())
        self.block_tables = torch.full((batch, self.max_blocks), -1, dtype=torch.int32)
        at = 0
        for b in range(batch):
            n = int(nblk[b])
            self.block_tables[b, :n] = perm[at:at + n].to(torch.int32)
            at += n
        self.q_host = torch.randn(batch, self.H, self.D, generator=g).to(self.dtype)
        if device is not None:
            self.q_host = self.q_host.pin_memory()
        self.batch, self.total_blocks = batch, total
        self.scale = 1.0 / self.D ** 0.5
        self.bytes_per_step = synth.decode_bytes(self.context_lens, batch, self.H, self.KVH, self.D, 2,
                                                 self.max_blocks)
        self.units_per_step = self.bytes_per_step  # metric unit: algorithmic GB/s
        if device is not None:
            gg = torch.Generator(device=device).manual_seed(200 + rank)
            shape = (total, self.bs, self.KVH, self.D)
            self.k_cache = torch.randn(shape, generator=gg, device=device, dtype=self.dtype)
            self.v_cache = torch.randn(shape, generator=gg, device=device, dtype=self.dtype)
            self.q = self.q_host.to(device)
            self.bt = self.block_tables.to(device)
            self.cl = self.context_lens.to(device)
            self.bt_host = self.block_tables.pin_memory()
            self.cl_host = self.context_lens.pin_memory()
            self.out_host = torch.empty_like(self.q_host).pin_memory()

    def step_resident(self):
        from minivllm_b200.layers import attention as A
        return A.paged_attention_decode(self.q, self.k_cache, self.v_cache, self.bt, self.cl, self.scale, self.H,
                                        self.KVH, self.D, self.bs)

    def step_e2e(self):
        from minivllm_b200.layers import attention as A
        q = self.q_host.to(self.device, non_blocking=True)
        bt = self.bt_host.to(self.device, non_blocking=True)
        cl = self.cl_host.to(self.device, non_blocking=True)
        out = A.paged_attention_decode(q, self.k_cache, self.v_cache, bt, cl, self.scale, self.H, self.KVH, self.D,
                                       self.bs)
        self.out_host.copy_(out, non_blocking=True)

    h2d_bytes = property(lambda s: s.q_host.numel() * 2 + s.block_tables.numel() * 4 + s.context_lens.numel() * 8)
    d2h_bytes = property(lambda s: s.q_host.numel() * 2)
    launches_per_step = 2  # split-K kernel + combine kernel

    def cpu_sample(self, nseq=8):
        """First `nseq` sequences with their own blocks gathered into a compact fp32 cache on the host."""
        from oracle import attention_oracle as oracle
        cl = self.context_lens[:nseq]
        bt = self.block_tables[:nseq]
        ids = bt[bt >= 0].long()
        remap = torch.full((self.total_blocks,), -1, dtype=torch.int32)
        remap[ids] = torch.arange(len(ids), dtype=torch.int32)
        bt2 = torch.where(bt >= 0, remap[bt.clamp(min=0).long()], torch.tensor(-1, dtype=torch.int32))
        if self.device is not None:
            kc = self.k_cache[ids.to(self.device)].float().cpu()
            vc = self.v_cache[ids.to(self.device)].float().cpu()
        else:
            g = torch.Generator().manual_seed(300)
            kc = torch.randn(len(ids), self.bs, self.KVH, self.D, generator=g).half().float()
            vc = torch.randn(len(ids), self.bs, self.KVH, self.D, generator=g).half().float()
        q = self.q_host[:nseq].float()
        nbytes = synth.decode_bytes(cl, nseq, self.H, self.KVH, self.D, 2, bt2.shape[1])

        def run():
            return oracle.paged_attention_decode(q, kc, vc, bt2, cl, self.scale, self.H, self.KVH, self.D, self.bs)
        return run, nbytes, f"first {nseq} of {self.batch} sequences ({int(cl.sum())} KV tokens), fp32"


def time_cpu(run, units, min_seconds=10.0, max_iters=50):
    run()
    t0 = time.perf_counter()
    n = 0
    while True:
        run()
        n += 1
        dt = time.perf_counter() - t0
        if dt >= min_seconds or n >= max_iters:
            break
    return units * n / dt, dt / n


def device_timed(fn, steps, warmup, dist_on):
    """W warm-up calls, then K calls each bracketed by CUDA events on the current stream."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    t0.record()
    for a, b in evs:
        a.record()
        fn()
        b.record()
    t1.record()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    total_ms = t0.elapsed_time(t1)
    per_call_ms = sum(a.elapsed_time(b) for a, b in evs) / steps
    if dist_on:
        t = torch.tensor([total_ms, per_call_ms], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, per_call_ms = float(t[0]), float(t[1])
    return total_ms, per_call_ms


def _time_calls(fns, iters, warmup=5):
    """Average device time (ms) of calls taken round-robin from `fns` (distinct inputs defeat L2 reuse)."""
    for i in range(warmup):
        fns[i % len(fns)]()
    torch.cuda.synchronize()
    a, b = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    a.record()
    for i in range(iters):
        fns[i % len(fns)]()
    b.record()
    torch.cuda.synchronize()
    return a.elapsed_time(b) / iters


def extras(device, pk):
    """Secondary numbers of the same run: the exact small decode configuration and store_kvcache."""
    from minivllm_b200.layers import attention as A
    out = {}
    # decode, exact configuration: batch 16, ctx [64,1024] (34 MB of KV, fits L2) -> rotate 8 cache copies
    d = synth.decode_inputs(seed=0)
    dt = torch.float16
    q, bt, cl = d["q"].to(dt).to(device), d["block_tables"].to(device), d["context_lens"].to(device)
    copies = [(d["k_cache"].to(dt).to(device).clone(), d["v_cache"].to(dt).to(device).clone()) for _ in range(8)]
    fns = [lambda kc=kc, vc=vc: A.paged_attention_decode(q, kc, vc, bt, cl, d["scale"], 16, 8, 128, 256)
           for kc, vc in copies]
    ms = _time_calls(fns, 200, 20)
    nbytes = synth.decode_bytes(d["context_lens"], 16, 16, 8, 128, 2, bt.shape[1])
    out["decode_batch16_ctx64_1024"] = {"us_per_call": ms * 1e3, "GBps": nbytes / ms / 1e6,
                                        "frac_of_measured_peak": nbytes / ms / 1e6 / pk["hbm_gbs"],
                                        "l2": "8 rotating cache copies (272 MB)", "bytes": nbytes}
    del copies, fns
    # store_kvcache: 65,536 tokens, 8 kv heads x 128, bf16, 4096 x 256-slot cache, ~3% padding
    s = synth.store_inputs()
    bf = torch.bfloat16
    slots = s["slot_mapping"].to(device)
    valid = int((s["slot_mapping"] >= 0).sum())
    shape = (s["num_blocks"], s["block_size"], 8, 128)
    kc, vc = torch.zeros(shape, dtype=bf, device=device), torch.zeros(shape, dtype=bf, device=device)
    srcs = [(s["k"].to(bf).to(device).clone(), s["v"].to(bf).to(device).clone()) for _ in range(2)]
    fns = [lambda k=k, v=v: A.store_kvcache(k, v, kc, vc, slots, 256) for k, v in srcs]
    ms = _time_calls(fns, 50)
    nbytes = valid * 8 * 128 * (2 * 2 + 2 * 2) + 65536 * 8
    out["store_kvcache_bf16"] = {"us_per_call": ms * 1e3, "GBps": nbytes / ms / 1e6,
                                 "frac_of_measured_peak": nbytes / ms / 1e6 / pk["hbm_gbs"], "bytes": nbytes}
    del kc, vc
    kq, vq = torch.zeros(shape, dtype=torch.int8, device=device), torch.zeros(shape, dtype=torch.int8, device=device)
    ks = torch.zeros(shape[:3], dtype=torch.float16, device=device)
    vs = torch.zeros(shape[:3], dtype=torch.float16, device=device)
    fns = [lambda k=k, v=v: A.store_kvcache(k, v, kq, vq, slots, 256, k_scale=ks, v_scale=vs) for k, v in srcs]
    ms = _time_calls(fns, 50)
    nbytes = valid * 8 * (128 * (2 * 2 + 2 * 1) + 2 * 2) + 65536 * 8
    out["store_kvcache_int8"] = {"us_per_call": ms * 1e3, "GBps": nbytes / ms / 1e6,
                                 "frac_of_measured_peak": nbytes / ms / 1e6 / pk["hbm_gbs"], "bytes": nbytes}
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=50)
    ap.add_argument("--warmup", type=int, default=5)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode", choices=["decode"])
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--small", action="store_true",
                    help="profiling case: batch 64, ctx [1024,4096] (~1.3 GB of KV), no e2e/CPU/extra legs")
    args = ap.parse_args()
    args.warmup = max(args.warmup, 3) if args.impl == "ours" else args.warmup

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    metric, unit = "paged-decode attention algorithmic HBM throughput", "GB/s"

    if args.impl == "reference":
        if rank != 0:
            return
        wl = DecodeWorkload(0, "cuda:0" if torch.cuda.is_available() else None)
        run, nbytes, sample = wl.cpu_sample()
        for _ in range(args.warmup):
            run()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            run()
        dt = time.perf_counter() - t0
        v = nbytes * args.steps / dt / 1e9
        line = {"impl": "reference", "metric": metric, "value": v, "unit": unit, "n_gpus": args.gpus,
                "steps": args.steps, "warmup": args.warmup, "ms_per_step": dt / args.steps * 1e3,
                "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f32",
                "data": "synthetic", "config": {"workload": wl.name},
                "cpu_baseline": {"value": v, "unit": unit, "cores": torch.get_num_threads(), "kind": "port",
                                 "sample": sample},
                "e2e": {"value": v, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
        print(json.dumps(line), flush=True)
        return

    assert torch.cuda.is_available(), "bench.py --impl ours needs a GPU (there is no CPU path)"
    dist_on = world > 1
    torch.cuda.set_device(local)
    device = torch.device("cuda", local)
    if dist_on:
        import torch.distributed as dist
        dist.init_process_group("nccl", device_id=device)
    from minivllm_b200 import _cabi
    _cabi.lib()

    if args.small:
        wl = DecodeWorkload(rank, device, batch=64, ctx_lo=1024, ctx_hi=4096)
        wl.name = wl.name.replace("batch 256, ctx uniform[1024,8192]", "batch 64, ctx uniform[1024,4096]")
    else:
        wl = DecodeWorkload(rank, device)
    with ClockSampler(local) as clocks:
        total_ms, call_ms = device_timed(wl.step_resident, args.steps, args.warmup, dist_on)
    if args.small:
        e2e_total_ms = float("nan")
    else:
        e2e_total_ms, _ = device_timed(wl.step_e2e, args.steps, args.warmup, dist_on)

    pk = peaks()
    units = wl.units_per_step * world
    value = units * args.steps / (total_ms * 1e-3) / 1e9
    e2e_value = units * args.steps / (e2e_total_ms * 1e-3) / 1e9
    achieved = wl.bytes_per_step / (call_ms * 1e-3) / 1e9
    line = {
        "metric": metric, "value": value, "unit": unit, "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": total_ms / args.steps, "higher_is_better": True, "scaling": "weak", "vs_baseline": None,
        "dtype": "f16", "data": "synthetic",
        "config": {"workload": wl.name, "l2": "inputs larger than L2 (KV read per step %.2f GB)" %
                   (wl.bytes_per_step / 1e9), "sharding": "independent batches per GPU, no collective"},
        "e2e": {"value": e2e_value, "unit": unit, "h2d_bytes_per_step": wl.h2d_bytes,
                "d2h_bytes_per_step": wl.d2h_bytes},
        "gpu_launches": wl.launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": wl.bytes_per_step * NCU_TRAFFIC_RATIO,
                     "traffic_note": "ncu dram bytes of the batch-64 case scaled by KV tokens", "peak_source": pk["src"],
                     "kernel": "paged_decode_kernel (+combine)", "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks.summary(),
    }
    if rank == 0:
        if world == 1 and not args.small:
            line["extra"] = extras(device, pk)
            run, nbytes, sample = wl.cpu_sample()
            v, _ = time_cpu(run, nbytes / 1e9, min_seconds=args.cpu_seconds)
            line["cpu_baseline"] = {"value": v, "unit": unit, "cores": torch.get_num_threads(), "kind": "port",
                                    "sample": sample}
        print(json.dumps(line), flush=True)
    if dist_on:
        import torch.distributed as dist
        dist.destroy_process_group()


if __name__ == "__main__":
    main()
