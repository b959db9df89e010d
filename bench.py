#!/usr/bin/env python
"""Benchmark of the ragged-batch attention path on B200.

    python bench.py [--gpus N] [--steps K] [--warmup W] [--impl ours|reference] [--workload engine|decode]

Prints ONE JSON line (rank 0).

--workload engine (default): engine output tokens/s.  Random-init Qwen3-8B-shaped
  model (hidden 4096, 36 layers, 32 q / 8 kv heads, head_dim 128, SwiGLU 12288,
  bf16), tensor parallel over the N GPUs (heads and MLP sharded, NCCL all-reduce
  after o_proj / down_proj), 512 requests of random token ids with prompt
  lengths uniform in [512, 1536], 512 greedy output tokens each, KV cache = 80 %
  of free HBM, continuous batching.  A step is one `generate()` over all 512
  requests (prefill waves included); value = output tokens / time.  Fixed total
  work as N grows: "strong" scaling.  `e2e` is the same run clocked on the host
  around the public `LLMEngine.generate` call: every engine step copies its
  inputs (prompt token ids, sequence slots) from pinned host memory and reads
  the sampled tokens back.  `roofline` is the paged-decode attention kernel, the
  largest HBM consumer of a decode step at this shape, timed with CUDA events in
  the same process on the engine's own KV pool.
--workload decode: the paged-decode attention operator alone (algorithmic GB/s),
  independent batches per GPU ("weak" scaling, no collective).

`--impl reference` times the CPU path (the oracle's restatement of the
reference's PyTorch operators inside the same harness model) on the host
cores, on a bounded sample of the workload.
"""
import argparse
import json
import os
import sys
import threading
import time

import torch

ROOT = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, ROOT)

from minivllm_b200 import synth  # noqa: E402

# dram__bytes_read+write / algorithmic bytes of paged_decode_kernel in an ncu capture of the batch-64 case
# (`--workload decode --small`: 652.4 MB measured against 652.1 MB algorithmic); traffic grows in proportion to
# the KV tokens read, so the ratio carries over to the larger cases that are too big to capture
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
    launches_per_step = 1  # one kernel: the last piece's CTA reduces a split sequence

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


def _graph_timed(fn, calls=20, replays=10):
    """Per-call device time (ms) of `fn` replayed inside a CUDA graph: no host work between launches."""
    s = torch.cuda.Stream()
    s.wait_stream(torch.cuda.current_stream())
    with torch.cuda.stream(s):
        fn()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g, stream=s):
            for _ in range(calls):
                fn()
    torch.cuda.current_stream().wait_stream(s)
    return _time_calls([g.replay], replays, 3) / calls


def _hbm(ms, nbytes, pk, **more):
    d = {"us_per_call": ms * 1e3, "GBps": nbytes / ms / 1e6, "frac_of_measured_peak": nbytes / ms / 1e6 / pk["hbm_gbs"],
         "bytes": nbytes}
    d.update(more)
    return d


def case_decode_cfg0(device, pk, iters=200):
    """Paged decode, the exact small configuration: batch 16, ctx [64,1024], 16q/8kv, fp16 (34 MB of KV fits L2:
    8 rotating cache copies).  Timed through the Python operator and, launch-only, inside a CUDA graph."""
    from minivllm_b200.layers import attention as A
    d = synth.decode_inputs(seed=0)
    dt = torch.float16
    q, bt, cl = d["q"].to(dt).to(device), d["block_tables"].to(device), d["context_lens"].to(device)
    copies = [(d["k_cache"].to(dt).to(device).clone(), d["v_cache"].to(dt).to(device).clone()) for _ in range(8)]
    fns = [lambda kc=kc, vc=vc: A.paged_attention_decode(q, kc, vc, bt, cl, d["scale"], 16, 8, 128, 256)
           for kc, vc in copies]
    ms = _time_calls(fns, iters, 20)
    nbytes = synth.decode_bytes(d["context_lens"], 16, 16, 8, 128, 2, bt.shape[1])
    state = {"i": 0}

    def rotate():
        fns[state["i"] % 8]()
        state["i"] += 1
    msg = _graph_timed(rotate, calls=16, replays=max(2, iters // 16))
    return _hbm(ms, nbytes, pk, l2="8 rotating cache copies (272 MB)", us_per_call_in_graph=msg * 1e3,
                GBps_in_graph=nbytes / msg / 1e6)


def case_decode_tp8_shape(device, pk, iters=20):
    """Paged decode at the per-rank shape of the engine under TP=8: batch 512, 4 q heads / 1 kv head, ctx
    uniform[768,1792] (prompt + 256), bf16, 256-token blocks (1.3 GB of KV per call)."""
    from minivllm_b200.layers import attention as A
    d = synth.decode_inputs(seed=4, batch=512, ctx_lo=768, ctx_hi=1792, num_heads=4, num_kv_heads=1)
    dt = torch.bfloat16
    q, bt, cl = d["q"].to(dt).to(device), d["block_tables"].to(device), d["context_lens"].to(device)
    kc, vc = d["k_cache"].to(dt).to(device), d["v_cache"].to(dt).to(device)
    ms = _time_calls([lambda: A.paged_attention_decode(q, kc, vc, bt, cl, d["scale"], 4, 1, 128, 256)], iters, 3)
    return _hbm(ms, synth.decode_bytes(d["context_lens"], 512, 4, 1, 128, 2, bt.shape[1]), pk)


def case_decode_int8(device, pk, iters=20):
    """Paged decode from an int8 cache (fp16 scales): batch 64, ctx [1024,4096], 16q/8kv, fp16 queries."""
    from minivllm_b200.layers import attention as A
    d = synth.decode_inputs(seed=3, batch=64, ctx_lo=1024, ctx_hi=4096, num_heads=16, num_kv_heads=8)
    nb, bs, kvh, hd = d["k_cache"].shape
    dt = torch.float16
    kq, vq = (torch.zeros(nb, bs, kvh, hd, dtype=torch.int8, device=device) for _ in range(2))
    ks, vs = (torch.zeros(nb, bs, kvh, dtype=torch.float16, device=device) for _ in range(2))
    slots = torch.arange(nb * bs, dtype=torch.int64, device=device)
    A.store_kvcache(d["k_cache"].reshape(-1, kvh, hd).to(dt).to(device), d["v_cache"].reshape(-1, kvh, hd).to(dt).to(device),
                    kq, vq, slots, bs, k_scale=ks, v_scale=vs)
    q, bt, cl = d["q"].to(dt).to(device), d["block_tables"].to(device), d["context_lens"].to(device)
    ms = _time_calls([lambda: A.paged_attention_decode(q, kq, vq, bt, cl, d["scale"], 16, 8, 128, 256, k_scale=ks,
                                                       v_scale=vs)], iters, 3)
    return _hbm(ms, synth.decode_bytes(d["context_lens"], 64, 16, 8, 128, 2, bt.shape[1], int8=True), pk)


def case_store(device, pk, iters=50, int8=False):
    """store_kvcache: 65,536 tokens, 8 kv heads x 128, bf16, 4096 x 256-slot cache, ~3 % padding slots."""
    from minivllm_b200.layers import attention as A
    s = synth.store_inputs()
    bf = torch.bfloat16
    slots = s["slot_mapping"].to(device)
    valid = int((s["slot_mapping"] >= 0).sum())
    shape = (s["num_blocks"], s["block_size"], 8, 128)
    srcs = [(s["k"].to(bf).to(device).clone(), s["v"].to(bf).to(device).clone()) for _ in range(2)]
    if int8:
        kq, vq = (torch.zeros(shape, dtype=torch.int8, device=device) for _ in range(2))
        ks, vs = (torch.zeros(shape[:3], dtype=torch.float16, device=device) for _ in range(2))
        fns = [lambda k=k, v=v: A.store_kvcache(k, v, kq, vq, slots, 256, k_scale=ks, v_scale=vs) for k, v in srcs]
        nbytes = valid * 8 * (128 * (2 * 2 + 2 * 1) + 2 * 2) + 65536 * 8
    else:
        kc, vc = torch.zeros(shape, dtype=bf, device=device), torch.zeros(shape, dtype=bf, device=device)
        fns = [lambda k=k, v=v: A.store_kvcache(k, v, kc, vc, slots, 256) for k, v in srcs]
        nbytes = valid * 8 * 128 * (2 * 2 + 2 * 2) + 65536 * 8
    return _hbm(_time_calls(fns, iters, 3), nbytes, pk)


def case_prefill(device, pk, iters=20, num_seqs=32, len_lo=128, len_hi=2048):
    """Varlen causal prefill: 32 sequences, lengths [128,2048], 32 q / 8 kv heads, head_dim 128, bf16."""
    from minivllm_b200.layers import attention as A
    p = synth.prefill_inputs(num_seqs=num_seqs, len_lo=len_lo, len_hi=len_hi)
    bf = torch.bfloat16
    q, k, v = (p[x].to(bf).to(device) for x in "qkv")
    cu = p["cu_seqlens"].to(device)
    ms = _time_calls([lambda: A.flash_attention_prefill(q, k, v, cu, p["scale"], 32, 8, 128)], iters, 5)
    fl = synth.prefill_flops(p["lens"], 32, 128)
    return {"ms_per_call": ms, "TFLOPs": fl / ms / 1e9, "tokens": int(q.shape[0]),
            "frac_of_measured_bf16_peak": fl / ms / 1e9 / pk["bf16_tflops"],
            "frac_of_nominal_2250": fl / ms / 1e9 / 2250.0, "flops": fl, "error_word": A.prefill_error_code(device)}


def case_prefill_paged(device, pk, iters=10):
    """Prefix-aware prefill: 16 sequences of [1024,2048] keys whose first half is already cached; the queries are
    the uncached half, K/V are read through the block tables (32q/8kv, bf16, 256-token blocks)."""
    from minivllm_b200.layers import attention as A
    g = torch.Generator().manual_seed(6)
    bf, H, KVH, D, bs = torch.bfloat16, 32, 8, 128, 256
    klen = torch.randint(1024, 2049, (16,), generator=g)
    qlen = klen // 2
    nblk = (klen + bs - 1) // bs
    total = int(nblk.sum())
    perm = torch.randperm(total, generator=g).to(torch.int32)
    bt = torch.full((16, int(nblk.max())), -1, dtype=torch.int32)
    at = 0
    for i, n in enumerate(nblk.tolist()):
        bt[i, :n] = perm[at:at + n]
        at += n
    cu_q = torch.zeros(17, dtype=torch.int32)
    cu_k = torch.zeros(17, dtype=torch.int32)
    cu_q[1:], cu_k[1:] = torch.cumsum(qlen, 0), torch.cumsum(klen, 0)
    gd = torch.Generator(device=device).manual_seed(6)
    q = torch.randn(int(cu_q[-1]), H, D, generator=gd, device=device, dtype=torch.float32).to(bf)
    kc = torch.randn(total, bs, KVH, D, generator=gd, device=device, dtype=torch.float32).to(bf)
    vc = torch.randn(total, bs, KVH, D, generator=gd, device=device, dtype=torch.float32).to(bf)
    args = (cu_q.to(device), cu_k.to(device), bt.to(device))
    ms = _time_calls([lambda: A.flash_attention_prefill_paged(q, kc, vc, *args, 1.0 / D ** 0.5, H, KVH, D)], iters, 3)
    fl = float(sum(4 * H * D * (int(ql) * (int(kl) - int(ql)) + int(ql) * (int(ql) + 1) // 2)
                   for ql, kl in zip(qlen, klen)))
    return {"ms_per_call": ms, "TFLOPs": fl / ms / 1e9, "query_tokens": int(cu_q[-1]), "key_tokens": int(cu_k[-1]),
            "frac_of_measured_bf16_peak": fl / ms / 1e9 / pk["bf16_tflops"], "flops": fl,
            "error_word": A.prefill_error_code(device)}


def case_pre_attention(device, pk, iters=20, int8=False):
    """Fused q/k RMSNorm + RoPE + K/V store: 16,384 tokens, 32q/8kv heads of 128, bf16 (int8: quantising store)."""
    from minivllm_b200.layers import attention as A
    g = torch.Generator().manual_seed(5)
    tokens, H, KVH, D = 16384, 32, 8, 128
    bf = torch.bfloat16
    qkv = torch.randn(tokens, (H + 2 * KVH) * D, generator=g).to(bf).to(device)
    gam = torch.ones(D, dtype=bf, device=device)
    pos = torch.randint(0, 2048, (tokens,), generator=g).to(device)
    inv = 1.0 / (1e6 ** (torch.arange(0, D, 2).float() / D))
    ang = torch.arange(2048).float()[:, None] * inv[None, :]
    cos, sin = torch.cos(ang).to(device), torch.sin(ang).to(device)
    kc = torch.zeros(128, 256, KVH, D, dtype=torch.int8 if int8 else bf, device=device)
    vc = torch.zeros_like(kc)
    ks = torch.zeros(128, 256, KVH, dtype=torch.float16, device=device) if int8 else None
    vs = torch.zeros_like(ks) if int8 else None
    slots = torch.randperm(128 * 256, generator=g)[:tokens].to(device)
    ms = _time_calls([lambda: A.qk_norm_rope_store(qkv, pos, cos, sin, gam, gam, 1e-5, H, KVH, D, kc, vc, slots,
                                                   k_scale=ks, v_scale=vs)], iters, 3)
    cache_row = (D + 2) if int8 else D * 2
    nbytes = tokens * ((H + 2 * KVH) * D * 2 + (H + KVH) * D * 2 + 2 * KVH * cache_row + 16)
    return _hbm(ms, nbytes, pk)


def case_argmax(device, pk, iters=20):
    """Greedy tail on decode-sized logits: 512 rows x 151,936 columns bf16."""
    from minivllm_b200.layers import sampler as S
    g = torch.Generator(device=device).manual_seed(5)
    x = torch.randn(512, 151936, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    ms = _time_calls([lambda: S.argmax_rows(x, want_keys=False, want_tokens=True)], iters, 3)
    ref = _time_calls([lambda: x.argmax(dim=-1)], iters, 3)
    same = bool((S.argmax_rows(x, want_keys=False, want_tokens=True)[1] == x.float().argmax(dim=-1)).all())
    return _hbm(ms, x.numel() * 2 + 512 * 8, pk, torch_argmax_us=ref * 1e3, same_tokens_as_torch=same)


def case_sample(device, pk, iters=20):
    """Temperature sampling tail (exponential race, Philox noise): 512 rows x 151,936 columns bf16, T = 0.6."""
    from minivllm_b200.layers import sampler as S
    g = torch.Generator(device=device).manual_seed(5)
    x = torch.randn(512, 151936, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    temps = torch.full((512,), 0.6, dtype=torch.float32, device=device)
    step = torch.zeros(1, dtype=torch.int64, device=device)
    ms = _time_calls([lambda: S.sample_rows(x, temps, 1234, step, want_keys=False, want_tokens=True)], iters, 3)

    def torch_race():       # what it replaces: softmax of fp32 logits, an exponential draw, a division, an argmax
        p = torch.softmax(x.float() / temps.unsqueeze(-1), dim=-1)
        return p.div_(torch.empty_like(p).exponential_(1).clamp_min_(1e-10)).argmax(dim=-1)
    ref = _time_calls([torch_race], max(2, iters // 4), 2)
    return _hbm(ms, x.numel() * 2 + 512 * 8, pk, torch_softmax_race_us=ref * 1e3,
                note="compute-bound (Philox + two logarithms per logit); the HBM figure is for scale only")


def case_allreduce_emulated(device, pk, iters=20):
    """Fused all-reduce + residual + RMSNorm, EMULATED world of 8 ranks on one GPU (one cooperative launch runs
    every rank's blocks): 128 rows x 4096 bf16.  A single-GPU stand-in for profilers (a multi-rank run may not be
    profiled); link traffic is replaced by local memory traffic, so only the instruction-level figures carry over."""
    from minivllm_b200.layers.allreduce import EmulatedCommunicator
    world, rows, hidden = 8, 128, 4096
    comm = EmulatedCommunicator(world, rows, hidden, torch.bfloat16, device)
    g = torch.Generator(device=device).manual_seed(3)
    for r in range(world):
        comm.inputs[r][:rows].copy_(torch.randn(rows, hidden, generator=g, device=device, dtype=torch.float32))
    shards = torch.zeros(world, rows // world, hidden, dtype=torch.bfloat16, device=device)
    gamma = torch.ones(hidden, dtype=torch.bfloat16, device=device)
    ms = _time_calls([lambda: comm.allreduce_residual_rmsnorm(rows, shards, gamma, 1e-5)], iters, 3)
    err = int(comm.error_word.item())
    comm.close()
    return {"us_per_call": ms * 1e3, "ranks_emulated": world, "rows": rows, "error_word": err}


def case_add_rmsnorm(device, pk, iters=20):
    """Fused residual add + RMSNorm (single-rank form): 16,384 rows x 4096 bf16, residual updated in place."""
    from minivllm_b200.layers.layernorm import add_rms_norm
    g = torch.Generator(device=device).manual_seed(8)
    x = torch.randn(16384, 4096, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    res = [torch.zeros_like(x) for _ in range(2)]
    gam = torch.ones(4096, dtype=torch.bfloat16, device=device)
    out = torch.empty_like(x)
    ms = _time_calls([lambda r=r: add_rms_norm(x, r, gam, 1e-5, residual_out=r, out=out) for r in res], iters, 3)
    return _hbm(ms, x.numel() * 2 * 4, pk)


def case_silu_mul(device, pk, iters=20):
    """SwiGLU activation: 16,384 rows x (2 x 12,288) bf16 -> 16,384 x 12,288."""
    from minivllm_b200.layers.activation import silu_and_mul
    g = torch.Generator(device=device).manual_seed(9)
    gu = torch.randn(16384, 2 * 12288, generator=g, device=device, dtype=torch.float32).to(torch.bfloat16)
    ms = _time_calls([lambda: silu_and_mul(gu)], iters, 3)
    return _hbm(ms, gu.numel() * 2 + gu.numel(), pk)


OP_CASES = {
    "decode_batch16_ctx64_1024": case_decode_cfg0,
    "decode_tp8_shape_b512_4q1kv": case_decode_tp8_shape,
    "decode_int8_b64_ctx1024_4096": case_decode_int8,
    "store_kvcache_bf16": case_store,
    "store_kvcache_int8": lambda device, pk, iters=50: case_store(device, pk, iters, int8=True),
    "prefill_varlen_bf16": case_prefill,
    "prefill_varlen_bf16_256seq_64_512": lambda device, pk, iters=20: case_prefill(device, pk, iters, 256, 64, 512),
    "prefill_paged_bf16_16seq_half_cached": case_prefill_paged,
    "qk_norm_rope_store_16384tok": case_pre_attention,
    "qk_norm_rope_store_int8_16384tok": lambda device, pk, iters=20: case_pre_attention(device, pk, iters, int8=True),
    "argmax_rows_512x151936": case_argmax,
    "sample_rows_512x151936": case_sample,
    "add_rmsnorm_16384x4096": case_add_rmsnorm,
    "allreduce_emulated_8ranks_128rows": case_allreduce_emulated,
    "silu_mul_16384x12288": case_silu_mul,
}


def extras(device, pk):
    """Secondary numbers of the same run: every operator of the library at its benchmark shape."""
    out = {}
    for name, fn in OP_CASES.items():
        out[name] = fn(device, pk)
        torch.cuda.empty_cache()
    return out


def run_ops(args, device, pk):
    """One operator case, a handful of launches: the command the ncu summaries under profiles/ are made with."""
    fn = OP_CASES[args.case]
    res = fn(device, pk, iters=max(1, args.steps))
    return {"metric": "operator case " + args.case, "value": res.get("us_per_call", res.get("ms_per_call")),
            "unit": "us" if "us_per_call" in res else "ms", "n_gpus": 1, "steps": args.steps, "warmup": 3,
            "higher_is_better": False, "data": "synthetic", "config": {"workload": (fn.__doc__ or args.case).strip()},
            "extra": {args.case: res}}


# ----------------------------------------------------------------------------
# engine workload
# ----------------------------------------------------------------------------
class EngineWorkload:
    name = ("engine output tok/s: random-init Qwen3-8B shape (hidden 4096, 36 layers, 32q/8kv heads, head_dim 128, "
            "intermediate 12288, vocab 151936, bf16), 512 requests, prompts uniform[512,1536] random ids, "
            "512 greedy output tokens each, KV cache 80% of free HBM, prefill waves of 16384 tokens")

    def __init__(self, rank, world, device, requests=512, new_tokens=512, **cfg_over):
        from minivllm_b200.engine import configs
        from minivllm_b200.engine.llm_engine import LLMEngine
        self.rank, self.world, self.device = rank, world, device
        if os.environ.get("MV_CUSTOM_ALLREDUCE", "1") == "0":      # A/B switch: the NCCL all-reduce path
            cfg_over.setdefault("custom_allreduce", False)
        if os.environ.get("MV_PREFILL_STREAMS"):                   # A/B switch: 2 = two prefill waves in flight
            cfg_over.setdefault("prefill_streams", int(os.environ["MV_PREFILL_STREAMS"]))
        self.cfg = configs.qwen3_8b_config(world_size=world, **cfg_over)
        self.prompts, self.sp = configs.qwen3_8b_requests(n=requests, new_tokens=new_tokens)
        self.engine = LLMEngine(self.cfg, rank=rank, world_size=world)
        self.out_tokens_per_step = requests * new_tokens
        self.units_per_step = self.out_tokens_per_step
        self.steps_run = 0

    def step(self):
        e = self.engine
        for k in e.stats:
            e.stats[k] = 0
        out = e.generate(self.prompts, self.sp)
        assert sum(len(t) for t in out["token_ids"]) == self.out_tokens_per_step
        self.last_stats = dict(e.stats)
        self.last_tokens = out["token_ids"]
        return out

    # host<->device traffic of one generate(): prompt ids + per-prefill-wave metadata, per decode step the slot
    # ids going down and the sampled tokens coming back
    @property
    def h2d_bytes(self):
        s = self.last_stats
        prompt_tokens = sum(len(p) for p in self.prompts)
        return prompt_tokens * 8 + s["steps"] * (self.cfg["max_num_seqs"] + 1) * 4 + len(self.prompts) * 24

    @property
    def d2h_bytes(self):
        return (self.out_tokens_per_step) * 8

    def launches_per_step(self):
        """Kernels of this library launched by one generate() (counted from the code path, see below), plus the
        metadata kernels of the step and its greedy sampling tail (row argmax; under tensor parallelism also the
        key decode after the all-reduce)."""
        s = self.last_stats
        layers = self.cfg["num_layers"]
        decode_steps = self.out_tokens_per_step // len(self.prompts) - 1
        prefill_waves = s["steps"] - decode_steps
        tail = (2 if self.world > 1 else 1) if self.cfg.get("greedy", False) else 0
        # per layer: fused q/k norm + RoPE + store, attention (one launch in decode and in prefill), two fused
        # (all-reduce +) add + norm kernels, SwiGLU activation; per step: the first norm and the metadata kernel(s).
        # A prefill wave on a side stream takes the copy-engine form of the all-reduce: two barrier kernels and
        # one reduction kernel per call instead of the one fused kernel.
        staged = 2 * 2 if self.engine.model_runner.prefill_lanes and self.world > 1 else 0
        return decode_steps * (layers * 5 + 2 + tail) + prefill_waves * (layers * (5 + staged) + 3 + tail)

    def decode_probe(self, iters=36):
        """Times paged_attention_decode with CUDA events on the engine's own KV pool at the shape of the
        middle of the run: every request decoding at context = prompt + new_tokens/2, physical blocks taken
        through a seeded permutation of the pool.  One call per layer cache, round robin, so consecutive calls
        read different memory (each call reads far more than L2 anyway)."""
        from minivllm_b200.layers import attention as A
        r = self.engine.model_runner
        c = r.model_cfg
        H, KVH, D, bs = c.num_heads // self.world, c.num_kv_heads // self.world, c.head_dim, r.block_size
        g = torch.Generator().manual_seed(7)
        ctx = torch.tensor([len(p) + self.sp.max_tokens // 2 for p in self.prompts], dtype=torch.int64)
        nblk = (ctx + bs - 1) // bs
        assert int(nblk.sum()) <= r.num_kv_blocks
        perm = torch.randperm(r.num_kv_blocks, generator=g)[:int(nblk.sum())].to(torch.int32)
        bt = torch.full((len(ctx), r.max_blocks_per_seq), -1, dtype=torch.int32)
        at = 0
        for b, n in enumerate(nblk.tolist()):
            bt[b, :n] = perm[at:at + n]
            at += n
        q = torch.randn(len(ctx), H, D, generator=g).to(r.dtype).to(self.device)
        bt, cl = bt.to(self.device), ctx.to(self.device)
        scale = 1.0 / D ** 0.5
        layers = [(r.kv_cache[0, l], r.kv_cache[1, l]) for l in range(c.num_layers)]
        fns = [lambda kc=kc, vc=vc: A.paged_attention_decode(q, kc, vc, bt, cl, scale, H, KVH, D, bs)
               for kc, vc in layers]
        ms = _time_calls(fns, iters, warmup=5)
        nbytes = synth.decode_bytes(ctx, len(ctx), H, KVH, D, 2, r.max_blocks_per_seq)
        return dict(ms=ms, bytes=nbytes, gbps=nbytes / ms / 1e6, batch=len(ctx), ctx_mean=float(ctx.float().mean()))

    def stream_check(self):
        """The first 32 generated tokens of every request against what a TP=1 run of this benchmark generated
        (tests/golden/engine_qwen3_8b_tp1_first32.npz, recorded from a single-GPU run): requests whose 32 tokens
        are identical, requests whose FIRST token is identical, and the mean length of the common prefix.
        A random-init model has nearly flat logits (the top two of 151,936 are often within a few bf16 steps),
        so any change of summation order -- another TP degree -- flips a near-tie sooner or later and the
        streams part there; the first-token and prefix figures are the informative ones.  Absent file -> nulls."""
        import hashlib
        import numpy as np
        first = np.array([list(t[:32]) + [-1] * (32 - len(t[:32])) for t in self.last_tokens], dtype=np.int32)
        out = {"requests": int(first.shape[0]), "digest_of_first32": hashlib.blake2b(first.tobytes(), digest_size=8).hexdigest(),
               "identical_to_tp1_first32": None, "first_token_identical_to_tp1": None, "mean_common_prefix_of_32": None}
        ref = os.path.join(ROOT, "tests", "golden", "engine_qwen3_8b_tp1_first32.npz")
        if os.path.exists(ref):
            want = np.load(ref)["tokens"]
            if want.shape == first.shape:
                eq = want == first
                prefix = np.where(eq.all(1), 32, (~eq).argmax(1))
                out.update(identical_to_tp1_first32=int(eq.all(1).sum()), first_token_identical_to_tp1=int(eq[:, 0].sum()),
                           mean_common_prefix_of_32=float(prefix.mean()))
        dump = os.environ.get("MV_WRITE_FIRST32_TOKENS")       # how the golden file is made (TP=1 run)
        if dump and self.rank == 0:
            np.savez_compressed(dump, tokens=first)
        return out

    def close(self):
        self.engine.exit()


CPU_SAMPLE = dict(requests=4, prompt_len=512, new_tokens=8)


def cpu_engine_reference(requests=CPU_SAMPLE["requests"], prompt_len=CPU_SAMPLE["prompt_len"],
                         new_tokens=CPU_SAMPLE["new_tokens"], repeats=1, warm=False):
    """The CPU path for the engine metric on a bounded sample: the same Qwen3-8B-shaped harness (same seeded
    weights, plain torch formulation) with every attention operator replaced by the CPU oracle, fp32 weights and
    activations (up-cast once, before the clock starts), all host cores, one batch of `requests` prompts of
    `prompt_len` tokens prefilled together and decoded together for `new_tokens` greedy tokens each.
    Both the `cpu_baseline` leg of the GPU run and `--impl reference` call this with the same sample.
    Returns (output tokens per second, seconds per repeat, description)."""
    from minivllm_b200.engine import configs
    from minivllm_b200.engine.qwen3 import Qwen3Config, Qwen3ForCausalLM
    from minivllm_b200.utils.context import reset_context, set_context
    from oracle.attention_module import swap_in_oracle_attention
    import psutil
    cores = os.cpu_count() or 1
    try:
        cores = len(os.sched_getaffinity(0))
    except (AttributeError, OSError):
        pass
    torch.set_num_threads(cores)      # torch.distributed.run exports OMP_NUM_THREADS=1; the CPU arm uses the host
    cfgd = configs.qwen3_8b_config(world_size=1)
    mc = Qwen3Config.from_dict(cfgd)
    build_dev = "cuda:0" if torch.cuda.is_available() else "cpu"   # weights are inputs: generate fast, then move
    model = Qwen3ForCausalLM(mc, 0, 1, torch.bfloat16, build_dev, seed=cfgd["seed"]).to("cpu")
    swap_in_oracle_attention(model)
    fp32 = psutil.virtual_memory().available > 56e9
    if fp32:
        model.float()   # the reference model is fp32-only; 33 GB of weights, converted before timing
    bs = mc.block_size
    nblk = (prompt_len + new_tokens + bs - 1) // bs
    kv = torch.zeros(2, mc.num_layers, requests * nblk, bs, mc.num_kv_heads, mc.head_dim, dtype=torch.float32)
    for l, layer in enumerate(model.layers):
        layer.attn.k_cache, layer.attn.v_cache = kv[0, l], kv[1, l]
    g = torch.Generator().manual_seed(0)
    ids = torch.randint(0, configs.VOCAB, (requests, prompt_len), generator=g)
    tables = torch.arange(requests * nblk, dtype=torch.int32).reshape(requests, nblk)

    def slots(pos_lo, pos_hi):
        return torch.cat([tables[r, p // bs].long() * bs + p % bs
                          for r in range(requests) for p in [torch.arange(pos_lo, pos_hi)]])

    def one_pass(new_tokens=new_tokens):
        with torch.inference_mode():
            cu = torch.arange(0, (requests + 1) * prompt_len, prompt_len, dtype=torch.int32)
            set_context(True, cu, cu, prompt_len, prompt_len, slots(0, prompt_len), None, None,
                        positions=torch.arange(prompt_len).repeat(requests),
                        last_token_index=(cu[1:] - 1).long())
            tok = model.compute_logits(model(ids.reshape(-1))).argmax(-1)
            produced = requests
            for t in range(1, new_tokens):
                pos = prompt_len + t - 1
                set_context(False, None, None, 0, 0, slots(pos, pos + 1), torch.full((requests,), pos + 1), tables,
                            positions=torch.full((requests,), pos))
                tok = model.compute_logits(model(tok)).argmax(-1)
                produced += requests
            reset_context()
        return produced

    if warm:
        one_pass(2)                   # untimed: touches every weight once
    t0 = time.perf_counter()
    produced = sum(one_pass() for _ in range(repeats))
    dt = (time.perf_counter() - t0) / repeats
    desc = (f"{requests} requests prefilled and decoded as one batch, prompt {prompt_len} tokens each (the low end of "
            f"the workload's [512,1536]), {new_tokens} greedy output tokens each, "
            f"{'fp32' if fp32 else 'bf16 weights (host RAM too small for fp32)'} on {cores} host threads; weights "
            f"built and converted before the clock starts")
    return produced / repeats / dt, dt, desc

def device_timed(fn, steps, warmup, dist_on):
    """W warm-up calls, then K calls each bracketed by CUDA events on the current stream; barrier and
    synchronize on both sides; returns (device ms over the K calls, mean per-call ms, host seconds), the
    first two as the MAX over ranks."""
    import torch.distributed as dist
    for _ in range(warmup):
        fn()
    torch.cuda.synchronize()
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize()
    evs = [(torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)) for _ in range(steps)]
    t0, t1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    h0 = time.perf_counter()
    t0.record()
    for a, b in evs:
        a.record()
        fn()
        b.record()
    t1.record()
    torch.cuda.synchronize()
    host_s = time.perf_counter() - h0
    if dist_on:
        dist.barrier()
    total_ms = t0.elapsed_time(t1)
    per_call_ms = sum(a.elapsed_time(b) for a, b in evs) / steps
    if dist_on:
        t = torch.tensor([total_ms, per_call_ms, host_s], device="cuda", dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        total_ms, per_call_ms, host_s = float(t[0]), float(t[1]), float(t[2])
    return total_ms, per_call_ms, host_s


def finish(line, rank):
    """Rank 0 prints the one JSON line."""
    if rank == 0:
        print(json.dumps(line), flush=True)
    sys.stdout.flush()
    sys.stderr.flush()


def teardown(dist_on, limit_s=120.0):
    """Normal shutdown: graphs and communicators are already closed by the workload; synchronise and destroy
    the process group, then return so that the interpreter exits through its regular exit path (exit hooks
    included).  A watchdog only guards against a teardown that blocks: after `limit_s` it runs the registered
    exit hooks itself and leaves."""
    def bail():
        import atexit
        sys.stderr.write("bench.py: teardown did not finish in %.0f s; running exit hooks and leaving\n" % limit_s)
        sys.stderr.flush()
        try:
            atexit._run_exitfuncs()
        finally:
            os._exit(0)
    timer = threading.Timer(limit_s, bail)
    timer.daemon = True
    timer.start()
    torch.cuda.synchronize()
    if dist_on:
        import torch.distributed as dist
        dist.barrier()
        dist.destroy_process_group()
    timer.cancel()


def run_reference(args, rank):
    """CPU arm: rank 0 alone works; the other ranks exit 0."""
    if rank != 0:
        return
    if args.workload == "engine":
        metric, unit = "engine output tokens/s", "tok/s"
        name = EngineWorkload.name
        # one model build, then an untimed pass and the timed passes of the same bounded sample
        value, dt, sample = cpu_engine_reference(repeats=args.steps, warm=args.warmup > 0)
        ms = dt * 1e3
        dtype, scaling = "f32", "strong"
    else:
        metric, unit = "paged-decode attention algorithmic HBM throughput", "GB/s"
        wl = DecodeWorkload(0, "cuda:0" if torch.cuda.is_available() else None)
        name = wl.name
        run, nbytes, sample = wl.cpu_sample()
        for _ in range(args.warmup):
            run()
        t0 = time.perf_counter()
        for _ in range(args.steps):
            run()
        dt = time.perf_counter() - t0
        value, ms = nbytes * args.steps / dt / 1e9, dt / args.steps * 1e3
        dtype, scaling = "f32", "weak"
    line = {"impl": "reference", "metric": metric, "value": value, "unit": unit, "n_gpus": args.gpus,
            "steps": args.steps, "warmup": args.warmup, "ms_per_step": ms, "higher_is_better": True,
            "scaling": scaling, "vs_baseline": None, "dtype": dtype, "data": "synthetic",
            "config": {"workload": name},
            "cpu_baseline": {"value": value, "unit": unit, "cores": torch.get_num_threads(), "kind": "port",
                             "sample": sample},
            "e2e": {"value": value, "unit": unit, "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0}}
    print(json.dumps(line), flush=True)


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=None)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="engine", choices=["engine", "decode", "allreduce", "ops"])
    ap.add_argument("--case", default="store_kvcache_bf16", help="operator case of --workload ops: " + ", ".join(OP_CASES))
    ap.add_argument("--cpu-seconds", type=float, default=10.0)
    ap.add_argument("--no-extras", action="store_true", help="skip the secondary operator numbers and the CPU leg")
    ap.add_argument("--small", action="store_true",
                    help="profiling case: decode workload batch 64, ctx [1024,4096]; engine workload 32 requests x 8 "
                         "tokens with eager decode; no e2e/CPU/extra legs")
    args = ap.parse_args()
    ours = args.impl == "ours"
    if args.workload == "engine":
        # a step is a whole generate() (tens of seconds): few steps by default
        args.steps = 2 if args.steps is None else args.steps
        args.warmup = (3 if ours else 0) if args.warmup is None else args.warmup
        if not ours:
            args.steps = min(args.steps, 2)      # each CPU step is ~20-40 s of host work
            args.warmup = min(args.warmup, 1)    # (a short pass that touches every weight once)
    elif args.workload == "ops":
        args.steps = 3 if args.steps is None else args.steps
        args.warmup = 3
    else:
        args.steps = 50 if args.steps is None else args.steps
        args.warmup = 5 if args.warmup is None else args.warmup
    if ours:
        args.warmup = max(args.warmup, 3)

    rank = int(os.environ.get("RANK", "0"))
    world = int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))

    if not ours:
        run_reference(args, rank)
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
    pk = peaks()

    if args.workload == "engine":
        line = run_engine(args, rank, world, local, device, dist_on, pk)
    elif args.workload == "allreduce":
        line = run_allreduce(args, rank, world, local, device, dist_on, pk)
    elif args.workload == "ops":
        line = run_ops(args, device, pk)
    else:
        line = run_decode(args, rank, world, local, device, dist_on, pk)
    finish(line, rank)
    teardown(dist_on)


def run_engine(args, rank, world, local, device, dist_on, pk):
    if args.small:
        # profiling case: same model and kernels, 32 requests x 8 tokens, eager decode (a launch list of a
        # graph-capturing run would be dominated by the captures)
        wl = EngineWorkload(rank, world, device, requests=32, new_tokens=8, enforce_eager=True, num_kv_blocks=512)
        total_ms, call_ms, host_s = device_timed(wl.step, 1, 1, dist_on)
        line = {"metric": "engine output tokens/s", "value": wl.units_per_step / (total_ms * 1e-3), "unit": "tok/s",
                "n_gpus": world, "steps": 1, "warmup": 1, "config": {"workload": "profiling case: 32 requests x 8 "
                "tokens of the engine workload, eager decode", "allreduce": wl.engine.model_runner.comm_note}}
        wl.close()
        return line
    wl = EngineWorkload(rank, world, device)
    with ClockSampler(local, period_s=0.05) as clocks:
        total_ms, call_ms, host_s = device_timed(wl.step, args.steps, args.warmup, dist_on)
    value = wl.units_per_step * args.steps / (total_ms * 1e-3)
    e2e_value = wl.units_per_step * args.steps / host_s
    probe = wl.decode_probe()
    s = wl.last_stats
    line = {
        "metric": "engine output tokens/s", "value": value, "unit": "tok/s", "n_gpus": world,
        "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "strong", "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": wl.name, "parallelism": f"tp{world}", "kv_blocks_per_gpu": wl.engine.model_runner.num_kv_blocks,
                   "l2": "inputs larger than L2 (weights 16.4 GB and KV pool far exceed 126 MB)",
                   "decode": "CUDA-graph replay of the whole step, one step of lookahead on the host",
                   "step": "one generate() over all requests", "allreduce": wl.engine.model_runner.comm_note},
        "e2e": {"value": e2e_value, "unit": "tok/s", "h2d_bytes_per_step": wl.h2d_bytes,
                "d2h_bytes_per_step": wl.d2h_bytes},
        "gpu_launches": wl.launches_per_step() * args.steps,
        "roofline": {"bound": "hbm", "achieved": probe["gbps"], "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": probe["gbps"] / pk["hbm_gbs"], "traffic": probe["bytes"] * NCU_TRAFFIC_RATIO,
                     "traffic_note": "ncu dram bytes of the batch-64 op case scaled by KV tokens",
                     "peak_source": pk["src"], "kernel": "paged_decode_kernel",
                     "how": "CUDA events around the operator on the engine's KV pool, batch %d, mean ctx %.0f, "
                            "one call per layer cache" % (probe["batch"], probe["ctx_mean"]),
                     "ms_per_launch": probe["ms"], "frac_of_nominal_8TBs": probe["gbps"] / 8000.0},
        "clocks": clocks.summary(),
        "phase_split": {"prefill_s": s["prefill_s"], "decode_s": s["decode_s"], "engine_steps": s["steps"],
                        "prefill_tokens": s["prefill_tokens"],
                        "note": "host clock between launches; with a step in flight the split is approximate"},
        "stream_check": wl.stream_check(),
    }
    wl.close()
    if rank == 0 and world == 1 and not args.no_extras:
        del wl
        torch.cuda.empty_cache()
        line["extra"] = extras(device, pk)
        torch.cuda.empty_cache()
        v, dt, sample = cpu_engine_reference(warm=True)
        line["cpu_baseline"] = {"value": v, "unit": "tok/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": sample}
    return line


def run_decode(args, rank, world, local, device, dist_on, pk):
    if args.small:
        wl = DecodeWorkload(rank, device, batch=64, ctx_lo=1024, ctx_hi=4096)
        wl.name = wl.name.replace("batch 256, ctx uniform[1024,8192]", "batch 64, ctx uniform[1024,4096]")
    else:
        wl = DecodeWorkload(rank, device)
    with ClockSampler(local) as clocks:
        total_ms, call_ms, _ = device_timed(wl.step_resident, args.steps, args.warmup, dist_on)
    e2e_total_ms = float("nan") if args.small else device_timed(wl.step_e2e, args.steps, args.warmup, dist_on)[0]
    units = wl.units_per_step * world
    value = units * args.steps / (total_ms * 1e-3) / 1e9
    achieved = wl.bytes_per_step / (call_ms * 1e-3) / 1e9
    line = {
        "metric": "paged-decode attention algorithmic HBM throughput", "value": value, "unit": "GB/s",
        "n_gpus": world, "steps": args.steps, "warmup": args.warmup, "ms_per_step": total_ms / args.steps,
        "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "f16", "data": "synthetic",
        "config": {"workload": wl.name, "l2": "inputs larger than L2 (KV read per step %.2f GB)" %
                   (wl.bytes_per_step / 1e9), "sharding": "independent batches per GPU, no collective"},
        "e2e": {"value": units * args.steps / (e2e_total_ms * 1e-3) / 1e9, "unit": "GB/s",
                "h2d_bytes_per_step": wl.h2d_bytes, "d2h_bytes_per_step": wl.d2h_bytes},
        "gpu_launches": wl.launches_per_step * args.steps,
        "roofline": {"bound": "hbm", "achieved": achieved, "peak": pk["hbm_gbs"], "unit": "GB/s",
                     "frac": achieved / pk["hbm_gbs"], "traffic": wl.bytes_per_step * NCU_TRAFFIC_RATIO,
                     "traffic_note": "ncu dram bytes of the batch-64 case scaled by KV tokens",
                     "peak_source": pk["src"], "kernel": "paged_decode_kernel",
                     "frac_of_nominal_8TBs": achieved / 8000.0},
        "clocks": clocks.summary(),
    }
    if rank == 0 and world == 1 and not args.small and not args.no_extras:
        line["extra"] = extras(device, pk)
        run, nbytes, sample = wl.cpu_sample()
        v, _ = time_cpu(run, nbytes / 1e9, min_seconds=args.cpu_seconds)
        line["cpu_baseline"] = {"value": v, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                                "sample": sample}
    return line


def run_allreduce(args, rank, world, local, device, dist_on, pk):
    """The tensor-parallel step after o_proj / down_proj at the engine's two message sizes: decode (512 rows x
    4096 bf16 = 4 MiB) and a prefill wave (16,384 rows = 128 MiB).  Times the fused all-reduce + residual +
    RMSNorm kernel against what it replaces (NCCL all-reduce, then the residual add and RMSNorm on all rows),
    CUDA events, max over ranks.  Link roofline: a rank moves (N-1)/N of the message in each direction."""
    import torch.distributed as dist
    import torch.nn.functional as F
    from minivllm_b200.layers.allreduce import TPCommunicator, shard_rows
    from minivllm_b200.layers.layernorm import add_rms_norm
    assert world > 1, "--workload allreduce needs --gpus >= 2 (torch.distributed.run)"
    hidden, dt = 4096, torch.bfloat16
    comm = TPCommunicator(rank, world, 16384, hidden, dt, device)
    gamma = torch.ones(hidden, dtype=dt, device=device)
    out = {}
    link_gbs = 770.0      # measured peer-copy bandwidth per direction on this pool (nominal 900)
    for label, rows, iters in (("decode_512rows", 512, 400), ("prefill_16384rows", 16384, 40)):
        g = torch.Generator(device=device).manual_seed(rank)
        x = torch.randn(rows, hidden, generator=g, device=device, dtype=torch.float32).to(dt)
        lo, hi = shard_rows(rows, rank, world)
        shard = torch.zeros(max(hi - lo, 1), hidden, dtype=dt, device=device)
        full_res = torch.zeros(rows, hidden, dtype=dt, device=device)
        comm.input_rows(rows).copy_(x)

        def fused():
            comm.allreduce_residual_rmsnorm(rows, shard, gamma, 1e-5)

        def nccl_fused_norm():       # NCCL + this library's local add+norm kernel on all rows
            dist.all_reduce(x)
            add_rms_norm(x, full_res, gamma, 1e-5, residual_out=full_res)

        def nccl_torch():            # what the harness did before: NCCL, torch add, torch rms_norm
            dist.all_reduce(x)
            r = full_res + x
            F.rms_norm(r, (hidden,), gamma, 1e-5)

        res = {}
        for name, fn in (("fused_kernel", fused), ("nccl_plus_add_norm_kernel", nccl_fused_norm),
                         ("nccl_plus_torch_add_norm", nccl_torch)):
            x.normal_()              # keep values finite across repeated in-place all-reduces
            x.mul_(1e-3)
            total_ms, _, _ = device_timed(lambda: [fn() for _ in range(iters)], 1, 3, dist_on)
            res[name + "_us"] = total_ms * 1e3 / iters
        torch.cuda.synchronize()
        assert int(comm.error_word.item()) == 0, "an all-reduce wait ran out of time"
        moved = rows * hidden * 2 * (world - 1) / world          # bytes per direction per rank
        res["bytes_per_direction"] = moved
        res["link_GBps_per_direction"] = moved / res["fused_kernel_us"] / 1e3
        res["frac_of_measured_peer_copy_770GBps"] = res["link_GBps_per_direction"] / link_gbs
        res["speedup_vs_nccl_torch"] = res["nccl_plus_torch_add_norm_us"] / res["fused_kernel_us"]
        out[label] = res
    # The same kernel over the row counts between the two: launched one by one, replayed from a CUDA graph of 20
    # launches (no launch gaps, as in the engine's decode graph), and the NCCL all-reduce alone for comparison.
    sweep = {}
    for rows in (1, 64, 256, 512, 1024, 4096, 16384):
        lo, hi = shard_rows(rows, rank, world)
        shard = torch.zeros(max(hi - lo, 1), hidden, dtype=dt, device=device)
        x = torch.zeros(rows, hidden, dtype=dt, device=device)
        iters = 200 if rows <= 4096 else 40
        comm.input_rows(rows).zero_()

        def fused(rows=rows, shard=shard):
            comm.allreduce_residual_rmsnorm(rows, shard, gamma, 1e-5)

        eager_ms, _, _ = device_timed(lambda: [fused() for _ in range(iters)], 1, 3, dist_on)
        graph, side = torch.cuda.CUDAGraph(), torch.cuda.Stream()
        with torch.cuda.stream(side):
            with torch.cuda.graph(graph, stream=side):
                for _ in range(20):
                    fused()
        graph_ms, _, _ = device_timed(lambda: [graph.replay() for _ in range(10)], 1, 3, dist_on)
        nccl_ms, _, _ = device_timed(lambda: [dist.all_reduce(x) for _ in range(iters // 2)], 1, 3, dist_on)
        sweep[str(rows)] = {"fused_us": eager_ms * 1e3 / iters, "fused_in_graph_us": graph_ms * 1e3 / 200,
                            "nccl_allreduce_only_us": nccl_ms * 1e3 / (iters // 2)}
        del graph
    torch.cuda.synchronize()
    assert int(comm.error_word.item()) == 0, "an all-reduce wait ran out of time"
    out["rows_sweep"] = sweep
    d = out["decode_512rows"]
    line = {"metric": "all-reduce + residual + RMSNorm latency (512 rows x 4096 bf16)", "value": d["fused_kernel_us"],
            "unit": "us", "n_gpus": world, "steps": args.steps, "warmup": args.warmup,
            "ms_per_step": d["fused_kernel_us"] / 1e3, "higher_is_better": False, "scaling": "strong",
            "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
            "config": {"workload": "tensor-parallel all-reduce + residual add + RMSNorm, hidden 4096 bf16, "
                                   "512 rows (decode step) and 16,384 rows (prefill wave)",
                       "l2": "the 4 MiB message is L2-resident by construction (the preceding GEMM just wrote it); "
                             "the 128 MiB message exceeds L2"},
            "gpu_launches": 2 * 3 * (400 + 40), "extra": out}
    comm.close()
    return line


if __name__ == "__main__":
    main()
