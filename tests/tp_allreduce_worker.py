"""One rank of the multi-GPU all-reduce test (launched by tests/test_allreduce_multigpu.py, one process per GPU).

Every rank fills its partial sums from a seed, runs the fused all-reduce + residual + RMSNorm kernel (and its
copy-engine form) on the real peer-mapped communicator, gathers every rank's partial sums bit for bit (NCCL all_gather) and checks its own
residual shard (bit-exact) and the gathered rows (one rounding step) against the CPU oracle; the rows must also be
identical on every rank.  Prints "TP_ALLREDUCE_OK <rank>" on success.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from minivllm_b200.layers.allreduce import TPCommunicator, shard_rows  # noqa: E402
from oracle import layers_oracle as oracle  # noqa: E402

EPS = 1e-5


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dev = torch.device("cuda", rank)
    dist.init_process_group("nccl", device_id=dev)
    dtype, hidden, max_rows = torch.bfloat16, 4096, 1024
    comm = TPCommunicator(rank, world, max_rows, hidden, dtype, dev, timeout_ms=2000)
    step = 2.0 ** -7
    # the fused kernel and the copy-engine form alternate on ONE communicator: they share flags and generations
    for it, rows in enumerate([512, 64, 5, 1, 1000, 512, 512, 64, 5, 1, 1000, 512]):
        comm.staged = it >= 5 and it % 2 == 1 or it >= 9
        g = torch.Generator().manual_seed(1000 + it)
        partials = [torch.randn(rows, hidden, generator=g).to(dtype) for _ in range(world)]
        residual = (torch.randn(rows, hidden, generator=g) * 2).to(dtype)
        gamma = (1 + 0.1 * torch.randn(hidden, generator=g)).to(dtype)
        lo, hi = shard_rows(rows, rank, world)
        shard = residual[lo:hi].to(dev).contiguous()       # empty (null pointer) on a rank without rows
        comm.input_rows(rows).copy_(partials[rank])
        out = comm.allreduce_residual_rmsnorm(rows, shard, gamma.to(dev), EPS)
        torch.cuda.synchronize()
        assert int(comm.error_word.item()) == 0, hex(int(comm.error_word.item()))
        want_h, want_r = oracle.allreduce_residual_rmsnorm(partials, residual, gamma, EPS)
        assert torch.equal(shard[:hi - lo].cpu(), want_r[lo:hi]), f"rank {rank} rows {rows}: residual shard"
        got = out.float().cpu()
        assert bool(((got - want_h.float()).abs() <= step * want_h.float().abs() * 1.001).all()), \
            f"rank {rank} rows {rows}: gathered rows"
        every = [torch.empty_like(out) for _ in range(world)]
        dist.all_gather(every, out.clone())
        assert all(torch.equal(e, every[0]) for e in every), "ranks hold different rows"
    dist.barrier()
    comm.close()
    dist.destroy_process_group()
    print("TP_ALLREDUCE_OK", rank, flush=True)


if __name__ == "__main__":
    main()
