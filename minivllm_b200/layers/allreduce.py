"""Tensor-parallel all-reduce over NVLink peer memory, fused with the residual
add and RMSNorm that follow it (C-ABI: mv_comm_*, mv_allreduce_residual_rmsnorm).

The reference ends `RowParallelLinear.forward` with `dist.all_reduce(result)`
(src/myvllm/layers/linear.py:216-221) and then every rank repeats the residual
add and RMSNorm on the full activations (src/myvllm/layers/layernorm.py:19-22).
Here the row-parallel GEMM writes its partial sums straight into the
communicator's input buffer (`input_rows`), one kernel reduces the rows this
rank owns across all peers, adds them to its shard of the residual stream,
normalises and stores the normalised rows into every rank's gather buffer
(`allreduce_residual_rmsnorm` returns that buffer as a tensor).

Set-up exchanges CUDA IPC handles through `torch.distributed` (any backend);
after that no collective library is involved.
"""
import ctypes

import torch
import torch.distributed as dist

from .. import _cabi
from .attention import _error_word


class _DeviceMemory:
    """Exposes a raw device pointer through the CUDA array interface so torch can wrap it without a copy."""

    def __init__(self, ptr, nbytes, owner):
        self.__cuda_array_interface__ = {"shape": (int(nbytes),), "typestr": "|u1", "data": (int(ptr), False),
                                         "version": 2, "strides": None}
        self._owner = owner   # keeps the communicator alive as long as the tensor


def shard_rows(rows, rank, world):
    """Rows [lo, hi) of a (rows, hidden) activation that `rank` owns: ceil(rows/world) each, the tail clipped."""
    per = (rows + world - 1) // world
    lo = min(rows, rank * per)
    return lo, min(rows, lo + per)


class _CommBase:
    def _wrap(self, ptr):
        mem = torch.as_tensor(_DeviceMemory(ptr, self.data_bytes, self), device=self.device)
        return mem.view(self.dtype)[:self.max_rows * self.hidden].view(self.max_rows, self.hidden)

    def close(self):
        if getattr(self, "_comm", None):
            _cabi.lib().mv_comm_destroy(self._comm)
            self._comm = None

    def reset(self):
        """After a timed-out wait, on every rank and with every rank idle: zero the flags and generations."""
        _cabi.check(_cabi.lib().mv_comm_reset(self._comm))

    def set_max_blocks(self, max_blocks):
        """Caps the grid of the following calls (0 = no cap): a block of the kernel holds a whole SM, and a
        caller that overlaps a bandwidth-bound call with another stream's GEMMs leaves them the rest."""
        _cabi.check(_cabi.lib().mv_comm_set_max_blocks(self._comm, int(max_blocks)))


class TPCommunicator(_CommBase):
    """One per rank.  `max_rows` x `hidden` bounds a single call (the largest prefill wave)."""

    def __init__(self, rank, world, max_rows, hidden, dtype, device, group=None, timeout_ms=5000, staged=False):
        L = _cabi.lib()
        self.staged = staged     # True: bulk transfers on the copy engines (mv_allreduce_residual_rmsnorm_staged)
        self.rank, self.world, self.max_rows, self.hidden, self.dtype = rank, world, max_rows, hidden, dtype
        self.device = torch.device(device)
        self.data_bytes = max_rows * hidden * 2
        self._comm = None
        hb = L.mv_comm_handle_bytes()
        handle = ctypes.create_string_buffer(hb)
        comm = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _cabi.check(L.mv_comm_create(rank, world, self.data_bytes, int(timeout_ms), ctypes.byref(comm), handle))
            self._comm = comm
            mine = torch.tensor(list(handle.raw), dtype=torch.uint8,
                                device=self.device if dist.get_backend(group) == "nccl" else "cpu")
            every = [torch.empty_like(mine) for _ in range(world)]
            dist.all_gather(every, mine, group=group)
            blob = ctypes.create_string_buffer(b"".join(bytes(t.cpu().tolist()) for t in every), hb * world)
            _cabi.check(L.mv_comm_connect(self._comm, blob))
            dist.barrier(group=group)        # nobody launches before everybody has mapped everybody
        self._in = self._wrap(L.mv_comm_input(self._comm, 0))
        self._out = self._wrap(L.mv_comm_output(self._comm, 0))
        self.error_word = _error_word(self.device)

    def input_rows(self, rows):
        """(rows, hidden) view of this rank's input buffer: the row-parallel GEMM writes its partial sums here."""
        return self._in[:rows]

    def allreduce_residual_rmsnorm(self, rows, residual_shard, gamma, eps):
        """Reduces the first `rows` rows of every rank's input buffer.  residual_shard (owned rows, hidden) is
        updated in place; returns the (rows, hidden) gather buffer holding the normalised rows of all ranks
        (valid until the next call)."""
        L = _cabi.lib()
        fn = L.mv_allreduce_residual_rmsnorm_staged if self.staged else L.mv_allreduce_residual_rmsnorm
        _cabi.check(fn(self._comm, residual_shard.data_ptr(), 0, gamma.data_ptr(), float(eps), rows, self.hidden,
                       self.error_word.data_ptr(), _cabi.dtype_code(self.dtype), _cabi.stream_ptr()))
        return self._out[:rows]


class EmulatedCommunicator(_CommBase):
    """All `world` ranks on ONE GPU, run by a single cooperative launch: a test vehicle for the protocol and
    the arithmetic (at most 148 blocks in total, so small row counts)."""

    def __init__(self, world, max_rows, hidden, dtype, device, timeout_ms=1000):
        L = _cabi.lib()
        self.world, self.max_rows, self.hidden, self.dtype = world, max_rows, hidden, dtype
        self.device = torch.device(device)
        self.data_bytes = max_rows * hidden * 2
        comm = ctypes.c_void_p()
        with torch.cuda.device(self.device):
            _cabi.check(L.mv_comm_create_emulated(world, self.data_bytes, int(timeout_ms), ctypes.byref(comm)))
        self._comm = comm
        self.inputs = [self._wrap(L.mv_comm_input(comm, r)) for r in range(world)]
        self.outputs = [self._wrap(L.mv_comm_output(comm, r)) for r in range(world)]
        self.error_word = torch.zeros(1, dtype=torch.int32, device=self.device)

    def allreduce_residual_rmsnorm(self, rows, residual_shards, gamma, eps, staged=False):
        """residual_shards (world, rows_per_rank, hidden) contiguous: rank r's shard is residual_shards[r].
        staged=True: the copy-engine form (the copies and the local kernel of every rank; the barrier kernels
        only exist between real ranks)."""
        assert residual_shards.is_contiguous() and residual_shards.shape[0] == self.world
        L = _cabi.lib()
        fn = L.mv_allreduce_residual_rmsnorm_staged if staged else L.mv_allreduce_residual_rmsnorm
        _cabi.check(fn(self._comm, residual_shards.data_ptr(), residual_shards.stride(0), gamma.data_ptr(), float(eps),
                       rows, self.hidden, self.error_word.data_ptr(), _cabi.dtype_code(self.dtype),
                       _cabi.stream_ptr()))
        return [o[:rows] for o in self.outputs]
