"""Device-resident per-sequence state and the step metadata built from it on
the GPU (C-ABI entry points mv_build_prefill_meta, mv_build_decode_meta,
mv_update_block_tables).

The reference's model runner rebuilds slot_mapping / context_lens /
block_tables on the host every step with Python loops and ships them through
pinned copies (src/myvllm/engine/model_runner.py:180-256), and every decoder
layer recomputes `positions` on the host (src/myvllm/models/qwen3.py:196-212).
Here a running sequence owns a *slot*: one row of a block table, a length and a
last-token word that stay in device memory.  Per step the host uploads only the
slot ids (and, in prefill, the prompt lengths and token ids); everything else
is written by one kernel launch and shared by all layers through the Context.
"""
import torch

from .. import _cabi


class SequenceStateTable:
    """tables (num_slots, max_blocks) int32, seq_lens (num_slots) int32, last_token (num_slots) int64."""

    def __init__(self, num_slots, max_blocks, block_size, device):
        self.num_slots, self.max_blocks, self.block_size = num_slots, max_blocks, block_size
        self.device = torch.device(device)
        self.tables = torch.full((num_slots, max_blocks), -1, dtype=torch.int32, device=device)
        self.seq_lens = torch.zeros(num_slots, dtype=torch.int32, device=device)
        self.last_token = torch.zeros(num_slots, dtype=torch.int64, device=device)

    # -- block table maintenance -------------------------------------------------
    def update_tables(self, triples):
        """triples: iterable of (slot, index, physical_block); one small upload + one launch."""
        triples = list(triples)
        if not triples:
            return
        upd = torch.tensor(triples, dtype=torch.int32).reshape(-1, 3)
        if self.device.type == "cuda":
            upd = upd.pin_memory().to(self.device, non_blocking=True)
        rc = _cabi.lib().mv_update_block_tables(upd.data_ptr(), upd.shape[0], self.tables.data_ptr(),
                                                self.tables.stride(0), self.max_blocks, self.num_slots,
                                                _cabi.stream_ptr())
        _cabi.check(rc)

    def assign_sequence(self, slot, block_table):
        """A sequence was (re)allocated: write its whole row, clearing the tail."""
        row = list(block_table) + [-1] * (self.max_blocks - len(block_table))
        if len(row) > self.max_blocks:
            raise ValueError(f"sequence needs {len(block_table)} blocks, the table holds {self.max_blocks}")
        self.update_tables((slot, i, b) for i, b in enumerate(row))

    # -- prefill -------------------------------------------------------------------
    def build_prefill(self, slots, seq_lens, num_cached=None):
        """slots / seq_lens / num_cached: host int lists, one entry per sequence of the wave.
        Returns cu_seqlens_q, cu_seqlens_k (int32), positions, slot_mapping, last_token_index (int64)."""
        n = len(slots)
        cached = [0] * n if num_cached is None else list(num_cached)
        total = sum(int(l) - int(c) for l, c in zip(seq_lens, cached))
        host = torch.tensor([list(slots), list(seq_lens), cached], dtype=torch.int32)
        dev = host.pin_memory().to(self.device, non_blocking=True)
        out = dict(cu_seqlens_q=torch.empty(n + 1, dtype=torch.int32, device=self.device),
                   cu_seqlens_k=torch.empty(n + 1, dtype=torch.int32, device=self.device),
                   positions=torch.empty(total, dtype=torch.int64, device=self.device),
                   slot_mapping=torch.empty(total, dtype=torch.int64, device=self.device),
                   last_token_index=torch.empty(n, dtype=torch.int64, device=self.device))
        rc = _cabi.lib().mv_build_prefill_meta(
            dev[0].data_ptr(), dev[1].data_ptr(), dev[2].data_ptr(), n, total, self.tables.data_ptr(),
            self.tables.stride(0), self.max_blocks, self.block_size, self.seq_lens.data_ptr(),
            out["cu_seqlens_q"].data_ptr(), out["cu_seqlens_k"].data_ptr(), out["positions"].data_ptr(),
            out["slot_mapping"].data_ptr(), out["last_token_index"].data_ptr(), _cabi.stream_ptr())
        _cabi.check(rc)
        out["max_seqlen_q"] = max(int(l) - int(c) for l, c in zip(seq_lens, cached))
        out["max_seqlen_k"] = max(int(l) for l in seq_lens)
        return out

    # -- decode --------------------------------------------------------------------
    def build_decode(self, slots_dev, n_active_dev, bufs):
        """slots_dev (batch_padded,) int32 and n_active_dev (1,) int32 on the device;
        bufs: dict of preallocated outputs input_ids, positions, slot_mapping, context_lens (int64, batch_padded)
        and block_tables (batch_padded, max_blocks) int32.  Graph-capturable."""
        bp = bufs["input_ids"].shape[0]
        rc = _cabi.lib().mv_build_decode_meta(
            slots_dev.data_ptr(), n_active_dev.data_ptr(), bp, self.tables.data_ptr(), self.tables.stride(0),
            self.max_blocks, self.block_size, self.seq_lens.data_ptr(), self.last_token.data_ptr(),
            bufs["input_ids"].data_ptr(), bufs["positions"].data_ptr(), bufs["slot_mapping"].data_ptr(),
            bufs["context_lens"].data_ptr(), bufs["block_tables"].data_ptr(), bufs["block_tables"].stride(0),
            _cabi.stream_ptr())
        _cabi.check(rc)

    def new_decode_buffers(self, batch_padded):
        d = self.device
        return dict(input_ids=torch.zeros(batch_padded, dtype=torch.int64, device=d),
                    positions=torch.zeros(batch_padded, dtype=torch.int64, device=d),
                    slot_mapping=torch.full((batch_padded,), -1, dtype=torch.int64, device=d),
                    context_lens=torch.zeros(batch_padded, dtype=torch.int64, device=d),
                    block_tables=torch.full((batch_padded, self.max_blocks), -1, dtype=torch.int32, device=d))
