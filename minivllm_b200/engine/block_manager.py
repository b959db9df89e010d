"""Paged-KV block allocator on the host: a free list of physical blocks and a
free list of device-state slots.  Same role as the reference's
src/myvllm/engine/block_manager.py without its prefix cache: a prefix hit makes
cu_seqlens_k differ from cu_seqlens_q, which the reference's own prefill
kernel ignores (it attends to the uncached suffix only), so prefix reuse is
left to a prefix-aware prefill kernel.
"""
from collections import deque


class BlockManager:
    def __init__(self, num_blocks, block_size, num_slots):
        self.block_size = block_size
        self.free_blocks = deque(range(num_blocks))
        self.free_slots = deque(range(num_slots))

    def can_allocate(self, seq):
        return len(self.free_blocks) >= seq.num_blocks and len(self.free_slots) > 0

    def allocate(self, seq):
        assert not seq.block_table
        seq.block_table = [self.free_blocks.popleft() for _ in range(seq.num_blocks)]
        seq.slot = self.free_slots.popleft()
        seq.synced_blocks = 0
        seq.num_cached_tokens = 0

    def deallocate(self, seq):
        self.free_blocks.extend(seq.block_table)
        seq.block_table = []
        if seq.slot >= 0:
            self.free_slots.append(seq.slot)
        seq.slot = -1
        seq.synced_blocks = 0

    def can_append(self, seq):
        """The decode step writes the KV of the last token (position len-1): it needs a new block
        exactly when the table is one short of ceil(len / block_size)."""
        return len(seq.block_table) >= seq.num_blocks or len(self.free_blocks) > 0

    def append(self, seq):
        """Called before the decode step that feeds the last token and writes its KV at position len-1."""
        if len(seq.block_table) < seq.num_blocks:
            seq.block_table.append(self.free_blocks.popleft())
