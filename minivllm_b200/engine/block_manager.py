"""Paged-KV block allocator on the host: a free list of physical blocks, a free list of device-state slots
and, when enabled, a prefix cache keyed by a chained hash of full blocks (same idea as the reference's
src/myvllm/engine/block_manager.py:39-97: xxh64 over the previous block's hash and the block's token ids).
A prefix hit makes the prefill step's keys outnumber its queries; that case is served by the paged prefill
kernel (the reference's own prefill kernel ignores the cached part).
"""
from collections import deque

import numpy as np

try:
    import xxhash

    def _hash_block(prev, token_ids):
        h = xxhash.xxh64()
        if prev != -1:
            h.update(prev.to_bytes(8, "little"))
        h.update(np.asarray(token_ids, dtype=np.int32).tobytes())
        return h.intdigest()
except ImportError:  # same chaining, different 64-bit hash
    import hashlib

    def _hash_block(prev, token_ids):
        h = hashlib.blake2b(digest_size=8)
        if prev != -1:
            h.update(prev.to_bytes(8, "little"))
        h.update(np.asarray(token_ids, dtype=np.int32).tobytes())
        return int.from_bytes(h.digest(), "little")


class _Block:
    __slots__ = ("ref", "hash", "tokens")

    def __init__(self):
        self.ref, self.hash, self.tokens = 0, -1, None


class BlockManager:
    def __init__(self, num_blocks, block_size, num_slots, prefix_caching=False):
        self.block_size = block_size
        self.prefix_caching = prefix_caching
        self.blocks = [_Block() for _ in range(num_blocks)]
        self.free_blocks = deque(range(num_blocks))
        self.free_slots = deque(range(num_slots))
        self.hash_to_block = {}
        self.cached_hits = 0     # blocks served from the prefix cache so far

    # ---- internals ----
    def _fresh(self):
        block_id = self.free_blocks.popleft()
        b = self.blocks[block_id]
        if b.hash != -1 and self.hash_to_block.get(b.hash) == block_id:
            del self.hash_to_block[b.hash]   # its old contents are about to be overwritten
        b.ref, b.hash, b.tokens = 1, -1, None
        return block_id

    def _blocks_needed(self, seq):
        return seq.num_blocks

    # ---- interface used by the scheduler ----
    def can_allocate(self, seq):
        return len(self.free_blocks) >= self._blocks_needed(seq) and len(self.free_slots) > 0

    def allocate(self, seq):
        assert not seq.block_table
        bs, n = self.block_size, len(seq)
        table, cached, prev, hitting = [], 0, -1, self.prefix_caching
        for i in range(seq.num_blocks):
            toks = seq.token_ids[i * bs:(i + 1) * bs]
            full = len(toks) == bs
            h = _hash_block(prev, toks) if (self.prefix_caching and full) else -1
            # the last block is always recomputed: the step needs at least one query token per sequence
            reuse = -1
            if hitting and full and i < seq.num_blocks - 1:
                cand = self.hash_to_block.get(h, -1)
                if cand != -1 and self.blocks[cand].tokens == toks:
                    reuse = cand
            if reuse != -1:
                b = self.blocks[reuse]
                if b.ref == 0:
                    self.free_blocks.remove(reuse)
                b.ref += 1
                cached += bs
                self.cached_hits += 1
                table.append(reuse)
            else:
                hitting = False
                bid = self._fresh()
                if h != -1:
                    b = self.blocks[bid]
                    b.hash, b.tokens = h, list(toks)
                    self.hash_to_block[h] = bid
                table.append(bid)
            prev = h
        seq.block_table = table
        seq.num_cached_tokens = cached
        seq.slot = self.free_slots.popleft()
        seq.synced_blocks = 0

    def deallocate(self, seq):
        for bid in seq.block_table:
            b = self.blocks[bid]
            b.ref -= 1
            if b.ref == 0:
                self.free_blocks.append(bid)     # contents (and hash) stay valid until the block is handed out again
        seq.block_table = []
        seq.num_cached_tokens = 0
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
            seq.block_table.append(self._fresh())
        if self.prefix_caching:
            bs = self.block_size
            # the block that the previous step completed becomes reusable
            done = (len(seq) - 1) // bs - 1
            if done >= 0 and (len(seq) - 1) % bs == 0:
                b = self.blocks[seq.block_table[done]]
                if b.hash == -1:
                    prev = self.blocks[seq.block_table[done - 1]].hash if done > 0 else -1
                    toks = seq.token_ids[done * bs:(done + 1) * bs]
                    if done == 0 or prev != -1:
                        b.hash, b.tokens = _hash_block(prev, toks), list(toks)
                        self.hash_to_block[b.hash] = seq.block_table[done]
