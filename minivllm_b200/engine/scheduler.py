"""Continuous-batching scheduler on the host, the policy of the reference's
src/myvllm/engine/scheduler.py:25-82: a prefill wave whenever waiting requests
fit (sequence and token budgets, free blocks), otherwise one decode token for
every running sequence, preempting from the tail when no block is free.
"""
from collections import deque

from .block_manager import BlockManager
from .sequence import Sequence, SequenceStatus


class Scheduler:
    def __init__(self, max_num_seqs, max_num_batched_tokens, num_blocks, block_size, eos, num_slots=None,
                 prefix_caching=False):
        self.max_num_seqs = max_num_seqs
        self.max_num_batched_tokens = max_num_batched_tokens
        self.block_manager = BlockManager(num_blocks, block_size, num_slots or max_num_seqs, prefix_caching)
        self.eos = eos
        self.waiting: deque[Sequence] = deque()
        self.running: deque[Sequence] = deque()

    def is_finished(self):
        return not self.waiting and not self.running

    def add_sequence(self, seq):
        self.waiting.append(seq)

    def schedule(self):
        """Returns (sequences, is_prefill)."""
        picked, tokens = [], 0
        while self.waiting and len(self.running) < self.max_num_seqs:
            seq = self.waiting[0]
            if not self.block_manager.can_allocate(seq) or tokens + len(seq) > self.max_num_batched_tokens:
                break
            self.waiting.popleft()
            self.block_manager.allocate(seq)
            seq.status = SequenceStatus.RUNNING
            self.running.append(seq)
            picked.append(seq)
            tokens += len(seq)
        if picked:
            return picked, True
        # decode: every running sequence that can get a slot for its next token
        survivors = deque()
        while self.running:
            seq = self.running.popleft()
            while not self.block_manager.can_append(seq):
                if self.running:
                    self.preempt(self.running.pop())
                else:
                    self.preempt(seq)
                    seq = None
                    break
            if seq is None:
                break
            self.block_manager.append(seq)
            survivors.append(seq)
        self.running = survivors
        return list(survivors), False

    def preempt(self, seq):
        self.block_manager.deallocate(seq)
        seq.status = SequenceStatus.WAITING
        self.waiting.appendleft(seq)

    def postprocess(self, seqs, token_ids):
        for seq, tok in zip(seqs, token_ids):
            seq.append_token(tok)
            if (not seq.ignore_eos and tok == self.eos) or seq.num_completion_tokens >= seq.max_tokens:
                self._finish(seq)

    def _finish(self, seq):
        seq.status = SequenceStatus.FINISHED
        self.block_manager.deallocate(seq)
        self.running.remove(seq)

    # ---- one step of lookahead: bookkeeping before the sampled tokens have reached the host ----
    def can_run_ahead(self, seqs):
        """True when the step after this one can be scheduled without knowing this step's tokens: no
        sequence of the batch can end on an EOS token, and no token value is hashed (prefix cache off)."""
        return not self.block_manager.prefix_caching and all(s.ignore_eos or self.eos < 0 for s in seqs)

    def no_preemption_next(self):
        """The next decode step finds a block for every running sequence, so nothing is preempted (a preempted
        sequence is prefilled again from its token ids, which must then be real)."""
        return len(self.block_manager.free_blocks) >= len(self.running)

    def advance(self, seqs):
        """postprocess() with the token values still unknown: appends a placeholder to every sequence and
        finishes those that reached max_tokens.  Returns the positions to hand to `fill_tokens`."""
        at = []
        for seq in seqs:
            at.append(len(seq.token_ids))
            seq.append_token(-1)
            if seq.num_completion_tokens >= seq.max_tokens:
                self._finish(seq)
        return at

    @staticmethod
    def fill_tokens(seqs, positions, token_ids):
        for seq, pos, tok in zip(seqs, positions, token_ids):
            seq.token_ids[pos] = int(tok)
