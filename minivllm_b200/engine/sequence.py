"""Host-side request state (out of the hot path; kept as thin Python like the
reference's src/myvllm/engine/sequence.py).  Differences: a full last block
counts block_size tokens (the reference counts zero), tokens are appended
through `append_token` only, and a running sequence owns a device-state `slot`.
"""
from dataclasses import dataclass
from enum import Enum, auto
from itertools import count


class SequenceStatus(Enum):
    WAITING = auto()
    RUNNING = auto()
    FINISHED = auto()


@dataclass
class SamplingParams:
    temperature: float = 1.0     # 0 selects greedy argmax (the reference has no greedy path)
    max_tokens: int = 64
    ignore_eos: bool = False


class Sequence:
    _ids = count()

    def __init__(self, token_ids, sampling_params=None, block_size=256):
        sp = sampling_params or SamplingParams()
        self.seq_id = next(Sequence._ids)
        self.status = SequenceStatus.WAITING
        self.token_ids = list(token_ids)
        self.num_prompt_tokens = len(self.token_ids)
        self.block_size = block_size
        self.block_table = []
        self.num_cached_tokens = 0
        self.slot = -1               # row of the device-resident state while running
        self.synced_blocks = 0       # how many block-table entries the device row already holds
        self.temperature, self.max_tokens, self.ignore_eos = sp.temperature, sp.max_tokens, sp.ignore_eos

    def __len__(self):
        return len(self.token_ids)

    @property
    def num_tokens(self):
        return len(self.token_ids)

    @property
    def last_token(self):
        return self.token_ids[-1]

    @property
    def num_completion_tokens(self):
        return len(self.token_ids) - self.num_prompt_tokens

    @property
    def completion_token_ids(self):
        return self.token_ids[self.num_prompt_tokens:]

    @property
    def num_blocks(self):
        return (len(self.token_ids) + self.block_size - 1) // self.block_size

    @property
    def is_finished(self):
        return self.status == SequenceStatus.FINISHED

    def append_token(self, token_id):
        self.token_ids.append(int(token_id))
