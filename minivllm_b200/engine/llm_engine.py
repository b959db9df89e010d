"""Engine front end: add prompts, step the scheduler and the model runner
until every request is finished.  Same call shape as the reference's
src/myvllm/engine/llm_engine.py (`add_prompt`, `step`, `generate`) with token
ids in and out (no tokenizer is bundled).  `step` always returns a 3-tuple.
Under tensor parallelism every rank constructs the same engine and calls the
same methods with the same prompts (SPMD); see engine/model_runner.py.
"""
import time

import torch

from .model_runner import ModelRunner, _cfg
from .scheduler import Scheduler
from .sequence import SamplingParams, Sequence


class LLMEngine:
    def __init__(self, config: dict, rank: int = 0, world_size: int = None, model=None):
        self.config = config
        self.model_runner = ModelRunner(config, rank=rank, world_size=world_size, model=model)
        self.block_size = config.get("block_size", 256)
        num_blocks = min(self.model_runner.num_kv_blocks, config.get("max_cached_blocks", 1 << 60))
        self.scheduler = Scheduler(
            max_num_seqs=self.model_runner.max_num_seqs,
            max_num_batched_tokens=_cfg(config, "max_num_batched_tokens", default=1024),
            num_blocks=num_blocks, block_size=self.block_size, eos=config.get("eos", -1),
            num_slots=self.model_runner.max_num_seqs,
            prefix_caching=config.get("enable_prefix_caching", False))
        self.stats = dict(prefill_tokens=0, decode_tokens=0, prefill_s=0.0, decode_s=0.0, steps=0)

    def add_prompt(self, token_ids, sampling_params: SamplingParams = None):
        seq = Sequence(token_ids, sampling_params, block_size=self.block_size)
        if len(seq) + seq.max_tokens > self.model_runner.max_model_len:
            raise ValueError("prompt + max_tokens exceeds max_model_length")
        self.scheduler.add_sequence(seq)
        return seq

    def step(self):
        seqs, is_prefill = self.scheduler.schedule()
        if not seqs:
            return [], 0, is_prefill
        t0 = time.perf_counter()
        tokens = self.model_runner.run(seqs, is_prefill)
        dt = time.perf_counter() - t0
        self.scheduler.postprocess(seqs, tokens)
        n = sum(len(s) - 1 - s.num_cached_tokens for s in seqs) if is_prefill else len(seqs)
        key = "prefill" if is_prefill else "decode"
        self.stats[key + "_tokens"] += n
        self.stats[key + "_s"] += dt
        self.stats["steps"] += 1
        done = [(s.seq_id, s.completion_token_ids) for s in seqs if s.is_finished]
        return done, n, is_prefill

    def generate(self, prompts, sampling_params: SamplingParams = None):
        """prompts: list of token-id lists.  Returns {'token_ids': completions in submission order}."""
        seqs = [self.add_prompt(p, sampling_params) for p in prompts]
        while not self.scheduler.is_finished():
            done, n, _ = self.step()
            if n == 0 and not done:
                raise RuntimeError("scheduler made no progress: the KV pool cannot hold a single request")
        return {"token_ids": [s.completion_token_ids for s in seqs]}

    def exit(self):
        self.model_runner.exit()
