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
        if self.model_runner.greedy and seq.temperature != 0:
            raise ValueError("this engine was configured with greedy=True (argmax for every request); "
                             "use temperature 0, or greedy=False for per-request temperatures")
        self.scheduler.add_sequence(seq)
        return seq

    def _account(self, seqs, is_prefill, dt):
        n = sum(len(s) - 1 - s.num_cached_tokens for s in seqs) if is_prefill else len(seqs)
        key = "prefill" if is_prefill else "decode"
        self.stats[key + "_tokens"] += n
        self.stats[key + "_s"] += dt
        self.stats["steps"] += 1
        return n

    def step(self):
        seqs, is_prefill = self.scheduler.schedule()
        if not seqs:
            return [], 0, is_prefill
        t0 = time.perf_counter()
        tokens = self.model_runner.run(seqs, is_prefill)
        dt = time.perf_counter() - t0
        self.scheduler.postprocess(seqs, tokens)
        n = self._account(seqs, is_prefill, dt)
        done = [(s.seq_id, s.completion_token_ids) for s in seqs if s.is_finished]
        return done, n, is_prefill

    def generate(self, prompts, sampling_params: SamplingParams = None):
        """prompts: list of token-id lists.  Returns {'token_ids': completions in submission order}.

        The loop keeps one step in flight: when no sequence of a batch can stop on an EOS token, the next step
        is scheduled and launched (lengths and finishes are known from counts; the last token of every
        sequence already sits in device memory) before the previous step's sampled tokens are read back, so
        the device->host read and the host bookkeeping overlap the GPU work."""
        seqs = [self.add_prompt(p, sampling_params) for p in prompts]
        sch, runner = self.scheduler, self.model_runner
        lookahead = self.config.get("lookahead", True)
        pending = None                       # (handle, seqs, positions) of the step in flight
        t_last = time.perf_counter()

        def resolve():
            nonlocal pending
            if pending is not None:
                handle, pseqs, at = pending
                sch.fill_tokens(pseqs, at, runner.finish(handle))
                pending = None

        while not sch.is_finished():
            if pending is not None and not sch.no_preemption_next():
                resolve()
            batch, is_prefill = sch.schedule()
            if not batch:
                resolve()
                if sch.is_finished():
                    break
                raise RuntimeError("scheduler made no progress: the KV pool cannot hold a single request")
            handle = runner.launch(batch, is_prefill)
            if lookahead and sch.can_run_ahead(batch):
                at = sch.advance(batch)
                resolve()                    # the previous step, while this one runs
                pending = (handle, batch, at)
            else:
                resolve()
                sch.postprocess(batch, runner.finish(handle))
            now = time.perf_counter()
            self._account(batch, is_prefill, now - t_last)
            t_last = now
        resolve()
        return {"token_ids": [s.completion_token_ids for s in seqs]}

    def exit(self):
        self.model_runner.exit()
