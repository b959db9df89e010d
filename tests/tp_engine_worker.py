"""One rank of the multi-GPU engine test (launched by tests/test_allreduce_multigpu.py, one process per GPU).

Runs the same requests through the engine at TP = world size (heads and MLP sharded, fused all-reduce + residual +
RMSNorm over peer memory, residual stream sharded by rows; eager and CUDA-graph decode must agree, and so must
two prefill waves in flight on two streams (prefill_streams=2, copy-engine all-reduce) against one stream) and through a
TP = 1 engine built on the same GPU, and compares the final hidden states that reach the LM head at every step in which both
engines fed the same tokens (a random-init model's logits are nearly flat, so greedy streams may part at a
near-tie; what must hold is that equal inputs give equal activations up to bf16 rounding).  Prints
"TP_ENGINE_OK <rank> <steps compared>" on success.
"""
import os
import sys

import torch
import torch.distributed as dist

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
sys.path.insert(0, ROOT)

from minivllm_b200.engine.llm_engine import LLMEngine  # noqa: E402
from minivllm_b200.engine.sequence import SamplingParams  # noqa: E402

CONFIG = dict(vocab_size=2048, hidden_size=512, num_layers=3, num_heads=8, num_kv_heads=8, head_dim=128,
              intermediate_size=1024, base=1e6, max_position=512, max_model_length=512, tie_word_embeddings=True,
              scale=1.0, block_size=16, max_num_seqs=8, max_num_batched_tokens=512, num_kv_blocks=128, greedy=True,
              eos=-1, seed=0, dtype=torch.bfloat16)


def run(world, rank, prompts, steps, eager=True, **over):
    eng = LLMEngine(dict(CONFIG, world_size=world, enforce_eager=eager, **over), rank=rank if world > 1 else 0,
                    world_size=world)
    model, seen = eng.model_runner.model, []
    inner = model.compute_logits

    def spy(hidden, *a, **k):
        from minivllm_b200.utils.context import get_context
        ctx = get_context()
        h = hidden[ctx.last_token_index] if ctx.is_prefill and ctx.last_token_index is not None else hidden
        seen.append(h.float().clone())
        return inner(hidden, *a, **k)
    model.compute_logits = spy
    out = eng.generate(prompts, SamplingParams(temperature=0.0, max_tokens=steps, ignore_eos=True))["token_ids"]
    note, waves = eng.model_runner.comm_note, eng.model_runner._prefill_at
    eng.exit()
    return out, seen, (note, waves) if over else note


def main():
    rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", device_id=torch.device("cuda", rank))
    g = torch.Generator().manual_seed(5)
    prompts = [torch.randint(0, CONFIG["vocab_size"], (n,), generator=g).tolist() for n in (7, 33, 16, 50, 3, 21)]
    steps = 12
    tp_tokens, tp_hidden, note = run(world, rank, prompts, steps)           # eager: every step passes the spy
    assert "fused all-reduce" in note, note
    one_tokens, one_hidden, _ = run(1, 0, prompts, steps)
    assert len(tp_hidden) == steps and len(one_hidden) == steps
    graph_tokens, _, _ = run(world, rank, prompts, steps, eager=False)      # CUDA-graph decode, same TP degree
    assert graph_tokens == tp_tokens, "graph decode and eager decode disagree under tensor parallelism"
    compared = 0
    for t in range(steps):
        same_history = all(a[:t] == b[:t] for a, b in zip(tp_tokens, one_tokens))
        if not same_history:
            break
        a, b = tp_hidden[t][:len(prompts)], one_hidden[t][:len(prompts)]
        err = float((a - b).abs().max())
        assert err <= 0.06 * float(b.abs().max()), f"step {t}: hidden states differ by {err}"
        compared += 1
    assert compared >= 1
    every = [None] * world
    dist.all_gather_object(every, tp_tokens)
    assert all(e == every[0] for e in every), "ranks generated different tokens"
    same = sum(a == b for a, b in zip(tp_tokens, one_tokens))
    # Several prefill waves: with prefill_streams=2 two of them are in flight on two streams, each with its own
    # communicator whose all-reduces take the copy-engine form (same sums, same roundings as the fused kernel):
    # the tokens must be those of the one-stream engine.
    two, _, (_, waves) = run(world, rank, prompts, steps, eager=False, max_num_batched_tokens=64, prefill_streams=2)
    one, _, (_, none) = run(world, rank, prompts, steps, eager=False, max_num_batched_tokens=64, prefill_streams=1)
    assert waves >= 3 and none == 0, (waves, none)
    assert two == one, "two prefill waves in flight changed the tokens"
    dist.barrier()
    dist.destroy_process_group()
    print("TP_ENGINE_OK", rank, compared, f"identical streams {same}/{len(prompts)}", flush=True)


if __name__ == "__main__":
    main()
