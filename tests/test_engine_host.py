"""Host-side engine logic without a GPU: block manager, scheduler policy, and the
tensor-parallel sharding of the harness model over 2 gloo ranks on the CPU."""
import os
import subprocess
import sys

import pytest
import torch

from minivllm_b200.engine.block_manager import BlockManager
from minivllm_b200.engine.scheduler import Scheduler
from minivllm_b200.engine.sequence import SamplingParams, Sequence, SequenceStatus

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def test_block_manager_allocates_and_grows_at_block_boundaries():
    bm = BlockManager(num_blocks=4, block_size=4, num_slots=2)
    s = Sequence(list(range(8)), block_size=4)       # exactly two full blocks
    assert bm.can_allocate(s)
    bm.allocate(s)
    assert s.block_table == [0, 1] and s.slot == 0
    s.append_token(99)                                # 9 tokens: the decode step writes position 8 -> third block
    assert bm.can_append(s)
    bm.append(s)
    assert s.block_table == [0, 1, 2]
    for t in range(3):
        s.append_token(t)
        bm.append(s)
    assert s.block_table == [0, 1, 2]                 # 12 tokens still fit three blocks
    s.append_token(5)
    bm.append(s)
    assert s.block_table == [0, 1, 2, 3]
    s.append_token(5); s.append_token(5); s.append_token(5); s.append_token(5)   # 17 tokens, no block left
    assert not bm.can_append(s)
    bm.deallocate(s)
    assert len(bm.free_blocks) == 4 and s.slot == -1 and list(bm.free_slots) == [1, 0]


def test_scheduler_prefill_first_then_decode_and_finish():
    sch = Scheduler(max_num_seqs=2, max_num_batched_tokens=10, num_blocks=8, block_size=4, eos=-1)
    a = Sequence([1, 2, 3], SamplingParams(max_tokens=2), block_size=4)
    b = Sequence([4, 5, 6, 7, 8], SamplingParams(max_tokens=1), block_size=4)
    c = Sequence([9] * 6, SamplingParams(max_tokens=1), block_size=4)
    for s in (a, b, c):
        sch.add_sequence(s)
    seqs, is_prefill = sch.schedule()
    assert is_prefill and seqs == [a, b]              # c does not fit: two sequences running
    sch.postprocess(seqs, [10, 11])
    assert b.is_finished and not a.is_finished        # b reached max_tokens = 1
    seqs, is_prefill = sch.schedule()
    assert is_prefill and seqs == [c]                 # prefill comes before decode
    sch.postprocess(seqs, [12])
    seqs, is_prefill = sch.schedule()
    assert not is_prefill and seqs == [a]
    sch.postprocess(seqs, [13])
    assert a.is_finished and sch.is_finished()
    assert a.completion_token_ids == [10, 13]


def test_scheduler_preempts_from_the_tail_when_blocks_run_out():
    sch = Scheduler(max_num_seqs=4, max_num_batched_tokens=100, num_blocks=2, block_size=4, eos=-1)
    a = Sequence([1, 2, 3, 4], SamplingParams(max_tokens=8), block_size=4)
    b = Sequence([5, 6, 7, 8], SamplingParams(max_tokens=8), block_size=4)
    sch.add_sequence(a); sch.add_sequence(b)
    seqs, _ = sch.schedule()
    assert seqs == [a, b]
    sch.postprocess(seqs, [9, 9])                     # both now need a second block; none is free
    seqs, is_prefill = sch.schedule()
    assert not is_prefill and seqs == [a]             # b was preempted, its block went to a
    assert b.status == SequenceStatus.WAITING and sch.waiting[0] is b and b.block_table == []
    assert len(a.block_table) == 2


TP_WORKER = r'''
import os, sys, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MV_ROOT"])
from minivllm_b200.engine.qwen3 import Qwen3Config, Qwen3ForCausalLM
from minivllm_b200.utils.context import set_context
from oracle.attention_module import swap_in_oracle_attention
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
cfg = Qwen3Config(vocab_size=97, hidden_size=64, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=16,
                  intermediate_size=96, max_position=64, block_size=4)
def logits_for(tp_rank, tp_size):
    m = swap_in_oracle_attention(Qwen3ForCausalLM(cfg, tp_rank, tp_size, torch.float32, "cpu", seed=3))
    ids = torch.tensor([5, 9, 2, 7, 7, 1, 3], dtype=torch.int64)
    cu = torch.tensor([0, 4, 7], dtype=torch.int32)
    set_context(True, cu, cu, 4, 4, None, None, None, positions=torch.tensor([0, 1, 2, 3, 0, 1, 2]),
                last_token_index=torch.tensor([3, 6]))
    with torch.inference_mode():
        return m.compute_logits(m(ids))
sharded = logits_for(rank, world)          # all-reduces over gloo inside
if rank == 0:
    dist.barrier()
    whole = logits_for(0, 1)               # tp_size 1: no collective
    err = (sharded - whole).abs().max().item()
    print("TP_MAXERR", err)
    assert err < 1e-4, err
else:
    dist.barrier()
# every rank holds the same logits (replicated head on all-reduced activations)
gathered = [torch.zeros_like(sharded) for _ in range(world)]
dist.all_gather(gathered, sharded)
assert all(torch.equal(g, gathered[0]) for g in gathered)
dist.destroy_process_group()
'''


def test_tensor_parallel_sharding_matches_single_rank_on_gloo(tmp_path):
    script = tmp_path / "tp_worker.py"
    script.write_text(TP_WORKER)
    env = dict(os.environ, MV_ROOT=ROOT, MASTER_ADDR="127.0.0.1", MASTER_PORT="29611", WORLD_SIZE="2",
               OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert "TP_MAXERR" in outs[0]


def test_prefix_cache_reuses_full_blocks_but_never_the_last_one():
    bm = BlockManager(num_blocks=16, block_size=4, num_slots=4, prefix_caching=True)
    a = Sequence(list(range(10)), block_size=4)          # blocks [0-3], [4-7], [8,9]
    bm.allocate(a)
    assert a.num_cached_tokens == 0 and len(a.block_table) == 3
    b = Sequence(list(range(8)) + [99, 98, 97], block_size=4)   # same first two blocks
    bm.allocate(b)
    assert b.num_cached_tokens == 8 and b.block_table[:2] == a.block_table[:2] and b.block_table[2] != a.block_table[2]
    c = Sequence(list(range(8)), block_size=4)           # exactly the shared blocks: the last one is recomputed
    bm.allocate(c)
    assert c.num_cached_tokens == 4 and c.block_table[0] == a.block_table[0] and c.block_table[1] != a.block_table[1]
    # shared blocks survive the release of one owner and are revived from the free list
    bm.deallocate(a); bm.deallocate(b); bm.deallocate(c)
    assert len(bm.free_blocks) == 16
    d = Sequence(list(range(8)) + [5], block_size=4)
    bm.allocate(d)
    assert d.num_cached_tokens == 8
    # a block filled during decode becomes reusable once complete
    e = Sequence([7, 7, 7], block_size=4)
    bm.allocate(e)
    for tok in (1, 2):
        e.append_token(tok)
        bm.append(e)            # 5 tokens: the step that writes position 4 finds block 0 complete
    f = Sequence([7, 7, 7, 1, 2, 3], block_size=4)
    bm.allocate(f)
    assert f.num_cached_tokens == 4 and f.block_table[0] == e.block_table[0]


def test_scheduler_lookahead_bookkeeping_without_token_values():
    """advance() is postprocess() with the tokens still on the GPU: lengths grow, sequences finish by count,
    blocks are released; fill_tokens() patches the values in afterwards, also into finished sequences."""
    sch = Scheduler(max_num_seqs=4, max_num_batched_tokens=100, num_blocks=8, block_size=4, eos=-1)
    a = Sequence([1, 2, 3], SamplingParams(max_tokens=2, ignore_eos=True), block_size=4)
    b = Sequence([4, 5, 6, 7, 8], SamplingParams(max_tokens=1, ignore_eos=True), block_size=4)
    sch.add_sequence(a); sch.add_sequence(b)
    seqs, is_prefill = sch.schedule()
    assert is_prefill and sch.can_run_ahead(seqs) and sch.no_preemption_next()
    at = sch.advance(seqs)
    assert at == [3, 5] and b.is_finished and not a.is_finished and len(a) == 4
    nxt, is_prefill = sch.schedule()                      # the next step is schedulable before the tokens arrive
    assert not is_prefill and nxt == [a]
    at2 = sch.advance(nxt)
    assert a.is_finished and sch.is_finished()
    sch.fill_tokens(seqs, at, [10, 11])
    sch.fill_tokens(nxt, at2, [12])
    assert a.completion_token_ids == [10, 12] and b.completion_token_ids == [11]
    # a sequence that may stop on EOS cannot be run ahead of, nor can anything with the prefix cache on
    sch2 = Scheduler(max_num_seqs=2, max_num_batched_tokens=100, num_blocks=8, block_size=4, eos=7)
    c = Sequence([1, 2], SamplingParams(max_tokens=4, ignore_eos=False), block_size=4)
    assert not sch2.can_run_ahead([c])
    sch3 = Scheduler(max_num_seqs=2, max_num_batched_tokens=100, num_blocks=8, block_size=4, eos=-1, prefix_caching=True)
    assert not sch3.can_run_ahead([a])
