"""CPU oracle for the step metadata.  TEST INFRASTRUCTURE ONLY (see
attention_oracle.py for the rules on who may import this).

Restates src/myvllm/engine/model_runner.py:180-256 (`prepare_prefill`,
`prepare_decode`) and the positions of src/myvllm/models/qwen3.py:196-212 as
plain loops over per-sequence records.  A record is a dict with
`num_tokens` (tokens of the sequence, including the one fed in decode),
`num_cached_tokens`, `block_table` (list of physical block ids) and, for
decode, `last_token`.

Pinned: tests/golden/metadata_*.npz hold what the reference's own functions
return for the same sequences (made by tests/golden/make_golden.py through the
reference's Sequence / BlockManager / ModelRunner code).  One deliberate
difference: the reference counts ZERO tokens in a last block that is exactly
full (src/myvllm/engine/sequence.py:69-72), which sends the decode write to
`block*bs - 1` and drops prefill slots; here a full last block holds
block_size tokens.  The tests compare everything else bit for bit and check
the differing entries against the intended value.
"""
import numpy as np


def prepare_prefill(seqs, block_size):
    input_positions, slot_mapping, cu_q, cu_k, last_index = [], [], [0], [0], []
    for s in seqs:
        n, c, bt = s["num_tokens"], s["num_cached_tokens"], s["block_table"]
        cu_q.append(cu_q[-1] + n - c)
        cu_k.append(cu_k[-1] + n)
        last_index.append(cu_q[-1] - 1)
        for p in range(c, n):
            input_positions.append(p)
            slot_mapping.append(bt[p // block_size] * block_size + p % block_size)
    max_blocks = max(len(s["block_table"]) for s in seqs)
    tables = np.full((len(seqs), max_blocks), -1, dtype=np.int32)
    for i, s in enumerate(seqs):
        tables[i, :len(s["block_table"])] = s["block_table"]
    return dict(cu_seqlens_q=np.array(cu_q, np.int32), cu_seqlens_k=np.array(cu_k, np.int32),
                positions=np.array(input_positions, np.int64), slot_mapping=np.array(slot_mapping, np.int64),
                last_token_index=np.array(last_index, np.int64), block_tables=tables,
                max_seqlen_q=max(s["num_tokens"] - s["num_cached_tokens"] for s in seqs),
                max_seqlen_k=max(s["num_tokens"] for s in seqs))


def prepare_decode(seqs, block_size):
    input_ids, context_lens, slot_mapping, positions = [], [], [], []
    for s in seqs:
        n, bt = s["num_tokens"], s["block_table"]
        p = n - 1  # the token being fed is the last one of the sequence
        input_ids.append(s["last_token"])
        context_lens.append(n)
        positions.append(p)
        slot_mapping.append(bt[p // block_size] * block_size + p % block_size)
    max_blocks = max(len(s["block_table"]) for s in seqs)
    tables = np.full((len(seqs), max_blocks), -1, dtype=np.int32)
    for i, s in enumerate(seqs):
        tables[i, :len(s["block_table"])] = s["block_table"]
    return dict(input_ids=np.array(input_ids, np.int64), context_lens=np.array(context_lens, np.int64),
                positions=np.array(positions, np.int64), slot_mapping=np.array(slot_mapping, np.int64),
                block_tables=tables)
