"""The metadata oracle against what the reference's own prepare_prefill /
prepare_decode returned for the same sequences (tests/golden/metadata_*.npz)."""
import ast

import numpy as np
import pytest

from oracle import metadata_oracle as mo


def load_case(golden_dir, name):
    z = np.load(f"{golden_dir}/{name}.npz")
    return z, ast.literal_eval(str(z["case"]))


def records(z, case, step=None):
    """Per-sequence records as the engine would hold them at prefill (step None) or after `step+1` appended tokens."""
    recs = []
    for i, prompt in enumerate(case["prompts"]):
        n = len(prompt) + (0 if step is None else step + 1)
        tables = z["prefill_tables" if step is None else f"decode{step}_tables_full"][i]
        rec = dict(num_tokens=n, num_cached_tokens=int(z["prefill_num_cached"][i]) if step is None else 0,
                   block_table=[int(b) for b in tables if b >= 0])
        if step is not None:
            rec["last_token"] = case["appended"][i][step]
        recs.append(rec)
    return recs


@pytest.mark.parametrize("name", ["metadata_bs4", "metadata_bs16"])
def test_prefill_metadata_matches_reference(golden_dir, name):
    z, case = load_case(golden_dir, name)
    bs = case["block_size"]
    got = mo.prepare_prefill(records(z, case), bs)
    assert np.array_equal(got["cu_seqlens_q"], z["prefill_cu_q"])
    assert np.array_equal(got["cu_seqlens_k"], z["prefill_cu_k"])
    assert np.array_equal(got["slot_mapping"], z["prefill_slot_mapping"])
    assert got["slot_mapping"].dtype == np.int64 and got["cu_seqlens_q"].dtype == np.int32


@pytest.mark.parametrize("name,steps", [("metadata_bs4", 1), ("metadata_bs16", 2)])
def test_decode_metadata_matches_reference(golden_dir, name, steps):
    z, case = load_case(golden_dir, name)
    bs = case["block_size"]
    for t in range(steps):
        recs = records(z, case, t)
        got = mo.prepare_decode(recs, bs)
        assert np.array_equal(got["input_ids"], z[f"decode{t}_input_ids"])
        assert np.array_equal(got["context_lens"], z[f"decode{t}_context_lens"])
        assert np.array_equal(got["block_tables"], z[f"decode{t}_block_tables"])
        ref_slots = z[f"decode{t}_slot_mapping"]
        for i, r in enumerate(recs):
            if r["num_tokens"] % bs == 0:
                # the reference counts zero tokens in an exactly full last block and writes to block*bs - 1;
                # the intended slot is the last one of that block
                assert ref_slots[i] == r["block_table"][-1] * bs - 1
                assert got["slot_mapping"][i] == r["block_table"][-1] * bs + bs - 1
            else:
                assert got["slot_mapping"][i] == ref_slots[i]


def test_known_answer_block_size_4(golden_dir):
    """The recorded known answer: seqs [1..10], [1..8,42], [7,7,7] allocated in that order."""
    z, case = load_case(golden_dir, "metadata_bs4")
    assert z["prefill_slot_mapping"].tolist() == list(range(10)) + [12, 16, 17, 18]
    assert z["decode0_slot_mapping"].tolist() == [10, 13, 15]          # 15 is the defect; intended 19
    got = mo.prepare_decode(records(z, case, 0), 4)
    assert got["slot_mapping"].tolist() == [10, 13, 19]
    assert got["positions"].tolist() == [10, 9, 3]
