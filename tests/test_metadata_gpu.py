"""On-GPU step metadata (C ABI) against the oracle and the reference's recorded outputs: bit-exact."""
import numpy as np
import pytest
import torch

from minivllm_b200.engine.metadata import SequenceStateTable
from oracle import metadata_oracle as mo
from tests.test_metadata_oracle import load_case, records

pytestmark = pytest.mark.gpu
DEV = "cuda:0"


def _state_for(recs, block_size, max_blocks=8, num_slots=16, slot_of=None):
    st = SequenceStateTable(num_slots, max_blocks, block_size, DEV)
    slots = slot_of or list(range(3, 3 + len(recs)))   # not slot == row, on purpose
    for s, r in zip(slots, recs):
        st.assign_sequence(s, r["block_table"])
    return st, slots


@pytest.mark.parametrize("name", ["metadata_bs4", "metadata_bs16"])
def test_prefill_metadata_on_gpu(golden_dir, name):
    z, case = load_case(golden_dir, name)
    bs = case["block_size"]
    recs = records(z, case)
    st, slots = _state_for(recs, bs)
    got = st.build_prefill(slots, [r["num_tokens"] for r in recs], [r["num_cached_tokens"] for r in recs])
    want = mo.prepare_prefill(recs, bs)
    torch.cuda.synchronize()
    for k in ("cu_seqlens_q", "cu_seqlens_k", "positions", "slot_mapping", "last_token_index"):
        assert np.array_equal(got[k].cpu().numpy(), want[k]), k
        assert got[k].cpu().numpy().dtype == want[k].dtype, k
    assert np.array_equal(got["slot_mapping"].cpu().numpy(), z["prefill_slot_mapping"])
    assert got["max_seqlen_q"] == want["max_seqlen_q"] and got["max_seqlen_k"] == want["max_seqlen_k"]
    assert st.seq_lens[slots].tolist() == [r["num_tokens"] for r in recs]


@pytest.mark.parametrize("name,steps", [("metadata_bs4", 1), ("metadata_bs16", 2)])
def test_decode_metadata_on_gpu(golden_dir, name, steps):
    z, case = load_case(golden_dir, name)
    bs = case["block_size"]
    recs0 = records(z, case)
    st, slots = _state_for(recs0, bs)
    st.build_prefill(slots, [r["num_tokens"] for r in recs0])      # sets seq_lens = prompt lengths
    pad = 8
    bufs = st.new_decode_buffers(pad)
    slots_dev = torch.zeros(pad, dtype=torch.int32, device=DEV)
    slots_dev[:len(slots)] = torch.tensor(slots, dtype=torch.int32)
    n_active = torch.tensor([len(slots)], dtype=torch.int32, device=DEV)
    for t in range(steps):
        recs = records(z, case, t)
        # host side of a step: new blocks go to the device table, sampled tokens to last_token
        st.update_tables((s, len(r["block_table"]) - 1, r["block_table"][-1]) for s, r in zip(slots, recs))
        st.last_token[torch.tensor(slots, device=DEV)] = torch.tensor([r["last_token"] for r in recs], device=DEV)
        st.build_decode(slots_dev, n_active, bufs)
        torch.cuda.synchronize()
        want = mo.prepare_decode(recs, bs)
        n = len(slots)
        for k in ("input_ids", "context_lens", "positions", "slot_mapping"):
            assert np.array_equal(bufs[k][:n].cpu().numpy(), want[k]), (t, k)
        wt = want["block_tables"]
        assert np.array_equal(bufs["block_tables"][:n, :wt.shape[1]].cpu().numpy(), wt)
        assert bool((bufs["block_tables"][:n, wt.shape[1]:] == -1).all())
        # padded rows of a captured batch
        assert bufs["slot_mapping"][n:].tolist() == [-1] * (pad - n)
        assert bufs["context_lens"][n:].tolist() == [0] * (pad - n)
        assert bool((bufs["block_tables"][n:] == -1).all())
        assert np.array_equal(bufs["context_lens"][:n].cpu().numpy(), z[f"decode{t}_context_lens"])


def test_metadata_large_ragged_batch():
    """600 sequences (more than one scan pass), random lengths, 256-token blocks."""
    g = torch.Generator().manual_seed(9)
    bs, nseq = 256, 600
    lens = torch.randint(1, 1500, (nseq,), generator=g).tolist()
    perm = torch.randperm(5000, generator=g).tolist()
    recs, at = [], 0
    for n in lens:
        nb = (n + bs - 1) // bs
        recs.append(dict(num_tokens=n, num_cached_tokens=0, block_table=perm[at:at + nb], last_token=n % 97))
        at += nb
    st = SequenceStateTable(1024, 8, bs, DEV)
    slots = torch.randperm(1024, generator=g)[:nseq].tolist()
    rows = torch.full((1024, 8), -1, dtype=torch.int32)
    for s, r in zip(slots, recs):
        rows[s, :len(r["block_table"])] = torch.tensor(r["block_table"], dtype=torch.int32)
    st.tables.copy_(rows)
    got = st.build_prefill(slots, lens)
    want = mo.prepare_prefill(recs, bs)
    torch.cuda.synchronize()
    for k in ("cu_seqlens_q", "cu_seqlens_k", "positions", "slot_mapping", "last_token_index"):
        assert np.array_equal(got[k].cpu().numpy(), want[k]), k
