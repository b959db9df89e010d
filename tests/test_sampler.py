"""Greedy sampling tail: the oracle against torch.argmax on CPU, and (GPU) the kernels against the oracle,
bit-exact, through the C ABI."""
import os
import subprocess
import sys

import numpy as np
import pytest
import torch

from oracle import sampler_oracle as oracle


def _logits(seed, rows, cols, dtype, ties=True):
    g = torch.Generator().manual_seed(seed)
    x = (torch.randn(rows, cols, generator=g) * 3).to(dtype)
    if ties and cols >= 8:      # plant equal maxima: the lowest index must win
        for r in range(rows):
            idx = torch.randint(0, cols, (3,), generator=g)
            x[r, idx] = 40.0
    return x


@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_oracle_follows_torch_argmax(dtype):
    x = _logits(1, 6, 777, dtype)
    x[2, 500] = float("nan")
    x[2, 600] = float("nan")
    want = torch.argmax(x.float(), dim=-1).numpy()
    assert np.array_equal(oracle.argmax_rows(x.float().numpy()), want)
    assert int(want[2]) == 500


def test_sharded_oracle_equals_full_argmax():
    x = _logits(2, 5, 1024, torch.bfloat16).float().numpy()
    for shards in (1, 2, 4, 8):
        assert np.array_equal(oracle.argmax_sharded(x, shards), oracle.argmax_rows(x))


MERGE_WORKER = r'''
import os, sys, numpy as np, torch, torch.distributed as dist
sys.path.insert(0, os.environ["MV_ROOT"])
from oracle import sampler_oracle as oracle
rank, world = int(os.environ["RANK"]), int(os.environ["WORLD_SIZE"])
dist.init_process_group("gloo", rank=rank, world_size=world)
g = torch.Generator().manual_seed(11)
x = (torch.randn(7, 64, generator=g) * 2).bfloat16().float()
x[0, :] = -3.0                      # all equal: token 0
x[1, 10] = x[1, 50] = 9.0           # equal maxima in different shards: the lower index
x[2, 40] = float("nan")             # NaN is the maximum
w = 64 // world
keys = torch.tensor(oracle.shard_keys(x[:, rank * w:(rank + 1) * w].numpy(), rank * w), dtype=torch.int64)
dist.all_reduce(keys, op=dist.ReduceOp.MAX)
tokens = np.array([oracle.token_of_key(k) for k in keys.tolist()])
want = oracle.argmax_rows(x.numpy())
assert np.array_equal(tokens, want), (tokens, want)
assert tokens[0] == 0 and tokens[1] == 10 and tokens[2] == 40
print("MERGE_OK", rank)
dist.destroy_process_group()
'''


def test_shard_keys_merge_by_integer_max_over_two_gloo_ranks(tmp_path):
    """The multi-rank protocol on the CPU: every rank contributes one key per row, all-reduce(MAX), decode."""
    script = tmp_path / "merge_worker.py"
    script.write_text(MERGE_WORKER)
    root = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))
    env = dict(os.environ, MV_ROOT=root, MASTER_ADDR="127.0.0.1", MASTER_PORT="29617", WORLD_SIZE="2",
               OMP_NUM_THREADS="1")
    procs = [subprocess.Popen([sys.executable, str(script)], env=dict(env, RANK=str(r)), stdout=subprocess.PIPE,
                              stderr=subprocess.STDOUT, text=True) for r in range(2)]
    outs = [p.communicate(timeout=240)[0] for p in procs]
    assert all(p.returncode == 0 for p in procs), "\n".join(outs)
    assert all("MERGE_OK" in o for o in outs)


@pytest.mark.gpu
def test_gpu_keys_equal_the_oracle_keys():
    from minivllm_b200.layers import sampler as S
    x = _logits(6, 5, 512, torch.bfloat16)
    x[4, 100] = float("nan")
    keys, _ = S.argmax_rows(x.cuda(), index_offset=1000)
    assert keys.cpu().tolist() == oracle.shard_keys(x.float().numpy(), 1000)


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
@pytest.mark.parametrize("rows,cols", [(1, 8), (3, 1000), (5, 4099), (17, 18992), (2, 151936)])
def test_argmax_rows_on_gpu(dtype, rows, cols):
    from minivllm_b200.layers import sampler as S
    x = _logits(3, rows, cols, dtype)
    pad = (-cols) % 8
    buf = torch.zeros(rows, cols + pad, dtype=dtype)    # rows must start on 16-byte boundaries
    buf[:, :cols] = x
    view = buf.cuda()[:, :cols]
    want = oracle.argmax_rows(x.float().numpy())
    _, tokens = S.argmax_rows(view, want_keys=False, want_tokens=True)
    assert np.array_equal(tokens.cpu().numpy(), want)
    keys, _ = S.argmax_rows(view, index_offset=7)
    assert np.array_equal(S.decode_keys(keys).cpu().numpy(), want + 7)


@pytest.mark.gpu
def test_argmax_nan_and_negative_rows_on_gpu():
    from minivllm_b200.layers import sampler as S
    x = -torch.rand(4, 512).half() - 1.0                  # all negative: order of negative floats
    x[1, 300] = float("nan")
    x[1, 17] = float("nan")
    x[3, :] = float("-inf")
    want = oracle.argmax_rows(x.float().numpy())
    got = S.argmax_rows(x.cuda(), want_keys=False, want_tokens=True)[1].cpu().numpy()
    assert np.array_equal(got, want) and got[1] == 17 and got[3] == 0


@pytest.mark.gpu
@pytest.mark.parametrize("shards", [2, 8])
def test_vocabulary_shards_merge_to_the_full_argmax(shards):
    """Each shard reduced on its own (as a tensor-parallel rank does), keys merged by MAX, decoded."""
    from minivllm_b200.layers import sampler as S
    rows, cols = 9, 4096
    x = _logits(4, rows, cols, torch.bfloat16)
    x[0, :] = 1.0                                         # one row of all-equal logits: token 0
    w = cols // shards
    xd = x.cuda()
    keys = torch.stack([S.argmax_rows(xd[:, s * w:(s + 1) * w], index_offset=s * w)[0] for s in range(shards)])
    want = oracle.argmax_sharded(x.float().numpy(), shards)
    assert np.array_equal(S.decode_keys(keys.contiguous()).cpu().numpy(), want)
    assert np.array_equal(S.decode_keys(keys.max(dim=0).values).cpu().numpy(), want)   # what an all-reduce(MAX) leaves
    assert np.array_equal(want, oracle.argmax_rows(x.float().numpy()))


@pytest.mark.gpu
def test_argmax_rows_that_do_not_start_on_16_bytes():
    from minivllm_b200.layers import sampler as S
    x = _logits(5, 3, 1001, torch.float16)
    want = oracle.argmax_rows(x.float().numpy())
    assert np.array_equal(S.argmax_rows(x.cuda(), want_keys=False, want_tokens=True)[1].cpu().numpy(), want)


def test_zero_of_either_sign_is_one_logit_value():
    """-0.0 and +0.0 compare equal, so torch.argmax returns the lower index; the keys must agree."""
    x = -np.ones((3, 64), dtype=np.float32)
    x[0, 5], x[0, 40] = -0.0, 0.0
    x[1, 5], x[1, 40] = 0.0, -0.0
    x[2, 33] = -0.0
    want = torch.argmax(torch.from_numpy(x), dim=-1).numpy()
    assert want.tolist() == [5, 5, 33]
    assert np.array_equal(oracle.argmax_rows(x), want)
    for shards in (1, 2, 8):
        assert np.array_equal(oracle.argmax_sharded(x, shards), want)
    assert oracle.make_key(-0.0, 7) == oracle.make_key(0.0, 7)
    # merged by integer MAX of the shard keys, as the ranks do
    keys = [oracle.shard_keys(x[:, s * 32:(s + 1) * 32], s * 32) for s in range(2)]
    merged = [oracle.token_of_key(max(a, b)) for a, b in zip(*keys)]
    assert merged == want.tolist()


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_zero_of_either_sign_on_gpu(dtype):
    from minivllm_b200.layers import sampler as S
    x = -torch.ones(3, 4096, dtype=dtype)
    x[0, 5], x[0, 3000] = -0.0, 0.0          # different threads of the row's CTA
    x[1, 5], x[1, 3000] = 0.0, -0.0
    x[2, 2049] = -0.0
    want = torch.argmax(x.float(), dim=-1).numpy()
    xd = x.cuda()
    assert np.array_equal(S.argmax_rows(xd, want_keys=False, want_tokens=True)[1].cpu().numpy(), want)
    keys = torch.stack([S.argmax_rows(xd[:, s * 2048:(s + 1) * 2048], index_offset=s * 2048)[0] for s in range(2)])
    assert np.array_equal(S.decode_keys(keys.contiguous()).cpu().numpy(), want)
    want_keys = oracle.shard_keys(x.float().numpy())
    assert S.argmax_rows(xd)[0].cpu().tolist() == want_keys


# ---- temperature sampling (exponential race) -----------------------------------------------------------------
def test_philox_known_answers():
    """Philox4x32-10 known-answer vectors of the Random123 distribution (kat_vectors), for the oracle's restatement
    and for the library's own generator evaluated on the host."""
    import ctypes
    from minivllm_b200 import _cabi
    kat = [((0, 0, 0, 0), (0, 0), (0x6627e8d5, 0xe169c58d, 0xbc57ac4c, 0x9b00dbd8)),
           ((0xffffffff,) * 4, (0xffffffff,) * 2, (0x408f276d, 0x41c83b0e, 0xa20bc7c6, 0x6d5451fd)),
           ((0x243f6a88, 0x85a308d3, 0x13198a2e, 0x03707344), (0xa4093822, 0x299f31d0),
            (0xd16cfe09, 0x94fdcceb, 0x5001e420, 0x24126ea1))]
    for ctr, key, want in kat:
        assert oracle.philox4x32_10(ctr, key) == want
        out = (ctypes.c_uint32 * 4)()
        seed, step = key[0] | (key[1] << 32), ctr[2] | (ctr[3] << 32)
        assert _cabi.lib().mv_philox4x32_10(seed, step, ctr[1], ctr[0], out) == 0
        assert tuple(out) == want


def test_race_oracle_draws_from_the_softmax():
    """The restated race is a sampler of softmax(logits / T): empirical frequencies over many rows."""
    logits = np.array([2.0, 1.0, 0.0, -1.0, 0.5, 0.5], dtype=np.float32)
    rows, temp = 4000, 0.7
    toks, _ = oracle.sample_rows(np.tile(logits, (rows, 1)), [temp] * rows, seed=99, step=3)
    p = np.exp(logits / temp) / np.exp(logits / temp).sum()
    freq = np.bincount(toks, minlength=len(logits)) / rows
    assert np.abs(freq - p).max() < 0.03
    greedy, _ = oracle.sample_rows(np.tile(logits, (4, 1)), [0.0] * 4, seed=1, step=0)
    assert greedy.tolist() == [0] * 4


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", [torch.float16, torch.bfloat16])
def test_sampled_tokens_match_the_race_oracle(dtype):
    """Same seed, step, rows and columns -> same noise: the kernel's choice equals the oracle's except where the
    oracle's two best scores are closer than the kernel's fp32 rounding; rows with temperature 0 are greedy.
    Shards merged by MAX give the same tokens as the whole vocabulary."""
    from minivllm_b200.layers import sampler as S
    rows, cols = 12, 2048
    x = _logits(6, rows, cols, dtype)
    temps = torch.tensor([0.6, 1.0, 0.0, 2.5] * 3, dtype=torch.float32)
    step = torch.tensor([41], dtype=torch.int64, device="cuda")
    want, scores = oracle.sample_rows(x.float().numpy(), temps.numpy(), seed=1234, step=41)
    xd, td = x.cuda(), temps.cuda()
    got = S.sampled_tokens(xd, td, 1234, step).cpu().numpy()
    for r in range(rows):
        if got[r] != want[r]:
            top2 = np.sort(scores[r])[-2:]
            assert top2[1] - top2[0] < 1e-4 * max(1.0, abs(top2[1])), f"row {r}: {got[r]} vs {want[r]}"
    assert np.array_equal(got[2::4], oracle.argmax_rows(x.float().numpy())[2::4])
    for shards in (2, 8):
        w = cols // shards
        keys = torch.stack([S.sample_rows(xd[:, s * w:(s + 1) * w], td, 1234, step, index_offset=s * w)[0]
                            for s in range(shards)])
        assert np.array_equal(S.decode_keys(keys.contiguous()).cpu().numpy(), got)
    step.add_(1)
    again = S.sampled_tokens(xd, td, 1234, step).cpu().numpy()
    assert not np.array_equal(again[0::4], got[0::4]) or not np.array_equal(again[1::4], got[1::4])   # new noise
    assert np.array_equal(again[2::4], got[2::4])                                                   # greedy rows


@pytest.mark.gpu
def test_sampled_token_frequencies_follow_the_softmax():
    from minivllm_b200.layers import sampler as S
    logits = torch.tensor([2.0, 1.0, 0.0, -1.0, 0.5, 0.5, -3.0, 1.5], dtype=torch.float32)
    rows, temp = 40000, 0.6
    x = logits.to(torch.bfloat16).repeat(rows, 1).cuda()
    t = torch.full((rows,), temp, dtype=torch.float32, device="cuda")
    step = torch.zeros(1, dtype=torch.int64, device="cuda")
    toks = S.sampled_tokens(x, t, 7, step).cpu().numpy()
    z = logits.to(torch.bfloat16).float().numpy() / temp
    p = np.exp(z) / np.exp(z).sum()
    freq = np.bincount(toks, minlength=8) / rows
    assert np.abs(freq - p).max() < 0.01, (freq, p)
