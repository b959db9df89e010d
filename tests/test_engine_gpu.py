"""Engine-level parity on the GPU: the same harness model, scheduler and runner,
with the CUDA attention path (eager and CUDA-graph decode) against the CPU-oracle
attention operators.  Greedy token streams must be identical for the first 32 tokens, up to near-ties of the
logits (see _assert_same_up_to_near_ties)."""
import pytest
import torch

from minivllm_b200.engine.llm_engine import LLMEngine
from minivllm_b200.engine.sequence import SamplingParams
from oracle.attention_module import swap_in_oracle_attention

pytestmark = pytest.mark.gpu

CONFIG = dict(vocab_size=2048, hidden_size=256, num_layers=2, num_heads=4, num_kv_heads=2, head_dim=128,
              intermediate_size=512, base=1e6, max_position=512, max_model_length=512, tie_word_embeddings=True,
              scale=1.0, block_size=16, max_num_seqs=8, max_num_batched_tokens=512, num_kv_blocks=64, greedy=True,
              eos=-1, seed=0, dtype=torch.bfloat16)


def _prompts(n=6, seed=0):
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(3, 40, (n,), generator=g).tolist()
    return [torch.randint(0, CONFIG["vocab_size"], (l,), generator=g).tolist() for l in lens]


def _run(enforce_eager, oracle=False, max_tokens=40, config=None):
    torch.cuda.set_device(0)
    cfg = dict(config or CONFIG, enforce_eager=enforce_eager)
    eng = LLMEngine(cfg)
    if oracle:
        swap_in_oracle_attention(eng.model_runner.model)
    out = eng.generate(_prompts(), SamplingParams(temperature=0.0, max_tokens=max_tokens, ignore_eos=True))
    eng.exit()
    return out["token_ids"], eng


def _assert_same_up_to_near_ties(ours, ref, what, config=None, prompts=None):
    """Greedy streams must agree token for token, except that a stream may leave the other one where the two
    candidate tokens are a near-tie: kernels that differ only in summation order (how the KV tokens of a batch
    are cut into work items depends on the batch) can order two almost equal bf16 logits differently.  At the
    first divergence of a request the logits are recomputed by a full forward pass over the common history
    with the CPU-oracle attention, and the two tokens must be within 3 bf16 rounding steps of each other and
    of the maximum.  Nothing after a legitimate divergence is compared: the histories differ from there on."""
    from minivllm_b200.utils.context import reset_context, set_context
    prompts = _prompts() if prompts is None else prompts
    config = CONFIG if config is None else config
    model, identical = None, 0
    for r, (x, y) in enumerate(zip(ours, ref)):
        assert len(x) == len(y)
        i = next((k for k, (a, b) in enumerate(zip(x, y)) if a != b), None)
        if i is None:
            identical += 1
            continue
        if model is None:
            eng = LLMEngine(dict(config, enforce_eager=True))
            model = swap_in_oracle_attention(eng.model_runner.model)
        ids = torch.tensor(prompts[r] + y[:i], dtype=torch.int64, device="cuda")
        n = ids.numel()
        cu = torch.tensor([0, n], dtype=torch.int32, device="cuda")
        set_context(True, cu, cu, n, n, None, None, None, positions=torch.arange(n, device="cuda"),
                    last_token_index=torch.tensor([n - 1], device="cuda"))
        with torch.inference_mode():
            logits = model.compute_logits(model(ids)).float()[0]
        reset_context()
        top = float(logits.max())
        la, lb = float(logits[x[i]]), float(logits[y[i]])
        step = 2.0 ** -8 * max(abs(top), 1e-6)
        assert abs(la - lb) <= 3 * step and top - min(la, lb) <= 3 * step, \
            f"{what}: request {r} diverges at token {i} ({x[i]} vs {y[i]}) and it is no near-tie: " \
            f"logits {la} / {lb}, maximum {top}"
    return identical


def test_graph_decode_equals_eager_decode():
    eager, _ = _run(True)
    graph, eng = _run(False)
    assert eager == graph
    assert all(len(t) == 40 for t in graph)
    assert eng.stats["decode_tokens"] > 0 and eng.stats["prefill_tokens"] > 0


def test_greedy_stream_matches_oracle_attention_for_32_tokens():
    ours, _ = _run(False, max_tokens=32)
    ref, _ = _run(True, oracle=True, max_tokens=32)
    _assert_same_up_to_near_ties(ours, ref, "CUDA attention against the oracle attention")


def test_continuous_batching_with_preemption_keeps_streams():
    """A KV pool too small for all requests at once: sequences are preempted and recomputed; the
    greedy streams must not change."""
    big, _ = _run(False, max_tokens=24)
    small_cfg = dict(CONFIG, num_kv_blocks=9)       # 6 requests x up to 4 blocks do not fit
    small, eng = _run(False, max_tokens=24, config=small_cfg)
    _assert_same_up_to_near_ties(small, big, "with preemption against without")


def test_temperature_sampling_runs_in_graph_mode():
    torch.cuda.set_device(0)
    eng = LLMEngine(dict(CONFIG, greedy=False, enforce_eager=False))
    out = eng.generate(_prompts(4), SamplingParams(temperature=0.6, max_tokens=8, ignore_eos=True))
    assert all(len(t) == 8 and all(0 <= x < CONFIG["vocab_size"] for x in t) for t in out["token_ids"])
    eng.exit()


def test_mixed_temperatures_in_one_batch():
    """Requests at temperature 0 and 0.6 in the same batches (greedy=False engine): the temperature-0 requests
    generate exactly what the all-greedy engine generates, the others draw valid tokens, and the same seed
    reproduces the whole run."""
    torch.cuda.set_device(0)
    prompts = _prompts()
    greedy, _ = _run(False, max_tokens=16)

    def mixed():
        eng = LLMEngine(dict(CONFIG, greedy=False, enforce_eager=False, sample_seed=77))
        seqs = [eng.add_prompt(p, SamplingParams(temperature=0.0 if i % 2 == 0 else 0.6, max_tokens=16, ignore_eos=True))
                for i, p in enumerate(prompts)]
        while not eng.scheduler.is_finished():
            eng.step()
        eng.exit()
        return [s.completion_token_ids for s in seqs]
    a, b = mixed(), mixed()
    assert a == b
    assert all(a[i] == greedy[i] for i in range(0, len(prompts), 2))
    assert any(a[i] != greedy[i] for i in range(1, len(prompts), 2))
    assert all(0 <= t < CONFIG["vocab_size"] for toks in a for t in toks)


def test_greedy_engine_refuses_a_temperature():
    torch.cuda.set_device(0)
    eng = LLMEngine(dict(CONFIG, enforce_eager=True))
    with pytest.raises(ValueError, match="greedy=True"):
        eng.add_prompt([1, 2, 3], SamplingParams(temperature=0.6, max_tokens=4))
    eng.exit()


def test_a_kernel_wait_that_runs_out_surfaces_from_the_engine_step():
    """Host-side injection: one prefill launch withholds an mbarrier arrival, its bounded wait (200 ms) runs out
    and sets the error word; the engine reads the word with the step's tokens and raises instead of returning
    tokens sampled from an output that was never written.  The next engine on the same context is clean."""
    import ctypes
    from minivllm_b200 import _cabi
    torch.cuda.set_device(0)
    eng = LLMEngine(dict(CONFIG, enforce_eager=True))
    eng.add_prompt(list(range(1, 130)), SamplingParams(temperature=0.0, max_tokens=4, ignore_eos=True))
    assert _cabi.lib().mv_debug_prefill_inject(ctypes.c_int(1)) == 0
    with pytest.raises(RuntimeError, match="ran out of time"):
        eng.step()
    eng.exit()
    again, _ = _run(True, max_tokens=4)
    assert all(len(t) == 4 for t in again)


def test_int8_kv_cache_engine_matches_the_oracle_on_the_dequantised_cache():
    """kv_cache_dtype='int8': K/V rows are quantised per token and head inside the fused pre-attention kernel
    and the decode kernel reads codes and scales.  The oracle engine quantises with the CPU definition and
    attends over float(code) * float(scale).  Codes and scales are bit-identical on both sides, so the two
    engines compute the same function up to rounding: greedy streams must agree for 32 tokens in all but at most
    one request (a near-tie of the quantised model's logits cannot be re-checked with the unquantised forward
    pass the other tests use), and the int8 engine's graph and eager decode agree exactly."""
    cfg = dict(CONFIG, kv_cache_dtype="int8")
    graph, eng = _run(False, max_tokens=32, config=cfg)
    assert eng.model_runner.kv_cache.dtype == torch.int8 and eng.model_runner.kv_scale is not None
    eager, _ = _run(True, max_tokens=32, config=cfg)
    assert graph == eager
    ref, _ = _run(True, oracle=True, max_tokens=32, config=cfg)
    same = sum(a == b for a, b in zip(graph, ref))
    print(f"\nint8 KV cache: {same}/{len(graph)} requests token-identical for 32 tokens")
    assert same >= len(graph) - 1
    with pytest.raises(ValueError, match="prefix caching"):
        LLMEngine(dict(cfg, enable_prefix_caching=True))


def test_prefix_caching_keeps_streams_and_hits_the_cache():
    """Prompts that share their first 48 tokens (3 blocks of 16): with the prefix cache on, later requests
    feed only their uncached suffix through the paged prefill kernel; greedy streams must not change."""
    torch.cuda.set_device(0)
    g = torch.Generator().manual_seed(3)
    shared = torch.randint(0, CONFIG["vocab_size"], (48,), generator=g).tolist()
    prompts = [shared + torch.randint(0, CONFIG["vocab_size"], (n,), generator=g).tolist() for n in (5, 17, 1, 30)]
    sp = SamplingParams(temperature=0.0, max_tokens=20, ignore_eos=True)
    outs = {}
    for caching in (False, True):
        eng = LLMEngine(dict(CONFIG, enforce_eager=False, enable_prefix_caching=caching, max_num_seqs=2))
        outs[caching] = eng.generate(prompts, sp)["token_ids"]
        hits = eng.scheduler.block_manager.cached_hits
        eng.exit()
        assert (hits > 0) == caching
    assert outs[True] == outs[False]


def test_engine_configuration_3_streams_against_oracle_attention():
    """The 1-GPU engine configuration of the benchmark plan (hidden 1024, 8 layers, 16q/8kv heads of 128,
    vocabulary 151,936, 60 prompts of 16-64 random tokens, greedy) for 32 tokens: the CUDA attention path
    (fused q/k norm + RoPE + store, varlen prefill, graph-replayed paged decode) against the same engine with the
    reference's separate q/k norm and RoPE and the CPU-oracle attention operators.  Counts and prints the
    requests whose 32 tokens are identical; every other request must part at a verified near-tie of the logits
    (a random-init model over 151,936 tokens has the top two logits within a few bf16 steps of each other in a
    sizeable share of positions)."""
    from minivllm_b200.engine import configs
    torch.cuda.set_device(0)
    cfg = configs.small_qwen3_config(greedy=True, num_kv_blocks=64, max_num_seqs=64)
    prompts, _ = configs.small_qwen3_requests()
    sp = SamplingParams(temperature=0.0, max_tokens=32, ignore_eos=True)

    def run(oracle):
        eng = LLMEngine(dict(cfg, enforce_eager=oracle))
        if oracle:
            swap_in_oracle_attention(eng.model_runner.model)
        out = eng.generate(prompts, sp)["token_ids"]
        eng.exit()
        return out
    ours, ref = run(False), run(True)
    assert all(len(t) == 32 for t in ours)
    identical = _assert_same_up_to_near_ties(ours, ref, "configuration 3", config=cfg, prompts=prompts)
    print(f"\nconfiguration 3: {identical}/{len(prompts)} requests token-identical for 32 tokens; the others part at "
          f"verified near-ties")
    assert identical >= 57


def test_two_prefill_waves_in_flight_keep_the_streams():
    """prefill_streams=2: prefill waves alternate between two side streams and overlap on the GPU; the token
    streams are those of the one-stream engine.  max_num_batched_tokens is small so that
    the six prompts make several waves, and the second configuration also preempts and prefills again."""
    for extra in (dict(max_num_batched_tokens=48), dict(max_num_batched_tokens=48, num_kv_blocks=9)):
        one, _ = _run(False, max_tokens=24, config=dict(CONFIG, prefill_streams=1, **extra))
        two, eng = _run(False, max_tokens=24, config=dict(CONFIG, prefill_streams=2, **extra))
        assert eng.model_runner._prefill_at >= 3, "the prompts were meant to take several waves"
        _assert_same_up_to_near_ties(two, one, "two prefill streams against one", config=dict(CONFIG, **extra))
