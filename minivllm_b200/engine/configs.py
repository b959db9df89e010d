"""The two engine configurations of the benchmark plan, as config dicts in the
reference's style (plain dict, R/main.py:15-41) plus seeded prompt generators.
Random-init weights (seed 0, N(0, 0.02)) and random token ids stand in for a
checkpoint and a dataset; nothing is downloaded.
"""
import torch

from .sequence import SamplingParams

VOCAB = 151936


def small_qwen3_config(world_size=1, **over):
    """hidden 1024, 8 layers, 16 q / 8 kv heads, head_dim 128, SwiGLU 3072, tied embeddings, bf16."""
    c = dict(vocab_size=VOCAB, hidden_size=1024, num_layers=8, num_heads=16, num_kv_heads=8, head_dim=128,
             intermediate_size=3072, base=1e6, max_model_length=1024, tie_word_embeddings=True, scale=1.0,
             block_size=256, max_num_seqs=256, max_num_batched_tokens=16384, gpu_memory_utilization=0.5,
             greedy=False, eos=-1, seed=0, world_size=world_size, dtype=torch.bfloat16)
    c.update(over)
    return c


def small_qwen3_requests(seed=0, n=60):
    """60 prompts of random token ids, lengths uniform in [16, 64]; 256 new tokens at temperature 0.6."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(16, 65, (n,), generator=g).tolist()
    prompts = [torch.randint(0, VOCAB, (l,), generator=g).tolist() for l in lens]
    return prompts, SamplingParams(temperature=0.6, max_tokens=256, ignore_eos=True)


def qwen3_8b_config(world_size=1, **over):
    """Qwen3-8B shape: hidden 4096, 36 layers, 32 q / 8 kv heads, head_dim 128, SwiGLU 12288, bf16,
    KV cache = 80 % of free HBM, 512 sequences, 16,384-token prefill waves."""
    c = dict(vocab_size=VOCAB, hidden_size=4096, num_layers=36, num_heads=32, num_kv_heads=8, head_dim=128,
             intermediate_size=12288, base=1e6, max_model_length=2048, tie_word_embeddings=False, scale=1.0,
             block_size=256, max_num_seqs=512, max_num_batched_tokens=16384, gpu_memory_utilization=0.8,
             greedy=True, eos=-1, seed=0, world_size=world_size, dtype=torch.bfloat16)
    c.update(over)
    return c


def qwen3_8b_requests(seed=0, n=512, new_tokens=512):
    """512 requests, prompt lengths uniform in [512, 1536] of random token ids, 512 greedy output tokens each."""
    g = torch.Generator().manual_seed(seed)
    lens = torch.randint(512, 1537, (n,), generator=g).tolist()
    prompts = [torch.randint(0, VOCAB, (l,), generator=g).tolist() for l in lens]
    return prompts, SamplingParams(temperature=0.0, max_tokens=new_tokens, ignore_eos=True)
