"""CPU restatement of the fused layer steps around the attention path.  Test infrastructure: only tests/,
the smoke run and the benchmark's CPU legs may import this module.

  * `add_rms_norm`: the reference's residual add + RMSNorm, src/myvllm/layers/layernorm.py:10-28
    (x = x + residual in the model dtype; x / sqrt(mean(x^2) + eps) * gamma, evaluated in fp32 and rounded
    once, as the reference's compiled kernel does for fp16/bf16 inputs);
  * `allreduce_residual_rmsnorm`: the same step behind the all-reduce that ends a row-parallel linear layer,
    src/myvllm/layers/linear.py:216-221: partial sums added in fp32 in rank order, rounded to the model dtype
    (the all-reduced tensor), added to the residual, normalised.  Also returns the row partition the CUDA
    kernel uses (rank r owns ceil(rows/N) rows from r*ceil(rows/N));
  * `silu_and_mul`: src/myvllm/layers/activation.py:17-20, fp32 inside, rounded once.
"""
import torch


def shard_rows(rows, rank, world):
    per = (rows + world - 1) // world
    lo = min(rows, rank * per)
    return lo, min(rows, lo + per)


def rms_norm(x, gamma, eps):
    xf = x.float()
    return (xf * torch.rsqrt(xf.pow(2).mean(-1, keepdim=True) + eps) * gamma.float()).to(x.dtype)


def add_rms_norm(x, residual, gamma, eps):
    """Returns (normalised, new residual), both in x's dtype."""
    s = x if residual is None else (x.float() + residual.float()).to(x.dtype)
    return rms_norm(s, gamma, eps), s


def allreduce_residual_rmsnorm(partials, residual, gamma, eps):
    """partials: list over ranks of (rows, hidden) tensors in the model dtype; residual (rows, hidden).
    Returns (normalised rows, new residual) as every rank sees them after the step."""
    acc = torch.zeros_like(partials[0], dtype=torch.float32)
    for p in partials:                      # rank order, fp32
        acc = acc + p.float()
    o = acc.to(partials[0].dtype)           # what all_reduce would have left in the model dtype
    return add_rms_norm(o, residual, gamma, eps)


def silu_and_mul(gate_up):
    g, u = gate_up.float().chunk(2, dim=-1)
    return (g / (1.0 + torch.exp(-g)) * u).to(gate_up.dtype)
