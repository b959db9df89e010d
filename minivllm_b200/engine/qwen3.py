"""Qwen3-shaped decoder used as the HARNESS that drives the attention path at
engine level (BASELINE configurations 3 and 4).  Everything here except the
`Attention` module is plain torch (cuBLAS GEMMs, torch's fused rms_norm) —
library code, out of the hot path's scope — with the tensor-parallel layout of
the reference (src/myvllm/models/qwen3.py, src/myvllm/layers/linear.py:83-221):
query/KV heads and the MLP are split across ranks, the only collectives are the
all-reduces after o_proj and down_proj, embedding and LM head are replicated.

Differences from the reference model, all forced by its defects: RoPE is
computed in fp32 and cast back to the model dtype (the reference promotes q/k
to fp32 and then fails in o_proj); positions come from the Context, built once
per step on the GPU (the reference rebuilds them on the host in every layer);
weights are seeded (the reference leaves them uninitialised).  Kept as in the
reference: RMSNorm eps 1e-5 whatever the config says, one shared gamma for the
q and k norms, tied embeddings when asked, and a residual stream that starts
from the normalised embedding (models/qwen3.py:186-190).  On CUDA the residual
adds, norms, SwiGLU activation and (under tensor parallelism) the all-reduces
run through the fused kernels of layers/layernorm.py, layers/activation.py and
layers/allreduce.py; CPU tensors take the plain torch formulation.
"""
import math
from dataclasses import dataclass

import torch
import torch.nn as nn
import torch.nn.functional as F

from ..layers.activation import silu_and_mul
from ..layers.allreduce import shard_rows
from ..layers.attention import Attention, qk_norm_rope_store
from ..layers.layernorm import add_rms_norm
from ..utils.context import get_context

RMS_EPS = 1e-5


@dataclass
class Qwen3Config:
    vocab_size: int = 151936
    hidden_size: int = 1024
    num_layers: int = 8
    num_heads: int = 16
    num_kv_heads: int = 8
    head_dim: int = 128
    intermediate_size: int = 3072
    rope_theta: float = 1e6
    max_position: int = 4096
    tie_word_embeddings: bool = True
    scale: float = 1.0
    block_size: int = 256
    fused_pre_attention: bool = True

    @staticmethod
    def from_dict(c):
        return Qwen3Config(vocab_size=c["vocab_size"], hidden_size=c["hidden_size"], num_layers=c["num_layers"],
                           num_heads=c["num_heads"], num_kv_heads=c["num_kv_heads"],
                           head_dim=c.get("head_dim", c["hidden_size"] // c["num_heads"]),
                           intermediate_size=c["intermediate_size"], rope_theta=c.get("base", 1e6),
                           max_position=c.get("max_position", c.get("max_model_length", 4096)),
                           tie_word_embeddings=c.get("tie_word_embeddings", True), scale=c.get("scale", 1.0),
                           block_size=c.get("block_size", 256),
                           fused_pre_attention=c.get("fused_pre_attention", True))


def _seeded_normal(shape, seed, device, std=0.02):
    """N(0, std) in fp32 from a generator keyed by `seed`: the FULL tensor, so that every
    tensor-parallel degree slices the same weights."""
    g = torch.Generator(device=device).manual_seed(seed)
    return torch.randn(shape, generator=g, device=device, dtype=torch.float32) * std


def _rope_cache(head_dim, max_position, theta, device):
    inv = 1.0 / (theta ** (torch.arange(0, head_dim, 2, dtype=torch.float32, device=device) / head_dim))
    ang = torch.arange(max_position, dtype=torch.float32, device=device)[:, None] * inv[None, :]
    return torch.cos(ang), torch.sin(ang)  # (max_position, head_dim/2) each


def apply_rope(x, cos, sin):
    """Rotate-half (neox) RoPE in fp32 on (tokens, heads, head_dim); cos/sin (tokens, head_dim/2)."""
    xf = x.float()
    x1, x2 = xf.chunk(2, dim=-1)
    c, s = cos[:, None, :], sin[:, None, :]
    return torch.cat([x1 * c - x2 * s, x2 * c + x1 * s], dim=-1).to(x.dtype)


class DecoderLayer(nn.Module):
    def __init__(self, cfg, layer, tp_rank, tp_size, dtype, device, seed):
        super().__init__()
        H, KVH, D, hid, inter = cfg.num_heads, cfg.num_kv_heads, cfg.head_dim, cfg.hidden_size, cfg.intermediate_size
        assert H % tp_size == 0 and KVH % tp_size == 0 and inter % tp_size == 0, "tp must divide heads and MLP"
        self.h, self.kvh, self.d, self.inter = H // tp_size, KVH // tp_size, D, inter // tp_size
        self.tp_size = tp_size
        base = seed * 1000003 + layer * 101
        r = tp_rank
        # column-parallel: rows of the (out, in) weight are sliced by head / by MLP column
        q_full = _seeded_normal((H * D, hid), base + 1, device)
        k_full = _seeded_normal((KVH * D, hid), base + 2, device)
        v_full = _seeded_normal((KVH * D, hid), base + 3, device)
        self.qkv_w = nn.Parameter(torch.cat([q_full[r * self.h * D:(r + 1) * self.h * D],
                                             k_full[r * self.kvh * D:(r + 1) * self.kvh * D],
                                             v_full[r * self.kvh * D:(r + 1) * self.kvh * D]]).to(dtype),
                                  requires_grad=False)
        del q_full, k_full, v_full
        # row-parallel: columns of the (out, in) weight are sliced
        o_full = _seeded_normal((hid, H * D), base + 4, device)
        self.o_w = nn.Parameter(o_full[:, r * self.h * D:(r + 1) * self.h * D].contiguous().to(dtype),
                                requires_grad=False)
        del o_full
        gate_full = _seeded_normal((inter, hid), base + 5, device)
        up_full = _seeded_normal((inter, hid), base + 6, device)
        self.gate_up_w = nn.Parameter(torch.cat([gate_full[r * self.inter:(r + 1) * self.inter],
                                                 up_full[r * self.inter:(r + 1) * self.inter]]).to(dtype),
                                      requires_grad=False)
        del gate_full, up_full
        down_full = _seeded_normal((hid, inter), base + 7, device)
        self.down_w = nn.Parameter(down_full[:, r * self.inter:(r + 1) * self.inter].contiguous().to(dtype),
                                   requires_grad=False)
        del down_full
        ones = lambda n: nn.Parameter(torch.ones(n, dtype=dtype, device=device), requires_grad=False)
        self.input_norm_w, self.post_norm_w, self.qk_norm_w = ones(hid), ones(hid), ones(D)
        self.attn = Attention(self.h, D, cfg.scale, self.kvh, cfg.block_size)
        # the fused kernel is CUDA-only and written for head_dim 128
        self.fused_pre_attention = cfg.fused_pre_attention and D == 128 and torch.device(device).type == "cuda"

    def forward(self, x, residual, cos, sin, rope=None):
        """Plain torch formulation (the reference's layer structure, src/myvllm/models/qwen3.py:186-217): the
        path of CPU tensors, i.e. of the tests and the CPU baseline that drive this harness with the oracle's
        attention.  CUDA tensors take `forward_fused`."""
        if residual is None:
            # first layer, as the reference has it (models/qwen3.py:186-190): the residual stream starts from
            # the NORMALISED embedding, not from the embedding itself
            h = F.rms_norm(x, (x.shape[-1],), self.input_norm_w, RMS_EPS)
            residual = h
        else:
            residual = residual + x
            h = F.rms_norm(residual, (residual.shape[-1],), self.input_norm_w, RMS_EPS)
        o = self._attention(F.linear(h, self.qkv_w), cos, sin, rope)
        o = F.linear(o, self.o_w)
        if self.tp_size > 1:
            torch.distributed.all_reduce(o)
        residual = residual + o
        h = F.rms_norm(residual, (residual.shape[-1],), self.post_norm_w, RMS_EPS)
        gu = F.linear(h, self.gate_up_w)
        act = F.silu(gu[:, :self.inter]) * gu[:, self.inter:]
        out = F.linear(act, self.down_w)
        if self.tp_size > 1:
            torch.distributed.all_reduce(out)
        return out, residual

    def _attention(self, qkv, cos, sin, rope):
        """q/k RMSNorm, RoPE, K/V store and attention on the fused qkv projection output."""
        v = qkv[:, (self.h + self.kvh) * self.d:].view(-1, self.kvh, self.d)   # v stays a strided view of qkv
        if self.fused_pre_attention:
            # one launch: q/k RMSNorm + RoPE + the K/V scatter into the paged cache
            ctx = get_context()
            a = self.attn
            q, k = qk_norm_rope_store(qkv, ctx.positions, rope[0], rope[1], self.qk_norm_w, self.qk_norm_w, RMS_EPS,
                                      self.h, self.kvh, self.d, a.k_cache, a.v_cache, ctx.slot_mapping,
                                      k_scale=a.k_scale, v_scale=a.v_scale)
            return a(q, k, v, store=False)
        # the reference's separate steps (src/myvllm/models/qwen3.py:104-110); the attention module stores K/V
        q, k, _ = qkv.split([self.h * self.d, self.kvh * self.d, self.kvh * self.d], dim=-1)
        q = F.rms_norm(q.reshape(-1, self.h, self.d), (self.d,), self.qk_norm_w, RMS_EPS)
        k = F.rms_norm(k.reshape(-1, self.kvh, self.d), (self.d,), self.qk_norm_w, RMS_EPS)
        q, k = apply_rope(q, cos, sin), apply_rope(k, cos, sin)
        return self.attn(q, k, v)

    def _reduce_add_norm(self, partial, residual, gamma, comm):
        """All-reduce of the row-parallel partial sums + residual add + RMSNorm with `gamma`.
        With a communicator: one kernel over NVLink peer memory; `partial` is the communicator's input buffer and
        `residual` this rank's row shard.  Without: NCCL (when sharded) and the local fused add + norm on the
        replicated residual.  Returns the normalised activations of ALL rows; `residual` is updated in place."""
        if comm is not None:
            return comm.allreduce_residual_rmsnorm(partial.shape[0], residual, gamma, RMS_EPS)
        if self.tp_size > 1:
            torch.distributed.all_reduce(partial)
        return add_rms_norm(partial, residual, gamma, RMS_EPS, residual_out=residual)

    def forward_fused(self, h, residual, next_gamma, rope, comm=None, cos=None, sin=None):
        """CUDA path.  `h` = normalised input of this layer (all rows), `residual` = the residual stream (this
        rank's row shard when `comm` is set, all rows otherwise), `next_gamma` = weight of the norm that follows
        this layer (next layer's input norm, or the final norm).  Returns the next layer's normalised input."""
        rows = h.shape[0]
        o = self._attention(F.linear(h, self.qkv_w), cos, sin, rope)
        partial = torch.mm(o, self.o_w.t(), out=comm.input_rows(rows)) if comm is not None else F.linear(o, self.o_w)
        h = self._reduce_add_norm(partial, residual, self.post_norm_w, comm)
        act = silu_and_mul(F.linear(h, self.gate_up_w))
        partial = torch.mm(act, self.down_w.t(), out=comm.input_rows(rows)) if comm is not None else \
            F.linear(act, self.down_w)
        return self._reduce_add_norm(partial, residual, next_gamma, comm)


class Qwen3ForCausalLM(nn.Module):
    def __init__(self, cfg: Qwen3Config, tp_rank=0, tp_size=1, dtype=torch.bfloat16, device="cuda", seed=0):
        super().__init__()
        self.cfg, self.tp_size, self.tp_rank, self.dtype = cfg, tp_size, tp_rank, dtype
        self.comm = None   # layers.allreduce.TPCommunicator, attached by the model runner under tensor parallelism
        self.embed = nn.Parameter(_seeded_normal((cfg.vocab_size, cfg.hidden_size), seed * 1000003 + 900001,
                                                 device).to(dtype), requires_grad=False)
        if cfg.tie_word_embeddings:
            self.lm_head = self.embed
        else:
            self.lm_head = nn.Parameter(_seeded_normal((cfg.vocab_size, cfg.hidden_size), seed * 1000003 + 900002,
                                                       device).to(dtype), requires_grad=False)
        self.layers = nn.ModuleList(DecoderLayer(cfg, l, tp_rank, tp_size, dtype, device, seed)
                                    for l in range(cfg.num_layers))
        self.final_norm_w = nn.Parameter(torch.ones(cfg.hidden_size, dtype=dtype, device=device), requires_grad=False)
        cos, sin = _rope_cache(cfg.head_dim, cfg.max_position, cfg.rope_theta, device)
        self.register_buffer("rope_cos", cos, persistent=False)
        self.register_buffer("rope_sin", sin, persistent=False)

    def forward(self, input_ids):
        """input_ids (tokens,) int64 -> hidden (tokens, hidden).  Positions come from the Context."""
        positions = get_context().positions
        if positions is None:
            raise ValueError("Context.positions must be set before the model runs")
        fused = all(l.fused_pre_attention for l in self.layers)
        x = F.embedding(input_ids, self.embed)
        cos, sin = (None, None) if fused else (self.rope_cos[positions], self.rope_sin[positions])
        if x.is_cuda:
            return self._forward_fused(x, cos, sin)
        residual = None
        for layer in self.layers:
            x, residual = layer(x, residual, cos, sin, (self.rope_cos, self.rope_sin))
        return F.rms_norm(residual + x, (x.shape[-1],), self.final_norm_w, RMS_EPS)

    def _forward_fused(self, x, cos=None, sin=None):
        """Every norm is fused with the add (and, under tensor parallelism, the all-reduce) in front of it, so a
        layer hands the next one its normalised input; with a communicator the residual stream is sharded by
        rows and never replicated."""
        rows = x.shape[0]
        comm = self.comm if self.comm is not None and rows <= self.comm.max_rows else None
        lo, hi = shard_rows(rows, self.tp_rank, self.tp_size) if comm is not None else (0, rows)
        h = add_rms_norm(x, None, self.layers[0].input_norm_w, RMS_EPS)
        residual = h[lo:hi].clone()      # the reference starts the residual stream from the normalised embedding
        rope = (self.rope_cos, self.rope_sin)
        for i, layer in enumerate(self.layers):
            nxt = self.layers[i + 1].input_norm_w if i + 1 < len(self.layers) else self.final_norm_w
            h = layer.forward_fused(h, residual, nxt, rope, comm, cos, sin)
        return h

    def compute_logits(self, hidden, vocab_shard=None):
        """Prefill keeps the last token of every sequence (Context.last_token_index); decode keeps all rows.
        vocab_shard = (rank, size): only that slice of the vocabulary rows of the (replicated) head, i.e.
        logits (rows, vocab / size) whose column 0 is token rank * vocab / size."""
        ctx = get_context()
        if ctx.is_prefill and ctx.last_token_index is not None:
            hidden = hidden[ctx.last_token_index]
        w = self.lm_head
        if vocab_shard is not None:
            rank, size = vocab_shard
            per = w.shape[0] // size
            w = w[rank * per:(rank + 1) * per]
        return F.linear(hidden, w)
