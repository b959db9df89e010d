"""Attention module with the same interface as minivllm_b200.layers.attention.Attention
whose three operators are the CPU oracle (fp32).  Test infrastructure: it lets the
engine-level tests run the SAME model, scheduler and runner with only the attention
operators swapped, on GPU tensors (moved to the CPU and back) or on CPU tensors."""
import torch
import torch.nn as nn

from minivllm_b200.utils.context import get_context
from oracle import attention_oracle as oracle


class OracleAttention(nn.Module):
    def __init__(self, num_heads, head_dim, scale=1.0, num_kv_heads=None, block_size=16):
        super().__init__()
        self.num_heads, self.head_dim, self.scale = num_heads, head_dim, scale
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.block_size = block_size
        self.k_cache = self.v_cache = torch.tensor([])
        self.k_scale = self.v_scale = None      # set: int8 caches (codes) with fp16 scales

    def forward(self, q, k, v, store=True):
        ctx = get_context()
        dev, dt = q.device, q.dtype
        kc, vc = self.k_cache, self.v_cache
        int8 = self.k_scale is not None
        if kc.numel() > 0 and ctx.slot_mapping is not None:
            kcc, vcc = kc.cpu(), vc.cpu()
            if int8:
                ksc, vsc = self.k_scale.cpu(), self.v_scale.cpu()
                oracle.store_kvcache_int8(k.cpu(), v.cpu(), kcc, vcc, ksc, vsc, ctx.slot_mapping.cpu())
                self.k_scale.copy_(ksc)
                self.v_scale.copy_(vsc)
            else:
                oracle.store_kvcache(k.cpu(), v.cpu(), kcc, vcc, ctx.slot_mapping.cpu())
            kc.copy_(kcc)
            vc.copy_(vcc)
        scale = self.scale / self.head_dim ** 0.5
        if ctx.is_prefill:
            o = oracle.flash_attention_prefill(q.cpu(), k.cpu(), v.cpu(), ctx.cu_seqlens_q.cpu(), scale,
                                               self.num_heads, self.num_kv_heads, self.head_dim)
        else:
            kf, vf = kc.cpu(), vc.cpu()
            if int8:      # the decode kernel's contract: attention over float(code) * float(scale)
                kf = oracle.dequantize_kv_int8(kf, self.k_scale.cpu())
                vf = oracle.dequantize_kv_int8(vf, self.v_scale.cpu())
            o = oracle.paged_attention_decode(q.cpu(), kf, vf, ctx.block_tables.cpu(),
                                              ctx.context_lens.cpu(), scale, self.num_heads, self.num_kv_heads,
                                              self.head_dim, kc.shape[1])
        return o.to(dt).to(dev).reshape(o.shape[0], self.num_heads * self.head_dim)


def swap_in_oracle_attention(model):
    """Replaces every Attention of a Qwen3ForCausalLM harness by an OracleAttention sharing its caches."""
    for layer in model.layers:
        a = layer.attn
        o = OracleAttention(a.num_heads, a.head_dim, a.scale, a.num_kv_heads, a.block_size)
        o.k_cache, o.v_cache = a.k_cache, a.v_cache
        o.k_scale, o.v_scale = getattr(a, "k_scale", None), getattr(a, "v_scale", None)
        layer.attn = o
        layer.fused_pre_attention = False   # the reference path: separate norm, RoPE and store
    return model
