"""Attention operators of the engine, routed through the C-ABI library into
hand-written sm_100a CUDA.

Same names and positional arguments as src/myvllm/layers/attention.py of the
reference (`store_kvcache` :67, `flash_attention_prefill` :212,
`paged_attention_decode` :418, `Attention` :476), so the reference's call
sites (src/myvllm/models/qwen3.py:110) work unchanged.  There is no Triton, no
PyTorch and no CPU path behind these functions: a missing library raises.

Differences from the reference, all deliberate:
  * no `.contiguous()` copies: token strides are passed to the kernels, so the
    non-contiguous `v` split view of a fused qkv projection is read in place;
  * the block size used to address the cache is the cache's own second
    dimension; the `block_size` argument is only checked against it (the
    reference module defaults it to 16 while the engine allocates 256-token
    blocks, which corrupts decode);
  * optional int8 caches (`k_scale` / `v_scale` keyword arguments).
"""
import torch
import torch.nn as nn

from .. import _cabi
from ..utils.context import get_context

_workspaces = {}


def _decode_workspace(device, nbytes):
    """Grow-only scratch per device for the split-K partial results (zero-filled: its first 64 KiB are the
    arrival counters of split sequences, which every call leaves zero)."""
    ws = _workspaces.get(device)
    if ws is None or ws.numel() < nbytes:
        ws = torch.zeros(max(nbytes, 1 << 20), dtype=torch.uint8, device=device)
        _workspaces[device] = ws
    return ws


def _row_stride(x, name):
    """Token stride (elements) of a (tokens, heads, head_dim) tensor whose last two dims are dense."""
    t, h, d = x.shape
    if x.stride(2) != 1 or (h > 1 and x.stride(1) != d):
        raise ValueError(f"{name}: heads and head_dim must be contiguous within a token")
    return x.stride(0) if t > 1 else h * d


def store_kvcache(key, value, k_cache, v_cache, slot_mapping, block_size, k_scale=None, v_scale=None):
    """Scatter `key`/`value` (tokens, kv_heads, head_dim) into the paged caches
    (blocks, block_size, kv_heads, head_dim) at `slot_mapping` (int64, -1 skips).

    With `k_scale`/`v_scale` (blocks, block_size, kv_heads) fp16 tensors the
    caches are int8 and rows are quantised per token and head on the way in.
    Reference: src/myvllm/layers/attention.py:67-108.
    """
    _cabi.require_cuda(key, value, k_cache, v_cache, slot_mapping)
    num_tokens, num_kv_heads, head_dim = key.shape
    assert value.shape == key.shape, "K and V shapes must match"
    assert k_cache.shape == v_cache.shape, "K and V cache shapes must match"
    assert slot_mapping.numel() == num_tokens, "Slot mapping size must match number of tokens"
    if k_cache.dim() != 4 or k_cache.shape[2] != num_kv_heads or k_cache.shape[3] != head_dim:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={num_kv_heads}, head_dim={head_dim}")
    if block_size != k_cache.shape[1]:
        raise ValueError(f"block_size {block_size} differs from the cache's block dimension {k_cache.shape[1]}")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches must be contiguous")
    if slot_mapping.dtype != torch.int64 or not slot_mapping.is_contiguous():
        raise ValueError("slot_mapping must be a contiguous int64 tensor")
    if value.dtype != key.dtype:
        raise ValueError("key and value dtypes differ")
    quant = k_scale is not None or v_scale is not None
    if quant:
        if k_scale is None or v_scale is None:
            raise ValueError("k_scale and v_scale must be given together")
        if k_cache.dtype != torch.int8 or v_cache.dtype != torch.int8:
            raise ValueError("int8 caches are required when scales are given")
        for s in (k_scale, v_scale):
            if s.dtype != torch.float16 or tuple(s.shape) != tuple(k_cache.shape[:3]) or not s.is_contiguous():
                raise ValueError("scales must be contiguous fp16 tensors of shape (blocks, block_size, kv_heads)")
    elif k_cache.dtype != key.dtype:
        raise ValueError(f"cache dtype {k_cache.dtype} differs from key dtype {key.dtype}")
    num_slots = k_cache.shape[0] * k_cache.shape[1]
    rc = _cabi.lib().mv_store_kvcache(
        key.data_ptr(), value.data_ptr(), _row_stride(key, "key"), _row_stride(value, "value"),
        k_cache.data_ptr(), v_cache.data_ptr(),
        k_scale.data_ptr() if quant else None, v_scale.data_ptr() if quant else None,
        slot_mapping.data_ptr(), num_tokens, num_slots, num_kv_heads, head_dim,
        _cabi.dtype_code(key.dtype), _cabi.stream_ptr())
    _cabi.check(rc)


def paged_attention_decode(query, k_cache, v_cache, block_tables, context_lens, scale, num_heads, num_kv_heads,
                           head_dim, block_size, k_scale=None, v_scale=None, workspace=None):
    """Decode attention of one new token per sequence over the paged cache.

    query (batch, heads, head_dim); block_tables (batch, max_blocks) int32,
    negative entries carry no tokens; context_lens (batch,) int32 or int64.
    Returns a new (batch, heads, head_dim) tensor in query's dtype.
    Reference: src/myvllm/layers/attention.py:418-473.
    """
    _cabi.require_cuda(query, k_cache, v_cache, block_tables, context_lens)
    batch = query.shape[0]
    if tuple(query.shape) != (batch, num_heads, head_dim):
        raise ValueError(f"query shape {tuple(query.shape)} is not (batch, {num_heads}, {head_dim})")
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape or k_cache.shape[2] != num_kv_heads or \
            k_cache.shape[3] != head_dim:
        raise ValueError(f"cache shape {tuple(k_cache.shape)} does not match kv_heads={num_kv_heads}, head_dim={head_dim}")
    if block_size != k_cache.shape[1]:
        raise ValueError(f"block_size {block_size} differs from the cache's block dimension {k_cache.shape[1]}")
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] != batch or \
            block_tables.stride(1) != 1:
        raise ValueError("block_tables must be a (batch, max_blocks) int32 tensor with dense rows")
    if context_lens.dtype not in (torch.int32, torch.int64) or context_lens.numel() != batch or \
            not context_lens.is_contiguous():
        raise ValueError("context_lens must be a contiguous (batch,) int32 or int64 tensor")
    quant = k_scale is not None or v_scale is not None
    if quant:
        if k_scale is None or v_scale is None:
            raise ValueError("k_scale and v_scale must be given together")
        if k_cache.dtype != torch.int8 or v_cache.dtype != torch.int8:
            raise ValueError("int8 caches are required when scales are given")
        for s in (k_scale, v_scale):
            if s.dtype != torch.float16 or tuple(s.shape) != tuple(k_cache.shape[:3]) or not s.is_contiguous():
                raise ValueError("scales must be contiguous fp16 tensors of shape (blocks, block_size, kv_heads)")
    elif k_cache.dtype != query.dtype or v_cache.dtype != query.dtype:
        raise ValueError(f"cache dtype {k_cache.dtype} differs from query dtype {query.dtype}")
    if not (k_cache.is_contiguous() and v_cache.is_contiguous()):
        raise ValueError("caches must be contiguous")
    if not query.is_contiguous():
        query = query.contiguous()
    out = torch.empty_like(query)
    if batch == 0:
        return out
    max_blocks = block_tables.shape[1]
    L = _cabi.lib()
    need = L.mv_paged_decode_workspace_bytes(batch, num_heads, num_kv_heads, head_dim, max_blocks, block_size)
    if need < 0:
        raise ValueError("paged_attention_decode: invalid shape")
    if workspace is None:
        workspace = _decode_workspace(query.device, need)
    rc = L.mv_paged_decode(
        out.data_ptr(), query.data_ptr(), k_cache.data_ptr(), v_cache.data_ptr(),
        k_scale.data_ptr() if quant else None, v_scale.data_ptr() if quant else None,
        block_tables.data_ptr(), block_tables.stride(0) if batch > 1 else max_blocks, max_blocks,
        context_lens.data_ptr(), 1 if context_lens.dtype == torch.int64 else 0,
        batch, num_heads, num_kv_heads, head_dim, block_size, k_cache.shape[0], float(scale),
        workspace.data_ptr(), workspace.numel() * workspace.element_size(),
        _cabi.dtype_code(query.dtype), _cabi.stream_ptr())
    _cabi.check(rc)
    return out


_error_words = {}


def _error_word(device):
    """One int32 per device that the prefill kernel sets when one of its bounded waits runs out."""
    w = _error_words.get(device)
    if w is None:
        w = torch.zeros(1, dtype=torch.int32, device=device)
        _error_words[device] = w
    return w


def prefill_error_code(device=None, clear=True):
    """Reads (synchronising) the prefill kernel's error word; 0 means every wait completed."""
    device = torch.device("cuda", torch.cuda.current_device()) if device is None else torch.device(device)
    w = _error_words.get(device)
    if w is None:
        return 0
    code = int(w.item())
    if code and clear:
        w.zero_()
    return code


def flash_attention_prefill(q, k, v, cu_seqlens, scale, num_heads, num_kv_heads, head_dim):
    """Causal attention over a packed batch of sequences (prefill).

    q (tokens, heads, head_dim), k/v (tokens, kv_heads, head_dim), cu_seqlens
    (num_seqs + 1,) int32 prefix sums.  Returns a new (tokens, heads, head_dim)
    tensor.  Unlike the reference (src/myvllm/layers/attention.py:212-280)
    there is no `.contiguous()` copy and no `cu_seqlens.cpu()` sync.
    """
    _cabi.require_cuda(q, k, v, cu_seqlens)
    total = q.shape[0]
    if tuple(q.shape) != (total, num_heads, head_dim) or tuple(k.shape) != (total, num_kv_heads, head_dim) or \
            tuple(v.shape) != tuple(k.shape):
        raise ValueError("q/k/v shapes do not match (tokens, heads, head_dim) / (tokens, kv_heads, head_dim)")
    if cu_seqlens.dtype != torch.int32 or cu_seqlens.dim() != 1 or not cu_seqlens.is_contiguous():
        raise ValueError("cu_seqlens must be a contiguous int32 vector")
    if k.dtype != q.dtype or v.dtype != q.dtype:
        raise ValueError("q, k and v dtypes differ")
    out = torch.empty((total, num_heads, head_dim), dtype=q.dtype, device=q.device)
    num_seqs = cu_seqlens.numel() - 1
    if total == 0 or num_seqs <= 0:
        return out
    rc = _cabi.lib().mv_prefill_varlen(
        out.data_ptr(), q.data_ptr(), k.data_ptr(), v.data_ptr(), _row_stride(q, "q"), _row_stride(k, "k"),
        _row_stride(v, "v"), cu_seqlens.data_ptr(), num_seqs, total, num_heads, num_kv_heads, head_dim, float(scale),
        _error_word(q.device).data_ptr(), _cabi.dtype_code(q.dtype), _cabi.stream_ptr())
    _cabi.check(rc)
    return out


def flash_attention_prefill_paged(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables, scale, num_heads,
                                  num_kv_heads, head_dim):
    """Prefill attention when part of every sequence is already in the paged cache (prefix hit, or a later
    chunk of a long prompt): q holds the packed uncached tokens, K and V are read from the cache through
    `block_tables`, which must already contain this step's tokens (store first).  Query i of sequence s sits at
    position (keys_s - queries_s + i) and attends to keys at positions <= its own.

    The reference builds exactly this metadata on a prefix hit (src/myvllm/engine/model_runner.py:198-215) but
    its kernel ignores it and attends to the uncached suffix only (src/myvllm/layers/attention.py:135-137).
    """
    _cabi.require_cuda(q, k_cache, v_cache, cu_seqlens_q, cu_seqlens_k, block_tables)
    total = q.shape[0]
    if tuple(q.shape) != (total, num_heads, head_dim):
        raise ValueError(f"q shape {tuple(q.shape)} is not (tokens, {num_heads}, {head_dim})")
    if k_cache.dim() != 4 or k_cache.shape != v_cache.shape or tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim) \
            or k_cache.dtype != q.dtype or v_cache.dtype != q.dtype or not k_cache.is_contiguous() \
            or not v_cache.is_contiguous():
        raise ValueError("caches must be contiguous (blocks, block_size, kv_heads, head_dim) tensors of q's dtype")
    for t in (cu_seqlens_q, cu_seqlens_k):
        if t.dtype != torch.int32 or t.dim() != 1 or not t.is_contiguous() or t.numel() != cu_seqlens_q.numel():
            raise ValueError("cu_seqlens_q / cu_seqlens_k must be contiguous int32 vectors of equal length")
    num_seqs = cu_seqlens_q.numel() - 1
    if block_tables.dtype != torch.int32 or block_tables.dim() != 2 or block_tables.shape[0] != num_seqs or \
            block_tables.stride(1) != 1:
        raise ValueError("block_tables must be a (num_seqs, max_blocks) int32 tensor with dense rows")
    out = torch.empty((total, num_heads, head_dim), dtype=q.dtype, device=q.device)
    if total == 0 or num_seqs <= 0:
        return out
    rc = _cabi.lib().mv_prefill_paged(
        out.data_ptr(), q.data_ptr(), _row_stride(q, "q"), k_cache.data_ptr(), v_cache.data_ptr(),
        cu_seqlens_q.data_ptr(), cu_seqlens_k.data_ptr(), block_tables.data_ptr(),
        block_tables.stride(0) if num_seqs > 1 else block_tables.shape[1], block_tables.shape[1], k_cache.shape[1],
        k_cache.shape[0], num_seqs, total, num_heads, num_kv_heads, head_dim, float(scale),
        _error_word(q.device).data_ptr(), _cabi.dtype_code(q.dtype), _cabi.stream_ptr())
    _cabi.check(rc)
    return out


def qk_norm_rope_store(qkv, positions, cos_table, sin_table, gamma_q, gamma_k, eps, num_heads, num_kv_heads,
                       head_dim, k_cache=None, v_cache=None, slot_mapping=None, k_scale=None, v_scale=None):
    """One launch for what the reference does in a dozen before attention: RMSNorm of the q and k heads,
    rotary embedding, and the scatter of k and v into the paged cache.

    qkv (tokens, (heads + 2*kv_heads) * head_dim) is the fused projection output (any token stride);
    positions (tokens,) int64; cos_table / sin_table (max_position, head_dim/2) fp32.
    Returns (q, k) as new contiguous (tokens, heads, head_dim) / (tokens, kv_heads, head_dim) tensors; v is
    still `qkv[..., -kv_heads*head_dim:]`.  With caches and a slot_mapping, k and v are also stored; with
    `k_scale` / `v_scale` (fp16, (blocks, block_size, kv_heads)) the caches are int8 and the rows are quantised on
    the way in, exactly as `store_kvcache(k, v, ..., k_scale=, v_scale=)` would.
    Reference: src/myvllm/models/qwen3.py:104-108 and src/myvllm/layers/attention.py:498-510.
    """
    _cabi.require_cuda(qkv, positions, cos_table, sin_table, gamma_q, gamma_k)
    tokens = qkv.shape[0]
    width = (num_heads + 2 * num_kv_heads) * head_dim
    if qkv.dim() != 2 or qkv.shape[1] != width or qkv.stride(1) != 1:
        raise ValueError(f"qkv must be (tokens, {width}) with dense rows")
    if positions.dtype != torch.int64 or positions.numel() != tokens or not positions.is_contiguous():
        raise ValueError("positions must be a contiguous int64 vector with one entry per token")
    for t in (cos_table, sin_table):
        if t.dtype != torch.float32 or t.dim() != 2 or t.shape[1] != head_dim // 2 or not t.is_contiguous():
            raise ValueError("cos/sin tables must be contiguous fp32 (max_position, head_dim/2)")
    q = torch.empty((tokens, num_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    k = torch.empty((tokens, num_kv_heads, head_dim), dtype=qkv.dtype, device=qkv.device)
    store = slot_mapping is not None and k_cache is not None and k_cache.numel() > 0
    quant = k_scale is not None or v_scale is not None
    if quant and (k_scale is None or v_scale is None or not store):
        raise ValueError("k_scale and v_scale must be given together, with caches and a slot_mapping")
    if store:
        want = torch.int8 if quant else qkv.dtype
        if k_cache.dtype != want or v_cache.dtype != want or tuple(k_cache.shape[2:]) != (num_kv_heads, head_dim) or \
                not (k_cache.is_contiguous() and v_cache.is_contiguous()):
            raise ValueError("fused store needs contiguous caches (blocks, block_size, kv_heads, head_dim) of the model "
                             "dtype, or int8 caches together with scales")
        if quant:
            for sc in (k_scale, v_scale):
                if sc.dtype != torch.float16 or tuple(sc.shape) != tuple(k_cache.shape[:3]) or not sc.is_contiguous():
                    raise ValueError("scales must be contiguous fp16 tensors of shape (blocks, block_size, kv_heads)")
        if slot_mapping.dtype != torch.int64 or slot_mapping.numel() != tokens:
            raise ValueError("slot_mapping must be int64 with one entry per token")
    rc = _cabi.lib().mv_qk_norm_rope_store(
        qkv.data_ptr(), qkv.stride(0) if tokens > 1 else width, positions.data_ptr(), cos_table.data_ptr(),
        sin_table.data_ptr(), cos_table.shape[0], gamma_q.data_ptr(), gamma_k.data_ptr(), float(eps), q.data_ptr(),
        k.data_ptr(), k_cache.data_ptr() if store else None, v_cache.data_ptr() if store else None,
        k_scale.data_ptr() if quant else None, v_scale.data_ptr() if quant else None,
        slot_mapping.data_ptr() if store else None, k_cache.shape[0] * k_cache.shape[1] if store else 0, tokens,
        num_heads, num_kv_heads, head_dim, _cabi.dtype_code(qkv.dtype), _cabi.stream_ptr())
    _cabi.check(rc)
    return q, k


class Attention(nn.Module):
    """Attention layer of the engine: stores the step's K/V into the paged cache
    and runs varlen prefill or paged decode, as told by the global Context.

    Same constructor arguments and attributes as the reference module
    (src/myvllm/layers/attention.py:476-557); `k_cache` / `v_cache` start as
    empty tensors and are assigned by the model runner's allocate_kv_cache,
    which finds the modules by these two attribute names.  Optional
    `k_scale` / `v_scale` attributes switch the layer to an int8 cache.
    The cache's own block dimension is used for addressing; `block_size` is
    only a default for callers that read it.
    """

    def __init__(self, num_heads: int, head_dim: int, scale: float = 1.0, num_kv_heads: int = None,
                 block_size: int = 16):
        super().__init__()
        self.num_heads = num_heads
        self.head_dim = head_dim
        self.scale = scale
        self.num_kv_heads = num_kv_heads if num_kv_heads is not None else num_heads
        self.block_size = block_size
        self.k_cache = self.v_cache = torch.tensor([])
        self.k_scale = self.v_scale = None

    def forward(self, q: torch.Tensor, k: torch.Tensor, v: torch.Tensor, store: bool = True) -> torch.Tensor:
        """`store=False` when the caller already wrote this step's K/V into the cache (qk_norm_rope_store)."""
        ctx = get_context()
        k_cache, v_cache = self.k_cache, self.v_cache
        if q.dim() == 4:  # (B, N, heads, head_dim) -> packed tokens; decode passes N == 1
            q = q.reshape(-1, q.shape[-2], q.shape[-1])
            k = k.reshape(-1, k.shape[-2], k.shape[-1])
            v = v.reshape(-1, v.shape[-2], v.shape[-1])
        has_cache = k_cache.numel() > 0 and v_cache.numel() > 0
        if store and has_cache and ctx.slot_mapping is not None:
            store_kvcache(k, v, k_cache, v_cache, ctx.slot_mapping, k_cache.shape[1],
                          k_scale=self.k_scale, v_scale=self.v_scale)
        scale = self.scale / (self.head_dim ** 0.5)
        if ctx.is_prefill:
            if ctx.cu_seqlens_q is None:
                raise ValueError("cu_seqlens_q must be provided for varlen attention")
            if ctx.block_tables is not None and ctx.cu_seqlens_k is not None and has_cache:
                # some sequence has a cached prefix: attend through the paged cache (this step's K/V are in it)
                o = flash_attention_prefill_paged(q, k_cache, v_cache, ctx.cu_seqlens_q, ctx.cu_seqlens_k,
                                                  ctx.block_tables, scale, self.num_heads, self.num_kv_heads,
                                                  self.head_dim)
            else:
                o = flash_attention_prefill(q, k, v, ctx.cu_seqlens_q, scale, self.num_heads, self.num_kv_heads,
                                            self.head_dim)
        else:
            o = paged_attention_decode(q, k_cache, v_cache, ctx.block_tables, ctx.context_lens, scale,
                                       self.num_heads, self.num_kv_heads, self.head_dim, k_cache.shape[1],
                                       k_scale=self.k_scale, v_scale=self.v_scale, workspace=ctx.decode_workspace)
        return o.reshape(o.shape[0], self.num_heads * self.head_dim)
