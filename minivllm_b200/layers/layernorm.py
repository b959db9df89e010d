"""RMSNorm with the residual add fused in, one launch of hand-written CUDA.

The reference's `LayerNorm.forward(x, residual)` (src/myvllm/layers/layernorm.py
:10-28) adds the residual, keeps the sum as the new residual and normalises it;
`add_rms_norm` does the same through `mv_add_rmsnorm`.  Under tensor parallelism
the same step is fused with the all-reduce that precedes it
(layers/allreduce.py), and the residual stream is then kept sharded by rows:
`residual_rows=(lo, hi)` stores the new residual only for the rows this rank owns.
"""
import torch

from .. import _cabi


def add_rms_norm(x, residual, gamma, eps, residual_out=None, residual_rows=None, out=None):
    """x (rows, hidden) fp16/bf16 contiguous.  s = x + residual (or x when residual is None);
    returns rms_norm(s) * gamma as a new tensor (or into `out`).  With `residual_out`, s is stored to
    residual_out[row - lo] for rows lo <= row < hi (`residual_rows`, default all rows); `residual_out` may be
    `residual` itself when lo == 0 (in-place update of the residual stream)."""
    _cabi.require_cuda(x, residual, gamma, residual_out, out)
    if x.dim() != 2 or not x.is_contiguous():
        raise ValueError("x must be a contiguous (rows, hidden) tensor")
    rows, hidden = x.shape
    if residual is not None and (residual.shape != x.shape or not residual.is_contiguous() or residual.dtype != x.dtype):
        raise ValueError("residual must match x in shape and dtype")
    if gamma.numel() != hidden or gamma.dtype != x.dtype or not gamma.is_contiguous():
        raise ValueError("gamma must be a contiguous (hidden,) tensor of x's dtype")
    lo, hi = (0, rows) if residual_rows is None else residual_rows
    if residual_out is not None:
        if residual_out.dtype != x.dtype or not residual_out.is_contiguous() or residual_out.dim() != 2 or \
                residual_out.shape[1] != hidden or residual_out.shape[0] < hi - lo:
            raise ValueError("residual_out must be a contiguous (>= hi-lo, hidden) tensor of x's dtype")
    if out is None:
        out = torch.empty_like(x)
    elif out.shape != x.shape or out.dtype != x.dtype or not out.is_contiguous():
        raise ValueError("out must match x")
    _cabi.check(_cabi.lib().mv_add_rmsnorm(
        out.data_ptr(), x.data_ptr(), residual.data_ptr() if residual is not None else None,
        residual_out.data_ptr() if residual_out is not None else None, lo, hi, gamma.data_ptr(), float(eps), rows,
        hidden, _cabi.dtype_code(x.dtype), _cabi.stream_ptr()))
    return out
