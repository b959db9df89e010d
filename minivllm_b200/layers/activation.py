"""SwiGLU activation of the fused gate_up projection in one launch.

Reference: `SiluAndMul.forward` (src/myvllm/layers/activation.py:17-20):
`x, y = x.chunk(2, -1); return F.silu(x) * y`.
"""
import torch

from .. import _cabi


def silu_and_mul(gate_up):
    """gate_up (rows, 2*inter) fp16/bf16 with dense rows -> (rows, inter): silu(first half) * second half."""
    _cabi.require_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.stride(1) != 1 or gate_up.shape[1] % 2:
        raise ValueError("gate_up must be (rows, 2*inter) with dense rows")
    rows, inter = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty((rows, inter), dtype=gate_up.dtype, device=gate_up.device)
    _cabi.check(_cabi.lib().mv_silu_mul(out.data_ptr(), gate_up.data_ptr(), gate_up.stride(0) if rows > 1 else 2 * inter,
                                        rows, inter, _cabi.dtype_code(gate_up.dtype), _cabi.stream_ptr()))
    return out
