"""Process-global attention metadata: the side channel from the model runner to
the Attention modules, the decoder layers (positions) and the LM head
(last-token selection).

Interface parity with src/myvllm/utils/context.py:5-27 of the reference: a
`Context` whose first eight fields have the reference's names and order, and
`get_context` / `set_context` / `reset_context` that swap the whole object, so
`set_context(True, cu_q, cu_k, max_q, max_k, slots, None, tables)` call sites
work unchanged.  The fields after the first eight are additions of this
package: they carry what the metadata kernels build on the GPU once per step
(the reference rebuilds positions on the host in every layer,
src/myvllm/models/qwen3.py:196-212) and default to None.
"""
from dataclasses import dataclass, fields
from typing import Optional

import torch


@dataclass
class Context:
    # --- the reference's eight fields, same order ---
    is_prefill: bool = False
    cu_seqlens_q: Optional[torch.Tensor] = None
    cu_seqlens_k: Optional[torch.Tensor] = None
    max_seqlen_q: int = 0
    max_seqlen_k: int = 0
    slot_mapping: Optional[torch.Tensor] = None
    context_lens: Optional[torch.Tensor] = None
    block_tables: Optional[torch.Tensor] = None
    # --- additions: built on the device once per step ---
    positions: Optional[torch.Tensor] = None        # (num_tokens,) int64 RoPE positions
    last_token_index: Optional[torch.Tensor] = None  # (num_seqs,) int64 rows fed to the LM head
    decode_workspace: Optional[torch.Tensor] = None  # split-K scratch shared by all layers


class _Holder:
    """Owns the current Context; replaced wholesale, never mutated in place."""

    def __init__(self):
        self.current = Context()


_holder = _Holder()
_FIELD_NAMES = tuple(f.name for f in fields(Context))


def get_context() -> Context:
    return _holder.current


def reset_context() -> None:
    _holder.current = Context()


def set_context(is_prefill, *args, **kwargs) -> None:
    """Positional order after `is_prefill` follows the dataclass fields."""
    if len(args) > len(_FIELD_NAMES) - 1:
        raise TypeError(f"set_context takes at most {len(_FIELD_NAMES)} positional arguments")
    values = dict(zip(_FIELD_NAMES[1:], args))
    for name, value in kwargs.items():
        if name not in _FIELD_NAMES or name in values:
            raise TypeError(f"set_context got an unexpected or duplicate argument '{name}'")
        values[name] = value
    _holder.current = Context(is_prefill=bool(is_prefill), **values)
