"""The C-ABI library loads without a GPU and exports exactly what the header declares."""
import ctypes
import os
import re

import pytest

from minivllm_b200 import _cabi

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))


def _declared():
    text = open(os.path.join(ROOT, "include", "minivllm_b200.h")).read()
    text = re.sub(r"/\*.*?\*/", "", text, flags=re.S)
    return sorted(set(re.findall(r"\b(mv_[a-z0-9_]+)\s*\(", text)))


def test_library_exports_every_declared_symbol():
    names = _declared()
    assert "mv_store_kvcache" in names and "mv_paged_decode" in names
    handle = ctypes.CDLL(_cabi.LIB_PATH)
    for n in names:
        assert hasattr(handle, n), f"{n} is declared in the header but not exported"


def test_binding_table_matches_header():
    assert sorted(_cabi.SIGNATURES) == _declared()


def test_abi_version_and_error_string():
    lib = _cabi.lib()
    assert lib.mv_abi_version() >= 1
    assert isinstance(lib.mv_last_error_string(), bytes)


def test_argument_validation_needs_no_gpu():
    """Bad arguments are rejected before any launch, so these calls are safe on a CPU-only host."""
    lib = _cabi.lib()
    # odd head_dim
    rc = lib.mv_store_kvcache(16, 16, 8, 8, 16, 16, None, None, 16, 4, 64, 1, 7, 0, None)
    assert rc == 3 and b"head_dim" in lib.mv_last_error_string()
    # null pointers
    rc = lib.mv_store_kvcache(None, None, 64, 64, None, None, None, None, None, 4, 64, 1, 64, 0, None)
    assert rc == 1
    # misaligned pointer
    rc = lib.mv_store_kvcache(8, 16, 64, 64, 16, 16, None, None, 16, 4, 64, 1, 64, 0, None)
    assert rc == 2
    # bad dtype
    rc = lib.mv_store_kvcache(16, 16, 64, 64, 16, 16, None, None, 16, 4, 64, 1, 64, 9, None)
    assert rc == 5
    # heads not divisible
    assert lib.mv_paged_decode_workspace_bytes(4, 6, 4, 128, 4, 256) == -1
    need = lib.mv_paged_decode_workspace_bytes(16, 16, 8, 128, 4, 256)
    assert need > 0
    rc = lib.mv_paged_decode(16, 16, 16, 16, None, None, 16, 4, 4, 16, 1, 16, 16, 8, 128, 256, 41, 0.1, 16, need - 1,
                             0, None)
    assert rc == 4 and b"workspace" in lib.mv_last_error_string()
    rc = lib.mv_paged_decode(16, 16, 16, 16, None, None, 16, 4, 4, 16, 1, 16, 16, 8, 96, 256, 41, 0.1, 16, need, 0,
                             None)
    assert rc == 3


def test_operators_refuse_cpu_tensors():
    import torch
    from minivllm_b200.layers import attention as A
    k = torch.zeros(2, 1, 64, dtype=torch.float16)
    c = torch.zeros(1, 16, 1, 64, dtype=torch.float16)
    with pytest.raises(RuntimeError, match="no CPU path"):
        A.store_kvcache(k, k, c, c, torch.zeros(2, dtype=torch.int64), 16)
