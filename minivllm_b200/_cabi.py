"""ctypes binding of libminivllm_b200.so, the C-ABI library declared in
include/minivllm_b200.h.

The library is the only compute path of this package: if it has not been built
(`python -m minivllm_b200.csrc.build`) importing an operator raises, there is
no PyTorch or CPU fallback.
"""
import ctypes
import os

import torch

_HERE = os.path.dirname(os.path.abspath(__file__))
LIB_PATH = os.path.join(_HERE, "csrc", "libminivllm_b200.so")

MV_F16, MV_BF16 = 0, 1

_c_i64 = ctypes.c_int64
_c_int = ctypes.c_int
_c_ptr = ctypes.c_void_p
_c_f32 = ctypes.c_float

# name -> (restype, argtypes); must list every symbol of include/minivllm_b200.h
SIGNATURES = {
    "mv_last_error_string": (ctypes.c_char_p, []),
    "mv_abi_version": (_c_int, []),
    "mv_store_kvcache": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr,
                                  _c_i64, _c_i64, _c_int, _c_int, _c_int, _c_ptr]),
    "mv_paged_decode_workspace_bytes": (_c_i64, [_c_int, _c_int, _c_int, _c_int, _c_int, _c_int]),
    "mv_paged_decode": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int,
                                 _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_i64, _c_f32,
                                 _c_ptr, _c_i64, _c_int, _c_ptr]),
    "mv_paged_decode_static_capacity": (_c_i64, []),
    "mv_paged_decode_static": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int,
                                        _c_ptr, _c_int, _c_int, _c_int, _c_int, _c_int, _c_int, _c_i64, _c_f32,
                                        _c_int, _c_ptr]),
    "mv_prefill_varlen": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_i64, _c_ptr, _c_int, _c_i64,
                                   _c_int, _c_int, _c_int, _c_f32, _c_ptr, _c_int, _c_ptr]),
    "mv_prefill_paged": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_int, _c_int,
                                  _c_i64, _c_int, _c_i64, _c_int, _c_int, _c_int, _c_f32, _c_ptr, _c_int, _c_ptr]),
    "mv_build_decode_meta": (_c_int, [_c_ptr, _c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_int, _c_ptr, _c_ptr,
                                      _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_ptr]),
    "mv_build_prefill_meta": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_int, _c_i64, _c_ptr, _c_i64, _c_int, _c_int,
                                       _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr]),
    "mv_update_block_tables": (_c_int, [_c_ptr, _c_int, _c_ptr, _c_i64, _c_int, _c_int, _c_ptr]),
    "mv_qk_norm_rope_store": (_c_int, [_c_ptr, _c_i64, _c_ptr, _c_ptr, _c_ptr, _c_int, _c_ptr, _c_ptr, _c_f32,
                                       _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_int,
                                       _c_int, _c_int, _c_int, _c_ptr]),
    "mv_argmax_rows": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, _c_ptr, _c_int, _c_ptr]),
    "mv_argmax_decode": (_c_int, [_c_ptr, _c_int, _c_i64, _c_ptr, _c_ptr]),
    "mv_sample_rows": (_c_int, [_c_ptr, _c_i64, _c_i64, _c_i64, _c_i64, _c_ptr, ctypes.c_uint64, _c_ptr, _c_ptr, _c_ptr,
                                _c_int, _c_ptr]),
    "mv_philox4x32_10": (_c_int, [ctypes.c_uint64, ctypes.c_uint64, ctypes.c_uint32, ctypes.c_uint32, _c_ptr]),
    "mv_comm_handle_bytes": (_c_i64, []),
    "mv_comm_create": (_c_int, [_c_int, _c_int, _c_i64, _c_int, ctypes.POINTER(_c_ptr), _c_ptr]),
    "mv_comm_connect": (_c_int, [_c_ptr, _c_ptr]),
    "mv_comm_create_emulated": (_c_int, [_c_int, _c_i64, _c_int, ctypes.POINTER(_c_ptr)]),
    "mv_comm_destroy": (_c_int, [_c_ptr]),
    "mv_comm_reset": (_c_int, [_c_ptr]),
    "mv_comm_set_max_blocks": (_c_int, [_c_ptr, _c_int]),
    "mv_comm_input": (_c_ptr, [_c_ptr, _c_int]),
    "mv_comm_output": (_c_ptr, [_c_ptr, _c_int]),
    "mv_allreduce_residual_rmsnorm": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_ptr, _c_f32, _c_int, _c_int, _c_ptr,
                                               _c_int, _c_ptr]),
    "mv_allreduce_residual_rmsnorm_staged": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_ptr, _c_f32, _c_int, _c_int, _c_ptr,
                                               _c_int, _c_ptr]),
    "mv_add_rmsnorm": (_c_int, [_c_ptr, _c_ptr, _c_ptr, _c_ptr, _c_i64, _c_i64, _c_ptr, _c_f32, _c_i64, _c_int,
                                _c_int, _c_ptr]),
    "mv_silu_mul": (_c_int, [_c_ptr, _c_ptr, _c_i64, _c_i64, _c_int, _c_int, _c_ptr]),
}

_lib = None


def lib():
    """Loads the shared library once; raises if it is missing."""
    global _lib
    if _lib is None:
        if not os.path.exists(LIB_PATH):
            raise RuntimeError(
                f"{LIB_PATH} is missing: build it with `python -m minivllm_b200.csrc.build` "
                "(this package has no fallback path)")
        handle = ctypes.CDLL(LIB_PATH)
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(handle, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = handle
    return _lib


def check(status, exc=RuntimeError):
    """Turns a non-zero mv_status into a Python exception carrying the library's message."""
    if status != 0:
        msg = lib().mv_last_error_string().decode()
        # shape / dtype / null problems are argument errors, as in the reference's asserts
        if status in (1, 2, 3, 5, 7):
            raise ValueError(f"minivllm_b200 status {status}: {msg}")
        raise exc(f"minivllm_b200 status {status}: {msg}")


def dtype_code(dt):
    if dt == torch.float16:
        return MV_F16
    if dt == torch.bfloat16:
        return MV_BF16
    raise ValueError(f"minivllm_b200 kernels take float16 or bfloat16 tensors, got {dt}")


def stream_ptr():
    return torch.cuda.current_stream().cuda_stream


def require_cuda(*tensors):
    for t in tensors:
        if t is not None and not t.is_cuda:
            raise RuntimeError("minivllm_b200 operators run on CUDA tensors only (no CPU path)")
