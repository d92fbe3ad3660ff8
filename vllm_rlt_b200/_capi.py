"""ctypes binding of ``librlt_verify.so`` (declared in ``include/rlt_verify.h``).

There is no CPU or PyTorch fallback behind this module: if the CUDA library has not been
built, or a call fails, the caller gets an exception.
"""

from __future__ import annotations

import ctypes
from ctypes import c_char_p, c_float, c_int, c_int64, c_size_t, c_void_p
from pathlib import Path

import torch

LIBRARY = Path(__file__).resolve().parent / "librlt_verify.so"

OK, ERR_INVALID, ERR_UNSUPPORTED, ERR_CUDA, ERR_WORKSPACE = 0, -1, -2, -3, -4
ROW_OK, ROW_ZERO_PROPOSAL, ROW_INVALID_RESIDUAL, ROW_BAD_LOGITS, ROW_SHARED_PAGE, ROW_BAD_POSITION = range(6)

DTYPE_CODES = {torch.float32: 0, torch.float16: 1, torch.bfloat16: 2}

# name -> (restype, argtypes); mirrors include/rlt_verify.h one to one.
_P, _I, _L, _Z, _F = c_void_p, c_int, c_int64, c_size_t, c_float
SIGNATURES = {
    "rlt_version": (c_char_p, []),
    "rlt_last_error": (c_char_p, []),
    "rlt_silu_and_mul": (_I, [_P, _P, _P, _L, _I, _P]),
    "rlt_silu_and_mul_packed": (_I, [_P, _L, _P, _L, _L, _I, _P]),
    "rlt_kv_write": (_I, [_P, _P, _L, _L, _L, _I, _I, _I, _I, _P, _P, _P, _P, _P, _P, _I, _P]),
    "rlt_verify_attention_workspace_bytes": (_Z, [_I, _I, _I, _I, _I, _I]),
    "rlt_verify_attention": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _I,
                                  _P, _Z, _P]),
    "rlt_verify_attention_plan": (_I, [_P, _I, _I, _P, _P, _I, _I, _I, _I, _I, _I, _P, _Z, _P]),
    "rlt_verify_attention_run": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _I,
                                      _P, _Z, _P]),
    "rlt_verify_attention_noalloc": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _I, _P]),
    "rlt_windowed_attention": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _P, _I, _I, _P]),
    "rlt_prefill_attention_workspace_bytes": (_Z, [_I, _I, _I, _I, _I, _I, _I]),
    "rlt_prefill_attention": (_I, [_P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _I,
                                   _P, _Z, _P]),
    "rlt_verify_attention_status": (_I, [_P, _P, _P]),
    "rlt_argmax_rows": (_I, [_P, _L, _I, _I, _I, _P, _P]),
    "rlt_accept_greedy": (_I, [_P, _L, _I, _I, _I, _P, _I, _P, _P, _I, _P, _P, _P, _P, _P]),
    "rlt_round_uniforms": (_I, [_P, _P, _I, _I, _P, _P, _P, _P]),
    "rlt_probabilities": (_I, [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P]),
    "rlt_sample_rows": (_I, [_P, _L, _I, _I, _I, _P, _P, _P, _P, _P, _P, _P]),
    "rlt_accept_rejection_workspace_bytes": (_Z, [_I]),
    "rlt_accept_rejection": (_I, [_P, _P, _L, _I, _I, _I, _P, _I, _P, _P, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P,
                                  _P, _P, _Z, _P]),
    "rlt_finalize_tokens": (_I, [_P, _P, _L, _L, _L, _L, _I, _I, _I, _I, _I, _P, _I, _I, _P, _P, _P, _I, _P]),
    "rlt_pipeline_shift": (_I, [_P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P, _P]),
    "rlt_rope_kv_write": (_I, [_P, _L, _P, _L, _P, _L, _P, _P, _P, _P, _P, _L, _L, _L, _I, _I, _I, _I, _I, _P, _P, _P, _P,
                               _I, _P]),
    "rlt_sandwich_norm": (_I, [_P, _P, _P, _P, _P, _P, _I, _I, _F, _I, _P]),
    "rlt_rollback": (_I, [_P, _P, _I, _P, _I, _I, _I, _P, _P, _L, _P, _I, _P, _P, _P, _P, _P, _P]),
}

_lib = None


class NativeLibraryMissing(RuntimeError):
    pass


def load() -> ctypes.CDLL:
    """Load the CUDA library once; raise if it has not been built."""
    global _lib
    if _lib is None:
        if not LIBRARY.exists():
            raise NativeLibraryMissing(
                f"{LIBRARY.name} is not built: run `python -m vllm_rlt_b200.build` "
                "(needs nvcc with sm_100a support). There is no fallback implementation."
            )
        lib = ctypes.CDLL(str(LIBRARY))
        for name, (restype, argtypes) in SIGNATURES.items():
            fn = getattr(lib, name)
            fn.restype = restype
            fn.argtypes = argtypes
        _lib = lib
    return _lib


def last_error() -> str:
    return load().rlt_last_error().decode()


def check(status: int, what: str) -> None:
    """Translate a C-ABI status into the exception the reference interface raises."""
    if status == OK:
        return
    detail = last_error()
    if status == ERR_INVALID:
        raise ValueError(f"{what}: {detail}")
    if status == ERR_UNSUPPORTED:
        raise NotImplementedError(f"{what}: {detail}")
    raise RuntimeError(f"{what}: status {status}: {detail}")


def ptr(tensor) -> c_void_p:
    return c_void_p(0 if tensor is None else tensor.data_ptr())


def stream_of(tensor) -> c_void_p:
    return c_void_p(torch.cuda.current_stream(tensor.device).cuda_stream)


def require_cuda(*tensors) -> torch.device:
    device = None
    for t in tensors:
        if t is None:
            continue
        if t.device.type != "cuda":
            raise ValueError("the B200 verify-step kernels require CUDA tensors")
        if device is None:
            device = t.device
        elif t.device != device:
            raise ValueError("all tensors of one call must live on the same device")
    return device
