"""SiLU-and-Mul of the Ouro MLP on the B200 kernel.

Host-side mirror of ``vllm_rlt/kernels/activation.py`` and of the native entry
``vllm_rlt::silu_and_mul_cuda`` (``csrc/activation/silu_and_mul.cu:220-247`` of the reference):
same argument meaning, same checks and error types, a new output tensor, launch on the
current stream of the inputs' device, no host synchronisation.
"""

from __future__ import annotations

import torch

from . import _capi

_SCHEMA = "silu_and_mul(Tensor gate, Tensor up) -> Tensor"
_libraries = []  # registrations are dropped when their Library object dies


def _validate_inputs(gate: torch.Tensor, up: torch.Tensor) -> None:
    if gate.shape != up.shape:
        raise ValueError("silu_and_mul expects inputs with the same shape")
    if gate.device != up.device:
        raise ValueError("silu_and_mul expects inputs on the same device")
    if gate.dtype != up.dtype:
        raise TypeError("silu_and_mul expects inputs with the same dtype")
    if gate.dtype not in _capi.DTYPE_CODES:
        raise TypeError("silu_and_mul supports float32, float16 and bfloat16")


def silu_and_mul(gate: torch.Tensor, up: torch.Tensor) -> torch.Tensor:
    """``F.silu(gate) * up`` with the activation rounded to the storage type first."""
    _validate_inputs(gate, up)
    _capi.require_cuda(gate, up)
    if not (gate.is_contiguous() and up.is_contiguous()):
        raise RuntimeError("silu_and_mul requires contiguous inputs")
    if torch.is_grad_enabled() and (gate.requires_grad or up.requires_grad):
        raise RuntimeError("silu_and_mul is inference-only")
    out = torch.empty_like(gate)
    if gate.numel() == 0:
        return out
    with torch.cuda.device(gate.device):
        status = _capi.load().rlt_silu_and_mul(
            _capi.ptr(gate), _capi.ptr(up), _capi.ptr(out), gate.numel(),
            _capi.DTYPE_CODES[gate.dtype], _capi.stream_of(gate))
    _capi.check(status, "silu_and_mul")
    return out


def silu_and_mul_packed(gate_up: torch.Tensor) -> torch.Tensor:
    """``F.silu(gate_up[:, :F]) * gate_up[:, F:]`` for the output ``[rows, 2 * F]`` of one GEMM over the
    concatenated gate and up weights (the two projections of ``OuroMLP``, ``vllm_rlt/models/ouro.py:196-197``,
    share their input).  Same arithmetic and bits as ``silu_and_mul`` on the two halves."""
    _capi.require_cuda(gate_up)
    if gate_up.dim() != 2 or gate_up.shape[1] % 2 or gate_up.stride(1) != 1:
        raise ValueError("silu_and_mul_packed expects [rows, 2 * features] with unit inner stride")
    if gate_up.dtype not in _capi.DTYPE_CODES:
        raise TypeError("silu_and_mul supports float32, float16 and bfloat16")
    if torch.is_grad_enabled() and gate_up.requires_grad:
        raise RuntimeError("silu_and_mul is inference-only")
    rows, cols = gate_up.shape[0], gate_up.shape[1] // 2
    out = torch.empty(rows, cols, dtype=gate_up.dtype, device=gate_up.device)
    if out.numel() == 0:
        return out
    with torch.cuda.device(gate_up.device):
        status = _capi.load().rlt_silu_and_mul_packed(_capi.ptr(gate_up), gate_up.stride(0), _capi.ptr(out), rows, cols,
                                                      _capi.DTYPE_CODES[gate_up.dtype], _capi.stream_of(gate_up))
    _capi.check(status, "silu_and_mul_packed")
    return out


def register_torch_op(namespace: str = "vllm_rlt") -> None:
    """Make ``torch.ops.<namespace>.silu_and_mul`` dispatch CUDA tensors to this kernel.

    This is the registration the reference's ``csrc/torch_bindings.cpp:7-13`` performs for
    its own kernel.  If the schema already exists (the reference's Python module defines it
    when its extension is absent, ``vllm_rlt/kernels/activation.py:33-37``) only the CUDA
    implementation is added; other dispatch keys are left alone.
    """
    _capi.load()
    library = torch.library.Library(namespace, "FRAGMENT")
    try:
        library.define(_SCHEMA)
    except RuntimeError as error:  # already defined by another fragment
        if "already" not in str(error) and "multiple" not in str(error).lower():
            raise
    library.impl("silu_and_mul", silu_and_mul, "CUDA")
    _libraries.append(library)
