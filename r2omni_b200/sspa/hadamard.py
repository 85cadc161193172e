"""128-point Walsh-Hadamard pre-conditioning of key/value rows on the GPU.

Mirrors ``triton_fwht_128`` (r2omni/sspa/kernels/triton_qwen_mrope.py:325-346) and the CPU form
``normalized_fwht`` (r2omni/sspa/runtime/int2_reference.py:18-31): fp32 butterflies over the last axis in stages
of stride 1, 2, ..., 64, scaled by 128**-0.5 and stored in the tensor's own 16-bit type.  The decode launch
applies the same transform to its output when ``output_hadamard`` is set; this entry covers the other side, the
new key/value rows of a decode step when the cache was built with ``key_hadamard`` / ``value_hadamard``.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L
from .cache import _ptr, _stream_ptr, dtype_code


def triton_fwht_128(tensor: torch.Tensor, *, output: torch.Tensor | None = None) -> torch.Tensor:
    """Normalised 128-wide FWHT in one launch; same name, arguments and errors as the reference's entry."""
    if tensor.shape[-1] != 128 or not torch.is_floating_point(tensor):
        raise ValueError("fused FWHT requires a floating tensor with last dimension 128")
    if not tensor.is_cuda:
        raise RuntimeError("fused FWHT requires a CUDA tensor")
    if tensor.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("fused FWHT runs on bf16 / fp16 rows (the cache's element types)")
    tensor = tensor.contiguous()
    if output is None:
        output = torch.empty_like(tensor)
    elif output.shape != tensor.shape or output.device != tensor.device or output.dtype != tensor.dtype:
        raise ValueError("fused FWHT output must match input shape, device, and dtype")
    if not output.is_contiguous():
        raise ValueError("fused FWHT output must be contiguous")
    rows = tensor.numel() // 128
    if rows == 0:
        return output
    L.check(L.lib().r2k_fwht128(_ptr(tensor), _ptr(output), dtype_code(tensor.dtype), C.c_int64(rows),
                                C.c_void_p(_stream_ptr(tensor.device))), "r2k_fwht128")
    return output


normalized_fwht = triton_fwht_128
