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


def qwen_qk_mrope(query: torch.Tensor, key: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor, mrope_section, *,
                  output=None, apply_hadamard: bool = False):
    """Qwen multimodal RoPE (and optionally the 128-point Hadamard) on the query and key rows of a step in one
    launch.  Same name, arguments and errors as the reference's entry
    (r2omni/sspa/kernels/triton_qwen_mrope.py:214-322): q ``[B,Hq,T,128]``, k ``[B,Hkv,T,128]``, cos / sin
    ``[3,B,T,128]`` (any strides; bf16, fp16 or fp32), three sections summing to 64."""
    if query.ndim != 4 or key.ndim != 4:
        raise ValueError("Qwen fused mRoPE requires rank-4 Q/K")
    if query.shape[0] != key.shape[0]:
        raise ValueError("Qwen fused mRoPE requires equal Q/K batch sizes")
    if query.shape[2] <= 0 or key.shape[2] != query.shape[2]:
        raise ValueError("Qwen fused mRoPE requires equal positive Q/K token counts")
    if query.shape[-1] != 128 or key.shape[-1] != 128:
        raise ValueError("Qwen fused mRoPE currently requires head_dim=128")
    if query.device != key.device or query.dtype != key.dtype:
        raise ValueError("Q/K device and dtype must match")
    if cos.device != query.device or sin.device != query.device:
        raise ValueError("Q/K and rotary tensors must share a device")
    if cos.shape != sin.shape or cos.ndim != 4 or cos.shape[0] != 3:
        raise ValueError("Qwen fused mRoPE requires cos/sin [3,B,S,D]")
    tokens, batch = int(query.shape[2]), int(query.shape[0])
    if cos.shape[1] != batch or tuple(cos.shape[-2:]) != (tokens, 128):
        raise ValueError("Qwen fused mRoPE rotary positions must match Q/K tokens")
    sections = tuple(int(v) for v in mrope_section)
    if len(sections) != 3 or sum(sections) != 64:
        raise ValueError("Qwen mRoPE sections must contain three values summing to 64")
    if not query.is_cuda:
        raise RuntimeError("fused Qwen mRoPE requires CUDA tensors")
    if query.dtype not in (torch.bfloat16, torch.float16):
        raise ValueError("fused Qwen mRoPE runs on bf16 / fp16 rows")
    if cos.dtype != sin.dtype or cos.dtype not in (torch.bfloat16, torch.float16, torch.float32):
        raise ValueError("rotary tables must share one of bf16 / fp16 / fp32")
    query, key = query.contiguous(), key.contiguous()
    if output is None:
        query_out, key_out = torch.empty_like(query), torch.empty_like(key)
    else:
        query_out, key_out = output
        if query_out.shape != query.shape or key_out.shape != key.shape:
            raise ValueError("fused Qwen mRoPE output shapes must match Q/K")
        if (query_out.device != query.device or key_out.device != key.device or query_out.dtype != query.dtype
                or key_out.dtype != key.dtype):
            raise ValueError("fused Qwen mRoPE outputs must match Q/K device and dtype")
        if not query_out.is_contiguous() or not key_out.is_contiguous():
            raise ValueError("fused Qwen mRoPE outputs must be contiguous")
    rot = 2 if cos.dtype == torch.float32 else dtype_code(cos.dtype)
    cs = (C.c_int64 * 4)(*[int(s) for s in cos.stride()])
    ss = (C.c_int64 * 4)(*[int(s) for s in sin.stride()])
    L.check(L.lib().r2k_qk_mrope(
        _ptr(query), _ptr(key), _ptr(query_out), _ptr(key_out), dtype_code(query.dtype), batch, int(query.shape[1]),
        int(key.shape[1]), tokens, _ptr(cos), _ptr(sin), rot, cs, ss, sections[0], sections[1], int(bool(apply_hadamard)),
        C.c_void_p(_stream_ptr(query.device))), "r2k_qk_mrope")
    return query_out, key_out
