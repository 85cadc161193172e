"""128-point Walsh-Hadamard pre-conditioning of key/value rows on the GPU.

Mirrors ``triton_fwht_128`` (r2omni/sspa/kernels/triton_qwen_mrope.py:325-346) and the CPU form
``normalized_fwht`` (r2omni/sspa/runtime/int2_reference.py:18-31): fp32 butterflies over the last axis in stages
of stride 1, 2, ..., 64, scaled by 128**-0.5 and stored in the tensor's own 16-bit type.  The decode launch
applies the same transform to its output when ``output_hadamard`` is set; this entry covers the other side, the
new key/value rows of a decode step when the cache was built with ``key_hadamard`` / ``value_hadamard``.
``qwen_qkv_prologue`` does the rotation of the query and key rows and the hand-over of the value rows of a decode
step in one launch, reading the three straight out of a fused projection.
"""
from __future__ import annotations

import ctypes as C

import torch

from .. import _lib as L
from .cache import _ptr, _stream_ptr, dtype_code


def _require(ok: bool, message: str, error=ValueError) -> None:
    if not ok:
        raise error(message)


_ROW_TYPES = (torch.bfloat16, torch.float16)


def triton_fwht_128(tensor: torch.Tensor, *, output: torch.Tensor | None = None) -> torch.Tensor:
    """Normalised 128-wide FWHT in one launch; same name, arguments and errors as the reference's entry."""
    _require(tensor.shape[-1] == 128 and torch.is_floating_point(tensor),
             "fused FWHT requires a floating tensor with last dimension 128")
    _require(tensor.is_cuda, "fused FWHT requires a CUDA tensor", RuntimeError)
    _require(tensor.dtype in _ROW_TYPES, "fused FWHT runs on bf16 / fp16 rows (the cache's element types)")
    tensor = tensor.contiguous()
    if output is None:
        output = torch.empty_like(tensor)
    else:
        same = (output.shape, output.device, output.dtype) == (tensor.shape, tensor.device, tensor.dtype)
        _require(same, "fused FWHT output must match input shape, device, and dtype")
        _require(output.is_contiguous(), "fused FWHT output must be contiguous")
    rows = tensor.numel() // 128
    if rows:
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
    _require(query.ndim == 4 and key.ndim == 4, "Qwen fused mRoPE requires rank-4 Q/K")
    batch, heads_q, tokens, width = (int(n) for n in query.shape)
    _require(key.shape[0] == batch, "Qwen fused mRoPE requires equal Q/K batch sizes")
    _require(tokens > 0 and key.shape[2] == tokens, "Qwen fused mRoPE requires equal positive Q/K token counts")
    _require(width == 128 and key.shape[-1] == 128, "Qwen fused mRoPE currently requires head_dim=128")
    _require((query.device, query.dtype) == (key.device, key.dtype), "Q/K device and dtype must match")
    _require(cos.device == query.device and sin.device == query.device,
             "Q/K and rotary tensors must share a device")
    _require(cos.ndim == 4 and cos.shape == sin.shape and cos.shape[0] == 3,
             "Qwen fused mRoPE requires cos/sin [3,B,S,D]")
    _require(tuple(cos.shape[1:]) == (batch, tokens, 128), "Qwen fused mRoPE rotary positions must match Q/K tokens")
    sections = tuple(int(v) for v in mrope_section)
    _require(len(sections) == 3 and sum(sections) == 64,
             "Qwen mRoPE sections must contain three values summing to 64")
    _require(query.is_cuda, "fused Qwen mRoPE requires CUDA tensors", RuntimeError)
    _require(query.dtype in _ROW_TYPES, "fused Qwen mRoPE runs on bf16 / fp16 rows")
    _require(cos.dtype == sin.dtype and cos.dtype in _ROW_TYPES + (torch.float32,),
             "rotary tables must share one of bf16 / fp16 / fp32")
    query, key = query.contiguous(), key.contiguous()
    if output is None:
        outs = (torch.empty_like(query), torch.empty_like(key))
    else:
        outs = tuple(output)
        for out, src in zip(outs, (query, key)):
            _require(out.shape == src.shape, "fused Qwen mRoPE output shapes must match Q/K")
        for out, src in zip(outs, (query, key)):
            _require((out.device, out.dtype) == (src.device, src.dtype),
                     "fused Qwen mRoPE outputs must match Q/K device and dtype")
        _require(all(out.is_contiguous() for out in outs), "fused Qwen mRoPE outputs must be contiguous")
    rot = 2 if cos.dtype == torch.float32 else dtype_code(cos.dtype)
    strides = [(C.c_int64 * 4)(*(int(n) for n in t.stride())) for t in (cos, sin)]
    L.check(L.lib().r2k_qk_mrope(
        _ptr(query), _ptr(key), _ptr(outs[0]), _ptr(outs[1]), dtype_code(query.dtype), batch, heads_q,
        int(key.shape[1]), tokens, _ptr(cos), _ptr(sin), rot, strides[0], strides[1], sections[0], sections[1],
        int(bool(apply_hadamard)), C.c_void_p(_stream_ptr(query.device))), "r2k_qk_mrope")
    return outs


def qwen_qkv_prologue(query: torch.Tensor, key: torch.Tensor, value: torch.Tensor, cos: torch.Tensor, sin: torch.Tensor,
                      mrope_section, *, key_hadamard: bool = False, value_hadamard: bool = False, output=None):
    """Everything between the projections and the decode launch of one step, in one launch: ``qwen_qk_mrope`` on
    the query and key rows (Hadamard when ``key_hadamard``) and the value rows brought along (``triton_fwht_128``
    when ``value_hadamard``), bit for bit what those calls give (r2omni/sspa/integration/qwen_sspa_attention.py:
    1216-1249 and the value rotation of :1780).

    ``query`` is ``[B,Hq,128]`` or ``[B,1,Hq*128]``-like, ``key`` / ``value`` ``[B,Hkv,128]``-like: any views whose
    last ``heads*128`` elements are contiguous per request -- slices of one fused projection output qualify, no copy
    is made.  Returns contiguous ``(q [B,Hq,1,128], k [B,Hkv,1,128], v [B,Hkv,1,128])``."""
    batch = int(query.shape[0])

    def rows(t: torch.Tensor, what: str):
        _require(t.is_cuda, "fused Qwen prologue requires CUDA tensors", RuntimeError)
        _require(t.shape[0] == batch and t.numel() % (batch * 128) == 0, f"{what} rows do not match the batch")
        heads = t.numel() // (batch * 128)
        flat = t.reshape(batch, heads * 128)      # a view wherever one exists (a slice of a fused projection is one)
        if flat.stride(1) != 1 or flat.stride(0) % 4 or flat.data_ptr() % 8:
            flat = flat.contiguous()
        return flat, heads

    q2, heads_q = rows(query, "query")
    k2, heads_kv = rows(key, "key")
    v2, heads_v = rows(value, "value")
    _require(heads_v == heads_kv, "key and value rows must have the same number of heads")
    _require(q2.dtype in _ROW_TYPES and k2.dtype == q2.dtype and v2.dtype == q2.dtype, "fused Qwen prologue runs on bf16 / fp16 rows")
    _require(cos.ndim == 4 and cos.shape == sin.shape and cos.shape[0] == 3 and tuple(cos.shape[1:]) == (batch, 1, 128),
             "Qwen fused prologue requires cos/sin [3,B,1,128]")
    _require(cos.device == q2.device and sin.device == q2.device, "Q/K and rotary tensors must share a device")
    _require(cos.dtype == sin.dtype and cos.dtype in _ROW_TYPES + (torch.float32,),
             "rotary tables must share one of bf16 / fp16 / fp32")
    sections = tuple(int(n) for n in mrope_section)
    _require(len(sections) == 3 and sum(sections) == 64, "Qwen mRoPE sections must contain three values summing to 64")
    if output is None:
        output = (torch.empty(batch, heads_q, 1, 128, device=q2.device, dtype=q2.dtype),
                  torch.empty(batch, heads_kv, 1, 128, device=q2.device, dtype=q2.dtype),
                  torch.empty(batch, heads_kv, 1, 128, device=q2.device, dtype=q2.dtype))
    else:
        wanted = ((batch, heads_q, 1, 128), (batch, heads_kv, 1, 128), (batch, heads_kv, 1, 128))
        for out, shape in zip(output, wanted):
            _require(tuple(out.shape) == shape and out.dtype == q2.dtype and out.device == q2.device and out.is_contiguous(),
                     "fused Qwen prologue outputs must be contiguous [B,H,1,128] of the input type")
    rot = 2 if cos.dtype == torch.float32 else dtype_code(cos.dtype)
    strides = [(C.c_int64 * 4)(*(int(n) for n in t.stride())) for t in (cos, sin)]
    L.check(L.lib().r2k_qkv_prologue(
        _ptr(q2), C.c_int64(q2.stride(0)), _ptr(k2), C.c_int64(k2.stride(0)), _ptr(v2), C.c_int64(v2.stride(0)),
        _ptr(output[0]), _ptr(output[1]), _ptr(output[2]), dtype_code(q2.dtype), batch, heads_q, heads_kv,
        _ptr(cos), _ptr(sin), rot, strides[0], strides[1], sections[0], sections[1], int(bool(key_hadamard)),
        int(bool(value_hadamard)), C.c_void_p(_stream_ptr(q2.device))), "r2k_qkv_prologue")
    return tuple(output)
