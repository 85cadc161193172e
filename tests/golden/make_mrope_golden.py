"""Golden vectors of the multimodal-RoPE prologue FROM THE REFERENCE'S OWN KERNEL.

The reference has this step only as a Triton kernel (r2omni/sspa/kernels/triton_qwen_mrope.py:44-212), so the
vectors are made on a CUDA machine that has the reference installed (oracle/install_reference.py):

    python tests/golden/make_mrope_golden.py [/path/to/installed/reference] [output directory]

Seeded inputs (see ``mrope_inputs``), the reference's ``qwen_qk_mrope`` on the GPU, outputs stored as raw 16-bit
patterns in ``mrope_reference.npz`` next to this script (or in the given directory).  The tests load only that file.
"""
from __future__ import annotations

import os
import sys

import numpy as np
import torch

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, HERE)
from recipe import digest  # noqa: E402

CASES = (   # name, batch, hq, hkv, tokens, row dtype, table dtype, hadamard
    ("b8_bf16_tables_bf16", 8, 16, 2, 1, torch.bfloat16, torch.bfloat16, False),
    ("b8_bf16_tables_f32", 8, 16, 2, 1, torch.bfloat16, torch.float32, False),
    ("b8_bf16_tables_f32_hadamard", 8, 16, 2, 1, torch.bfloat16, torch.float32, True),
    ("b2_gqa7_fp16_three_tokens_hadamard", 2, 28, 4, 3, torch.float16, torch.float16, True),
)
SECTIONS = (16, 24, 24)


def mrope_inputs(name, batch, hq, hkv, tokens, dtype, rot_dtype):
    g = torch.Generator().manual_seed(sum(name.encode()))
    q = torch.randn(batch, hq, tokens, 128, generator=g).to(dtype)
    k = torch.randn(batch, hkv, tokens, 128, generator=g).to(dtype)
    angle = torch.rand(3, batch, tokens, 128, generator=g) * 6.2831853
    return q, k, torch.cos(angle).to(rot_dtype), torch.sin(angle).to(rot_dtype)


def main():
    ref = sys.argv[1] if len(sys.argv) > 1 else os.path.join(os.path.dirname(os.path.dirname(HERE)), "baseline", "_ref")
    out_dir = sys.argv[2] if len(sys.argv) > 2 else HERE
    sys.path.insert(0, ref)
    sys.dont_write_bytecode = True
    from r2omni.sspa.kernels.triton_qwen_mrope import qwen_qk_mrope
    out = {}
    for name, batch, hq, hkv, tokens, dtype, rot_dtype, hadamard in CASES:
        q, k, cos, sin = mrope_inputs(name, batch, hq, hkv, tokens, dtype, rot_dtype)
        rq, rk = qwen_qk_mrope(q.cuda(), k.cuda(), cos.cuda(), sin.cuda(), list(SECTIONS), apply_hadamard=hadamard)
        out[name + "_q"] = rq.cpu().contiguous().view(torch.int16).numpy()
        out[name + "_k"] = rk.cpu().contiguous().view(torch.int16).numpy()
        out[name + "_digest"] = np.asarray(digest(q, k, cos.float(), sin.float()))
    path = os.path.join(out_dir, "mrope_reference.npz")
    np.savez_compressed(path, **out)
    print(path, os.path.getsize(path), "bytes")


if __name__ == "__main__":
    main()
