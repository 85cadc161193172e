"""Qwen multimodal RoPE (+ Hadamard) prologue kernel against the oracle's restatement of _qwen_qk_mrope_kernel
(r2omni/sspa/kernels/triton_qwen_mrope.py:44-212), which is itself pinned by outputs of the reference's kernel
(tests/golden/mrope_reference.npz), and against those outputs directly: bit-exact."""
import pytest
import torch

import r2omni_b200 as R
from oracle import sspa_oracle as O

pytestmark = pytest.mark.gpu


def _inputs(batch, hq, hkv, tokens, dtype, rot_dtype, seed):
    g = torch.Generator().manual_seed(seed)
    q = torch.randn(batch, hq, tokens, 128, generator=g).to(dtype)
    k = torch.randn(batch, hkv, tokens, 128, generator=g).to(dtype)
    angle = torch.rand(3, batch, tokens, 128, generator=g) * 6.2831853
    return q, k, torch.cos(angle).to(rot_dtype), torch.sin(angle).to(rot_dtype)


@pytest.mark.parametrize("dtype,rot_dtype", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                             (torch.float16, torch.float16)])
@pytest.mark.parametrize("batch,hq,hkv,tokens", [(1, 16, 2, 1), (8, 16, 2, 1), (2, 28, 4, 3)])
@pytest.mark.parametrize("hadamard", [False, True])
def test_mrope_matches_the_oracle_bit_for_bit(dtype, rot_dtype, batch, hq, hkv, tokens, hadamard):
    q, k, cos, sin = _inputs(batch, hq, hkv, tokens, dtype, rot_dtype, seed=batch * 100 + hq + tokens)
    sections = (16, 24, 24)
    want_q, want_k = O.qk_mrope(q, k, cos, sin, sections, hadamard)
    got_q, got_k = R.qwen_qk_mrope(q.cuda(), k.cuda(), cos.cuda(), sin.cuda(), sections, apply_hadamard=hadamard)
    assert torch.equal(got_q.cpu().view(torch.int16), want_q.view(torch.int16))
    assert torch.equal(got_k.cpu().view(torch.int16), want_k.view(torch.int16))


def test_mrope_strided_tables_in_place_output_and_errors():
    q, k, cos, sin = _inputs(2, 16, 2, 1, torch.bfloat16, torch.float32, seed=9)
    table = torch.zeros(3, 2, 5, 128)          # position tables are usually slices of longer ones
    table_s = torch.zeros(3, 2, 5, 128)
    table[:, :, 3:4] = cos
    table_s[:, :, 3:4] = sin
    want_q, want_k = O.qk_mrope(q, k, cos, sin, (16, 24, 24), True)
    qd, kd = q.cuda(), k.cuda()
    out = R.qwen_qk_mrope(qd, kd, table.cuda()[:, :, 3:4], table_s.cuda()[:, :, 3:4], (16, 24, 24), output=(qd, kd),
                          apply_hadamard=True)
    assert out[0] is qd and out[1] is kd
    assert torch.equal(qd.cpu(), want_q) and torch.equal(kd.cpu(), want_k)
    with pytest.raises(ValueError):
        R.qwen_qk_mrope(qd, kd, cos.cuda(), sin.cuda(), (16, 24, 20))
    with pytest.raises(ValueError):
        R.qwen_qk_mrope(qd[0], kd, cos.cuda(), sin.cuda(), (16, 24, 24))
    with pytest.raises(ValueError):
        R.qwen_qk_mrope(qd, kd, cos.cuda()[:2], sin.cuda()[:2], (16, 24, 24))
    with pytest.raises(RuntimeError):
        R.qwen_qk_mrope(q, k, cos, sin, (16, 24, 24))


def test_mrope_matches_the_reference_kernel_fixture():
    import os

    import numpy as np
    from make_mrope_golden import CASES, SECTIONS, mrope_inputs
    z = np.load(os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "mrope_reference.npz"))
    for name, batch, hq, hkv, tokens, dtype, rot_dtype, hadamard in CASES:
        q, k, cos, sin = mrope_inputs(name, batch, hq, hkv, tokens, dtype, rot_dtype)
        got_q, got_k = R.qwen_qk_mrope(q.cuda(), k.cuda(), cos.cuda(), sin.cuda(), SECTIONS, apply_hadamard=hadamard)
        assert np.array_equal(got_q.cpu().view(torch.int16).numpy(), z[name + "_q"]), name
        assert np.array_equal(got_k.cpu().view(torch.int16).numpy(), z[name + "_k"]), name


@pytest.mark.parametrize("dtype,rot_dtype", [(torch.bfloat16, torch.bfloat16), (torch.bfloat16, torch.float32),
                                             (torch.float16, torch.float16)])
@pytest.mark.parametrize("batch,hq,hkv", [(1, 16, 2), (8, 16, 2), (3, 28, 4), (2, 3, 1)])
@pytest.mark.parametrize("key_hadamard,value_hadamard", [(False, False), (True, False), (False, True), (True, True)])
def test_one_launch_prologue_equals_the_separate_calls(dtype, rot_dtype, batch, hq, hkv, key_hadamard, value_hadamard):
    """Query, key and value rows read in place from one fused projection output (rows 4 elements apart from where a
    contiguous tensor would have them, to make sure the stride is used): the same bits as the rotation call on
    contiguous copies and the Hadamard call on the value rows, and as the oracle."""
    g = torch.Generator().manual_seed(1000 + batch * 37 + hq)
    width = (hq + 2 * hkv) * 128
    fused = torch.randn(batch, 1, width + 4, generator=g).to(dtype).cuda()[..., :width]
    q, k, v = fused[..., : hq * 128], fused[..., hq * 128 : (hq + hkv) * 128], fused[..., (hq + hkv) * 128 :]
    assert not q.is_contiguous() or batch == 1
    _, _, cos, sin = _inputs(batch, hq, hkv, 1, dtype, rot_dtype, seed=batch + hq)
    sections = (16, 24, 24)
    cos, sin = cos.cuda(), sin.cuda()
    got_q, got_k, got_v = R.qwen_qkv_prologue(q, k, v, cos, sin, sections, key_hadamard=key_hadamard,
                                              value_hadamard=value_hadamard)
    qc = q.reshape(batch, 1, hq, 128).transpose(1, 2).contiguous()
    kc = k.reshape(batch, 1, hkv, 128).transpose(1, 2).contiguous()
    vc = v.reshape(batch, 1, hkv, 128).transpose(1, 2).contiguous()
    want_q, want_k = R.qwen_qk_mrope(qc, kc, cos, sin, sections, apply_hadamard=key_hadamard)
    want_v = R.triton_fwht_128(vc) if value_hadamard else vc
    for got, want in ((got_q, want_q), (got_k, want_k), (got_v, want_v)):
        assert got.shape == want.shape and got.is_contiguous()
        assert torch.equal(got.view(torch.int16), want.view(torch.int16))
    oq, ok = O.qk_mrope(qc.cpu(), kc.cpu(), cos.cpu(), sin.cpu(), sections, key_hadamard)
    assert torch.equal(got_q.cpu().view(torch.int16), oq.view(torch.int16))
    assert torch.equal(got_k.cpu().view(torch.int16), ok.view(torch.int16))
    if value_hadamard:
        assert torch.equal(got_v.cpu().view(torch.int16), O.fwht128(vc.cpu().float()).to(dtype).view(torch.int16))


def test_one_launch_prologue_rejects_bad_arguments():
    fused = torch.randn(2, 1, 20 * 128).to(torch.bfloat16).cuda()
    q, k, v = fused[..., :2048], fused[..., 2048:2304], fused[..., 2304:]
    _, _, cos, sin = _inputs(2, 16, 2, 1, torch.bfloat16, torch.float32, seed=4)
    cos, sin = cos.cuda(), sin.cuda()
    R.qwen_qkv_prologue(q, k, v, cos, sin, (16, 24, 24))
    with pytest.raises(ValueError):
        R.qwen_qkv_prologue(q, k, v[..., :128], cos, sin, (16, 24, 24))          # key and value heads differ
    with pytest.raises(ValueError):
        R.qwen_qkv_prologue(q, k, v, cos[:, :1], sin[:, :1], (16, 24, 24))      # tables of another batch
    with pytest.raises(ValueError):
        R.qwen_qkv_prologue(q, k, v, cos, sin, (16, 24, 20))
    with pytest.raises(RuntimeError):
        R.qwen_qkv_prologue(q.cpu(), k.cpu(), v.cpu(), cos.cpu(), sin.cpu(), (16, 24, 24))
