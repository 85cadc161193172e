"""The attention manager's decode path on this library's kernels (kernel_backend "cuda_sm100"), driven without model
weights: the attention module is a stand-in object with random projection layers, as the reference's own tests
stand in for models (tests/test_release_core.py of the reference).  Every step of the manager -- project, rotate,
fused append or flush, attend, project out -- is held against the same step composed from the CPU oracle."""
from types import SimpleNamespace

import pytest
import torch

import r2omni_b200 as R
from gpu_helpers import assert_close, build_gpu_cache
from oracle import sspa_oracle as O
from recipe import make_inputs

pytestmark = pytest.mark.gpu

HQ, HKV, HIDDEN, SECTIONS = 16, 2, 256, (16, 24, 24)


def _module(seed):
    g = torch.Generator().manual_seed(seed)
    def linear(n_in, n_out):
        layer = torch.nn.Linear(n_in, n_out, bias=True)
        with torch.no_grad():
            layer.weight.copy_(torch.randn(n_out, n_in, generator=g) * n_in ** -0.5)
            layer.bias.copy_(torch.randn(n_out, generator=g) * 0.1)
        return layer.to(torch.bfloat16)
    return SimpleNamespace(head_dim=128, q_proj=linear(HIDDEN, HQ * 128), k_proj=linear(HIDDEN, HKV * 128),
                           v_proj=linear(HIDDEN, HKV * 128), o_proj=linear(HQ * 128, HIDDEN))


def _to(module, device):
    return SimpleNamespace(head_dim=128, **{n: getattr(module, n).to(device) for n in ("q_proj", "k_proj", "v_proj", "o_proj")})


def _rotary(batch, position, generator):
    angle = torch.rand(3, batch, 1, 128, generator=generator) * 6.2831853 + position
    return torch.cos(angle), torch.sin(angle)


@pytest.mark.parametrize("batch,value_hadamard", [(1, False), (2, False), (2, True)])
def test_manager_decode_steps_match_the_oracle_composition(batch, value_hadamard):
    pages, page = 24, 64
    seq = pages * page
    r = torch.rand(pages, generator=torch.Generator().manual_seed(2))
    classes = torch.where(r < 0.25, 1, torch.where(r < 0.75, 2, 5))
    manager = R.PackedKVAttentionManager(num_query_heads=HQ, mrope_section=SECTIONS, value_hadamard=value_hadamard)
    assert manager.kernel_backend == "cuda_sm100"
    gcaches, ocaches = [], []
    for b in range(batch):
        key, value, _, _, _ = make_inputs(seed=90 + b, hq=HQ, hkv=HKV, tokens=seq, appends=1, n_queries=1)
        if value_hadamard:   # values are rotated before packing; the decode epilogue rotates the output back
            value = O.fwht128(value.float()).to(value.dtype)
        gcaches.append(build_gpu_cache(key, value, classes, page_size=page, append_capacity=256))
        ocaches.append(O.build_cache(key, value, classes, page_size=page, append_capacity=256))
    state = manager.adopt_layer(0, gcaches, seq)
    cpu_module = _module(5)
    gpu_module = _to(cpu_module, "cuda")
    g = torch.Generator().manual_seed(11)
    steps = 131     # through one flush of the 128-token window
    for i in range(steps):
        hidden = torch.randn(batch, 1, HIDDEN, generator=g).to(torch.bfloat16)
        cos, sin = _rotary(batch, float(i), g)
        out = manager.active_forward(0, gpu_module, hidden.cuda(), (cos.cuda(), sin.cuda()), cache_position=seq + i)
        if i % 26 and i not in (127, 128, 129):
            # the oracle cache still has to follow every append
            check = False
        else:
            check = True
        hd = hidden.cuda()   # projections on the GPU (same GEMMs as the manager ran), everything after on the host
        q = gpu_module.q_proj(hd).view(batch, 1, -1, 128).transpose(1, 2).contiguous().cpu()
        k = gpu_module.k_proj(hd).view(batch, 1, -1, 128).transpose(1, 2).contiguous().cpu()
        v = gpu_module.v_proj(hd).view(batch, 1, -1, 128).transpose(1, 2).contiguous().cpu()
        q, k = O.qk_mrope(q, k, cos, sin, SECTIONS, False)
        if value_hadamard:
            v = O.fwht128(v.float()).to(v.dtype)
        rows = []
        for b in range(batch):
            O.append_token(ocaches[b], k[b, :, 0], v[b, :, 0], seq + i, seq + i)
            if check:
                rows.append(O.decode(q[b : b + 1, :, 0], ocaches[b], output_hadamard=value_hadamard))
        if check:
            mixed = torch.cat(rows, 0)      # [B,Hq,128] bf16
            want = gpu_module.o_proj(mixed.reshape(batch, 1, -1).cuda())
            # the attention tolerance, carried through the output projection (rows of unit-variance weights)
            err = (out.float() - want.float()).abs().max().item()
            assert err < 0.05, f"step {i}: {err}"
            if not value_hadamard:
                attn = state.fourq_executor.workspace.output
                assert_close(attn, mixed, f"step {i} attention rows")
    stats = manager.get_stats()[0]
    assert stats["kernel_calls"] == steps and stats["append_count"] == steps
    assert stats["generated_recompress_count"] == 1 and stats["flushed_tokens"] == 128
    assert stats["sequence_length"] == seq + steps and stats["recent_fp_tokens"] == steps - 128
    assert state.fourq_executor.device_status() == 0


@pytest.mark.parametrize("value_hadamard", [False, True])
def test_fused_projection_module_gives_the_same_steps(value_hadamard):
    """A module with one ``qkv_proj`` (weights of the three projections stacked) goes through the one-launch
    prologue; a twin manager with the three projections goes through the reference's sequence of calls.  Same
    attention rows, bit for bit, step after step, through a flush."""
    pages, page, batch = 12, 64, 2
    seq = pages * page
    classes = torch.tensor([1, 2, 5, 2, 2, 1, 5, 2, 1, 2, 5, 2])
    managers = [R.PackedKVAttentionManager(num_query_heads=HQ, mrope_section=SECTIONS, value_hadamard=value_hadamard)
                for _ in range(2)]
    for m in managers:
        caches = []
        for b in range(batch):
            key, value, _, _, _ = make_inputs(seed=60 + b, hq=HQ, hkv=HKV, tokens=seq, appends=1, n_queries=1)
            caches.append(build_gpu_cache(key, value, classes, page_size=page, append_capacity=256))
        m.adopt_layer(0, caches, seq)
    split = _to(_module(7), "cuda")
    qkv = torch.nn.Linear(HIDDEN, (HQ + 2 * HKV) * 128, bias=True, device="cuda", dtype=torch.bfloat16)
    with torch.no_grad():
        qkv.weight.copy_(torch.cat([split.q_proj.weight, split.k_proj.weight, split.v_proj.weight], 0))
        qkv.bias.copy_(torch.cat([split.q_proj.bias, split.k_proj.bias, split.v_proj.bias], 0))
    fused = SimpleNamespace(head_dim=128, qkv_proj=qkv, o_proj=split.o_proj)
    g = torch.Generator().manual_seed(13)
    for i in range(131):
        hidden = torch.randn(batch, 1, HIDDEN, generator=g).to(torch.bfloat16).cuda()
        cos, sin = _rotary(batch, float(i), g)
        a = managers[0].active_forward(0, split, hidden, (cos.cuda(), sin.cuda()), cache_position=seq + i).clone()
        rows_a = managers[0]._states[0].fourq_executor.workspace.output.clone()
        b = managers[1].active_forward(0, fused, hidden, (cos.cuda(), sin.cuda()), cache_position=seq + i)
        rows_b = managers[1]._states[0].fourq_executor.workspace.output
        # one GEMM over the stacked weights and three GEMMs may round differently in the last bit of a projection;
        # the attention tolerance covers what that does to the rows
        assert_close(rows_b, rows_a, f"step {i}")
        assert (a.float() - b.float()).abs().max().item() < 0.05
    assert managers[1].get_stats()[0]["generated_recompress_count"] == 1
    for m in managers:
        assert m._states[0].fourq_executor.device_status() == 0


def test_manager_rejects_what_the_reference_manager_rejects():
    manager = R.PackedKVAttentionManager(num_query_heads=HQ)
    key, value, _, _, _ = make_inputs(seed=95, hq=HQ, hkv=HKV, tokens=512, appends=1, n_queries=1)
    classes = torch.tensor([2, 5, 1, 2, 5, 2, 1, 5])
    manager.adopt_layer(0, build_gpu_cache(key, value, classes, page_size=64), 512)
    module = _to(_module(6), "cuda")
    g = torch.Generator().manual_seed(1)
    cos, sin = _rotary(1, 0.0, g)
    hidden = torch.randn(1, 2, HIDDEN, generator=g).to(torch.bfloat16).cuda()
    with pytest.raises(ValueError):
        manager.active_forward(0, module, hidden, (cos.cuda(), sin.cuda()))              # two tokens per request
    with pytest.raises(ValueError):
        manager.active_forward(0, module, hidden[:, :1], None)                            # no rotary tables
    with pytest.raises(RuntimeError):
        manager.active_forward(0, module, hidden[:, :1], (cos.cuda(), sin.cuda()), cache_position=700)   # not the append position
    with pytest.raises(TypeError):
        manager.adopt_layer(1, object(), 512)
