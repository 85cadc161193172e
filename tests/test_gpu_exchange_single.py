"""The fused cross-rank merge of r2k_decode_exchange on ONE GPU: the test plays the second rank from the host.

Rank 0 is a real launch over the first half of a sequence.  "Rank 1" is the second half decoded to its un-normalised
state rows (r2k_decode with R2K_FLAG_OUT_STATE), which the test writes into rank 0's exchange buffer as
(value, step) words, exactly where a peer's stores over NVLink would put them; rank 1's own exchange buffer is a
local scratch tensor that receives rank 0's rows.  The merged output must equal the all-gather variant
(r2k_merge_states) bit for bit and the single-cache oracle within tolerance.

The same call WITHOUT the peer's rows and with a short wait budget is the failure case: the bounded wait runs out,
the kernel returns, the status word reads R2K_ERR_DEVICE_TIMEOUT, the output is the finite merge of the ranks that
did arrive, and the next step after r2k_decode_workspace_init is correct again.  No wait is unbounded and nothing
faults: the missing rank is simply a buffer nobody writes.
"""
import ctypes as C

import pytest
import torch

import r2omni_b200 as R
from r2omni_b200 import _lib as L
from r2omni_b200.sspa.cache import _stream_ptr
from gpu_helpers import assert_close, build_gpu_cache, make_executor
from oracle import sspa_oracle as O
from recipe import make_inputs

pytestmark = pytest.mark.gpu

HQ, HKV, TOKENS, PAGE = 16, 2, 8192, 64
ROWS = HQ   # batch 1


def _setup():
    r = torch.rand(TOKENS // PAGE, generator=torch.Generator().manual_seed(3))
    classes = torch.where(r < 0.25, 1, torch.where(r < 0.75, 2, 5))
    key, value, _, _, queries = make_inputs(seed=61, hq=HQ, hkv=HKV, tokens=TOKENS, appends=1, n_queries=4)
    half = TOKENS // 2
    shards = []
    for rank in range(2):
        sl = slice(rank * half, (rank + 1) * half)
        cache = build_gpu_cache(key[:, sl].contiguous(), value[:, sl].contiguous(),
                                classes[sl.start // PAGE : sl.stop // PAGE], page_size=PAGE)
        shards.append(make_executor(cache, HQ))
    whole = O.build_cache(key, value, classes, page_size=PAGE)
    first_half = O.build_cache(key[:, :half].contiguous(), value[:, :half].contiguous(), classes[: half // PAGE],
                               page_size=PAGE)
    return shards, whole, first_half, queries


def _exchange(ex0, seq, wait_us=0):
    geom = ex0.arenas.geom(HQ)
    need = C.c_size_t(0)
    L.check(L.lib().r2k_exchange_bytes(C.byref(geom), 2, C.byref(need)), "r2k_exchange_bytes")
    mine = torch.zeros(need.value, device="cuda", dtype=torch.uint8)
    peer = torch.zeros(need.value, device="cuda", dtype=torch.uint8)
    x = L.Exchange()
    x.buffers[0], x.buffers[1] = mine.data_ptr(), peer.data_ptr()
    x.rank, x.world, x.seq, x.wait_us = 0, 2, seq, wait_us
    return x, mine, peer


def _rows_offset(step, rank):
    """First (value, step) word of `rank`'s rows in the half of an exchange buffer that step `step` uses."""
    return (((step & 1) * 2 + rank) * ROWS) * 130


def _deliver(buffer, state, step, rank=1):
    """What a peer's stores leave behind: every float of `state` [1,Hq,130] as a (bits, step) word."""
    words = torch.stack((state.contiguous().view(torch.int32).flatten(),
                         torch.full((ROWS * 130,), step, dtype=torch.int32, device=state.device)), dim=1)
    view = buffer.view(torch.int32).view(-1, 2)
    off = _rows_offset(step, rank)
    view[off : off + ROWS * 130] = words


def _merge_states(states):
    stacked = torch.stack(states).contiguous()
    out = torch.empty(1, HQ, 128, device="cuda", dtype=torch.bfloat16)
    L.check(L.lib().r2k_merge_states(C.c_void_p(stacked.data_ptr()), len(states), C.c_int64(ROWS * 130), ROWS, L.DTYPE_BF16,
                                     C.c_void_p(out.data_ptr()), C.c_uint32(0), C.c_void_p(_stream_ptr(out.device))),
            "r2k_merge_states")
    return out


def test_fused_exchange_with_a_host_played_peer():
    (ex0, ex1), whole, _, queries = _setup()
    x, mine, peer = _exchange(ex0, seq=0)
    out = torch.empty(1, HQ, 128, device="cuda", dtype=torch.bfloat16)
    for step in (1, 2, 3):   # both halves of the buffer, and the first one again with a newer tag
        q = queries[step].cuda()
        state0, state1 = ex0.decode_state(q).clone(), ex1.decode_state(q).clone()
        _deliver(mine, state1, step)
        x.seq = step
        ex0.decode_exchange(q, x, out)
        torch.cuda.synchronize()
        assert ex0.device_status() == 0
        want = _merge_states([state0, state1])
        assert torch.equal(out.view(torch.int16), want.view(torch.int16)), f"step {step}: fused merge differs from the all-gather merge"
        assert_close(out, O.decode(queries[step], whole), f"step {step} against the single-cache oracle")
        # what rank 0 stored into its peer's buffer: its own rows, tagged with the step
        got = peer.view(torch.int32).view(-1, 2)[_rows_offset(step, 0) : _rows_offset(step, 0) + ROWS * 130]
        assert torch.equal(got[:, 1], torch.full_like(got[:, 1], step))
        assert torch.equal(got[:, 0], state0.view(torch.int32).flatten())


def test_device_step_counter_advances_once_per_launch():
    (ex0, ex1), whole, _, queries = _setup()
    x, mine, peer = _exchange(ex0, seq=0)
    counter = mine.view(torch.int32)[(mine.numel() - 128) // 4 :]
    out = torch.empty(1, HQ, 128, device="cuda", dtype=torch.bfloat16)
    for launch in range(3):
        step = int(counter[0]) + 1
        assert step == launch + 1 and int(counter[1]) == 0
        q = queries[launch].cuda()
        _deliver(mine, ex1.decode_state(q).clone(), step)
        ex0.decode_exchange(q, x, out)     # seq = 0: the kernel reads and moves the counter kept in the buffer
        torch.cuda.synchronize()
        assert ex0.device_status() == 0
        assert_close(out, O.decode(queries[launch], whole), f"launch {launch}")


def test_missing_peer_times_out_and_the_next_step_is_clean():
    (ex0, ex1), whole, first_half, queries = _setup()
    x, mine, peer = _exchange(ex0, seq=1, wait_us=1000)
    out = torch.full((1, HQ, 128), float("nan"), device="cuda", dtype=torch.bfloat16)
    q = queries[0].cuda()
    ex0.decode_exchange(q, x, out)          # nobody delivers rank 1's rows
    torch.cuda.synchronize()
    assert ex0.device_status() == L.ERR_DEVICE_TIMEOUT
    assert torch.isfinite(out.float()).all()
    assert_close(out, O.decode(queries[0], first_half), "the ranks that did arrive")
    ws = ex0.workspace.buffer
    L.check(L.lib().r2k_decode_workspace_init(C.c_void_p(ws.data_ptr()), C.c_size_t(ws.numel()),
                                              C.c_void_p(_stream_ptr(ws.device))), "r2k_decode_workspace_init")
    assert ex0.device_status() == 0
    x.seq, x.wait_us = 2, 0
    q = queries[1].cuda()
    _deliver(mine, ex1.decode_state(q).clone(), 2)
    ex0.decode_exchange(q, x, out)
    torch.cuda.synchronize()
    assert ex0.device_status() == 0
    assert_close(out, O.decode(queries[1], whole), "step after the timeout")
    assert_close(ex0(q), O.decode(queries[1], first_half), "plain decode on the same workspace")
