"""The sequence-sharded protocol on CPU ranks (gloo, world_size 2 and 3): contiguous page-aligned shards,
residual window on the last rank, one all-gather of (max, sum-exp, out) states, exact merge on every rank.
The per-rank attention here is the oracle; the CUDA path of the same protocol runs in the GPU tests."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

import r2omni_b200 as R
from oracle import sspa_oracle as O
from recipe import make_inputs


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, tokens, results):
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world)
    try:
        torch.set_num_threads(1)
        page = 64
        r = torch.rand(tokens // page, generator=torch.Generator().manual_seed(3))
        classes = torch.where(r < 0.25, 1, torch.where(r < 0.75, 2, 5))
        key, value, new_k, new_v, queries = make_inputs(seed=60, hq=16, hkv=2, tokens=tokens, appends=5, n_queries=1)
        start, end = R.shard_token_range(tokens, world, rank, align=128)
        shard = O.build_cache(key[:, start:end].contiguous(), value[:, start:end].contiguous(),
                              classes[start // page : end // page], page_size=page)
        if rank == world - 1:
            for i in range(5):
                O.append_token(shard, new_k[i], new_v[i], tokens + i, tokens + i)
        q = queries[0].float()
        if shard.n_fp + shard.n_i4 + shard.i2_active + shard.recent_len:
            top, den, acc = O.decode_state(q, shard)
        else:
            top, den, acc = torch.full((1, 16), float("-inf")), torch.zeros(1, 16), torch.zeros(1, 16, 128)
        state = torch.cat((top.unsqueeze(-1), den.unsqueeze(-1), acc), -1).contiguous()      # [1,16,130]
        gathered = torch.empty(world, 16, 130)
        dist.all_gather_into_tensor(gathered, state)
        merged = None
        for s in gathered:
            part = (s[..., 0], s[..., 1], s[..., 2:])
            merged = part if merged is None else O.merge_state(merged, part)
        out = merged[2] / merged[1].unsqueeze(-1)
        whole = O.build_cache(key, value, classes, page_size=page)
        for i in range(5):
            O.append_token(whole, new_k[i], new_v[i], tokens + i, tokens + i)
        want = O.decode_fp32(q, whole)
        results[rank] = float((out - want).abs().max())
        # per-shard packing is bit-identical to the slice of the single cache (pages and key blocks do not straddle)
        whole_k = O.dequantize_k_int4(whole.k_packed, whole.k_scale, whole.k_zero, 0, whole.k_active, 32)
        assert whole_k.shape[1] == tokens
    finally:
        dist.destroy_process_group()


@pytest.mark.parametrize("world,tokens", [(2, 2048), (3, 1536)])
def test_sharded_decode_protocol_on_cpu_ranks(world, tokens):
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(world, port, tokens, results), nprocs=world, join=True)
    assert len(results) == world
    assert max(results.values()) < 2e-6, dict(results)


def _worker_with_absent_rank(rank, world, port, results):
    """The last rank joins the group and then never contributes its state.  The others must come back from the
    exchange step with an error inside the group's (short) timeout and report it; nobody waits for ever."""
    import datetime
    import time
    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    dist.init_process_group("gloo", rank=rank, world_size=world, timeout=datetime.timedelta(seconds=5))
    t0 = time.monotonic()
    try:
        if rank == world - 1:
            results[rank] = "absent"
            time.sleep(1.0)          # alive, between steps, but silent
            return
        state = torch.zeros(1, 16, 130)
        gathered = torch.empty(world, 16, 130)
        try:
            dist.all_gather_into_tensor(gathered, state)
            results[rank] = "completed"
        except Exception:   # noqa: BLE001 -- gloo reports a timeout or a closed connection, depending on timing
            results[rank] = f"exchange failed after {time.monotonic() - t0:.1f} s"
    finally:
        try:
            dist.destroy_process_group()
        except Exception:   # noqa: BLE001 -- the group is already broken on the survivors
            pass


def test_a_rank_that_never_contributes_is_reported_not_waited_for():
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker_with_absent_rank, args=(3, port, results), nprocs=3, join=True)
    assert results[2] == "absent"
    for rank in (0, 1):
        assert results[rank].startswith("exchange failed"), dict(results)
