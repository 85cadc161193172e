"""Sequence-sharded decode on 2 GPUs over NCCL (skipped when fewer than two devices are visible):
per-rank CUDA decode to un-normalised states, one all-gather, CUDA merge; checked against the
single-cache oracle.  The fused variant (peer stores and merge inside the decode launch) must give the same bits
as the all-gather variant, step after step."""
import os
import socket

import pytest
import torch
import torch.distributed as dist
import torch.multiprocessing as mp

pytestmark = pytest.mark.gpu


def _free_port() -> int:
    with socket.socket() as s:
        s.bind(("127.0.0.1", 0))
        return s.getsockname()[1]


def _worker(rank, world, port, results, fused=False):
    import r2omni_b200 as R
    from gpu_helpers import build_gpu_cache, make_executor
    from oracle import sspa_oracle as O
    from recipe import make_inputs

    os.environ.update(MASTER_ADDR="127.0.0.1", MASTER_PORT=str(port))
    torch.cuda.set_device(rank)
    dist.init_process_group("nccl", rank=rank, world_size=world, device_id=torch.device("cuda", rank))
    try:
        tokens, page = 8192, 64
        r = torch.rand(tokens // page, generator=torch.Generator().manual_seed(3))
        classes = torch.where(r < 0.25, 1, torch.where(r < 0.75, 2, 5))
        key, value, new_k, new_v, queries = make_inputs(seed=61, hq=16, hkv=2, tokens=tokens, appends=3, n_queries=2)
        start, end = R.shard_token_range(tokens, world, rank, align=128)
        cache = build_gpu_cache(key[:, start:end].contiguous(), value[:, start:end].contiguous(),
                                classes[start // page : end // page], page_size=page, device=f"cuda:{rank}")
        sharded = R.SequenceShardedExecutor(make_executor(cache, 16), fused=fused)
        twin = None
        if fused:   # the all-gather path over an identical cache: same states, same merge order
            twin_cache = build_gpu_cache(key[:, start:end].contiguous(), value[:, start:end].contiguous(),
                                         classes[start // page : end // page], page_size=page, device=f"cuda:{rank}")
            twin = R.SequenceShardedExecutor(make_executor(twin_cache, 16))
        whole = O.build_cache(key, value, classes, page_size=page)
        dev = torch.device("cuda", rank)
        err = 0.0
        for i in range(3):   # the fused append lands on the last rank only; every rank makes the same call
            out = sharded(queries[0].to(dev), append=(new_k[i].unsqueeze(0).contiguous().to(dev),
                                                      new_v[i].unsqueeze(0).contiguous().to(dev), tokens + i, tokens + i))
            if twin is not None:
                ref = twin(queries[0].to(dev), append=(new_k[i].unsqueeze(0).contiguous().to(dev),
                                                       new_v[i].unsqueeze(0).contiguous().to(dev), tokens + i, tokens + i))
                if not torch.equal(out, ref):
                    err = max(err, 1.0 + float((out.float() - ref.float()).abs().max()))
                if rank == world - 1:
                    twin_cache.recent_fp_pool.active_length += 1
                if sharded.local.device_status() != 0:
                    err += 100.0
            if rank == world - 1:
                cache.recent_fp_pool.active_length += 1
            O.append_token(whole, new_k[i], new_v[i], tokens + i, tokens + i)
            want = O.decode(queries[0], whole).float()
            err = max(err, float(((out.float().cpu() - want).abs() - (2e-3 + 1e-2 * want.abs())).max()))
        results[rank] = err
        if fused:
            sharded.close()
    finally:
        dist.destroy_process_group()


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_sequence_sharded_decode():
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results), nprocs=2, join=True)
    assert len(results) == 2 and max(results.values()) <= 0.0, dict(results)


@pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")
def test_two_gpu_fused_exchange_matches_all_gather():
    port = _free_port()
    manager = mp.Manager()
    results = manager.dict()
    mp.spawn(_worker, args=(2, port, results, True), nprocs=2, join=True)
    assert len(results) == 2 and max(results.values()) <= 0.0, dict(results)


def test_single_rank_sharded_executor_equals_plain_decode():
    import r2omni_b200 as R
    from gpu_helpers import assert_close, build_gpu_cache, make_executor
    from recipe import make_inputs
    classes = torch.tensor([2, 5, 1, 2, 5, 5, 2, 1])
    key, value, _, _, queries = make_inputs(seed=62, hq=16, hkv=2, tokens=512, appends=1, n_queries=1)
    cache = build_gpu_cache(key, value, classes, page_size=64)
    ex = make_executor(cache, 16)
    plain = ex(queries[0].cuda()).clone()
    assert_close(R.SequenceShardedExecutor(ex)(queries[0].cuda()), plain, "world-1 sharded")
