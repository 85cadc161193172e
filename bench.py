#!/usr/bin/env python
"""Benchmark of the SSPA packed-KV decode path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference]

Workload "decode_32k_b8" (default): one layer, 16 query / 2 KV heads of 128 dims,
batch 8, 32768 cached tokens per request in 64-token pages whose value precision is
drawn from a seed as bf16 25 % / INT4 50 % / INT2 25 %, INT4 keys in 32-token
blocks, a 128-token bf16 residual window.  A step is one decode launch over the
whole batch that also appends one new token per request; every 128 steps the
residual window is quantized and packed (flush).  Four distinct cache sets are
visited round-robin (4 x ~98 MB > L2), so every step reads from HBM.

``value`` is the whole-job algorithmic GB/s with inputs resident in HBM
(CUDA-graph replays, device-timed); ``e2e`` is the same metric through the public
operator call with host query/key/value buffers and a host read of the output
inside the timed region.  With N > 1 every rank runs its own replica (requests
are independent: no data-path collective) and the line also carries the
sequence-sharded 1M-token decode, which does exchange (max, sum-exp, out) states.
"""
from __future__ import annotations

import argparse
import json
import os
import subprocess
import sys
import threading
import time

ROOT = os.path.dirname(os.path.abspath(__file__))
for _p in (ROOT, os.path.join(ROOT, "tests"), os.path.join(ROOT, "tests", "golden")):
    if _p not in sys.path:
        sys.path.insert(0, _p)

import torch  # noqa: E402

HQ, HKV, D = 16, 2, 128
PAGE, K_BLOCK, V2_GROUP, RING = 64, 32, 32, 128
METRIC = "packed_kv_decode_effective_hbm_gbps"


def page_classes(n_pages: int, seed: int, p_fp: float, p_i4: float) -> torch.Tensor:
    r = torch.rand(n_pages, generator=torch.Generator().manual_seed(seed))
    return torch.where(r < p_fp, 1, torch.where(r < p_fp + p_i4, 2, 5))


def synth_kv(tokens: int, seed: int, device, hkv: int = HKV):
    """K/V ~ N(0,1) in bf16; key channels scaled by per-(head, channel) lognormal(0,1) factors."""
    g = torch.Generator(device=device).manual_seed(seed)
    key = torch.randn(hkv, tokens, D, generator=g, device=device)
    key = (key * torch.exp(torch.randn(hkv, 1, D, generator=g, device=device))).to(torch.bfloat16)
    value = torch.randn(hkv, tokens, D, generator=g, device=device).to(torch.bfloat16)
    return key, value


def algorithmic_bytes(n_fp, n_i4, n_i2, ring_len, batch, hq=HQ, hkv=HKV, append=True) -> int:
    """Bytes one decode step has to move: 76 B/token of keys, 256/68/44 B/token of
    values, 512 B per residual token, query in / output out, appended rows."""
    hist = n_fp + n_i4 + n_i2
    per_head = hist * (64 + 3 * D // K_BLOCK) + n_fp * 256 + n_i4 * 68 + n_i2 * (32 + 3 * D // V2_GROUP) + ring_len * 512
    return batch * (hkv * per_head + 4 * hq * D + (8 * hkv * D if append else 0))


class ClockSampler:
    """SM clock and throttle reasons sampled through NVML while the timed region runs."""

    def __init__(self, index: int, period: float = 0.004):
        self.index, self.period = index, period
        self.mhz, self.reasons, self.max_mhz = [], 0, None
        self._stop, self._thread = threading.Event(), None

    def _run(self):
        try:
            import pynvml as nv
            nv.nvmlInit()
            visible = os.environ.get("CUDA_VISIBLE_DEVICES")
            phys = int(visible.split(",")[self.index]) if visible and visible.split(",")[self.index].isdigit() else self.index
            h = nv.nvmlDeviceGetHandleByIndex(phys)
            self.max_mhz = int(nv.nvmlDeviceGetMaxClockInfo(h, nv.NVML_CLOCK_SM))
            while not self._stop.is_set():
                self.mhz.append(int(nv.nvmlDeviceGetClockInfo(h, nv.NVML_CLOCK_SM)))
                self.reasons |= int(nv.nvmlDeviceGetCurrentClocksEventReasons(h))
                self._stop.wait(self.period)
        except Exception as exc:  # reading clocks must never break the benchmark
            self.error = repr(exc)

    def __enter__(self):
        self._thread = threading.Thread(target=self._run, daemon=True)
        self._thread.start()
        time.sleep(0.02)
        return self

    def __exit__(self, *exc):
        self._stop.set()
        self._thread.join(timeout=10)

    def summary(self) -> dict:
        mhz = sorted(self.mhz)
        bits = {"hw_slowdown": 0x8, "hw_thermal_slowdown": 0x40, "sw_thermal_slowdown": 0x20, "sw_power_cap": 0x4,
                "hw_power_brake_slowdown": 0x80}
        out = {"sm_mhz": mhz[len(mhz) // 2] if mhz else None, "sm_max_mhz": self.max_mhz,
               "reasons": [n for n, b in bits.items() if self.reasons & b], "samples": len(mhz)}
        if hasattr(self, "error"):
            out["error"] = self.error
        return out


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch on the default workload, from the ncu
# capture summarised in profiles/decode_kernel_b8_32k.md (96.55 MB read + 3.09 MB written, mean of two launches).
NCU_DRAM_BYTES_PER_LAUNCH = 99_630_000


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


# --------------------------------------------------------------------------- #
# this library
# --------------------------------------------------------------------------- #
def build_batched_executor(batch, tokens, seed, device, p_fp=0.25, p_i4=0.5):
    import r2omni_b200 as R
    from gpu_helpers import make_plan

    singles = []
    classes = page_classes(tokens // PAGE, seed, p_fp, p_i4)
    for b in range(batch):
        key, value = synth_kv(tokens, seed * 1000 + b, device)
        cache = R.build_three_precision_cache(key, value, make_plan(classes, PAGE, RING), page_size=PAGE,
                                              key_quantization_superblock=K_BLOCK, int2_group_size=V2_GROUP,
                                              compact_key_append_capacity=RING, recent_flush_size=RING)
        ws = R.allocate_splitk_workspace(cache, num_query_heads=HQ)
        singles.append(R.prepare_splitk_executor(cache, ws))
        del key, value
    if batch == 1:
        return singles[0]
    ex = R.stack_homogeneous_splitk_executors(singles)
    del singles
    return ex


class ReplicaBench:
    """Round-robin over `sets` batched caches; decode+append every step, flush every 128 steps per set."""

    def __init__(self, device, batch=8, tokens=32768, sets=4, p_fp=0.25, p_i4=0.5):
        import r2omni_b200 as R
        self.R, self.device, self.batch, self.tokens = R, device, batch, tokens
        self.ex = [build_batched_executor(batch, tokens, 11 + s, device, p_fp, p_i4) for s in range(sets)]
        g = torch.Generator(device=device).manual_seed(5)
        self.q = torch.randn(batch, HQ, D, generator=g, device=device).to(torch.bfloat16)
        self.k = torch.randn(batch, HKV, D, generator=g, device=device).to(torch.bfloat16)
        self.v = torch.randn(batch, HKV, D, generator=g, device=device).to(torch.bfloat16)
        self.stats = R.DynamicCacheStats()
        self.base = [(e.arenas.k_active, e.arenas.i2_active) for e in self.ex]
        self.step_graphs, self.flush_graphs = [], []
        # prefill the rings half way so that flushes fall inside short runs too
        for e in self.ex:
            for i in range(RING // 2):
                e(self.q, append=(self.k, self.v, tokens + i, tokens + i))
        torch.cuda.synchronize(device)
        for e in self.ex:
            gs, gf = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            ring = e.arenas.recent_len
            with torch.cuda.graph(gs):
                e(self.q, append=(self.k, self.v, tokens, tokens))
            e.arenas.recent_len = ring                     # capture does not run the kernel
            with torch.cuda.graph(gf):
                e.arenas.recent_len = RING
                R.flush_recent(e.arenas)
            # flushed tokens overwrite the same arena rows on every replay: the context stays at `tokens` + ring
            e.arenas.k_active, e.arenas.i2_active = self.base[len(self.step_graphs)]
            e.arenas.recent_len = ring
            self.step_graphs.append(gs)
            self.flush_graphs.append(gf)
        # one graph per round (a step on every set, back to back): consecutive decode launches are joined by
        # programmatic dependent launch edges, as consecutive layers of a model are
        rings = [e.arenas.recent_len for e in self.ex]
        self.round_graph = torch.cuda.CUDAGraph()
        with torch.cuda.graph(self.round_graph):
            for e in self.ex:
                e(self.q, append=(self.k, self.v, tokens, tokens))
        for e, ring in zip(self.ex, rings):
            e.arenas.recent_len = ring
        self.launches_per_step = 1
        self.launches_per_flush = 3
        a = self.ex[0].arenas
        self.geom = (a.n_fp, a.n_i4, a.i2_active)


    def step_bytes(self, ring_len):
        return algorithmic_bytes(*self.geom, ring_len, self.batch)

    def run_graph_steps(self, steps, start=0):
        """Enqueue `steps` steps; returns (bytes moved, decode launches, flushes)."""
        total, flushes = 0, 0
        n, i, end = len(self.ex), start, start + steps
        while i < end:
            s = i % n
            whole_round = s == 0 and i + n <= end
            for t in (range(n) if whole_round else (s,)):
                a = self.ex[t].arenas
                if a.recent_len == RING:
                    self.flush_graphs[t].replay()
                    a.recent_len = 0
                    flushes += 1
                total += self.step_bytes(a.recent_len + 1)
                a.recent_len += 1
            if whole_round:
                self.round_graph.replay()
                i += n
            else:
                self.step_graphs[s].replay()
                i += 1
        return total, steps, flushes

    def run_api_steps(self, steps, host_in, host_out, start=0, torch_copies=False):
        """Public operator call with host buffers, one call per step (SplitKExecutor.step_host = r2k_decode_host):
        H2D of q/k/v from pinned memory, decode+append, D2H of the output, wait.  `torch_copies` issues the same
        step as three torch calls around the device-tensor operator instead (timed beside it for comparison)."""
        total = 0
        nq, nk = self.q.numel(), self.k.numel()
        dev_in = self._dev_in
        for i in range(start, start + steps):
            s = i % len(self.ex)
            e = self.ex[s]
            a = e.arenas
            if a.recent_len == RING:
                self.R.flush_recent(a)
                a.k_active, a.i2_active = self.base[s]
            total += self.step_bytes(a.recent_len + 1)
            if not torch_copies:
                e.step_host(host_in, host_out, append_indices=(self.tokens + i, self.tokens + i))
                continue
            dev_in.copy_(host_in, non_blocking=True)
            q = dev_in[:nq].view(self.batch, HQ, D)
            k = dev_in[nq : nq + nk].view(self.batch, HKV, D)
            v = dev_in[nq + nk :].view(self.batch, HKV, D)
            out = e(q, append=(k, v, self.tokens + i, self.tokens + i))
            host_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()   # the caller reads the result
        return total

    def prepare_api(self):
        n = self.q.numel() + 2 * self.k.numel()
        host_in = torch.empty(n, dtype=torch.bfloat16).pin_memory()
        host_in[: self.q.numel()] = self.q.flatten().cpu()
        host_in[self.q.numel() : self.q.numel() + self.k.numel()] = self.k.flatten().cpu()
        host_in[self.q.numel() + self.k.numel() :] = self.v.flatten().cpu()
        host_out = torch.empty(self.batch, HQ, D, dtype=torch.bfloat16).pin_memory()
        self._dev_in = torch.empty(n, dtype=torch.bfloat16, device=self.device)
        return host_in, host_out


def time_region(device, fn, dist_on):
    """Barrier + synchronize on both sides; CUDA-event time in ms, max over ranks."""
    import torch.distributed as dist
    if dist_on:
        dist.barrier()
    torch.cuda.synchronize(device)
    e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
    e0.record()
    result = fn()
    e1.record()
    torch.cuda.synchronize(device)
    ms = e0.elapsed_time(e1)
    if dist_on:
        t = torch.tensor([ms], device=device, dtype=torch.float64)
        dist.all_reduce(t, op=dist.ReduceOp.MAX)
        ms = float(t.item())
        dist.barrier()
    return ms, result


def sharded_1m(device, rank, world, steps, warmup, dist_on):
    """Sequence-sharded decode of a 1,048,576-token cache (INT4/INT2 value pages 50/50,
    128-token residual window on the last rank).  With more than one rank the merge is fused into the decode
    launch (peer stores over NVLink, r2k_decode_exchange); the all-gather + merge-launch variant is timed
    beside it for comparison."""
    import torch.distributed as dist

    import r2omni_b200 as R
    from gpu_helpers import make_plan

    total = 1 << 20
    per = total // world
    classes = page_classes(total // PAGE, 77, 0.0, 0.5)[rank * (per // PAGE) : (rank + 1) * (per // PAGE)]
    key, value = synth_kv(per, 900 + rank, device)
    cache = R.build_three_precision_cache(key, value, make_plan(classes, PAGE, RING), page_size=PAGE,
                                          key_quantization_superblock=K_BLOCK, int2_group_size=V2_GROUP,
                                          compact_key_append_capacity=RING, recent_flush_size=RING)
    del key, value
    ex = R.prepare_splitk_executor(cache, R.allocate_splitk_workspace(cache, num_query_heads=HQ))
    g = torch.Generator(device=device).manual_seed(6)
    q = torch.randn(1, HQ, D, generator=g, device=device).to(torch.bfloat16)
    if rank == world - 1:
        st = R.DynamicCacheStats()
        nk = torch.randn(RING, HKV, 1, D, generator=g, device=device).to(torch.bfloat16)
        for i in range(RING):
            R.append_generated_token(cache, nk[i], nk[(i + 1) % RING], global_token_index=total + i,
                                     logical_position=total + i, stats=st)
    a = cache.arenas
    my_bytes = algorithmic_bytes(a.n_fp, a.n_i4, a.i2_active, a.recent_len, 1, append=False)
    def timed(one_step, steps):
        """(us per step, graphed?) for `steps` steps; eight steps per CUDA graph, eager launches if capture is refused."""
        for _ in range(max(warmup, 3)):
            one_step()
        torch.cuda.synchronize(device)
        graph, per_replay = None, 8
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for _ in range(per_replay):
                    one_step()
            graph.replay()
            torch.cuda.synchronize(device)
        except Exception:
            graph = None
            torch.cuda.synchronize(device)
        if graph is not None:
            steps = max(per_replay, steps // per_replay * per_replay)
            ms, _ = time_region(device, lambda: [graph.replay() for _ in range(steps // per_replay)], dist_on)
        else:
            ms, _ = time_region(device, lambda: [one_step() for _ in range(steps)], dist_on)
        return ms * 1e3 / steps, graph is not None, steps

    nccl_us = None
    if world == 1:
        us, graphed, steps = timed(lambda: ex(q), steps)
    else:
        gathered = R.SequenceShardedExecutor(ex)
        local_us, _, _ = timed(lambda: ex.decode_state(q, out=gathered.state), steps)   # this rank's shard alone
        nccl_us, _, _ = timed(lambda: gathered(q), steps)
        # the fused variant is the one reported; if it cannot be set up or times out on this box, every rank
        # agrees on that and the all-gather number is reported instead (with the reason)
        fused_error, fused = None, None
        try:
            fused = R.SequenceShardedExecutor(ex, fused=True, device_step_counter=True)
            fused(q)                                   # one step first: a broken exchange shows up as a bounded
            probe = torch.tensor([float(ex.device_status())], device=device)   # wait here, not 300 times over
            dist.all_reduce(probe, op=dist.ReduceOp.MAX)
            if float(probe.item()) != 0.0:
                fused_error = "device-side timeout in the cross-rank wait"
            else:
                us, graphed, steps = timed(lambda: fused(q), steps)
                if ex.device_status() != 0:
                    fused_error = "device-side timeout in the cross-rank wait"
        except Exception as exc:   # noqa: BLE001 -- reported in the JSON line
            fused_error = repr(exc)[:200]
        ok = torch.tensor([0.0 if fused_error else 1.0], device=device)
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)
        if fused is not None and fused_error is None:
            fused.close()
        if float(ok.item()) < 1.0:
            us, graphed, steps = nccl_us, True, steps
            fused_error = fused_error or "another rank failed"
    bytes_all = torch.tensor([float(my_bytes)], device=device, dtype=torch.float64)
    if dist_on:
        dist.all_reduce(bytes_all)
    out = {"workload": "sharded_1m_b1", "tokens": total, "n_gpus": world, "us_per_step": round(us, 2),
           "gbps": round(float(bytes_all.item()) / (us * 1e-6) / 1e9, 1), "steps": steps,
           "collective": "none" if world == 1 else "fused: tagged peer stores over NVLink inside the decode launch",
           "launches_per_step": 1, "cuda_graph": graphed}
    if nccl_us is not None:
        out["us_per_step_nccl_all_gather"] = round(nccl_us, 2)
        out["us_per_step_local_shard_only"] = round(local_us, 2)
        if fused_error:
            out.update(collective="nccl all_gather of [Hq,130] fp32 per rank", launches_per_step=2, fused_error=fused_error)
    return out


def cpu_baseline_sample(tokens, seconds=12.0):
    """The oracle (a port of the reference's dequantise-then-attend CPU path) on ONE
    request of the workload, all host threads."""
    from oracle import sspa_oracle as O
    torch.set_num_threads(os.cpu_count() or 1)
    classes = page_classes(tokens // PAGE, 11, 0.25, 0.5)
    key, value = synth_kv(tokens, 11000, "cpu")
    cache = O.build_cache(key, value, classes, page_size=PAGE, recent_capacity=RING, k_block=K_BLOCK, v2_group=V2_GROUP,
                          append_capacity=RING)
    g = torch.Generator().manual_seed(5)
    nk = torch.randn(RING // 2, HKV, D, generator=g).to(torch.bfloat16)
    for i in range(RING // 2):
        O.append_token(cache, nk[i], nk[i], tokens + i, tokens + i)
    q = torch.randn(1, HQ, D, generator=g).to(torch.bfloat16)
    O.decode(q, cache)
    best, reps, t_end = float("inf"), 0, time.perf_counter() + seconds
    while time.perf_counter() < t_end or reps < 3:
        t0 = time.perf_counter()
        O.append_token(cache, nk[0], nk[0], 0, 0) if cache.recent_len < RING else None
        O.decode(q, cache)
        best = min(best, time.perf_counter() - t0)
        reps += 1
    nbytes = algorithmic_bytes(cache.n_fp, cache.n_i4, cache.i2_active, cache.recent_len, 1)
    return {"value": round(nbytes / best / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
            "sample": f"1 of 8 requests ({tokens} tokens, same page mix), best of {reps} decode+append steps, "
                      f"{best * 1e3:.1f} ms per request-step"}


def run_reference_arm(args):
    """The reference's CPU implementation of the path (oracle port; the reference is Python and
    does not travel to the GPU box), all host threads, one request per step."""
    from oracle import sspa_oracle as O
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    torch.set_num_threads(os.cpu_count() or 1)
    tokens = 32768
    classes = page_classes(tokens // PAGE, 11, 0.25, 0.5)
    key, value = synth_kv(tokens, 11000, "cpu")
    cache = O.build_cache(key, value, classes, page_size=PAGE, recent_capacity=RING, k_block=K_BLOCK, v2_group=V2_GROUP,
                          append_capacity=RING)
    base = (cache.k_active, cache.i2_active)
    g = torch.Generator().manual_seed(5)
    nk = torch.randn(RING, HKV, D, generator=g).to(torch.bfloat16)
    q = torch.randn(1, HQ, D, generator=g).to(torch.bfloat16)
    for i in range(RING // 2):
        O.append_token(cache, nk[i], nk[i], tokens + i, tokens + i)
    steps = min(args.steps, 200)

    def step(i):
        if O.append_token(cache, nk[i % RING], nk[(i + 1) % RING], tokens + i, tokens + i):
            cache.k_active, cache.i2_active = base[0], base[1]     # keep the context at 32768 + residual
            cache.i2_global, cache.i2_logical = cache.i2_global[: base[1]], cache.i2_logical[: base[1]]
        O.decode(q, cache)
        return algorithmic_bytes(cache.n_fp, cache.n_i4, cache.i2_active, cache.recent_len, 1)

    for i in range(max(1, min(args.warmup, 3))):
        step(i)
    t0 = time.perf_counter()
    nbytes = sum(step(10 + i) for i in range(steps))
    sec = time.perf_counter() - t0
    value = round(nbytes / sec / 1e9, 3)
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(sec * 1e3 / steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "bf16", "data": "synthetic",
        "config": {"workload": "decode_32k_b8", "sample": "one request (32768 tokens) per step", "heads": "16q/2kv x128"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": "port",
                         "sample": "one of the 8 requests per step (32768 tokens, bf16/INT4/INT2 pages 25/50/25), "
                                   "decode + one-token append, flush when the residual window fills"},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=8192)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_32k_b8", choices=["decode_32k_b8", "small"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--page-mix", default="25,50,25", help="percent of bf16,INT4,INT2 value pages (kernel studies)")
    args = ap.parse_args()
    if args.impl == "reference":
        run_reference_arm(args)
        return

    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist_on = world > 1
    if dist_on:
        dist.init_process_group("nccl", device_id=device)
    from r2omni_b200 import _lib as L
    L.lib()   # fails loudly when the CUDA library is missing: there is no fallback

    warmup = max(args.warmup, 3)
    tokens, batch = (32768, 8) if args.workload == "decode_32k_b8" else (4096, 2)
    mix = [float(x) / 100.0 for x in args.page_mix.split(",")]
    bench = ReplicaBench(device, batch=batch, tokens=tokens, sets=4, p_fp=mix[0], p_i4=mix[1])
    bench.run_graph_steps(warmup)
    launches0 = L.lib().r2k_launch_count()
    with ClockSampler(local) as clocks:
        ms, (nbytes, decodes, flushes) = time_region(device, lambda: bench.run_graph_steps(args.steps, start=warmup), dist_on)
    value = nbytes * world / (ms * 1e-3) / 1e9
    gpu_launches = decodes * bench.launches_per_step + flushes * bench.launches_per_flush

    # the decode kernel alone: same graphs, no flush in the window
    probe_steps = 0
    def make_room():
        for s, e in enumerate(bench.ex):
            if e.arenas.recent_len > RING - 33:
                bench.flush_graphs[s].replay()
                e.arenas.recent_len = 0
    def decode_only(rounds=True):
        nonlocal probe_steps
        b = 0
        for r in range(32):
            for e in bench.ex:
                b += bench.step_bytes(e.arenas.recent_len + 1)
                e.arenas.recent_len += 1
                probe_steps += 1
            if rounds:
                bench.round_graph.replay()
            else:
                for g in bench.step_graphs:
                    g.replay()
        return b
    # launches separated by graph boundaries (no overlap between consecutive launches), for comparison
    make_room()
    iso_ms, _ = time_region(device, lambda: decode_only(False), dist_on)
    iso_us = iso_ms * 1e3 / max(probe_steps, 1)
    probe_steps = 0
    make_room()
    k_ms, k_bytes = time_region(device, decode_only, dist_on)
    peak, peak_kind = measured_peak_gbs()
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "decode_kernel<bf16>", "achieved": round(achieved, 1), "peak": peak,
                "peak_source": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "frac_of_nominal_8000": round(achieved / 8000.0, 4), "us_per_launch": round(k_ms * 1e3 / max(probe_steps, 1), 2),
                "us_per_launch_isolated": round(iso_us, 2),
                "bytes_per_launch": int(k_bytes / max(probe_steps, 1)),
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH if args.workload == "decode_32k_b8" and args.page_mix == "25,50,25" else None}

    # the flush alone (quantize-and-pack of the 128-token residual window: 3 launches, launch-bound)
    def flush_only():
        for r in range(8):
            for s_, e in enumerate(bench.ex):
                bench.flush_graphs[s_].replay()
                e.arenas.recent_len = 0
    f_ms, _ = time_region(device, flush_only, dist_on)
    flush = {"us_per_flush": round(f_ms * 1e3 / (8 * len(bench.ex)), 2), "launches": bench.launches_per_flush,
             "amortised_us_per_step": round(f_ms * 1e3 / (8 * len(bench.ex)) / RING, 3)}

    # end to end through the operator call with host buffers
    e2e = None
    if not args.no_e2e:
        host_in, host_out = bench.prepare_api()
        bench.run_api_steps(warmup, host_in, host_out)
        e2e_steps = min(args.steps, 512)
        e_ms, e_bytes = time_region(device, lambda: bench.run_api_steps(e2e_steps, host_in, host_out, start=warmup), dist_on)
        e2e = {"value": round(e_bytes * world / (e_ms * 1e-3) / 1e9, 1), "unit": "GB/s",
               "us_per_step": round(e_ms * 1e3 / e2e_steps, 2), "steps": e2e_steps,
               "h2d_bytes_per_step": int(host_in.numel() * 2), "d2h_bytes_per_step": int(host_out.numel() * 2),
               "call": "SplitKExecutor.step_host (r2k_decode_host): H2D copy kernel from the pinned block, decode+append writing the pinned result over PCIe, stream wait"}
        t_steps = min(e2e_steps, 256)
        t_ms, _ = time_region(device, lambda: bench.run_api_steps(t_steps, host_in, host_out, start=warmup + e2e_steps,
                                                                  torch_copies=True), dist_on)
        e2e["us_per_step_three_torch_calls"] = round(t_ms * 1e3 / t_steps, 2)
    del bench
    torch.cuda.empty_cache()

    sharded = None if args.no_sharded or args.workload != "decode_32k_b8" else \
        sharded_1m(device, rank, world, steps=min(args.steps, 256), warmup=warmup, dist_on=dist_on)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample(tokens)

    if rank == 0:
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(ms / args.steps, 5), "us_per_step": round(ms * 1e3 / args.steps, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 tensor-core products, f32 accumulation (u4/u2 codes, bf16 pages)",
            "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": batch, "tokens_per_request": tokens, "heads": "16q/2kv x128",
                       "pages": f"64 tokens; bf16/INT4/INT2 = {args.page_mix} % from a seed", "keys": "INT4 per channel, 32-token blocks",
                       "residual_window": RING, "append_per_step": 1, "flush_every": RING,
                       "l2": "4 cache sets of ~98 MB visited round-robin (inputs larger than L2)",
                       "parallelism": f"{world} independent replicas" if world > 1 else "1 GPU",
                       "step_bytes": bench_bytes_note(tokens, batch)},
            "gpu_launches": int(gpu_launches), "flushes_in_region": int(flushes), "flush": flush,
            "roofline": roofline, "e2e": e2e, "clocks": clocks.summary(),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if sharded is not None:
            line["seq_sharded"] = sharded
        print(json.dumps(line))
    if dist_on:
        dist.destroy_process_group()


def bench_bytes_note(tokens, batch):
    return f"sum over {batch} requests x 2 kv heads of 76 B/token keys + 256/68/44 B/token values + 512 B/residual token"


if __name__ == "__main__":
    main()
