#!/usr/bin/env python
"""Benchmark of the SSPA packed-KV decode path on B200.

    python bench.py --gpus N --steps K --warmup W [--impl reference] [--workload NAME]

Workloads (``config.workload``):

* ``decode_32k_b8`` (default): one layer, 16 query / 2 KV heads of 128 dims, batch 8, 32768 cached tokens per
  request in 64-token pages whose value precision is drawn from a seed as bf16 25 % / INT4 50 % / INT2 25 %, INT4
  keys in 32-token blocks, a 128-token bf16 residual window.  A step is one decode launch over the whole batch that
  also appends one new token per request; every 128 steps the residual window is quantized and packed (flush).
  Four distinct cache sets are visited round-robin (4 x ~98 MB > L2), so every step reads from HBM.
* ``decode_4k_b1``: batch 1, 4096 INT4-value tokens in 32-token pages plus a full 128-token residual window; a step
  is one decode launch (launch-bound: 1.3 MB).  128 cache sets are visited round-robin (168 MB > L2).
* ``decode_7b_28l``: 28 layers of the 28-query / 4-KV-head shape, batch 16, 65536 tokens per request, mixed pages as
  above (~21.8 GB resident).  A step is the attention of ALL layers: 28 decode launches with fused append, joined by
  programmatic dependent launch; every 128 steps all layers flush.

* ``decode_3b_36l``: the attention of the thinker workload below alone: 36 layers of 16 query / 2 KV heads, batch 32,
  16384 tokens per request (~7.6 GB resident); a step is 36 decode launches.
* ``thinker_3b_b32``: greedy decode of a random-weight 36-layer Qwen2.5-Omni-3B-shaped decoder (hidden 2048, MLP
  11008, vocabulary 151936), batch 32, 16384 prefilled tokens per request and layer, 256 generated tokens, with this
  library's attention manager path in every layer; its line reports tokens/s.

``value`` is the whole-job algorithmic GB/s with inputs resident in HBM (CUDA-graph replays, device-timed); ``e2e``
is the same metric through the public operator call with host query/key/value buffers and a host read of the output
inside the timed region.  After the timed regions one decode of the benchmarked caches is compared with the CPU
oracle (``parity``).  With N > 1 every rank runs its own replica (requests are independent: no data-path collective)
and the line also carries the sequence-sharded 1M-token decode, which does exchange (max, sum-exp, out) states and
is checked against the oracle's per-shard states at every N.  ``triton_reference`` times the reference's own Triton
decoder on the same GPU and the same seeded workload when the reference is installed under ``baseline/_ref``.
"""
from __future__ import annotations

import argparse
import json
import os
import statistics
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
ATOL, RTOL = 2e-3, 1e-2   # attention tolerance: max-abs 2e-3 + rel 1e-2

WORKLOADS = {
    # name: heads, batch, tokens, cache sets, page, (bf16, INT4) page fractions, what a step is, append per step
    "decode_32k_b8": dict(hq=16, hkv=2, batch=8, tokens=32768, sets=4, page=64, mix=(0.25, 0.5), step="launch", append=True),
    "decode_4k_b1": dict(hq=16, hkv=2, batch=1, tokens=4096, sets=128, page=32, mix=(0.0, 1.0), step="launch", append=False),
    "decode_7b_28l": dict(hq=28, hkv=4, batch=16, tokens=65536, sets=28, page=64, mix=(0.25, 0.5), step="round", append=True),
    "decode_3b_36l": dict(hq=16, hkv=2, batch=32, tokens=16384, sets=36, page=64, mix=(0.25, 0.5), step="round", append=True),
    "small": dict(hq=16, hkv=2, batch=2, tokens=4096, sets=4, page=64, mix=(0.25, 0.5), step="launch", append=True),
}


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


# dram__bytes_read.sum + dram__bytes_write.sum of one decode_kernel launch on the default workload, taken from an
# ncu capture of this command (96.55 MB read + 3.09 MB written, mean of two launches); a constant, not measured here.
NCU_DRAM_BYTES_PER_LAUNCH = 99_630_000


def measured_peak_gbs():
    path = os.path.join(ROOT, "MEASURED_PEAKS.json")
    if os.path.exists(path):
        with open(path) as f:
            return float(json.load(f)["hbm_gbs"]), "measured"
    return 6650.0, "fallback"


def spread(samples) -> dict:
    """min / median / max of repeated measurements (so that an outlier can be told from a regression)."""
    s = sorted(samples)
    return {"repeats": len(s), "min": round(s[0], 2), "median": round(statistics.median(s), 2), "max": round(s[-1], 2)}


def tolerance_excess(got: torch.Tensor, want: torch.Tensor):
    """(max-abs error, worst excess over atol + rtol*|want|): the result passes when the excess is <= 0."""
    got, want = got.float().cpu(), want.float().cpu()
    err = (got - want).abs()
    return float(err.max()), float((err - (ATOL + RTOL * want.abs())).max())


# --------------------------------------------------------------------------- #
# the unmodified reference, when it is installed beside the repository
# --------------------------------------------------------------------------- #
_REFERENCE = None


def load_reference():
    """Modules of the reference package installed in baseline/_ref (oracle/install_reference.py), or the reason why
    they cannot be used.  Nothing of the product goes through them: they are the baseline being measured."""
    global _REFERENCE
    if _REFERENCE is not None:
        return _REFERENCE
    path = os.path.join(ROOT, "baseline", "_ref")
    if not os.path.isdir(os.path.join(path, "r2omni")):
        _REFERENCE = (None, "the reference is not installed under baseline/_ref")
        return _REFERENCE
    if path not in sys.path:
        sys.path.insert(0, path)
    sys.dont_write_bytecode = True
    try:
        import types
        ns = types.SimpleNamespace()
        from r2omni.sspa.kernels.triton_fourq_attention import triton_mixed_reference
        from r2omni.sspa.runtime.cache_plan import LayerCompressionPlan
        from r2omni.sspa.runtime.dynamic_fourq_cache import DynamicCacheStats, append_generated_token
        from r2omni.sspa.runtime.precision_pool import build_three_precision_cache
        ns.triton_mixed_reference, ns.LayerCompressionPlan = triton_mixed_reference, LayerCompressionPlan
        ns.DynamicCacheStats, ns.append_generated_token = DynamicCacheStats, append_generated_token
        ns.build_three_precision_cache = build_three_precision_cache
        _REFERENCE = (ns, None)
    except Exception as exc:  # noqa: BLE001 -- reported in the JSON line
        _REFERENCE = (None, f"the reference under baseline/_ref does not import: {exc!r}"[:300])
    return _REFERENCE


def reference_plan(ns, classes: torch.Tensor, page: int, recent_capacity: int, device="cpu"):
    """The reference's plan type; its index tensors live where the key/value tensors do."""
    n = int(classes.numel())
    pos = torch.arange(n * page, device=device)
    classes = classes.to(device)
    sel = lambda c: (classes == c).nonzero().flatten()  # noqa: E731
    return ns.LayerCompressionPlan(
        layer_id=0, fp_pages=sel(1), int4_pages=sel(2), int2_pages=sel(5), evicted_pages=sel(0),
        protected_pages=torch.empty(0, dtype=torch.long, device=device), recent_fp_capacity=recent_capacity,
        logical_positions=pos, global_token_indices=pos.clone(),
        page_offsets=torch.arange(n, device=device) * page, page_lengths=torch.full((n,), page, device=device),
        page_classes=classes)


# --------------------------------------------------------------------------- #
# this library
# --------------------------------------------------------------------------- #
def build_batched_executor(batch, tokens, seed, device, p_fp=0.25, p_i4=0.5, hq=HQ, hkv=HKV, page=PAGE):
    import r2omni_b200 as R
    from gpu_helpers import make_plan

    singles = []
    classes = page_classes(tokens // page, seed, p_fp, p_i4)
    for b in range(batch):
        key, value = synth_kv(tokens, seed * 1000 + b, device, hkv=hkv)
        cache = R.build_three_precision_cache(key, value, make_plan(classes, page, RING), page_size=page,
                                              key_quantization_superblock=K_BLOCK, int2_group_size=V2_GROUP,
                                              compact_key_append_capacity=RING, recent_flush_size=RING)
        ws = R.allocate_splitk_workspace(cache, num_query_heads=hq)
        singles.append(R.prepare_splitk_executor(cache, ws))
        del key, value
    if batch == 1:
        return singles[0]
    ex = R.stack_homogeneous_splitk_executors(singles)
    del singles
    return ex


class ReplicaBench:
    """`sets` batched caches visited in order.  A "visit" is one decode launch on one set (with a fused one-token
    append when the workload appends); a step is one visit, or -- for a multi-layer workload -- one visit of every
    set.  When a set's residual window is full it is flushed before its next visit."""

    def __init__(self, device, *, hq=HQ, hkv=HKV, batch=8, tokens=32768, sets=4, page=PAGE, mix=(0.25, 0.5),
                 step="launch", append=True, seed0=11):
        import r2omni_b200 as R
        self.R, self.device, self.batch, self.tokens = R, device, batch, tokens
        self.hq, self.hkv, self.page, self.mix, self.seed0 = hq, hkv, page, mix, seed0
        self.append, self.visits_per_step = append, (sets if step == "round" else 1)
        self.ex = [build_batched_executor(batch, tokens, seed0 + s, device, mix[0], mix[1], hq, hkv, page) for s in range(sets)]
        g = torch.Generator(device=device).manual_seed(5)
        self.q = torch.randn(batch, hq, D, generator=g, device=device).to(torch.bfloat16)
        self.k = torch.randn(batch, hkv, D, generator=g, device=device).to(torch.bfloat16)
        self.v = torch.randn(batch, hkv, D, generator=g, device=device).to(torch.bfloat16)
        self.stats = R.DynamicCacheStats()
        self.base = [(e.arenas.k_active, e.arenas.i2_active) for e in self.ex]
        self.step_graphs, self.flush_graphs = [], []
        # appending workloads start with the windows half full, so that flushes fall inside short runs too; the
        # static workload decodes against a full window
        for e in self.ex:
            for i in range(RING // 2 if append else RING):
                if append:
                    e(self.q, append=(self.k, self.v, tokens + i, tokens + i))
                    if batch == 1:
                        e.arenas.recent_len += 1     # a single-request caller advances the host mirror itself
                else:
                    R.append_generated_token(e.arenas, self.k if batch > 1 else self.k[0].unsqueeze(1),
                                             self.v if batch > 1 else self.v[0].unsqueeze(1),
                                             global_token_index=tokens + i, logical_position=tokens + i, stats=self.stats)
        torch.cuda.synchronize(device)
        for e in self.ex:
            gs, gf = torch.cuda.CUDAGraph(), torch.cuda.CUDAGraph()
            ring = e.arenas.recent_len
            with torch.cuda.graph(gs):
                self._visit(e)
            e.arenas.recent_len = ring                     # capture does not run the kernel
            if append:
                with torch.cuda.graph(gf):
                    e.arenas.recent_len = RING
                    R.flush_recent(e.arenas)
                # flushed tokens overwrite the same arena rows on every replay: the context stays at `tokens` + ring
                e.arenas.k_active, e.arenas.i2_active = self.base[len(self.step_graphs)]
                e.arenas.recent_len = ring
            self.step_graphs.append(gs)
            self.flush_graphs.append(gf if append else None)
        # one graph per round (a visit of every set, back to back): consecutive decode launches are joined by
        # programmatic dependent launch edges, as consecutive layers of a model are.  Large rounds are split into
        # graphs of at most 32 launches.
        rings = [e.arenas.recent_len for e in self.ex]
        self.round_graphs = []
        for lo in range(0, len(self.ex), 32):
            gr = torch.cuda.CUDAGraph()
            with torch.cuda.graph(gr):
                for e in self.ex[lo : lo + 32]:
                    self._visit(e)
            self.round_graphs.append(gr)
        for e, ring in zip(self.ex, rings):
            e.arenas.recent_len = ring
        # and one graph of several rounds (about as many launches as a model has layers), used while every
        # window has room for them: launches inside a graph are chained by programmatic dependent launch, two graph
        # replays are not
        self.chain_rounds = max(1, 32 // len(self.ex)) if append else max(1, 128 // len(self.ex))
        self.chain_graph = None
        if self.chain_rounds > 1:
            self.chain_graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(self.chain_graph):
                for _ in range(self.chain_rounds):
                    for e in self.ex:
                        self._visit(e)
            for e, ring in zip(self.ex, rings):
                e.arenas.recent_len = ring
        self.launches_per_visit = 1
        self.launches_per_flush = 3
        a = self.ex[0].arenas
        self.geom = (a.n_fp, a.n_i4, a.i2_active)

    def _visit(self, e):
        if self.append:
            e(self.q, append=(self.k, self.v, self.tokens, self.tokens))
            if self.batch == 1:
                e.arenas.recent_len += 1
        else:
            e(self.q)

    def visit_bytes(self, ring_len):
        return algorithmic_bytes(*self.geom, ring_len, self.batch, self.hq, self.hkv, self.append)

    def _account(self, a, t):
        """Host bookkeeping of one visit of set t: flush if the window is full; returns (bytes, flushed)."""
        flushed = 0
        if self.append and a.recent_len == RING:
            self.flush_graphs[t].replay()
            a.recent_len = 0
            flushed = 1
        ring_after = a.recent_len + (1 if self.append else 0)
        nbytes = self.visit_bytes(ring_after)
        if self.append:
            a.recent_len += 1
        return nbytes, flushed

    def run_graph_steps(self, steps, start=0):
        """Enqueue `steps` steps; returns (bytes moved, decode launches, flushes)."""
        total, flushes = 0, 0
        n = len(self.ex)
        i, end = start * self.visits_per_step, (start + steps) * self.visits_per_step
        while i < end:
            s = i % n
            whole_round = s == 0 and i + n <= end
            r = self.chain_rounds
            if whole_round and self.chain_graph is not None and i + r * n <= end and \
                    (not self.append or all(e.arenas.recent_len + r <= RING for e in self.ex)):
                for e in self.ex:      # r rounds without a flush: one replay of the chained graph
                    a = e.arenas
                    for _ in range(r):
                        total += self.visit_bytes(a.recent_len + (1 if self.append else 0))
                        if self.append:
                            a.recent_len += 1
                self.chain_graph.replay()
                i += r * n
                continue
            for t in (range(n) if whole_round else (s,)):
                nbytes, flushed = self._account(self.ex[t].arenas, t)
                total += nbytes
                flushes += flushed
            if whole_round:
                for gr in self.round_graphs:
                    gr.replay()
                i += n
            else:
                self.step_graphs[s].replay()
                i += 1
        return total, steps * self.visits_per_step, flushes

    def run_api_steps(self, steps, host_in, host_out, start=0, torch_copies=False):
        """Public operator call with host buffers, one call per visit (SplitKExecutor.step_host = r2k_decode_host):
        H2D of q/k/v from pinned memory, decode+append, D2H of the output, wait.  `torch_copies` issues the same
        visit as three torch calls around the device-tensor operator instead (timed beside it for comparison)."""
        total = 0
        nq, nk = self.q.numel(), self.k.numel()
        dev_in = self._dev_in
        first, last = start * self.visits_per_step, (start + steps) * self.visits_per_step
        for i in range(first, last):
            s = i % len(self.ex)
            e = self.ex[s]
            a = e.arenas
            if self.append and a.recent_len == RING:
                self.R.flush_recent(a)
                a.k_active, a.i2_active = self.base[s]
            total += self.visit_bytes(a.recent_len + (1 if self.append else 0))
            idx = (self.tokens + i, self.tokens + i) if self.append else None
            if not torch_copies:
                e.step_host(host_in, host_out, append_indices=idx)
                if self.append and self.batch == 1:
                    a.recent_len += 1
                continue
            dev_in.copy_(host_in, non_blocking=True)
            q = dev_in[:nq].view(self.batch, self.hq, D)
            if self.append:
                k = dev_in[nq : nq + nk].view(self.batch, self.hkv, D)
                v = dev_in[nq + nk :].view(self.batch, self.hkv, D)
                out = e(q, append=(k, v, idx[0], idx[1]))
                if self.batch == 1:
                    a.recent_len += 1
            else:
                out = e(q)
            host_out.copy_(out, non_blocking=True)
            torch.cuda.current_stream(self.device).synchronize()   # the caller reads the result
        return total

    def prepare_api(self):
        n = self.q.numel() + (2 * self.k.numel() if self.append else 0)
        host_in = torch.empty(n, dtype=torch.bfloat16).pin_memory()
        host_in[: self.q.numel()] = self.q.flatten().cpu()
        if self.append:
            host_in[self.q.numel() : self.q.numel() + self.k.numel()] = self.k.flatten().cpu()
            host_in[self.q.numel() + self.k.numel() :] = self.v.flatten().cpu()
        host_out = torch.empty(self.batch, self.hq, D, dtype=torch.bfloat16).pin_memory()
        self._dev_in = torch.empty(n, dtype=torch.bfloat16, device=self.device)
        return host_in, host_out

    def oracle_cache(self, s, b):
        """The oracle's cache of request b of set s in the state the benchmark has left the GPU cache in: the static
        pools as built (flushes of the benchmark overwrite rows outside the attended extent) plus a residual
        window of `recent_len` copies of the request's appended row."""
        from oracle import sspa_oracle as O
        seed = self.seed0 + s
        classes = page_classes(self.tokens // self.page, seed, self.mix[0], self.mix[1])
        key, value = synth_kv(self.tokens, seed * 1000 + b, self.device, hkv=self.hkv)
        cache = O.build_cache(key.cpu(), value.cpu(), classes, page_size=self.page, recent_capacity=RING, k_block=K_BLOCK,
                              v2_group=V2_GROUP, append_capacity=RING)
        k, v = self.k[b].cpu(), self.v[b].cpu()
        for i in range(self.ex[s].arenas.recent_len):
            O.append_token(cache, k, v, self.tokens + i, self.tokens + i)
        return cache

    def parity(self, requests=None, s=0):
        """One decode (no append) of set s on the benchmarked caches against the oracle, for the given requests."""
        from oracle import sspa_oracle as O
        e = self.ex[s]
        requests = sorted(set(requests if requests is not None else (0, self.batch - 1)))
        out = e.decode_f32(self.q).cpu()
        worst_abs, worst_excess = 0.0, -1.0
        for b in requests:
            want = O.decode_fp32(self.q[b : b + 1].float().cpu(), self.oracle_cache(s, b))
            err, excess = tolerance_excess(out[b : b + 1], want)
            worst_abs, worst_excess = max(worst_abs, err), max(worst_excess, excess)
        return {"ok": bool(worst_excess <= 0 and e.device_status() == 0), "max_abs_err": float(f"{worst_abs:.3e}"),
                "tolerance": f"max-abs {ATOL} + rel {RTOL}", "checked": f"requests {requests} of cache set {s} after the timed "
                f"regions ({self.tokens} tokens + {e.arenas.recent_len} residual), fp32 output against the CPU oracle"}


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


def sharded_1m(device, rank, world, steps, warmup, dist_on, check=True):
    """Sequence-sharded decode of a 1,048,576-token cache (INT4/INT2 value pages 50/50,
    128-token residual window on the last rank).  With more than one rank the merge is fused into the decode
    launch (peer stores over NVLink, r2k_decode_exchange); the all-gather + merge-launch variant is timed
    beside it for comparison.  Every variant's output is compared with the oracle: every rank runs the oracle's
    un-normalised state over its own shard on the host, the states are gathered and merged in rank order."""
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
    host_kv = (key.cpu(), value.cpu()) if check else None
    del key, value
    ex = R.prepare_splitk_executor(cache, R.allocate_splitk_workspace(cache, num_query_heads=HQ))
    g = torch.Generator(device=device).manual_seed(6)
    q = torch.randn(1, HQ, D, generator=g, device=device).to(torch.bfloat16)
    nk = None
    if rank == world - 1:
        st = R.DynamicCacheStats()
        nk = torch.randn(RING, HKV, 1, D, generator=g, device=device).to(torch.bfloat16)
        for i in range(RING):
            R.append_generated_token(cache, nk[i], nk[(i + 1) % RING], global_token_index=total + i,
                                     logical_position=total + i, stats=st)
    a = cache.arenas
    my_bytes = algorithmic_bytes(a.n_fp, a.n_i4, a.i2_active, a.recent_len, 1, append=False)

    def timed(one_step, steps, repeats=5):
        """(median us per step, graphed?, steps, spread) over `repeats` timed regions of `steps` steps; eight steps
        per CUDA graph, eager launches if capture is refused."""
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
        samples = []
        for _ in range(repeats):
            if graph is not None:
                steps = max(per_replay, steps // per_replay * per_replay)
                ms, _ = time_region(device, lambda: [graph.replay() for _ in range(steps // per_replay)], dist_on)
            else:
                ms, _ = time_region(device, lambda: [one_step() for _ in range(steps)], dist_on)
            samples.append(ms * 1e3 / steps)
        return statistics.median(samples), graph is not None, steps, spread(samples)

    nccl_us, fused_out, gathered_out, us_spread = None, None, None, None
    fused_error = None
    if world == 1:
        us, graphed, steps, us_spread = timed(lambda: ex(q), steps)
        fused_out = ex.decode_f32(q).clone()
    else:
        gathered = R.SequenceShardedExecutor(ex)
        local_us, _, _, _ = timed(lambda: ex.decode_state(q, out=gathered.state), steps)   # this rank's shard alone
        nccl_us, _, _, _ = timed(lambda: gathered(q), steps)
        gathered_out = gathered(q).clone()
        # the fused variant is the one reported; if it cannot be set up or times out on this box, every rank
        # agrees on that and the all-gather number is reported instead (with the reason)
        fused = None
        try:
            fused = R.SequenceShardedExecutor(ex, fused=True, device_step_counter=True)
            fused(q)                                   # one step first: a broken exchange shows up as a bounded
            probe = torch.tensor([float(ex.device_status())], device=device)   # wait here, not 300 times over
            dist.all_reduce(probe, op=dist.ReduceOp.MAX)
            if float(probe.item()) != 0.0:
                fused_error = "device-side timeout in the cross-rank wait"
            else:
                us, graphed, steps, us_spread = timed(lambda: fused(q), steps)
                fused_out = fused(q).clone()
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
            fused_out = None
    bytes_all = torch.tensor([float(my_bytes)], device=device, dtype=torch.float64)
    if dist_on:
        dist.all_reduce(bytes_all)
    out = {"workload": "sharded_1m_b1", "tokens": total, "n_gpus": world, "us_per_step": round(us, 2),
           "gbps": round(float(bytes_all.item()) / (us * 1e-6) / 1e9, 1), "steps": steps,
           "collective": "none" if world == 1 else "fused: tagged peer stores over NVLink inside the decode launch",
           "launches_per_step": 1, "cuda_graph": graphed}
    if us_spread is not None:
        out["us_per_step_spread"] = us_spread
    if nccl_us is not None:
        out["us_per_step_nccl_all_gather"] = round(nccl_us, 2)
        out["us_per_step_local_shard_only"] = round(local_us, 2)
        if fused_error:
            out.update(collective="nccl all_gather of [Hq,130] fp32 per rank", launches_per_step=2, fused_error=fused_error)
    if check:
        out["parity"] = sharded_parity(device, rank, world, dist_on, host_kv, classes, nk, total, q, fused_out, gathered_out)
    return out


def sharded_parity(device, rank, world, dist_on, host_kv, classes, nk, total, q, fused_out, gathered_out):
    """Every rank: the oracle's un-normalised (max, sum-exp, out) over its own shard, on the host; then one gather
    and the oracle's merge in rank order on every rank.  The GPU outputs (fused exchange, all-gather variant) are
    held against that, and against each other bit for bit."""
    import torch.distributed as dist
    from oracle import sspa_oracle as O
    torch.set_num_threads(max(1, (os.cpu_count() or 1) // max(world, 1)))
    per = host_kv[0].shape[1]
    shard = O.build_cache(host_kv[0], host_kv[1], classes, page_size=PAGE, recent_capacity=RING, k_block=K_BLOCK,
                          v2_group=V2_GROUP, append_capacity=RING)
    if nk is not None:
        rows = nk.cpu()
        for i in range(RING):
            O.append_token(shard, rows[i][:, 0], rows[(i + 1) % RING][:, 0], total + i, total + i)
    top, den, acc = O.decode_state(q.float().cpu(), shard, chunk=65536)
    state = torch.cat((top.unsqueeze(-1), den.unsqueeze(-1), acc), -1).contiguous().to(device)   # [1,Hq,130]
    states = torch.empty((world,) + tuple(state.shape), device=device)
    if dist_on:
        dist.all_gather_into_tensor(states, state)
    else:
        states[0] = state
    merged = None
    for s in states.cpu():
        part = (s[..., 0], s[..., 1], s[..., 2:])
        merged = part if merged is None else O.merge_state(merged, part)
    want = merged[2] / merged[1].unsqueeze(-1)
    res = {"tolerance": f"max-abs {ATOL} + rel {RTOL}",
           "checked": f"oracle state of every rank's shard ({per} tokens) on the host, gathered and merged in rank order"}
    flags = []
    for name, got in (("fused" if world > 1 else "decode", fused_out), ("all_gather", gathered_out)):
        if got is None:
            continue
        err, excess = tolerance_excess(got, want.to(torch.bfloat16) if got.dtype == torch.bfloat16 else want)
        res[f"{name}_max_abs_err"] = float(f"{err:.3e}")
        flags.append(excess <= 0)
    if fused_out is not None and gathered_out is not None:
        res["fused_equals_all_gather_bitwise"] = bool(torch.equal(fused_out.view(torch.int16), gathered_out.view(torch.int16)))
        flags.append(res["fused_equals_all_gather_bitwise"])
    ok = torch.tensor([1.0 if flags and all(flags) else 0.0], device=device)
    if dist_on:
        dist.all_reduce(ok, op=dist.ReduceOp.MIN)     # every rank holds the same output; all must agree
    res["ok"] = bool(ok.item() > 0)
    return res


# --------------------------------------------------------------------------- #
# CPU baselines
# --------------------------------------------------------------------------- #
class CpuRequest:
    """One request of a workload on the host: the reference's own CPU path (its torch quantisers, append/flush
    state machine and dequantise-then-attend decoder) when the reference is installed, else the oracle port."""

    def __init__(self, w, horizon_steps):
        self.w = w
        hq, hkv, tokens, page = w["hq"], w["hkv"], w["tokens"], w["page"]
        torch.set_num_threads(os.cpu_count() or 1)
        classes = page_classes(tokens // page, 11, w["mix"][0], w["mix"][1])
        key, value = synth_kv(tokens, 11000, "cpu", hkv=hkv)
        g = torch.Generator().manual_seed(5)
        self.nk = torch.randn(RING, hkv, D, generator=g).to(torch.bfloat16)
        self.q = torch.randn(1, hq, D, generator=g).to(torch.bfloat16)
        self.ns, self.why_port = load_reference()
        self.kind = "reference" if self.ns is not None else "port"
        # room for every flush of the run: the context grows by 128 tokens per flush
        room = RING * (horizon_steps // RING + 2)
        if self.ns is not None:
            ns = self.ns
            self.cache = ns.build_three_precision_cache(
                key, value, reference_plan(ns, classes, page, RING), page_size=page, key_quantization_superblock=K_BLOCK,
                int2_group_size=V2_GROUP, compact_key_append_capacity=room, recent_flush_size=RING)
            self.stats = ns.DynamicCacheStats()
        else:
            from oracle import sspa_oracle as O
            self.O = O
            self.cache = O.build_cache(key, value, classes, page_size=page, recent_capacity=RING, k_block=K_BLOCK,
                                       v2_group=V2_GROUP, append_capacity=room)
        self.i = 0
        for _ in range(RING // 2 if w["append"] else RING):
            self.append()

    def append(self):
        i, t = self.i, self.w["tokens"]
        k, v = self.nk[i % RING], self.nk[(i + 1) % RING]
        if self.ns is not None:
            self.ns.append_generated_token(self.cache, k.unsqueeze(1), v.unsqueeze(1), global_token_index=t + i,
                                           logical_position=t + i, stats=self.stats)
        else:
            self.O.append_token(self.cache, k, v, t + i, t + i)
        self.i += 1

    def step(self):
        """One decode step of the workload for this request; returns its algorithmic bytes."""
        if self.w["append"]:
            self.append()
        if self.ns is not None:
            self.ns.triton_mixed_reference(self.q, self.cache)
            c = self.cache
            n = (c.fp_pool.token_count, c.int4_pool.token_count, c.int2_pool.token_count, c.recent_fp_pool.token_count)
        else:
            self.O.decode(self.q, self.cache)
            c = self.cache
            n = (c.n_fp, c.n_i4, c.i2_active, c.recent_len)
        return algorithmic_bytes(n[0], n[1], n[2], n[3], 1, self.w["hq"], self.w["hkv"], self.w["append"])

    def describe(self):
        what = ("the reference's own CPU path (triton_mixed_reference + append_generated_token, imported unmodified)"
                if self.ns is not None else f"the oracle port ({self.why_port})")
        return what


def cpu_baseline_sample(w, seconds=12.0):
    """A bounded sample of the workload on the host cores: ONE request of one layer, all host threads."""
    req = CpuRequest(w, horizon_steps=4096)
    req.step()
    best, reps, t_end, nbytes = float("inf"), 0, time.perf_counter() + seconds, 0
    while (time.perf_counter() < t_end or reps < 3) and reps < 4000:
        t0 = time.perf_counter()
        nbytes = req.step()
        best = min(best, time.perf_counter() - t0)
        reps += 1
    return {"value": round(nbytes / best / 1e9, 3), "unit": "GB/s", "cores": torch.get_num_threads(), "kind": req.kind,
            "sample": f"1 of {w['batch']} requests of one layer ({w['tokens']} tokens, same page mix), best of {reps} "
                      f"decode{'+append' if w['append'] else ''} steps, {best * 1e3:.2f} ms per request-step; {req.describe()}"}


def run_reference_arm(args):
    """The reference's CPU implementation of the path on the host cores (imported unmodified from baseline/_ref
    when it is installed there, else the oracle port), all host threads, one request per step."""
    rank = int(os.environ.get("RANK", "0"))
    if rank != 0:
        return
    w = WORKLOADS[args.workload]
    steps = min(args.steps, 200)
    req = CpuRequest(w, horizon_steps=steps + 16)
    for _ in range(max(1, min(args.warmup, 3))):
        req.step()
    t0 = time.perf_counter()
    nbytes = sum(req.step() for _ in range(steps))
    sec = time.perf_counter() - t0
    value = round(nbytes / sec / 1e9, 3)
    sample = (f"one of the {w['batch']} requests of one layer per step ({w['tokens']} tokens, same page mix), decode"
              f"{' + one-token append, flush when the residual window fills' if w['append'] else ''}; {req.describe()}")
    line = {
        "impl": "reference", "metric": METRIC, "value": value, "unit": "GB/s", "n_gpus": args.gpus, "steps": steps,
        "warmup": args.warmup, "ms_per_step": round(sec * 1e3 / steps, 3), "higher_is_better": True, "scaling": "weak",
        "vs_baseline": None, "dtype": "f32 (dequantise-then-attend on the host)", "data": "synthetic",
        "config": {"workload": args.workload, "sample": f"one request ({w['tokens']} tokens) per step",
                   "heads": f"{w['hq']}q/{w['hkv']}kv x128"},
        "cpu_baseline": {"value": value, "unit": "GB/s", "cores": torch.get_num_threads(), "kind": req.kind, "sample": sample},
        "e2e": {"value": value, "unit": "GB/s", "h2d_bytes_per_step": 0, "d2h_bytes_per_step": 0},
    }
    print(json.dumps(line))


# --------------------------------------------------------------------------- #
# the reference's Triton decoder on this GPU
# --------------------------------------------------------------------------- #
def triton_reference_record(device, bench, steps=200, sets=3):
    """The reference's fused split-K decoder (Triton, JIT-compiled for this GPU) on the benchmark's workload, built
    from the same seeds through the reference's own build_three_precision_cache -> allocate_splitk_workspace ->
    prepare_splitk_executor -> stack_homogeneous_splitk_executors, launch policy as its attention manager
    chooses it (block_n 64 beyond 6144 tokens, fp16 partials, hierarchical reduce), CUDA events around `steps`
    eager steps over `sets` cache sets; plus the largest difference between its output and this library's on the
    same state.  Any failure to import, compile or run is recorded as text instead."""
    ns, why = load_reference()
    if ns is None:
        return {"unavailable": why}
    try:
        from r2omni.sspa.kernels import triton_fourq_splitk as T
        w = dict(hq=bench.hq, hkv=bench.hkv, batch=bench.batch, tokens=bench.tokens, page=bench.page, mix=bench.mix)
        block_n = 64 if w["tokens"] > 6144 else 128
        stacked = []
        t_build = time.perf_counter()
        for s in range(sets):
            seed = bench.seed0 + s
            classes = page_classes(w["tokens"] // w["page"], seed, w["mix"][0], w["mix"][1])
            singles = []
            for b in range(w["batch"]):
                key, value = synth_kv(w["tokens"], seed * 1000 + b, device, hkv=w["hkv"])
                cache = ns.build_three_precision_cache(
                    key, value, reference_plan(ns, classes, w["page"], RING, device), page_size=w["page"],
                    key_quantization_superblock=K_BLOCK, int2_group_size=V2_GROUP, compact_key_append_capacity=RING,
                    recent_flush_size=RING)
                ws = T.allocate_splitk_workspace(cache, block_n=block_n, num_query_heads=w["hq"],
                                                 partial_output_dtype=torch.float16, hierarchical_group_blocks=64)
                singles.append(T.prepare_splitk_executor(
                    cache, ws, block_n=block_n, num_warps=8, num_stages=1, reduce_num_warps=8 if block_n == 64 else 4,
                    broadcast_k_metadata=True, use_tensor_cores_qk=True, use_tensor_cores_pv=False, output_hadamard=False,
                    hierarchical_reduce=True))
                del key, value
            if s == 0:
                probe = singles[0]       # request 0 alone: decoded by both libraries from the very same tensors below
            stacked.append(T.stack_homogeneous_splitk_executors(singles) if w["batch"] > 1 else singles[0])
            del singles
        build_s = time.perf_counter() - t_build
        q, k, v = bench.q, bench.k, bench.v
        ring_target = bench.ex[0].arenas.recent_len     # bring set 0 to the state this library's set 0 is in
        for s, ex in enumerate(stacked):
            for i in range(ring_target if s == 0 else RING // 2):
                ex(q, append=(k, v, w["tokens"] + i, w["tokens"] + i))
        torch.cuda.synchronize(device)
        theirs = stacked[0](q).float().clone()
        ours = bench.ex[0](q).float().clone()
        diff = float((theirs - ours).abs().max())
        # the same bytes through both decoders: this library adopts the reference-built cache of request 0 in place
        import r2omni_b200 as R
        adopted = R.adopt_reference_cache(probe.cache)
        mine = R.prepare_splitk_executor(adopted, R.allocate_splitk_workspace(adopted, num_query_heads=w["hq"]))
        q0 = q[0:1].contiguous()
        same_cache_diff = float((probe(q0).float() - mine(q0).float()).abs().max())
        oracle_diff = float((ns.triton_mixed_reference(q0, probe.cache).float() - mine(q0).float()).abs().max())
        # timed: decode without append (the window of a set would fill after 64 steps and the reference must then
        # be unstacked to flush); the appended row is 0.5 % of the traffic
        for _ in range(3):
            for ex in stacked:
                ex(q)
        torch.cuda.synchronize(device)
        e0, e1 = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        samples = []
        for _ in range(5):
            e0.record()
            for i in range(steps):
                stacked[i % sets](q)
            e1.record()
            torch.cuda.synchronize(device)
            samples.append(e0.elapsed_time(e1) * 1e3 / steps)
        us = statistics.median(samples)
        # the same calls captured into one CUDA graph (takes the Python launch path out of the measurement), if
        # the reference's call can be captured at all
        graph_us, graph_note = None, None
        try:
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                for ex in stacked:
                    ex(q)
            graph.replay()
            torch.cuda.synchronize(device)
            gs = []
            for _ in range(5):
                e0.record()
                for i in range(max(1, steps // sets)):
                    graph.replay()
                e1.record()
                torch.cuda.synchronize(device)
                gs.append(e0.elapsed_time(e1) * 1e3 / (max(1, steps // sets) * sets))
            graph_us = statistics.median(gs)
        except Exception as exc:  # noqa: BLE001
            graph_note = f"not capturable: {exc!r}"[:200]
            torch.cuda.synchronize(device)
        a = bench.ex[0].arenas
        nbytes = algorithmic_bytes(a.n_fp, a.n_i4, a.i2_active, RING // 2, w["batch"], w["hq"], w["hkv"], append=False)
        import triton
        best = min(us, graph_us) if graph_us is not None else us
        return {"us_per_step": round(best, 2), "us_per_step_eager": round(us, 2), "us_per_step_spread_eager": spread(samples),
                "us_per_step_cuda_graph": None if graph_us is None else round(graph_us, 2), "cuda_graph_note": graph_note,
                "gbps": round(nbytes / (best * 1e-6) / 1e9, 1),
                "launches_per_step": 3, "block_n": block_n, "triton": triton.__version__, "cache_sets": sets,
                "max_abs_diff_same_cache": float(f"{same_cache_diff:.3e}"),
                "max_abs_diff_same_cache_vs_reference_torch_decoder": float(f"{oracle_diff:.3e}"),
                "max_abs_diff_own_caches": float(f"{diff:.3e}"),
                "diff_note": "same_cache: request 0 of the reference-built cache decoded by the reference's Triton kernel and, "
                             "adopted in place, by this library (bf16 outputs).  own_caches: each library decoding the cache it "
                             "packed itself; the reference's Triton pack kernels break rounding ties differently from its "
                             "torch pack routine (which this library reproduces bit for bit), so the two caches differ",
                "steps": steps, "build_seconds": round(build_s, 1),
                "what": "reference SplitKExecutor.__call__ (stacked batch, no append) on the same seeded caches, eager "
                        "launches from Python and replayed from a CUDA graph; this library's comparable figure is "
                        "roofline.us_per_launch_isolated"}
    except Exception as exc:  # noqa: BLE001 -- the record of the failure is the deliverable
        import traceback
        return {"error": repr(exc)[:400], "where": traceback.format_exc().strip().splitlines()[-3:]}


# --------------------------------------------------------------------------- #
# greedy decode of a random-weight thinker with the packed-KV attention in the loop
# --------------------------------------------------------------------------- #
THINKER = dict(layers=36, hidden=2048, hq=16, hkv=2, mlp=11008, vocab=151936, theta=1.0e6, batch=32, tokens=16384,
               new_tokens=256, page=64, mix=(0.25, 0.5))


class SyntheticThinker:
    """A Qwen2.5-Omni-3B-shaped text decoder with random weights (~N(0, 0.02), bf16): RMSNorm, q/k/v projections
    with bias (one GEMM), multimodal RoPE (text positions: the three axes agree), packed-KV attention through
    PackedKVAttentionManager (kernel_backend "cuda_sm100"), output projection, SwiGLU MLP; final norm, LM head,
    argmax.  Every layer's cache holds `tokens` prefilled tokens per request, packed from random bf16
    activations with seeded page precisions.  One decode step is captured into a CUDA graph: token ids,
    positions and append indices live on the device and are advanced inside the graph."""

    def __init__(self, device, cfg):
        import types

        import r2omni_b200 as R
        from gpu_helpers import make_plan
        self.R, self.device, self.cfg = R, device, cfg
        c = cfg
        g = torch.Generator(device=device).manual_seed(1234)
        def w(*shape):
            return (torch.randn(*shape, generator=g, device=device) * 0.02).to(torch.bfloat16)
        def linear(n_in, n_out, bias):
            layer = torch.nn.Linear(n_in, n_out, bias=bias, device=device, dtype=torch.bfloat16)
            with torch.no_grad():
                layer.weight.copy_(w(n_out, n_in))
                if bias:
                    layer.bias.copy_(w(n_out))
            return layer
        self.embed, self.lm_head = w(c["vocab"], c["hidden"]), w(c["vocab"], c["hidden"])
        self.final_norm = torch.ones(c["hidden"], device=device, dtype=torch.bfloat16)
        self.manager = R.PackedKVAttentionManager(num_query_heads=c["hq"], mrope_section=(16, 24, 24), device_positions=True)
        self.layers = []
        t_build = time.perf_counter()
        for l in range(c["layers"]):
            # query, key and value projections as one GEMM: the manager hands its output to the one-launch prologue
            attn = types.SimpleNamespace(
                head_dim=128, qkv_proj=linear(c["hidden"], (c["hq"] + 2 * c["hkv"]) * 128, True),
                o_proj=linear(c["hq"] * 128, c["hidden"], False))
            self.layers.append(types.SimpleNamespace(
                attn=attn, ln1=torch.ones(c["hidden"], device=device, dtype=torch.bfloat16),
                ln2=torch.ones(c["hidden"], device=device, dtype=torch.bfloat16),
                gate_up=linear(c["hidden"], 2 * c["mlp"], False),    # gate and up projections as one GEMM
                down=linear(c["mlp"], c["hidden"], False)))
            classes = page_classes(c["tokens"] // c["page"], 300 + l, c["mix"][0], c["mix"][1])
            caches = []
            for b in range(c["batch"]):
                key, value = synth_kv(c["tokens"], (300 + l) * 1000 + b, device, hkv=c["hkv"])
                caches.append(R.build_three_precision_cache(
                    key, value, make_plan(classes, c["page"], RING), page_size=c["page"], key_quantization_superblock=K_BLOCK,
                    int2_group_size=V2_GROUP, compact_key_append_capacity=RING * (c["new_tokens"] // RING + 2),
                    recent_flush_size=RING))
                del key, value
            self.manager.adopt_layer(l, caches, c["tokens"])
            del caches
        self.build_seconds = time.perf_counter() - t_build
        B = c["batch"]
        self.inv_freq = 1.0 / (c["theta"] ** (torch.arange(0, 128, 2, device=device, dtype=torch.float32) / 128.0))
        self.tok = torch.randint(0, c["vocab"], (B,), generator=g, device=device)
        self.pos = torch.full((B,), float(c["tokens"]), device=device, dtype=torch.float32)
        self.idx = torch.full((B, 2), c["tokens"], device=device, dtype=torch.int64)
        self.graphs, self.phase = [], 0

    def _step(self):
        """One decode step on the current stream; advances tok / pos / idx on the device."""
        c, F = self.cfg, torch.nn.functional
        B = c["batch"]
        x = self.embed[self.tok].view(B, 1, c["hidden"])
        angle = self.pos[:, None] * self.inv_freq[None, :]
        emb = torch.cat((angle, angle), dim=-1)                       # [B,128]
        cos = emb.cos().view(1, B, 1, 128).expand(3, B, 1, 128)
        sin = emb.sin().view(1, B, 1, 128).expand(3, B, 1, 128)
        for l, layer in enumerate(self.layers):
            h = F.rms_norm(x, (c["hidden"],), layer.ln1, 1e-6)
            x = x + self.manager.active_forward(l, layer.attn, h, (cos, sin), append_indices=self.idx)
            h = F.rms_norm(x, (c["hidden"],), layer.ln2, 1e-6)
            gate, up = layer.gate_up(h).chunk(2, dim=-1)
            x = x + layer.down(F.silu(gate) * up)
        h = F.rms_norm(x, (c["hidden"],), self.final_norm, 1e-6)
        logits = h.view(B, c["hidden"]) @ self.lm_head.t()
        self.tok.copy_(logits.argmax(dim=-1))
        self.pos.add_(1.0)
        self.idx.add_(1)

    def _host_mirrors(self):
        return [(s.original_seq_len, s.append_count, s.last_cache_position, s.calls, s.kernel_calls,
                 s.dynamic_stats.appended_tokens, s.fourq_executor.arenas.recent_len) for s in self.manager._states.values()]

    def capture(self, phases):
        """Capture one decode step per cache geometry: the launch geometry is part of a captured graph, and every
        flush moves 128 tokens per request from the residual window into the INT2-value pool, so phase k (after k
        flushes) gets its own graph, captured ahead of time with the pool extents it will have.  The host-side
        bookkeeping a step does runs once per capture and is undone; `advance` redoes it after every replay."""
        for _ in range(2):      # eager steps first: library handles, workspaces
            self.flush_if_needed()
            self._step()
        torch.cuda.synchronize(self.device)
        self.flush_if_needed()
        self.graphs, self.phase = [], 0
        arenas = [s.fourq_executor.arenas for s in self.manager._states.values()]
        base = [(a.k_active, a.i2_active) for a in arenas]
        for k in range(phases):
            before = self._host_mirrors()
            for a, (ka, ia) in zip(arenas, base):
                a.k_active, a.i2_active = ka + RING * k, ia + RING * k
            graph = torch.cuda.CUDAGraph()
            with torch.cuda.graph(graph):
                self._step()
            self.graphs.append(graph)
            for s, m in zip(self.manager._states.values(), before):
                (s.original_seq_len, s.append_count, s.last_cache_position, s.calls, s.kernel_calls,
                 s.dynamic_stats.appended_tokens, s.fourq_executor.arenas.recent_len) = m
        for a, (ka, ia) in zip(arenas, base):
            a.k_active, a.i2_active = ka, ia

    def advance(self):
        for s in self.manager._states.values():
            s.last_cache_position = s.original_seq_len
            s.original_seq_len += 1
            s.append_count += 1
            s.calls += 1
            s.kernel_calls += 1
            s.dynamic_stats.appended_tokens += 1
            s.fourq_executor.arenas.recent_len += 1

    def flush_if_needed(self):
        return sum(1 for l in range(len(self.layers)) if self.manager.flush_if_full(l))

    def generate(self, steps, host_loop=False, host_tok=None):
        """`steps` replays of the captured step (flushes of full residual windows in between).  host_loop: the token
        ids go through pinned host memory every step, as a serving loop with a host-side sampler / stop check does."""
        flushes = 0
        for _ in range(steps):
            flushed = self.flush_if_needed()
            if flushed:
                flushes += flushed
                self.phase += 1
            if host_loop:
                self.tok.copy_(host_tok, non_blocking=True)
            self.graphs[self.phase].replay()
            self.advance()
            if host_loop:
                host_tok.copy_(self.tok, non_blocking=True)
                torch.cuda.current_stream(self.device).synchronize()
        return flushes


def run_thinker(args):
    import torch.distributed as dist
    rank, world = int(os.environ.get("RANK", "0")), int(os.environ.get("WORLD_SIZE", "1"))
    local = int(os.environ.get("LOCAL_RANK", "0"))
    device = torch.device("cuda", local)
    torch.cuda.set_device(device)
    dist_on = world > 1
    if dist_on:
        dist.init_process_group("nccl", device_id=device)
    from r2omni_b200 import _lib as L
    L.lib()
    cfg = dict(THINKER)
    steps = args.steps if args.steps else cfg["new_tokens"]
    model = SyntheticThinker(device, cfg)
    warm = max(3, min(args.warmup, 8))
    model.capture(phases=(warm + steps + min(steps, 64) + 4) // RING + 2)
    model.generate(warm)
    with ClockSampler(local) as clocks:
        ms, flushes = time_region(device, lambda: model.generate(steps), dist_on)
    tokens_per_s = cfg["batch"] * steps * world / (ms * 1e-3)
    host_tok = torch.empty(cfg["batch"], dtype=torch.int64).pin_memory()
    host_tok.copy_(model.tok)
    e_steps = min(steps, 64)
    e_ms, _ = time_region(device, lambda: model.generate(e_steps, host_loop=True, host_tok=host_tok), dist_on)
    a = model.manager._states[0].fourq_executor.arenas
    kv_bytes = cfg["layers"] * algorithmic_bytes(a.n_fp, a.n_i4, a.i2_active, RING // 2, cfg["batch"], cfg["hq"], cfg["hkv"], True)
    per_layer = cfg["hidden"] * (cfg["hq"] + 2 * cfg["hkv"]) * 128 + cfg["hq"] * 128 * cfg["hidden"] + 3 * cfg["hidden"] * cfg["mlp"]
    weight_bytes = 2 * (cfg["layers"] * per_layer + cfg["vocab"] * cfg["hidden"])
    peak, peak_kind = measured_peak_gbs()
    if rank == 0:
        line = {
            "metric": "greedy_decode_tokens_per_s", "value": round(tokens_per_s, 1), "unit": "tokens/s", "n_gpus": world,
            "steps": steps, "warmup": warm, "ms_per_step": round(ms / steps, 4), "higher_is_better": True, "scaling": "weak",
            "vs_baseline": None, "dtype": "bf16 weights and activations; packed INT4 keys, bf16/INT4/INT2 value pages",
            "data": "synthetic",
            "config": {"workload": "thinker_3b_b32", "layers": cfg["layers"], "hidden": cfg["hidden"], "heads": "16q/2kv x128",
                       "mlp": cfg["mlp"], "vocab": cfg["vocab"], "rope_theta": cfg["theta"], "batch_per_gpu": cfg["batch"],
                       "prefilled_tokens": cfg["tokens"], "generated_tokens": steps,
                       "pages": "64 tokens; bf16/INT4/INT2 = 25,50,25 % from a seed", "weights": "random ~N(0, 0.02), bf16",
                       "attention": "PackedKVAttentionManager, kernel_backend cuda_sm100: fused mRoPE launch + one decode launch "
                                    "with fused append per layer; flush of all layers every 128 steps",
                       "step": "one CUDA-graph replay (36 layers, LM head, argmax); token ids, positions and append "
                               "indices advance on the device", "l2": "7 GB of caches + 6.7 GB of weights per step (larger than L2)",
                       "parallelism": f"{world} independent replicas" if world > 1 else "1 GPU"},
            "gpu_launches": int(steps * cfg["layers"] * 2 + flushes * 3),
            "flushes_in_region": int(flushes),
            "roofline": {"bound": "hbm", "kernel": "whole decode step (attention + GEMV-like projections)",
                         "achieved": round((kv_bytes + weight_bytes) / (ms / steps * 1e-3) / 1e9, 1), "peak": peak,
                         "peak_source": peak_kind, "unit": "GB/s",
                         "frac": round((kv_bytes + weight_bytes) / (ms / steps * 1e-3) / 1e9 / peak, 4),
                         "bytes_per_step": {"packed_kv": int(kv_bytes), "weights": int(weight_bytes)}, "traffic": None},
            "e2e": {"value": round(cfg["batch"] * e_steps * world / (e_ms * 1e-3), 1), "unit": "tokens/s",
                    "ms_per_step": round(e_ms / e_steps, 4), "steps": e_steps,
                    "h2d_bytes_per_step": cfg["batch"] * 8, "d2h_bytes_per_step": cfg["batch"] * 8,
                    "call": "token ids from pinned host memory in, graph replay, sampled ids back to the host, stream wait"},
            "build_seconds": round(model.build_seconds, 1), "clocks": clocks.summary(),
            "stats_layer0": model.manager.get_stats()[0],
        }
        print(json.dumps(line))
    if dist_on:
        dist.destroy_process_group()


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=None)
    ap.add_argument("--warmup", type=int, default=16)
    ap.add_argument("--impl", default="ours", choices=["ours", "reference"])
    ap.add_argument("--workload", default="decode_32k_b8", choices=sorted(WORKLOADS) + ["thinker_3b_b32"])
    ap.add_argument("--no-cpu-baseline", action="store_true")
    ap.add_argument("--no-sharded", action="store_true")
    ap.add_argument("--no-e2e", action="store_true")
    ap.add_argument("--no-parity", action="store_true")
    ap.add_argument("--no-triton-reference", action="store_true")
    ap.add_argument("--page-mix", default=None, help="percent of bf16,INT4,INT2 value pages (kernel studies)")
    args = ap.parse_args()
    if args.workload == "thinker_3b_b32":
        if args.impl == "reference":
            args.workload = "decode_32k_b8"      # the CPU arm times the attention path, whatever drives it
        else:
            run_thinker(args)
            return
    w = dict(WORKLOADS[args.workload])
    if args.steps is None:
        args.steps = {"decode_7b_28l": 256, "decode_3b_36l": 256, "decode_4k_b1": 16384}.get(args.workload, 8192)
    if args.page_mix is not None:
        mix = [float(x) / 100.0 for x in args.page_mix.split(",")]
        w["mix"] = (mix[0], mix[1])
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
    default_workload = args.workload == "decode_32k_b8" and args.page_mix is None
    bench = ReplicaBench(device, hq=w["hq"], hkv=w["hkv"], batch=w["batch"], tokens=w["tokens"], sets=w["sets"],
                         page=w["page"], mix=w["mix"], step=w["step"], append=w["append"])
    n_sets, vps = len(bench.ex), bench.visits_per_step
    bench.run_graph_steps(warmup)
    with ClockSampler(local) as clocks:
        ms, (nbytes, decodes, flushes) = time_region(device, lambda: bench.run_graph_steps(args.steps, start=warmup), dist_on)
    value = nbytes * world / (ms * 1e-3) / 1e9
    gpu_launches = decodes * bench.launches_per_visit + flushes * bench.launches_per_flush

    # the decode kernel alone: same graphs, no flush in the window
    probe_visits = 0
    rounds = 32 if w["append"] else 8      # visits of every set inside the window (it must fit the residual window)
    rounds = max(bench.chain_rounds, rounds // bench.chain_rounds * bench.chain_rounds)
    def make_room():
        if not w["append"]:
            return
        for s, e in enumerate(bench.ex):
            if e.arenas.recent_len > RING - rounds - 1:
                bench.flush_graphs[s].replay()
                e.arenas.recent_len = 0
    def decode_only(whole_rounds=True):
        nonlocal probe_visits
        b = 0
        for r in range(rounds):
            for e in bench.ex:
                b += bench.visit_bytes(e.arenas.recent_len + (1 if w["append"] else 0))
                if w["append"]:
                    e.arenas.recent_len += 1
                probe_visits += 1
            if not whole_rounds:
                for g in bench.step_graphs:
                    g.replay()
            elif bench.chain_graph is None:
                for gr in bench.round_graphs:
                    gr.replay()
            elif (r + 1) % bench.chain_rounds == 0:
                bench.chain_graph.replay()
        return b
    # launches separated by graph boundaries (no overlap between consecutive launches), for comparison
    make_room()
    iso_ms, _ = time_region(device, lambda: decode_only(False), dist_on)
    iso_us = iso_ms * 1e3 / max(probe_visits, 1)
    probe_visits = 0
    make_room()
    k_ms, k_bytes = time_region(device, decode_only, dist_on)
    peak, peak_kind = measured_peak_gbs()
    achieved = k_bytes / (k_ms * 1e-3) / 1e9
    roofline = {"bound": "hbm", "kernel": "decode_kernel<bf16>", "achieved": round(achieved, 1), "peak": peak,
                "peak_source": peak_kind, "unit": "GB/s", "frac": round(achieved / peak, 4),
                "frac_of_nominal_8000": round(achieved / 8000.0, 4), "us_per_launch": round(k_ms * 1e3 / max(probe_visits, 1), 2),
                "us_per_launch_isolated": round(iso_us, 2),
                "bytes_per_launch": int(k_bytes / max(probe_visits, 1)),
                "traffic": NCU_DRAM_BYTES_PER_LAUNCH if default_workload else None}

    # the flush alone (quantize-and-pack of the 128-token residual window: 3 launches, launch-bound)
    flush = None
    if w["append"]:
        def flush_only():
            for r in range(8):
                for s_, e in enumerate(bench.ex):
                    bench.flush_graphs[s_].replay()
                    e.arenas.recent_len = 0
        f_ms, _ = time_region(device, flush_only, dist_on)
        flush = {"us_per_flush": round(f_ms * 1e3 / (8 * n_sets), 2), "launches": bench.launches_per_flush,
                 "amortised_us_per_step": round(f_ms * 1e3 / (8 * n_sets) / RING * vps, 3)}

    # end to end through the operator call with host buffers
    e2e = None
    if not args.no_e2e:
        host_in, host_out = bench.prepare_api()
        bench.run_api_steps(max(1, warmup // vps), host_in, host_out)
        e2e_steps = max(1, min(args.steps, 512 // vps))
        cursor = warmup
        samples, e_bytes_ms = [], []
        for _ in range(5):
            e_ms, e_bytes = time_region(device, lambda: bench.run_api_steps(e2e_steps, host_in, host_out, start=cursor), dist_on)
            cursor += e2e_steps
            samples.append(e_ms * 1e3 / e2e_steps)
            e_bytes_ms.append(e_bytes / (e_ms * 1e-3))
        e_us = statistics.median(samples)
        e2e = {"value": round(statistics.median(e_bytes_ms) * world / 1e9, 1), "unit": "GB/s",
               "us_per_step": round(e_us, 2), "us_per_step_spread": spread(samples), "steps": e2e_steps,
               "h2d_bytes_per_step": int(host_in.numel() * 2 * vps), "d2h_bytes_per_step": int(host_out.numel() * 2 * vps),
               "call": "SplitKExecutor.step_host (r2k_decode_host), one call per launch: H2D copy kernel from the pinned block, "
                       "decode+append writing the pinned result over PCIe, stream wait"}
        t_steps = max(1, min(e2e_steps, 256 // vps))
        t_ms, _ = time_region(device, lambda: bench.run_api_steps(t_steps, host_in, host_out, start=cursor, torch_copies=True),
                              dist_on)
        e2e["us_per_step_three_torch_calls"] = round(t_ms * 1e3 / t_steps, 2)

    parity = None
    if not args.no_parity:
        ok_local = bench.parity()
        flag = torch.tensor([1.0 if ok_local["ok"] else 0.0], device=device)
        if dist_on:
            dist.all_reduce(flag, op=dist.ReduceOp.MIN)
            ok_local["ok"] = bool(flag.item() > 0)
            ok_local["checked"] += "; every rank checks its own replica"
        parity = ok_local

    triton_ref = None
    if rank == 0 and world == 1 and not args.no_triton_reference and args.workload in ("decode_32k_b8", "small"):
        triton_ref = triton_reference_record(device, bench)

    config_note = bench_bytes_note(w)
    chain_launches = bench.chain_rounds * n_sets
    set_mb = bench.visit_bytes(RING) / 1e6
    del bench
    torch.cuda.empty_cache()

    sharded = None if args.no_sharded or args.workload != "decode_32k_b8" else \
        sharded_1m(device, rank, world, steps=min(args.steps, 256), warmup=warmup, dist_on=dist_on, check=not args.no_parity)
    cpu = None
    if rank == 0 and world == 1 and not args.no_cpu_baseline:
        cpu = cpu_baseline_sample(w)

    if rank == 0:
        mix_pct = ",".join(str(int(round(100 * x))) for x in (w["mix"][0], w["mix"][1], 1.0 - w["mix"][0] - w["mix"][1]))
        line = {
            "metric": METRIC, "value": round(value, 1), "unit": "GB/s", "n_gpus": world, "steps": args.steps, "warmup": warmup,
            "ms_per_step": round(ms / args.steps, 5), "us_per_step": round(ms * 1e3 / args.steps, 2), "higher_is_better": True,
            "scaling": "weak", "vs_baseline": None, "dtype": "f16 tensor-core products, f32 accumulation (u4/u2 codes, bf16 pages)",
            "data": "synthetic",
            "config": {"workload": args.workload, "batch_per_gpu": w["batch"], "tokens_per_request": w["tokens"],
                       "heads": f"{w['hq']}q/{w['hkv']}kv x128", "layers": n_sets if w["step"] == "round" else 1,
                       "pages": f"{w['page']} tokens; bf16/INT4/INT2 = {mix_pct} % from a seed",
                       "keys": "INT4 per channel, 32-token blocks",
                       "residual_window": RING, "append_per_step": 1 if w["append"] else 0,
                       "flush_every": RING if w["append"] else None,
                       "step": "one decode launch" if vps == 1 else f"{vps} decode launches (all layers)",
                       "l2": f"{n_sets} cache sets of ~{set_mb:.1f} MB visited in order (inputs larger than L2)",
                       "graphs": f"{chain_launches} decode launches per CUDA-graph replay, chained by programmatic dependent launch",
                       "parallelism": f"{world} independent replicas" if world > 1 else "1 GPU",
                       "step_bytes": config_note},
            "gpu_launches": int(gpu_launches), "flushes_in_region": int(flushes),
            "flush": flush, "roofline": roofline, "e2e": e2e, "parity": parity, "clocks": clocks.summary(),
        }
        if cpu is not None:
            line["cpu_baseline"] = cpu
        if triton_ref is not None:
            line["triton_reference"] = triton_ref
        if sharded is not None:
            line["seq_sharded"] = sharded
        print(json.dumps(line))
    if dist_on:
        dist.destroy_process_group()


def bench_bytes_note(w):
    return (f"sum over {w['batch']} requests x {w['hkv']} kv heads of 76 B/token keys + 256/68/44 B/token values + "
            "512 B/residual token" + (f", x {w['sets']} layers per step" if w["step"] == "round" else ""))


if __name__ == "__main__":
    main()
