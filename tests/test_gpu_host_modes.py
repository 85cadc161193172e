"""The host-buffer decode call under each of its transfer modes, and the library with programmatic dependent launch
turned off.  Both switches are environment variables that the library reads once, so every mode runs in a child
process: the same seeded steps, bitwise the same results as the default mode and oracle parity."""
import os
import subprocess
import sys

import pytest

pytestmark = pytest.mark.gpu

ROOT = os.path.dirname(os.path.dirname(os.path.abspath(__file__)))

CHILD = r"""
import hashlib, sys, os
root = sys.argv[1]
sys.path.insert(0, root); sys.path.insert(0, os.path.join(root, "tests")); sys.path.insert(0, os.path.join(root, "tests", "golden"))
import torch
import r2omni_b200 as R
from gpu_helpers import assert_close, build_gpu_cache, make_executor
from oracle import sspa_oracle as O
from recipe import make_inputs

hq, hkv, s, steps = 16, 2, 20 * 64, 132            # 132 steps: through a flush of the full residual window
r = torch.rand(20, generator=torch.Generator().manual_seed(9))
classes = torch.tensor([1 if x < 0.25 else 2 if x < 0.75 else 5 for x in r.tolist()])
key, value, new_k, new_v, queries = make_inputs(seed=123, hq=hq, hkv=hkv, tokens=s, appends=steps, n_queries=steps)
ocache = O.build_cache(key, value, classes, page_size=64, append_capacity=256)
gcache = build_gpu_cache(key, value, classes, page_size=64, append_capacity=256)
ex = make_executor(gcache, hq)
host_in = torch.empty(hq * 128 + 2 * hkv * 128, dtype=torch.bfloat16).pin_memory()
host_out = torch.empty(1, hq, 128, dtype=torch.bfloat16).pin_memory()
digest = hashlib.sha256()
stats = R.DynamicCacheStats()
for i in range(steps):
    q = queries[i].reshape(1, hq, 128)
    ring = gcache.recent_fp_pool
    if ring.active_length == ring.capacity:      # full: flush and append on the device, then a step without append
        R.append_generated_token(gcache, new_k[i].cuda().unsqueeze(1), new_v[i].cuda().unsqueeze(1),
                                 global_token_index=s + i, logical_position=s + i, stats=stats)
        host_in[: hq * 128] = q.flatten()
        got = ex.step_host(host_in, host_out)
    else:
        host_in[: hq * 128] = q.flatten()
        host_in[hq * 128 : hq * 128 + hkv * 128] = new_k[i].flatten()
        host_in[hq * 128 + hkv * 128 :] = new_v[i].flatten()
        got = ex.step_host(host_in, host_out, append_indices=(s + i, s + i))
        ring.active_length += 1
    O.append_token(ocache, new_k[i], new_v[i], s + i, s + i)
    digest.update(got.view(torch.int16).numpy().tobytes())
    if i % 40 == 0 or i >= steps - 3:
        assert_close(got.float(), O.decode_fp32(q.float(), ocache), f"step {i}")
assert ex.device_status() == 0
print("DIGEST", digest.hexdigest())
"""


def run_child(extra_env):
    env = dict(os.environ)
    env.update(extra_env)
    out = subprocess.run([sys.executable, "-c", CHILD, ROOT], env=env, capture_output=True, text=True, timeout=600)
    assert out.returncode == 0, out.stdout[-2000:] + out.stderr[-2000:]
    lines = [ln for ln in out.stdout.splitlines() if ln.startswith("DIGEST ")]
    assert len(lines) == 1, out.stdout[-2000:]
    return lines[0]


def test_every_transfer_mode_and_no_dependent_launch_give_the_same_bits():
    """R2K_HOST_ZERO_COPY bit 0: the kernel reads the pinned inputs in place; bit 1: it writes the pinned result in
    place; bit 2: a copy kernel instead of a memcpy brings the inputs in.  R2K_DISABLE_PDL=1: ordinary launches."""
    base = run_child({})
    for mode in ("0", "1", "2", "3", "4", "5"):
        assert run_child({"R2K_HOST_ZERO_COPY": mode}) == base, f"transfer mode {mode}"
    assert run_child({"R2K_DISABLE_PDL": "1"}) == base, "programmatic dependent launch off"
