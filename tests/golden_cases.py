"""Load the committed golden fixtures (produced from the reference by
tests/golden/make_golden.py) and rebuild their seeded inputs."""
from __future__ import annotations

import os

import numpy as np
import torch

from recipe import digest, make_inputs

GOLDEN_DIR = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
CASES = ("tiers_page32", "mixed_page64", "page16_tail", "gqa7_fp16", "kblock64_group64", "int4_only")


class GoldenCase:
    def __init__(self, name: str):
        self.name = name
        self.z = np.load(os.path.join(GOLDEN_DIR, name + ".npz"))
        z = self.z
        self.hq, self.hkv, self.page = int(z["hq"]), int(z["hkv"]), int(z["page"])
        self.k_block, self.group = int(z["k_block"]), int(z["group"])
        self.recent_capacity = int(z["recent_capacity"])
        self.append_capacity = None if int(z["append_capacity"]) < 0 else int(z["append_capacity"])
        self.dtype = torch.bfloat16 if int(z["is_bf16"]) else torch.float16
        self.classes = torch.from_numpy(z["classes"])
        self.appends = int(z["appends"])
        self.marks = [int(v) for v in z["snapshots"]]
        self.key, self.value, self.new_k, self.new_v, self.queries = make_inputs(
            seed=int(z["seed"]), hq=self.hq, hkv=self.hkv, tokens=int(self.classes.numel()) * self.page,
            appends=self.appends, n_queries=len(self.marks) + 1, dtype=self.dtype, outliers=bool(z["outliers"]))
        got = digest(self.key, self.value, self.new_k, self.new_v, self.queries)
        if got != str(z["input_digest"]):
            raise RuntimeError(
                f"golden case {name}: regenerated inputs differ from the ones the fixture was made from "
                "(random generator changed?) - regenerate the fixtures with tests/golden/make_golden.py")

    def tensor(self, key: str, dtype=None) -> torch.Tensor:
        t = torch.from_numpy(self.z[key])
        return t.view(dtype) if dtype is not None else t

    def has(self, key: str) -> bool:
        return key in self.z.files

    def build_kwargs(self) -> dict:
        return dict(page_size=self.page, recent_capacity=self.recent_capacity, k_block=self.k_block,
                    v2_group=self.group, append_capacity=self.append_capacity)


def snapshot_arrays(prefix, *, k_packed, k_scale, k_zero, k_active, k_offsets, i2_packed, i2_scale, i2_zero,
                    i2_active, i4_packed, i4_scale, fp_v, recent_k, recent_v, recent_len, recent_global,
                    recent_logical, recent_page_lengths, i2_global, i2_logical) -> dict:
    """Arrange a cache image under the fixture's key names (CPU tensors in)."""
    def raw(t):
        t = t.contiguous()
        return (t.view(torch.int16) if t.dtype in (torch.bfloat16, torch.float16) else t).numpy()
    out = {
        "k_packed": raw(k_packed), "k_scale": raw(k_scale), "k_zero": raw(k_zero), "k_active": np.int64(k_active),
        "k_offsets": np.asarray(k_offsets, dtype=np.int64),
        "i2_packed": raw(i2_packed[:, :i2_active]), "i2_scale": raw(i2_scale[:, :i2_active]),
        "i2_zero": raw(i2_zero[:, :i2_active]), "i2_active": np.int64(i2_active),
        "fp_v": raw(fp_v), "recent_k": raw(recent_k), "recent_v": raw(recent_v), "recent_len": np.int64(recent_len),
        "recent_global": raw(recent_global), "recent_logical": raw(recent_logical),
        "recent_page_lengths": raw(recent_page_lengths), "i2_global": raw(i2_global), "i2_logical": raw(i2_logical),
    }
    if i4_packed.shape[1]:
        out["i4_packed"] = raw(i4_packed)
        out["i4_scale"] = raw(i4_scale)
    return {prefix + k: v for k, v in out.items()}


def compare_snapshot(case: GoldenCase, prefix: str, got: dict, skip=()) -> None:
    """Bit-exact comparison of a cache image with fixture snapshot ``prefix``."""
    for name, value in got.items():
        short = name[len(prefix):]
        if short in skip:
            continue
        if case.has(name):
            want = case.z[name]
            assert want.shape == np.asarray(value).shape, (case.name, name, want.shape, np.asarray(value).shape)
            assert np.array_equal(want, value), (case.name, name, "mismatching elements",
                                                 int((want != value).sum()))
        elif case.has(name + "_digest"):
            assert digest(value) == str(case.z[name + "_digest"]), (case.name, name, "digest differs")
