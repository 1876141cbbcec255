"""Binding a model's tensors by name, from files or from a seeded generator.

A model description lists the tensors it expects (``TensorSpec`` by full
name).  ``load_tensors`` fetches exactly those from a source and fails with
ONE error that lists every missing name, every unexpected name and every
wrong shape -- the reference stops at the first (``need_tensor`` "missing
tensor NAME", src/model.c:158-170; ``check_shape`` got/expected,
src/model.c:193-205), which makes a broken checkpoint slow to diagnose.

Storage rule: a tensor stored as bfloat16 stays bfloat16, one stored in 32 bit
stays 32 bit, float16 is widened to float32 (exact), integer tables become
int32.  Parts that compute with a vector in float32 (norm weights, as the
reference's ``tensor_to_f32``, src/model.c:139-144) widen their own copy when
they bind.
"""
from __future__ import annotations

import hashlib
from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsFile, open_model_files


@dataclass(frozen=True)
class TensorSpec:
    shape: Tuple[int, ...]
    kind: str = "matrix"          # "matrix" | "vector" | "table" (integers)
    init: str = "normal"          # random mode: "normal" | "ones" | "ones_jitter" | "zeros"


class WeightsError(ValueError):
    """The source does not hold the tensors the model expects."""

    def __init__(self, where: str, missing: List[str], unexpected: List[str],
                 wrong: List[Tuple[str, Tuple[int, ...], Tuple[int, ...]]], bad_dtype: List[Tuple[str, str]]):
        self.missing, self.unexpected, self.wrong_shape, self.bad_dtype = missing, unexpected, wrong, bad_dtype
        lines = [f"{where}: tensors do not match the model"]
        if missing:
            lines.append(f"  missing ({len(missing)}): " + ", ".join(missing))
        if unexpected:
            lines.append(f"  unexpected ({len(unexpected)}): " + ", ".join(unexpected))
        for name, got, want in wrong:
            lines.append(f"  wrong shape: {name} is {list(got)}, expected {list(want)}")
        for name, dt in bad_dtype:
            lines.append(f"  wrong dtype: {name} is {dt}")
        super().__init__("\n".join(lines))


class TensorSource:
    """Where tensors come from.  `where` names the source in error messages."""
    where = "weights"

    def listing(self) -> Mapping[str, Tuple[torch.dtype, Tuple[int, ...]]]:
        raise NotImplementedError

    def fetch(self, name: str, device: torch.device) -> torch.Tensor:
        raise NotImplementedError


class FolderSource(TensorSource):
    """model.safetensors (or the shards named by model.safetensors.index.json) of a folder."""

    def __init__(self, model_dir: str):
        self.where = model_dir
        self.files: List[SafetensorsFile] = open_model_files(model_dir)
        self._owner: Dict[str, SafetensorsFile] = {}
        dup = []
        for f in self.files:
            for n in f.names():
                if n in self._owner:
                    dup.append(n)
                self._owner[n] = f
        if dup:
            raise WeightsError(model_dir, [], [f"{n} (stored twice)" for n in dup], [], [])

    def listing(self):
        return {n: (f.tensors[n].dtype, f.tensors[n].shape) for n, f in self._owner.items()}

    def fetch(self, name, device):
        return self._owner[name].get(name).to(device, non_blocking=False)


def tensor_seed(seed: int, name: str) -> int:
    """Seed of one tensor's stream: every tensor draws independently of the others' sizes."""
    return int.from_bytes(hashlib.sha256(f"{seed}:{name}".encode()).digest()[:7], "little")


class RandomSource(TensorSource):
    """Seeded random tensors for a list of specs.

    Matrices ~ N(0, std); vectors marked "ones_jitter" are 1 + N(0, jitter)
    (with jitter 0 they are exactly 1, the reference fixture's norm weights,
    scripts/make-test-model.py:276,287).  Values are drawn in float32 and
    rounded to `dtype` (nearest even).  Streams differ between generator
    devices, so a folder is always written from the CPU generator.
    """

    def __init__(self, specs: Mapping[str, TensorSpec], seed: int, dtype: torch.dtype,
                 std: float = 0.02, norm_jitter: float = 0.01, gen_device: str = "cpu"):
        self.where = f"random(seed={seed})"
        self.specs, self.seed, self.dtype, self.std, self.jitter = dict(specs), seed, dtype, std, norm_jitter
        self.gen_device = torch.device(gen_device)

    def dtype_of(self, spec: TensorSpec) -> torch.dtype:
        return torch.int32 if spec.kind == "table" else self.dtype

    def listing(self):
        return {n: (self.dtype_of(s), tuple(s.shape)) for n, s in self.specs.items()}

    def fetch(self, name, device):
        spec = self.specs[name]
        g = torch.Generator(device=self.gen_device)
        g.manual_seed(tensor_seed(self.seed, name))
        if spec.init == "zeros" or spec.kind == "table":
            t = torch.zeros(spec.shape, dtype=torch.float32, device=self.gen_device)
        elif spec.init == "ones":
            t = torch.ones(spec.shape, dtype=torch.float32, device=self.gen_device)
        else:
            t = torch.empty(spec.shape, dtype=torch.float32, device=self.gen_device)
            # drawn row by row for big matrices so that the float32 staging copy stays small
            if t.dim() == 2 and t.numel() > (1 << 26):
                out = torch.empty(spec.shape, dtype=self.dtype, device=device)
                rows = max(1, (1 << 26) // t.shape[1])
                del t
                for r0 in range(0, spec.shape[0], rows):
                    r1 = min(spec.shape[0], r0 + rows)
                    blk = torch.empty((r1 - r0, spec.shape[1]), dtype=torch.float32, device=self.gen_device)
                    blk.normal_(0.0, self.std, generator=g)
                    out[r0:r1] = blk.to(device=device, dtype=self.dtype)
                return out
            if spec.init == "ones_jitter":
                if self.jitter > 0:
                    t.normal_(1.0, self.jitter, generator=g)
                else:
                    t.fill_(1.0)
            else:
                t.normal_(0.0, self.std, generator=g)
        return t.to(device=device, dtype=self.dtype_of(spec))


def load_tensors(expected: Mapping[str, TensorSpec], source: TensorSource,
                 device: torch.device) -> Dict[str, torch.Tensor]:
    """Fetch exactly the expected tensors; raise one WeightsError for every mismatch."""
    have = source.listing()
    missing = [n for n in expected if n not in have]
    unexpected = sorted(n for n in have if n not in expected)
    wrong, bad = [], []
    for n, spec in expected.items():
        if n not in have:
            continue
        dt, shape = have[n]
        if tuple(shape) != tuple(spec.shape):
            wrong.append((n, tuple(shape), tuple(spec.shape)))
        if spec.kind == "table":
            if dt not in (torch.int32, torch.int64):
                bad.append((n, f"{dt}, expected an integer table"))
        elif dt not in (torch.float32, torch.bfloat16, torch.float16):
            bad.append((n, f"{dt}, expected float32, bfloat16 or float16"))
    if missing or unexpected or wrong or bad:
        raise WeightsError(source.where, missing, unexpected, wrong, bad)
    out: Dict[str, torch.Tensor] = {}
    for n, spec in expected.items():
        t = source.fetch(n, device)
        if spec.kind == "table":
            t = t.to(torch.int32)
        elif t.dtype == torch.float16:
            t = t.to(torch.float32)
        out[n] = t.contiguous()
    return out


def write_model_folder(path: str, config_dict: dict, specs: Mapping[str, TensorSpec], seed: int,
                       dtype: torch.dtype, std: float = 0.02, norm_jitter: float = 0.01) -> None:
    """Random-weights mode: write config.json and model.safetensors for `specs`."""
    import json
    import os
    from .safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    src = RandomSource(specs, seed, dtype, std=std, norm_jitter=norm_jitter)
    layout = [(n, src.dtype_of(s), tuple(s.shape)) for n, s in specs.items()]
    cpu = torch.device("cpu")
    write_safetensors(os.path.join(path, "model.safetensors"),
                      ((n, src.fetch(n, cpu)) for n in specs), metadata={"format": "pt"}, layout=layout)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=1)
