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
import os
from dataclasses import dataclass
from typing import Dict, List, Mapping, Tuple

import torch

from .safetensors_io import SafetensorsFile, open_model_files, read_weight_map


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
        wm = read_weight_map(model_dir)
        odd: List[str] = []
        for f in self.files:
            shard = os.path.basename(f.path)
            for n in f.names():
                if n in self._owner:
                    odd.append(f"{n} (stored twice: {os.path.basename(self._owner[n].path)} and {shard})")
                elif wm is not None and n not in wm:
                    odd.append(f"{n} (in {shard} but not in the index)")
                elif wm is not None and wm[n] != shard:
                    odd.append(f"{n} (in {shard}, the index says {wm[n]})")
                self._owner[n] = f
        # a name that the index lists but no shard holds is simply absent from the listing: load_tensors reports it
        # as missing together with everything else
        self.index_only = sorted(n for n in (wm or {}) if n not in self._owner)
        if odd:
            raise WeightsError(model_dir, [f"{n} (in the index, in no shard)" for n in self.index_only], odd, [], [])

    def listing(self):
        return {n: (f.tensors[n].dtype, f.tensors[n].shape) for n, f in self._owner.items()}

    def fetch(self, name, device):
        return self._owner[name].get(name).to(device, non_blocking=False)


class RandomSource(TensorSource):
    """Seeded random tensors for a list of specs.

    Matrices ~ N(0, std); vectors marked "ones_jitter" are 1 + N(0, jitter)
    (with jitter 0 they are exactly 1, the reference fixture's norm weights,
    scripts/make-test-model.py:276,287).  Values are drawn in float32 by the
    counter-based generator of ``weights.random_fill`` -- element i of tensor
    `name` is a function of (seed, name, i) alone -- and rounded to `dtype`
    (nearest even).  `gen_device` "cpu" draws with numpy, a CUDA device with
    the kernel of the same recipe; the bits are the same, so a model drawn on
    the device for a measurement can be re-made anywhere, whole or tensor by
    tensor, without a folder.
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

    def law(self, spec: TensorSpec):
        """(mean, std) of a spec's values, or a constant."""
        if spec.init == "zeros" or spec.kind == "table":
            return 0.0
        if spec.init == "ones":
            return 1.0
        if spec.init == "ones_jitter":
            return (1.0, self.jitter) if self.jitter > 0 else 1.0
        return (0.0, self.std)

    def fetch(self, name, device):
        from . import random_fill
        spec = self.specs[name]
        law = self.law(spec)
        dt = self.dtype_of(spec)
        if not isinstance(law, tuple):
            return torch.full(tuple(spec.shape), law, dtype=dt, device=device)
        key = random_fill.tensor_key(self.seed, name)
        count = 1
        for s in spec.shape:
            count *= int(s)
        if self.gen_device.type == "cuda":
            from .. import kernels
            out = torch.empty(tuple(spec.shape), dtype=dt, device=self.gen_device)
            kernels.random_normal(out, key, law[0], law[1])
            return out.to(device)
        vals = torch.from_numpy(random_fill.normal_values(key, 0, count, law[0], law[1])).view(tuple(spec.shape))
        return vals.to(dt).to(device)


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
                       dtype: torch.dtype, std: float = 0.02, norm_jitter: float = 0.01, gen_device: str = "cpu") -> None:
    """Random-weights mode: write config.json and model.safetensors for `specs` (the same file whichever device
    draws the values)."""
    import json
    import os
    from .safetensors_io import write_safetensors
    os.makedirs(path, exist_ok=True)
    src = RandomSource(specs, seed, dtype, std=std, norm_jitter=norm_jitter, gen_device=gen_device)
    layout = [(n, src.dtype_of(s), tuple(s.shape)) for n, s in specs.items()]
    cpu = torch.device("cpu")
    write_safetensors(os.path.join(path, "model.safetensors"),
                      ((n, src.fetch(n, cpu)) for n in specs), metadata={"format": "pt"}, layout=layout)
    with open(os.path.join(path, "config.json"), "w", encoding="utf-8") as f:
        json.dump(config_dict, f, indent=1)
