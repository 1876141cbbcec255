"""Trace replay: drive the engine's step function with given token ids and collect the logits.

A trace is a sequence of steps, each ``{"step": k, "entries": [{"id", "tokens", "want"}], "end": [...]}``.
All entries of a step are one batch for ``Engine.step``; requests named in `end` give their pages and
slot back after the step.  Nothing is sampled, and there is no forward pass here: the reference's
analogues are its teacher-forced passes (`--score`, src/main.c:1344-1433; tests/test_gpu_identity.c:70-108),
which call the model's own forward the same way.
"""
from __future__ import annotations

import json
import os
from typing import Callable, Dict, Iterable, Optional

import numpy as np

from .engine import Engine, StepEntry


def replay(engine: Engine, steps: Iterable, out_dir: Optional[str] = None,
           on_done: Optional[Callable[[object], None]] = None) -> Dict[object, np.ndarray]:
    """Run `steps` (dicts or JSON lines).  Returns {step: float32 [wanted, vocab]} for steps that wanted
    logits; with `out_dir` each is also written to <out_dir>/<step>.f32 (little-endian)."""
    results: Dict[object, np.ndarray] = {}
    for rec in steps:
        if isinstance(rec, (str, bytes)):
            if not rec.strip():
                continue
            rec = json.loads(rec)
        step = rec["step"]
        entries = [StepEntry(e["id"], e["tokens"], e.get("want", ())) for e in rec.get("entries", ())]
        logits = engine.step(entries)
        if logits.shape[0] > 0:
            arr = logits.cpu().numpy().astype("<f4", copy=False)
            engine.check_status()
            if out_dir is not None:
                arr.tofile(os.path.join(out_dir, f"{step}.f32"))
            else:
                results[step] = arr.copy()
        for rid in rec.get("end", ()):
            if engine.is_live(rid):
                engine.end(rid)
        if on_done is not None:
            on_done(step)
    return results
