"""The engine: a loaded model, its cache, and ONE step function.

``Engine.step`` takes a batch of (request, its next tokens, the places whose
logits are wanted): portions of prompts beside single decoded tokens, cut
anywhere.  It runs exactly the tokens it is given, as one flat batch, against
the keys and values that earlier steps left in the pages, and returns float32
logits at the wanted places.  The reference has two disjoint primitives for
this -- ``model_forward_batch`` (n consecutive tokens of one sequence, logits
of the last, src/model.h:667-670) and ``model_batch_decode`` (one token of each
of n sequences, src/model.h:796-807) -- and carries the rule that a token's
result must not depend on what else is in the batch (src/gpu.h:127-131); that
rule holds here for any mixture.

All token-parallel work (norms, products, rotation, SwiGLU) runs on the flat
token axis; attention runs per token over its request's block table with the
causal limit of its own position; the head runs on the gathered wanted rows
only (the reference's `want_logits`, src/model.c:6478-6481, generalised).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence

import numpy as np
import torch

from .. import architectures  # noqa: F401  (registers the built-in architectures)
from .. import kernels
from ..cache.pages import CacheManager, OutOfPages
from ..config import registry
from ..parts.base import Runtime
from ..weights.loader import FolderSource, RandomSource, TensorSource
from .model import LayerRuntime, LoadedModel, ModelPlan

_DTYPES = {"bfloat16": torch.bfloat16, "bf16": torch.bfloat16, "float32": torch.float32, "fp32": torch.float32}


@dataclass
class EngineParams:
    dtype: str = "bfloat16"            # "bfloat16": serving kernels; "float32": everything in true 32 bit
    max_tokens: int = 4096             # tokens the page pool holds (rounded up to whole pages)
    page_size: int = 64                # tokens per page
    max_requests: int = 4              # live requests (state slots)
    max_request_tokens: Optional[int] = None   # longest request; default min(model limit, max_tokens)
    max_step_tokens: int = 8192        # sizing hint for the step's buffers (they grow if a step brings more)
    cuda_graphs: bool = True           # decode-only steps are captured once per (batch, context bucket) and replayed
    device: str = "cuda:0"


@dataclass
class StepEntry:
    request: object
    tokens: Sequence[int]
    want: Sequence[int] = ()           # indices into `tokens` whose logits are wanted


class StepContext:
    """What the parts see of one step.  Tensors are on the device; `host` holds the same as numpy."""

    def __init__(self, eng: "Engine"):
        self._eng = eng
        self.act_dtype = eng.act_dtype
        self.page_size = eng.params.page_size
        self.max_pages = eng.cache.max_pages_per_request
        self.n = 0
        self.n_seg = 0
        self.token_ids = self.positions = self.tok_seg = self.logit_rows = None
        self.token_feed = None          # tokens that an earlier step left on the device (Engine.step's `feed`)
        self.seg_start = self.seg_len = self.seg_pos0 = self.seg_slot = None
        self.block_tables: List[torch.Tensor] = []
        self.host: Dict[str, np.ndarray] = {}
        self.max_kv_len = 0            # longest key range any token of the step reads
        self._pending = {}
        self._views: Dict[tuple, torch.Tensor] = {}
        self._memo: Dict[object, object] = {}
        self.decode_only = False       # every segment is a single token
        self.uneven = False            # the requests' lengths differ much (a hint for kernels that split work by request)

    def buf(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        # (every layer asks for the same few views: made once a step)
        key = (name, tuple(shape), dtype)
        t = self._views.get(key)
        if t is None:
            t = self._views[key] = self._eng._buf(name, shape, dtype)
        return t

    def once(self, key, make):
        """make() the first time `key` is asked for in this step, the same value afterwards: for what a part works out
        from the step's description on the host and every layer would work out again."""
        v = self._memo.get(key)
        if v is None:
            v = self._memo[key] = make()
        return v

    # A part whose last product was split along K may leave the sum unfinished ("pending") on the residual
    # stream; the next norm finishes it in its own pass.  Anything else that reads or writes that tensor
    # directly calls ``materialize`` first.
    def set_pending(self, x: torch.Tensor, pending) -> None:
        if pending is not None:
            self.materialize(x)
            self._pending[x.data_ptr()] = pending

    def take_pending(self, x: torch.Tensor):
        return self._pending.pop(x.data_ptr(), None)

    def materialize(self, x: torch.Tensor) -> None:
        p = self._pending.pop(x.data_ptr(), None)
        if p is not None:
            p.finish()

    def cache_layer(self, lay: LayerRuntime):
        """(pointer to this layer's K block of page 0, elements between pages, elements from K to V)."""
        return self._eng._cache_layer[lay.entry]

    def cache_group(self, lay: LayerRuntime):
        """(pointer to the whole array of the layer's cache group, its pages, its layers, this layer's index)."""
        t = self._eng.kv[lay.group]
        return (t.data_ptr(), t.shape[0], t.shape[1], lay.layer_in_group)


class Engine:
    def __init__(self, model_dir: Optional[str] = None, params: Optional[EngineParams] = None, *,
                 config=None, architecture: Optional[str] = None, source: Optional[TensorSource] = None):
        """Load from `model_dir` (config.json + model.safetensors), or from a typed `config` plus a tensor
        `source` (e.g. ``RandomSource``) for an architecture name."""
        self.params = params or EngineParams()
        p = self.params
        if p.dtype not in _DTYPES:
            raise ValueError(f"dtype '{p.dtype}': choose bfloat16 or float32")
        self.act_dtype = _DTYPES[p.dtype]
        if not torch.cuda.is_available():
            raise RuntimeError("the engine runs on a CUDA device only; none is visible")
        self.device = torch.device(p.device)
        torch.cuda.set_device(self.device)
        kernels.lib()                      # fail now, and loudly, if the kernels cannot be built or loaded
        if model_dir is not None:
            arch, self.config = registry.load_config(model_dir)
            source = FolderSource(model_dir)
        else:
            if config is None or source is None:
                raise ValueError("give model_dir, or config and source")
            arch = registry.resolve(architecture or config.architecture)
            self.config = config
        plan: ModelPlan = arch.build_plan(self.config)
        rt = Runtime(self.device, self.act_dtype, p.page_size, p.max_step_tokens, p.max_requests)
        self.model = LoadedModel(plan, source, rt)
        self.plan = plan
        n_pages = max(1, -(-p.max_tokens // p.page_size))
        max_req = p.max_request_tokens or min(plan.max_positions, n_pages * p.page_size)
        self.cache = CacheManager([g.spec for g in self.model.groups] or [], n_pages, p.page_size,
                                  p.max_requests, max_req)
        # device arrays of keys and values: [page][layer in group][K|V][kv head][token in page][head_dim].  One page
        # more than the pool hands out: the rows that fill a decode step up to a repeating size write there.
        self.kv: List[torch.Tensor] = []
        self._filler_page = n_pages
        for g in self.model.groups:
            self.kv.append(torch.zeros((n_pages + 1, g.n_layers, 2, g.kv_heads, p.page_size, g.head_dim),
                                       dtype=self.act_dtype, device=self.device))
        self._cache_layer: Dict[int, tuple] = {}
        for lay in self.model.layers:
            if lay.group >= 0:
                t = self.kv[lay.group]
                es = t.element_size()
                self._cache_layer[lay.entry] = (t.data_ptr() + lay.layer_in_group * t.stride(1) * es,
                                                t.stride(0), t.stride(2))
        for entry, need in self.model.state_needs:
            self.model.layers[entry].state = torch.zeros((p.max_requests,) + tuple(need.shape), dtype=need.dtype,
                                                         device=self.device)
        self._bufs: Dict[tuple, torch.Tensor] = {}
        # step descriptions go through a small ring of pinned buffers; an event per buffer says when the
        # copy that read it has run, so the host never rewrites memory that a copy in flight still reads
        self._pinned: List[Optional[torch.Tensor]] = [None] * 3
        self._pinned_done: List[Optional[torch.cuda.Event]] = [None] * 3
        self._pinned_next = 0
        self._slot_generation = np.zeros(p.max_requests, dtype=np.int64)
        self.steps_run = 0
        self.h2d_bytes = 0               # bytes of step descriptions copied to the device so far
        # CUDA graphs of decode-only steps, keyed by (tokens, wanted rows, context bucket).  A graph holds the
        # addresses of the step's buffers, so any buffer that is made anew invalidates all graphs.
        self._graphs: Dict[tuple, object] = {}
        self._uneven_of_shape: Dict[tuple, bool] = {}      # decode-only steps: the unevenness hint a shape was first seen with
        self._graph_ok = p.cuda_graphs and all(part.graph_safe for part in plan.parts())
        # Decode-only steps of more than 8 requests are filled up to a multiple of 8 with rows of a request that does
        # not exist (one token at position 0, keys and values in the spare page, logits dropped), so that a few graphs
        # serve every batch size.  Not with per-request state: a filler row has no slot of its own.
        self._fill_ok = self._graph_ok and not self.model.state_needs
        self._graph_seen: Dict[tuple, int] = {}
        self._buf_generation = 0
        self.graph_replays = 0
        self._graph_launches: Dict[tuple, int] = {}
        # the step description's device buffer is made once for the largest step the parameters name
        T, S = p.max_step_tokens, p.max_requests
        torch.cuda.synchronize(self.device)       # weights are at rest before the first product reads them
        self._buf("step_description", (4 * (T + 4) + 4 * (S + 4) + len(self.cache.groups) * (S * self.cache.max_pages_per_request + 4),),
                  torch.int32)

    # ---- buffers ---------------------------------------------------------------
    def _buf(self, name: str, shape, dtype: torch.dtype) -> torch.Tensor:
        n = 1
        for s in shape:
            n *= int(s)
        key = (name, dtype)
        t = self._bufs.get(key)
        if t is None or t.numel() < n:
            cap = n
            if t is None and len(shape) == 2 and shape[0] < self.params.max_step_tokens and name != "logits":
                cap = self.params.max_step_tokens * int(shape[1])
            t = torch.empty(max(cap, 1), dtype=dtype, device=self.device)
            self._bufs[key] = t
            self._buf_generation += 1
            self._graphs.clear()
            self._uneven_of_shape.clear()
        return t[:n].view(*shape)

    # ---- requests ----------------------------------------------------------------
    def is_live(self, request) -> bool:
        return self.cache.is_open(request)

    def length(self, request) -> int:
        return self.cache.length(request)

    def end(self, request) -> None:
        """The request is finished: its pages and its state slot are given back."""
        self.cache.close(request)

    def adopt(self, request, n_tokens: int) -> None:
        """Open `request` as if `n_tokens` had been run: pages are taken, nothing is computed, and the keys
        and values in those pages are whatever the pool holds.  For measurements that need a long context
        without paying for its prefill."""
        self._open(request)
        self.cache.reserve(request, n_tokens)
        self.cache.commit(request)

    def _open(self, request) -> int:
        slot = self.cache.open(request)
        for lay in self.model.layers:
            if lay.state is not None:
                lay.state[slot].zero_()
        return slot

    # ---- the step ----------------------------------------------------------------
    def step(self, entries: Sequence[StepEntry], reserved: bool = False, feed: Optional[torch.Tensor] = None,
             commit: bool = True) -> torch.Tensor:
        """Run one batch.  Returns float32 logits [number of wanted places, vocab] on the device, in the
        order of the entries and of each entry's `want`; the tensor is reused by the next step.

        `feed`: int32 tokens on the device; a token id -(1 + j) in an entry stands for
        feed[j] as it is when this step runs, e.g. what the step before sampled, which the host has not read yet.

        Unless `reserved`, pages for every entry's tokens are taken here (all or nothing: on
        ``OutOfPages`` the cache is as before the call).  A request not seen before is opened.

        A step that fails owns no row of the cache (the reference's rule for a position handed out for a forward
        that never ran, src/engine.c:1917-1925): whatever is raised between the reservation and the last launch --
        a kernel refusing its sizes, the runtime refusing a launch, an allocation that fails -- the reservations
        of every entry are given back, the caller's too when `reserved`, requests that this call opened are closed,
        and the exception goes on to the caller; the same entries can then be run again.  With ``commit=False``
        the caller finishes the step itself: ``commit_step`` once everything that belongs to it (sampling) has
        been launched, ``cancel_step`` if that failed."""
        entries = [e for e in entries if len(e.tokens) > 0]
        if not entries:
            return torch.empty((0, self.plan.vocab_size), dtype=torch.float32, device=self.device)
        seen = set()
        for e in entries:
            if e.request in seen:
                raise ValueError(f"request {e.request!r} appears twice in one step")
            seen.add(e.request)
            for w in e.want:
                if not (0 <= w < len(e.tokens)):
                    raise ValueError(f"request {e.request!r}: wanted place {w} is outside its {len(e.tokens)} tokens")
        opened: List[object] = []
        try:
            if not reserved:
                for e in entries:
                    if not self.cache.is_open(e.request):
                        self._open(e.request)
                        opened.append(e.request)
                    self.cache.reserve(e.request, len(e.tokens))
            ctx = self._describe(entries)
            ctx.token_feed = feed
            if ctx.decode_only and self._graph_ok:
                logits = self._forward_graphed(ctx)
            else:
                logits = self._forward(ctx)
        except BaseException:
            self.cancel_step(entries, opened)
            raise
        if ctx.real_rows != ctx.n_rows:
            logits = logits[:ctx.real_rows]          # the filler rows' logits are nobody's
        if commit:
            self.commit_step(entries)
        return logits

    def commit_step(self, entries: Sequence[StepEntry]) -> None:
        """The step's launches are all queued: its tokens now count as held by their requests."""
        for e in entries:
            if len(e.tokens) > 0:
                self.cache.commit(e.request)
        self.steps_run += 1

    def cancel_step(self, entries: Sequence[StepEntry], opened: Sequence[object] = ()) -> None:
        """The step did not run to its end: give back what was reserved for it and close the requests in `opened`.
        Rows that its kernels may have written lie beyond every request's length and are nobody's."""
        for e in entries:
            if self.cache.is_open(e.request):
                self.cache.cancel(e.request)
        for r in opened:
            if self.cache.is_open(r):
                self.cache.close(r)

    def _describe(self, entries: Sequence[StepEntry]) -> StepContext:
        """Flatten the batch and bring its description to the device in one copy."""
        kernels.tc_workspace_reset(self.device)      # no deferred sum outlives its step
        cache = self.cache
        S_real = len(entries)
        i32 = np.int32
        counts = np.fromiter((len(e.tokens) for e in entries), i32, S_real)
        want_counts = np.fromiter((len(e.want) for e in entries), i32, S_real)
        slots = np.fromiter((cache.slot_of(e.request) for e in entries), i32, S_real)
        n_real, R_real = int(counts.sum()), int(want_counts.sum())
        if n_real == S_real:
            tokens = np.fromiter((e.tokens[0] for e in entries), np.int64, S_real).astype(i32)
        else:
            tokens = np.concatenate([np.asarray(e.tokens, dtype=np.int64) for e in entries]).astype(i32)
        wants = np.fromiter((w for e in entries for w in e.want), i32, R_real)
        fill = 0
        if self._fill_ok and S_real > 8 and n_real == S_real:
            fill = min(-(-S_real // 8) * 8, max(self.params.max_requests, S_real)) - S_real
        S, n, R = S_real + fill, n_real + fill, R_real + fill
        G = len(cache.groups)
        mp = cache.max_pages_per_request
        sizes = [n, n, n, max(R, 1), S, S, S, S] + [S * mp] * G
        offs = np.concatenate([[0], np.cumsum([(s + 3) // 4 * 4 for s in sizes])]).astype(np.int64)
        total = int(offs[-1])
        slot_i = self._pinned_next
        self._pinned_next = (slot_i + 1) % len(self._pinned)
        if self._pinned_done[slot_i] is not None:
            self._pinned_done[slot_i].synchronize()
        if self._pinned[slot_i] is None or self._pinned[slot_i].numel() < total:
            self._pinned[slot_i] = torch.empty(max(total, 1 << 16), dtype=torch.int32).pin_memory()
        pinned = self._pinned[slot_i]
        host = pinned.numpy()
        tok, pos, seg, rows, s_start, s_len, s_pos0, s_slot = (host[offs[i]:offs[i] + sizes[i]] for i in range(8))
        # the flattening itself is native (csrc/host/page_cache.cpp: xrh_describe); it writes into the pinned buffer
        base = host.ctypes.data
        max_kv = cache.describe_step(slots, counts, tokens, want_counts, wants, fill, self._filler_page,
                                     [base + 4 * int(offs[i]) for i in range(8)], [base + 4 * int(offs[8 + g]) for g in range(G)])
        decode_only = n_real == S_real
        dev = self._buf("step_description", (total,), torch.int32)
        dev.copy_(pinned[:total], non_blocking=True)
        self.h2d_bytes += total * 4
        if self._pinned_done[slot_i] is None:
            self._pinned_done[slot_i] = torch.cuda.Event()
        self._pinned_done[slot_i].record()
        ctx = StepContext(self)
        ctx.n, ctx.n_seg, ctx.n_rows, ctx.real_rows = n, S, R, R_real
        view = lambda i: dev[int(offs[i]):int(offs[i]) + sizes[i]]
        ctx.token_ids, ctx.positions, ctx.tok_seg, ctx.logit_rows = view(0), view(1), view(2), view(3)
        ctx.seg_start, ctx.seg_len, ctx.seg_pos0, ctx.seg_slot = view(4), view(5), view(6), view(7)
        ctx.block_tables = [view(8 + g).view(S, mp) for g in range(G)]
        # (views of the pinned buffer: valid until this buffer's turn in the ring comes again, three steps on)
        ctx.host = {"token_ids": tok, "positions": pos, "tok_seg": seg, "logit_rows": rows[:R], "seg_start": s_start,
                    "seg_len": s_len, "seg_pos0": s_pos0, "seg_slot": s_slot}
        if decode_only:
            max_kv = -(-max_kv // 1024) * 1024      # a bucket, so that launch shapes repeat from step to step
        ctx.max_kv_len, ctx.decode_only = max_kv, decode_only
        # equal spans of the longest request would be more than a quarter empty
        ends = s_pos0[:S_real].astype(np.int64) + s_len[:S_real]
        ctx.uneven = S_real > 1 and int(ends.max()) * S_real > 1.25 * int(ends.sum())
        if decode_only:
            # a step graph holds the kernels that were chosen when it was captured: the answer at the first step of a
            # shape stands for all later steps of that shape, so that a shape has one graph
            ctx.uneven = self._uneven_of_shape.setdefault((n, R, max_kv), ctx.uneven)
        return ctx

    def _forward_graphed(self, ctx: StepContext) -> torch.Tensor:
        """Decode-only steps have the same launches whenever batch size and context bucket repeat: the
        first such step runs plainly (and makes every buffer), the second is captured, later ones replay.
        Everything that changes from step to step is in the step description, which is copied before."""
        key = (ctx.n, ctx.n_rows, ctx.max_kv_len, None if ctx.token_feed is None else ctx.token_feed.data_ptr())
        g = self._graphs.get(key)
        if g is not None:
            g.replay()
            self.graph_replays += 1
            kernels.launch_count += self._graph_launches[key]
            return self._bufs[("logits", torch.float32)][:ctx.n_rows * self.plan.vocab_size].view(ctx.n_rows, -1)
        seen = self._graph_seen.get(key, 0)
        self._graph_seen[key] = seen + 1
        if seen == 0 or ctx.n_rows == 0:
            return self._forward(ctx)
        gen = self._buf_generation
        graph = torch.cuda.CUDAGraph()
        torch.cuda.synchronize(self.device)
        launches0 = kernels.launch_count
        with torch.cuda.graph(graph):
            logits = self._forward(ctx)
        self._graph_launches[key] = kernels.launch_count - launches0
        if self._buf_generation != gen:
            # a buffer was made during capture: the graph may hold a stale address; run plainly this time
            self._graph_seen[key] = 1
            return self._forward(ctx)
        self._graphs[key] = graph
        graph.replay()
        self.graph_replays += 1
        return logits

    def _forward(self, ctx: StepContext) -> torch.Tensor:
        plan = self.plan
        x = ctx.buf("residual", (ctx.n, plan.width), torch.float32)
        plan.embedding.forward(ctx, ctx.token_ids, x)
        for lay in self.model.layers:
            plan.blocks[plan.schedule[lay.entry].layer].forward(ctx, x, lay)
        if ctx.n_rows == 0:
            ctx.materialize(x)
            return torch.empty((0, plan.vocab_size), dtype=torch.float32, device=self.device)
        hn = ctx.buf("head_normed", (ctx.n_rows, plan.width), ctx.act_dtype)
        # a step of single tokens that all want their logits: the wanted rows are all rows, in order
        every_row = ctx.decode_only and ctx.n_rows == ctx.n
        plan.final_norm.forward(ctx, x, hn, rows=None if every_row else ctx.logit_rows)
        logits = ctx.buf("logits", (ctx.n_rows, plan.vocab_size), torch.float32)
        plan.head.forward(ctx, hn, logits)
        return logits

    def check_status(self) -> None:
        """Raise if a kernel reported a failure since the last check (one small read from the device)."""
        kernels.tc_check_status(self.device)

    # ---- accounting (bench) ---------------------------------------------------------
    def weight_bytes_per_step(self) -> int:
        return self.model.weight_bytes_per_step()

    def kv_bytes_per_token(self) -> int:
        return self.model.kv_bytes_per_token(2 if self.act_dtype == torch.bfloat16 else 4)


def random_engine(config, seed: int, params: EngineParams, std: float = 0.02, norm_jitter: float = 0.01,
                  weight_dtype: Optional[torch.dtype] = None) -> Engine:
    """An engine with seeded random weights generated on the device (nothing is written to disk)."""
    arch = registry.resolve(config.architecture)
    plan = arch.build_plan(config)
    wd = weight_dtype or _DTYPES.get(getattr(config, "torch_dtype", "bfloat16"), torch.bfloat16)
    src = RandomSource(plan.tensor_specs(), seed, wd, std=std, norm_jitter=norm_jitter, gen_device=params.device)
    return Engine(params=params, config=config, source=src)
