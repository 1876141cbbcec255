"""The Python entry point: a model folder (or a seeded random model) in, generated token ids out.

It is the same path as the command line: requests go to the scheduler, the scheduler plans steps for the
engine's step function, the device sampler picks tokens.  Option names follow the reference's command
line (src/main.c:188-340): ``n`` (-n, max new tokens, default 256), ``temp`` (--temp, 0 = greedy),
``top_k``, ``top_p``, ``min_p``, ``repeat_penalty``, ``seed`` (-s), ``ignore_eos``; ``ctx`` (-c) and
``batch`` (-b) size the engine.
"""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Dict, List, Optional, Sequence, Union

import torch

from .. import kernels
from ..sampling.sampler import DeviceSampler, SamplingParams
from .engine import Engine, EngineParams, StepEntry, random_engine
from .scheduler import Request, Scheduler, SchedulerParams, StepPlan


@dataclass
class GenerationResult:
    tokens: List[int]
    finish_reason: str
    prompt_tokens: int
    preemptions: int = 0


@dataclass
class InFlight:
    """A step that has been launched: who gets a token from it, where the tokens will arrive, and when."""
    wanting: list
    host: Optional[torch.Tensor]
    done: Optional[torch.cuda.Event]


class EngineExecutor:
    """Runs a scheduler's plan on the engine and samples on the device.

    `launch` queues a step and returns at once; `wait` blocks until its tokens are on the host.  The sampled ids
    of every step stay in one device array (`feed`), so that the step after it can be launched before the host
    has read them: an entry whose token is the scheduler's IN_FLIGHT mark is fed row `feed_rows[request]` of it."""

    # A request whose sampling penalises recent tokens can be stepped ahead all the same: the token that is still on the
    # device is put into its window there (DeviceSampler.pick, in_flight=).
    windows_on_device = True

    def __init__(self, engine: Engine):
        self.engine = engine
        self.sampler = DeviceSampler(engine.device)
        self.feed = torch.zeros(max(engine.params.max_requests, 1), dtype=torch.int32, device=engine.device)
        self.picked = torch.zeros_like(self.feed)       # where a step's tokens go first when its sampling reads `feed`
        self._host = [torch.empty(self.feed.numel(), dtype=torch.int32).pin_memory() for _ in range(3)]
        self._next = 0

    def launch(self, plan: StepPlan, feed_rows: Optional[Dict[object, int]] = None) -> InFlight:
        entries = []
        for e in plan.entries:
            toks = e.tokens
            if feed_rows is not None and e.request.id in feed_rows:
                assert e.count == 1
                toks = [-(1 + feed_rows[e.request.id])]
            entries.append(StepEntry(e.request.id, toks, [e.count - 1] if e.wants_token else []))
        # the engine gives the plan's reservations back if anything in the step fails; so does this method when the
        # sampling that belongs to the step fails, and only then is the step committed
        logits = self.engine.step(entries, reserved=True, feed=self.feed, commit=False)
        wanting = [e.request for e in plan.entries if e.wants_token]
        draws = [r.sampler.rng for r in wanting]
        try:
            if not wanting:
                step = InFlight([], None, None)
            else:
                in_flight = [feed_rows.get(r.id, -1) if feed_rows is not None else -1 for r in wanting]
                if any(j >= 0 and r.sampler.needs_window() for j, r in zip(in_flight, wanting)):
                    ids = self.sampler.pick(logits, [r.sampler for r in wanting], out=self.picked, in_flight=in_flight, feed=self.feed)
                    self.feed[:len(wanting)].copy_(ids)
                else:
                    ids = self.sampler.pick(logits, [r.sampler for r in wanting], out=self.feed)
                host = self._host[self._next]
                self._next = (self._next + 1) % len(self._host)
                host[:len(wanting)].copy_(ids, non_blocking=True)                       # device -> host
                done = torch.cuda.Event()
                done.record()
                step = InFlight(wanting, host, done)
        except BaseException:
            self.engine.cancel_step(entries)
            for r, state in zip(wanting, draws):
                r.sampler.rng = state          # a draw made for a step that did not happen is made again
            raise
        self.engine.commit_step(entries)
        return step

    def wait(self, step: InFlight) -> Dict[object, int]:
        if not step.wanting:
            return {}
        step.done.synchronize()
        picked = step.host[:len(step.wanting)].tolist()
        return {r.id: t for r, t in zip(step.wanting, picked)}

    def run(self, plan: StepPlan) -> Dict[object, int]:
        return self.wait(self.launch(plan))


class Runner:
    STATUS_EVERY = 64        # generate() reads the kernels' status word every so many steps (one small device read)

    def __init__(self, model: Optional[str] = None, *, config=None, random_seed: Optional[int] = None,
                 dtype: str = "bfloat16", ctx: Optional[int] = None, batch: int = 2048, parallel: int = 8,
                 max_tokens: Optional[int] = None, page_size: int = 64, prefill_chunk: Optional[int] = None,
                 device: str = "cuda:0", engine: Optional[Engine] = None, rope_base: Optional[float] = None,
                 rope_scale: Optional[float] = None):
        """model: folder with config.json + model.safetensors.  Or `config` (a typed configuration) with
        `random_seed` for seeded random weights.  ctx: longest request (default min(model limit, 4096), the
        reference's -c default, src/model.c:3075; 0: as long as the model allows and the free memory holds, its -c 0).  batch: token budget of a step (-b).  parallel: live
        requests.  max_tokens: tokens the page pool holds (default parallel * ctx).  rope_base: use this
        frequency base instead of the configuration's (--rope-base, src/model.c:282).  rope_scale: force linear
        position scaling by this factor instead of the configuration's scaling (--rope-scale, src/model.c:324-326)."""
        if engine is None:
            from ..config import registry
            if model is not None:
                arch, cfg = registry.load_config(model)
            else:
                cfg = config
                arch = registry.resolve(cfg.architecture)
            if rope_base is not None or rope_scale is not None:
                if arch.override is None:
                    raise ValueError(f"architecture '{arch.name}' takes no rope_base / rope_scale override")
                cfg = arch.override(cfg, rope_base=rope_base, rope_scale=rope_scale)
            model_limit = arch.build_plan(cfg).max_positions        # (parts only, no weights: cheap)
            if ctx == 0:
                ctx = self._fit_context(arch, cfg, model_limit, parallel, page_size, dtype, device)
            ctx = ctx or min(model_limit, 4096)
            ep = EngineParams(dtype=dtype, max_tokens=max_tokens or parallel * ctx, page_size=page_size,
                              max_requests=parallel, max_request_tokens=ctx, max_step_tokens=batch, device=device)
            if model is not None and (rope_base is not None or rope_scale is not None):
                from ..weights.loader import FolderSource
                engine = Engine(params=ep, config=cfg, source=FolderSource(model))
            elif model is not None:
                engine = Engine(model, ep)
            else:
                engine = random_engine(cfg, random_seed or 0, ep)
        self.engine = engine
        self.executor = EngineExecutor(engine)
        self.scheduler = Scheduler(engine.cache, self.executor,
                                   SchedulerParams(max_step_tokens=max(batch, engine.params.max_requests),
                                                   prefill_chunk=prefill_chunk),
                                   open_request=engine._open)
        self._next_id = 0
        self.timing: Dict[str, float] = {}

    @staticmethod
    def _fit_context(arch, cfg, model_limit: int, parallel: int, page_size: int, dtype: str, device: str) -> int:
        """ctx=0, the reference's auto-fit (-c 0, src/main.c:512): the longest context, up to the model's limit, whose
        keys and values for `parallel` requests fit the device memory that is free now beside the weights (nine
        tenths of it: the step's buffers need room too)."""
        plan = arch.build_plan(cfg)
        elem = 2 if dtype in ("bfloat16", "bf16") else 4
        wbytes = 0
        wdt = 2 if getattr(cfg, "torch_dtype", "bfloat16") == "bfloat16" else 4
        for spec in plan.tensor_specs().values():
            n = 1
            for s_ in spec.shape:
                n *= int(s_)
            wbytes += n * wdt
        per_token = 0
        for e in plan.schedule:
            need = plan.blocks[e.layer].mixer.kv_need()
            if need is not None and e.cache_from is None:
                per_token += 2 * need.kv_heads * need.head_dim * elem
        free, _ = torch.cuda.mem_get_info(torch.device(device))
        room = int(0.9 * free) - 2 * wbytes                      # (packing a matrix needs a second copy for a moment)
        if per_token == 0:
            return model_limit
        fit = room // (per_token * parallel) // page_size * page_size
        if fit < page_size:
            raise ValueError(f"-c 0: no context fits beside the weights ({free >> 20} MiB free, weights {wbytes >> 20} MiB)")
        return int(min(model_limit, fit))

    def submit(self, prompt: Sequence[int], n: int = 256, temp: float = 0.0, top_k: int = 0, top_p: float = 1.0,
               min_p: float = 0.0, repeat_penalty: float = 1.0, seed: Optional[int] = None,
               ignore_eos: bool = False, stop_ids: Optional[Sequence[int]] = None) -> object:
        rid = self._next_id
        self._next_id += 1
        sp = SamplingParams(temperature=temp, top_k=top_k, top_p=top_p, min_p=min_p, repeat_penalty=repeat_penalty,
                            seed=seed)
        stops = tuple(stop_ids) if stop_ids is not None else tuple(self.engine.plan.stop_ids)
        self.scheduler.add(Request(rid, [int(t) for t in prompt], max_new_tokens=n, sampling=sp, stop_ids=stops,
                                   ignore_eos=ignore_eos))
        return rid

    def abort(self, request_id) -> bool:
        """End a submitted request now; its pages and slot are free when this returns (see Scheduler.abort)."""
        return self.scheduler.abort(request_id)

    def generate(self, prompts: Union[Sequence[int], Sequence[Sequence[int]]], n: int = 256, temp: float = 0.0,
                 top_k: int = 0, top_p: float = 1.0, min_p: float = 0.0, repeat_penalty: float = 1.0,
                 seed: Optional[int] = None, ignore_eos: bool = False, on_token=None):
        """Generate for one prompt (a list of ids) or several (a list of lists), all scheduled together.
        With several prompts and a seed, request i samples with seed + i.  `on_token(request, token, finished)` is
        called for every token as it arrives; returning False ends that request there (finish reason "abort").
        Returns GenerationResult(s)."""
        single = len(prompts) > 0 and isinstance(prompts[0], int)
        plist = [prompts] if single else list(prompts)
        ids = [self.submit(p, n, temp, top_k, top_p, min_p, repeat_penalty,
                           None if seed is None else seed + i, ignore_eos) for i, p in enumerate(plist)]
        t0 = time.perf_counter()
        sch = self.scheduler
        steps = 0
        try:
            while sch.has_work():
                before = len(sch.finished)
                res = sch.step()
                if on_token is not None:
                    for rid, tok, done in res:
                        if on_token(rid, tok, done) is False and not done:
                            sch.abort(rid)       # the callback asked for the end of this request (src/engine.c:1844-1848)
                if not res and not sch.live and sch.waiting and len(sch.finished) == before:
                    r = sch.waiting.popleft()
                    sch._finish(r, "rejected")
                steps += 1
                if steps % self.STATUS_EVERY == 0:
                    self.engine.check_status()   # a kernel that gave up a wait: stop now, not after a run of garbage
            torch.cuda.synchronize(self.engine.device)
            self.engine.check_status()
        except BaseException:
            # the call ends here: its requests give back their pages and slots, and the runner can be used again
            for rid in ids:
                if rid not in sch.finished:
                    sch.abort(rid)
            for rid in ids:
                sch.finished.pop(rid, None)
            raise
        self.timing["generate_s"] = time.perf_counter() - t0
        out = []
        for rid in ids:
            r = sch.finished.pop(rid)
            out.append(GenerationResult(list(r.generated), r.finish_reason, len(r.prompt), r.preemptions))
        return out[0] if single else out

    def score(self, tokens: Sequence[int], portion: int = 256) -> List[float]:
        """Teacher-forced scoring, the reference's --score mode (src/main.c:1344-1433): log P(tokens[i + 1] | tokens[:i + 1])
        for every i, in float32 from the logits (float maximum, double sum of exponentials).  The tokens run through
        the step function in portions of at most `portion` (each portion's logits are [portion, vocabulary] float32);
        by the engine's exactness rule the result does not depend on the portion beyond rounding.  Nothing is sampled."""
        toks = [int(t) for t in tokens]
        if len(toks) < 2:
            raise ValueError(f"scoring needs at least 2 tokens to score a transition (got {len(toks)})")
        if len(toks) > self.engine.cache.max_pages_per_request * self.engine.cache.page_size:
            raise ValueError(f"the prompt is {len(toks)} tokens, the context is "
                             f"{self.engine.cache.max_pages_per_request * self.engine.cache.page_size}")
        eng = self.engine
        portion = max(1, min(portion, eng.params.max_step_tokens))
        rid = ("score", self._next_id)
        self._next_id += 1
        out: List[float] = []
        n_score = len(toks) - 1
        target = torch.tensor(toks[1:], dtype=torch.int32, device=eng.device)
        lp = torch.empty(n_score, dtype=torch.float32, device=eng.device)
        try:
            for at in range(0, n_score, portion):
                m = min(portion, n_score - at)
                logits = eng.step([StepEntry(rid, toks[at:at + m], list(range(m)))])
                kernels.logprob(logits, target[at:at + m], lp[at:at + m])
            out = lp.cpu().tolist()
        finally:
            if eng.is_live(rid):
                eng.end(rid)
        eng.check_status()
        return out
