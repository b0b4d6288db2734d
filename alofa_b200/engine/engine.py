"""The engine loop and the Python entry point.

:class:`Engine` joins the scheduler, the cache manager and the step function:
requests are submitted with their prompt tokens, every :meth:`Engine.step`
asks the scheduler what to run, translates its action into one batch for the
step function, samples, and settles the outcome (tokens appended, finished
requests released, preempted requests reset to be recomputed from their
prompt).  The reference's counterpart is ``EngineCore``
(src/alofa/engine/core.mojo:83-790: submit, cancel, prepare/decide/settle,
tick, run, output, release).

    engine = Engine("path/to/model", dtype="bfloat16")
    outputs = engine.generate([[1, 2, 3], [4, 5]], max_new_tokens=16)
"""
from __future__ import annotations

import time
from collections import OrderedDict

import torch
from dataclasses import dataclass, field, replace
from typing import Optional, Sequence

from ..config.engine_config import EngineConfig
from ..errors import AlofaError
from ..sampling.params import SamplingParams
from ..sampling.rng import SplitMix64
from .loading import load_model, random_model
from .scheduler import Action, SchedConfig, SchedInput, Scheduler, format_config, format_tick
from .step import StepEntry, StepRunner


@dataclass
class Request:
    id: int
    prompt: list
    params: SamplingParams
    rng: SplitMix64
    output: list = field(default_factory=list)
    slot: Optional[int] = None
    done: bool = False
    preemptions: int = 0


@dataclass
class InFlight:
    """A step that was launched and whose tokens the host has not read yet."""

    owners: list        # the requests whose next token each wanted row yields, in row order
    epochs: list        # their preemption counts at launch: a request preempted since is skipped
    row_of: dict        # request id -> row
    host: "torch.Tensor"  # pinned; the tokens arrive here
    status: "torch.Tensor"  # pinned [1]; the kernels' status word arrives here with the tokens
    event: "torch.cuda.Event"
    finishing: list     # requests the scheduler ended with this step
    kind: str
    rows: int
    t0: float


class Engine:
    """One model on one GPU, serving token-id requests.

    Steps overlap: when every request of a step samples by temperature alone,
    the step is launched with its decoded tokens taken on the device from the
    step before, and only then does the host read that earlier step's tokens.
    The host's bookkeeping thus runs beside the GPU.  A request that meets a
    stop token is seen one step late; the extra row it ran is dropped."""

    def __init__(self, model=None, dtype: Optional[str] = None, config: Optional[EngineConfig] = None, device=None, admission: str = "committed", trace_out=None, _loaded=None, **overrides):
        cfg = replace(config) if config is not None else EngineConfig()
        if dtype is not None:
            cfg.dtype = {"bf16": "bfloat16", "fp32": "float32"}.get(dtype, dtype)
        for key, value in overrides.items():
            if not hasattr(cfg, key):
                raise AlofaError("invalid_argument", "unknown engine setting", f"name={key}")
            setattr(cfg, key, value)
        cfg.validate()
        self.config = cfg
        if _loaded is not None:
            self.model, self.model_config, self.architecture = _loaded
        else:
            if model is None:
                raise AlofaError("invalid_argument", "Engine needs a model folder")
            self.model, self.model_config, self.architecture = load_model(model, cfg.dtype, device)
        spec = self.model.spec
        self.max_tokens = min(cfg.max_tokens, spec.max_position)
        blocks_per_request = -(-self.max_tokens // cfg.block_size)
        capacity = cfg.capacity_blocks or cfg.max_batch * blocks_per_request
        step_tokens = max(cfg.token_budget, cfg.max_batch, 1)
        self.runner = StepRunner(self.model, cfg.block_size, capacity, cfg.max_batch, self.max_tokens, step_tokens, cfg.cuda_graphs)
        groups = [(g.block_size, g.window or 0, g.num_pages) for g in self.runner.group_specs]
        self.sched_config = SchedConfig(
            token_budget=cfg.token_budget, max_chunk=min(cfg.max_chunk, step_tokens), max_batch=cfg.max_batch, max_tokens=self.max_tokens,
            watermark_permille=cfg.watermark_permille, max_wait_ticks=cfg.max_wait_ticks, admission=admission, groups=groups,
        )
        self.scheduler = Scheduler(self.sched_config)
        self._pending = OrderedDict()  # submitted, not yet admitted by the scheduler
        self._live = {}  # admitted
        self._finished = OrderedDict()  # done, output not yet taken
        self._cancels, self._ended = [], []
        self._next_id = 1
        self._trace = open(trace_out, "w") if trace_out else None
        if self._trace:
            self._trace.write(format_config(self.sched_config) + "\n")
        self._inflight: Optional[InFlight] = None
        on_gpu = self.runner.rt.device.type == "cuda"
        pin = (lambda t: t.pin_memory()) if on_gpu else (lambda t: t)
        self._pinned = [pin(torch.zeros(max(step_tokens, 1), dtype=torch.int32)) for _ in range(2)]
        # the status word the kernels raise (a wait that ran out, a token id outside the vocabulary)
        # comes to the host with every step's tokens, behind the same event
        self._pinned_status = [pin(torch.zeros(1, dtype=torch.int32)) for _ in range(2)]
        self._pin_flip = 0
        self.overlap = bool(cfg.overlap_steps) and self.runner.feeds_tokens
        # set to a callable (request ids, logits [rows, vocab] as a float32 numpy array) to see the
        # logits every token is sampled from; steps then run one after the other
        self.logits_sink = None
        self.marks = []  # (time a step's tokens reached the host, kind, rows)
        self.counters = {"ticks": 0, "rows_run": 0, "prefill_rows": 0, "decode_rows": 0, "preempt_total": 0, "steps_prefill": 0, "steps_decode": 0}
        self.timings = {"prefill_ms": [], "decode_ms": []}

    @classmethod
    def from_random(cls, architecture: str, model_config, seed: int, dtype: str = "bfloat16", device=None, generate_on_device: bool = False, **kwargs):
        """An engine over seeded random weights of a typed model configuration."""
        loaded = random_model(architecture, model_config, seed, dtype, device, generate_on_device)
        return cls(dtype=dtype, _loaded=loaded, **kwargs)

    # -- requests -----------------------------------------------------------
    def add_request(self, prompt: Sequence[int], params: Optional[SamplingParams] = None) -> int:
        """Queue a request; returns its id.  Refused at once if it could never
        run: empty prompt, ids outside the vocabulary, longer than the context
        window, or larger than the whole cache."""
        params = params or SamplingParams(temperature=0.0, seed=self.config.seed)
        prompt = [int(t) for t in prompt]
        vocab = self.model.spec.vocab_size
        if not prompt:
            raise AlofaError("invalid_argument", "prompt must hold at least one token")
        if min(prompt) < 0 or max(prompt) >= vocab:
            raise AlofaError("out_of_range", "token id outside the vocabulary", f"vocab={vocab}")
        params.validate(vocab)
        self.scheduler.can_ever_fit(len(prompt), params.max_new_tokens)
        rid = self._next_id
        self._next_id += 1
        self._pending[rid] = Request(rid, prompt, params, SplitMix64(params.seed))
        return rid

    def cancel(self, request_id: int) -> None:
        """Drop a request wherever it is; its pages come back at once."""
        if request_id in self._pending:
            del self._pending[request_id]
            return
        req = self._live.pop(request_id, None)
        if req is None:
            return
        if req.slot is not None:
            self.runner.release(req.slot)
        self._cancels.append(request_id)

    def has_work(self) -> bool:
        return bool(self._pending or self._live or self._inflight is not None)

    def pop_finished(self) -> list:
        """(request id, generated token ids) of requests that ended since the last call."""
        out = [(rid, list(req.output)) for rid, req in self._finished.items()]
        self._finished.clear()
        return out

    # -- one tick -----------------------------------------------------------
    def step(self) -> Action:
        offered = list(self._pending.values())[: self.config.max_batch]
        inp = SchedInput(
            arrivals=[(r.id, len(r.prompt), r.params.max_new_tokens) for r in offered],
            cancels=self._cancels, finished=self._ended, free_pages=self.runner.manager.free_pages(),
        )
        self._cancels, self._ended = [], []
        act = self.scheduler.step(inp)
        if self._trace:
            self._trace.write(format_tick(inp, act) + "\n")
        self.counters["ticks"] += 1
        self.counters["preempt_total"] = act.preempt_total
        for req, status in zip(offered, act.arrival_status):
            if status == 1:
                self._live[req.id] = self._pending.pop(req.id)
            elif status < 0:
                del self._pending[req.id]
                raise AlofaError("capacity", "the scheduler refused a request for good", f"request={req.id} status={status}")
        for rid in act.preempted:  # recompute later from the prompt
            req = self._live[rid]
            self.runner.release(req.slot)
            req.slot = None
            req.output.clear()
            req.rng = SplitMix64(req.params.seed)
            req.preemptions += 1
        # who runs: decoded tokens first, then prompt portions
        plan = []  # (request, prompt range or None, samples)
        for rid in act.decode:
            req = self._live.get(rid)
            if req is not None:
                plan.append((req, None, True))
        for rid, start, end in act.prefill:
            req = self._live[rid]
            if req.slot is None:
                req.slot = self.runner.admit(rid)
            plan.append((req, (start, end), end == len(req.prompt)))
        owners = [req for req, _, samples in plan if samples]
        overlap = self.overlap and self.logits_sink is None and bool(plan) and all(req.params.plain() for req in owners)
        if not overlap:
            self._settle()  # every token is on the host before this step is put together
        fl = self._inflight
        entries = []
        for req, span, samples in plan:
            if span is not None:
                entries.append(self._entry(req, req.prompt[span[0] : span[1]], samples))
            elif req.done or req.id not in self._live:
                owners.remove(req)  # ended by a stop token that settling has just shown
            elif fl is not None and fl.row_of.get(req.id, -1) >= 0 and fl.epochs[fl.row_of[req.id]] == req.preemptions:
                entry = self._entry(req, [0], True)
                entry.feed = fl.row_of[req.id]  # its token is still on the device
                entries.append(entry)
            else:
                entries.append(self._entry(req, [req.output[-1]], True))
        if entries:
            kind = "prefill" if act.prefill else "decode"
            if overlap:
                launched = self._launch(entries, owners, kind, list(act.finished))
                for rid in act.finished:  # their pages come back now (the stream keeps later users behind this step) ...
                    req = self._live.get(rid)
                    if req is not None and req.slot is not None:
                        self.runner.release(req.slot)
                        req.slot = None
                self._settle()
                self._inflight = launched  # ... and their last tokens with this step's
            else:
                self._launch_and_wait(entries, owners, kind)
                for rid in act.finished:
                    self._finish(rid)
        else:
            self._settle()
            for rid in act.finished:
                self._finish(rid)
        return act

    def _entry(self, req: Request, tokens, sample: bool) -> StepEntry:
        if not sample:
            return StepEntry(req.slot, tokens, ())
        p = req.params
        u = req.rng.next_uniform() if p.temperature > 0.0 else 0.0
        return StepEntry(req.slot, tokens, (len(tokens) - 1,), p.temperature, u)

    def _launch(self, entries, owners, kind: str, finishing: list) -> InFlight:
        """Run a step whose rows all sample by temperature alone; its tokens
        are copied to pinned memory behind it and read by :meth:`_settle`."""
        t0 = time.perf_counter()
        rows = sum(len(e.tokens) for e in entries)
        ctx, logits, tokens = self.runner.forward_sampled(entries)
        host, status = self._pinned[self._pin_flip], self._pinned_status[self._pin_flip]
        self._pin_flip ^= 1
        n = len(owners)
        if n:
            host[:n].copy_(tokens[:n], non_blocking=True)
        self.runner.copy_status(status)
        event = torch.cuda.Event()
        event.record()
        return InFlight(owners, [r.preemptions for r in owners], {r.id: i for i, r in enumerate(owners)}, host, status, event, finishing, kind, rows, t0)

    def _settle(self) -> None:
        """Read the tokens of the step in flight, if any, and act on them."""
        fl = self._inflight
        if fl is None:
            return
        self._inflight = None
        fl.event.synchronize()
        self.runner.raise_status(int(fl.status[0]))  # tokens of a step whose kernels gave up are not handed out
        picked = fl.host[: len(fl.owners)].tolist()
        self._account(fl.kind, fl.rows, fl.t0)
        for req, epoch, tok in zip(fl.owners, fl.epochs, picked):
            if req.done or req.preemptions != epoch or req.id not in self._live:
                continue  # cancelled, preempted, or ended a step earlier: the row is dropped
            self._take(req, int(tok))
        for rid in fl.finishing:
            self._finish(rid)

    def _launch_and_wait(self, entries, owners, kind: str) -> None:
        from ..sampling.sampler import sample_rows

        t0 = time.perf_counter()
        rows = sum(len(e.tokens) for e in entries)
        ctx, logits, tokens = self.runner.forward_sampled(entries)
        picked = []
        status = self._pinned_status[self._pin_flip]
        if logits is not None:
            if not all(req.params.plain() for req in owners):
                tokens = sample_rows(ctx, logits, owners)
            self.runner.copy_status(status)
            picked = tokens.cpu().tolist()  # waits for the stream: the status word is on the host too
            if self.logits_sink is not None:
                self.logits_sink([req.id for req in owners], logits[: len(owners)].float().cpu().numpy())
            self.runner.raise_status(int(status[0]))
        # (a portion of a prompt nobody samples from is not waited for: the word stays raised
        # until it is read, so the step that yields the request's first token reports it)
        self._account(kind, rows, t0)
        for req, tok in zip(owners, picked):
            self._take(req, int(tok))

    def _take(self, req: Request, tok: int) -> None:
        req.output.append(tok)
        if tok in req.params.stop_token_ids and len(req.output) < req.params.max_new_tokens:
            self._ended.append(req.id)  # tells the scheduler on the next tick
            self._finish(req.id)

    def _account(self, kind: str, rows: int, t0: float) -> None:
        """Book a step whose tokens have just reached the host.  Its time runs
        from its launch or, if later, from the arrival of the step before: the
        times of overlapping steps then add up to the wall clock."""
        now = time.perf_counter()
        start = max(t0, self.marks[-1][0]) if self.marks else t0
        self.counters["rows_run"] += rows
        self.counters[f"steps_{kind}"] += 1
        self.counters[f"{kind}_rows"] += rows
        self.timings[f"{kind}_ms"].append((now - start) * 1e3)
        self.marks.append((now, kind, rows))
        if len(self.marks) > 4096:
            del self.marks[:2048]

    def _finish(self, rid: int) -> None:
        req = self._live.pop(rid, None)
        if req is None:
            return
        if req.slot is not None:
            self.runner.release(req.slot)
            req.slot = None
        req.done = True
        self._finished[rid] = req

    def run(self, max_ticks: int = 1 << 30) -> None:
        ticks = 0
        while self.has_work():
            self.step()
            ticks += 1
            if ticks >= max_ticks:
                raise AlofaError("state", "engine did not finish within the tick limit", f"max_ticks={max_ticks}")

    # -- the call a user makes ------------------------------------------------
    def generate(self, prompts: Sequence[Sequence[int]], max_new_tokens: int = 16, temperature: float = 0.0, seed: Optional[int] = None,
                 eos_token_id: Optional[int] = None, sampling: Optional[SamplingParams] = None) -> list:
        """Generate for every prompt (token ids in, token ids out); requests
        that do not fit at once wait their turn.  ``sampling`` overrides the
        simple arguments; request ``i`` draws from seed ``seed + i``."""
        base = seed if seed is not None else self.config.seed
        ids = []
        for i, prompt in enumerate(prompts):
            if sampling is not None:
                params = replace(sampling, seed=sampling.seed + i)
            else:
                stops = (eos_token_id,) if eos_token_id is not None else ()
                params = SamplingParams(temperature=temperature, seed=base + i, max_new_tokens=max_new_tokens, stop_token_ids=stops)
            ids.append(self.add_request(prompt, params))
        self.run()
        done = dict(self.pop_finished())
        return [done[rid] for rid in ids]

    def stats(self) -> dict:
        mgr = self.runner.manager
        out = dict(self.counters)
        out.update(self.scheduler.counts())
        out["pending"] = len(self._pending)
        out["free_pages"] = mgr.free_pages()
        out["used_pages"] = [mgr.used_pages(g) for g in range(len(self.runner.group_specs))]
        out["cache_bytes"] = self.runner.storage.bytes
        out["defects"] = mgr.defects()
        return out

    def close(self) -> None:
        if self._trace:
            self._trace.close()
            self._trace = None
