"""The scheduler's Python face and its text traces.

The state machine itself is C++ (``csrc/host/scheduler.cpp``): a pure
``step(state, input) -> action`` with no I/O, clock or allocation, after the
reference's ``Scheduler.step`` (src/alofa/engine/scheduler.mojo:639-767).  This
module wraps it in dataclasses and records or replays its decisions as text,
one line per tick, in the manner of the reference's trace format
(src/alofa/engine/trace.mojo:63-238): integers only, ``-`` for an empty list."""
from __future__ import annotations

import ctypes
from dataclasses import dataclass, field

from ..csrc.build import load_library
from ..errors import AlofaError

ADMISSION = {"committed": 0, "optimistic": 1}
_lib = None


def _native():
    global _lib
    if _lib is None:
        lib = load_library("alofa_scheduler", ["host/scheduler.cpp"], cuda=False)
        P, I = ctypes.c_void_p, ctypes.c_int
        lib.sched_create.restype = P
        lib.sched_create.argtypes = [P, I]
        lib.sched_destroy.restype = None
        lib.sched_destroy.argtypes = [P]
        lib.sched_can_ever_fit.restype = I
        lib.sched_can_ever_fit.argtypes = [P, I, I]
        lib.sched_step.restype = I
        lib.sched_step.argtypes = [P, P, P, P, I, P, I, P, I, P, P, P, P, P, P, P, P, P, P]
        lib.sched_counts.restype = None
        lib.sched_counts.argtypes = [P, P]
        lib.sched_request.restype = I
        lib.sched_request.argtypes = [P, ctypes.c_int64, P]
        _lib = lib
    return _lib


@dataclass
class SchedConfig:
    """``groups``: one ``(page_size, window, capacity_pages)`` per cache group
    (window 0 = all keys).  ``admission``: "committed" admits a request only
    if every live request could grow to its full length beside it (nothing is
    ever preempted); "optimistic" admits while the prompts fit and lets decode
    growth preempt the newest running request."""

    token_budget: int = 256
    max_chunk: int = 64
    max_batch: int = 32
    max_tokens: int = 4096
    watermark_permille: int = 900
    max_wait_ticks: int = 8
    admission: str = "committed"
    groups: list = field(default_factory=lambda: [(16, 0, 1024)])

    def as_ints(self) -> list:
        if self.admission not in ADMISSION:
            raise AlofaError("invalid_argument", "admission must be committed or optimistic", f"admission={self.admission}")
        out = [self.token_budget, self.max_chunk, self.max_batch, self.max_tokens, self.watermark_permille, self.max_wait_ticks, ADMISSION[self.admission], len(self.groups)]
        for ps, win, cap in self.groups:
            out += [ps, win or 0, cap]
        return out


@dataclass
class SchedInput:
    """What happened since the last tick.  ``free_pages``: the cache manager's
    count per group at the moment of the call (the one book of pages)."""

    arrivals: list = field(default_factory=list)  # (id, prompt_len, max_new)
    cancels: list = field(default_factory=list)
    finished: list = field(default_factory=list)  # ended by the engine (stop token)
    free_pages: list = field(default_factory=list)


@dataclass
class Action:
    """What to run this tick.  ``arrival_status`` per arrival: 1 admitted,
    0 deferred (offer again), 2 blocked by a cancel, negative refused."""

    prefill: list  # (id, start, end)
    decode: list
    preempted: list
    finished: list
    arrival_status: list
    tick_seq: int
    preempt_total: int
    digest: int

    def tokens(self) -> int:
        return len(self.decode) + sum(e - s for _, s, e in self.prefill)


_STEP_ERRORS = {-2: ("invalid_argument", "bad scheduler call"), -4: ("capacity", "kv pool too small for this batch"), -5: ("out_of_range", "request is longer than max_tokens")}


class Scheduler:
    def __init__(self, cfg: SchedConfig):
        self.cfg = cfg
        ints = cfg.as_ints()
        arr = (ctypes.c_int * len(ints))(*ints)
        self._h = _native().sched_create(arr, len(ints))
        if not self._h:
            raise AlofaError("invalid_argument", "scheduler refused its configuration", f"cfg={cfg}")
        n = cfg.max_batch
        L, I = ctypes.c_int64, ctypes.c_int
        self._p_id, self._d_id, self._x_id, self._f_id = (L * n)(), (L * n)(), (L * n)(), (L * n)()
        self._p_start, self._p_end = (I * n)(), (I * n)()
        self._counts, self._info = (I * 4)(), (L * 3)()

    def __del__(self):
        h, self._h = getattr(self, "_h", None), None
        if h and _lib is not None:
            _lib.sched_destroy(h)

    def can_ever_fit(self, prompt_len: int, max_new: int) -> None:
        rc = _lib.sched_can_ever_fit(self._h, prompt_len, max_new)
        if rc != 0:
            code, text = _STEP_ERRORS.get(rc, ("invalid_argument", "request refused"))
            if rc == -4:
                text = "request does not fit in the kv pool even alone"
            raise AlofaError(code, text, f"prompt_len={prompt_len} max_new={max_new}")

    def step(self, inp: SchedInput) -> Action:
        L, I = ctypes.c_int64, ctypes.c_int
        na, nc, nf = len(inp.arrivals), len(inp.cancels), len(inp.finished)
        if len(inp.free_pages) != len(self.cfg.groups):
            raise AlofaError("invalid_argument", "free_pages must have one count per cache group", f"got={inp.free_pages}")
        a_id = (L * max(na, 1))(*[a[0] for a in inp.arrivals])
        a_pl = (I * max(na, 1))(*[a[1] for a in inp.arrivals])
        a_mn = (I * max(na, 1))(*[a[2] for a in inp.arrivals])
        a_st = (I * max(na, 1))()
        c_id = (L * max(nc, 1))(*inp.cancels)
        f_id = (L * max(nf, 1))(*inp.finished)
        free = (I * len(inp.free_pages))(*inp.free_pages)
        rc = _lib.sched_step(
            self._h, a_id, a_pl, a_mn, na, c_id, nc, f_id, nf, free, a_st,
            self._p_id, self._p_start, self._p_end, self._d_id, self._x_id, self._f_id, self._counts, self._info,
        )
        if rc != 0:
            code, text = _STEP_ERRORS.get(rc, ("state", "scheduler error"))
            raise AlofaError(code, text, f"rc={rc}")
        npf, nd, nx, nfin = self._counts
        return Action(
            prefill=[(self._p_id[i], self._p_start[i], self._p_end[i]) for i in range(npf)],
            decode=list(self._d_id[:nd]),
            preempted=list(self._x_id[:nx]),
            finished=list(self._f_id[:nfin]),
            arrival_status=list(a_st[:na]),
            tick_seq=self._info[0],
            preempt_total=self._info[1],
            digest=self._info[2],
        )

    def counts(self) -> dict:
        out = (ctypes.c_int * 3)()
        _lib.sched_counts(self._h, out)
        return {"live": out[0], "waiting": out[1], "running": out[2]}

    def request(self, request_id: int):
        out = (ctypes.c_int * 8)()
        if _lib.sched_request(self._h, request_id, out) != 0:
            return None
        keys = ("state", "prompt_len", "max_new", "done", "n_out", "wait_ticks", "preempt_count", "cache_len")
        return dict(zip(keys, out))


# -- text traces ------------------------------------------------------------
def _ids(values) -> str:
    return ",".join(str(v) for v in values) if values else "-"


def _triples(values) -> str:
    return ",".join(":".join(str(x) for x in t) for t in values) if values else "-"


def format_config(cfg: SchedConfig) -> str:
    return (
        f"CFG b={cfg.token_budget} c={cfg.max_chunk} n={cfg.max_batch} m={cfg.max_tokens} w={cfg.watermark_permille} "
        f"t={cfg.max_wait_ticks} a={ADMISSION[cfg.admission]} G={_triples([(p, w or 0, c) for p, w, c in cfg.groups])}"
    )


def format_tick(inp: SchedInput, act: Action) -> str:
    return (
        f"IN=A={_triples(inp.arrivals)}|C={_ids(inp.cancels)}|F={_ids(inp.finished)}|R={_ids(inp.free_pages)} "
        f"OUT=t={act.tick_seq} S={_ids(act.arrival_status)} P={_triples(act.prefill)} D={_ids(act.decode)} "
        f"X={_ids(act.preempted)} F={_ids(act.finished)} C={act.preempt_total} K={act.digest}"
    )


def _parse_ids(text: str) -> list:
    return [] if text == "-" else [int(x) for x in text.split(",")]


def _parse_triples(text: str) -> list:
    return [] if text == "-" else [tuple(int(x) for x in t.split(":")) for t in text.split(",")]


def parse_config(line: str) -> SchedConfig:
    if not line.startswith("CFG "):
        raise AlofaError("parse", "a scheduler trace starts with a CFG line", f"line={line!r}")
    kv = dict(item.split("=", 1) for item in line[4:].split())
    try:
        names = {v: k for k, v in ADMISSION.items()}
        return SchedConfig(
            token_budget=int(kv["b"]), max_chunk=int(kv["c"]), max_batch=int(kv["n"]), max_tokens=int(kv["m"]),
            watermark_permille=int(kv["w"]), max_wait_ticks=int(kv["t"]), admission=names[int(kv["a"])],
            groups=[tuple(t) for t in _parse_triples(kv["G"])],
        )
    except (KeyError, ValueError) as err:
        raise AlofaError("parse", "malformed CFG line", f"line={line!r}: {err}") from err


def parse_tick(line: str) -> SchedInput:
    """The input half of a tick line."""
    try:
        head = line.split(" OUT=", 1)[0]
        if not head.startswith("IN="):
            raise ValueError("no IN=")
        fields = dict(item.split("=", 1) for item in head[3:].split("|"))
        return SchedInput(_parse_triples(fields["A"]), _parse_ids(fields["C"]), _parse_ids(fields["F"]), _parse_ids(fields["R"]))
    except (KeyError, ValueError) as err:
        raise AlofaError("parse", "malformed tick line", f"line={line!r}: {err}") from err


def replay_trace(text: str) -> list:
    """Run a recorded trace through a fresh scheduler; returns the lines
    (number, recorded, replayed) that differ."""
    lines = [ln for ln in text.splitlines() if ln.strip()]
    sched = Scheduler(parse_config(lines[0]))
    bad = []
    for no, line in enumerate(lines[1:], start=2):
        inp = parse_tick(line)
        again = format_tick(inp, sched.step(inp))
        if again != line:
            bad.append((no, line, again))
    return bad
