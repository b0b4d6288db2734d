"""Building and running replay schedules for the tests.

A schedule is a list of steps in the JSON form ``bin/trace_run`` reads.  The
builders below cut the same requests in different ways; ``run_inprocess``
drives a StepRunner the way bin/trace_run does, ``run_trace_program`` drives
the program itself.  ``collect`` turns a run's outputs into, per request, the
logits at every position, for comparison with the plain implementation."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np

ROOT = Path(__file__).resolve().parents[1]


def whole(requests):
    """Each request alone, all its tokens in one step."""
    steps = []
    for rid, toks in requests.items():
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks, "want": list(range(len(toks)))}], "end": [rid]})
    return steps


def tail_decoded(requests, tail=32):
    """Most of a request in one step, its last ``tail`` tokens one by one."""
    steps = []
    for rid, toks in requests.items():
        head = max(1, len(toks) - tail)
        steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[:head], "want": list(range(head))}], "end": []})
        for i in range(head, len(toks)):
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": [toks[i]], "want": [0]}], "end": [rid] if i == len(toks) - 1 else []})
        if head == len(toks):
            steps[-1]["end"] = [rid]
    return steps


def portions(requests, sizes=(7, 2, 16, 3, 2, 33, 5, 2, 64, 2, 9)):
    """Each request alone, in portions of changing size, down to two tokens."""
    steps = []
    k = 0
    for rid, toks in requests.items():
        at = 0
        while at < len(toks):
            n = min(sizes[k % len(sizes)], len(toks) - at)
            k += 1
            last = at + n == len(toks)
            steps.append({"step": len(steps), "entries": [{"id": rid, "tokens": toks[at : at + n], "want": list(range(n))}], "end": [rid] if last else []})
            at += n
    return steps


def mixed(requests, prompt_lens, max_tokens, block, seed=0, max_live=4):
    """Up to ``max_live`` requests at a time: portions of prompts beside single
    decoded tokens, requests skipping steps, admitted only while the pool of
    ``max_tokens`` (each request rounded up to ``block``) holds them, so pages
    are given back and used again."""
    rng = np.random.default_rng(seed)
    waiting = list(requests)
    live, fed, steps = [], {}, []

    def need(rid):
        return -(-len(requests[rid]) // block) * block

    while waiting or live:
        while waiting and len(live) < max_live and sum(need(r) for r in live) + need(waiting[0]) <= max_tokens:
            rid = waiting.pop(0)
            live.append(rid)
            fed[rid] = 0
        assert live, "pool too small for the next request"
        chosen = [r for r in live if rng.random() < 0.75] or [live[int(rng.integers(len(live)))]]
        entries, ended = [], []
        for rid in chosen:
            toks, at = requests[rid], fed[rid]
            if at < prompt_lens[rid]:
                left = prompt_lens[rid] - at
                n = int(min(left, rng.choice([2, 3, 5, 8, 16, 17, 31, 40])))
                if left - n == 1:  # never leave a single prompt token over
                    n += 1
            else:
                n = 1
            entries.append({"id": rid, "tokens": toks[at : at + n], "want": list(range(n))})
            fed[rid] = at + n
            if fed[rid] == len(toks):
                ended.append(rid)
        steps.append({"step": len(steps), "entries": entries, "end": ended})
        for rid in ended:
            live.remove(rid)
    return steps


def run_inprocess(runner, steps):
    """The loop of bin/trace_run over a StepRunner; step -> logits array."""
    from alofa_b200.engine.step import StepEntry

    slots, out, next_id = {}, {}, 0
    for step in steps:
        entries = []
        for e in step["entries"]:
            if e["id"] not in slots:
                slots[e["id"]] = runner.admit(next_id)
                next_id += 1
            entries.append(StepEntry(slots[e["id"]], e["tokens"], e.get("want", [])))
        if entries:
            logits = runner.forward(entries)
            if logits is not None:
                out[step["step"]] = logits.float().cpu().numpy()
        for rid in step.get("end", []):
            runner.release(slots.pop(rid))
    runner.check_status()
    assert runner.manager.defects() == 0
    return out


def run_trace_program(model, dtype, steps, out_dir, max_tokens, extra=()):
    """Feed ``steps`` to bin/trace_run one by one, waiting for each ``done``."""
    out_dir = Path(out_dir)
    cmd = [sys.executable, str(ROOT / "bin" / "trace_run"), "--model", str(model), "--dtype", dtype, "--out", str(out_dir), "--max-tokens", str(max_tokens), *extra]
    proc = subprocess.Popen(cmd, stdin=subprocess.PIPE, stdout=subprocess.PIPE, text=True)
    try:
        for step in steps:
            proc.stdin.write(json.dumps(step) + "\n")
            proc.stdin.flush()
            line = proc.stdout.readline().strip()
            assert line == f"done {step['step']}", f"trace_run said {line!r} (exit {proc.poll()})"
        proc.stdin.close()
        assert proc.wait(timeout=120) == 0
    finally:
        if proc.poll() is None:
            proc.kill()
    out = {}
    for step in steps:
        path = out_dir / f"{step['step']}.f32"
        if path.exists():
            out[step["step"]] = np.fromfile(path, dtype="<f4")
    return out


def collect(steps, outputs, vocab):
    """request -> [positions, vocab] logits, from a run's per-step outputs."""
    rows = {}
    for step in steps:
        wanted = sum(len(e.get("want", [])) for e in step["entries"])
        if not wanted:
            continue
        block = np.asarray(outputs[step["step"]]).reshape(wanted, vocab)
        at = 0
        for e in step["entries"]:
            for _ in e.get("want", []):
                rows.setdefault(e["id"], []).append(block[at])
                at += 1
    return {rid: np.stack(r) for rid, r in rows.items()}
