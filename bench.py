#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B] [--shape 0.5b|1.5b|7b] [--no-extra]

The default run has the layer sizes of the Qwen2.5-0.5B shape with random
weights, a batch of 8 requests with 2,048-token prompts inside a 4,096-token
context, and times K decode steps on the device after W warm-up steps.  One
JSON line is printed:

* ``value``: decoded tokens per second at the default batch (device time of K
  steps of the engine's own step function, CUDA events);
* ``e2e``: the same through ``Engine.generate`` (host token ids in, host token
  ids out, every step copying its inputs to the device and its tokens back);
* ``prefill``: one 2,048-token prompt in one step;
* ``roofline``: bytes a decode step has to read (every weight once, the cache
  of the live requests) over its time, against the measured copy bandwidth;
* ``points``: decode at batch 1 and 64, and, unless ``--no-extra``, the other
  measurements: decode at batch 8 and 64 with prompts that fill the 4,096-token
  context; the Qwen2.5-1.5B shape serving 64 requests with prompt lengths
  uniform in [128, 2048] and 256 new tokens each through ``Engine.generate``
  (scheduler included); the Qwen2.5-7B shape at batch 1, 8 and 64 and its
  2,048-token prefill.  ``points_detail`` gives each point's time per step
  (median, min, max over the steps, each step timed by its own event pair), its
  fraction of the roofline from the same formula, and the scheduler's counts.

Method, after the reference's own benchmark (src/alofa/cli.mojo:62-82,
819-850): warm-up first, then every repetition timed on its own and the median
reported with the span; ``value`` itself is the contract's figure, K steps
between one pair of events.

Peaks come from MEASURED_PEAKS.json beside this file when present, else from
the fallback figures 6.65 TB/s and 1.59 PFLOP/s.  Every decode step reads more
than a gigabyte of weights and cache, far more than the 126 MB L2, so no L2
flush is needed between steps (``config.l2``)."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import subprocess
import sys
import threading
import time
from pathlib import Path

ROOT = Path(__file__).resolve().parent
sys.path.insert(0, str(ROOT))

METRIC = "decode tok/s @ batch 8 (Qwen2.5-0.5B shape, 2,048-token prompts, context 4096)"
FALLBACK_PEAKS = {"hbm_gbs": 6650.0, "bf16_tflops": 1590.0}

# the shapes the measurements are quoted on (their published config.json values)
SHAPES = {
    "0.5b": ("Qwen2.5-0.5B shape", dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
                                        intermediate_size=4864, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True,
                                        max_position_embeddings=32768)),
    "1.5b": ("Qwen2.5-1.5B shape", dict(num_hidden_layers=28, hidden_size=1536, num_attention_heads=12, num_key_value_heads=2, head_dim=128,
                                        intermediate_size=8960, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True,
                                        max_position_embeddings=32768)),
    "7b": ("Qwen2.5-7B shape", dict(num_hidden_layers=28, hidden_size=3584, num_attention_heads=28, num_key_value_heads=4, head_dim=128,
                                    intermediate_size=18944, vocab_size=152064, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=False,
                                    max_position_embeddings=32768)),
}
SHAPE = SHAPES["0.5b"][1]
PROMPT_LEN = 2048
CONTEXT = 4096


def _find_number(raw, key):
    """The number under ``key`` anywhere in a nested JSON value (a figure may be
    a bare number or an object with a ``value``); None when absent."""
    if isinstance(raw, dict):
        if key in raw:
            v = raw[key]
            if isinstance(v, dict):
                v = v.get("value")
            try:
                return float(v)
            except (TypeError, ValueError):
                return None
        for v in raw.values():
            found = _find_number(v, key)
            if found is not None:
                return found
    elif isinstance(raw, list):
        for v in raw:
            found = _find_number(v, key)
            if found is not None:
                return found
    return None


def peaks() -> tuple:
    path = ROOT / "MEASURED_PEAKS.json"
    if path.exists():
        try:
            raw = json.loads(path.read_text())
        except ValueError:
            raw = None
        hbm = _find_number(raw, "hbm_gbs")
        # the prefill is timed over a few milliseconds: the burst figure is its denominator
        flops = _find_number(raw, "bf16_tflops") or _find_number(raw, "bf16_tflops_sustained")
        if hbm and flops:
            return {"hbm_gbs": hbm, "bf16_tflops": flops}, "measured"
    return dict(FALLBACK_PEAKS), "fallback"


class ClockSampler:
    """Samples SM clocks and throttle reasons with nvidia-smi while timing."""

    QUERY = "clocks.sm,clocks.max.sm,clocks_event_reasons.hw_slowdown,clocks_event_reasons.hw_thermal_slowdown,clocks_event_reasons.sw_thermal_slowdown,clocks_event_reasons.sw_power_cap"

    def __init__(self):
        self.samples = []
        self.proc = None
        self.begin = 0.0

    def start(self):
        """Start sampling; nvidia-smi takes a moment to give its first line, so
        this goes before the warm-up and :meth:`mark` before the timed steps."""
        try:
            self.proc = subprocess.Popen(["nvidia-smi", "-i", "0", f"--query-gpu={self.QUERY}", "--format=csv,noheader,nounits", "-lms", "20"],
                                         stdout=subprocess.PIPE, stderr=subprocess.DEVNULL, text=True)
        except OSError:
            self.proc = None
            return
        threading.Thread(target=self._read, daemon=True).start()

    def _read(self):
        for line in self.proc.stdout:
            parts = [p.strip() for p in line.split(",")]
            if len(parts) == 6:
                self.samples.append((time.perf_counter(), parts))

    def mark(self):
        """The timed region starts now: only samples from here on count."""
        self.begin = time.perf_counter()

    def stop(self) -> dict:
        if self.proc is None:
            return {"sm_mhz": None, "sm_max_mhz": None, "reasons": ["nvidia-smi unavailable"]}
        self.proc.terminate()
        try:
            self.proc.wait(timeout=5)
        except subprocess.TimeoutExpired:
            self.proc.kill()
        clocks, reasons, max_mhz = [], set(), None
        names = ["hw_slowdown", "hw_thermal_slowdown", "sw_thermal_slowdown", "sw_power_cap"]
        for at, s in self.samples:
            if at < self.begin:
                continue
            try:
                clocks.append(int(s[0]))
                max_mhz = int(s[1])
            except ValueError:
                continue
            for name, flag in zip(names, s[2:]):
                if flag.lower().startswith("active"):
                    reasons.add(name)
        return {"sm_mhz": int(statistics.median(clocks)) if clocks else None, "sm_max_mhz": max_mhz, "reasons": sorted(reasons), "samples": len(clocks)}


def model_numbers(cfg, layers: int) -> dict:
    """Bytes a decode step reads and flops a prefill does, from the sizes."""
    H, I, V = cfg.hidden_size, cfg.intermediate_size, cfg.vocab_size
    q, kv = cfg.num_attention_heads * cfg.head_dim, cfg.num_key_value_heads * cfg.head_dim
    per_layer_params = H * (q + 2 * kv) + (q + 2 * kv) + q * H + 3 * H * I + 2 * H
    weight_bytes = 2 * (layers * per_layer_params + V * H + H)  # bf16; the head (tied table) is read once
    kv_bytes_per_token = layers * 2 * kv * 2
    return {"weight_bytes": weight_bytes, "kv_bytes_per_token": kv_bytes_per_token, "per_layer_matmul_params": H * (q + 2 * kv) + q * H + 3 * H * I, "q": q}


def prefill_flops(cfg, layers: int, tokens: int, numbers: dict) -> float:
    gemm = 2.0 * tokens * layers * numbers["per_layer_matmul_params"]
    attn = layers * 4.0 * numbers["q"] * tokens * (tokens + 1) / 2
    head = 2.0 * cfg.hidden_size * cfg.vocab_size
    return gemm + attn + head


class Bench:
    """One engine of one shape and the measurements made on it."""

    def __init__(self, shape: str, layers: int, max_batch: int, context: int = CONTEXT):
        import numpy as np

        from alofa_b200.engine.engine import Engine
        from alofa_b200.models.qwen2 import NAME, Qwen2Config

        self.label, values = SHAPES[shape]
        values = dict(values)
        self.full_layers = values["num_hidden_layers"]
        values["num_hidden_layers"] = layers or self.full_layers
        self.cfg = Qwen2Config(**values)
        self.layers = self.cfg.num_hidden_layers
        self.engine = Engine.from_random(NAME, self.cfg, seed=0, dtype="bfloat16", generate_on_device=True, block_size=64, max_batch=max_batch,
                                         max_tokens=context, token_budget=PROMPT_LEN + max_batch, max_chunk=PROMPT_LEN)
        self.runner = self.engine.runner
        self.numbers = model_numbers(self.cfg, self.layers)
        self.peaks, self.peaks_kind = peaks()
        self.rng = np.random.default_rng(0)

    def prompt(self, n: int) -> list:
        return [int(t) for t in self.rng.integers(0, self.cfg.vocab_size, size=n)]

    @staticmethod
    def timed_each(fn, reps: int) -> tuple:
        """(mean ms over one pair of events around all repetitions, [ms of each
        repetition by its own pair of events])."""
        import torch

        marks = [torch.cuda.Event(enable_timing=True) for _ in range(reps + 1)]
        torch.cuda.synchronize()
        marks[0].record()
        for i in range(reps):
            fn()
            marks[i + 1].record()
        torch.cuda.synchronize()
        each = [marks[i].elapsed_time(marks[i + 1]) for i in range(reps)]
        return marks[0].elapsed_time(marks[reps]) / reps, each

    @staticmethod
    def spread(each: list) -> dict:
        return {"median": round(statistics.median(each), 4), "min": round(min(each), 4), "max": round(max(each), 4), "n": len(each)}

    def prefill(self, warmup: int, reps: int = 10) -> dict:
        """One 2,048-token prompt in one step, `reps` times; the median."""
        from alofa_b200.engine.step import StepEntry

        tokens = self.prompt(PROMPT_LEN)

        def one():
            slot = self.runner.admit(10_000)
            self.runner.forward_logits([StepEntry(slot, tokens, (PROMPT_LEN - 1,))])
            self.runner.release(slot)

        for _ in range(max(3, warmup)):  # a shape met a third time is recorded as a graph: time what serving replays
            one()
        _, each = self.timed_each(one, reps)
        ms = statistics.median(each)
        flops = prefill_flops(self.cfg, self.layers, PROMPT_LEN, self.numbers)
        return {"value": round(PROMPT_LEN / ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(ms, 4),
                "frac": round(flops / (ms * 1e-3) / (self.peaks["bf16_tflops"] * 1e12), 4), "reps": self.spread(each)}

    def decode(self, batch: int, steps: int, warmup: int, prompt_len: int = PROMPT_LEN, clocks=None) -> dict:
        """`steps` decode steps of `batch` requests whose prompts of `prompt_len`
        tokens were run first, one request per step."""
        import torch

        from alofa_b200.csrc import ops
        from alofa_b200.engine.step import StepEntry

        runner = self.runner
        slots = [runner.admit(20_000 + i) for i in range(batch)]
        for s in slots:
            toks = self.prompt(prompt_len)
            for lo in range(0, prompt_len, PROMPT_LEN):
                runner.forward_logits([StepEntry(s, toks[lo : lo + PROMPT_LEN], ())])
        feed = self.rng.integers(0, self.cfg.vocab_size, size=(steps + warmup, batch))
        state = {"i": 0}

        def one_step():
            toks = feed[state["i"]]
            state["i"] += 1
            runner.forward_sampled([StepEntry(s, (int(t),), (0,)) for s, t in zip(slots, toks)])

        if clocks:
            clocks.start()
        for _ in range(warmup):
            one_step()
        if clocks:
            torch.cuda.synchronize()
            time.sleep(0.3)  # the sampler's first lines
            clocks.mark()
        launches0 = ops.launch_count()
        ms, each = self.timed_each(one_step, steps)
        clock_report = clocks.stop() if clocks else None
        launches = ops.launch_count() - launches0
        mean_kv = prompt_len + warmup + steps / 2
        for s in slots:
            runner.release(s)
        step_bytes = self.numbers["weight_bytes"] + self.numbers["kv_bytes_per_token"] * mean_kv * batch
        achieved = step_bytes / (ms * 1e-3) / 1e9
        return {"ms": ms, "tok_s": batch / ms * 1e3, "bytes": step_bytes, "launches": launches, "clocks": clock_report, "step_ms": self.spread(each),
                "gbs": achieved, "frac": achieved / self.peaks["hbm_gbs"]}

    def detail(self, point: dict) -> dict:
        return {"tok_s": round(point["tok_s"], 1), "ms_per_step": round(point["ms"], 4), "step_ms": point["step_ms"],
                "hbm_gbs": round(point["gbs"], 1), "hbm_frac": round(point["frac"], 4)}

    def serve(self, n_requests: int, new_tokens: int, lo: int, hi: int) -> dict:
        """`n_requests` with prompt lengths uniform in [lo, hi] and `new_tokens`
        new tokens each through Engine.generate, scheduler included; run once
        untimed (records the graphs), then timed by the wall clock."""
        engine = self.engine
        prompts = [self.prompt(int(n)) for n in self.rng.integers(lo, hi + 1, size=n_requests)]
        engine.generate(prompts, max_new_tokens=new_tokens)
        engine.marks.clear()
        before = dict(engine.counters)
        for key in engine.timings:
            engine.timings[key].clear()
        t0 = time.perf_counter()
        outs = engine.generate(prompts, max_new_tokens=new_tokens)
        wall = time.perf_counter() - t0
        made = sum(len(o) for o in outs)
        by_rows = {}
        for _, kind, rows in engine.marks:
            bucket = kind + ":" + ("1-16" if rows <= 16 else "17-64" if rows <= 64 else "65-512" if rows <= 512 else "513+")
            by_rows[bucket] = by_rows.get(bucket, 0) + 1
        stats = engine.stats()
        return {"tok_s": round(made / wall, 1), "wall_s": round(wall, 3), "requests": n_requests, "new_tokens": made,
                "prompt_tokens": sum(len(p) for p in prompts), "ticks": stats["ticks"] - before["ticks"],
                "preemptions": stats["preempt_total"], "steps_by_rows": by_rows,
                "decode_step_ms_median": round(statistics.median(engine.timings["decode_ms"]), 4) if engine.timings["decode_ms"] else None}

    def close(self) -> None:
        import gc

        import torch

        self.engine.close()
        self.engine = self.runner = None
        gc.collect()
        torch.cuda.empty_cache()


def extra_points(args, first: Bench) -> tuple:
    """The measurements beside the headline; each guarded, so that a failure of
    one is reported under its own name and costs nothing else."""
    points, detail = {}, {}

    def guarded(name, fn):
        try:
            fn()
        except Exception as err:  # noqa: BLE001 - reported in the line, never fatal to the headline
            detail[name] = {"error": f"{type(err).__name__}: {err}"[:300]}

    steps = max(64, args.steps // 2)

    def long_context():
        fill = CONTEXT - steps - args.warmup - 8  # prompts that leave room for the timed steps only
        for batch in (8, 64):
            point = first.decode(batch, steps, args.warmup, prompt_len=fill)
            points[f"decode_b{batch}_ctx4096"] = round(point["tok_s"], 1)
            detail[f"decode_b{batch}_ctx4096"] = dict(first.detail(point), prompt_len=fill)

    guarded("decode_ctx4096", long_context)
    first.close()

    def shape_15b():
        bench = Bench("1.5b", 0, 64)
        try:
            served = bench.serve(64, 256, 128, 2048)
            points["qwen2.5-1.5b_serve64_tok_s"] = served["tok_s"]
            detail["qwen2.5-1.5b_serve64"] = served
            point = bench.decode(8, steps, args.warmup)
            points["qwen2.5-1.5b_decode_b8"] = round(point["tok_s"], 1)
            detail["qwen2.5-1.5b_decode_b8"] = bench.detail(point)
        finally:
            bench.close()

    def shape_7b():
        bench = Bench("7b", 0, 64)
        try:
            for batch in (1, 8, 64):
                point = bench.decode(batch, steps, args.warmup)
                points[f"qwen2.5-7b_decode_b{batch}"] = round(point["tok_s"], 1)
                detail[f"qwen2.5-7b_decode_b{batch}"] = bench.detail(point)
            pre = bench.prefill(args.warmup)
            points["qwen2.5-7b_prefill_tok_s"] = pre["value"]
            detail["qwen2.5-7b_prefill"] = pre
        finally:
            bench.close()

    guarded("qwen2.5-1.5b", shape_15b)
    guarded("qwen2.5-7b", shape_7b)
    return points, detail


def run(args) -> dict:
    from alofa_b200.engine.context import Layout

    bench = Bench(args.shape, args.layers, max(64, args.batch))
    cfg, layers, engine, runner = bench.cfg, bench.layers, bench.engine, bench.runner

    if args.phase == "decode":
        prefill = None
    else:
        prefill = bench.prefill(args.warmup)
    if args.phase == "prefill":
        print(json.dumps({"phase": "prefill", "ms": prefill["ms"], "tok_s": prefill["value"], "reps": prefill["reps"]}))
        raise SystemExit(0)

    main = bench.decode(args.batch, args.steps, args.warmup, clocks=ClockSampler())
    if args.phase == "decode":
        print(json.dumps({"phase": "decode", "batch": args.batch, "ms_per_step": main["ms"], "tok_s": main["tok_s"], "launches": main["launches"], "step_ms": main["step_ms"]}))
        raise SystemExit(0)
    b1 = bench.decode(1, max(8, args.steps // 2), args.warmup)
    b64 = bench.decode(64, max(8, args.steps // 2), args.warmup)

    # -- end to end: Engine.generate, host tokens in and out --------------------
    # as many new tokens as timed steps: the requests start and end a tick apart each, so a short
    # run is mostly steps with fewer rows than the batch
    e2e_new = max(8, min(256, args.steps))
    prompts = [bench.prompt(PROMPT_LEN) for _ in range(args.batch)]
    engine.generate(prompts, max_new_tokens=e2e_new)  # the same run once untimed: records the CUDA graphs it uses
    engine.marks.clear()
    rows_before = engine.counters["decode_rows"]
    t0 = time.perf_counter()
    outs = engine.generate(prompts, max_new_tokens=e2e_new)
    wall = time.perf_counter() - t0
    # wall clock of the decoding part: from the arrival of the last step that held a prompt portion
    # to the arrival of the last tokens, scheduler and bookkeeping included
    last_prefill = max((t for t, kind, _ in engine.marks if kind == "prefill"), default=t0)
    decode_wall = max((t for t, kind, _ in engine.marks if kind == "decode"), default=last_prefill) - last_prefill
    decode_rows = sum(rows for t, kind, rows in engine.marks if kind == "decode" and t > last_prefill)
    assert decode_rows <= engine.counters["decode_rows"] - rows_before
    e2e_value = decode_rows / decode_wall if decode_wall > 0 else None

    h2d = Layout.make(args.batch, args.batch, args.batch, runner._group_shapes).total * 4
    points = {"decode_b1": round(b1["tok_s"], 1), "decode_b64": round(b64["tok_s"], 1)}
    detail = {"decode_b1": bench.detail(b1), f"decode_b{args.batch}": bench.detail(main), "decode_b64": bench.detail(b64)}
    if args.extra and args.shape == "0.5b" and not args.layers:
        more_points, more_detail = extra_points(args, bench)
        points.update(more_points)
        detail.update(more_detail)
    metric = METRIC if args.shape == "0.5b" else METRIC.replace("Qwen2.5-0.5B shape", bench.label)
    result = {
        "metric": metric, "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, uniform random token ids", "impl": "alofa_b200",
        "config": {
            "model": bench.label, "layers": layers, "layers_full": bench.full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "block_size": 64, "parallelism": "single GPU",
            "l2": "inputs>L2 (each step reads >1 GB)", "peaks": bench.peaks_kind,
        },
        "e2e": {"value": round(e2e_value, 1) if e2e_value else None, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch + 4,
                "new_tokens": e2e_new, "wall_s_with_prefill": round(wall, 3), "outputs": len(outs)},
        "gpu_launches": main["launches"],
        "prefill": {k: v for k, v in prefill.items() if k != "reps"},
        "roofline": {"bound": "hbm", "achieved": round(main["gbs"], 1), "peak": bench.peaks["hbm_gbs"], "unit": "GB/s", "frac": round(main["frac"], 4)},
        "points": points,
        "step_ms": main["step_ms"],
        "prefill_reps": prefill["reps"],
        "points_detail": detail,
        "clocks": main["clocks"],
    }
    return result


def reference_arm() -> dict:
    """The reference is a Mojo project: it has no Python package to install and
    neither `mojo` nor `pixi` exists in this image, so it cannot run here."""
    return {"impl": "reference", "unavailable": "mojothon/alofa is pure Mojo (no setup.py/pyproject; pip finds nothing to install) and no Mojo toolchain is in the image; CPU-only in any case"}


def main() -> int:
    ap = argparse.ArgumentParser()
    ap.add_argument("--gpus", type=int, default=1)
    ap.add_argument("--steps", type=int, default=256)
    ap.add_argument("--warmup", type=int, default=4)
    ap.add_argument("--impl", default="alofa_b200")
    ap.add_argument("--batch", type=int, default=8)
    ap.add_argument("--layers", type=int, default=0, help="fewer layers than the full shape (named in config)")
    ap.add_argument("--phase", choices=["all", "decode", "prefill"], default="all", help="profiling aid: run only one part; the JSON line then lacks the others")
    ap.add_argument("--shape", choices=sorted(SHAPES), default="0.5b", help="whose layer sizes the headline run has")
    ap.add_argument("--no-extra", dest="extra", action="store_false", help="leave out the measurements beside the headline (long contexts, the 1.5B and 7B shapes)")
    args = ap.parse_args()
    if args.impl == "reference":
        print(json.dumps(reference_arm()))
        return 0
    if args.gpus != 1 or int(os.environ.get("WORLD_SIZE", "1")) != 1:
        print(f"bench.py: this engine runs on one GPU; --gpus {args.gpus} is not supported")
        return 2
    args.warmup = max(args.warmup, 3)
    print(json.dumps(run(args)))
    return 0


if __name__ == "__main__":
    sys.exit(main())
