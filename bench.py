#!/usr/bin/env python3
"""Decode and prefill throughput of the engine on one B200.

    python bench.py [--gpus 1] [--steps K] [--warmup W] [--layers L] [--batch B]

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
* ``points``: decode at batch 1 and 64.

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

# Qwen2.5-0.5B shape
SHAPE = dict(num_hidden_layers=24, hidden_size=896, num_attention_heads=14, num_key_value_heads=2, head_dim=64,
             intermediate_size=4864, vocab_size=151936, rms_norm_eps=1e-6, rope_theta=1e6, tie_word_embeddings=True,
             max_position_embeddings=32768)
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


def run(args) -> dict:
    import numpy as np
    import torch

    from alofa_b200.csrc import ops
    from alofa_b200.engine.engine import Engine
    from alofa_b200.engine.step import StepEntry
    from alofa_b200.models.qwen2 import NAME, Qwen2Config

    shape = dict(SHAPE)
    full_layers = shape["num_hidden_layers"]
    shape["num_hidden_layers"] = args.layers or full_layers
    cfg = Qwen2Config(**shape)
    layers = cfg.num_hidden_layers
    max_batch = max(64, args.batch)
    engine = Engine.from_random(NAME, cfg, seed=0, dtype="bfloat16", generate_on_device=True, block_size=64, max_batch=max_batch,
                                max_tokens=CONTEXT, token_budget=PROMPT_LEN + max_batch, max_chunk=PROMPT_LEN)
    runner = engine.runner
    numbers = model_numbers(cfg, layers)
    pk, pk_kind = peaks()
    rng = np.random.default_rng(0)
    vocab = cfg.vocab_size

    def prompt(n):
        return [int(t) for t in rng.integers(0, vocab, size=n)]

    def timed(fn, reps):
        start, end = torch.cuda.Event(enable_timing=True), torch.cuda.Event(enable_timing=True)
        torch.cuda.synchronize()
        start.record()
        for _ in range(reps):
            fn()
        end.record()
        torch.cuda.synchronize()
        return start.elapsed_time(end) / reps

    # -- prefill: one 2,048-token prompt in one step --------------------------
    def one_prefill():
        slot = runner.admit(10_000)
        runner.forward_logits([StepEntry(slot, prefill_tokens, (PROMPT_LEN - 1,))])
        runner.release(slot)

    prefill_tokens = prompt(PROMPT_LEN)
    if args.phase == "decode":
        prefill_ms = float("nan")
    else:
        for _ in range(max(1, min(args.warmup, 3))):
            one_prefill()
        prefill_ms = timed(one_prefill, 5)
    if args.phase == "prefill":
        print(json.dumps({"phase": "prefill", "ms": prefill_ms, "tok_s": PROMPT_LEN / prefill_ms * 1e3}))
        raise SystemExit(0)
    pf = prefill_flops(cfg, layers, PROMPT_LEN, numbers)
    prefill = {"value": round(PROMPT_LEN / prefill_ms * 1e3, 1), "tokens": PROMPT_LEN, "ms": round(prefill_ms, 4),
               "frac": round(pf / (prefill_ms * 1e-3) / (pk["bf16_tflops"] * 1e12), 4)}

    # -- decode ---------------------------------------------------------------
    def decode_point(batch, steps, warmup, clocks=None):
        slots = [runner.admit(20_000 + i) for i in range(batch)]
        for s in slots:  # 2,048-token prompts, one request per step
            runner.forward_logits([StepEntry(s, prompt(PROMPT_LEN), ())])
        feed = rng.integers(0, vocab, size=(steps + warmup, batch))
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
        ms = timed(one_step, steps)
        clock_report = clocks.stop() if clocks else None
        launches = ops.launch_count() - launches0
        mean_kv = PROMPT_LEN + warmup + steps / 2
        for s in slots:
            runner.release(s)
        step_bytes = numbers["weight_bytes"] + numbers["kv_bytes_per_token"] * mean_kv * batch
        return {"ms": ms, "tok_s": batch / ms * 1e3, "bytes": step_bytes, "launches": launches, "clocks": clock_report}

    main = decode_point(args.batch, args.steps, args.warmup, ClockSampler())
    if args.phase == "decode":
        print(json.dumps({"phase": "decode", "batch": args.batch, "ms_per_step": main["ms"], "tok_s": main["tok_s"], "launches": main["launches"]}))
        raise SystemExit(0)
    b1 = decode_point(1, max(8, args.steps // 2), args.warmup)
    b64 = decode_point(64, max(8, args.steps // 2), args.warmup)
    achieved = main["bytes"] / (main["ms"] * 1e-3) / 1e9

    # -- end to end: Engine.generate, host tokens in and out --------------------
    # as many new tokens as timed steps: the requests start and end a tick apart each, so a short
    # run is mostly steps with fewer rows than the batch
    e2e_new = max(8, min(256, args.steps))
    prompts = [prompt(PROMPT_LEN) for _ in range(args.batch)]
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
    from alofa_b200.engine.context import Layout

    h2d = Layout.make(args.batch, args.batch, args.batch, runner._group_shapes).total * 4
    result = {
        "metric": METRIC, "value": round(main["tok_s"], 1), "unit": "tok/s", "n_gpus": 1, "steps": args.steps, "warmup": args.warmup,
        "ms_per_step": round(main["ms"], 4), "higher_is_better": True, "scaling": "weak", "vs_baseline": None, "dtype": "bf16",
        "data": "synthetic: seeded random weights, uniform random token ids", "impl": "alofa_b200",
        "config": {
            "model": "Qwen2.5-0.5B shape", "layers": layers, "layers_full": full_layers, "hidden": cfg.hidden_size, "heads": cfg.num_attention_heads,
            "kv_heads": cfg.num_key_value_heads, "head_dim": cfg.head_dim, "intermediate": cfg.intermediate_size, "vocab": cfg.vocab_size,
            "global_batch": args.batch, "prompt_len": PROMPT_LEN, "seq_len": CONTEXT, "block_size": 64, "parallelism": "single GPU",
            "l2": "inputs>L2 (each step reads >1 GB)", "peaks": pk_kind,
        },
        "e2e": {"value": round(e2e_value, 1) if e2e_value else None, "unit": "tok/s", "h2d_bytes_per_step": h2d, "d2h_bytes_per_step": 4 * args.batch,
                "new_tokens": e2e_new, "wall_s_with_prefill": round(wall, 3), "outputs": len(outs)},
        "gpu_launches": main["launches"],
        "prefill": prefill,
        "roofline": {"bound": "hbm", "achieved": round(achieved, 1), "peak": pk["hbm_gbs"], "unit": "GB/s", "frac": round(achieved / pk["hbm_gbs"], 4)},
        "points": {"decode_b1": round(b1["tok_s"], 1), "decode_b64": round(b64["tok_s"], 1)},
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
