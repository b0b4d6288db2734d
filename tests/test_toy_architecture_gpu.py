"""A second architecture without a change to the package: ``ToyForCausalLM``
(tests/toy_architecture.py) is registered by importing a module, its folder is
written by the stock random-weights writer, and it runs through
``Engine.generate``, ``bin/generate`` and ``bin/trace_run`` (which find it
through ALOFA_PLUGINS), against its own plain restatement.  One variant keeps
fixed-size state only: it gets no page group at all, and the scheduler admits
by request slots alone.  The other mixes paged attention (layer 0) with state
(layer 1) in a pool so small that requests owning a state slot are preempted
and recomputed."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import replay

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


@pytest.fixture(scope="module")
def toy(tmp_path_factory):
    import toy_architecture as t
    from alofa_b200.weights.random_init import write_random_model
    from alofa_b200.weights.safetensors_io import SafeTensorFile

    base = tmp_path_factory.mktemp("toy_models")
    out = {}
    for name, cfg, seed in (("state", t.ToyConfig(("mean", "mean", "mean")), 5), ("mixed", t.ToyConfig(("attention", "mean")), 6)):
        folder = write_random_model(base / name, t.NAME, cfg, seed, torch.bfloat16)
        st = SafeTensorFile(folder / "model.safetensors")
        w = {n: st.tensor(n).to(torch.float64).numpy() for n in st.names()}
        st.close()
        out[name] = (folder, cfg, w)
    return out


def plugin_env():
    env = dict(os.environ)
    env["ALOFA_PLUGINS"] = "toy_architecture"
    env["PYTHONPATH"] = str(ROOT / "tests") + os.pathsep + env.get("PYTHONPATH", "")
    return env


def prompts_for(cfg, lengths, seed=0):
    rng = np.random.default_rng(seed)
    return [[int(t) for t in rng.integers(0, cfg.vocab, n)] for n in lengths]


def test_state_only_model_books_no_pages_and_generates(toy):
    import toy_architecture as t
    from alofa_b200.engine.engine import Engine

    folder, cfg, w = toy["state"]
    eng = Engine(str(folder), dtype="float32", block_size=16, max_batch=3, token_budget=32, max_chunk=16, max_tokens=96)
    assert eng.architecture.name == t.NAME
    assert eng.runner.group_specs == [] and eng.sched_config.groups == [] and not eng.runner.has_paged
    prompts = prompts_for(cfg, [5, 17, 33, 1, 9])  # five requests through three slots: admission is bounded by slots alone
    want = [t.plain_greedy(p, 6, w, cfg) for p in prompts]
    assert eng.generate(prompts, max_new_tokens=6) == want
    stats = eng.stats()
    assert stats["defects"] == 0 and stats["live"] == 0 and stats["used_pages"] == [] and stats["free_pages"] == [] and stats["preempt_total"] == 0
    assert stats["cache_bytes"] == 3 * 3 * (cfg.hidden + 1) * 4  # three layers, three slots, the state alone


def test_state_slot_owner_is_preempted_and_recomputed(toy):
    import toy_architecture as t
    from alofa_b200.engine.engine import Engine

    folder, cfg, w = toy["mixed"]
    prompts = prompts_for(cfg, [30, 31, 29], seed=1)
    want = [t.plain_greedy(p, 20, w, cfg) for p in prompts]
    eng = Engine(str(folder), dtype="float32", block_size=16, max_batch=4, token_budget=64, max_chunk=32, max_tokens=96, capacity_blocks=7, admission="optimistic")
    assert len(eng.runner.group_specs) == 1
    assert eng.generate(prompts, max_new_tokens=20) == want
    stats = eng.stats()
    assert stats["preempt_total"] > 0, "the pool was meant to be too small"
    assert stats["defects"] == 0 and stats["free_pages"] == [7]


@pytest.mark.parametrize("name", ["state", "mixed"])
def test_command_line_programs_find_the_architecture_through_the_plugin_variable(toy, tmp_path, name):
    import toy_architecture as t

    folder, cfg, w = toy[name]
    prompts = prompts_for(cfg, [9, 21], seed=2)
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--model", str(folder), "--dtype", "float32", "--max-new-tokens", "5", "--block-size", "16",
           "--max-tokens", "96", "--token-budget", "32", "--max-chunk", "16", "--max-batch", "2", "--json"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env=plugin_env())
    assert out.returncode == 0, out.stderr[-2000:]
    assert json.loads(out.stdout.strip().splitlines()[-1])["out_ids"] == [t.plain_greedy(p, 5, w, cfg) for p in prompts]
    # without the plugin the architecture is unknown, and the refusal lists what is known
    bare = subprocess.run(cmd, capture_output=True, text=True, timeout=300, env={k: v for k, v in plugin_env().items() if k != "ALOFA_PLUGINS"})
    assert bare.returncode != 0 and "ToyForCausalLM" in bare.stderr and "Qwen2ForCausalLM" in bare.stderr


@pytest.mark.parametrize("name", ["state", "mixed"])
def test_trace_replay_of_the_toy_architecture(toy, tmp_path, monkeypatch, name):
    import toy_architecture as t

    folder, cfg, w = toy[name]
    for key, value in plugin_env().items():
        if key in ("ALOFA_PLUGINS", "PYTHONPATH"):
            monkeypatch.setenv(key, value)
    reqs = {f"r{i}": p for i, p in enumerate(prompts_for(cfg, [40, 23, 61, 12], seed=3))}
    prompt_lens = {rid: len(p) - 8 for rid, p in reqs.items()}
    steps = replay.mixed(reqs, prompt_lens, 192, 64, seed=1)
    assert max(len(s["entries"]) for s in steps) > 1
    out = replay.run_trace_program(folder, "float32", steps, tmp_path / "out", 192)
    got = replay.collect(steps, out, cfg.vocab)
    for rid, toks in reqs.items():
        ref = t.plain_forward(toks, w, cfg)
        diff = np.abs(got[rid] - ref).max()
        assert diff <= 2e-5 * max(1.0, float(np.abs(ref).max())), f"{name}/{rid}: {diff:.3e}"
