"""Generation through the entry points: greedy against the plain
implementation, sampling that does not depend on the batch, what happens when
pages run out, the command line, and refusals."""
import json
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import tiny

pytestmark = pytest.mark.gpu
ROOT = Path(__file__).resolve().parents[1]


def engine(folder, dtype="float32", **kw):
    from alofa_b200.engine.engine import Engine

    args = dict(block_size=16, max_batch=4, token_budget=24, max_chunk=16, max_tokens=128)
    args.update(kw)
    return Engine(str(folder), dtype=dtype, **args)


def near_plain_maximum(prompt, out, wts, cfg, tol=4e-2):
    seq = list(prompt)
    for tok in out:
        row = plain.forward(seq, wts, cfg)[-1]
        assert row.max() - row[tok] <= tol * max(1.0, float(np.abs(row).max()))
        seq.append(tok)


@pytest.mark.parametrize("name", ["A", "B", "C"])
def test_greedy_generation_matches_plain(model_folders, name):
    wts, cfg = plain.load(model_folders[name])
    prompts = [tiny.tokens(name, n, seed=i) for i, n in enumerate([5, 17, 33, 1, 9, 40])]
    want = [plain.greedy(p, 8, wts, cfg) for p in prompts]
    eng = engine(model_folders[name])
    assert eng.generate(prompts, max_new_tokens=8) == want  # six requests through four slots: some wait their turn
    stats = eng.stats()
    assert stats["defects"] == 0 and stats["live"] == 0 and all(u == 0 for u in stats["used_pages"])
    got16 = engine(model_folders[name], "bfloat16").generate(prompts, max_new_tokens=8)
    for p, out in zip(prompts, got16):
        near_plain_maximum(p, out, wts, cfg)


def test_float32_checkpoint_in_bfloat16_mode(tmp_path):
    """A checkpoint stored in 32-bit keeps its weights in 32-bit."""
    folder = tiny.write(tmp_path / "A32", "A", dtype=torch.float32)
    wts, cfg = plain.load(folder)
    eng = engine(folder, "bfloat16")
    assert eng.model.embedding.weight.dtype == torch.float32
    prompt = tiny.tokens("A", 12)
    near_plain_maximum(prompt, eng.generate([prompt], max_new_tokens=5)[0], wts, cfg)


@pytest.mark.parametrize("overlap", [True, False])
def test_a_raised_status_word_stops_generation(model_folders, overlap):
    """The kernels report a wait that ran out, or a token id outside the
    vocabulary, in a status word and skip their work; the engine reads the word
    with every step's tokens and raises instead of handing out those tokens."""
    from alofa_b200.errors import AlofaError

    eng = engine(model_folders["A"], "bfloat16", overlap_steps=overlap)
    prompt = tiny.tokens("A", 9)
    assert len(eng.generate([prompt], max_new_tokens=3)[0]) == 3
    eng.runner._status.fill_(2)  # what a kernel whose wait ran out leaves behind
    with pytest.raises(AlofaError, match="gave up waiting"):
        eng.generate([prompt], max_new_tokens=3)
    assert int(eng.runner._status.item()) == 0  # cleared: the engine can be used again


def test_pages_run_out_preempted_requests_are_recomputed(model_folders):
    wts, cfg = plain.load(model_folders["B"])
    prompts = [tiny.tokens("B", n, seed=i) for i, n in enumerate([30, 31, 29])]
    want = [plain.greedy(p, 20, wts, cfg) for p in prompts]
    eng = engine(model_folders["B"], capacity_blocks=7, admission="optimistic", max_tokens=256, token_budget=64, max_chunk=32)
    got = eng.generate(prompts, max_new_tokens=20)
    stats = eng.stats()
    assert stats["preempt_total"] > 0, "the pool was meant to run out"
    assert got == want and stats["defects"] == 0 and stats["free_pages"] == [7]
    # the same with room for everything: no preemption, same tokens
    calm = engine(model_folders["B"], max_tokens=256, token_budget=64, max_chunk=32)
    assert calm.generate(prompts, max_new_tokens=20) == want and calm.stats()["preempt_total"] == 0


def test_sampling_does_not_depend_on_the_batch(model_folders):
    from alofa_b200.sampling.params import SamplingParams

    prompts = [tiny.tokens("A", n, seed=i) for i, n in enumerate([7, 19, 3, 12])]
    params = SamplingParams(temperature=0.9, top_k=40, top_p=0.95, repetition_penalty=1.1, seed=77, max_new_tokens=12)
    together = engine(model_folders["A"]).generate(prompts, sampling=params)
    from dataclasses import replace

    for i, p in enumerate(prompts):
        alone = engine(model_folders["A"]).generate([p], sampling=replace(params, seed=77 + i))
        assert alone[0] == together[i]
    hot = engine(model_folders["A"]).generate(prompts, max_new_tokens=12, temperature=1.5, seed=5)
    assert hot != engine(model_folders["A"]).generate(prompts, max_new_tokens=12, temperature=1.5, seed=6)
    assert hot == engine(model_folders["A"]).generate(prompts, max_new_tokens=12, temperature=1.5, seed=5)


def test_tiny_temperature_equals_greedy_and_draws_follow_the_plain_chain(model_folders):
    wts, cfg = plain.load(model_folders["A"])
    prompt = tiny.tokens("A", 10)
    greedy = engine(model_folders["A"]).generate([prompt], max_new_tokens=6)
    assert engine(model_folders["A"]).generate([prompt], max_new_tokens=6, temperature=0.01, seed=3) == greedy
    # temperature sampling: replay the engine's draws through the plain chain
    out = engine(model_folders["A"]).generate([prompt], max_new_tokens=6, temperature=1.3, seed=11)[0]
    rng, seq = plain.SplitMix64(11), list(prompt)
    for tok in out:
        dist = plain.sample_distribution(plain.forward(seq, wts, cfg)[-1], temperature=1.3)
        u = rng.next_uniform()
        cdf = np.cumsum(dist)
        assert (cdf[tok - 1] if tok else 0.0) - 1e-4 <= u < cdf[tok] + 1e-4
        seq.append(tok)


def test_stop_token_cancel_and_refusals(model_folders):
    from alofa_b200.errors import AlofaError
    from alofa_b200.sampling.params import SamplingParams

    wts, cfg = plain.load(model_folders["A"])
    prompt = tiny.tokens("A", 10)
    free_run = plain.greedy(prompt, 8, wts, cfg)
    stop = free_run[3]
    first = free_run.index(stop)
    eng = engine(model_folders["A"])
    assert eng.generate([prompt], max_new_tokens=8, eos_token_id=stop)[0] == free_run[: first + 1]
    assert eng.stats()["live"] == 0 or not eng.has_work()
    a = eng.add_request(prompt, SamplingParams(temperature=0.0, max_new_tokens=30))
    b = eng.add_request(tiny.tokens("A", 5), SamplingParams(temperature=0.0, max_new_tokens=4))
    eng.step()
    eng.cancel(a)
    eng.run()
    done = dict(eng.pop_finished())
    assert a not in done and len(done[b]) == 4 and eng.stats()["used_pages"] == [0] and eng.stats()["defects"] == 0
    for bad in ([], [256], [-1]):
        with pytest.raises(AlofaError):
            eng.add_request(bad)
    with pytest.raises(AlofaError):
        eng.add_request(tiny.tokens("A", 100), SamplingParams(temperature=0.0, max_new_tokens=100))  # longer than the context window


@pytest.mark.parametrize("name, dtype", [("A", "float32"), ("B", "bfloat16"), ("C", "bfloat16")])
def test_overlapped_steps_give_the_same_tokens(model_folders, name, dtype):
    """Steps launched before the host has read the tokens of the step before
    (fed on the device) against steps run one after the other: greedy with a
    stop token that ends requests early, temperature sampling, more requests
    than slots, and a pool so small that requests are preempted."""
    from alofa_b200.sampling.params import SamplingParams

    prompts = [tiny.tokens(name, n, seed=i) for i, n in enumerate([5, 17, 33, 1, 9, 26, 3])]
    probe = engine(model_folders[name], dtype, overlap_steps=False).generate(prompts, max_new_tokens=12)
    stop = probe[1][4]  # a token that some requests meet on their way
    cases = {
        "greedy with a stop": dict(max_new_tokens=12, eos_token_id=stop),
        "temperature": dict(sampling=SamplingParams(temperature=0.8, seed=5, max_new_tokens=10, stop_token_ids=(stop,))),
    }
    for what, kw in cases.items():
        runs = {}
        for overlap in (True, False):
            eng = engine(model_folders[name], dtype, overlap_steps=overlap)
            runs[overlap] = eng.generate(prompts, **kw)
            stats = eng.stats()
            assert stats["defects"] == 0 and stats["live"] == 0 and all(u == 0 for u in stats["used_pages"]) and not eng.has_work()
            assert eng.overlap == overlap
        assert runs[True] == runs[False], what
        if "stop" in what:
            assert any(len(out) < 12 for out in runs[True]), "the stop token was meant to end a request early"
    tight = dict(capacity_blocks=7, admission="optimistic", max_tokens=256, token_budget=64, max_chunk=32)
    a = engine(model_folders[name], dtype, overlap_steps=True, **tight)
    b = engine(model_folders[name], dtype, overlap_steps=False, **tight)
    long_prompts = [tiny.tokens(name, n, seed=i) for i, n in enumerate([30, 31, 29])]
    assert a.generate(long_prompts, max_new_tokens=20) == b.generate(long_prompts, max_new_tokens=20)
    assert a.stats()["preempt_total"] > 0 and a.stats()["defects"] == 0 and a.stats()["free_pages"] == [7] * len(a.stats()["free_pages"])


def test_scheduler_trace_of_a_run_replays(model_folders, tmp_path):
    from alofa_b200.engine.scheduler import replay_trace

    trace = tmp_path / "sched.trace"
    eng = engine(model_folders["A"], trace_out=str(trace), capacity_blocks=6, admission="optimistic")
    eng.generate([tiny.tokens("A", n, seed=i) for i, n in enumerate([30, 25, 28])], max_new_tokens=25)
    eng.close()
    text = trace.read_text()
    assert text.startswith("CFG ") and len(text.splitlines()) > 10 and replay_trace(text) == []


def test_generate_command_line(model_folders):
    prompt = tiny.tokens("B", 9)
    wts, cfg = plain.load(model_folders["B"])
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--model", str(model_folders["B"]), "--dtype", "float32", "--prompt-ids", ",".join(map(str, prompt)),
           "--max-new-tokens", "5", "--block-size", "16", "--max-tokens", "128", "--token-budget", "32", "--max-chunk", "16", "--json"]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    report = json.loads(out.stdout.strip().splitlines()[-1])
    assert report["out_ids"] == [plain.greedy(prompt, 5, wts, cfg)] and report["ticks"] >= 5 and report["preemptions"] == 0


def test_generate_from_a_random_config_dumps_the_logits_it_sampled_from(model_folders, tmp_path):
    """--random-config makes the weights in memory from a config.json and a
    seed (the same numbers the folder writer draws); --dump-logits writes the
    rows every token was picked from, which must be the plain logits."""
    name = "B"
    seed = tiny.CONFIGS[name][1]
    prompts = [tiny.tokens(name, 9), tiny.tokens(name, 21, seed=1)]
    wts, cfg = plain.load(model_folders[name])
    dump = tmp_path / "logits.f32"
    cmd = [sys.executable, str(ROOT / "bin" / "generate"), "--random-config", str(model_folders[name] / "config.json"), "--weights-seed", str(seed),
           "--dtype", "float32", "--max-new-tokens", "4", "--block-size", "16", "--max-tokens", "128", "--token-budget", "32", "--max-chunk", "16",
           "--dump-logits", str(dump), "--json"]
    for p in prompts:
        cmd += ["--prompt-ids", ",".join(map(str, p))]
    out = subprocess.run(cmd, capture_output=True, text=True, timeout=300)
    assert out.returncode == 0, out.stderr[-2000:]
    report = json.loads(out.stdout.strip().splitlines()[-1])
    assert report["out_ids"] == [plain.greedy(p, 4, wts, cfg) for p in prompts]
    vocab = tiny.CONFIGS[name][0].vocab_size
    rows = np.fromfile(dump, dtype="<f4").reshape(-1, vocab)
    index = [tuple(int(x) for x in line.split("\t")) for line in Path(str(dump) + ".tsv").read_text().splitlines()]
    assert len(rows) == len(index) == 8 and sorted(index) == [(r, k) for r in range(2) for k in range(4)]
    for row, (r, k) in zip(rows, index):
        seq = prompts[r] + report["out_ids"][r][:k]
        ref = plain.forward(seq, wts, cfg)[-1]
        assert np.abs(row - ref).max() <= 1e-5 * max(1.0, float(np.abs(ref).max()))
        assert int(np.argmax(row)) == report["out_ids"][r][k]


def test_no_cpu_path():
    from alofa_b200.csrc import ops
    from alofa_b200.errors import AlofaError

    with pytest.raises(AlofaError, match="CUDA tensors only"):
        ops.rmsnorm(torch.zeros(2, 8), torch.zeros(2, 8), torch.ones(8), 1e-5)
