"""Replay on the GPU: the same requests whole, with the last 32 tokens decoded
one by one, in portions of changing size, and mixed with other requests in a
pool so small that pages are used again, in 32-bit and in bfloat16, against the
plain implementation.  The logits at a position must not depend on how the
tokens were cut into steps, on what else was in the batch, or on which pages
were used, beyond rounding."""
import numpy as np
import pytest

import plain_qwen2 as plain
import replay
import tiny

pytestmark = pytest.mark.gpu

# Largest |engine - plain| allowed on logits, times max(1, max|plain|).
# float32: fp32 sums against the plain implementation's float64 (worst seen over all runs of
# this file: 7.9e-7).  bfloat16: activations and cache entries are rounded to 8 bits of
# mantissa; the bound is about twice the worst seen (4.5e-3 against plain, 3.2e-3 between
# cuts), and the reference's own gate for reduced precision (cosine and largest logit, see
# check) is applied beside it.
TOL = {"float32": 1e-5, "bfloat16": 1e-2}
# between two cuts of the same request inside one dtype
TOL_CUT = {"float32": 2e-6, "bfloat16": 7e-3}

LENGTHS = {"A": [5, 17, 33, 70], "B": [1, 9, 64, 127, 143], "C": [3, 40, 75, 130]}


def make_requests(name, decoded=16):
    reqs, prompts = {}, {}
    for i, n in enumerate(LENGTHS[name]):
        rid = f"r{i}"
        reqs[rid] = tiny.tokens(name, n + decoded, seed=i)
        prompts[rid] = n
    return reqs, prompts


@pytest.fixture(scope="module")
def plain_logits(model_folders):
    out = {}
    for name, folder in model_folders.items():
        wts, cfg = plain.load(folder)
        reqs, _ = make_requests(name)
        out[name] = {rid: plain.forward(toks, wts, cfg) for rid, toks in reqs.items()}
    return out


def runner_for(folder, dtype, block, pages):
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    model, *_ = load_model(folder, dtype)
    return StepRunner(model, block_size=block, num_pages=pages, max_requests=8, max_tokens=model.spec.max_position, max_step_tokens=512)


def check(got, want, tol, what, gate=False):
    """Largest absolute difference against ``tol * max(1, max|ref|)``.  With
    ``gate`` (bfloat16 against plain) also the reference's own gate for reduced
    precision (tests/unit/test_model_parity.mojo:49-51): every row's cosine
    with the plain row at least 0.999, and the same largest logit - or, where
    plain has a near-tie at the top, one of the tied."""
    for rid, ref in want.items():
        assert rid in got, f"{what}: request {rid} has no output"
        assert got[rid].shape == ref.shape, f"{what}: {rid} shape {got[rid].shape} vs {ref.shape}"
        diff = np.abs(got[rid] - ref)
        bound = tol * max(1.0, float(np.abs(ref).max()))
        record_worst(what, float(diff.max()) / max(1.0, float(np.abs(ref).max())))
        if diff.max() > bound:
            pos = int(np.argmax(diff.max(axis=1) > bound))
            raise AssertionError(f"{what}: request {rid} first differs at position {pos}: {diff[pos].max():.3e} > {bound:.3e}")
        if gate:
            mine = got[rid].astype(np.float64)
            cosine = (mine * ref).sum(axis=1) / (np.linalg.norm(mine, axis=1) * np.linalg.norm(ref, axis=1))
            assert cosine.min() >= 0.999, f"{what}: request {rid} position {int(cosine.argmin())}: cosine {cosine.min():.5f}"
            picked = mine.argmax(axis=1)
            short = ref.max(axis=1) - ref[np.arange(len(ref)), picked]
            assert short.max() <= 2 * bound, f"{what}: request {rid} position {int(short.argmax())}: picks a logit {short.max():.3e} below the plain maximum"


def record_worst(what, ratio):
    """ALOFA_RECORD_WORST=FILE appends every comparison's worst difference (as a
    fraction of max(1, max|ref|)): the bounds above were set from such a run."""
    import os

    path = os.environ.get("ALOFA_RECORD_WORST")
    if path:
        with open(path, "a") as fh:
            fh.write(f"{what}\t{ratio:.6e}\n")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["A", "B", "C"])
@pytest.mark.parametrize("block", [16, 64])
def test_every_cut_matches_plain(model_folders, plain_logits, name, dtype, block):
    reqs, prompts = make_requests(name)
    vocab = tiny.CONFIGS[name][0].vocab_size
    ref = plain_logits[name]
    longest = max(-(-len(t) // block) * block for t in reqs.values())
    runner = runner_for(model_folders[name], dtype, block, pages=longest // block)
    results = {}
    for what, steps in (("whole", replay.whole(reqs)), ("tail", replay.tail_decoded(reqs)), ("portions", replay.portions(reqs))):
        results[what] = replay.collect(steps, replay.run_inprocess(runner, steps), vocab)
        check(results[what], ref, TOL[dtype], f"{name}/{dtype}/{what}", gate=dtype == "bfloat16")
    # so few pages that they are used again: room for about two and a half requests
    pool = longest + max(block * 3, longest // 2)
    runner = runner_for(model_folders[name], dtype, block, pages=pool // block)
    for seed in (0, 1):
        steps = replay.mixed(reqs, prompts, pool, block, seed=seed)
        assert max(len(s["entries"]) for s in steps) > 1
        out = replay.run_inprocess(runner, steps)
        results["mixed"] = replay.collect(steps, out, vocab)
        check(results["mixed"], ref, TOL[dtype], f"{name}/{dtype}/mixed{seed}", gate=dtype == "bfloat16")
    counters = runner.manager.counters(0)
    assert counters["allocs"] > runner.group_specs[0].num_pages, "the pool was never reused"
    assert runner.manager.free_pages(0) == runner.group_specs[0].num_pages
    for what in ("tail", "portions", "mixed"):
        check(results[what], results["whole"], TOL_CUT[dtype], f"{name}/{dtype}/{what} vs whole")


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_trace_program(model_folders, plain_logits, tmp_path, dtype):
    """bin/trace_run itself, as a user calls it."""
    name = "B"
    reqs, prompts = make_requests(name)
    vocab = tiny.CONFIGS[name][0].vocab_size
    steps = replay.mixed(reqs, prompts, 384, 64, seed=3)
    out = replay.run_trace_program(model_folders[name], dtype, steps, tmp_path / "out", 384)
    check(replay.collect(steps, out, vocab), plain_logits[name], TOL[dtype], f"trace_run/{dtype}")


def test_long_decoding_and_first_tokens(model_folders):
    """A sequence decoded token by token from its very first token up to the
    context limit equals the whole sequence in one step."""
    name = "A"
    cfg = tiny.CONFIGS[name][0]
    wts, pcfg = plain.load(model_folders[name])
    toks = tiny.tokens(name, cfg.max_position_embeddings, seed=9)
    ref = plain.forward(toks, wts, pcfg)
    for dtype in ("float32", "bfloat16"):
        runner = runner_for(model_folders[name], dtype, 16, pages=8)
        steps = [{"step": i, "entries": [{"id": "x", "tokens": [t], "want": [0]}], "end": []} for i, t in enumerate(toks)]
        got = replay.collect(steps, replay.run_inprocess(runner, steps), cfg.vocab_size)
        check(got, {"x": ref}, TOL[dtype], f"long decode {dtype}")
        with pytest.raises(Exception):
            from alofa_b200.engine.step import StepEntry

            runner.forward([StepEntry(0, [1], [0])])  # one past the context limit
