"""Schedules beyond the replay tests: decode-only steps of 17 to 64 requests
(the steps that run 32- and 64-token weight tiles, add their split sums in
kernels of their own and are replayed as graphs of those batch sizes), contexts
of more than 4,096 keys in decode (more than 16 key splits), a step that the
cache refuses, and controls that MUST fail: a block table that names another
request's page, the wrong map from query heads to KV heads, and two requests'
prompts exchanged."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
import tiny

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-5, "bfloat16": 2e-2}


def configs():
    from alofa_b200.models.qwen2 import Qwen2Config

    return {
        # 2 layers, 3 heads on 1, head 64, tied head, vocabulary 333
        "P": (Qwen2Config(2, 192, 3, 1, 64, 160, 333, 1e-6, 1e4, True, 1024), 11),
        # 3 layers, 2 heads on 2, head 128, untied head, layers 1.. see the last 300 keys
        "Q": (Qwen2Config(3, 256, 2, 2, 128, 96, 200, 1e-5, 1e6, False, 2048, True, 300, 1), 12),
        # as P with positions up to 8,192
        "L": (Qwen2Config(2, 192, 3, 1, 64, 160, 333, 1e-6, 1e4, True, 8192), 13),
    }


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from alofa_b200.models.qwen2 import NAME
    from alofa_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("schedule_models")
    return {name: write_random_model(base / name, NAME, cfg, seed, torch.bfloat16) for name, (cfg, seed) in configs().items()}


def runner_for(folder, dtype, pages, max_requests, max_tokens, max_step_tokens=768, graphs=True):
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    model, _, _ = load_model(folder, dtype)
    return StepRunner(model, block_size=64, num_pages=pages, max_requests=max_requests, max_tokens=max_tokens, max_step_tokens=max_step_tokens, cuda_graphs=graphs)


def assert_rows(got, want, tol, what):
    got, want = np.asarray(got, dtype=np.float64), np.asarray(want, dtype=np.float64)
    bound = tol * max(1.0, float(np.abs(want).max()))
    diff = np.abs(got - want).max()
    assert diff <= bound, f"{what}: {diff:.3e} > {bound:.3e}"


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
@pytest.mark.parametrize("name", ["P", "Q"])
def test_decode_only_steps_of_17_to_64_requests(folders, name, dtype):
    """64 requests with prompts of mixed lengths (page edges and split edges
    among them), then eight decode-only steps with 64, 64, 33, 33, 33, 17, 17
    and 17 of them live: every row against plain.  The second and later steps
    of a batch size replay its graph."""
    from alofa_b200.engine.step import StepEntry

    vocab = configs()[name][0].vocab_size
    wts, cfg = plain.load(folders[name])
    rng = np.random.default_rng(17)
    lens = [1, 2, 63, 64, 65, 127, 128, 129, 255, 256, 257, 300] + [int(n) for n in rng.integers(1, 280, 52)]
    n_new = 8
    seqs = [[int(t) for t in rng.integers(0, vocab, n + n_new)] for n in lens]
    want = [plain.forward(s, wts, cfg, rows=range(n, n + n_new)) for s, n in zip(seqs, lens)]
    runner = runner_for(folders[name], dtype, pages=64 * 6, max_requests=64, max_tokens=512)
    slots = [runner.admit(i) for i in range(64)]
    batch, used = [], 0
    for i in rng.permutation(64):  # prompts several to a step, in an order that scatters the pages
        if used + lens[i] > 700:
            runner.forward(batch)
            batch, used = [], 0
        batch.append(StepEntry(slots[i], seqs[i][: lens[i]], []))
        used += lens[i]
    runner.forward(batch)
    done = [0] * 64
    for live in (64, 64, 33, 33, 33, 17, 17, 17):
        chosen = list(range(live))
        logits = runner.forward([StepEntry(slots[i], [seqs[i][lens[i] + done[i]]], [0]) for i in chosen]).float().cpu().numpy()
        for row, i in zip(logits, chosen):
            assert_rows(row, want[i][done[i]], TOL[dtype], f"{name}/{dtype} {live} live, request {i} (prompt {lens[i]}), token {done[i]}")
            done[i] += 1
    runner.check_status()
    assert runner.manager.defects() == 0
    if dtype == "bfloat16":
        assert {key[0] for key in runner._graphs if key[2] == "decode"} == {64, 33, 17}


@pytest.mark.parametrize("name", ["P", "Q"])
def test_generate_with_64_slots(folders, name):
    """Through the entry point with 64 request slots: 70 requests, eight new
    tokens each, greedy in 32-bit against plain, and bfloat16 close to it."""
    from alofa_b200.engine.engine import Engine

    vocab = configs()[name][0].vocab_size
    wts, cfg = plain.load(folders[name])
    rng = np.random.default_rng(33)
    prompts = [[int(t) for t in rng.integers(0, vocab, int(n))] for n in rng.integers(1, 120, 70)]
    want = [plain.greedy(p, 8, wts, cfg) for p in prompts]
    eng = Engine(str(folders[name]), dtype="float32", block_size=64, max_batch=64, token_budget=512, max_chunk=256, max_tokens=256)
    assert eng.generate(prompts, max_new_tokens=8) == want
    eng16 = Engine(str(folders[name]), dtype="bfloat16", block_size=64, max_batch=64, token_budget=512, max_chunk=256, max_tokens=256)
    got = eng16.generate(prompts, max_new_tokens=8)
    eng16.runner.check_status()
    for p, out in zip(prompts, got):  # bfloat16 may swap near-ties: the first token must be within rounding of the plain maximum
        row = plain.forward(p, wts, cfg)[-1]
        assert len(out) == 8 and row.max() - row[out[0]] <= 4e-2 * max(1.0, float(np.abs(row).max()))
    assert any(key[0] > 16 for key in eng16.runner._graphs if key[2] == "decode"), "no decode graph of more than 16 requests was recorded"
    assert eng16.stats()["defects"] == 0


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_decode_over_more_than_4096_keys(folders, dtype):
    """One request of 4,200 tokens, then six decoded: 17 key splits of 256, one
    more than the output product merges by itself, so the splits are combined
    by their own kernel.  A 300-key request in the same engine is decoded
    inside a graph recorded for its own bucket of context lengths."""
    from alofa_b200.engine.step import StepEntry

    name = "L"
    vocab = configs()[name][0].vocab_size
    wts, cfg = plain.load(folders[name])
    rng = np.random.default_rng(5)
    n, n_new = 4200, 6
    seq = [int(t) for t in rng.integers(0, vocab, n + n_new)]
    want = plain.forward(seq, wts, cfg, rows=range(n, n + n_new))
    short = [int(t) for t in rng.integers(0, vocab, 300 + n_new)]
    want_short = plain.forward(short, wts, cfg, rows=range(300, 300 + n_new))
    runner = runner_for(folders[name], dtype, pages=80, max_requests=2, max_tokens=8192, max_step_tokens=1024)
    a, b = runner.admit(1), runner.admit(2)
    for lo in range(0, n, 1000):
        runner.forward([StepEntry(a, seq[lo : min(lo + 1000, n)], [])])
    runner.forward([StepEntry(b, short[:300], [])])
    for k in range(n_new):
        row = runner.forward([StepEntry(a, [seq[n + k]], [0])]).float().cpu().numpy()[0]
        assert_rows(row, want[k], TOL[dtype], f"{dtype} long request, token {k}")
        row = runner.forward([StepEntry(b, [short[300 + k]], [0])]).float().cpu().numpy()[0]
        assert_rows(row, want_short[k], TOL[dtype], f"{dtype} short request, token {k}")
    both = runner.forward([StepEntry(a, [seq[n + n_new - 1]], [0])])  # one past what plain was asked for: only the shape matters here
    runner.check_status()
    if dtype == "bfloat16":
        assert {(key[0], key[1]) for key in runner._graphs if key[2] == "decode"} == {(1, 8192), (1, 512)}


def test_a_step_the_cache_refuses_leaves_the_runner_as_it_was(folders):
    """Two entries of which the second does not fit: nothing is reserved, the
    lengths stand, and a smaller step runs and is right."""
    from alofa_b200.engine.step import StepEntry
    from alofa_b200.errors import AlofaError

    name = "P"
    vocab = configs()[name][0].vocab_size
    wts, cfg = plain.load(folders[name])
    rng = np.random.default_rng(2)
    a_toks = [int(t) for t in rng.integers(0, vocab, 150)]
    b_toks = [int(t) for t in rng.integers(0, vocab, 150)]
    runner = runner_for(folders[name], "float32", pages=4, max_requests=2, max_tokens=512)
    a, b = runner.admit(1), runner.admit(2)
    with pytest.raises(AlofaError, match="too few free pages"):
        runner.forward([StepEntry(a, a_toks, []), StepEntry(b, b_toks, [])])  # 3 + 3 pages of 4
    assert runner.length(a) == 0 and runner.length(b) == 0 and runner.manager.free_pages() == [4] and runner.manager.defects() == 0
    got = runner.forward([StepEntry(a, a_toks[:100], [99]), StepEntry(b, b_toks[:120], [119])]).float().cpu().numpy()
    assert_rows(got[0], plain.forward(a_toks[:100], wts, cfg)[-1], 1e-5, "after the refusal, a")
    assert_rows(got[1], plain.forward(b_toks[:120], wts, cfg)[-1], 1e-5, "after the refusal, b")
    assert runner.manager.defects() == 0


# -- controls that must fail -------------------------------------------------------
def run_two(runner, toks_a, toks_b, corrupt=None):
    """Two requests prefilled together, then one decode step of both; the
    logits of that decode step.  ``corrupt(host_meta, layout)`` edits the
    decode step's metadata on the host before it is copied to the device."""
    from alofa_b200.engine.step import StepEntry

    a, b = runner.admit(1), runner.admit(2)
    runner.forward([StepEntry(a, toks_a[:-1], []), StepEntry(b, toks_b[:-1], [])])
    if corrupt is not None:
        real = runner.manager.plan_step

        def planned(slots, counts, want_counts, wants, meta_ptr, offsets, max_blocks):
            out = real(slots, counts, want_counts, wants, meta_ptr, offsets, max_blocks)
            corrupt(runner, offsets)
            return out

        runner.manager.plan_step = planned
    got = runner.forward([StepEntry(a, toks_a[-1:], [0]), StepEntry(b, toks_b[-1:], [0])]).float().cpu().numpy()
    runner.release(a)
    runner.release(b)
    return got


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_a_block_table_that_names_another_requests_page_is_caught(model_folders, dtype):
    """One entry of request a's block table is exchanged for a page of request
    b (a valid page holding other tokens' keys): the comparison with plain,
    which passes untouched, must fail.  A comparison this cannot fail would
    not notice a wrong page either."""
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    name = "A"
    wts, cfg = plain.load(model_folders[name])
    toks_a, toks_b = tiny.tokens(name, 50, seed=1), tiny.tokens(name, 60, seed=2)
    want = np.stack([plain.forward(toks_a, wts, cfg)[-1], plain.forward(toks_b, wts, cfg)[-1]])
    bound = TOL[dtype] * max(1.0, float(np.abs(want).max()))
    model, _, _ = load_model(model_folders[name], dtype)

    def fresh():
        return StepRunner(model, block_size=16, num_pages=12, max_requests=2, max_tokens=128, max_step_tokens=128, cuda_graphs=False)

    assert np.abs(run_two(fresh(), toks_a, toks_b) - want).max() <= bound

    def corrupt(runner, offsets):
        host = runner._host_meta[runner._flip ^ 1].numpy()  # the buffer the step in preparation uses
        table_at = int(offsets[7])  # block table of group 0: [requests, max_blocks]
        mb = runner.manager.max_blocks
        mine, theirs = host[table_at + 1], host[table_at + mb + 1]
        assert mine >= 0 and theirs >= 0 and mine != theirs
        host[table_at + 1] = theirs  # request a's second page := request b's second page

    got = run_two(fresh(), toks_a, toks_b, corrupt)
    assert np.abs(got[0] - want[0]).max() > bound, "a wrong page went unnoticed"
    assert np.abs(got[1] - want[1]).max() <= bound  # the other request is untouched


def test_the_wrong_head_map_is_caught(model_folders, monkeypatch):
    """Plain attention with query head h reading KV head h % kv_heads instead
    of h // group (tiny A: 4 heads on 2) must NOT agree with the engine."""
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    name = "A"
    wts, cfg = plain.load(model_folders[name])
    toks_a, toks_b = tiny.tokens(name, 50, seed=1), tiny.tokens(name, 60, seed=2)
    model, _, _ = load_model(model_folders[name], "float32")
    got = run_two(StepRunner(model, block_size=16, num_pages=12, max_requests=2, max_tokens=128, max_step_tokens=128), toks_a, toks_b)
    right = plain.forward(toks_a, wts, cfg)[-1]
    real = plain.attention

    def wrong(q, k, v, nh, nkv, hd, window=None):
        out = np.zeros((q.shape[0], nh * hd))
        for h in range(nh):
            kh = h % nkv
            out[:, h * hd : (h + 1) * hd] = real(q[:, h * hd : (h + 1) * hd], k[:, kh * hd : (kh + 1) * hd], v[:, kh * hd : (kh + 1) * hd], 1, 1, hd, window)
        return out

    monkeypatch.setattr(plain, "attention", wrong)
    mapped = plain.forward(toks_a, wts, cfg)[-1]
    bound = 1e-5 * max(1.0, float(np.abs(right).max()))
    assert np.abs(got[0] - right).max() <= bound
    assert np.abs(got[0] - mapped).max() > bound, "the wrong head map went unnoticed"


def test_exchanged_prompts_are_caught(model_folders):
    """The engine is given two requests' prompts exchanged: the comparison that
    passes otherwise must fail for both."""
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    name = "B"
    wts, cfg = plain.load(model_folders[name])
    toks_a, toks_b = tiny.tokens(name, 50, seed=1), tiny.tokens(name, 50, seed=2)
    want = np.stack([plain.forward(toks_a, wts, cfg)[-1], plain.forward(toks_b, wts, cfg)[-1]])
    bound = 1e-5 * max(1.0, float(np.abs(want).max()))
    model, _, _ = load_model(model_folders[name], "float32")
    runner = StepRunner(model, block_size=16, num_pages=12, max_requests=2, max_tokens=128, max_step_tokens=128)
    assert np.abs(run_two(runner, toks_a, toks_b) - want).max() <= bound
    swapped = run_two(runner, toks_b[:-1] + toks_a[-1:], toks_a[:-1] + toks_b[-1:])  # the prompts exchanged, the decoded tokens kept
    assert np.abs(swapped[0] - want[0]).max() > bound and np.abs(swapped[1] - want[1]).max() > bound
