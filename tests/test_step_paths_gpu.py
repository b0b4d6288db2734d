"""The ways a step can be issued, against the plain implementation and against
each other: kernel by kernel, as CUDA graphs (decode steps; prompt steps of a
repeated shape), and overlapped with the step before.  Two small configurations
that the tensor-core kernels take (head sizes 64 and 128, widths that are
multiples of 32, a vocabulary that is no multiple of 8, a window), one to five
requests of different lengths per step, pages used in a scattered order, and
contexts that span several 256-key splits."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu


def configs():
    from alofa_b200.models.qwen2 import Qwen2Config

    return {
        # 2 layers, 3 heads on 1, head 64, tied head, vocabulary 333 (the last weight tile is ragged)
        "P": (Qwen2Config(2, 192, 3, 1, 64, 160, 333, 1e-6, 1e4, True, 1024), 11),
        # 3 layers, 2 heads on 2, head 128, untied head, layers 1.. see the last 300 keys
        "Q": (Qwen2Config(3, 256, 2, 2, 128, 96, 200, 1e-5, 1e6, False, 2048, True, 300, 1), 12),
    }


@pytest.fixture(scope="module")
def folders(tmp_path_factory):
    from alofa_b200.models.qwen2 import NAME
    from alofa_b200.weights.random_init import write_random_model

    base = tmp_path_factory.mktemp("step_path_models")
    return {name: write_random_model(base / name, NAME, cfg, seed, torch.bfloat16) for name, (cfg, seed) in configs().items()}


def runner_for(folder, graphs: bool, pages: int, dtype="bfloat16", max_requests=5, max_tokens=1024):
    from alofa_b200.engine.loading import load_model
    from alofa_b200.engine.step import StepRunner

    model, _, _ = load_model(folder, dtype)
    return StepRunner(model, block_size=64, num_pages=pages, max_requests=max_requests, max_tokens=max_tokens, max_step_tokens=768, cuda_graphs=graphs)


@pytest.mark.parametrize("name", ["P", "Q"])
def test_decode_graphs_against_plain_and_launches(folders, name):
    from alofa_b200.engine.step import StepEntry

    wts, cfg = plain.load(folders[name])
    vocab = configs()[name][0].vocab_size
    rng = np.random.default_rng(3)
    lens = [5, 300, 64, 611, 255]  # prompts: inside one block, past a split, on a page's edge, three splits, one short of a split
    n_new = 6
    seqs = [[int(t) for t in rng.integers(0, vocab, n + n_new)] for n in lens]
    want = [plain.forward(s, wts, cfg) for s in seqs]
    results = {}
    for graphs in (True, False):
        runner = runner_for(folders[name], graphs, pages=40)
        slots = [runner.admit(i) for i in range(len(seqs))]
        # prompts in an order that scatters the pages, one of them in two portions
        for i in (3, 0, 4):
            runner.forward([StepEntry(slots[i], seqs[i][: lens[i]], [])])
        runner.forward([StepEntry(slots[1], seqs[1][:130], [])])
        runner.forward([StepEntry(slots[2], seqs[2][: lens[2]], []), StepEntry(slots[1], seqs[1][130 : lens[1]], [])])
        got = [[] for _ in seqs]
        for step in range(n_new):
            live = range(len(seqs)) if step % 2 == 0 else (1, 3)  # five requests, then two: two batch sizes, two graphs
            logits = runner.forward([StepEntry(slots[i], [seqs[i][lens[i] + len(got[i])]], [0]) for i in live]).float().cpu().numpy()
            for row, i in zip(logits, live):
                got[i].append(row)
        runner.check_status()
        used = {key[0] if isinstance(key, tuple) else key for key in runner._graphs}
        assert used == ({2, 5} if graphs else set()), f"batch sizes replayed as graphs: {used}"
        results[graphs] = got
    for i, rows in enumerate(results[True]):
        ref = want[i][lens[i] : lens[i] + len(rows)]
        bound = 2e-2 * max(1.0, float(np.abs(ref).max()))
        diff = np.abs(np.stack(rows).astype(np.float64) - ref)
        assert diff.max() <= bound, f"{name} request {i}: decoded token {int(np.argmax(diff.max(axis=1) > bound))} differs from plain by {diff.max():.3e} > {bound:.3e}"
        other = np.abs(np.stack(rows) - np.stack(results[False][i])).max()
        assert other <= bound, f"{name} request {i}: graph replay and launches differ by {other:.3e}"


@pytest.mark.parametrize("name", ["P", "Q"])
def test_decode_with_more_work_than_the_device_holds_at_once(folders, name, monkeypatch):
    """When a decode step's (request, KV head) pairs times 256-key splits are
    more than the CTAs the device holds at a time, the splits grow and a warp
    takes several key blocks in turn.  Made to happen at this size by a device
    that claims room for few CTAs: twenty requests merged by the combine
    kernel, then eight whose splits the output product merges."""
    from alofa_b200.csrc import ops
    from alofa_b200.engine.step import StepEntry
    from alofa_b200.parts.attention import GQAttention

    wts, cfg = plain.load(folders[name])
    vocab = configs()[name][0].vocab_size
    rng = np.random.default_rng(5)
    lens = [1, 63, 255, 256, 257, 511, 512, 513, 767, 768, 769, 900] + [int(n) for n in rng.integers(2, 900, 8)]
    n_new = 4
    seqs = [[int(t) for t in rng.integers(0, vocab, n + n_new)] for n in lens]
    want = [plain.forward(s, wts, cfg) for s in seqs]
    asked, one_wide_split = [], []
    real = ops.attention_bf16

    def watch(*args, **kwargs):
        asked.append(args[17])  # split_keys
        if args[16] == 1 and args[17] % (64 * ops.attention_decode_wide_warps(args[13])) == 0:
            one_wide_split.append(args[17])
        return real(*args, **kwargs)

    monkeypatch.setattr(ops, "attention_bf16", watch)
    real_slots = ops.attention_decode_slots
    for graphs in (True, False):
        runner = runner_for(folders[name], graphs, pages=20 * 16, max_requests=20, max_tokens=20 * 1024)
        slots = [runner.admit(i) for i in range(len(seqs))]
        for i in rng.permutation(len(seqs)):
            for lo in range(0, lens[i], 700):
                runner.forward([StepEntry(slots[i], seqs[i][lo : min(lens[i], lo + 700)], [])])
        got = [[] for _ in seqs]
        del asked[:]
        # (requests, room for four-warp CTAs, room for eight-warp CTAs): twenty with splits of 512 merged by the combine
        # kernel; eight, twice, whose splits the output product merges; nineteen with one split each on the wide kernel's eight or six warps
        for step, (live, room, wide) in enumerate(((range(20), 40, 0), (range(4, 12), 16, 0), (range(4, 12), 16, 0), (range(19), 40, 40))):  # nineteen: a graph of its own
            monkeypatch.setattr(ops, "attention_decode_slots",
                                lambda hd, page, warps=4, room=room, wide=wide: room if warps == 4 else min(wide, real_slots(hd, page, warps)))
            logits = runner.forward([StepEntry(slots[i], [seqs[i][lens[i] + len(got[i])]], [0]) for i in live]).float().cpu().numpy()
            for row, i in zip(logits, live):
                got[i].append(row)
        runner.check_status()
        assert max(asked) >= 512 and GQAttention.SPLIT_KEYS == 256, f"splits asked for: {sorted(set(asked))}"
        assert one_wide_split, "the last step should have run one split per request on the wide kernel"
        for i, rows in enumerate(got):
            ref = want[i][lens[i] : lens[i] + len(rows)]
            bound = 2e-2 * max(1.0, float(np.abs(ref).max()))
            diff = np.abs(np.stack(rows).astype(np.float64) - ref) if rows else np.zeros(1)
            assert diff.max() <= bound, f"{name} graphs={graphs} request {i} ({lens[i]} keys): differs from plain by {diff.max():.3e} > {bound:.3e}"


@pytest.mark.parametrize("name", ["P", "Q"])
def test_prompt_steps_of_a_repeated_shape_are_replayed_as_graphs(folders, name):
    """Steps with prompt portions whose shape (tokens, requests, wanted rows)
    repeats are recorded as CUDA graphs at the third occurrence and replayed
    after it: the same shape with the tokens divided differently among the
    requests, with a decode token beside a prompt, and with earlier context,
    against the plain implementation."""
    from alofa_b200.engine.step import StepEntry

    wts, cfg = plain.load(folders[name])
    vocab = configs()[name][0].vocab_size
    rng = np.random.default_rng(9)
    runner = runner_for(folders[name], True, pages=60)
    assert runner.prompt_graphs
    key = (200, 2, 2)
    # (tokens of the first request, of the second) per step: always 200 tokens, two requests, two wanted rows
    for step, (a, b) in enumerate([(120, 80), (10, 190), (199, 1), (150, 50), (64, 136), (1, 199)]):
        seqs = [[int(t) for t in rng.integers(0, vocab, n + 3)] for n in (a + 70, b + 70)]
        want = [plain.forward(s, wts, cfg) for s in seqs]
        slots = [runner.admit(10 * step + i) for i in range(2)]
        # 70 earlier tokens each (a step of another shape), then the step of the repeated shape, then a decoded token
        runner.forward([StepEntry(slots[0], seqs[0][:70], []), StepEntry(slots[1], seqs[1][:70], [])])
        got = runner.forward([StepEntry(slots[0], seqs[0][70 : 70 + a], [a - 1]), StepEntry(slots[1], seqs[1][70 : 70 + b], [b - 1])]).float().cpu().numpy()
        assert (key in runner._graphs) == (step >= 2), f"step {step}: graphs {list(runner._graphs)}"
        nxt = runner.forward([StepEntry(slots[0], [seqs[0][70 + a]], [0]), StepEntry(slots[1], [seqs[1][70 + b]], [0])]).float().cpu().numpy()
        for i, n in enumerate((a, b)):
            for row, ref in ((got[i], want[i][70 + n - 1]), (nxt[i], want[i][70 + n])):
                bound = 2e-2 * max(1.0, float(np.abs(ref).max()))
                assert np.abs(row - ref).max() <= bound, f"{name} step {step} request {i}: {np.abs(row - ref).max():.3e} > {bound:.3e}"
        for s in slots:
            runner.release(s)
    runner.check_status()
    assert runner.manager.defects() == 0


@pytest.mark.parametrize("name", ["P", "Q"])
def test_engine_variants_generate_the_same_tokens(folders, name):
    """Random workloads (prompt lengths, new-token counts, a stop token, greedy
    and temperature rows, more requests than slots, a pool small enough to
    preempt) through engines that differ only in how steps are issued -
    overlapped or one after the other, CUDA graphs or plain launches: the
    kernels and their order are the same, so every token must be."""
    from alofa_b200.engine.engine import Engine
    from alofa_b200.sampling.params import SamplingParams

    vocab = configs()[name][0].vocab_size
    rng = np.random.default_rng(21)
    rounds = []
    for _ in range(3):
        reqs = []
        for i in range(int(rng.integers(3, 9))):
            prompt = [int(t) for t in rng.integers(0, vocab, int(rng.integers(1, 400)))]
            temp = float(rng.choice([0.0, 0.0, 0.7]))
            reqs.append((prompt, SamplingParams(temperature=temp, seed=int(rng.integers(1, 1 << 30)), max_new_tokens=int(rng.integers(1, 40)),
                                                stop_token_ids=(int(rng.integers(0, vocab)), int(rng.integers(0, vocab))))))
        rounds.append(reqs)
    outputs = {}
    for overlap in (True, False):
        for graphs in (True, False):
            eng = Engine(str(folders[name]), dtype="bfloat16", block_size=64, max_batch=4, token_budget=160, max_chunk=128, max_tokens=512,
                         capacity_blocks=14, admission="optimistic", overlap_steps=overlap, cuda_graphs=graphs)
            got = []
            for reqs in rounds:  # the same engine serves round after round: graphs and pages are reused
                ids = [eng.add_request(p, params) for p, params in reqs]
                eng.run()
                done = dict(eng.pop_finished())
                got.append([done[i] for i in ids])
                stats = eng.stats()
                assert stats["defects"] == 0 and stats["live"] == 0 and all(u == 0 for u in stats["used_pages"])
            eng.runner.check_status()
            outputs[(overlap, graphs)] = got
    first = outputs[(False, False)]
    for key, got in outputs.items():
        assert got == first, f"overlap={key[0]} graphs={key[1]} differs from plain stepping"
    assert any(len(out) > 5 for round_out in first for out in round_out)
