"""The layer sizes of the benchmarked shape (hidden 896, 14 heads on 2, head 64,
intermediate 4864, vocabulary 151936, tied head), two layers deep, against the
plain implementation: whole prompt, decoded tail, and a mixed step.  These are
the sizes the tensor-core kernels are tuned for (tiles of 128/256 with tails:
1152 = 9 x 128, 4864 = 38 x 128, 151936 = 1187 x 128)."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain

pytestmark = pytest.mark.gpu

TOL = {"float32": 1e-5, "bfloat16": 2e-2}


@pytest.fixture(scope="module")
def shaped():
    from alofa_b200.models.qwen2 import Qwen2Config, build_spec
    from alofa_b200.parts import expected_tensors
    from alofa_b200.weights.random_init import random_state

    cfg = Qwen2Config(2, 896, 14, 2, 64, 4864, 151936, 1e-6, 1e6, True, 32768)
    state = random_state(expected_tensors(build_spec(cfg)), 5, torch.bfloat16)
    wts = {k: v.to(torch.float64).numpy() for k, v in state.items()}
    pcfg = {"L": 2, "H": 896, "nh": 14, "nkv": 2, "hd": 64, "I": 4864, "V": 151936, "eps": 1e-6, "theta": 1e6, "tied": True, "window": None, "first_window_layer": 2}
    rng = np.random.default_rng(0)
    a = [int(t) for t in rng.integers(0, 151936, 150)]
    b = [int(t) for t in rng.integers(0, 151936, 70)]
    ref = {"a": plain.forward(a, wts, pcfg), "b": plain.forward(b, wts, pcfg)}
    return cfg, state, {"a": a, "b": b}, ref


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_benchmark_layer_sizes_against_plain(shaped, dtype):
    from alofa_b200.engine.loading import compute_dtype
    from alofa_b200.engine.step import StepEntry, StepRunner
    from alofa_b200.models.qwen2 import build_spec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.model import Model
    from alofa_b200.weights.loader import load_state

    cfg, state, toks, ref = shaped
    model = Model(build_spec(cfg), Runtime(torch.device("cuda"), compute_dtype(dtype)))
    model.load(load_state(model.tensors(), state, model.rt.dtype, model.rt.device))
    runner = StepRunner(model, block_size=64, num_pages=8, max_requests=4, max_tokens=512, max_step_tokens=256)
    a, b = toks["a"], toks["b"]
    sa, sb = runner.admit(1), runner.admit(2)
    got = {"a": [], "b": []}
    got["a"].append(runner.forward([StepEntry(sa, a[:130], list(range(130)))]).cpu().numpy())  # a prompt portion past one 128-token tile
    mixed = runner.forward([StepEntry(sa, a[130:131], [0]), StepEntry(sb, b[:67], list(range(67)))]).cpu().numpy()  # a decoded token beside a prompt
    got["a"].append(mixed[:1])
    got["b"].append(mixed[1:])
    for i in range(131, 150):  # decoded one by one (CUDA graph of batch 1 in bfloat16)
        got["a"].append(runner.forward([StepEntry(sa, a[i : i + 1], [0])]).cpu().numpy())
    both = runner.forward([StepEntry(sb, b[67:68], [0])]).cpu().numpy()
    got["b"].append(both)
    got["b"].append(runner.forward([StepEntry(sb, b[68:], [0, 1])]).cpu().numpy())
    runner.check_status()
    for rid in ("a", "b"):
        mine = np.concatenate(got[rid]).astype(np.float64)
        want = ref[rid]
        bound = TOL[dtype] * max(1.0, float(np.abs(want).max()))
        diff = np.abs(mine - want)
        assert diff.max() <= bound, f"{dtype} request {rid}: position {int(np.argmax(diff.max(axis=1) > bound))} differs by {diff.max():.3e} > {bound:.3e}"
        assert (mine.argmax(axis=1) == want.argmax(axis=1)).mean() > 0.9


@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_the_benchmarked_prompt_step_against_plain(shaped, dtype):
    """The benchmark's own prompt step at its real widths, two layers deep: one
    2,048-token prompt in one step, and in portions of 512, logits wanted at
    the first row, either side of a 128-token tile edge and the last row.
    This is where the persistent gate/up kernel has more tiles than SMs, the
    tensor-core attention runs several waves and the down product splits its
    depth."""
    from alofa_b200.engine.loading import compute_dtype
    from alofa_b200.engine.step import StepEntry, StepRunner
    from alofa_b200.models.qwen2 import build_spec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.model import Model
    from alofa_b200.weights.loader import load_state

    cfg, state, _, _ = shaped
    wts = {k: v.to(torch.float64).numpy() for k, v in state.items()}
    pcfg = {"L": 2, "H": 896, "nh": 14, "nkv": 2, "hd": 64, "I": 4864, "V": 151936, "eps": 1e-6, "theta": 1e6, "tied": True, "window": None, "first_window_layer": 2}
    toks = [int(t) for t in np.random.default_rng(7).integers(0, 151936, 2048)]
    rows = [0, 127, 128, 2047]
    want = plain.forward(toks, wts, pcfg, rows=rows)
    model = Model(build_spec(cfg), Runtime(torch.device("cuda"), compute_dtype(dtype)))
    model.load(load_state(model.tensors(), state, model.rt.dtype, model.rt.device))
    runner = StepRunner(model, block_size=64, num_pages=70, max_requests=2, max_tokens=4096, max_step_tokens=2112)
    bound = TOL[dtype] * max(1.0, float(np.abs(want).max()))
    whole = runner.admit(1)
    got = runner.forward([StepEntry(whole, toks, rows)]).cpu().numpy().astype(np.float64)
    assert np.abs(got - want).max() <= bound, f"{dtype} whole: {np.abs(got - want).max():.3e} > {bound:.3e}"
    cut = runner.admit(2)
    parts = []
    for lo in range(0, 2048, 512):
        local = [r - lo for r in rows if lo <= r < lo + 512]
        out = runner.forward([StepEntry(cut, toks[lo : lo + 512], local)])
        if local:
            parts.append(out.cpu().numpy().astype(np.float64))
    got = np.concatenate(parts)
    runner.check_status()
    assert np.abs(got - want).max() <= bound, f"{dtype} portions of 512: {np.abs(got - want).max():.3e} > {bound:.3e}"
    assert (got.argmax(axis=1) == want.argmax(axis=1)).all()


def test_steps_allocate_nothing(shaped):
    """Every buffer a step needs comes from the runner's arena: once a step of
    a shape has run, prompt steps, mixed steps and decode steps leave the
    device memory the tensor library holds exactly as it was."""
    from alofa_b200.engine.loading import compute_dtype
    from alofa_b200.engine.step import StepEntry, StepRunner
    from alofa_b200.models.qwen2 import build_spec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.model import Model
    from alofa_b200.weights.loader import load_state

    cfg, state, toks, _ = shaped
    model = Model(build_spec(cfg), Runtime(torch.device("cuda"), compute_dtype("bfloat16")))
    model.load(load_state(model.tensors(), state, model.rt.dtype, model.rt.device))
    runner = StepRunner(model, block_size=64, num_pages=16, max_requests=4, max_tokens=512, max_step_tokens=256, cuda_graphs=False)
    a, b = toks["a"], toks["b"]

    def steps():
        sa, sb = runner.admit(1), runner.admit(2)
        runner.forward([StepEntry(sa, a[:130], [129])])
        runner.forward([StepEntry(sa, a[130:131], [0]), StepEntry(sb, b[:67], [66])])
        for k in range(3):  # both decode, three steps
            runner.forward([StepEntry(sa, a[131 + k : 132 + k], [0]), StepEntry(sb, b[67 + k : 68 + k], [0])])
        runner.release(sa)
        runner.release(sb)

    steps()  # kernels loaded, the arena grown to what these shapes need
    torch.cuda.synchronize()
    grown = runner.arena.grown
    before = torch.cuda.memory_allocated()
    peak = torch.cuda.max_memory_allocated()
    torch.cuda.reset_peak_memory_stats()
    steps()
    torch.cuda.synchronize()
    assert torch.cuda.memory_allocated() == before and torch.cuda.max_memory_allocated() == before
    assert runner.arena.grown == grown
    runner.check_status()


@pytest.mark.parametrize("n", [8, 40])
def test_decode_steps_on_the_accumulator_stream_give_the_same_bits_every_run(shaped, n):
    """Requests decoded together (eight: the five-kernel layer; forty: the
    layer of larger steps), whose residual products add their split sums with
    atomic integer adds in whatever order their CTAs finish: two runs from the
    same state must give the same logits bit for bit, and the accumulators are
    zero between steps."""
    from alofa_b200.engine.loading import compute_dtype
    from alofa_b200.engine.step import StepEntry, StepRunner
    from alofa_b200.models.qwen2 import build_spec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.model import Model
    from alofa_b200.weights.loader import load_state

    cfg, state, _, _ = shaped
    model = Model(build_spec(cfg), Runtime(torch.device("cuda"), compute_dtype("bfloat16")))
    model.load(load_state(model.tensors(), state, model.rt.dtype, model.rt.device))
    rng = np.random.default_rng(11)
    prompts = [[int(t) for t in rng.integers(0, 151936, int(k))] for k in rng.integers(20, 200, n)]
    feed = rng.integers(0, 151936, size=(4, n))
    runs = []
    for graphs in (True, True, False):
        runner = StepRunner(model, block_size=64, num_pages=5 * n, max_requests=n, max_tokens=512, max_step_tokens=256, cuda_graphs=graphs)
        assert runner._stream_acc is not None and n <= runner.STREAM_TOKENS
        slots = [runner.admit(i) for i in range(n)]
        for s, p in zip(slots, prompts):
            runner.forward([StepEntry(s, p, [])])
        rows = []
        for step in feed:
            rows.append(runner.forward([StepEntry(s, [int(t)], [0]) for s, t in zip(slots, step)]).clone())
            assert int(runner._stream_acc.abs().sum()) == 0, "an accumulator was left with a value after the step"
        runner.check_status()
        runs.append(torch.stack(rows))
    assert torch.equal(runs[0], runs[1]), "two runs of the same steps differ"
    assert torch.equal(runs[0], runs[2]), "graph replay and plain launches differ"
