"""Each part alone against the plain implementation, and the generality of the
assembly: a toy mixer with state of its own, a toy routed feed-forward and a
toy position encoding are registered, built and stepped from this file alone;
a run list that names a layer twice and a layer that reads another layer's
cache."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from gpu_util import assert_close, rounded

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
TOL = {F32: 1e-5, BF16: 2e-2}


def runtime(dtype):
    from alofa_b200.parts.base import Runtime

    return Runtime(torch.device("cuda"), dtype)


def toy_spec(layers=2, run=None, mixer_kind="gqa_attention", ffn_kind="gated_mlp", position_kind="rotary_neox", hidden=40, nh=5, nkv=1, hd=8, inter=56, vocab=97, window=None, max_pos=96):
    """A small model description built by hand: nothing here is an architecture
    of anyone's, it only exercises the assembly."""
    from alofa_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

    specs = []
    for i in range(layers):
        p = f"layers.{i}."
        pos = PartSpec(position_kind, {"head_dim": hd, "rotary_dim": hd, "theta": 777.0, "max_position": max_pos}, prefix=p + "pos.")
        mixer = PartSpec(mixer_kind, {"hidden_size": hidden, "num_heads": nh, "num_kv_heads": nkv, "head_dim": hd, "qkv_bias": i % 2 == 0, "out_bias": i % 2 == 1, "window": window, "position": pos}, prefix=p + "attn.")
        ffn = PartSpec(ffn_kind, {"hidden_size": hidden, "intermediate_size": inter, "activation": "silu", "experts": 3}, prefix=p + "ffn.")
        norm = lambda name: PartSpec("rmsnorm", {"size": hidden, "eps": 2e-5}, prefix=p + name + ".")
        specs.append(LayerSpec(PartSpec("prenorm_residual", {"mixer": mixer, "feed_forward": ffn, "mixer_norm": norm("n1"), "feed_forward_norm": norm("n2")}, prefix=p)))
    run = run or [RunEntry(i, i) for i in range(layers)]
    return ModelSpec("Toy", hidden, vocab, max_pos, PartSpec("token_embedding", {"vocab_size": vocab, "hidden_size": hidden}, prefix="embed."), specs, run,
                     PartSpec("rmsnorm", {"size": hidden, "eps": 2e-5}, prefix="norm."), PartSpec("linear_head", {"vocab_size": vocab, "hidden_size": hidden, "tied_to": None}, prefix="head."))


def build(spec, dtype, seed=0):
    from alofa_b200.engine.step import StepRunner
    from alofa_b200.parts.model import Model
    from alofa_b200.weights.loader import load_state
    from alofa_b200.weights.random_init import random_state

    model = Model(spec, runtime(dtype))
    state = random_state(model.tensors(), seed, torch.bfloat16)
    model.load(load_state(model.tensors(), state, dtype, model.rt.device))
    runner = StepRunner(model, block_size=16, num_pages=24, max_requests=4, max_tokens=spec.max_position, max_step_tokens=128)
    return model, runner, {k: v.to(torch.float64).numpy() for k, v in state.items()}


def toy_plain_layer(h, positions, w, p, spec_layer, k_from=None):
    """The plain restatement of one toy layer with the stock parts."""
    mp = spec_layer.block.params["mixer"].params
    nh, nkv, hd = mp["num_heads"], mp["num_kv_heads"], mp["head_dim"]
    x = plain.rmsnorm(h, w[p + "n1.weight"], 2e-5)
    a = p + "attn."
    bias = lambda n: w.get(a + n + "_proj.bias")
    q = plain.rope(plain.linear(x, w[a + "q_proj.weight"], bias("q")), positions, nh, hd, 777.0)
    if k_from is None:
        k = plain.rope(plain.linear(x, w[a + "k_proj.weight"], bias("k")), positions, nkv, hd, 777.0)
        v = plain.linear(x, w[a + "v_proj.weight"], bias("v"))
    else:
        k, v = k_from
    att = plain.attention(q, k, v, nh, nkv, hd, mp["window"])
    h = h + plain.linear(att, w[a + "o_proj.weight"], bias("o"))
    x = plain.rmsnorm(h, w[p + "n2.weight"], 2e-5)
    f = p + "ffn."
    return h + plain.swiglu_mlp(x, w[f + "gate_proj.weight"], w[f + "up_proj.weight"], w[f + "down_proj.weight"]), (k, v)


def toy_plain(ids, w, spec, run=None):
    run = run or [(e.layer, e.cache) for e in spec.run]
    positions = np.arange(len(ids))
    h = plain.embed(ids, w["embed.weight"])
    kvs = {}
    for i, (layer, cache) in enumerate(run):
        h, kv = toy_plain_layer(h, positions, w, f"layers.{layer}.", spec.layers[layer], None if cache == i else kvs[cache])
        kvs[i] = kv
    return plain.linear(plain.rmsnorm(h, w["norm.weight"], 2e-5), w["head.weight"])


def step_whole_then_one_by_one(runner, ids, cut):
    from alofa_b200.engine.step import StepEntry

    slot = runner.admit(1)
    rows = [runner.forward([StepEntry(slot, ids[:cut], list(range(cut)))]).cpu().numpy()]
    for t in ids[cut:]:
        rows.append(runner.forward([StepEntry(slot, [t], [0])]).cpu().numpy())
    runner.release(slot)
    return np.concatenate(rows).astype(np.float64)


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_stock_parts_in_a_hand_made_model(dtype):
    """Norm, attention (with q/k/v bias or with output bias), gated MLP, block,
    embedding and head, at sizes no test model has (5 heads on 1, head 8,
    hidden 40, vocabulary 97), each layer alone and all together."""
    spec = toy_spec(layers=2)
    model, runner, w = build(spec, dtype)
    ids = [int(t) for t in np.random.default_rng(0).integers(0, 97, 50)]
    assert_close(step_whole_then_one_by_one(runner, ids, 31), toy_plain(ids, w, spec), TOL[dtype], "toy model")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_each_part_alone(dtype):
    from alofa_b200.config.spec import PartSpec
    from alofa_b200.engine.step import StepEntry
    from alofa_b200.parts.base import build_part

    spec = toy_spec(layers=1)
    model, runner, w = build(spec, dtype)
    ids = [int(t) for t in np.random.default_rng(1).integers(0, 97, 21)]
    slot = runner.admit(1)
    ctx = runner.prepare([StepEntry(slot, ids, [20])])
    # embedding
    h = ctx.buf((21, 40), F32)
    model.embedding.forward(ctx, h)
    want_h = plain.embed(ids, w["embed.weight"])
    assert_close(h.cpu(), want_h, 0.0, "embedding")
    block = model.layers[0]
    # norm
    x = block.mixer_norm.forward(ctx, h)
    want_x = plain.rmsnorm(want_h, w["layers.0.n1.weight"], 2e-5)
    assert_close(x.float().cpu(), want_x, TOL[dtype], "norm")
    # mixer alone: h2 = h + attention(x)
    h2 = h.clone()
    block.mixer.forward(ctx, x, h2, runner.storage.caches[0], True)
    ctx.flush_pending()  # a part may leave split-K partial sums owed to the stream
    xin = rounded(x.float().cpu().numpy(), dtype)
    a = "layers.0.attn."
    pos = np.arange(21)
    q = plain.rope(plain.linear(xin, w[a + "q_proj.weight"], w[a + "q_proj.bias"]), pos, 5, 8, 777.0)
    k = plain.rope(plain.linear(xin, w[a + "k_proj.weight"], w[a + "k_proj.bias"]), pos, 1, 8, 777.0)
    v = plain.linear(xin, w[a + "v_proj.weight"], w[a + "v_proj.bias"])
    want_h2 = want_h + plain.linear(plain.attention(q, k, v, 5, 1, 8), w[a + "o_proj.weight"])
    assert_close(h2.cpu(), want_h2, TOL[dtype], "mixer")
    # feed-forward alone
    h3 = torch.zeros_like(h)
    block.feed_forward.forward(ctx, x, h3)
    ctx.flush_pending()
    f = "layers.0.ffn."
    assert_close(h3.cpu(), plain.swiglu_mlp(xin, w[f + "gate_proj.weight"], w[f + "up_proj.weight"], w[f + "down_proj.weight"]), TOL[dtype], "feed-forward")
    # head on the wanted row
    xr = model.final_norm.forward(ctx, h, ctx.logit_rows)
    logits = model.head.forward(ctx, xr)
    want = plain.linear(rounded(xr.float().cpu().numpy(), dtype), w["head.weight"])
    assert_close(logits.cpu(), want, TOL[dtype], "head")
    # a position encoding that leaves q and k alone
    none = build_part("position", PartSpec("none", {}), runtime(dtype))
    assert none.rotary_table() == (None, 0)


def test_run_list_names_a_layer_twice_and_a_layer_reads_anothers_cache():
    from alofa_b200.config.spec import RunEntry

    ids = [int(t) for t in np.random.default_rng(2).integers(0, 97, 40)]
    # layer 0 runs twice (its own cache each time), then layer 1
    spec = toy_spec(layers=2, run=[RunEntry(0, 0), RunEntry(0, 1), RunEntry(1, 2)])
    model, runner, w = build(spec, F32)
    assert sorted(model.cache_plan()) == [0, 1, 2]
    assert_close(step_whole_then_one_by_one(runner, ids, 17), toy_plain(ids, w, spec), TOL[F32], "layer twice")
    # entry 2 (layer 1) reads the cache that entry 0 wrote and writes none
    spec = toy_spec(layers=2, run=[RunEntry(0, 0), RunEntry(1, 1), RunEntry(1, 0)])
    model, runner, w = build(spec, F32)
    assert sorted(model.cache_plan()) == [0, 1]
    assert_close(step_whole_then_one_by_one(runner, ids, 17), toy_plain(ids, w, spec), TOL[F32], "shared cache")
    with pytest.raises(Exception):
        toy_spec(layers=2, run=[RunEntry(0, 1), RunEntry(1, 1)]).validate()  # may only read an earlier entry


def register_toy_parts():
    """Toy parts, defined in the tests only (tests/toy_architecture.py): a mixer
    that keeps a running mean of its inputs per request (state of fixed size,
    no pages), a feed-forward that routes every token to one of several small
    experts, and a position encoding that is not rotary."""
    import toy_architecture

    toy_architecture.register_parts()


def test_toy_mixer_with_state_of_its_own_is_registered_built_and_stepped():
    """No file of the package changes: the toy kinds are registered here, named
    in a hand-made spec, built by the stock assembly, given state slots by the
    stock cache code, and stepped in portions and mixed batches."""
    from alofa_b200.engine.step import StepEntry

    register_toy_parts()
    spec = toy_spec(layers=2, mixer_kind="toy_running_mean", ffn_kind="toy_routed")
    model, runner, w = build(spec, F32)
    assert all(type(s).__name__ == "SlotState" for s in model.cache_plan().values()) and not runner.has_paged

    def plain_toy(ids):
        h = plain.embed(ids, w["embed.weight"])
        for i in range(2):
            p = f"layers.{i}."
            x = plain.rmsnorm(h, w[p + "n1.weight"], 2e-5)
            mean = np.cumsum(x, axis=0) / np.arange(1, len(ids) + 1)[:, None]
            h = h + mean @ w[p + "attn.mix.weight"].T
            x = plain.rmsnorm(h, w[p + "n2.weight"], 2e-5)
            choice = (x @ w[p + "ffn.router.weight"].T).argmax(axis=1)
            out = np.stack([x[t] @ w[p + f"ffn.experts.{choice[t]}.weight"].T for t in range(len(ids))])
            h = h + out
        return plain.linear(plain.rmsnorm(h, w["norm.weight"], 2e-5), w["head.weight"])

    rng = np.random.default_rng(3)
    a = [int(t) for t in rng.integers(0, 97, 30)]
    b = [int(t) for t in rng.integers(0, 97, 22)]
    sa, sb = runner.admit(1), runner.admit(2)
    # (a step's logits live in the runner's arena until the next step: copy what is kept)
    got_a = [runner.forward([StepEntry(sa, a[:7], list(range(7)))]).clone()]
    mixed = runner.forward([StepEntry(sa, a[7:9], [0, 1]), StepEntry(sb, b[:20], list(range(20)))]).clone()
    got_a.append(mixed[:2])
    got_b = [mixed[2:]]
    mixed = runner.forward([StepEntry(sb, b[20:21], [0]), StepEntry(sa, a[9:], list(range(21)))]).clone()
    got_b.append(mixed[:1])
    got_a.append(mixed[1:])
    got_b.append(runner.forward([StepEntry(sb, b[21:], [0])]).clone())
    assert_close(torch.cat(got_a).cpu(), plain_toy(a), 2e-5, "toy request a")
    assert_close(torch.cat(got_b).cpu(), plain_toy(b), 2e-5, "toy request b")
    # a new request in a used slot starts from zeroed state
    runner.release(sa)
    sc = runner.admit(3)
    assert sc == sa
    assert_close(runner.forward([StepEntry(sc, b, list(range(22)))]).cpu(), plain_toy(b), 2e-5, "state is zeroed on reuse")


def test_toy_position_encoding_goes_through_the_stock_attention():
    register_toy_parts()
    spec = toy_spec(layers=1, position_kind="toy_added")
    model, runner, w = build(spec, F32)
    ids = [int(t) for t in np.random.default_rng(4).integers(0, 97, 25)]
    positions = np.arange(25)
    h = plain.embed(ids, w["embed.weight"])
    x = plain.rmsnorm(h, w["layers.0.n1.weight"], 2e-5)
    a = "layers.0.attn."
    shift = (positions.astype(np.float32) * np.float32(0.01)).astype(np.float64)[:, None]
    q = plain.linear(x, w[a + "q_proj.weight"], w[a + "q_proj.bias"]) + shift
    k = plain.linear(x, w[a + "k_proj.weight"], w[a + "k_proj.bias"]) + shift
    v = plain.linear(x, w[a + "v_proj.weight"], w[a + "v_proj.bias"])
    h = h + plain.linear(plain.attention(q, k, v, 5, 1, 8), w[a + "o_proj.weight"])
    x = plain.rmsnorm(h, w["layers.0.n2.weight"], 2e-5)
    f = "layers.0.ffn."
    h = h + plain.swiglu_mlp(x, w[f + "gate_proj.weight"], w[f + "up_proj.weight"], w[f + "down_proj.weight"])
    want = plain.linear(plain.rmsnorm(h, w["norm.weight"], 2e-5), w["head.weight"])
    assert_close(step_whole_then_one_by_one(runner, ids, 11), want, 2e-5, "toy position")
