"""The plain implementation, and through it the kernels, held against the
reference project's own fixtures: its sampler cases over real logits rows of
Qwen2.5-0.5B, its paged-attention cases with their negative controls, and its
layer-0 capture (tests/test_plain.py).  The differences were derived once from
a checkout of the reference by the scripts under tests/golden/ and are
committed there; with ALOFA_REFERENCE_CHECKOUT set they are derived again and
must come out the same.  The GPU tests run the engine's own kernels on the
committed inputs."""
import json
import os
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_qwen2 as plain

GOLDEN = Path(__file__).parent / "golden"
sys.path.insert(0, str(GOLDEN))
REFERENCE = os.environ.get("ALOFA_REFERENCE_CHECKOUT", "")
needs_reference = pytest.mark.skipif(not (REFERENCE and Path(REFERENCE, "tests/fixtures/paged/cases.tsv").exists()),
                                     reason="set ALOFA_REFERENCE_CHECKOUT to a checkout of the reference project to re-derive the anchors")


# -- sampler -------------------------------------------------------------------
def test_sampler_anchor_is_committed_and_exact():
    """SplitMix64 reproduces the reference's 64 raw outputs; for all nine cases
    the plain chain gives the reference's surviving set (count, first ids,
    fingerprint of all ids), its probabilities to fp32 rounding, and the same
    32 ids drawn; top-k on a row full of ties keeps every tied value."""
    result = json.loads((GOLDEN / "sampler_anchor.json").read_text())
    assert result["splitmix64"] == {"outputs": 64, "mismatches": 0}
    assert sorted(result["cases"]) == [f"c{i}" for i in range(9)]
    for name, c in result["cases"].items():
        assert c["survivors"] == c["survivors_ref"] and c["first_survivors_equal"] and c["fingerprint_equal"], name
        assert c["max_abs_prob_diff"] <= 1e-9, name
        assert c["sampled"] == 32 and c["sampled_mismatches"] == 0, name
    assert all(t["equal"] for t in result["ties"].values()) and len(result["ties"]) == 4


@needs_reference
def test_sampler_anchor_reproduces():
    import make_sampler_anchor

    result, _ = make_sampler_anchor.derive(REFERENCE)
    assert json.loads(json.dumps(result, sort_keys=True)) == json.loads((GOLDEN / "sampler_anchor.json").read_text())


def sampler_rows():
    arrays = np.load(GOLDEN / "sampler_rows.npz")
    table = json.loads((GOLDEN / "sampler_rows.json").read_text())
    return arrays, table


def test_cut_rows_give_the_reference_ids_through_the_plain_chain():
    """The committed rows are the reference's logits cut to their largest
    entries; wherever a top-k bounds the survivors the ids drawn from the cut
    row are the reference's own (recorded as such by the script)."""
    arrays, table = sampler_rows()
    from_reference = [name for name, e in table["expected"].items() if e["from"] == "reference"]
    assert sorted(from_reference) == ["c0", "c2", "c3", "c4", "c7", "c8"]
    case = next(c for c in table["cases"] if c["name"] == "c3")
    ids = arrays["row0_ids"]
    probs = plain.sample_distribution(arrays["row0_logits"], temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"])
    rng = plain.SplitMix64(table["seed"])
    drawn = [int(ids[plain.pick_from(probs, rng.next_uniform())]) for _ in range(4)]
    assert drawn == table["expected"]["c3"]["ids"][:4]


@pytest.mark.gpu
def test_device_sampling_chain_draws_the_reference_ids():
    """The device chain (bias, penalties, temperature, top-k, top-p, min-p,
    draw) on the reference's logits rows with the reference's uniform numbers:
    the ids of sampled.tsv.  The chain computes in fp32 where the reference
    uses fp64, so a draw may differ only where its uniform number lies within
    fp32 rounding of a step of the distribution."""
    from alofa_b200.sampling.params import SamplingParams
    from alofa_b200.sampling.sampler import sample_chain_rows
    from gpu_util import dev

    arrays, table = sampler_rows()
    rows, logits, want, dists = [], [], [], []
    for case in table["cases"]:
        ids = arrays[f"row{case['prompt']}_ids"]
        where = {int(t): i for i, t in enumerate(ids)}
        x = arrays[f"row{case['prompt']}_logits"]
        hist = [where[t] for t in case["history"]]
        bias = {where[i]: v for i, v in case["logit_bias"]}
        p = SamplingParams(temperature=case["temperature"], top_k=case["top_k"], top_p=case["top_p"], min_p=case["min_p"],
                           repetition_penalty=case["repetition_penalty"], frequency_penalty=case["frequency_penalty"],
                           presence_penalty=case["presence_penalty"], min_tokens_to_keep=1, logit_bias=bias)
        dist = plain.sample_distribution(x, hist, p.temperature, p.top_k, p.top_p, p.min_p, p.repetition_penalty, p.frequency_penalty,
                                         p.presence_penalty, 1, list(bias.items()))
        rng = plain.SplitMix64(table["seed"])
        for expected in table["expected"][case["name"]]["ids"]:
            u = rng.next_uniform()
            rows.append((p, u, hist))
            logits.append(x)
            want.append((where[expected], u))
            dists.append(dist)
    width = max(len(x) for x in logits)
    batch = np.full((len(logits), width), -1e30, dtype=np.float32)  # rows differ by a few entries: pad with what no case keeps
    for i, x in enumerate(logits):
        batch[i, : len(x)] = x
    got = sample_chain_rows(dev(batch), rows).cpu().tolist()
    off = 0
    for g, (w, u), dist in zip(got, want, dists):
        if g != w:
            cdf = np.cumsum(dist)
            assert g < len(dist) and dist[g] > 0 and min(abs(u - cdf[w]), abs(u - (cdf[w - 1] if w else 0.0))) < 1e-5, (g, w)
            off += 1
    assert off <= len(got) // 50, f"{off} of {len(got)} draws sit on a step of the distribution: too many to be rounding"


# -- paged attention -------------------------------------------------------------
def test_paged_anchor_is_committed_and_inside_the_gate():
    result = json.loads((GOLDEN / "paged_anchor.json").read_text())
    assert len(result["cases"]) == 11
    for name, c in result["cases"].items():
        assert c["ok"] and c["max_abs_diff"] <= c["bound"], name
    assert result["controls"] == {"moved_element_is_caught": True, "wrong_head_map_is_caught": True, "wrong_head_map_reproduced": True}


@needs_reference
def test_paged_anchor_reproduces():
    import make_paged_anchor

    result, _ = make_paged_anchor.derive(REFERENCE)
    assert json.loads(json.dumps(result, sort_keys=True)) == json.loads((GOLDEN / "paged_anchor.json").read_text())


def paged_cases():
    arrays = np.load(GOLDEN / "paged_cases.npz")
    nh, nkv, hd, page = (int(x) for x in arrays["config"])
    names = sorted({k.split(".")[0] for k in arrays.files if k.endswith(".q")})
    cases = {n: {key: arrays[f"{n}.{key}"].astype(np.float64) for key in "qkvy"} for n in names}
    return (nh, nkv, hd, page), cases, arrays["control.bad"].astype(np.float64), arrays["control.hmap"].astype(np.float64)


def test_negative_controls_fail_the_comparison_of_the_plain_implementation():
    """The reference's two controls (one element moved by 0.05; the head map
    h % kv_heads) must NOT pass the gate its cases pass."""
    (nh, nkv, hd, _), cases, bad, hmap = paged_cases()
    first = cases["s01_c3_r1"]
    q_len, kv_len = first["q"].shape[0], first["k"].shape[0]
    q = np.zeros((kv_len, nh * hd))
    q[kv_len - q_len :] = first["q"]
    got = plain.attention(q, first["k"], first["v"], nh, nkv, hd)[kv_len - q_len :]
    bound = 1e-5 * max(1.0, float(np.abs(first["y"]).max()))
    assert np.abs(got - first["y"]).max() <= bound
    assert np.abs(got - bad).max() > bound and np.abs(got - hmap).max() > bound


@pytest.mark.gpu
@pytest.mark.parametrize("dtype", ["float32", "bfloat16"])
def test_paged_attention_kernel_on_the_reference_cases(dtype):
    """All eleven cases as one batch through the engine's paged-attention
    kernel (every head size; the tensor-core kernel starts at head 16, these
    are head 8), pages scattered by a random block table, against the
    reference's expected outputs; its two controls must fail."""
    import torch
    from alofa_b200.csrc import ops
    from gpu_util import dev, paged_from_sequences, rounded

    tdt = {"float32": torch.float32, "bfloat16": torch.bfloat16}[dtype]
    tol = {"float32": 1e-5, "bfloat16": 6e-3}[dtype]
    (nh, nkv, hd, page), cases, bad, hmap = paged_cases()
    rng = np.random.default_rng(5)
    names = list(cases)
    ks = [rounded(cases[n]["k"], tdt) for n in names]
    vs = [rounded(cases[n]["v"], tdt) for n in names]
    k_cache, v_cache, table = paged_from_sequences(ks, vs, page, nkv, hd, tdt, rng)
    q_rows, positions, seq_of, want = [], [], [], []
    for s, n in enumerate(names):
        q_len, kv_len = cases[n]["q"].shape[0], cases[n]["k"].shape[0]
        for t in range(q_len):
            q_rows.append(rounded(cases[n]["q"][t], tdt))
            positions.append(kv_len - q_len + t)
            seq_of.append(s)
            want.append(cases[n]["y"][t])
    q = dev(np.stack(q_rows), tdt)
    out = torch.empty_like(q)
    ops.paged_attention_generic(out, q, k_cache, v_cache, dev(np.array(positions, dtype=np.int32)), dev(np.array(seq_of, dtype=np.int32)),
                                table, page, nh, nkv, hd, None, 1.0 / np.sqrt(hd))
    got = out.float().cpu().numpy().astype(np.float64)
    want = np.stack(want)
    bound = tol * max(1.0, float(np.abs(want).max()))
    assert np.abs(got - want).max() <= bound, f"{np.abs(got - want).max():.3e} > {bound:.3e}"
    first = got[: cases[names[0]]["q"].shape[0]]
    assert names[0] == "s01_c3_r1"
    assert np.abs(first - bad).max() > bound, "the moved element went unnoticed"
    assert np.abs(first - hmap).max() > bound, "the wrong head map went unnoticed"
