"""The plain implementation itself: its anchor on the reference's layer-0
capture, and properties its formulas must have."""
import json
import os
import subprocess
import sys
from pathlib import Path

import numpy as np
import pytest

import plain_qwen2 as plain
import tiny

GOLDEN = Path(__file__).parent / "golden"


def test_layer0_anchor_is_committed_and_inside_the_gate():
    result = json.loads((GOLDEN / "layer0_anchor.json").read_text())
    assert set(result) >= {"rmsnorm", "q_proj", "k_proj", "v_proj", "rope_q", "rope_k", "rope_cos_table", "attention", "o_proj", "swiglu"}
    for name, r in result.items():
        assert r["ok"] and r["max_abs_diff"] <= r["bound"], name


REFERENCE = os.environ.get("ALOFA_REFERENCE_CHECKOUT", "")


@pytest.mark.skipif(not (REFERENCE and Path(REFERENCE, "tests/fixtures/qwen2.5-0.5b/layer0/tensors.f32").exists()),
                    reason="set ALOFA_REFERENCE_CHECKOUT to a checkout of the reference project to re-derive the anchor")
def test_layer0_anchor_reproduces(tmp_path):
    before = (GOLDEN / "layer0_anchor.json").read_text()
    subprocess.run([sys.executable, str(GOLDEN / "make_layer0_anchor.py"), REFERENCE], check=True, capture_output=True)
    assert (GOLDEN / "layer0_anchor.json").read_text() == before


def test_rope_table_is_fp32_arithmetic():
    cos, sin = plain.rope_table([0, 1, 500], 64, 1e6)
    assert cos.shape == (3, 32) and np.all(cos[0] == 1.0) and np.all(sin[0] == 0.0)
    inv = np.float32(1.0) / np.float32(1e6 ** (2 * 5 / 64))
    angle = np.float32(500) * inv
    assert cos[2, 5] == np.float32(np.cos(np.float64(angle)))


def test_rope_rotates_pairs_d_and_d_plus_half():
    x = np.zeros((1, 8))
    x[0, 1], x[0, 5] = 1.0, 2.0
    y = plain.rope(x, [3], 1, 8, 10000.0)
    cos, sin = plain.rope_table([3], 8, 10000.0)
    assert np.isclose(y[0, 1], 1.0 * cos[0, 1] - 2.0 * sin[0, 1]) and np.isclose(y[0, 5], 2.0 * cos[0, 1] + 1.0 * sin[0, 1])
    assert y[0, 0] == 0 and y[0, 4] == 0


def test_attention_is_causal_grouped_and_windowed():
    rng = np.random.default_rng(0)
    n, nh, nkv, hd = 12, 4, 2, 8
    q, k, v = rng.normal(size=(n, nh * hd)), rng.normal(size=(n, nkv * hd)), rng.normal(size=(n, nkv * hd))
    out = plain.attention(q, k, v, nh, nkv, hd)
    k2, v2 = k.copy(), v.copy()
    k2[7:], v2[7:] = 0.0, 9.0
    assert np.allclose(plain.attention(q, k2, v2, nh, nkv, hd)[:7], out[:7])  # later keys do not matter
    assert np.allclose(out[0], np.repeat(v[0].reshape(nkv, hd), nh // nkv, axis=0).reshape(-1))  # head h reads kv head h // g
    w = plain.attention(q, k, v, nh, nkv, hd, window=3)
    assert np.allclose(w[:3], out[:3]) and not np.allclose(w[5], out[5])
    k3, v3 = k.copy(), v.copy()
    k3[:6], v3[:6] = 5.0, -5.0
    assert np.allclose(plain.attention(q, k3, v3, nh, nkv, hd, window=3)[8:], w[8:])  # keys behind the window do not matter


def test_forward_is_causal_and_head_is_tied_or_not(model_folders):
    for name in ("A", "B"):
        wts, cfg = plain.load(model_folders[name])
        ids = tiny.tokens(name, 20)
        full = plain.forward(ids, wts, cfg)
        assert np.allclose(plain.forward(ids[:11], wts, cfg), full[:11], atol=1e-12)
        assert ("lm_head.weight" in wts) == (not cfg["tied"])
    wts, cfg = plain.load(model_folders["C"])
    assert cfg["window"] == 24 and cfg["first_window_layer"] == 1


def test_sampling_chain_examples():
    x = np.array([2.0, 1.0, 1.0, 0.0, -1.0])
    assert plain.sample_distribution(x, temperature=0.0).tolist() == [1, 0, 0, 0, 0]
    p = plain.sample_distribution(x, top_k=2)
    assert (p > 0).tolist() == [True, True, True, False, False]  # ties at the k-th value survive
    p = plain.sample_distribution(x, top_p=0.5)
    assert (p > 0).tolist() == [True, False, False, False, False]
    p = plain.sample_distribution(x, top_p=0.5, min_tokens_to_keep=2)
    assert (p > 0).tolist() == [True, True, False, False, False]  # the tie goes to the lower index
    p = plain.sample_distribution(x, min_p=0.3)
    assert (p > 0).tolist() == [True, True, True, False, False]
    p = plain.sample_distribution(x, history=[4, 4, 0], repetition_penalty=2.0)
    q = plain.sample_distribution(np.array([1.0, 1.0, 1.0, 0.0, -2.0]))
    assert np.allclose(p, q)
    p = plain.sample_distribution(x, history=[1, 1], frequency_penalty=0.5, presence_penalty=0.25)
    assert np.allclose(p, plain.sample_distribution(np.array([2.0, -0.25, 1.0, 0.0, -1.0])))
    assert plain.pick_from([0.2, 0.3, 0.5], 0.2) == 1 and plain.pick_from([0.2, 0.3, 0.5], 0.1999) == 0


def test_splitmix64_first_draws():
    rng = plain.SplitMix64(0)
    assert rng.next_u64() == 0xE220A8397B1DCDAF  # the generator's published first output for seed 0
    u = plain.SplitMix64(1234).next_uniform()
    assert 0.0 <= u < 1.0
    from alofa_b200.sampling.rng import SplitMix64

    a, b = plain.SplitMix64(20260918), SplitMix64(20260918)
    assert [a.next_uniform() for _ in range(5)] == [b.next_uniform() for _ in range(5)]
