"""Anchor the plain implementation's formulas on the reference's layer-0 capture.

The reference project ships Hugging Face forward-hook captures of layer 0 of
Qwen2.5-0.5B for 16 tokens (tests/fixtures/qwen2.5-0.5b/layer0/tensors.tsv and
tensors.f32 in the mojothon/alofa tree) together with that layer's real
weights.  This script feeds the captured inputs through the functions of
tests/plain_qwen2.py and writes the largest absolute differences to
layer0_anchor.json beside it.  The reference's own gate for these operators is
1e-5 * max(1, max|ref|) (tests/unit/test_layer0_parity.mojo:12-16).

The reference's model code is Mojo and cannot be run where this script runs;
only its captured tensors are read.

    python tests/golden/make_layer0_anchor.py <path to the reference checkout>
"""
import json
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import plain_qwen2 as plain  # noqa: E402


def read_capture(folder: Path) -> dict:
    blob = np.fromfile(folder / "tensors.f32", dtype="<f4")
    out = {}
    for line in (folder / "tensors.tsv").read_text().splitlines():
        name, shape, offset, count = line.split("\t")
        dims = tuple(int(d) for d in shape.split("x"))
        start = int(offset) // 4
        out[name] = blob[start : start + int(count)].reshape(dims).astype(np.float64)
    return out


def main(ref_root: str) -> None:
    cap = read_capture(Path(ref_root) / "tests/fixtures/qwen2.5-0.5b/layer0")
    nh, nkv, hd, eps, theta = 14, 2, 64, 1e-6, 1e6
    n = cap["embed_out"].shape[0]
    pos = np.arange(n)
    result = {}

    def gate(name, got, want):
        diff = float(np.abs(got - want).max())
        bound = 1e-5 * max(1.0, float(np.abs(want).max()))
        result[name] = {"max_abs_diff": diff, "bound": bound, "ok": diff <= bound}

    gate("rmsnorm", plain.rmsnorm(cap["embed_out"], cap["norm_w"], eps), cap["norm_out"])
    gate("q_proj", plain.linear(cap["norm_out"], cap["q_w"], cap["q_b"]), cap["q_out"])
    gate("k_proj", plain.linear(cap["norm_out"], cap["k_w"], cap["k_b"]), cap["k_out"])
    gate("v_proj", plain.linear(cap["norm_out"], cap["v_w"], cap["v_b"]), cap["v_out"])
    cos, sin = plain.rope_table(pos, hd, theta)
    gate("rope_cos_table", cos, cap["cos"][:, : hd // 2])
    gate("rope_sin_table", sin, cap["sin"][:, : hd // 2])
    gate("rope_q", plain.rope(cap["q_out"], pos, nh, hd, theta), cap["q_rot"])
    gate("rope_k", plain.rope(cap["k_out"], pos, nkv, hd, theta), cap["k_rot"])
    gate(
        "attention",
        plain.attention(cap["q_rot"], cap["k_rot"], cap["v_out"], nh, nkv, hd),
        cap["attn_out"],
    )
    gate("o_proj", plain.linear(cap["attn_out"], cap["o_w"]), cap["o_out"])
    gate("residual", cap["embed_out"] + cap["o_out"], cap["hidden1"])
    gate("rmsnorm2", plain.rmsnorm(cap["hidden1"], cap["norm2_w"], eps), cap["norm2_out"])
    gate("silu", plain.silu(cap["gate_out"]), cap["silu_out"])
    gate("swiglu", plain.silu(cap["gate_out"]) * cap["up_out"], cap["swiglu_out"])
    out = Path(__file__).with_name("layer0_anchor.json")
    out.write_text(json.dumps(result, indent=1, sort_keys=True) + "\n")
    bad = [k for k, v in result.items() if not v["ok"]]
    print("wrote", out, "failed:", bad)
    sys.exit(1 if bad else 0)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_layer0_anchor.py <path to the reference checkout>")
    main(sys.argv[1])
