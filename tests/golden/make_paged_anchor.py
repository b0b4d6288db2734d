"""Anchor the plain implementation's attention on the reference's paged fixtures.

The reference project ships eleven paged-attention cases under
tests/fixtures/paged/ in the mojothon/alofa tree (4 heads on 2 KV heads, head
8, pages of 16): for each case the queries of its last q_len positions
(<case>.q.tsv), the keys and values of its whole context gathered through its
page table (<case>.kv.tsv), and the expected output (<case>.y.tsv) computed by
a reference written from the definition of causal grouped-query attention
(scripts/dump_paged_reference.py:111-160), which is what the reference's own
paged kernel (src/alofa/kernels/cpu/paged.mojo:249-336) is held to within
1e-5 (tests/unit/test_paged_attention.mojo:60-63).  Two negative controls
come with them: the first case's output with one element moved by 0.05
(expected_bad.tsv) and computed with the wrong head map h % kv_heads
(expected_hmap.tsv); a comparison that accepts either is broken.

This script feeds the cases through `attention` of tests/plain_qwen2.py and
writes the differences to paged_anchor.json; it also packs the cases into
paged_cases.npz (q, k, v, y per case, the two controls) so that the GPU tests
can run the engine's own paged-attention kernel on them.

    python tests/golden/make_paged_anchor.py <path to the reference checkout>
"""
import json
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import plain_qwen2 as plain  # noqa: E402

TOLERANCE = 1e-5  # the reference's own gate, relative to max(1, max|expected|)


def floats(path: Path) -> np.ndarray:
    return np.array([float(x) for x in path.read_text().split()], dtype=np.float64)


def read_cases(ref_root: str):
    folder = Path(ref_root) / "tests/fixtures/paged"
    cfg = {k: int(v) for k, v in (line.split("\t") for line in (folder / "config.tsv").read_text().splitlines())}
    nh, nkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    cases = {}
    for line in (folder / "cases.tsv").read_text().splitlines():
        if line.startswith("#"):
            continue
        fields = line.split("\t")
        name, q_len, n_entries = fields[0], int(fields[4]), int(fields[5])
        runs = [tuple(int(x) for x in fields[6 + 3 * i : 9 + 3 * i]) for i in range(n_entries)]
        kv_len = sum(r[2] for r in runs)
        kv = floats(folder / f"{name}.kv.tsv")
        cases[name] = {
            "q": floats(folder / f"{name}.q.tsv").reshape(q_len, nh * hd),
            "k": kv[: kv_len * nkv * hd].reshape(kv_len, nkv * hd),
            "v": kv[kv_len * nkv * hd :].reshape(kv_len, nkv * hd),
            "y": floats(folder / f"{name}.y.tsv").reshape(q_len, nh * hd),
        }
    first = next(iter(cases))
    controls = {"first": first, "bad": floats(folder / "expected_bad.tsv").reshape(cases[first]["y"].shape),
                "hmap": floats(folder / "expected_hmap.tsv").reshape(cases[first]["y"].shape)}
    return cfg, cases, controls


def plain_output(case, nh, nkv, hd, head_map=None):
    """plain.attention takes whole sequences: the case's queries are its last
    q_len positions, the earlier rows are padding whose output is dropped."""
    q_len, kv_len = case["q"].shape[0], case["k"].shape[0]
    q = np.zeros((kv_len, nh * hd))
    q[kv_len - q_len :] = case["q"]
    k, v = case["k"], case["v"]
    if head_map is not None:  # a deliberately wrong map, for the control: permute the KV heads each query head reads
        g = nh // nkv
        out = np.zeros((q_len, nh * hd))
        for h in range(nh):
            kh = head_map(h)
            one = plain.attention(q[:, h * hd : (h + 1) * hd], k[:, kh * hd : (kh + 1) * hd], v[:, kh * hd : (kh + 1) * hd], 1, 1, hd)
            out[:, h * hd : (h + 1) * hd] = one[kv_len - q_len :]
        return out
    return plain.attention(q, k, v, nh, nkv, hd)[kv_len - q_len :]


def derive(ref_root: str):
    cfg, cases, controls = read_cases(ref_root)
    nh, nkv, hd = cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"]
    result = {"config": cfg, "cases": {}}
    for name, case in cases.items():
        got = plain_output(case, nh, nkv, hd)
        diff = float(np.abs(got - case["y"]).max())
        bound = TOLERANCE * max(1.0, float(np.abs(case["y"]).max()))
        result["cases"][name] = {"max_abs_diff": diff, "bound": bound, "ok": diff <= bound, "q_len": int(case["q"].shape[0]), "kv_len": int(case["k"].shape[0])}
    first = cases[controls["first"]]
    got = plain_output(first, nh, nkv, hd)
    bound = TOLERANCE * max(1.0, float(np.abs(first["y"]).max()))
    wrong = plain_output(first, nh, nkv, hd, head_map=lambda h: h % nkv)
    result["controls"] = {
        "moved_element_is_caught": bool(np.abs(got - controls["bad"]).max() > bound),
        "wrong_head_map_is_caught": bool(np.abs(got - controls["hmap"]).max() > bound),
        "wrong_head_map_reproduced": bool(np.abs(wrong - controls["hmap"]).max() <= bound),  # the plain implementation with h % kv_heads gives the control's numbers
    }
    return result, (cfg, cases, controls)


def main(ref_root: str) -> None:
    result, (cfg, cases, controls) = derive(ref_root)
    here = Path(__file__).parent
    arrays = {"config": np.array([cfg["n_heads"], cfg["n_kv_heads"], cfg["head_dim"], cfg["block_size"]], dtype=np.int32)}
    for name, case in cases.items():
        for key, value in case.items():
            arrays[f"{name}.{key}"] = value.astype(np.float32)
    arrays["control.bad"] = controls["bad"].astype(np.float32)
    arrays["control.hmap"] = controls["hmap"].astype(np.float32)
    np.savez_compressed(here / "paged_cases.npz", **arrays)
    (here / "paged_anchor.json").write_text(json.dumps(result, indent=1, sort_keys=True) + "\n")
    print(json.dumps(result, indent=1, sort_keys=True))
    sys.exit(0 if all(c["ok"] for c in result["cases"].values()) and all(result["controls"].values()) else 1)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_paged_anchor.py <path to the reference checkout>")
    main(sys.argv[1])
