"""Anchor the plain implementation's sampler on the reference's sampler fixtures.

The reference project ships, under tests/fixtures/qwen2.5-0.5b/sampler/ in the
mojothon/alofa tree, nine sampling cases over four real logits rows of
Qwen2.5-0.5B (../logits_last.f32): for each case its parameters (cases.tsv,
bias.tsv, history.tsv), the final probability vector (probs.f32), the
surviving set (count, first ids and an FNV-1a fingerprint of all ids:
sets.tsv) and the 32 ids drawn with SplitMix64 of a named seed (sampled.tsv),
plus the generator's first 64 raw outputs (draws.tsv) and top-k sets on a row
full of ties (ties/).  They were written by the reference's
scripts/dump_sampler_reference.py (format: its lines 40-66) and are what its
own sampler (src/alofa/runtime/sampler.mojo:308-481) is tested against.

This script feeds the same inputs through tests/plain_qwen2.py
(`SplitMix64`, `sample_distribution`, `pick_from`) and writes what differs to
sampler_anchor.json beside it.  It also writes sampler_rows.npz: the four
logits rows cut down to their 8,192 largest entries (plus every id that a
case's history or bias names), with the reference's expected ids mapped into
the cut rows, so that a GPU test can run the device sampling chain on real
logits without the 2.4 MB file.  For the cases with a top-k the cut changes
nothing (everything that survives lies inside it), so their expected ids are
the reference's own; for the three cases where the whole vocabulary survives
the expected ids come from the plain implementation on the cut row.

    python tests/golden/make_sampler_anchor.py <path to the reference checkout>
"""
import json
import sys
from pathlib import Path

import numpy as np

sys.path.insert(0, str(Path(__file__).resolve().parents[1]))
import plain_qwen2 as plain  # noqa: E402

MASK64 = (1 << 64) - 1
KEEP = 8192


def fnv1a64(indices) -> int:
    """The fingerprint of a set of ids as the fixture's writer computes it
    (scripts/dump_sampler_reference.py:126-141): FNV-1a over the eight bytes of
    every id, lowest byte first."""
    h = 0xCBF29CE484222325
    for i in indices:
        v = int(i)
        for _ in range(8):
            h = ((h ^ (v & 0xFF)) * 0x100000001B3) & MASK64
            v >>= 8
    return h


def read_cases(folder: Path):
    biases, histories = {}, {}
    for line in (folder / "bias.tsv").read_text().splitlines():
        name, idx, val = line.split("\t")
        biases.setdefault(name, []).append((int(idx), float(val)))
    for line in (folder / "history.tsv").read_text().splitlines():
        name, ids = line.split("\t")
        histories[name] = [int(t) for t in ids.split(",")]
    cases = []
    for line in (folder / "cases.tsv").read_text().splitlines():
        name, prompt, temp, top_k, top_p, min_p, rep, freq, pres, bias, hist = line.split("\t")
        cases.append(dict(name=name, prompt=int(prompt), temperature=float(temp), top_k=int(top_k), top_p=float(top_p), min_p=float(min_p),
                          repetition_penalty=float(rep), frequency_penalty=float(freq), presence_penalty=float(pres),
                          logit_bias=biases.get(bias, []), history=histories.get(hist, [])))
    return cases


def distribution(case, row):
    args = {k: case[k] for k in ("history", "temperature", "top_k", "top_p", "min_p", "repetition_penalty", "frequency_penalty", "presence_penalty", "logit_bias")}
    return plain.sample_distribution(row, min_tokens_to_keep=1, **args)


def draw_ids(probs, seed: int, count: int):
    """`count` ids by plain.pick_from; zero entries are left out of the walk
    (they add nothing to the running sum) and the hit is mapped back."""
    alive = np.nonzero(probs)[0]
    weights = [float(w) for w in probs[alive]]
    rng = plain.SplitMix64(seed)
    return [int(alive[plain.pick_from(weights, rng.next_uniform())]) for _ in range(count)]


def derive(ref_root: str, with_rows: bool = False):
    fixtures = Path(ref_root) / "tests/fixtures/qwen2.5-0.5b"
    folder = fixtures / "sampler"
    manifest = dict(line.split("\t") for line in (folder / "manifest.tsv").read_text().splitlines())
    vocab, seed, n_ids = int(manifest["vocab"]), int(manifest["seed"]), int(manifest["n_sample_ids"])
    logits = np.fromfile(fixtures / "logits_last.f32", dtype="<f4").reshape(-1, vocab)
    result = {"seed": seed, "vocab": vocab}

    # the generator: the first 64 raw outputs of the named seed
    lines = (folder / "draws.tsv").read_text().splitlines()
    assert lines[0] == f"seed\t{seed}"
    want = [int(line.split("\t")[1]) for line in lines[1:]]
    rng = plain.SplitMix64(seed)
    got = [rng.next_u64() for _ in want]
    result["splitmix64"] = {"outputs": len(want), "mismatches": sum(a != b for a, b in zip(got, want))}

    probs_ref = np.fromfile(folder / "probs.f32", dtype="<f4")
    offsets = {l.split("\t")[0]: int(l.split("\t")[2]) for l in (folder / "probs.tsv").read_text().splitlines()}
    sets = {l.split("\t")[0]: l.split("\t")[1:] for l in (folder / "sets.tsv").read_text().splitlines()}
    sampled = {l.split("\t")[0]: [int(t) for t in l.split("\t")[1].split(",")] for l in (folder / "sampled.tsv").read_text().splitlines()}
    cases = read_cases(folder)
    result["cases"] = {}
    rows_out = {}
    for case in cases:
        name = case["name"]
        probs = distribution(case, logits[case["prompt"]])
        ref = probs_ref[offsets[name] : offsets[name] + vocab].astype(np.float64)
        alive = np.nonzero(probs)[0]
        count, head, digest = sets[name]
        ids = draw_ids(probs, seed, n_ids)
        result["cases"][name] = {
            "max_abs_prob_diff": float(np.abs(probs.astype(np.float32).astype(np.float64) - ref).max()),
            "survivors": int(alive.size), "survivors_ref": int(count),
            "first_survivors_equal": [int(i) for i in alive[:16]] == [int(t) for t in head.split(",")],
            "fingerprint_equal": fnv1a64(alive) == int(digest),
            "sampled_mismatches": sum(a != b for a, b in zip(ids, sampled[name])), "sampled": n_ids,
        }
        if with_rows:
            rows_out[name] = (case, ids)

    # top-k on a row full of ties: only the sets (every value >= the k-th largest survives)
    ties = folder / "ties"
    row = np.fromfile(ties / "logits.f32", dtype="<f4")
    result["ties"] = {}
    for line in (ties / "sets.tsv").read_text().splitlines():
        name, count, ids = line.split("\t")
        k = int(name[1:])
        probs = plain.sample_distribution(row, temperature=1.0, top_k=k)
        result["ties"][name] = {"equal": [int(i) for i in np.nonzero(probs)[0]] == [int(t) for t in ids.split(",")], "survivors_ref": int(count)}
    return result, (logits, cases, rows_out, seed, n_ids)


def cut_rows(logits, cases, rows_out, seed, n_ids):
    """The logits rows reduced to their largest KEEP entries (see the header)."""
    keep_ids, cut = [], []
    for r in range(logits.shape[0]):
        named = set()
        for case in cases:
            if case["prompt"] == r:
                named.update(case["history"])
                named.update(i for i, _ in case["logit_bias"])
        order = np.argsort(-logits[r], kind="stable")[:KEEP]
        ids = np.array(sorted(set(int(i) for i in order) | named), dtype=np.int64)
        keep_ids.append(ids)
        cut.append(logits[r][ids])
    out = {"seed": np.array([seed], dtype=np.uint64)}
    for r, (ids, vals) in enumerate(zip(keep_ids, cut)):
        out[f"row{r}_ids"] = ids.astype(np.int32)
        out[f"row{r}_logits"] = vals.astype(np.float32)
    expected = {}
    for case in cases:
        ids = keep_ids[case["prompt"]]
        where = {int(t): i for i, t in enumerate(ids)}
        local = dict(case)
        local["history"] = [where[t] for t in case["history"]]
        local["logit_bias"] = [(where[i], v) for i, v in case["logit_bias"]]
        row = cut[case["prompt"]]
        plain_ids = [int(ids[i]) for i in draw_ids(distribution(local, row), seed, n_ids)]
        ref_ids = rows_out[case["name"]][1]
        whole_vocabulary = case["top_k"] == 0 and case["temperature"] > 0.0
        expected[case["name"]] = {"ids": plain_ids, "from": "plain implementation on the cut row" if whole_vocabulary else "reference"}
        if not whole_vocabulary:
            assert plain_ids == ref_ids, case["name"]
    return out, expected


def main(ref_root: str) -> None:
    result, rest = derive(ref_root, with_rows=True)
    logits, cases, rows_out, seed, n_ids = rest
    arrays, expected = cut_rows(logits, cases, rows_out, seed, n_ids)
    here = Path(__file__).parent
    np.savez_compressed(here / "sampler_rows.npz", **arrays)
    case_table = [{k: v for k, v in case.items()} for case in cases]
    (here / "sampler_rows.json").write_text(json.dumps({"cases": case_table, "expected": expected, "seed": seed, "draws": n_ids}, indent=1) + "\n")
    (here / "sampler_anchor.json").write_text(json.dumps(result, indent=1, sort_keys=True) + "\n")
    print(json.dumps(result, indent=1, sort_keys=True))


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_sampler_anchor.py <path to the reference checkout>")
    main(sys.argv[1])
