"""Pack the reference's scheduler traces for the test that replays them.

The reference project ships seven recorded runs of its scheduler under
tests/fixtures/scheduler/ in the mojothon/alofa tree (written by its
scripts/dump_scheduler_reference.py, an implementation of the same policy that
is independent of its Mojo scheduler; line format
src/alofa/engine/trace.mojo:63-238): a CFG line (token budget b, largest chunk
c, block size s, capacity in blocks k, watermark in permille w, latency guard
t) and per tick what came in (arrivals id:prompt:max_new, cancels, completions
the engine saw, blocks its prefix cache gave back) and what the scheduler
decided (prompt portions P, decoded requests D, preempted X, finished F).

This script parses the seven files into scheduler_fixtures.json beside it;
tests/test_scheduler.py feeds the inputs to this package's scheduler and says
tick by tick which decisions are the same and which differ on purpose.

    python tests/golden/make_scheduler_anchor.py <path to the reference checkout>
"""
import json
import sys
from pathlib import Path


def ids(text):
    return [] if text == "-" else [int(x) for x in text.split(",")]


def triples(text):
    return [] if text == "-" else [[int(x) for x in item.split(":")] for item in text.split(",")]


def parse(path: Path) -> dict:
    lines = path.read_text().splitlines()
    cfg = {k: int(v) for k, v in (item.split("=") for item in lines[0].split()[1:])}
    ticks = []
    for line in lines[1:]:
        head, tail = line.split(" OUT=")
        fin = dict(item.split("=", 1) for item in head[3:].split("|"))
        out = dict(item.split("=", 1) for item in tail.split())
        ticks.append({"A": triples(fin["A"]), "C": ids(fin["C"]), "F": ids(fin["F"]), "R": int(fin["R"]),
                      "P": triples(out["P"]), "D": ids(out["D"]), "X": ids(out["X"]), "Fout": ids(out["F"]), "preempt_total": int(out["C"])})
    return {"cfg": cfg, "ticks": ticks}


def main(ref_root: str) -> None:
    folder = Path(ref_root) / "tests/fixtures/scheduler"
    out = {p.stem: parse(p) for p in sorted(folder.glob("s0*.trace"))}
    assert len(out) == 7, sorted(out)
    Path(__file__).with_name("scheduler_fixtures.json").write_text(json.dumps(out, separators=(",", ":"), sort_keys=True) + "\n")
    print({k: len(v["ticks"]) for k, v in out.items()})


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_scheduler_anchor.py <path to the reference checkout>")
    main(sys.argv[1])
