"""``generate``: token ids in, token ids out, with timing.

    python -m alofa_b200.cli.generate --model DIR --prompt-ids 1,2,3 --max-new-tokens 16
    python -m alofa_b200.cli.generate --random-config config.json --weights-seed 0 --prompt-len 100

The reference's ``generate`` (src/alofa/cli.mojo:361-560, 1054-1119) has no
flags (a compiled Mojo binary sees no argv; its settings are constants,
cli.mojo:109-171, and the server's are environment variables,
src/alofa/srv/config.mojo:73-107).  This command keeps those names and
meanings as flags, with the environment variables as defaults: ALOFA_WEIGHTS
(the model folder), ALOFA_MAX_TOKENS (context window per request),
ALOFA_MAX_PROMPT_TOKENS, ALOFA_SEED.  It prints what the reference prints:
prompt ids, generated ids, ticks, preemptions, prefill time, decode time per
token (mean and median) and tokens per second (cli.mojo:319-358, 530-535).
Text goes through no tokenizer: prompts are token ids.

``--random-config FILE`` runs a model of seeded random weights made in memory
from a config.json (no folder is written; ``--weights-seed`` names the seed),
and ``--dump-logits FILE`` writes the logits every generated token was sampled
from: little-endian float32 rows ``[tokens, vocab]`` in the order the tokens
were produced, as ``bin/trace_run`` writes them, with ``FILE.tsv`` naming each
row's request (its index among the prompts) and which of its tokens it is."""
from __future__ import annotations

import argparse
import json
import os
import statistics
import sys
import time

# defaults of the reference's command line (src/alofa/cli.mojo:109-171)
DEFAULT_NEW = 16
SEED = 20260918


def _env_int(name: str, default: int, lo: int, hi: int) -> int:
    raw = os.environ.get(name, "")
    if not raw:
        return default
    try:
        value = int(raw)
    except ValueError:
        raise SystemExit(f"environment variable is not an integer: {name}={raw}")
    if not lo <= value <= hi:
        raise SystemExit(f"environment variable is out of range: {name}={value} not in [{lo}, {hi}]")
    return value


def build_parser() -> argparse.ArgumentParser:
    ap = argparse.ArgumentParser(prog="generate", description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--model", default=os.environ.get("ALOFA_WEIGHTS"), help="folder with config.json and model.safetensors [ALOFA_WEIGHTS]")
    ap.add_argument("--random-config", metavar="FILE", help="instead of --model: a config.json; the weights are seeded random numbers, made in memory")
    ap.add_argument("--weights-seed", type=int, default=0, help="seed of the random weights of --random-config")
    ap.add_argument("--dump-logits", metavar="FILE", help="write the logits each generated token was sampled from (float32 rows), and FILE.tsv")
    ap.add_argument("--prompt-ids", action="append", help="comma-separated token ids; repeat for several requests")
    ap.add_argument("--prompt-len", type=int, help="instead of --prompt-ids: this many uniform random token ids")
    ap.add_argument("--num-prompts", type=int, default=1, help="how many random prompts with --prompt-len")
    ap.add_argument("--max-new-tokens", type=int, default=DEFAULT_NEW)
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16")
    # sampling: the reference's SampleParams (src/alofa/runtime/sampler.mojo:93-118)
    ap.add_argument("--temperature", type=float, default=0.0, help="0 = greedy")
    ap.add_argument("--top-k", type=int, default=0)
    ap.add_argument("--top-p", type=float, default=1.0)
    ap.add_argument("--min-p", type=float, default=0.0)
    ap.add_argument("--repetition-penalty", type=float, default=1.0)
    ap.add_argument("--frequency-penalty", type=float, default=0.0)
    ap.add_argument("--presence-penalty", type=float, default=0.0)
    ap.add_argument("--min-tokens-to-keep", type=int, default=1)
    ap.add_argument("--logit-bias", action="append", default=[], metavar="ID:VALUE[,ID:VALUE...]",
                    help="added to the logit of token ID before anything else; repeatable")
    ap.add_argument("--seed", "--sample-seed", dest="seed", type=int, default=_env_int("ALOFA_SEED", SEED, 0, 2_147_483_647), help="sampling seed [ALOFA_SEED]")
    ap.add_argument("--eos-token-id", type=int, default=None)
    # engine: the reference's SchedConfig (src/alofa/engine/scheduler.mojo:139-192)
    ap.add_argument("--max-tokens", type=int, default=_env_int("ALOFA_MAX_TOKENS", 4096, 1, 1 << 20), help="context window per request [ALOFA_MAX_TOKENS]")
    ap.add_argument("--max-prompt-tokens", type=int, default=_env_int("ALOFA_MAX_PROMPT_TOKENS", 1 << 20, 1, 1 << 20), help="longest prompt accepted [ALOFA_MAX_PROMPT_TOKENS]")
    ap.add_argument("--token-budget", type=int, default=2112)
    ap.add_argument("--max-chunk", type=int, default=2048)
    ap.add_argument("--block-size", type=int, default=64)
    ap.add_argument("--capacity-blocks", type=int, default=0, help="pages per cache group; 0 = max_batch full contexts")
    ap.add_argument("--watermark-permille", type=int, default=1000)
    ap.add_argument("--max-wait-ticks", type=int, default=8)
    ap.add_argument("--max-batch", type=int, default=8)
    ap.add_argument("--admission", choices=["committed", "optimistic"], default="committed")
    ap.add_argument("--trace-out", help="write the scheduler's decisions, one line per tick")
    ap.add_argument("--json", action="store_true", help="print one JSON object instead of text")
    return ap


def parse_logit_bias(items) -> dict:
    """``["5:1.5,7:-2", "9:0.25"]`` -> ``{5: 1.5, 7: -2.0, 9: 0.25}`` (the
    reference's ``LogitBias(index, value)`` list, sampler.mojo:93-118); a token
    named twice has its values added, as a list of additive entries would."""
    bias: dict = {}
    for item in items:
        for pair in item.split(","):
            if not pair.strip():
                continue
            index, sep, value = pair.partition(":")
            try:
                if not sep:
                    raise ValueError
                token, offset = int(index), float(value)
            except ValueError:
                raise SystemExit(f"generate: --logit-bias wants ID:VALUE, got {pair.strip()!r}") from None
            bias[token] = bias.get(token, 0.0) + offset
    return bias


def main(argv=None) -> int:
    args = build_parser().parse_args(argv)
    if args.random_config and args.model and not os.environ.get("ALOFA_WEIGHTS") == args.model:
        raise SystemExit("generate: give --model or --random-config, not both")
    if not args.model and not args.random_config:
        raise SystemExit("generate: --model (or ALOFA_WEIGHTS) or --random-config is required")
    from alofa_b200.engine.engine import Engine
    from alofa_b200.sampling.params import SamplingParams

    settings = dict(
        dtype=args.dtype, max_tokens=args.max_tokens, token_budget=args.token_budget, max_chunk=args.max_chunk,
        block_size=args.block_size, capacity_blocks=args.capacity_blocks, watermark_permille=args.watermark_permille,
        max_wait_ticks=args.max_wait_ticks, max_batch=args.max_batch, admission=args.admission, trace_out=args.trace_out,
    )
    if args.random_config:
        from alofa_b200.config.registry import read_model_config_file

        arch, cfg = read_model_config_file(args.random_config)
        engine = Engine.from_random(arch.name, cfg, args.weights_seed, **settings)
    else:
        engine = Engine(args.model, **settings)
    dump = None
    if args.dump_logits:
        dump = {"file": open(args.dump_logits, "wb"), "rows": [], "count": {}}

        def sink(request_ids, rows):
            dump["file"].write(rows.astype("<f4").tobytes())
            for rid in request_ids:
                dump["rows"].append((rid, dump["count"].get(rid, 0)))
                dump["count"][rid] = dump["count"].get(rid, 0) + 1

        engine.logits_sink = sink
    vocab = engine.model.spec.vocab_size
    if args.prompt_ids:
        prompts = [[int(t) for t in p.split(",") if t.strip()] for p in args.prompt_ids]
    elif args.prompt_len:
        import numpy as np

        rng = np.random.default_rng(args.seed)
        prompts = [[int(t) for t in rng.integers(0, vocab, size=args.prompt_len)] for _ in range(args.num_prompts)]
    else:
        raise SystemExit("generate: give --prompt-ids or --prompt-len")
    for p in prompts:
        if len(p) > args.max_prompt_tokens:
            raise SystemExit(f"generate: prompt of {len(p)} tokens is longer than --max-prompt-tokens {args.max_prompt_tokens}")
    sampling = SamplingParams(
        temperature=args.temperature, top_k=args.top_k, top_p=args.top_p, min_p=args.min_p, repetition_penalty=args.repetition_penalty,
        frequency_penalty=args.frequency_penalty, presence_penalty=args.presence_penalty, min_tokens_to_keep=args.min_tokens_to_keep,
        logit_bias=parse_logit_bias(args.logit_bias), seed=args.seed, max_new_tokens=args.max_new_tokens, stop_token_ids=(args.eos_token_id,) if args.eos_token_id is not None else (),
    )
    t0 = time.perf_counter()
    outputs = engine.generate(prompts, sampling=sampling)
    wall = time.perf_counter() - t0
    engine.close()
    if dump is not None:
        dump["file"].close()
        first = min((rid for rid, _ in dump["rows"]), default=0)  # request ids are handed out in prompt order
        with open(args.dump_logits + ".tsv", "w") as fh:
            for rid, k in dump["rows"]:
                fh.write(f"{rid - first}\t{k}\n")
    stats = engine.stats()
    prefill_ms = sum(engine.timings["prefill_ms"])
    decode = engine.timings["decode_ms"]
    n_out = sum(len(o) for o in outputs)
    report = {
        "prompt_ids": prompts, "out_ids": outputs, "ticks": stats["ticks"], "preemptions": stats["preempt_total"],
        "prefill_ms": round(prefill_ms, 3), "decode_ms_per_step_mean": round(statistics.fmean(decode), 4) if decode else None,
        "decode_ms_per_step_median": round(statistics.median(decode), 4) if decode else None,
        "tok_per_s": round(n_out / wall, 2) if wall > 0 else None, "rows_run": stats["rows_run"],
    }
    if args.json:
        print(json.dumps(report))
        return 0
    for p, o in zip(prompts, outputs):
        print("prompt ids:", " ".join(map(str, p)))
        print("out ids   :", " ".join(map(str, o)))
    print(f"ticks {report['ticks']}  preemptions {report['preemptions']}  rows {report['rows_run']}")
    print(f"prefill {report['prefill_ms']} ms  decode {report['decode_ms_per_step_mean']} ms/step mean, {report['decode_ms_per_step_median']} median  {report['tok_per_s']} tok/s")
    return 0


if __name__ == "__main__":
    sys.exit(main())
