"""The command line's options, parsed without building an engine (no GPU):
the reference's names and defaults for sampling (src/alofa/runtime/sampler.mojo:93-118)
and scheduling (src/alofa/engine/scheduler.mojo:139-192)."""
import pytest

from alofa_b200.cli.generate import build_parser, parse_logit_bias
from alofa_b200.sampling.params import SamplingParams


def test_sampling_defaults_are_the_references_except_greedy_temperature():
    args = build_parser().parse_args(["--model", "m", "--prompt-ids", "1,2"])
    ref = SamplingParams()
    assert args.temperature == 0.0  # the command line decodes greedily unless told otherwise
    for name in ("top_k", "top_p", "min_p", "repetition_penalty", "frequency_penalty", "presence_penalty", "min_tokens_to_keep"):
        assert getattr(args, name) == getattr(ref, name), name
    assert args.logit_bias == [] and args.eos_token_id is None


def test_environment_gives_defaults_and_flags_win(monkeypatch):
    monkeypatch.setenv("ALOFA_WEIGHTS", "/somewhere")
    monkeypatch.setenv("ALOFA_MAX_TOKENS", "777")
    monkeypatch.setenv("ALOFA_SEED", "99")
    args = build_parser().parse_args(["--prompt-len", "5"])
    assert (args.model, args.max_tokens, args.seed) == ("/somewhere", 777, 99)
    args = build_parser().parse_args(["--model", "x", "--max-tokens", "64", "--seed", "3", "--prompt-len", "5"])
    assert (args.model, args.max_tokens, args.seed) == ("x", 64, 3)


def test_logit_bias_pairs():
    assert parse_logit_bias([]) == {}
    assert parse_logit_bias(["5:1.5,7:-2", " 9:0.25 "]) == {5: 1.5, 7: -2.0, 9: 0.25}
    assert parse_logit_bias(["5:1", "5:2.5"]) == {5: 3.5}  # additive entries add up
    for bad in ("5", "a:1", "5:x", "5:1:2"):
        with pytest.raises(SystemExit):
            parse_logit_bias([bad])
    args = build_parser().parse_args(["--model", "m", "--prompt-ids", "1", "--logit-bias", "3:1", "--logit-bias", "4:-1"])
    params = SamplingParams(logit_bias=parse_logit_bias(args.logit_bias))
    assert not params.plain()  # a bias takes the whole sampling chain
    params.validate(vocab_size=5)
    with pytest.raises(Exception):
        SamplingParams(logit_bias={5: 1.0}).validate(vocab_size=5)


def test_several_prompts_and_scheduler_options():
    args = build_parser().parse_args(["--model", "m", "--prompt-ids", "1,2,3", "--prompt-ids", "4,5", "--token-budget", "32", "--max-chunk", "16",
                                      "--block-size", "16", "--max-batch", "4", "--watermark-permille", "900", "--max-wait-ticks", "8",
                                      "--admission", "optimistic"])
    assert args.prompt_ids == ["1,2,3", "4,5"]
    assert (args.token_budget, args.max_chunk, args.block_size, args.max_batch, args.watermark_permille, args.max_wait_ticks, args.admission) == (
        32, 16, 16, 4, 900, 8, "optimistic")


def test_random_config_and_dump_logits_flags():
    args = build_parser().parse_args(["--random-config", "cfg.json", "--weights-seed", "4", "--prompt-len", "5", "--dump-logits", "out.f32", "--sample-seed", "11"])
    assert (args.random_config, args.weights_seed, args.dump_logits, args.seed, args.model) == ("cfg.json", 4, "out.f32", 11, None)
