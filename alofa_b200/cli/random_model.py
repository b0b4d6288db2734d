"""Write a model folder with seeded random weights.

    python -m alofa_b200.cli.random_model --config config.json --seed 0 --out DIR [--dtype bfloat16|float32]

``--config`` is a config.json of a registered architecture (its own keys);
the folder gets that config.json and a model.safetensors whose matrices and
biases are drawn from N(0, 0.02) and whose norm weights from 1 + N(0, 0.01),
every tensor from its own generator seeded by (seed, tensor name)."""
from __future__ import annotations

import argparse
import sys
from pathlib import Path


def main(argv=None) -> int:
    ap = argparse.ArgumentParser(description=__doc__, formatter_class=argparse.RawDescriptionHelpFormatter)
    ap.add_argument("--config", required=True, help="config.json naming the architecture and its sizes")
    ap.add_argument("--seed", type=int, default=0)
    ap.add_argument("--out", required=True, help="folder to write")
    ap.add_argument("--dtype", choices=["bfloat16", "float32"], default="bfloat16", help="dtype the tensors are stored in")
    args = ap.parse_args(argv)
    import torch

    from alofa_b200.config.registry import read_model_config_file
    from alofa_b200.weights.random_init import write_random_model

    arch, cfg = read_model_config_file(args.config)
    folder = write_random_model(args.out, arch.name, cfg, args.seed, torch.bfloat16 if args.dtype == "bfloat16" else torch.float32)
    print(folder)
    return 0


if __name__ == "__main__":
    sys.exit(main())
