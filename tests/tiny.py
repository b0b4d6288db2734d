"""The tests' own small configurations of the Qwen2 architecture.  They differ
in every size and option: head counts and groups, sizes that are no power of
two, number of layers, vocabulary, eps, theta, tied head, window."""
import numpy as np
import torch

from alofa_b200.models.qwen2 import NAME, Qwen2Config
from alofa_b200.weights.random_init import write_random_model

CONFIGS = {
    # 2 layers, grouped (4 heads on 2 kv heads), head 16, tied head
    "A": (Qwen2Config(2, 64, 4, 2, 16, 128, 256, 1e-6, 1e4, True, 128), 0),
    # 3 layers, multi-query (3 heads on 1), head 32, odd vocabulary, untied head
    "B": (Qwen2Config(3, 96, 3, 1, 32, 320, 379, 1e-5, 1e6, False, 256), 1),
    # 3 layers, 5 heads on 5, head 48, layers 1.. see only the last 24 keys
    "C": (Qwen2Config(3, 240, 5, 5, 48, 200, 500, 3e-6, 5e4, False, 512, True, 24, 1), 2),
}


def write(folder, name, dtype=torch.bfloat16):
    cfg, seed = CONFIGS[name]
    return write_random_model(folder, NAME, cfg, seed, dtype)


def tokens(name, n, seed=0):
    cfg, _ = CONFIGS[name]
    rng = np.random.default_rng(1000 + seed)
    return [int(t) for t in rng.integers(0, cfg.vocab_size, size=n)]
