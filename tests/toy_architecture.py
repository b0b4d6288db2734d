"""A toy architecture, defined in the tests only, that the package has never
heard of: a mixer that keeps a running mean of its inputs per request (state
of fixed size, no pages), a feed-forward that routes every token to one of a
few small experts, and an architecture ``ToyForCausalLM`` whose config.json
says, layer by layer, whether the mixer is the running mean or the stock paged
attention.  Importing this module registers all of it; nothing in the package
changes.  It is nobody's model: it exercises the registry, the loader, the
cache manager, the scheduler and the entry points with parts they do not know.
A plain restatement of the same arithmetic (NumPy float64) stands beside it."""
from dataclasses import dataclass

import numpy as np
import torch

import plain_qwen2 as plain
from alofa_b200.config.registry import Architecture, register_architecture
from alofa_b200.config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from alofa_b200.parts.base import Part, SlotState, TensorSpec, register_part

NAME = "ToyForCausalLM"
EPS, THETA = 2e-5, 777.0


class RunningMeanMixer(Part):
    family = "mixer"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden = int(self.param("hidden_size"))

    def tensors(self):
        return {self.prefix + "mix.weight": TensorSpec((self.hidden, self.hidden))}

    def load(self, state):
        self.w = state[self.prefix + "mix.weight"].float()

    def cache_spec(self):
        return SlotState((self.hidden + 1,), torch.float32)  # sum of inputs and their count

    def forward(self, ctx, x, h, cache, writes=True):
        starts = ctx.host_field("q_start")
        slots = ctx.host_field("state_slots")
        xf = x.float()
        for s in range(ctx.n_seqs):
            lo, hi = int(starts[s]), int(starts[s + 1])
            st = cache.state[int(slots[s])]
            sums = st[: self.hidden] + torch.cumsum(xf[lo:hi], dim=0)
            counts = st[self.hidden] + torch.arange(1, hi - lo + 1, device=x.device, dtype=torch.float32)
            h[lo:hi] += (sums / counts[:, None]) @ self.w.T
            st[: self.hidden] = sums[-1]
            st[self.hidden] = counts[-1]


class RoutedToyMLP(Part):
    family = "feed_forward"

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        self.hidden, self.experts = int(self.param("hidden_size")), int(self.param("experts"))

    def tensors(self):
        t = {self.prefix + "router.weight": TensorSpec((self.experts, self.hidden))}
        for e in range(self.experts):
            t[self.prefix + f"experts.{e}.weight"] = TensorSpec((self.hidden, self.hidden))
        return t

    def load(self, state):
        self.router = state[self.prefix + "router.weight"].float()
        self.w = [state[self.prefix + f"experts.{e}.weight"].float() for e in range(self.experts)]

    def forward(self, ctx, x, h):
        xf = x.float()
        choice = (xf @ self.router.T).argmax(dim=1)
        for e in range(self.experts):
            rows = (choice == e).nonzero().flatten()
            if rows.numel():
                h[rows] += xf[rows] @ self.w[e].T


class AddedPosition(Part):
    family = "position"

    def rotary_table(self):
        return None, 0

    def apply(self, ctx, q, k):
        shift = (ctx.positions.float() * 0.01)[:, None, None]
        q += shift.to(q.dtype)
        if k.shape[1]:
            k += shift.to(k.dtype)


def register_parts():
    for family, kind, cls in (("mixer", "toy_running_mean", RunningMeanMixer), ("feed_forward", "toy_routed", RoutedToyMLP), ("position", "toy_added", AddedPosition)):
        register_part(family, kind, cls, replace=True)


@dataclass
class ToyConfig:
    mixers: tuple  # per layer: "mean" (state of its own) or "attention" (paged keys and values)
    hidden: int = 40
    heads: int = 5
    kv_heads: int = 1
    head_dim: int = 8
    experts: int = 3
    vocab: int = 97
    max_position: int = 96


def read_config(obj: dict, origin: str) -> ToyConfig:
    return ToyConfig(tuple(obj["toy_mixers"]), int(obj["toy_hidden"]), int(obj["toy_heads"]), int(obj["toy_kv_heads"]), int(obj["toy_head_dim"]),
                     int(obj["toy_experts"]), int(obj["toy_vocab"]), int(obj["toy_max_position"]))


def to_json(cfg: ToyConfig) -> dict:
    return {"architectures": [NAME], "toy_mixers": list(cfg.mixers), "toy_hidden": cfg.hidden, "toy_heads": cfg.heads, "toy_kv_heads": cfg.kv_heads,
            "toy_head_dim": cfg.head_dim, "toy_experts": cfg.experts, "toy_vocab": cfg.vocab, "toy_max_position": cfg.max_position}


def build_spec(cfg: ToyConfig) -> ModelSpec:
    layers = []
    for i, kind in enumerate(cfg.mixers):
        p = f"layers.{i}."
        if kind == "mean":
            mixer = PartSpec("toy_running_mean", {"hidden_size": cfg.hidden}, prefix=p + "attn.")
        else:
            pos = PartSpec("rotary_neox", {"head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": THETA, "max_position": cfg.max_position}, prefix=p + "pos.")
            mixer = PartSpec("gqa_attention", {"hidden_size": cfg.hidden, "num_heads": cfg.heads, "num_kv_heads": cfg.kv_heads, "head_dim": cfg.head_dim,
                                               "qkv_bias": True, "out_bias": False, "window": None, "position": pos}, prefix=p + "attn.")
        ffn = PartSpec("toy_routed", {"hidden_size": cfg.hidden, "experts": cfg.experts}, prefix=p + "ffn.")
        norm = lambda name: PartSpec("rmsnorm", {"size": cfg.hidden, "eps": EPS}, prefix=p + name + ".")
        layers.append(LayerSpec(PartSpec("prenorm_residual", {"mixer": mixer, "feed_forward": ffn, "mixer_norm": norm("n1"), "feed_forward_norm": norm("n2")}, prefix=p)))
    return ModelSpec(NAME, cfg.hidden, cfg.vocab, cfg.max_position, PartSpec("token_embedding", {"vocab_size": cfg.vocab, "hidden_size": cfg.hidden}, prefix="embed."),
                     layers, [RunEntry(i, i) for i in range(len(layers))], PartSpec("rmsnorm", {"size": cfg.hidden, "eps": EPS}, prefix="norm."),
                     PartSpec("linear_head", {"vocab_size": cfg.vocab, "hidden_size": cfg.hidden, "tied_to": None}, prefix="head."))


register_parts()
register_architecture(Architecture(NAME, read_config, build_spec, to_json), replace=True)


# -- the plain restatement -------------------------------------------------------
def plain_forward(ids, w, cfg: ToyConfig):
    """Logits [n, vocab] of one whole sequence (float64)."""
    n = len(ids)
    positions = np.arange(n)
    h = plain.embed(ids, w["embed.weight"])
    for i, kind in enumerate(cfg.mixers):
        p = f"layers.{i}."
        x = plain.rmsnorm(h, w[p + "n1.weight"], EPS)
        if kind == "mean":
            mean = np.cumsum(x, axis=0) / np.arange(1, n + 1)[:, None]
            h = h + mean @ w[p + "attn.mix.weight"].T
        else:
            a = p + "attn."
            q = plain.rope(plain.linear(x, w[a + "q_proj.weight"], w[a + "q_proj.bias"]), positions, cfg.heads, cfg.head_dim, THETA)
            k = plain.rope(plain.linear(x, w[a + "k_proj.weight"], w[a + "k_proj.bias"]), positions, cfg.kv_heads, cfg.head_dim, THETA)
            v = plain.linear(x, w[a + "v_proj.weight"], w[a + "v_proj.bias"])
            h = h + plain.linear(plain.attention(q, k, v, cfg.heads, cfg.kv_heads, cfg.head_dim), w[a + "o_proj.weight"])
        x = plain.rmsnorm(h, w[p + "n2.weight"], EPS)
        choice = (x @ w[p + "ffn.router.weight"].T).argmax(axis=1)
        h = h + np.stack([x[t] @ w[p + f"ffn.experts.{choice[t]}.weight"].T for t in range(n)])
    return plain.linear(plain.rmsnorm(h, w["norm.weight"], EPS), w["head.weight"])


def plain_greedy(ids, n_new, w, cfg):
    seq, out = list(ids), []
    for _ in range(n_new):
        tok = plain.argmax(plain_forward(seq, w, cfg)[-1])
        out.append(tok)
        seq.append(tok)
    return out
