"""The Qwen2 dense grouped-query decoder (``Qwen2ForCausalLM``).

RMSNorm, q/k/v projections with bias and an output projection without,
NeoX-style rotary position encoding, a SiLU-gated feed-forward, and a tied or
untied output head, arranged as pre-norm residual layers
(src/alofa/model/arch/qwen.mojo:1362-1525).  This file only reads the
architecture's config keys and describes the model as a
:class:`~alofa_b200.config.spec.ModelSpec`; the parts it names live in
:mod:`alofa_b200.parts` and know nothing about Qwen2."""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

from ..config.json_reader import Keys
from ..config.registry import Architecture, register_architecture
from ..config.spec import LayerSpec, ModelSpec, PartSpec, RunEntry
from ..errors import AlofaError

NAME = "Qwen2ForCausalLM"


@dataclass
class Qwen2Config:
    """The numbers of ``config.json`` (src/alofa/model/arch/qwen.mojo:915-998
    reads the first ten; the rest are read here in addition)."""

    num_hidden_layers: int
    hidden_size: int
    num_attention_heads: int
    num_key_value_heads: int
    head_dim: int
    intermediate_size: int
    vocab_size: int
    rms_norm_eps: float
    rope_theta: float
    tie_word_embeddings: bool
    max_position_embeddings: int
    use_sliding_window: bool = False
    sliding_window: Optional[int] = None
    max_window_layers: Optional[int] = None
    hidden_act: str = "silu"

    def validate(self, origin: str = "") -> None:
        """The reference's checks (qwen.mojo:970-994, 852-857) and a few more."""

        def need(ok, what, detail):
            if not ok:
                raise AlofaError("parse", what, f"{detail} config={origin}")

        c = self
        need(c.num_hidden_layers > 0, "num_hidden_layers must be positive", f"num_hidden_layers={c.num_hidden_layers}")
        need(c.hidden_size > 0, "hidden_size must be positive", f"hidden_size={c.hidden_size}")
        need(c.num_attention_heads > 0, "num_attention_heads must be positive", f"num_attention_heads={c.num_attention_heads}")
        need(
            c.num_key_value_heads > 0 and c.num_attention_heads % c.num_key_value_heads == 0,
            "num_key_value_heads must be positive and divide num_attention_heads",
            f"num_attention_heads={c.num_attention_heads} num_key_value_heads={c.num_key_value_heads}",
        )
        need(c.head_dim > 0 and c.head_dim % 2 == 0, "head_dim must be positive and even", f"head_dim={c.head_dim}")
        need(
            c.num_attention_heads * c.head_dim == c.hidden_size,
            "num_attention_heads * head_dim must equal hidden_size",
            f"num_attention_heads={c.num_attention_heads} head_dim={c.head_dim} hidden_size={c.hidden_size}",
        )
        need(c.intermediate_size > 0, "intermediate_size must be positive", f"intermediate_size={c.intermediate_size}")
        need(c.vocab_size > 0, "vocab_size must be positive", f"vocab_size={c.vocab_size}")
        need(c.rms_norm_eps > 0, "rms_norm_eps must be positive", f"rms_norm_eps={c.rms_norm_eps}")
        need(c.rope_theta > 0, "rope_theta must be positive", f"rope_theta={c.rope_theta}")
        need(c.max_position_embeddings > 0, "max_position_embeddings must be positive", f"max_position_embeddings={c.max_position_embeddings}")
        need(c.hidden_act == "silu", "hidden_act must be silu", f"hidden_act={c.hidden_act}")
        if c.use_sliding_window:
            need(c.sliding_window is not None and c.sliding_window > 0, "use_sliding_window needs a positive sliding_window", f"sliding_window={c.sliding_window}")
            need(
                c.max_window_layers is not None and 0 <= c.max_window_layers <= c.num_hidden_layers,
                "max_window_layers must lie in [0, num_hidden_layers]",
                f"max_window_layers={c.max_window_layers}",
            )

    def window_of_layer(self, i: int) -> Optional[int]:
        """Layers from ``max_window_layers`` on attend to the last
        ``sliding_window`` keys when ``use_sliding_window`` is set; all other
        layers see every key.  The reference never reads these keys and every
        configuration it ships leaves the option off."""
        if self.use_sliding_window and i >= self.max_window_layers:
            return self.sliding_window
        return None


def read_config(obj: dict, origin: str) -> Qwen2Config:
    k = Keys(obj, origin)
    heads = k.integer("num_attention_heads")
    hidden = k.integer("hidden_size")
    if heads <= 0:
        raise AlofaError("parse", "num_attention_heads must be positive", f"num_attention_heads={heads} config={origin}")
    cfg = Qwen2Config(
        num_hidden_layers=k.integer("num_hidden_layers"),
        hidden_size=hidden,
        num_attention_heads=heads,
        num_key_value_heads=k.integer("num_key_value_heads"),
        # optional: hidden // heads when absent (qwen.mojo:943-949)
        head_dim=k.integer("head_dim", hidden // heads),
        intermediate_size=k.integer("intermediate_size"),
        vocab_size=k.integer("vocab_size"),
        rms_norm_eps=k.number("rms_norm_eps"),
        rope_theta=k.number("rope_theta"),
        tie_word_embeddings=k.boolean("tie_word_embeddings"),
        max_position_embeddings=k.integer("max_position_embeddings"),
        use_sliding_window=k.boolean("use_sliding_window", False),
        sliding_window=k.integer("sliding_window") if k.has("sliding_window") else None,
        max_window_layers=k.integer("max_window_layers") if k.has("max_window_layers") else None,
        hidden_act=k.string("hidden_act", "silu"),
    )
    cfg.validate(origin)
    return cfg


def to_json(cfg: Qwen2Config) -> dict:
    out = {
        "architectures": [NAME],
        "model_type": "qwen2",
        "hidden_act": cfg.hidden_act,
        "hidden_size": cfg.hidden_size,
        "intermediate_size": cfg.intermediate_size,
        "max_position_embeddings": cfg.max_position_embeddings,
        "num_attention_heads": cfg.num_attention_heads,
        "num_hidden_layers": cfg.num_hidden_layers,
        "num_key_value_heads": cfg.num_key_value_heads,
        "head_dim": cfg.head_dim,
        "rms_norm_eps": cfg.rms_norm_eps,
        "rope_theta": cfg.rope_theta,
        "tie_word_embeddings": cfg.tie_word_embeddings,
        "use_sliding_window": cfg.use_sliding_window,
        "vocab_size": cfg.vocab_size,
    }
    if cfg.sliding_window is not None:
        out["sliding_window"] = cfg.sliding_window
    if cfg.max_window_layers is not None:
        out["max_window_layers"] = cfg.max_window_layers
    return out


def build_spec(cfg: Qwen2Config) -> ModelSpec:
    """Tensor names are the checkpoint's own, read without renaming
    (qwen.mojo:9-13, 1168-1189)."""
    layers = []
    for i in range(cfg.num_hidden_layers):
        p = f"model.layers.{i}."
        rotary = PartSpec(
            "rotary_neox",
            {"head_dim": cfg.head_dim, "rotary_dim": cfg.head_dim, "theta": cfg.rope_theta, "max_position": cfg.max_position_embeddings},
        )
        mixer = PartSpec(
            "gqa_attention",
            {
                "hidden_size": cfg.hidden_size,
                "num_heads": cfg.num_attention_heads,
                "num_kv_heads": cfg.num_key_value_heads,
                "head_dim": cfg.head_dim,
                "qkv_bias": True,
                "out_bias": False,
                "window": cfg.window_of_layer(i),
                "position": rotary,
            },
            prefix=p + "self_attn.",
        )
        ffn = PartSpec(
            "gated_mlp",
            {"hidden_size": cfg.hidden_size, "intermediate_size": cfg.intermediate_size, "activation": cfg.hidden_act},
            prefix=p + "mlp.",
        )
        norm = {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}
        block = PartSpec(
            "prenorm_residual",
            {
                "mixer": mixer,
                "feed_forward": ffn,
                "mixer_norm": PartSpec("rmsnorm", dict(norm), prefix=p + "input_layernorm."),
                "feed_forward_norm": PartSpec("rmsnorm", dict(norm), prefix=p + "post_attention_layernorm."),
            },
            prefix=p,
        )
        layers.append(LayerSpec(block))
    spec = ModelSpec(
        architecture=NAME,
        hidden_size=cfg.hidden_size,
        vocab_size=cfg.vocab_size,
        max_position=cfg.max_position_embeddings,
        embedding=PartSpec("token_embedding", {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size}, prefix="model.embed_tokens."),
        layers=layers,
        run=[RunEntry(i, i) for i in range(cfg.num_hidden_layers)],
        final_norm=PartSpec("rmsnorm", {"size": cfg.hidden_size, "eps": cfg.rms_norm_eps}, prefix="model.norm."),
        # the head is lm_head.weight if the file has it, else the embedding
        # when tied (qwen.mojo:1077-1089)
        head=PartSpec(
            "linear_head",
            {"vocab_size": cfg.vocab_size, "hidden_size": cfg.hidden_size, "tied_to": "model.embed_tokens.weight" if cfg.tie_word_embeddings else None},
            prefix="lm_head.",
        ),
    )
    spec.validate()
    return spec


register_architecture(Architecture(NAME, read_config, build_spec, to_json), replace=True)
