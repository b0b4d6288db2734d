"""Plain, slow restatement of the Qwen2 decoder used as the oracle of every test.

Whole sequences, no cache, one function per part, NumPy float64 accumulation.
It shares no code with the product package: it has its own config reader, its
own safetensors reader and its own arithmetic.  Each function cites the
reference file and lines (paths inside the mojothon/alofa project) whose
formula it restates.

The reference's model code is Mojo and can be neither imported nor compiled on
a machine without the Mojo toolchain, so this file rests on the formulas; the
formulas themselves are anchored on the reference's Hugging Face capture of
layer 0 by `tests/golden/make_layer0_anchor.py`.
"""
from __future__ import annotations

import json
import math
import struct
from pathlib import Path

import numpy as np


# ----------------------------------------------------------------------------
# files
# ----------------------------------------------------------------------------
def read_config(folder) -> dict:
    """Flat scalar keys of config.json (src/alofa/model/arch/qwen.mojo:929-968)."""
    raw = json.loads((Path(folder) / "config.json").read_text())
    cfg = {
        "L": int(raw["num_hidden_layers"]),
        "H": int(raw["hidden_size"]),
        "nh": int(raw["num_attention_heads"]),
        "nkv": int(raw["num_key_value_heads"]),
        "I": int(raw["intermediate_size"]),
        "V": int(raw["vocab_size"]),
        "eps": float(raw["rms_norm_eps"]),
        "theta": float(raw["rope_theta"]),
        "tied": bool(raw["tie_word_embeddings"]),
    }
    # head_dim is optional: hidden // heads when absent (qwen.mojo:943-949)
    cfg["hd"] = int(raw.get("head_dim", cfg["H"] // cfg["nh"]))
    cfg["window"] = None
    cfg["first_window_layer"] = cfg["L"]
    if raw.get("use_sliding_window", False):
        cfg["window"] = int(raw["sliding_window"])
        cfg["first_window_layer"] = int(raw.get("max_window_layers", cfg["L"]))
    return cfg


def _bf16_to_f64(raw: np.ndarray) -> np.ndarray:
    """bf16 widening = the 16 bits shifted into the top of an fp32
    (src/alofa/model/safetensors.mojo:123-137)."""
    return (raw.astype(np.uint32) << 16).view(np.float32).astype(np.float64)


def read_safetensors(path) -> dict:
    """8-byte little-endian header length, JSON header, raw data
    (src/alofa/model/safetensors.mojo:147-303)."""
    blob = Path(path).read_bytes()
    (hlen,) = struct.unpack("<Q", blob[:8])
    header = json.loads(blob[8 : 8 + hlen])
    base = 8 + hlen
    out = {}
    for name, meta in header.items():
        if name == "__metadata__":
            continue
        lo, hi = meta["data_offsets"]
        buf = blob[base + lo : base + hi]
        shape = tuple(meta["shape"])
        if meta["dtype"] == "F32":
            arr = np.frombuffer(buf, dtype="<f4").astype(np.float64)
        elif meta["dtype"] == "BF16":
            arr = _bf16_to_f64(np.frombuffer(buf, dtype="<u2"))
        else:
            raise ValueError(f"plain reader: dtype {meta['dtype']} of {name}")
        out[name] = arr.reshape(shape)
    return out


# ----------------------------------------------------------------------------
# parts
# ----------------------------------------------------------------------------
def rmsnorm(x, w, eps):
    """y = x * (1/sqrt(mean(x^2) + eps)) * w per row; no bias, no mean
    subtraction, weight used as is (src/alofa/kernels/cpu/scalar.mojo:93-129)."""
    x = np.asarray(x, dtype=np.float64)
    scale = 1.0 / np.sqrt((x * x).mean(axis=-1, keepdims=True) + eps)
    return x * scale * np.asarray(w, dtype=np.float64)


def linear(x, w, b=None):
    """y = x @ W^T (+ b); W is [out, in] row-major; the accumulator starts at
    the bias (src/alofa/kernels/cpu/scalar.mojo:132-205)."""
    y = np.asarray(x, dtype=np.float64) @ np.asarray(w, dtype=np.float64).T
    if b is not None:
        y = y + np.asarray(b, dtype=np.float64)
    return y


def rope_table(positions, hd, theta):
    """cos/sin [n, hd/2]: inv = f32(1)/f32(theta^(2i/hd)) with the power in
    f64; angle = f32(p) * inv as an fp32 product; cos/sin taken in f64 and
    rounded to fp32 (src/alofa/model/arch/qwen.mojo:830-880)."""
    half = hd // 2
    i = np.arange(half, dtype=np.float64)
    inv = np.float32(1.0) / np.power(np.float64(theta), 2.0 * i / hd).astype(np.float32)
    pos = np.asarray(positions).astype(np.float32)
    angle = (pos[:, None] * inv[None, :]).astype(np.float32)
    cos = np.cos(angle.astype(np.float64)).astype(np.float32).astype(np.float64)
    sin = np.sin(angle.astype(np.float64)).astype(np.float32).astype(np.float64)
    return cos, sin


def rope(x, positions, n_heads, hd, theta):
    """NeoX (half-split) rotation per head: y[d] = a*cos - b*sin,
    y[d+half] = b*cos + a*sin with a=x[d], b=x[d+half]
    (src/alofa/kernels/cpu/scalar.mojo:283-344; per-row position
    src/alofa/kernels/cpu/segments.mojo:48-130)."""
    n = x.shape[0]
    half = hd // 2
    cos, sin = rope_table(positions, hd, theta)
    xh = np.asarray(x, dtype=np.float64).reshape(n, n_heads, hd)
    a, b = xh[..., :half], xh[..., half:]
    out = np.empty_like(xh)
    out[..., :half] = a * cos[:, None, :] - b * sin[:, None, :]
    out[..., half:] = b * cos[:, None, :] + a * sin[:, None, :]
    return out.reshape(n, n_heads * hd)


def attention(q, k, v, nh, nkv, hd, window=None):
    """Causal grouped-query attention over a whole sequence: query head h reads
    KV head h // (nh/nkv); keys 0..P visible to the query at position P (causal
    by loop bound); score = dot * (1/sqrt(hd)); softmax with the row maximum
    subtracted; normalisation after the weighted sum
    (src/alofa/kernels/cpu/scalar.mojo:392-470).  `window`, when given, keeps
    only the last `window` keys (P-window < j <= P); the reference has no such
    option and every published configuration leaves it off."""
    n = q.shape[0]
    g = nh // nkv
    scale = 1.0 / math.sqrt(hd)
    qh = np.asarray(q, dtype=np.float64).reshape(n, nh, hd)
    kh = np.asarray(k, dtype=np.float64).reshape(n, nkv, hd)
    vh = np.asarray(v, dtype=np.float64).reshape(n, nkv, hd)
    out = np.zeros((n, nh, hd), dtype=np.float64)
    for h in range(nh):
        kvh = h // g
        s = (qh[:, h, :] @ kh[:, kvh, :].T) * scale  # [n, n]
        j = np.arange(n)
        visible = j[None, :] <= j[:, None]
        if window is not None:
            visible &= j[None, :] > (j[:, None] - window)
        s = np.where(visible, s, -np.inf)
        m = s.max(axis=1, keepdims=True)
        e = np.exp(s - m)
        z = e.sum(axis=1, keepdims=True)
        out[:, h, :] = (e @ vh[:, kvh, :]) / z
    return out.reshape(n, nh * hd)


def silu(z):
    """silu(z) = z / (1 + exp(-z)) (src/alofa/kernels/cpu/scalar.mojo:208-217)."""
    z = np.asarray(z, dtype=np.float64)
    return z / (1.0 + np.exp(-z))


def swiglu_mlp(x, w_gate, w_up, w_down):
    """down(silu(gate(x)) * up(x)), no biases
    (src/alofa/model/arch/qwen.mojo:1481-1510; scalar.mojo:219-231)."""
    return linear(silu(linear(x, w_gate)) * linear(x, w_up), w_down)


def embed(ids, table):
    """h[r] = table[id_r]; ids outside [0, V) are refused
    (src/alofa/model/arch/qwen.mojo:1391-1413)."""
    ids = np.asarray(ids)
    if ids.min() < 0 or ids.max() >= table.shape[0]:
        raise ValueError("token id outside the vocabulary")
    return np.asarray(table, dtype=np.float64)[ids]


def decoder_layer(h, positions, wts, prefix, cfg, window=None):
    """Pre-norm residual layer: h += Attn(RMS1(h)); h += MLP(RMS2(h))
    (src/alofa/model/arch/qwen.mojo:1418-1510)."""
    p = prefix
    x = rmsnorm(h, wts[p + "input_layernorm.weight"], cfg["eps"])
    q = linear(x, wts[p + "self_attn.q_proj.weight"], wts[p + "self_attn.q_proj.bias"])
    k = linear(x, wts[p + "self_attn.k_proj.weight"], wts[p + "self_attn.k_proj.bias"])
    v = linear(x, wts[p + "self_attn.v_proj.weight"], wts[p + "self_attn.v_proj.bias"])
    q = rope(q, positions, cfg["nh"], cfg["hd"], cfg["theta"])
    k = rope(k, positions, cfg["nkv"], cfg["hd"], cfg["theta"])
    a = attention(q, k, v, cfg["nh"], cfg["nkv"], cfg["hd"], window)
    h = h + linear(a, wts[p + "self_attn.o_proj.weight"])
    x = rmsnorm(h, wts[p + "post_attention_layernorm.weight"], cfg["eps"])
    h = h + swiglu_mlp(
        x,
        wts[p + "mlp.gate_proj.weight"],
        wts[p + "mlp.up_proj.weight"],
        wts[p + "mlp.down_proj.weight"],
    )
    return h


def head_weight(wts, cfg):
    """lm_head.weight if the file has it, else the embedding when tied, else an
    error (src/alofa/model/arch/qwen.mojo:1077-1089)."""
    if "lm_head.weight" in wts:
        return wts["lm_head.weight"]
    if cfg["tied"]:
        return wts["model.embed_tokens.weight"]
    raise ValueError("no lm_head.weight and embeddings are not tied")


def forward(ids, wts, cfg, rows=None):
    """Logits [n, V] (float64) at every position of one whole sequence, or at
    the positions ``rows`` only
    (src/alofa/model/arch/qwen.mojo:1362-1525; the reference projects the last
    row only, the same final norm and head are applied to every row here)."""
    n = len(ids)
    positions = np.arange(n)
    h = embed(ids, wts["model.embed_tokens.weight"])
    for i in range(cfg["L"]):
        window = cfg["window"] if i >= cfg["first_window_layer"] else None
        h = decoder_layer(h, positions, wts, f"model.layers.{i}.", cfg, window)
    if rows is not None:
        h = h[np.asarray(rows, dtype=np.int64)]
    x = rmsnorm(h, wts["model.norm.weight"], cfg["eps"])
    return linear(x, head_weight(wts, cfg))


def load(folder):
    """(weights as float64 arrays by name, config dict) of a model folder."""
    cfg = read_config(folder)
    wts = read_safetensors(Path(folder) / "model.safetensors")
    return wts, cfg


def argmax(row) -> int:
    """Largest logit, ties to the lowest index
    (src/alofa/model/arch/qwen.mojo:1527-1541)."""
    return int(np.argmax(np.asarray(row)))


def greedy(ids, n_new, wts, cfg):
    """Teacher-free greedy continuation by whole-sequence recomputation."""
    seq = list(ids)
    out = []
    for _ in range(n_new):
        tok = argmax(forward(seq, wts, cfg)[-1])
        out.append(tok)
        seq.append(tok)
    return out


# ----------------------------------------------------------------------------
# sampling
# ----------------------------------------------------------------------------
class SplitMix64:
    """SplitMix64; next_uniform = top 53 bits * 2^-53
    (src/alofa/core/rng.mojo:37-78)."""

    MASK = (1 << 64) - 1

    def __init__(self, seed: int):
        self.state = seed & self.MASK

    def next_u64(self) -> int:
        self.state = (self.state + 0x9E3779B97F4A7C15) & self.MASK
        z = self.state
        z = ((z ^ (z >> 30)) * 0xBF58476D1CE4E5B9) & self.MASK
        z = ((z ^ (z >> 27)) * 0x94D049BB133111EB) & self.MASK
        return z ^ (z >> 31)

    def next_uniform(self) -> float:
        return (self.next_u64() >> 11) * 1.1102230246251565e-16


def sample_distribution(
    logits,
    history=(),
    temperature=1.0,
    top_k=0,
    top_p=1.0,
    min_p=0.0,
    repetition_penalty=1.0,
    frequency_penalty=0.0,
    presence_penalty=0.0,
    min_tokens_to_keep=1,
    logit_bias=(),
):
    """Probability vector after the reference's chain: bias, repetition,
    frequency/presence, temperature, top-k, top-p, min-p, softmax
    (src/alofa/runtime/sampler.mojo:308-477)."""
    x = np.asarray(logits, dtype=np.float64).copy()
    n = x.shape[0]
    floor = -1.0e300
    for idx, val in logit_bias:
        x[idx] += val
    counts = {}
    for t in history:
        counts[t] = counts.get(t, 0) + 1
    if repetition_penalty != 1.0:
        for t in counts:
            x[t] = x[t] * repetition_penalty if x[t] < 0 else x[t] / repetition_penalty
    if frequency_penalty != 0.0 or presence_penalty != 0.0:
        for t, c in counts.items():
            x[t] -= frequency_penalty * c
            x[t] -= presence_penalty
    if temperature == 0.0:
        p = np.zeros(n)
        p[int(np.argmax(x))] = 1.0
        return p
    if temperature != 1.0:
        x = x / temperature
    keep = max(1, min_tokens_to_keep)

    def softmax(v):
        e = np.exp(v - v.max())
        e[v <= floor] = 0.0
        return e / e.sum()

    order = np.argsort(-x, kind="stable")
    if 0 < top_k < n:
        kth = x[order[top_k - 1]]
        x[x < kth] = floor
    if top_p < 1.0:
        w = softmax(x)
        acc = np.cumsum(w[order])
        taken = int(np.argmax(acc >= top_p)) + 1 if (acc >= top_p).any() else n
        taken = max(taken, keep)
        x[order[taken:]] = floor
    if min_p > 0.0:
        w = softmax(x)
        drop = w < min_p * w.max()
        drop[order[:keep]] = False
        x[drop] = floor
    return softmax(x)


def pick_from(weights, u: float) -> int:
    """Inverse CDF: first index whose running sum exceeds u
    (src/alofa/runtime/sampler.mojo:152-164)."""
    acc = 0.0
    for i, w in enumerate(weights):
        acc += float(w)
        if u < acc:
            return i
    return len(weights) - 1
