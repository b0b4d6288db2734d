"""From a step's logits to one token per wanted row, on the device.

Rows whose settings are temperature only go through the fused argmax /
softmax-draw kernel with the temperatures and uniform numbers that came up
with the step's metadata.  If any row uses the rest of the chain (bias,
penalties, top-k, top-p, min-p) the whole batch goes through the chain kernel,
whose per-row settings and token histories are uploaded here.  Sampling sits
outside the step function, as in the reference (``decide`` runs the forward,
the caller picks, ``settle`` consumes: src/alofa/engine/core.mojo:584-674)."""
from __future__ import annotations

import numpy as np
import torch

from ..csrc import ops


def chain_inputs(rows: list, device) -> dict:
    """Device arrays for the chain kernel.  ``rows``: per row a tuple
    (SamplingParams, uniform, history token list)."""
    n = len(rows)
    fparams = np.zeros((n, 8), dtype=np.float32)
    iparams = np.zeros((n, 4), dtype=np.int32)
    bias_start, bias_index, bias_value = [0], [], []
    hist_start, hist_token, hist_count = [0], [], []
    for r, (p, u, history) in enumerate(rows):
        fparams[r, :7] = (p.temperature, p.top_p, p.min_p, p.repetition_penalty, p.frequency_penalty, p.presence_penalty, u)
        iparams[r, :2] = (p.top_k, p.min_tokens_to_keep)
        for idx, val in p.logit_bias.items():
            bias_index.append(int(idx))
            bias_value.append(float(val))
        bias_start.append(len(bias_index))
        if p.repetition_penalty != 1.0 or p.frequency_penalty != 0.0 or p.presence_penalty != 0.0:
            toks, counts = np.unique(np.asarray(history, dtype=np.int64), return_counts=True)
            hist_token.extend(int(t) for t in toks)
            hist_count.extend(int(c) for c in counts)
        hist_start.append(len(hist_token))

    def dev(values, dtype):
        arr = np.asarray(values if len(values) else [0], dtype=dtype)
        return torch.from_numpy(arr).to(device)

    return {
        "fparams": torch.from_numpy(fparams).to(device), "iparams": torch.from_numpy(iparams).to(device),
        "bias_start": dev(bias_start, np.int32), "bias_index": dev(bias_index, np.int32), "bias_value": dev(bias_value, np.float32),
        "hist_start": dev(hist_start, np.int32), "hist_token": dev(hist_token, np.int32), "hist_count": dev(hist_count, np.int32),
    }


def sample_chain_rows(logits: torch.Tensor, rows: list) -> torch.Tensor:
    """tokens int32 [n] on the device for ``rows`` of (params, uniform, history)."""
    tokens = torch.empty(logits.shape[0], dtype=torch.int32, device=logits.device)
    work = torch.empty_like(logits)
    ops.sample_chain(tokens, logits, work, **chain_inputs(rows, logits.device))
    return tokens


def sample_rows(ctx, logits: torch.Tensor, owners: list) -> torch.Tensor:
    """One token per wanted row of a step through the whole chain;
    ``owners`` are the engine's requests in row order (``params``, ``prompt``,
    ``output``).  Rows shaped by temperature alone are served by the step
    itself (StepRunner.forward_sampled)."""
    uniform = ctx.host_field("uniform").view(np.float32)
    # history for the penalties = prompt + generated so far (src/alofa/cli.mojo:475-492)
    rows = [(req.params, float(uniform[i]), req.prompt + req.output) for i, req in enumerate(owners)]
    return sample_chain_rows(logits, rows)
