"""Choice of the tensor-core matrix product for bfloat16 operands.

``plan(linear)`` returns a callable ``(out, x) -> bool`` that runs the
tcgen05 kernel and returns True, or returns False, having launched nothing,
when the call's sizes are ones that kernel refuses (the caller then uses the
generic kernel), or None when the weight can never go that way (depth not a
multiple of 8: a TMA row must start on a 16-byte boundary).

Tokens per CTA and the number of k-splits are chosen from the token count and
the weight's shape so that even a handful of decode tokens pulls the weight
through most of the 148 SMs; the split partial sums are added in a fixed
order, so a given (tokens, weight) pair always sums the same way."""
from __future__ import annotations

import torch

from ..csrc import ops

SMS = 148
K_SLICE = 64


def _tokens_per_cta(tokens: int, feature_tiles: int) -> int:
    for bn in (16, 32, 64, 128):
        if tokens <= bn:
            return bn
    # prompts: smaller token tiles while the grid would not fill the GPU twice over
    return 128 if feature_tiles * -(-tokens // 256) < 2 * SMS else 256


def _splits(tokens: int, feature_tiles: int, bn: int, depth: int) -> int:
    ctas = feature_tiles * -(-tokens // bn)
    slices = -(-depth // K_SLICE)
    if ctas >= SMS // 2 or slices < 2:
        return 1
    return max(1, min(slices, SMS // ctas))


def plan(linear):
    w = linear.weight
    depth = linear.in_features
    if depth % 8 or w.data_ptr() % 16:
        return None
    feature_tiles = -(-linear.out_features // 128)
    n_acc = 2 if linear.epi == ops.EPI_GATED else 1

    def run(out: torch.Tensor, x: torch.Tensor) -> bool:
        tokens = x.shape[0]
        if tokens == 0:
            return True
        if x.data_ptr() % 16 or not x.is_contiguous():
            return False
        bn = _tokens_per_cta(tokens, feature_tiles)
        splits = ops.gemm_tc_splits(depth, _splits(tokens, feature_tiles, bn, depth))
        partial = None
        if splits > 1:
            partial = torch.empty(splits * n_acc * tokens * linear.out_features, dtype=torch.float32, device=x.device)
        return ops.gemm_tc(out, x, w, linear.bias, linear.epi, bn, splits, partial)

    return run
