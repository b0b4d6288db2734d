"""Choice of the tensor-core matrix product for bfloat16 operands.

``plan(linear)`` returns a callable ``(out, x, defer) -> True | Partial | False``
that runs the tcgen05 kernel, or returns False, having launched nothing, when
the call's sizes are ones that kernel refuses (the caller then uses the generic
kernel), or None when the weight can never go that way (depth not a multiple
of 8: a TMA row must start on a 16-byte boundary).

Tokens per CTA and the number of k-splits are chosen from the token count and
the weight's shape so that even a handful of decode tokens pulls the weight
through most of the 148 SMs; the split partial sums are added in a fixed
order, so a given (tokens, weight) pair always sums the same way."""
from __future__ import annotations

import torch

from ..csrc import ops
from ..errors import AlofaError

SMS = 148  # streaming multiprocessors the grids are sized for: a B200's, replaced by the device's own count at first use
K_SLICE = 64
_asked_device = False


def _sms_of_device(device) -> None:
    """The tile and split choices below fill the GPU once: they go by the
    number of SMs the device reports."""
    global SMS, _asked_device
    if not _asked_device and device.type == "cuda":
        _asked_device = True
        SMS = torch.cuda.get_device_properties(device).multi_processor_count


def _tile(tokens: int, features: int, gated: bool) -> int:
    """The kernel's tile argument.  Positive: weights on the M side of the MMA
    with that many tokens per CTA (decode: few tokens, weights streamed).
    Negative: tokens on the M side (128 per CTA) with that many weight rows
    per MMA (prompt portions: an MMA of M = 128 costs the same for any N up to
    256, so wide feature tiles are what pays)."""
    for bn in (16, 32, 64):
        if tokens <= bn:
            # a very tall weight (an output head) fills the GPU several times over
            # either way; wide tiles with the tokens on the M side stream it faster
            if not gated and -(-features // 128) > 4 * SMS:
                return -256
            return bn
    if gated:
        return -256  # 128 gate rows and their 128 up rows
    # narrow outputs: 128-wide tiles keep more SMs busy
    return -128 if -(-features // 256) * -(-tokens // 128) < SMS else -256


def _ctas(tokens: int, features: int, tile: int, gated: bool) -> int:
    if tile > 0:
        return -(-features // 128) * -(-tokens // tile)
    per_cta = -tile // 2 if gated else -tile
    return -(-features // per_cta) * -(-tokens // 128)


def _splits(ctas: int, depth: int, deferrable: bool = False) -> int:
    slices = -(-depth // K_SLICE)
    if slices < 2:
        return 1
    if ctas >= SMS // 2:
        # a deep product that does not fill the GPU once: two halves of the depth
        # side by side, when the consumer adds the halves up for free
        return 2 if deferrable and ctas < SMS and slices >= 32 else 1
    return max(1, min(slices, SMS // ctas))


def plan(linear):
    from .linear import Partial

    w = linear.weight
    depth = linear.in_features
    if depth % 8 or w.data_ptr() % 16:
        return None
    _sms_of_device(w.device)
    gated = linear.epi == ops.EPI_GATED
    n_acc = 2 if gated else 1

    def run(out, x, defer: bool = False, buf=None, acc=None):
        from .linear import ACCUMULATED

        tokens = x.shape[0]
        if tokens == 0:
            return True
        bn = _tile(tokens, linear.out_features, gated)
        lazy = None if isinstance(x, torch.Tensor) else x
        if lazy is not None:
            x = None
        splits = ops.gemm_tc_splits(depth, _splits(_ctas(tokens, linear.out_features, bn, gated), depth, defer and n_acc == 1))
        computed = None
        if lazy is not None:
            # Rows still to be made.  The weights-on-M kernel makes them as it loads, a k-slice at a
            # time and each a trip to L2: worth it while a CTA has a few slices, else they are made first.
            per_cta = -(-(-(-depth // K_SLICE)) // splits)
            kind = getattr(lazy, "kind", "merged")
            if kind == "merged" and bn == 16 and linear.epi == ops.EPI_RESIDUAL and per_cta <= 2 and lazy.fits_kernel():
                computed = lazy.computed()
            elif kind == "normed" and bn == 16 and gated and splits <= 8 and per_cta <= 6 and lazy.fits_kernel():
                computed = lazy.computed()  # the norm folded into a gated product whose splits are one cluster
            else:
                x = lazy.rows()
        if x is not None and (x.data_ptr() % 16 or not x.is_contiguous()):
            return False
        normed = computed is not None and computed[0] == ops.B_NORMED
        partial = None
        if splits > 1 and acc is None and not normed:
            shape = (splits * n_acc, tokens, linear.out_features)
            partial = buf(shape, torch.float32) if buf is not None else torch.empty(shape, dtype=torch.float32, device=w.device)
        deferred = defer and splits > 1 and n_acc == 1 and acc is None
        dst = partial[0] if deferred else out  # a deferred product writes partial sums only
        if not ops.gemm_tc(dst, x, w, linear.bias, linear.epi, bn, splits, partial, reduce=not deferred, computed=computed, acc=acc):
            if normed:
                lazy.undo()
                return run(out, lazy.rows(), defer, buf)
            if computed is not None or acc is not None:
                raise AlofaError("state", "the tensor-core product refused an operand it had accepted")
            return False
        if normed:
            lazy.done(computed)
        if acc is not None:
            return ACCUMULATED
        return Partial(partial, splits, linear.bias) if deferred else True

    run.weights_on_m = lambda tokens: _tile(tokens, linear.out_features, gated) > 0
    return run
