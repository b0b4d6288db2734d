"""Python face of the CUDA kernels.

Each function checks what the kernel cannot check for itself (device, dtype,
contiguity, matching sizes), then launches on the current CUDA stream through
the library's C entry point.  There is no fallback of any kind: tensors that
are not on a CUDA device are refused, and a library that cannot be built or
loaded raises when it is first needed."""
from __future__ import annotations

import ctypes

import torch

from ..errors import AlofaError
from .build import load_library

EPI_STORE, EPI_RESIDUAL, EPI_GATED = 0, 1, 2

_P, _I, _F = ctypes.c_void_p, ctypes.c_int, ctypes.c_float
_libs: dict = {}
_launches = 0  # kernels launched through this module (graph replays add their kernels)


def launch_count() -> int:
    """How many of this package's kernels have been launched so far."""
    return _launches


def count_launches(n: int) -> None:
    global _launches
    _launches += n


def _generic():
    lib = _libs.get("generic")
    if lib is None:
        lib = load_library("alofa_generic", ["kernels/generic.cu"])
        sigs = {
            "alofa_embed_gather": [_P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P],
            "alofa_rmsnorm": [_P, _P, _P, _P, _I, _I, _F, _I, _P],
            "alofa_gemm_generic": [_P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
            "alofa_rope_store": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _P],
            "alofa_paged_attention_generic": [_P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _F, _I, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["generic"] = lib
    return lib


def _sampling():
    lib = _libs.get("sampling")
    if lib is None:
        lib = load_library("alofa_sampling", ["kernels/sampling.cu"])
        sigs = {
            "alofa_sample": [_P, _P, _P, _P, _I, _I, _P, _I, _P],
            "alofa_sample_chain": [_P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _P, _P, _P],
        }
        for name, args in sigs.items():
            fn = getattr(lib, name)
            fn.restype = _I
            fn.argtypes = args
        _libs["sampling"] = lib
    return lib


def _gemm_tc():
    lib = _libs.get("gemm_tc")
    if lib is None:
        lib = load_library("alofa_gemm_tc", ["kernels/gemm_tc.cu"])
        lib.alofa_gemm_tc.restype = _I
        lib.alofa_gemm_tc.argtypes = [_P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _P, _I, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _F, _P, _P, _P]
        lib.alofa_splitk_reduce.restype = _I
        lib.alofa_splitk_reduce.argtypes = [_P, _P, _P, _I, _I, _I, _I, _I, _P]
        lib.alofa_gemm_tc_reduces_in_cluster.restype = _I
        lib.alofa_gemm_tc_reduces_in_cluster.argtypes = [_I, _I, _I]
        lib.alofa_gemm_tc_rope.restype = _I
        lib.alofa_gemm_tc_rope.argtypes = [_P, _P, _P, _I, _I, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _P, _P, _P, _P, _F, _P, _P, _P]
        lib.alofa_gemm_tc_rope_resident_clusters.restype = _I
        lib.alofa_gemm_tc_rope_resident_clusters.argtypes = [_I, _I]
        lib.alofa_gemm_tc_splits.restype = _I
        lib.alofa_gemm_tc_splits.argtypes = [_I, _I]
        _libs["gemm_tc"] = lib
    return lib


def _attention(head_dim: int):
    key = f"attention_hd{head_dim}"
    lib = _libs.get(key)
    if lib is None:
        lib = load_library(f"alofa_attention_hd{head_dim}", ["kernels/attention_bf16.cu"], defines={"HEAD_DIM": head_dim})
        lib.alofa_attention_bf16.restype = _I
        lib.alofa_attention_bf16.argtypes = [_P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _I, _I, _F, _I, _I, _P, _P, _I, ctypes.c_longlong, _P, _I, _P]
        lib.alofa_attention_combine.restype = _I
        lib.alofa_attention_combine.argtypes = [_P, _P, _P, _P, _I, _I, _I, _I, _P]
        lib.alofa_attention_decode_wide_warps.restype = _I
        lib.alofa_attention_decode_wide_warps.argtypes = []
        lib.alofa_attention_decode_slots.restype = _I
        lib.alofa_attention_decode_slots.argtypes = [_I, _I]
        _libs[key] = lib
    return lib


_decode_slots = {}


def attention_decode_wide_warps(head_dim: int) -> int:
    """Warps of the decode attention kernel's wide form at this head size (one
    CTA per SM; its splits are multiples of 64 keys a warp), 0 when it has none."""
    return _attention(head_dim).alofa_attention_decode_wide_warps()


def attention_decode_slots(head_dim: int, page_size: int, warps: int = 4) -> int:
    """How many CTAs of the decode attention kernel with ``warps`` warps (4, or
    the wide form's) the device holds at a time, 0 when that kernel is not
    built for this head size and kind of page (asked once each)."""
    key = (head_dim, page_size % 64 == 0, warps)
    if key not in _decode_slots:
        _decode_slots[key] = max(0, _attention(head_dim).alofa_attention_decode_slots(page_size, warps))
    return _decode_slots[key]


def attention_bf16_supported(head_dim: int) -> bool:
    """Head sizes the bfloat16 attention kernel is built for."""
    return head_dim % 16 == 0 and 16 <= head_dim <= 128


def _elementwise():
    lib = _libs.get("elementwise")
    if lib is None:
        lib = load_library("alofa_elementwise_bf16", ["kernels/elementwise_bf16.cu"])
        lib.alofa_norm_fused.restype = _I
        lib.alofa_norm_fused.argtypes = [_P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _F, _I, _P, _P, _P, _P]
        lib.alofa_stream_settle.restype = _I
        lib.alofa_stream_settle.argtypes = [_P, _P, _P, _P, _I, _P]
        lib.alofa_rope_store_fused.restype = _I
        lib.alofa_rope_store_fused.argtypes = [_P, _P, _P, _P, _P, _P, _P, _P, _P, _I, _I, _I, _I, _I, _I, _P]
        _libs["elementwise"] = lib
    return lib


_bound_stream = None  # the stream handle of the step in progress, looked up once per step


def _stream() -> int:
    return _bound_stream if _bound_stream is not None else torch.cuda.current_stream().cuda_stream


class bound_stream:
    """Within the block, every launch of this module goes to the stream that is
    current on entry, without asking torch for it at each launch (the lookup
    costs as much as a launch).  The caller must not switch streams inside."""

    def __enter__(self):
        global _bound_stream
        self._before = _bound_stream
        _bound_stream = torch.cuda.current_stream().cuda_stream
        return self

    def __exit__(self, *exc):
        global _bound_stream
        _bound_stream = self._before
        return False


def _dev(t: torch.Tensor, name: str, dtype=None) -> int:
    if not t.is_cuda:
        raise AlofaError("unsupported", "kernels run on CUDA tensors only", f"{name} is on {t.device}")
    if not t.is_contiguous():
        raise AlofaError("invalid_argument", "kernel operand must be contiguous", name)
    if dtype is not None and t.dtype != dtype:
        raise AlofaError("invalid_argument", "kernel operand has the wrong dtype", f"{name} is {t.dtype}, want {dtype}")
    return t.data_ptr()


def _is_bf16(t: torch.Tensor, name: str) -> int:
    if t.dtype == torch.bfloat16:
        return 1
    if t.dtype == torch.float32:
        return 0
    raise AlofaError("unsupported", "kernel operand must be float32 or bfloat16", f"{name} is {t.dtype}")


def _done(rc: int, what: str, detail: str = "") -> None:
    global _launches
    if rc == 0:
        _launches += 1
        return
    if rc == 1:
        raise AlofaError("unsupported", f"{what}: the kernel does not take these sizes", detail)
    raise AlofaError("state", f"{what}: the CUDA runtime refused the launch", detail + " " + str(torch.cuda.get_device_name()))


def embed_gather(out, table, ids, status=None, src=None, fed=None) -> None:
    """out[t] = table[ids[t]] widened to fp32; out [T, H] fp32.  With ``src``
    and ``fed`` (int32 on the device) token t is ``fed[src[t]]`` where
    ``src[t] >= 0``: a token the step before sampled, never seen by the host."""
    n, hidden = out.shape
    _done(
        _generic().alofa_embed_gather(
            _dev(out, "out", torch.float32), _dev(table, "table"), _dev(ids, "ids", torch.int32),
            _dev(src, "src", torch.int32) if src is not None else None, _dev(fed, "fed", torch.int32) if src is not None else None,
            n, hidden, table.shape[0],
            _is_bf16(table, "table"), _dev(status, "status", torch.int32) if status is not None else None, _stream(),
        ),
        "embed_gather",
    )


def rmsnorm(out, x, weight, eps: float, rows=None) -> None:
    """out[r] = rmsnorm(x[rows[r] or r]) * weight; x fp32, weight fp32."""
    n, hidden = out.shape
    if x.shape[-1] != hidden or weight.shape[0] != hidden:
        raise AlofaError("invalid_argument", "rmsnorm sizes disagree", f"out={tuple(out.shape)} x={tuple(x.shape)} w={tuple(weight.shape)}")
    _done(
        _generic().alofa_rmsnorm(
            _dev(out, "out"), _dev(x, "x", torch.float32), _dev(weight, "weight", torch.float32),
            _dev(rows, "rows", torch.int32) if rows is not None else None, n, hidden, float(eps), _is_bf16(out, "out"), _stream(),
        ),
        "rmsnorm",
    )


def gemm_generic(out, x, w, bias, epi: int) -> None:
    """out = x @ w.T (+bias) with the epilogue ``epi``; any sizes."""
    m, k = x.shape
    n = out.shape[1]
    rows_w = 2 * n if epi == EPI_GATED else n
    if w.shape != (rows_w, k) or out.shape[0] != m or (bias is not None and bias.shape[0] != rows_w):
        raise AlofaError("invalid_argument", "gemm sizes disagree", f"out={tuple(out.shape)} x={tuple(x.shape)} w={tuple(w.shape)} epi={epi}")
    _done(
        _generic().alofa_gemm_generic(
            _dev(out, "out"), _dev(x, "x"), _dev(w, "w"), _dev(bias, "bias", torch.float32) if bias is not None else None,
            m, n, k, epi, _is_bf16(x, "x"), _is_bf16(w, "w"), _is_bf16(out, "out"), _stream(),
        ),
        "gemm_generic", f"M={m} N={n} K={k} epi={epi}",
    )


def rope_store(q_out, k_cache, v_cache, qkv, cos_sin, positions, slot_map, nh, nkv, hd, rot, write_cache=True) -> None:
    """Rotate q and k, write k and v into the cache slots of ``slot_map``."""
    n = qkv.shape[0]
    if qkv.shape[1] != (nh + 2 * nkv) * hd or q_out.shape != (n, nh * hd):
        raise AlofaError("invalid_argument", "rope_store sizes disagree", f"qkv={tuple(qkv.shape)} q_out={tuple(q_out.shape)}")
    if rot and cos_sin.shape[1] * 2 != rot:
        raise AlofaError("invalid_argument", "rotary table does not match rotary_dim", f"table={tuple(cos_sin.shape)} rot={rot}")
    dt = qkv.dtype
    _done(
        _generic().alofa_rope_store(
            _dev(q_out, "q_out", dt), _dev(k_cache, "k_cache", dt) if write_cache else None,
            _dev(v_cache, "v_cache", dt) if write_cache else None, _dev(qkv, "qkv"),
            _dev(cos_sin, "cos_sin", torch.float32) if rot else None, _dev(positions, "positions", torch.int32),
            _dev(slot_map, "slot_map", torch.int32) if write_cache else None, n, nh, nkv, hd, rot, 1 if write_cache else 0,
            _is_bf16(qkv, "qkv"), _stream(),
        ),
        "rope_store", f"hd={hd} rot={rot}",
    )


def paged_attention_generic(out, q, k_cache, v_cache, positions, seq_of_token, block_table, page_size, nh, nkv, hd, window, scale) -> None:
    """Causal GQA over the paged cache, any head size up to 256."""
    n = q.shape[0]
    dt = q.dtype
    _done(
        _generic().alofa_paged_attention_generic(
            _dev(out, "out", dt), _dev(q, "q"), _dev(k_cache, "k_cache", dt), _dev(v_cache, "v_cache", dt),
            _dev(positions, "positions", torch.int32), _dev(seq_of_token, "seq_of_token", torch.int32),
            _dev(block_table, "block_table", torch.int32), block_table.shape[1], page_size, n, nh, nkv, hd,
            int(window or 0), float(scale), _is_bf16(q, "q"), _stream(),
        ),
        "paged_attention_generic", f"hd={hd} nh={nh} nkv={nkv}",
    )


ARGMAX_PARTS = 32


def sample(tokens, logits, temperature, uniform, scratch=None, any_hot: bool = True) -> None:
    """tokens[r] = argmax (temperature 0) or inverse-CDF draw of softmax(x/T).
    With ``scratch`` (fp32, 2 * rows * ARGMAX_PARTS words) greedy rows are found
    in two stages over many blocks; ``any_hot`` False promises that no row has a
    positive temperature, so the draw kernel is not launched at all."""
    n, vocab = logits.shape
    if scratch is not None and scratch.numel() < 2 * n * ARGMAX_PARTS:
        raise AlofaError("invalid_argument", "sample scratch is too small", f"have={scratch.numel()} need={2 * n * ARGMAX_PARTS}")
    _done(
        _sampling().alofa_sample(
            _dev(tokens, "tokens", torch.int32), _dev(logits, "logits", torch.float32),
            _dev(temperature, "temperature", torch.float32) if temperature is not None else None,
            _dev(uniform, "uniform", torch.float32) if uniform is not None else None, n, vocab,
            _dev(scratch, "scratch", torch.float32) if scratch is not None else None, 1 if any_hot else 0, _stream(),
        ),
        "sample",
    )
    if scratch is not None:
        count_launches(2 if any_hot else 1)


def sample_chain(tokens, logits, work, fparams, iparams, bias_start, bias_index, bias_value, hist_start, hist_token, hist_count) -> None:
    """The whole sampling chain per row (bias, penalties, temperature, top-k,
    top-p, min-p, draw); ``work`` is fp32 scratch of the logits' shape."""
    n, vocab = logits.shape
    if work.shape != logits.shape or fparams.shape != (n, 8) or iparams.shape != (n, 4):
        raise AlofaError("invalid_argument", "sample_chain sizes disagree", f"logits={tuple(logits.shape)} work={tuple(work.shape)}")
    f32, i32 = torch.float32, torch.int32
    _done(
        _sampling().alofa_sample_chain(
            _dev(tokens, "tokens", i32), _dev(logits, "logits", f32), _dev(work, "work", f32), n, vocab,
            _dev(fparams, "fparams", f32), _dev(iparams, "iparams", i32), _dev(bias_start, "bias_start", i32),
            _dev(bias_index, "bias_index", i32), _dev(bias_value, "bias_value", f32), _dev(hist_start, "hist_start", i32),
            _dev(hist_token, "hist_token", i32), _dev(hist_count, "hist_count", i32), _stream(),
        ),
        "sample_chain", f"vocab={vocab}",
    )


_rope_clusters = {}


def gemm_tc_rope_splits(m_tiles: int, normed: bool, most: int = 8) -> int:
    """The largest depth split (a cluster of that many CTAs per 128-row tile)
    of the q/k/v kernel for which all ``m_tiles`` clusters are resident
    together: a GPC holds whole clusters only, so the answer comes from the
    runtime's occupancy of clusters, asked once per size."""
    for splits in range(most, 1, -1):
        key = (splits, bool(normed))
        if key not in _rope_clusters:
            _rope_clusters[key] = _gemm_tc().alofa_gemm_tc_rope_resident_clusters(splits, 1 if normed else 0)
        if _rope_clusters[key] >= m_tiles:
            return splits
    return 1


def gemm_tc_splits(k: int, splits: int) -> int:
    """The number of k-splits gemm_tc really uses for depth ``k``."""
    return _gemm_tc().alofa_gemm_tc_splits(k, splits)


B_ROWS, B_MERGED_SPLITS, B_NORMED = 0, 1, 2


def gemm_tc(out, x, w, bias, epi: int, bn: int, splits: int = 1, partial=None, status=None, reduce: bool = True, computed=None, acc=None) -> bool:
    """Tensor-core product ``out = x @ w.T`` (bf16 operands, fp32 sums) with
    the epilogue fused.  Returns False, having launched nothing, when the
    kernel does not take these sizes (depth not a multiple of 8, unaligned).

    ``computed`` (residual products with ``bn`` = 16 only) replaces ``x`` by
    rows the kernel makes as it goes: ``(B_MERGED_SPLITS, partial_o,
    partial_ml, positions, heads, head_dim, window, split_keys)``, the
    attention output of decode tokens whose key splits are not merged yet; or,
    for gated products, ``(B_NORMED, base, acc or None, gamma, eps, new_base,
    zero or None)``: the RMSNorm of the residual stream ``base + acc``, which
    is also written to ``new_base`` while ``zero`` is cleared.

    ``acc`` (residual products, weights on M): the sums are added into this
    int64 accumulator ``[tokens, features]`` (units of 2^-32) with atomic adds
    instead of into ``out``; nothing else is written."""
    n = out.shape[1]
    rows_w = 2 * n if epi == EPI_GATED else n
    k = w.shape[1]
    m = out.shape[0]
    if w.shape[0] != rows_w or (x is not None and tuple(x.shape) != (m, k)) or (bias is not None and bias.shape[0] != rows_w):
        raise AlofaError("invalid_argument", "gemm sizes disagree", f"out={tuple(out.shape)} w={tuple(w.shape)} epi={epi}")
    f32, i64 = torch.float32, torch.int64
    b_kind, b_src, b_ml, b_pos, heads, hd, window, split_keys = B_ROWS, None, None, None, 0, 0, 0, 0
    n_acc = n_gamma = n_out = n_zero = None
    n_eps = 0.0
    if computed is not None and computed[0] == B_NORMED:
        b_kind, base, acc_in, gamma, n_eps, new_base, zero = computed
        if tuple(base.shape) != (m, k) or tuple(new_base.shape) != (m, k) or gamma.shape[0] != k:
            raise AlofaError("invalid_argument", "normed operand sizes disagree", f"base={tuple(base.shape)} gamma={tuple(gamma.shape)} k={k}")
        b_src, n_gamma, n_out = _dev(base, "base", f32), _dev(gamma, "gamma", f32), _dev(new_base, "new_base", f32)
        n_acc = _dev(acc_in, "acc", i64) if acc_in is not None else None
        n_zero = _dev(zero, "zero", i64) if zero is not None else None
    elif computed is not None:
        b_kind, po, pml, positions, heads, hd, window, split_keys = computed
        b_src, b_ml, b_pos, window = _dev(po, "partial_o", f32), _dev(pml, "partial_ml", f32), _dev(positions, "positions", torch.int32), int(window or 0)
    elif x is None:
        raise AlofaError("invalid_argument", "gemm without a token operand")
    rc = _gemm_tc().alofa_gemm_tc(
        _dev(out, "out"), _dev(x, "x", torch.bfloat16) if x is not None else None, _dev(w, "w", torch.bfloat16),
        _dev(bias, "bias", f32) if bias is not None else None,
        _dev(partial, "partial", f32) if partial is not None else None,
        m, n, k, epi, _is_bf16(out, "out"), bn, splits, 1 if reduce else 0,
        _dev(status, "status", torch.int32) if status is not None else None,
        b_kind, b_src, b_ml, b_pos, heads, hd, window, split_keys,
        _dev(acc, "acc", i64) if acc is not None else None, n_acc, n_gamma, float(n_eps), n_out, n_zero, _stream(),
    )
    if rc == 1:
        return False
    _done(rc, "gemm_tc", f"M={m} N={n} K={k} epi={epi} bn={bn} splits={splits}")
    if splits > 1 and reduce and acc is None and b_kind != B_NORMED and not _gemm_tc().alofa_gemm_tc_reduces_in_cluster(epi, bn, splits):
        count_launches(1)  # the kernel that adds the split sums up
    return True


def gemm_tc_rope(x, w, bias, q_out, k_cache, v_cache, slot_map, positions, cos_sin, nh: int, nkv: int, hd: int, splits: int, status=None, normed=None) -> bool:
    """q/k/v of up to 16 tokens in one kernel: ``x @ w.T + bias`` for the
    stacked weight [q; k; v] (``nkv`` = 0: q only), q and k rotated, q to
    ``q_out``, k and v to their cache slots.  With ``normed`` = ``(base, acc or
    None, gamma, eps, new_base, zero or None)`` the operand is not ``x`` (None
    then) but the RMSNorm of the residual stream ``base + acc``, made in the
    kernel; the stream is also written to ``new_base`` and ``zero`` cleared.
    False, having launched nothing, when the kernel does not take these sizes."""
    bf, f32, i64 = torch.bfloat16, torch.float32, torch.int64
    t, k = (x.shape if normed is None else normed[0].shape)
    if t > 16 or 128 % hd or w.shape != ((nh + 2 * nkv) * hd, k):
        return False
    n_base = n_acc = n_gamma = n_out = n_zero = None
    n_eps = 0.0
    if normed is not None:
        base, acc_in, gamma, n_eps, new_base, zero = normed
        if tuple(new_base.shape) != (t, k) or gamma.shape[0] != k:
            raise AlofaError("invalid_argument", "normed operand sizes disagree", f"base={tuple(base.shape)} gamma={tuple(gamma.shape)}")
        n_base, n_gamma, n_out = _dev(base, "base", f32), _dev(gamma, "gamma", f32), _dev(new_base, "new_base", f32)
        n_acc = _dev(acc_in, "acc", i64) if acc_in is not None else None
        n_zero = _dev(zero, "zero", i64) if zero is not None else None
    rc = _gemm_tc().alofa_gemm_tc_rope(
        _dev(x, "x", bf) if x is not None else None, _dev(w, "w", bf), _dev(bias, "bias", f32) if bias is not None else None, t, k, _dev(q_out, "q_out", bf),
        _dev(k_cache, "k_cache", bf) if nkv else None, _dev(v_cache, "v_cache", bf) if nkv else None,
        _dev(slot_map, "slot_map", torch.int32) if nkv else None, _dev(positions, "positions", torch.int32), _dev(cos_sin, "cos_sin", f32),
        nh, nkv, hd, splits, _dev(status, "status", torch.int32) if status is not None else None,
        n_base, n_acc, n_gamma, float(n_eps), n_out, n_zero, _stream(),
    )
    if rc == 1:
        return False
    _done(rc, "gemm_tc_rope", f"T={t} K={k} heads={nh}+2x{nkv} hd={hd}")
    return True


def attention_bf16(out, q, k_cache, v_cache, q_start, kv_len, positions, block_table, page_size, n_seqs, max_q_len, nh, nkv, hd, window, scale,
                   n_splits: int = 0, split_keys: int = 0, partial_o=None, partial_ml=None, max_kv_len: int = 0, status=None, combine: bool = True) -> None:
    """Causal GQA over the paged bf16 cache for a step's requests; with
    ``n_splits`` > 0 the keys of each request (decode tokens) or of each query
    tile (prompt portions) are split over several CTAs and merged - unless
    ``combine`` is False (decode tokens only): then ``partial_o`` / ``partial_ml``
    keep the splits for :func:`attention_combine` or a product that merges them."""
    n = q.shape[0]
    bf = torch.bfloat16
    g = nh // nkv
    tiles = -(-(max_q_len * g) // 64)
    rc = _attention(hd).alofa_attention_bf16(
        _dev(out, "out", bf), _dev(q, "q", bf), _dev(k_cache, "k_cache", bf), _dev(v_cache, "v_cache", bf),
        _dev(q_start, "q_start", torch.int32), _dev(kv_len, "kv_len", torch.int32), _dev(positions, "positions", torch.int32),
        _dev(block_table, "block_table", torch.int32),
        block_table.shape[1], page_size, n_seqs, n, tiles, nh, nkv, int(window or 0), float(scale), n_splits, split_keys,
        _dev(partial_o, "partial_o", torch.float32) if partial_o is not None else None,
        _dev(partial_ml, "partial_ml", torch.float32) if partial_ml is not None else None,
        int(max_kv_len) if max_kv_len else block_table.shape[1] * page_size, k_cache.shape[0],
        _dev(status, "status", torch.int32) if status is not None else None, 1 if combine else 0, _stream(),
    )
    _done(rc, "attention_bf16", f"hd={hd} nh={nh} nkv={nkv} splits={n_splits}")
    if n_splits > 1 and combine:
        count_launches(1)


def attention_combine(out, partial_o, partial_ml, positions, nh: int, hd: int, window, split_keys: int) -> None:
    """Merge the key splits of decode tokens: out [T, nh * hd] bf16."""
    rc = _attention(hd).alofa_attention_combine(
        _dev(out, "out", torch.bfloat16), _dev(partial_o, "partial_o", torch.float32), _dev(partial_ml, "partial_ml", torch.float32),
        _dev(positions, "positions", torch.int32), out.shape[0], nh, int(window or 0), split_keys, _stream(),
    )
    _done(rc, "attention_combine")


def norm_fused(out, h, weight, eps: float, rows=None, partial=None, splits: int = 0, bias=None, base=None, acc=None, other=None) -> bool:
    """RMSNorm of rows of the fp32 stream ``h`` (vectorised; hidden % 4 == 0).
    With ``partial`` [splits, T, hidden] the pending partial sums (and bias)
    are first added into ``h``.  With ``base`` the stream's values are read
    from there (``h`` is written, complete), with ``acc`` (int64, units of
    2^-32; every row, ``rows`` None) that accumulator is added on top and left
    zero, as is ``other``.  Returns False when the size is not taken."""
    n, hidden = out.shape
    if hidden % 4:
        return False
    f32, i64 = torch.float32, torch.int64
    rc = _elementwise().alofa_norm_fused(
        _dev(out, "out"), _dev(h, "h", f32), _dev(weight, "weight", f32), _dev(partial, "partial", f32) if partial is not None else None,
        _dev(bias, "bias", f32) if bias is not None else None, _dev(rows, "rows", torch.int32) if rows is not None else None,
        n, h.shape[0], hidden, splits, float(eps), _is_bf16(out, "out"),
        _dev(base, "base", f32) if base is not None else None, _dev(acc, "acc", i64) if acc is not None else None,
        _dev(other, "other", i64) if other is not None else None, _stream(),
    )
    if rc == 1:
        return False
    _done(rc, "norm_fused")
    return True


def stream_settle(h, base, acc, other=None) -> None:
    """``h = base + acc`` (the residual stream of a small decode step brought
    back to one fp32 tensor); ``acc`` and ``other`` (int64, units of 2^-32) are
    left zero."""
    f32, i64 = torch.float32, torch.int64
    _done(
        _elementwise().alofa_stream_settle(_dev(h, "h", f32), _dev(base, "base", f32), _dev(acc, "acc", i64),
                                           _dev(other, "other", i64) if other is not None else None, h.numel(), _stream()),
        "stream_settle",
    )


def rope_store_fused(q_out, k_cache, v_cache, qkv, partial, splits, bias, cos_sin, positions, slot_map, nh, nkv, hd, write_cache=True) -> None:
    """bf16 rotate-and-store with full rotary (rot == hd, hd % 16 == 0); the
    source is ``qkv`` (bf16) or split-K ``partial`` sums [splits, T, C] + bias."""
    n = q_out.shape[0]
    bf, f32 = torch.bfloat16, torch.float32
    _done(
        _elementwise().alofa_rope_store_fused(
            _dev(q_out, "q_out", bf), _dev(k_cache, "k_cache", bf) if write_cache else None, _dev(v_cache, "v_cache", bf) if write_cache else None,
            _dev(qkv, "qkv", bf) if qkv is not None else None, _dev(partial, "partial", f32) if partial is not None else None,
            _dev(bias, "bias", f32) if bias is not None else None, _dev(cos_sin, "cos_sin", f32), _dev(positions, "positions", torch.int32),
            _dev(slot_map, "slot_map", torch.int32) if write_cache else None, n, nh, nkv, hd, splits, 1 if write_cache else 0, _stream(),
        ),
        "rope_store_fused", f"hd={hd}",
    )


def splitk_reduce(out, partial, bias, splits: int, epi: int) -> None:
    """out (op)= bias + sum of ``partial`` [splits, T, N] in split order."""
    t, n = out.shape
    _done(
        _gemm_tc().alofa_splitk_reduce(
            _dev(out, "out"), _dev(partial, "partial", torch.float32), _dev(bias, "bias", torch.float32) if bias is not None else None,
            t, n, splits, epi, _is_bf16(out, "out"), _stream(),
        ),
        "splitk_reduce",
    )
