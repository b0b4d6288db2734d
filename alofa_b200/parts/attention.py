"""Grouped-query attention over a paged key/value cache.

``q = x Wq^T + bq`` (and k, v), heads packed along the channel axis (channel
``h * head_dim + d``); q and k are position-encoded, k and v are appended to
the cache through the block table, query head ``h`` reads KV head
``h // (heads / kv_heads)``, keys up to the query's own position are visible
(all of them, or the last ``window``), scores are ``dot / sqrt(head_dim)``,
softmax in fp32, and the output projection is added into the residual stream
(src/alofa/kernels/cpu/scalar.mojo:132-193, 392-470;
src/alofa/kernels/cpu/paged.mojo:208-336; src/alofa/engine/executor.mojo:745-795).

At load the q, k and v weights are stacked into one matrix so that one product
yields all three; the checkpoint's tensors are read under their own names."""
from __future__ import annotations

import math

import torch

from ..csrc import ops
from ..errors import AlofaError
from . import fast_linear
from .base import PagedKV, Part, TensorSpec, as_float32_vector, build_part, register_part
from .linear import RESIDUAL, STORE, Linear, MergedSplits, add_into_stream


class GQAttention(Part):
    family = "mixer"

    @property
    def graph_safe(self):
        return self.position.graph_safe

    def __init__(self, spec, rt):
        super().__init__(spec, rt)
        p = self.param
        self.hidden = int(p("hidden_size"))
        self.nh = int(p("num_heads"))
        self.nkv = int(p("num_kv_heads"))
        self.hd = int(p("head_dim"))
        self.qkv_bias = bool(p("qkv_bias", False))
        self.out_bias = bool(p("out_bias", False))
        self.window = self.params.get("window")
        if self.nkv <= 0 or self.nh % self.nkv:
            raise AlofaError("invalid_argument", "kv heads must divide heads", f"heads={self.nh} kv_heads={self.nkv}")
        if self.hd <= 0 or self.hd % 2 or self.hd > 256:
            raise AlofaError("unsupported", "head_dim must be even and at most 256", f"head_dim={self.hd}")
        self.q_dim, self.kv_dim = self.nh * self.hd, self.nkv * self.hd
        self.scale = 1.0 / math.sqrt(self.hd)
        self.position = build_part("position", p("position"), rt)
        self.qkv = self.q_only = self.out = None

    def cache_spec(self):
        return PagedKV(self.nkv, self.hd, self.window)

    def scratch_row_bytes(self) -> int:
        # q/k/v, q, the attention output, and the output product's split sums
        return 4 * (self.q_dim + 2 * self.kv_dim) + 2 * 4 * self.q_dim + 2 * 4 * self.hidden

    def tensors(self):
        pre = self.prefix
        t = {
            pre + "q_proj.weight": TensorSpec((self.q_dim, self.hidden)),
            pre + "k_proj.weight": TensorSpec((self.kv_dim, self.hidden)),
            pre + "v_proj.weight": TensorSpec((self.kv_dim, self.hidden)),
            pre + "o_proj.weight": TensorSpec((self.hidden, self.q_dim)),
        }
        if self.qkv_bias:
            t[pre + "q_proj.bias"] = TensorSpec((self.q_dim,))
            t[pre + "k_proj.bias"] = TensorSpec((self.kv_dim,))
            t[pre + "v_proj.bias"] = TensorSpec((self.kv_dim,))
        if self.out_bias:
            t[pre + "o_proj.bias"] = TensorSpec((self.hidden,))
        t.update(self.position.tensors())
        return t

    def load(self, state):
        pre = self.prefix
        w = torch.cat([state[pre + f"{n}_proj.weight"] for n in "qkv"], dim=0)
        b = None
        if self.qkv_bias:
            b = as_float32_vector(torch.cat([state[pre + f"{n}_proj.bias"] for n in "qkv"], dim=0))
        self.qkv = Linear(w, b, STORE)
        # a run of this layer that reads another run's cache needs q only
        self.q_only = Linear(w[: self.q_dim], b[: self.q_dim] if b is not None else None, STORE)
        ob = as_float32_vector(state[pre + "o_proj.bias"]) if self.out_bias else None
        self.out = Linear(state[pre + "o_proj.weight"], ob, RESIDUAL)
        self.position.load(state)

    takes_normed_rows = True  # ``x`` may be rows still to be made: the q/k/v kernel of a few tokens folds the norm in

    def forward(self, ctx, x, h, cache, writes=True):
        """h += Attention(x).  ``cache`` is the layer cache (k, v, group)."""
        n = x.shape[0]
        dt = self.rt.dtype
        group = ctx.groups[cache.group]
        nkv_in = self.nkv if writes else 0
        table, rot = self.position.rotary_table()
        custom = getattr(self.position, "apply", None)
        # the vectorised rotate-and-store: bf16, the whole head rotated, head size a multiple of 16
        vectorised = dt == torch.bfloat16 and custom is None and rot == self.hd and self.hd % 16 == 0
        lin = self.qkv if writes else self.q_only
        q = ctx.buf((n, self.q_dim), dt)
        # a handful of tokens: product, bias, rotation and the cache write in one kernel
        # (its depth split over a cluster of up to eight CTAs: the largest for which every tile's cluster is
        # resident at once - a GPC holds whole clusters only, 16 clusters of 8 ran in two waves where 16 of 6 run
        # in one: 1.52 -> 1.41 ms per step at hidden 1,536) and only while a CTA then has a few k-slices: on deep
        # products (3,584 wide) the cluster measured slower
        lazy = None if isinstance(x, torch.Tensor) else x
        depth_splits = 1
        if vectorised and n <= 16 and x.dtype == torch.bfloat16:
            depth_splits = ops.gemm_tc_rope_splits(-(-lin.weight.shape[0] // 128), lazy is not None)
        shallow = -(-(-(-self.hidden // fast_linear.K_SLICE)) // depth_splits) <= 4
        one_kernel = vectorised and shallow and n <= 16 and lin.weight.dtype == torch.bfloat16 and x.dtype == torch.bfloat16
        done = False
        if lazy is not None:
            if one_kernel and lazy.fits_kernel():
                normed = lazy.computed()  # the norm folded into the q/k/v kernel
                done = ops.gemm_tc_rope(None, lin.weight, lin.bias, q, cache.k, cache.v, group.slot_map, ctx.positions, table, self.nh, nkv_in, self.hd,
                                        depth_splits, ctx.status, normed=normed[1:])
                if done:
                    lazy.done(normed)
                else:
                    lazy.undo()
            if not done:
                x = lazy.rows()
        if not done and one_kernel:
            done = ops.gemm_tc_rope(x, lin.weight, lin.bias, q, cache.k, cache.v, group.slot_map, ctx.positions, table, self.nh, nkv_in, self.hd,
                                    depth_splits, ctx.status)
        if not done:
            qkv = ctx.buf((n, (self.nh + 2 * nkv_in) * self.hd), dt)
            owed = lin(qkv, x, defer=vectorised, buf=ctx.buf)
            self._rotate_and_store(ctx, q, qkv, owed, cache, group, table, rot, custom, vectorised, nkv_in, writes)
        attn = self.attend(ctx, q, cache, group)
        add_into_stream(ctx, self.out, h, attn)

    def _rotate_and_store(self, ctx, q, qkv, owed, cache, group, table, rot, custom, vectorised, nkv_in, writes):
        n = q.shape[0]
        if vectorised:
            ops.rope_store_fused(
                q, cache.k, cache.v, None if owed is not None else qkv, owed.sums if owed is not None else None,
                owed.splits if owed is not None else 0, owed.bias if owed is not None else None,
                table, ctx.positions, group.slot_map, self.nh, nkv_in, self.hd, writes,
            )
        else:
            if custom is not None:
                q_view = qkv[:, : self.q_dim].view(n, self.nh, self.hd)
                k_view = qkv[:, self.q_dim : self.q_dim + nkv_in * self.hd].view(n, nkv_in, self.hd)
                custom(ctx, q_view, k_view)
            ops.rope_store(q, cache.k, cache.v, qkv, table, ctx.positions, group.slot_map, self.nh, nkv_in, self.hd, rot, writes)

    # Keys per CTA, at least, when a decode-only step splits each request's keys: four 64-key
    # blocks, one per warp.  Splits grow in steps of this (a warp then takes several blocks in
    # turn, fetching the next behind its work on this one) until the step's CTAs are resident
    # together: CTAs that queue for an SM load, then compute, wave after wave (batch 64 at
    # 2,048 keys: 1.58 -> 1.47 ms per step for 14 heads of 64 on 2, 5.90 -> 5.08 ms for 28 heads
    # of 128 on 4).
    SPLIT_KEYS = 256
    # On pages of whole key blocks head sizes 64 and 128 have a wide form of the kernel, one CTA per SM with
    # eight or six warps (what shared memory holds tiles for), whose splits grow by 64 keys a warp: fewer,
    # larger CTAs and fewer splits to merge (14 heads of 64 on 2, batch 8: nine splits of 256 keys 0.780 ms per
    # step, five of 512 0.758; batch 12: 0.819 -> 0.788; 28 heads of 128 on 4, batch 64: 5.03 -> 4.90 ms).  With
    # three tenths as many (request, KV head) pairs as SMs or more, in steps of more than 16 tokens, one split
    # per pair (14 heads of 64 on 2, batch 64: 1.40 -> 1.34 ms; batch 32: 1.065 -> 1.027; the merge kernel and
    # the partial sums go).
    # Keys per CTA when a step with prompt portions splits the keys of its query tiles; 0 = never.
    # Measured at 2,048-token prompts the round trip of the partial sums costs more than the
    # long tiles' tail saves (4.9 ms against 4.5 ms for the step), so it is off.
    PROMPT_SPLIT_KEYS = 0

    # Decode tokens in at most this many key splits are handed to the output product unmerged: it
    # merges them while it loads its operand, which saves a kernel; with more splits every CTA of
    # the product would re-read too many partial outputs.
    MERGE_IN_PRODUCT_SPLITS = 16

    @classmethod
    def decode_split_keys(cls, n_tokens: int, pairs: int, longest: int, longest_now: int, wide_slots: int, slots: int, wide_unit: int = 512) -> int:
        """Keys per CTA of a decode-only step.  ``pairs``: (request, KV head)
        pairs; ``longest``: the context the launch must cover (a graph's
        bucket), ``longest_now``: the longest context of this step;
        ``wide_slots`` / ``slots``: CTAs of the wide / four-warp kernel the
        device holds at a time (0: that kernel is not built here);
        ``wide_unit``: the keys the wide kernel's splits grow by."""
        pairs = max(1, pairs)
        # the unit a split grows by, and how many CTAs of that kernel are resident together
        unit, room = (wide_unit, wide_slots) if wide_slots > 0 else (cls.SPLIT_KEYS, slots)
        whole = unit * -(-longest // unit)
        if wide_slots > 0 and n_tokens > 16 and 10 * pairs >= 3 * wide_slots:
            # enough pairs to keep the SMs busy with one CTA each: the whole context in one split, no partial
            # sums and no kernel that merges them
            return whole
        # as many splits as are resident together, by the longest context of this step (a graph keeps what the
        # step that recorded it chose; every length its bucket holds is covered either way)
        blocks = -(-max(1, longest_now) // unit)
        per_split = unit * -(-blocks // max(1, room // pairs))
        if per_split >= blocks * unit:
            return whole  # one split: let it reach to the end of the bucket, so that nothing is merged
        if n_tokens <= 16 and longest <= 4 * cls.MERGE_IN_PRODUCT_SPLITS * cls.SPLIT_KEYS:
            # few enough splits that the output product merges them, while a warp has at most a few blocks
            per_split = max(per_split, unit * -(-longest // (unit * cls.MERGE_IN_PRODUCT_SPLITS)))
        return per_split

    def attend(self, ctx, q, cache, group):
        """Attention of the step's rows over the cache: the tensor-core kernels
        for bfloat16 and head sizes they are built for, else the generic one.
        Returns the output rows, or a :class:`MergedSplits` for the product
        that follows to merge."""
        out = ctx.buf((q.shape[0], self.q_dim), q.dtype)
        if q.dtype == torch.bfloat16 and ops.attention_bf16_supported(self.hd):
            splits, po, pml = 0, None, None
            longest = ctx.max_context if ctx.capturing else ctx.max_kv_len
            per_split = self.SPLIT_KEYS
            group_size = self.nh // self.nkv
            if ctx.decode_only and group_size <= 16:
                wide_warps = ops.attention_decode_wide_warps(self.hd)
                per_split = self.decode_split_keys(ctx.n_tokens, ctx.n_seqs * self.nkv, longest, ctx.max_kv_len,
                                                   ops.attention_decode_slots(self.hd, group.page_size, wide_warps) if wide_warps else 0,
                                                   ops.attention_decode_slots(self.hd, group.page_size), 64 * wide_warps)
            if not ctx.decode_only:
                per_split = self.PROMPT_SPLIT_KEYS or (1 << 30)
            if ctx.decode_only and self.nh // self.nkv <= 64 and (longest > per_split or self.nh // self.nkv <= 16):
                splits = max(1, -(-longest // per_split))
            elif not ctx.decode_only and longest > per_split:
                splits = -(-longest // per_split)
            if splits:
                po = ctx.buf((splits, ctx.n_tokens * self.nh, self.hd), torch.float32)
                pml = ctx.buf((splits, ctx.n_tokens * self.nh, 2), torch.float32)
            unmerged = ctx.decode_only and 1 < splits <= self.MERGE_IN_PRODUCT_SPLITS and self.nh // self.nkv <= 16 and ctx.n_tokens <= 16
            ops.attention_bf16(
                out, q, cache.k, cache.v, ctx.q_start, ctx.kv_len, ctx.positions, group.block_table, group.page_size, ctx.n_seqs, ctx.max_q_len,
                self.nh, self.nkv, self.hd, self.window, self.scale, splits, per_split, po, pml, longest, ctx.status, combine=not unmerged,
            )
            if unmerged:
                return MergedSplits(po, pml, ctx.positions, ctx.n_tokens, self.nh, self.hd, self.window, per_split, ctx.buf)
            return out
        ops.paged_attention_generic(
            out, q, cache.k, cache.v, ctx.positions, ctx.seq_of_token, group.block_table, group.page_size,
            self.nh, self.nkv, self.hd, self.window, self.scale,
        )
        return out


register_part("mixer", "gqa_attention", GQAttention)
