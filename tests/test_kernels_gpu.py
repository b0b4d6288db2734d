"""Each kernel alone against its plain fp64 reference, at sizes other than the
engine's test models: odd widths, head sizes in steps of 16, partial rotary,
scattered pages, and inputs made so that a wrong key or a wrong edge shows."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from gpu_util import assert_close, dev, paged_from_sequences, rounded

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
# kernel-level bounds, times max(1, max|reference|): fp32 sums against fp64;
# bf16 outputs are rounded once to 8 bits of mantissa (2^-9 relative)
TOL = {F32: 1e-5, BF16: 6e-3}


@pytest.fixture(scope="module")
def ops():
    from alofa_b200.csrc import ops

    return ops


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_embed_gather(ops, dtype):
    rng = np.random.default_rng(0)
    table = rounded(rng.normal(size=(301, 72)), dtype)
    ids = np.array([0, 300, 17, 17, 5], dtype=np.int32)
    out = torch.empty(5, 72, dtype=F32, device="cuda")
    status = torch.zeros(1, dtype=torch.int32, device="cuda")
    ops.embed_gather(out, dev(table, dtype), dev(ids), status)
    assert np.array_equal(out.cpu().numpy(), table[ids].astype(np.float32)) and int(status.item()) == 0
    ops.embed_gather(out, dev(table, dtype), dev(np.array([1, 301, -1, 2, 3], dtype=np.int32)), status)
    assert int(status.item()) == 1 and float(out[1].abs().max()) == 0.0


@pytest.mark.parametrize("out_dtype", [F32, BF16])
@pytest.mark.parametrize("hidden", [100, 896, 1000])
def test_rmsnorm(ops, out_dtype, hidden):
    rng = np.random.default_rng(1)
    x = rng.normal(size=(9, hidden)).astype(np.float32) * 3
    w = (1 + 0.1 * rng.normal(size=hidden)).astype(np.float32)
    out = torch.empty(9, hidden, dtype=out_dtype, device="cuda")
    ops.rmsnorm(out, dev(x), dev(w), 1e-5)
    assert_close(out.float().cpu(), plain.rmsnorm(x, w, 1e-5), TOL[out_dtype], "rmsnorm")
    rows = np.array([8, 0, 3], dtype=np.int32)
    out = torch.empty(3, hidden, dtype=out_dtype, device="cuda")
    ops.rmsnorm(out, dev(x), dev(w), 1e-5, dev(rows))
    assert_close(out.float().cpu(), plain.rmsnorm(x[rows], w, 1e-5), TOL[out_dtype], "rmsnorm rows")


@pytest.mark.parametrize("dtypes", [(F32, F32, F32), (BF16, BF16, BF16), (BF16, BF16, F32), (BF16, F32, BF16)])
@pytest.mark.parametrize("shape", [(37, 53, 71), (1, 130, 64), (70, 64, 200)])
def test_gemm_generic_epilogues(ops, dtypes, shape):
    xd, wd, od = dtypes
    m, n, k = shape
    rng = np.random.default_rng(2)
    x = rounded(rng.normal(size=(m, k)), xd)
    w = rounded(rng.normal(size=(2 * n, k)) / np.sqrt(k), wd)
    bias = rng.normal(size=2 * n).astype(np.float32)
    out = torch.empty(m, n, dtype=od, device="cuda")
    ops.gemm_generic(out, dev(x, xd), dev(w[:n], wd), dev(bias[:n]), ops.EPI_STORE)
    assert_close(out.float().cpu(), plain.linear(x, w[:n], bias[:n]), TOL[od], "store")
    ops.gemm_generic(out, dev(x, xd), dev(w, wd), None, ops.EPI_GATED)
    assert_close(out.float().cpu(), plain.silu(plain.linear(x, w[:n])) * plain.linear(x, w[n:]), TOL[od], "gated")
    res = rng.normal(size=(m, n)).astype(np.float32)
    acc = dev(res)
    ops.gemm_generic(acc, dev(x, xd), dev(w[:n], wd), None, ops.EPI_RESIDUAL)
    assert_close(acc.cpu(), res + plain.linear(x, w[:n]), TOL[F32], "residual")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("hd, rot", [(48, 48), (48, 32), (16, 16), (128, 64)])
def test_rope_store(ops, dtype, hd, rot):
    from alofa_b200.config.spec import PartSpec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.position import RotaryNeox

    rng = np.random.default_rng(3)
    n, nh, nkv = 11, 3, 1
    part = RotaryNeox(PartSpec("rotary_neox", {"head_dim": hd, "rotary_dim": rot, "theta": 5e4, "max_position": 600}), Runtime(torch.device("cuda"), dtype))
    table = part.build_table(600)
    qkv = rounded(rng.normal(size=(n, (nh + 2 * nkv) * hd)), dtype)
    positions = np.array([0, 1, 2, 599, 64, 63, 17, 300, 5, 5, 128], dtype=np.int32)
    slots = np.array([4, 9, 0, 31, -1, 2, 7, 30, 12, 13, 1], dtype=np.int32)
    k_cache = torch.full((32, nkv, hd), 3.0, dtype=dtype, device="cuda")
    v_cache = torch.full((32, nkv, hd), 3.0, dtype=dtype, device="cuda")
    q_out = torch.empty(n, nh * hd, dtype=dtype, device="cuda")
    ops.rope_store(q_out, k_cache, v_cache, dev(qkv, dtype), table, dev(positions), dev(slots), nh, nkv, hd, rot)

    def rotate(x, heads):
        x = x.reshape(n, heads, hd)
        out = x.copy()
        out[..., :rot] = plain.rope(x[..., :rot].reshape(n, heads * rot), positions, heads, rot, 5e4).reshape(n, heads, rot)
        return out.reshape(n, heads * hd)

    q, k, v = qkv[:, : nh * hd], qkv[:, nh * hd : (nh + nkv) * hd], qkv[:, (nh + nkv) * hd :]
    assert_close(q_out.float().cpu(), rotate(q, nh), TOL[dtype], "q")
    want_k = np.full((32, nkv * hd), 3.0)
    want_v = np.full((32, nkv * hd), 3.0)
    rk = rotate(k, nkv)
    for t, s in enumerate(slots):
        if s >= 0:
            want_k[s], want_v[s] = rk[t], v[t]
    assert_close(k_cache.float().cpu().reshape(32, -1), want_k, TOL[dtype], "k cache")
    assert_close(v_cache.float().cpu().reshape(32, -1), want_v, 0.0, "v cache")


@pytest.mark.parametrize("out_dtype", [F32, BF16])
def test_norm_fused_adds_owed_partial_sums(ops, out_dtype):
    rng = np.random.default_rng(11)
    hidden, tokens, splits = 896, 9, 5
    h = rng.normal(size=(tokens, hidden)).astype(np.float32)
    partial = rng.normal(size=(splits, tokens, hidden)).astype(np.float32)
    bias = rng.normal(size=hidden).astype(np.float32)
    w = (1 + 0.1 * rng.normal(size=hidden)).astype(np.float32)
    hd = dev(h)
    out = torch.empty(tokens, hidden, dtype=out_dtype, device="cuda")
    assert ops.norm_fused(out, hd, dev(w), 1e-6, None, dev(partial), splits, dev(bias))
    total = h.astype(np.float64) + partial.astype(np.float64).sum(axis=0) + bias
    assert_close(hd.cpu(), total, 1e-6, "stream after the sums")
    assert_close(out.float().cpu(), plain.rmsnorm(total, w, 1e-6), TOL[out_dtype], "norm of the summed stream")
    rows = np.array([7, 2], dtype=np.int32)
    out = torch.empty(2, hidden, dtype=out_dtype, device="cuda")
    assert ops.norm_fused(out, dev(h), dev(w), 1e-6, dev(rows), dev(partial), splits, None)
    assert_close(out.float().cpu(), plain.rmsnorm((h.astype(np.float64) + partial.astype(np.float64).sum(axis=0))[rows], w, 1e-6), TOL[out_dtype], "gathered rows")
    assert not ops.norm_fused(torch.empty(2, 6, dtype=out_dtype, device="cuda"), dev(h[:, :6].copy()), dev(w[:6].copy()), 1e-6)  # width not a multiple of 4
    # a handful of rows that owe many split sums (one round of loads for up to 24, then rounds of 8)
    for width, n_splits, n in ((896, 19, 8), (100, 30, 1), (3584, 9, 16)):
        hh = rng.normal(size=(n, width)).astype(np.float32)
        pp = rng.normal(size=(n_splits, n, width)).astype(np.float32)
        bb = rng.normal(size=width).astype(np.float32)
        ww = (1 + 0.1 * rng.normal(size=width)).astype(np.float32)
        hdev = dev(hh)
        out = torch.empty(n, width, dtype=out_dtype, device="cuda")
        assert ops.norm_fused(out, hdev, dev(ww), 1e-6, None, dev(pp), n_splits, dev(bb))
        total = hh.astype(np.float64) + pp.astype(np.float64).sum(axis=0) + bb
        assert_close(hdev.cpu(), total, 2e-6, f"stream after {n_splits} sums")
        assert_close(out.float().cpu(), plain.rmsnorm(total, ww, 1e-6), TOL[out_dtype], f"norm after {n_splits} sums of {width}")
    # many rows take the warp-per-row form (a row in 8, 16 or 32 register groups per lane; wider rows a block each)
    for width in (200, 1000, 1536, 3588, 5120):
        many = rng.normal(size=(259, width)).astype(np.float32)
        part = rng.normal(size=(2, 259, width)).astype(np.float32)
        bm = rng.normal(size=width).astype(np.float32)
        wm = (1 + 0.1 * rng.normal(size=width)).astype(np.float32)
        hm = dev(many)
        out = torch.empty(259, width, dtype=out_dtype, device="cuda")
        assert ops.norm_fused(out, hm, dev(wm), 1e-5, None, dev(part), 2, dev(bm))
        total = many.astype(np.float64) + part.astype(np.float64).sum(axis=0) + bm
        assert_close(hm.cpu(), total, 1e-6, f"stream after the sums (many rows of {width})")
        assert_close(out.float().cpu(), plain.rmsnorm(total, wm, 1e-5), TOL[out_dtype], f"norm (many rows of {width})")
        out = torch.empty(259, width, dtype=out_dtype, device="cuda")
        assert ops.norm_fused(out, dev(many), dev(wm), 1e-5)
        assert_close(out.float().cpu(), plain.rmsnorm(many, wm, 1e-5), TOL[out_dtype], f"plain norm (many rows of {width})")
    picked = np.array([258, 0, 77] * 90, dtype=np.int32)  # gathered rows, many of them
    out = torch.empty(270, 5120, dtype=out_dtype, device="cuda")
    assert ops.norm_fused(out, dev(many), dev(wm), 1e-5, dev(picked))
    assert_close(out.float().cpu(), plain.rmsnorm(many[picked], wm, 1e-5), TOL[out_dtype], "gathered rows (many)")
    many = many[:, :1000].copy()
    out = torch.empty(270, 1000, dtype=out_dtype, device="cuda")
    assert ops.norm_fused(out, dev(many), dev(wm[:1000].copy()), 1e-5, dev(picked))
    assert_close(out.float().cpu(), plain.rmsnorm(many[picked], wm[:1000], 1e-5), TOL[out_dtype], "gathered rows (many, a warp each)")


@pytest.mark.parametrize("hd", [16, 48, 64, 128])
def test_rope_store_fused_from_tensor_and_from_partial_sums(ops, hd):
    from alofa_b200.config.spec import PartSpec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.position import RotaryNeox

    rng = np.random.default_rng(hd)
    n, nh, nkv, splits = 13, 3, 2, 4
    C = (nh + 2 * nkv) * hd
    table = RotaryNeox(PartSpec("rotary_neox", {"head_dim": hd, "theta": 1e6, "max_position": 700}), Runtime(torch.device("cuda"), BF16)).build_table(700)
    positions = rng.integers(0, 700, n).astype(np.int32)
    slots = rng.permutation(40)[:n].astype(np.int32)
    slots[3] = -1
    partial = rng.normal(size=(splits, n, C)).astype(np.float32)
    bias = rng.normal(size=C).astype(np.float32)
    summed = partial.astype(np.float64).sum(axis=0) + bias
    for source in ("partial", "tensor"):
        k_cache = torch.full((40, nkv, hd), 3.0, dtype=BF16, device="cuda")
        v_cache = torch.full((40, nkv, hd), 3.0, dtype=BF16, device="cuda")
        q_out = torch.empty(n, nh * hd, dtype=BF16, device="cuda")
        if source == "partial":
            qkv = summed
            ops.rope_store_fused(q_out, k_cache, v_cache, None, dev(partial), splits, dev(bias), table, dev(positions), dev(slots), nh, nkv, hd)
        else:
            qkv = rounded(summed, BF16)
            ops.rope_store_fused(q_out, k_cache, v_cache, dev(qkv, BF16), None, 0, None, table, dev(positions), dev(slots), nh, nkv, hd)
        q, k, v = qkv[:, : nh * hd], qkv[:, nh * hd : (nh + nkv) * hd], qkv[:, (nh + nkv) * hd :]
        assert_close(q_out.float().cpu(), plain.rope(q, positions, nh, hd, 1e6), TOL[BF16], f"q {source}")
        want_k, want_v = np.full((40, nkv * hd), 3.0), np.full((40, nkv * hd), 3.0)
        rk = plain.rope(k, positions, nkv, hd, 1e6)
        for t, s_ in enumerate(slots):
            if s_ >= 0:
                want_k[s_], want_v[s_] = rk[t], v[t]
        assert_close(k_cache.float().cpu().reshape(40, -1), want_k, TOL[BF16], f"k {source}")
        assert_close(v_cache.float().cpu().reshape(40, -1), want_v, TOL[BF16], f"v {source}")


@pytest.mark.parametrize("hd, nh, nkv, k", [(64, 14, 2, 896), (32, 3, 1, 96), (128, 4, 2, 512), (64, 3, 0, 192), (16, 5, 5, 64)])
def test_qkv_product_rotates_and_stores(ops, hd, nh, nkv, k):
    """q/k/v of a few tokens in one kernel (product, bias, rotation, cache
    write; the depth split over a cluster) against fp64, and bit for bit
    against the product followed by the rotate-and-store kernel."""
    from alofa_b200.config.spec import PartSpec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.position import RotaryNeox

    rng = np.random.default_rng(hd + k)
    table = RotaryNeox(PartSpec("rotary_neox", {"head_dim": hd, "theta": 1e4, "max_position": 900}), Runtime(torch.device("cuda"), BF16)).build_table(900)
    C = (nh + 2 * nkv) * hd
    w = rounded(rng.normal(size=(C, k)) / np.sqrt(k), BF16)
    bias = rng.normal(size=C).astype(np.float32)
    for n in (1, 7, 16):
        x = rounded(rng.normal(size=(n, k)), BF16)
        positions = rng.integers(0, 900, n).astype(np.int32)
        slots = rng.permutation(40)[:n].astype(np.int32)
        if n > 3:
            slots[3] = -1
        for splits in (1, 8):
            kc = torch.full((40, max(nkv, 1), hd), 3.0, dtype=BF16, device="cuda")
            vc = torch.full((40, max(nkv, 1), hd), 3.0, dtype=BF16, device="cuda")
            q_out = torch.empty(n, nh * hd, dtype=BF16, device="cuda")
            assert ops.gemm_tc_rope(dev(x, BF16), dev(w, BF16), dev(bias), q_out, kc, vc, dev(slots), dev(positions), table, nh, nkv, hd, splits)
            qkv = plain.linear(x, w, bias)
            q, kk, vv = qkv[:, : nh * hd], qkv[:, nh * hd : (nh + nkv) * hd], qkv[:, (nh + nkv) * hd :]
            assert_close(q_out.float().cpu(), plain.rope(q, positions, nh, hd, 1e4), TOL[BF16], f"q n={n} splits={splits}")
            if nkv:
                want_k, want_v = np.full((40, nkv * hd), 3.0), np.full((40, nkv * hd), 3.0)
                rk = plain.rope(kk, positions, nkv, hd, 1e4)
                for t, s_ in enumerate(slots):
                    if s_ >= 0:
                        want_k[s_], want_v[s_] = rk[t], vv[t]
                assert_close(kc.float().cpu().reshape(40, -1), want_k, TOL[BF16], f"k n={n} splits={splits}")
                assert_close(vc.float().cpu().reshape(40, -1), want_v, TOL[BF16], f"v n={n} splits={splits}")
    assert not ops.gemm_tc_rope(torch.zeros(17, k, dtype=BF16, device="cuda"), dev(w, BF16), None, torch.empty(17, nh * hd, dtype=BF16, device="cuda"),
                                kc, vc, dev(np.zeros(17, dtype=np.int32)), dev(np.zeros(17, dtype=np.int32)), table, nh, nkv, hd, 4), "more than 16 tokens"


def test_qkv_cluster_size_is_what_the_device_holds_at_once(ops):
    """The depth split of the q/k/v kernel: the largest cluster size for which
    the runtime reports every tile's cluster resident together, so it can only
    shrink as the tiles grow in number, and one tile gets the largest."""
    sizes = [ops.gemm_tc_rope_splits(tiles, normed) for normed in (True, False) for tiles in (1, 9, 16, 24, 36, 74, 148, 400)]
    for half in (sizes[:8], sizes[8:]):
        assert half[0] == 8 and all(1 <= s <= 8 for s in half)
        assert all(a >= b for a, b in zip(half, half[1:])), half
        assert half[-1] == 1  # more tiles than SMs: no cluster of two fits them all
    sms = torch.cuda.get_device_properties(0).multi_processor_count
    for tiles, split in zip((1, 9, 16, 24, 36, 74), sizes[:6]):
        assert tiles * split <= sms


@pytest.mark.parametrize("shape", [(5, 128, 64, 16, 1), (33, 379, 96, 64, 1), (300, 1152, 896, 128, 3), (8, 896, 4864, 16, 19), (513, 640, 320, 256, 2),
                                   (8, 512, 896, 16, 3), (13, 200, 320, 16, 5), (16, 131, 512, 16, 8), (29, 640, 896, 32, 3),  # gated: the splits add up inside a cluster
                                   (5, 128, 64, -64, 1), (130, 379, 96, -128, 1), (300, 1152, 896, -256, 3), (513, 650, 320, -256, 2), (257, 200, 240, -128, 1),
                                   (5, 40000, 96, -256, 1), (40, 40000, 96, -256, 1), (130, 39996, 64, -256, 1),  # more tiles than SMs: one resident CTA per SM, tiles cut evenly (5 and 40 tokens: 32 and 64 rows of the token tile fetched)
                                   (8, 2048, 1536, 16, 8), (8, 1536, 8960, 16, 12), (64, 1536, 1536, 64, 6), (300, 8960, 1536, -256, 1),  # widths of the 1.5B shape
                                   (8, 4608, 3584, 16, 4), (8, 3584, 18944, 16, 5), (33, 3584, 3584, 64, 2), (200, 4608, 3584, -256, 1),  # and of the 7B shape
                                   # deep and wide over several token tiles: pairs of CTAs with MMAs of M = 256 (ragged depth and width, a pair's
                                   # second token tile partly or wholly past the end)
                                   (300, 13000, 2056, -256, 1), (129, 20000, 1024, -256, 1)])
def test_gemm_tc_epilogues_and_split_depth(ops, shape):
    """The tcgen05 product against fp64: every epilogue, ragged sizes, split
    depth; weights on the M side (tile > 0) and tokens on the M side (tile < 0)."""
    m, n, k, bn, splits = shape
    rng = np.random.default_rng(m + n)
    x = rounded(rng.normal(size=(m, k)), BF16)
    w = rounded(rng.normal(size=(2 * n, k)) / np.sqrt(k), BF16)
    bias = rng.normal(size=2 * n).astype(np.float32)
    real = ops.gemm_tc_splits(k, splits)

    def ws(n_acc):
        return torch.empty(real * n_acc, m, n, device="cuda") if real > 1 else None

    for od in (BF16, F32):
        out = torch.empty(m, n, dtype=od, device="cuda")
        assert ops.gemm_tc(out, dev(x, BF16), dev(w[:n], BF16), dev(bias[:n]), ops.EPI_STORE, bn, splits, ws(1))
        assert_close(out.float().cpu(), plain.linear(x, w[:n], bias[:n]), TOL[od], "store")
        assert ops.gemm_tc(out, dev(x, BF16), dev(w, BF16), None, ops.EPI_GATED, bn, splits, ws(2))
        assert_close(out.float().cpu(), plain.silu(plain.linear(x, w[:n])) * plain.linear(x, w[n:]), TOL[od], "gated")
    res = rng.normal(size=(m, n)).astype(np.float32)
    acc = dev(res)
    assert ops.gemm_tc(acc, dev(x, BF16), dev(w[:n], BF16), None, ops.EPI_RESIDUAL, bn, splits, ws(1))
    assert_close(acc.cpu(), res + plain.linear(x, w[:n]), 2e-5, "residual")
    if real > 1:  # deferred: the partial sums alone, added up by the caller
        part = ws(1)
        assert ops.gemm_tc(part[0], dev(x, BF16), dev(w[:n], BF16), None, ops.EPI_RESIDUAL, bn, splits, part, reduce=False)
        assert_close(part.sum(dim=0).cpu(), plain.linear(x, w[:n]), 2e-5, "partial sums")
    assert not ops.gemm_tc(torch.empty(4, 8, dtype=BF16, device="cuda"), torch.zeros(4, 12, dtype=BF16, device="cuda"), torch.zeros(8, 12, dtype=BF16, device="cuda"), None, ops.EPI_STORE, 16)


def attention_case(ops, dtype, hd, nh, nkv, lens, q_lens, page, window, rng, craft=None, given=None, fast=False, split_keys=0):
    """Sequences of ``lens`` keys; the last ``q_lens[i]`` positions of each are
    queries in this launch.  Returns (got, want) as float64 arrays."""
    if given is not None:
        qs, ks, vs = given
    else:
        ks = [rounded(rng.normal(size=(n, nkv * hd)), dtype) for n in lens]
        vs = [rounded(rng.normal(size=(n, nkv * hd)), dtype) for n in lens]
        qs = [rounded(rng.normal(size=(n, nh * hd)), dtype) for n in lens]
    if craft:
        craft(qs, ks, vs)
        ks = [rounded(k, dtype) for k in ks]
        qs = [rounded(q, dtype) for q in qs]
    k_cache, v_cache, table = paged_from_sequences(ks, vs, page, nkv, hd, dtype, rng)
    q_rows, positions, seq_of = [], [], []
    want = []
    for s, (n, ql) in enumerate(zip(lens, q_lens)):
        full = plain.attention(qs[s], ks[s], vs[s], nh, nkv, hd, window)
        for p in range(n - ql, n):
            q_rows.append(qs[s][p])
            positions.append(p)
            seq_of.append(s)
            want.append(full[p])
    q = dev(np.stack(q_rows), dtype)
    out = torch.empty_like(q)
    if fast:
        q_start = np.concatenate([[0], np.cumsum(q_lens)]).astype(np.int32)
        n_splits, po, pml = 0, None, None
        if split_keys:
            n_splits = -(-max(lens) // split_keys)
            po = torch.empty(n_splits, len(q_rows) * nh, hd, device="cuda")
            pml = torch.empty(n_splits, len(q_rows) * nh, 2, device="cuda")
        ops.attention_bf16(out, q, k_cache, v_cache, dev(q_start), dev(np.array(lens, dtype=np.int32)), dev(np.array(positions, dtype=np.int32)), table, page, len(lens), max(q_lens),
                           nh, nkv, hd, window, 1.0 / np.sqrt(hd), n_splits, split_keys, po, pml)
        return out.float().cpu().numpy().astype(np.float64), np.stack(want)
    ops.paged_attention_generic(out, q, k_cache, v_cache, dev(np.array(positions, dtype=np.int32)), dev(np.array(seq_of, dtype=np.int32)),
                                table, page, nh, nkv, hd, window, 1.0 / np.sqrt(hd))
    return out.float().cpu().numpy().astype(np.float64), np.stack(want)


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("hd, nh, nkv", [(16, 4, 2), (48, 6, 2), (80, 5, 5), (128, 8, 1), (256, 2, 1)])
def test_paged_attention_generic_sizes(ops, dtype, hd, nh, nkv):
    rng = np.random.default_rng(hd)
    got, want = attention_case(ops, dtype, hd, nh, nkv, lens=[1, 37, 300, 129], q_lens=[1, 37, 2, 1], page=16, window=None, rng=rng)
    assert_close(got, want, TOL[dtype], f"hd={hd}")


@pytest.mark.parametrize("dtype", [F32, BF16])
def test_attention_finds_one_far_key_among_hundreds(ops, dtype):
    """One key far back is made to dominate the softmax: the output must be its
    value.  A kernel that skips a page, a chunk edge or a block-table entry
    misses it."""
    hd, nh, nkv = 32, 2, 1
    for far in (0, 15, 16, 127, 128, 255, 256, 400, 650):
        rng = np.random.default_rng(far)

        def craft(qs, ks, vs, far=far):
            direction = rng.normal(size=hd)
            direction /= np.linalg.norm(direction)
            for h in range(nh):
                qs[0][-1, h * hd : (h + 1) * hd] = 12.0 * direction
            ks[0][far, :hd] = 12.0 * direction
            vs[0][far, :hd] = 100.0

        got, want = attention_case(ops, dtype, hd, nh, nkv, lens=[700], q_lens=[1], page=16, window=None, rng=rng, craft=craft)
        assert np.abs(want[0]).min() > 90.0  # the plain output is that key's value
        assert_close(got, want, TOL[dtype], f"far key at {far}")


@pytest.mark.parametrize("dtype", [F32, BF16])
@pytest.mark.parametrize("window", [1, 16, 24, 129])
def test_attention_window_edge(ops, dtype, window):
    """A dominating key exactly at the window's oldest place is seen; one
    place older it is not."""
    hd, nh, nkv, n = 16, 2, 2, 300
    for offset, seen in ((window - 1, True), (window, False)):
        rng = np.random.default_rng(window)

        def craft(qs, ks, vs, offset=offset):
            direction = np.ones(hd) / np.sqrt(hd)
            qs[0][-1, :] = np.tile(14.0 * direction, nh)
            ks[0][n - 1 - offset, :] = np.tile(14.0 * direction, nkv)
            vs[0][n - 1 - offset, :] = 50.0

        got, want = attention_case(ops, dtype, hd, nh, nkv, lens=[n], q_lens=[1], page=16, window=window, rng=rng, craft=craft)
        assert (np.abs(want[0]).min() > 45.0) == seen
        assert_close(got, want, TOL[dtype], f"window {window} offset {offset}")


@pytest.mark.parametrize("hd, nh, nkv, window", [(64, 14, 2, None), (32, 3, 1, 300), (128, 4, 4, None), (48, 5, 5, 700)])
def test_output_product_merges_the_key_splits(ops, hd, nh, nkv, window):
    """Decode tokens whose key splits are left unmerged, and the residual
    product that merges them while it loads its operand, against the merge
    kernel followed by the plain product, and against fp64: one to sixteen
    tokens, lengths on both sides of the split edges, products with one and
    with several k-slices per CTA."""
    rng = np.random.default_rng(hd)
    for lens in ([600], [1, 255, 256, 257, 900, 3000, 512, 64, 4000, 33, 1023, 1024, 1025, 2047, 2048, 2049]):
        n = len(lens)
        ks = [rounded(rng.normal(size=(m, nkv * hd)), BF16) for m in lens]
        vs = [rounded(rng.normal(size=(m, nkv * hd)), BF16) for m in lens]
        qs = [rounded(rng.normal(size=(m, nh * hd)), BF16) for m in lens]
        k_cache, v_cache, table = paged_from_sequences(ks, vs, 64, nkv, hd, BF16, rng)
        q = dev(np.stack([qs[i][-1] for i in range(n)]), BF16)
        positions = dev(np.array([m - 1 for m in lens], dtype=np.int32))
        kv_len = dev(np.array(lens, dtype=np.int32))
        q_start = dev(np.arange(n + 1, dtype=np.int32))
        splits = -(-max(lens) // 256)
        po = torch.zeros(splits, n * nh, hd, device="cuda")
        pml = torch.zeros(splits, n * nh, 2, device="cuda")
        unused = torch.full((n, nh * hd), 7.0, dtype=BF16, device="cuda")
        ops.attention_bf16(unused, q, k_cache, v_cache, q_start, kv_len, positions, table, 64, n, 1, nh, nkv, hd, window, hd ** -0.5, splits, 256, po, pml, combine=False)
        assert float(unused.float().min()) == 7.0, "the attention kernel was told not to merge"
        merged = torch.empty(n, nh * hd, dtype=BF16, device="cuda")
        ops.attention_combine(merged, po, pml, positions, nh, hd, window, 256)
        want_attn = np.stack([plain.attention(qs[i], ks[i], vs[i], nh, nkv, hd, window)[-1] for i in range(n)])
        assert_close(merged.float().cpu(), want_attn, TOL[BF16], "merged splits")
        feats = 200
        w = rounded(rng.normal(size=(feats, nh * hd)) / np.sqrt(nh * hd), BF16)
        res = rng.normal(size=(n, feats)).astype(np.float32)
        for k_splits in (1, 4, ops.gemm_tc_splits(nh * hd, 64)):
            real = ops.gemm_tc_splits(nh * hd, k_splits)
            if splits > 16:
                continue  # more key splits than the product merges: the caller merges first
            part = torch.empty(real, n, feats, device="cuda") if real > 1 else None
            fused, plain_way = dev(res), dev(res)
            computed = (ops.B_MERGED_SPLITS, po, pml, positions, nh, hd, window, 256)
            assert ops.gemm_tc(fused, None, dev(w, BF16), None, ops.EPI_RESIDUAL, 16, k_splits, part, computed=computed)
            part2 = torch.empty(real, n, feats, device="cuda") if real > 1 else None
            assert ops.gemm_tc(plain_way, merged, dev(w, BF16), None, ops.EPI_RESIDUAL, 16, k_splits, part2)
            assert torch.equal(fused, plain_way), f"merging in the product changes bits (k splits {real})"
            assert_close(fused.cpu(), res + plain.linear(rounded(want_attn, BF16), w), 2e-2, f"product of merged splits (k splits {real})")


@pytest.mark.parametrize("hd, nh, nkv", [(16, 4, 2), (32, 3, 1), (48, 5, 5), (64, 14, 2), (80, 6, 3), (128, 8, 1)])
@pytest.mark.parametrize("page", [16, 48, 64])
def test_attention_bf16_sizes_portions_and_windows(ops, hd, nh, nkv, page):
    """The tensor-core kernel: whole prompts, portions that start mid-sequence,
    single tokens, in one launch; with and without a window."""
    for window in (None, 40):
        rng = np.random.default_rng(hd + page)
        got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[1, 37, 300, 129, 200, 64], q_lens=[1, 37, 2, 1, 131, 64], page=page, window=window, rng=rng, fast=True)
        assert_close(got, want, TOL[BF16], f"hd={hd} page={page} window={window}")


@pytest.mark.parametrize("hd, nh, nkv", [(64, 14, 2), (32, 3, 1), (128, 8, 8)])
def test_attention_bf16_split_keys(ops, hd, nh, nkv):
    """Decode tokens with each request's keys split over several CTAs: splits of
    128 keys (blocks one after the other) and of 256 (one block per warp)."""
    for window in (None, 300):
        for split, page in ((128, 16), (256, 16), (256, 64), (256, 48)):
            rng = np.random.default_rng(hd)
            lens = [1, 63, 64, 65, 300, 1000, 129, 256, 257, 511]
            got, want = attention_case(ops, BF16, hd, nh, nkv, lens=lens, q_lens=[1] * len(lens), page=page, window=window, rng=rng, fast=True, split_keys=split)
            assert_close(got, want, TOL[BF16], f"split {split} hd={hd} window={window} page={page}")
            whole, _ = attention_case(ops, BF16, hd, nh, nkv, lens=lens, q_lens=[1] * len(lens), page=page, window=window, rng=np.random.default_rng(hd), fast=True)
            assert_close(got, whole, TOL[BF16], "split vs unsplit")
    # a single split writes the output itself
    got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[200, 7], q_lens=[1, 1], page=16, window=None, rng=np.random.default_rng(1), fast=True, split_keys=256)
    assert_close(got, want, TOL[BF16], "one split")


@pytest.mark.parametrize("hd, nh, nkv", [(64, 14, 2), (128, 7, 1), (32, 6, 2)])
def test_attention_bf16_long_splits(ops, hd, nh, nkv):
    """Splits of several blocks per warp (512 to 1,280 keys): a warp refills its
    key tile and its value tile while it works on the block before.  Lengths
    either side of every edge: one block, one round of the warps, a split."""
    lens = [1, 65, 256, 257, 513, 769, 1025, 2049, 2600]
    # 3,072 keys: one split for every request here; multiples of 512 keys run on eight warps at head size 64, multiples
    # of 384 on six at head size 128 (384 itself: one block per warp), on pages of whole blocks
    for window, cases in ((None, ((512, 64), (768, 128), (1280, 64), (512, 16), (3072, 64), (384, 64))), (700, ((1024, 64), (768, 48), (3072, 128)))):
        for split, page in cases:
            got, want = attention_case(ops, BF16, hd, nh, nkv, lens=lens, q_lens=[1] * len(lens), page=page, window=window, rng=np.random.default_rng(hd + split), fast=True, split_keys=split)
            assert_close(got, want, TOL[BF16], f"split {split} hd={hd} window={window} page={page}")
    # one far key, in every block of a 1,024-key split in turn, among 2,049
    for far in range(1024 + 5, 2049, 128 if hd != 64 else 64):
        rng = np.random.default_rng(far)

        def craft(qs, ks, vs, far=far):
            direction = rng.normal(size=hd)
            direction /= np.linalg.norm(direction)
            qs[0][-1, :] = np.tile(12.0 * direction, nh)
            ks[0][far, :] = np.tile(12.0 * direction, nkv)
            vs[0][far, :] = 100.0

        got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[2049], q_lens=[1], page=64, window=None, rng=rng, craft=craft, fast=True, split_keys=1024)
        assert np.abs(want[0]).min() > 90.0
        assert_close(got, want, TOL[BF16], f"far key at {far}")


def test_attention_bf16_prompt_portions_with_split_keys(ops):
    """Prompt portions (and decode tokens beside them) whose query tiles split
    their keys over several CTAs."""
    for hd, nh, nkv in ((64, 14, 2), (32, 3, 1), (128, 8, 8)):
        for window in (None, 200):
            rng = np.random.default_rng(hd)
            lens, q_lens = [700, 37, 300, 129, 1, 450], [300, 37, 2, 1, 1, 450]
            got, want = attention_case(ops, BF16, hd, nh, nkv, lens=lens, q_lens=q_lens, page=16, window=window, rng=rng, fast=True, split_keys=192)
            assert_close(got, want, TOL[BF16], f"prompt split hd={hd} window={window}")


def test_attention_bf16_far_key_and_window_edge(ops):
    hd, nh, nkv = 64, 4, 2
    for split in (0, 64, 256):
        for far in (0, 63, 64, 127, 128, 500, 699):
            rng = np.random.default_rng(far)

            def craft(qs, ks, vs, far=far):
                direction = rng.normal(size=hd)
                direction /= np.linalg.norm(direction)
                qs[0][-1, :] = np.tile(12.0 * direction, nh)
                ks[0][far, :] = np.tile(12.0 * direction, nkv)
                vs[0][far, :] = 100.0

            got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[700], q_lens=[1], page=16, window=None, rng=rng, craft=craft, fast=True, split_keys=split)
            assert np.abs(want[0]).min() > 90.0
            assert_close(got, want, TOL[BF16], f"far key at {far} split {split}")
        for window in (1, 64, 65, 129):
            for offset, seen in ((window - 1, True), (window, False)):
                rng = np.random.default_rng(window)

                def craft(qs, ks, vs, offset=offset):
                    direction = np.ones(hd) / np.sqrt(hd)
                    qs[0][-1, :] = np.tile(14.0 * direction, nh)
                    ks[0][299 - offset, :] = np.tile(14.0 * direction, nkv)
                    vs[0][299 - offset, :] = 50.0

                got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[300], q_lens=[1], page=16, window=window, rng=rng, craft=craft, fast=True, split_keys=split)
                assert (np.abs(want[0]).min() > 45.0) == seen
                assert_close(got, want, TOL[BF16], f"window {window} offset {offset} split {split}")


@pytest.mark.parametrize("hd, nh, nkv", [(64, 14, 2), (64, 3, 3), (128, 8, 2), (128, 5, 1)])
def test_attention_prompt_portions_on_tcgen05(ops, hd, nh, nkv):
    """Prompt portions with pages of 64 and 128 keys (the tcgen05 kernel's
    shapes): long portions that wrap its ring of key blocks, portions that
    start mid-sequence, row counts that are no multiple of its 128-row tile,
    a decode token beside them, windows shorter and longer than a key block;
    and a far key and a window's edge made to stand out in a long portion."""
    for page in (64, 128):
        for window in (None, 70, 333):
            rng = np.random.default_rng(hd + page)
            lens, q_lens = [1000, 130, 64, 777, 129], [700, 130, 1, 777, 2]
            got, want = attention_case(ops, BF16, hd, nh, nkv, lens=lens, q_lens=q_lens, page=page, window=window, rng=rng, fast=True)
            assert_close(got, want, TOL[BF16], f"hd={hd} page={page} window={window}")
    for far in (0, 127, 128, 500, 895):
        rng = np.random.default_rng(far)

        def craft(qs, ks, vs, far=far):
            direction = rng.normal(size=hd)
            direction /= np.linalg.norm(direction)
            qs[0][-1, :] = np.tile(12.0 * direction, nh)
            qs[0][-300, :] = np.tile(12.0 * direction, nh)
            ks[0][far, :] = np.tile(12.0 * direction, nkv)
            vs[0][far, :] = 100.0

        got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[900], q_lens=[400], page=64, window=None, rng=rng, craft=craft, fast=True)
        assert (np.abs(want[-1]).min() > 90.0) and ((np.abs(want[-300]).min() > 90.0) == (far <= 600))
        # the two rows made for it; rows that see the value of 100 by chance are only as exact as
        # bfloat16 weights times 100 can be, which the bound of the random cases does not describe
        assert_close(got[[-1, -300]], want[[-1, -300]], TOL[BF16], f"far key at {far}")
    for window in (1, 128, 129, 200):
        for offset, seen in ((window - 1, True), (window, False)):
            rng = np.random.default_rng(window)

            def craft(qs, ks, vs, offset=offset):
                direction = np.ones(hd) / np.sqrt(hd)
                qs[0][-1, :] = np.tile(14.0 * direction, nh)
                ks[0][599 - offset, :] = np.tile(14.0 * direction, nkv)
                vs[0][599 - offset, :] = 50.0

            got, want = attention_case(ops, BF16, hd, nh, nkv, lens=[600], q_lens=[300], page=64, window=window, rng=rng, craft=craft, fast=True)
            assert (np.abs(want[-1]).min() > 45.0) == seen
            assert_close(got[-1:], want[-1:], TOL[BF16], f"window {window} offset {offset}")


def test_attention_rows_do_not_depend_on_the_batch(ops):
    """The same query gives the same bits alone or among other requests, and
    whatever the page size and the pages are."""
    rng = np.random.default_rng(5)
    hd, nh, nkv, lens = 48, 6, 2, [200, 77, 301]
    ks = [rounded(rng.normal(size=(n, nkv * hd)), F32) for n in lens]
    vs = [rounded(rng.normal(size=(n, nkv * hd)), F32) for n in lens]
    qs = [rounded(rng.normal(size=(n, nh * hd)), F32) for n in lens]
    first = ([qs[0]], [ks[0]], [vs[0]])
    alone16, want = attention_case(ops, F32, hd, nh, nkv, [200], [3], 16, None, np.random.default_rng(1), given=first)
    alone64, _ = attention_case(ops, F32, hd, nh, nkv, [200], [3], 64, None, np.random.default_rng(2), given=first)
    mixed, _ = attention_case(ops, F32, hd, nh, nkv, lens, [3, 77, 1], 16, None, np.random.default_rng(3), given=(qs, ks, vs))
    assert_close(alone16, want, TOL[F32])
    assert np.array_equal(alone16, alone64) and np.array_equal(alone16, mixed[:3])


def test_sample_greedy_ties_and_temperature(ops):
    rng = np.random.default_rng(6)
    V = 1187
    logits = rng.normal(size=(6, V)).astype(np.float32)
    logits[0, [5, 900]] = 9.0  # a tie at the top goes to the lower index
    logits[1, V - 1] = 8.0
    tokens = torch.empty(6, dtype=torch.int32, device="cuda")
    ops.sample(tokens, dev(logits), dev(np.zeros(6, dtype=np.float32)), dev(np.zeros(6, dtype=np.float32)))
    assert tokens.cpu().tolist() == [int(np.argmax(r)) for r in logits] and tokens[0] == 5 and tokens[1] == V - 1
    temps = np.array([0.01, 0.5, 1.0, 1.0, 2.0, 0.0], dtype=np.float32)
    us = np.array([0.3, 0.3, 0.0, 0.999999, 0.5, 0.4], dtype=np.float32)  # row 0: two tied maxima, u below one half picks the first
    ops.sample(tokens, dev(logits), dev(temps), dev(us))
    got = tokens.cpu().tolist()
    staged = torch.empty(6, dtype=torch.int32, device="cuda")  # the two-stage form gives the same tokens
    ops.sample(staged, dev(logits), dev(temps), dev(us), torch.empty(2 * 6 * ops.ARGMAX_PARTS, device="cuda"), True)
    assert staged.cpu().tolist() == got
    ops.sample(staged, dev(logits), dev(np.zeros(6, dtype=np.float32)), dev(us), torch.empty(2 * 6 * ops.ARGMAX_PARTS, device="cuda"), False)
    assert staged.cpu().tolist() == [int(np.argmax(r)) for r in logits]
    assert got[0] == 5 and got[5] == int(np.argmax(logits[5]))  # tiny temperature = greedy
    for r in range(1, 5):
        dist = plain.sample_distribution(logits[r], temperature=float(temps[r]))
        cdf = np.cumsum(dist)
        lo = cdf[got[r] - 1] if got[r] else 0.0
        assert lo - 1e-5 <= us[r] < cdf[got[r]] + 1e-5, f"row {r}: {got[r]} is not where the CDF passes u"


@pytest.mark.parametrize("vocab", [379, 5000])
def test_sample_chain_against_plain(ops, vocab):
    from alofa_b200.sampling.params import SamplingParams
    from alofa_b200.sampling.sampler import sample_chain_rows

    rng = np.random.default_rng(vocab)
    rows, logits, want = [], [], []
    for trial in range(64):
        x = rng.normal(0, 2, size=vocab).astype(np.float32)
        if trial % 4 == 0:
            x[rng.integers(0, vocab, 40)] = x[0]  # ties
        p = SamplingParams(
            temperature=float(rng.choice([0.0, 0.5, 1.0, 1.7])), top_k=int(rng.choice([0, 1, 5, 50])), top_p=float(rng.choice([1.0, 0.9, 0.5, 0.1])),
            min_p=float(rng.choice([0.0, 0.05, 0.3])), repetition_penalty=float(rng.choice([1.0, 1.3])), frequency_penalty=float(rng.choice([0.0, 0.2])),
            presence_penalty=float(rng.choice([0.0, 0.4])), min_tokens_to_keep=int(rng.choice([1, 1, 3])), logit_bias={int(rng.integers(vocab)): 2.5} if trial % 3 == 0 else {},
        )
        hist = [int(t) for t in rng.integers(0, vocab, 30)]
        u = float(rng.random())
        dist = plain.sample_distribution(x, hist, p.temperature, p.top_k, p.top_p, p.min_p, p.repetition_penalty, p.frequency_penalty, p.presence_penalty, p.min_tokens_to_keep, list(p.logit_bias.items()))
        rows.append((p, u, hist))
        logits.append(x)
        want.append((plain.pick_from(dist, u), dist, u))
    got = sample_chain_rows(dev(np.stack(logits)), rows).cpu().tolist()
    for g, (w, dist, u) in zip(got, want):
        if g != w:  # allowed only when u sits within fp32 rounding of a CDF step
            cdf = np.cumsum(dist)
            assert dist[g] > 0 and min(abs(u - cdf[w]), abs(u - (cdf[w - 1] if w else 0.0))) < 1e-5, (g, w)
