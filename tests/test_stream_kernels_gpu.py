"""The kernels behind the residual stream of small decode steps, each alone
against fp64: residual products that add their split sums into a 64-bit
fixed-point accumulator (the same bits every run, whatever order the CTAs
finish in), the gate/up and q/k/v products that make their own operand from
base + accumulator with the RMSNorm folded in, and the kernels that bring the
stream back to one tensor."""
import numpy as np
import pytest
import torch

import plain_qwen2 as plain
from gpu_util import assert_close, dev, rounded

pytestmark = pytest.mark.gpu

F32, BF16 = torch.float32, torch.bfloat16
SCALE = 4294967296.0


@pytest.fixture(scope="module")
def ops():
    from alofa_b200.csrc import ops

    return ops


def acc_of(values):
    """float values as the accumulator holds them."""
    return torch.from_numpy(np.rint(np.asarray(values, dtype=np.float64) * SCALE).astype(np.int64)).cuda()


@pytest.mark.parametrize("m, n, k, splits", [(8, 896, 4864, 19), (1, 896, 896, 7), (16, 131, 512, 8), (5, 200, 64, 1), (13, 379, 320, 3)])
def test_residual_product_adds_into_the_accumulator(ops, m, n, k, splits):
    rng = np.random.default_rng(m + n + k)
    x = rounded(rng.normal(size=(m, k)), BF16)
    w = rounded(rng.normal(size=(n, k)) / np.sqrt(k), BF16)
    bias = rng.normal(size=n).astype(np.float32)
    want = plain.linear(x, w, bias)
    seen = []
    for run in range(3):
        acc = torch.zeros(m, n, dtype=torch.int64, device="cuda")
        h = torch.full((m, n), 7.0, device="cuda")
        assert ops.gemm_tc(h, dev(x, BF16), dev(w, BF16), dev(bias), ops.EPI_RESIDUAL, 16, splits, None, acc=acc)
        assert torch.all(h == 7.0), "the product must write the accumulator only"
        assert_close(acc.cpu().numpy() / SCALE, want, 2e-5, f"accumulated product, run {run}")
        seen.append(acc.clone())
    assert torch.equal(seen[0], seen[1]) and torch.equal(seen[0], seen[2]), "integer adds must give the same bits in any order"
    again = seen[0].clone()
    assert ops.gemm_tc(h, dev(x, BF16), dev(w, BF16), None, ops.EPI_RESIDUAL, 16, splits, None, acc=again)  # on top of what is there
    assert_close(again.cpu().numpy() / SCALE, want + plain.linear(x, w), 4e-5, "a second product on top")


def test_output_product_merges_key_splits_into_the_accumulator(ops):
    """The merged-splits operand (attention output still in key splits) feeding
    a product that adds into the accumulator: the two new pieces together."""
    rng = np.random.default_rng(3)
    t, nh, hd, n_splits, split_keys = 5, 4, 64, 3, 256
    positions = np.array([10, 300, 600, 767, 520], dtype=np.int32)
    po = rng.normal(size=(n_splits, t * nh, hd)).astype(np.float32)
    pml = np.stack([rng.normal(size=(n_splits, t * nh)), rng.uniform(0.5, 2.0, size=(n_splits, t * nh))], axis=-1).astype(np.float32)
    for i, p in enumerate(positions):  # splits past the token's position hold nothing
        for s in range(n_splits):
            if s * split_keys > p:
                pml[s, i * nh : (i + 1) * nh, 0] = -np.inf
                pml[s, i * nh : (i + 1) * nh, 1] = 0.0
    m = pml[..., 0].max(axis=0)
    wgt = np.where(np.isfinite(pml[..., 0]), np.exp2(pml[..., 0] - m), 0.0)
    merged = ((po * wgt[..., None]).sum(axis=0) / (pml[..., 1] * wgt).sum(axis=0)[:, None]).reshape(t, nh * hd)
    w = rounded(rng.normal(size=(200, nh * hd)) / 16, BF16)
    acc = torch.zeros(t, 200, dtype=torch.int64, device="cuda")
    out = torch.zeros(t, 200, device="cuda")
    computed = (ops.B_MERGED_SPLITS, dev(po), dev(pml), dev(positions), nh, hd, None, split_keys)
    assert ops.gemm_tc(out, None, dev(w, BF16), None, ops.EPI_RESIDUAL, 16, 4, None, computed=computed, acc=acc)
    assert_close(acc.cpu().numpy() / SCALE, plain.linear(rounded(merged, BF16), w), 6e-3, "merged splits into the accumulator")


def stream_sum(base, owed):
    """base + accumulator as the kernels take it (common.cuh, stream_add): the
    accumulator split into the nearest whole number and a signed fraction, the
    whole part added to the base first, the fraction after, all in fp32; the
    result as float64."""
    acc = np.rint(np.asarray(owed, dtype=np.float64) * SCALE).astype(np.int64)
    whole = (acc + (1 << 31)) >> 32
    fraction = (acc - (whole << 32)).astype(np.int32).astype(np.float32) * np.float32(1.0 / SCALE)
    return ((np.asarray(base, dtype=np.float32) + whole.astype(np.float32)) + fraction).astype(np.float64)


def stream_inputs(rng, t, k, with_acc):
    base = rng.normal(size=(t, k)).astype(np.float32)
    owed = rng.normal(size=(t, k)) * 0.3 if with_acc else np.zeros((t, k))
    gamma = (1 + 0.1 * rng.normal(size=k)).astype(np.float32)
    stream = stream_sum(base, owed)
    exact = base.astype(np.float64) + np.rint(owed * SCALE) / SCALE
    small = np.abs(owed) < 0.49
    assert (np.abs(stream - exact)[small] <= (2.0 ** -24 * np.maximum(1.0, np.abs(exact)) + 2.0 ** -26)[small]).all()  # rounded once, and the fraction's own rounding
    assert (np.abs(stream - exact) <= 2.0 ** -22 * np.maximum(1.0, np.abs(exact))).all()  # two roundings where the accumulator has a whole part
    return base, owed, gamma, stream


@pytest.mark.parametrize("t, n, k, splits", [(8, 4864, 896, 3), (1, 640, 320, 5), (16, 131, 512, 8), (13, 200, 64, 1), (7, 256, 200, 2)])
@pytest.mark.parametrize("with_acc", [True, False])
def test_gated_product_folds_the_norm_in(ops, t, n, k, splits, with_acc):
    rng = np.random.default_rng(t + n + k)
    base, owed, gamma, stream = stream_inputs(rng, t, k, with_acc)
    eps = 1e-5
    w = rounded(rng.normal(size=(2 * n, k)) / np.sqrt(k), BF16)
    # the kernel rounds (stream * gamma) to bfloat16 and applies the row's factor to the sums
    rstd = 1.0 / np.sqrt((stream * stream).mean(axis=1, keepdims=True) + eps)
    x = rounded(stream * gamma, BF16)
    want = plain.silu(plain.linear(x, w[:n]) * rstd) * (plain.linear(x, w[n:]) * rstd)
    exact = plain.rmsnorm(stream, gamma, eps)
    want_exact = plain.silu(plain.linear(exact, w[:n])) * plain.linear(exact, w[n:])
    acc = acc_of(owed) if with_acc else None
    other = torch.full((t, k), 5, dtype=torch.int64, device="cuda")
    new_base = torch.zeros(t, k, device="cuda")
    out = torch.empty(t, n, dtype=BF16, device="cuda")
    computed = (ops.B_NORMED, dev(base), acc, dev(gamma), eps, new_base, other)
    assert ops.gemm_tc(out, None, dev(w, BF16), None, ops.EPI_GATED, 16, splits, None, computed=computed)
    assert_close(out.float().cpu(), want, 6e-3, "gated product of the normed stream")
    assert_close(out.float().cpu(), want_exact, 2e-2, "against the norm applied before rounding")
    assert np.array_equal(new_base.cpu().numpy().astype(np.float64), stream), "the stream's new base is base + accumulator"
    assert int(other.abs().sum()) == 0, "the accumulator that was not read is cleared"
    if with_acc:
        assert torch.equal(acc, acc_of(owed)), "the accumulator that was read is left as it was"


@pytest.mark.parametrize("hd, nh, nkv, k", [(64, 14, 2, 896), (32, 3, 1, 96), (128, 4, 2, 512), (64, 3, 0, 192), (16, 5, 5, 64)])
def test_qkv_product_folds_the_norm_in(ops, hd, nh, nkv, k):
    from alofa_b200.config.spec import PartSpec
    from alofa_b200.parts.base import Runtime
    from alofa_b200.parts.position import RotaryNeox

    rng = np.random.default_rng(hd + k)
    table = RotaryNeox(PartSpec("rotary_neox", {"head_dim": hd, "theta": 1e4, "max_position": 900}), Runtime(torch.device("cuda"), BF16)).build_table(900)
    C = (nh + 2 * nkv) * hd
    w = rounded(rng.normal(size=(C, k)) / np.sqrt(k), BF16)
    bias = rng.normal(size=C).astype(np.float32)
    eps = 1e-6
    for n in (1, 7, 16):
        base, owed, gamma, stream = stream_inputs(rng, n, k, True)
        rstd = 1.0 / np.sqrt((stream * stream).mean(axis=1, keepdims=True) + eps)
        qkv = plain.linear(rounded(stream * gamma, BF16), w) * rstd + bias
        positions = rng.integers(0, 900, n).astype(np.int32)
        slots = rng.permutation(40)[:n].astype(np.int32)
        for splits in (1, 8):
            kc = torch.full((40, max(nkv, 1), hd), 3.0, dtype=BF16, device="cuda")
            vc = torch.full((40, max(nkv, 1), hd), 3.0, dtype=BF16, device="cuda")
            q_out = torch.empty(n, nh * hd, dtype=BF16, device="cuda")
            other = torch.full((n, k), -9, dtype=torch.int64, device="cuda")
            new_base = torch.zeros(n, k, device="cuda")
            normed = (dev(base), acc_of(owed), dev(gamma), eps, new_base, other)
            assert ops.gemm_tc_rope(None, dev(w, BF16), dev(bias), q_out, kc, vc, dev(slots), dev(positions), table, nh, nkv, hd, splits, normed=normed)
            q, kk, vv = qkv[:, : nh * hd], qkv[:, nh * hd : (nh + nkv) * hd], qkv[:, (nh + nkv) * hd :]
            assert_close(q_out.float().cpu(), plain.rope(q, positions, nh, hd, 1e4), 6e-3, f"q n={n} splits={splits}")
            if nkv:
                want_k, want_v = np.full((40, nkv * hd), 3.0), np.full((40, nkv * hd), 3.0)
                rk = plain.rope(kk, positions, nkv, hd, 1e4)
                for t, s_ in enumerate(slots):
                    want_k[s_], want_v[s_] = rk[t], vv[t]
                assert_close(kc.float().cpu().reshape(40, -1), want_k, 6e-3, f"k n={n} splits={splits}")
                assert_close(vc.float().cpu().reshape(40, -1), want_v, 6e-3, f"v n={n} splits={splits}")
            assert np.array_equal(new_base.cpu().numpy().astype(np.float64), stream) and int(other.abs().sum()) == 0


@pytest.mark.parametrize("out_dtype", [F32, BF16])
def test_norm_kernel_and_settle_read_base_plus_accumulator(ops, out_dtype):
    rng = np.random.default_rng(9)
    t, k = 11, 896
    base, owed, gamma, stream = stream_inputs(rng, t, k, True)
    want = plain.rmsnorm(stream, gamma, 1e-6)
    for moved in (False, True):
        h = torch.full((t, k), 4.0, device="cuda") if moved else dev(base)
        acc, other = acc_of(owed), torch.full((t, k), 3, dtype=torch.int64, device="cuda")
        out = torch.empty(t, k, dtype=out_dtype, device="cuda")
        assert ops.norm_fused(out, h, dev(gamma), 1e-6, None, base=dev(base) if moved else None, acc=acc, other=other)
        assert_close(out.float().cpu(), want, 1e-5 if out_dtype == F32 else 6e-3, f"norm, base moved={moved}")
        assert np.array_equal(h.cpu().numpy().astype(np.float64), stream) and int(acc.abs().sum()) == 0 and int(other.abs().sum()) == 0
    # with split sums left as planes on top of a moved base
    planes = rng.normal(size=(5, t, k)).astype(np.float32)
    h = torch.zeros(t, k, device="cuda")
    out = torch.empty(t, k, dtype=out_dtype, device="cuda")
    assert ops.norm_fused(out, h, dev(gamma), 1e-6, None, dev(planes), 5, None, base=dev(base))
    total = base.astype(np.float64) + planes.astype(np.float64).sum(axis=0)
    assert_close(h.cpu(), total, 1e-5, "planes on a moved base")
    assert_close(out.float().cpu(), plain.rmsnorm(total, gamma, 1e-6), 1e-5 if out_dtype == F32 else 6e-3, "norm of it")
    # settle alone
    h = torch.zeros(t, k, device="cuda")
    acc, other = acc_of(owed), torch.full((t, k), 3, dtype=torch.int64, device="cuda")
    ops.stream_settle(h, dev(base), acc, other)
    assert np.array_equal(h.cpu().numpy().astype(np.float64), stream) and int(acc.abs().sum()) == 0 and int(other.abs().sum()) == 0
