"""Helpers of the GPU tests: paged caches from whole sequences, tolerances."""
import numpy as np
import torch


def dev(x, dtype=None):
    t = torch.as_tensor(np.asarray(x))
    if dtype is not None:
        t = t.to(dtype)
    return t.cuda().contiguous()


def rounded(x, dtype):
    """Values as the kernel sees them: rounded to ``dtype``, back in float64."""
    return torch.as_tensor(np.asarray(x)).to(dtype).to(torch.float64).numpy()


def paged_from_sequences(ks, vs, page_size, nkv, hd, dtype, rng, extra_pages=3):
    """Scatter per-sequence keys/values [n_i, nkv*hd] into one paged cache
    through random, non-ascending block tables.  Returns (k_cache, v_cache,
    block_table [n_seqs, max_blocks] int32 tensor)."""
    blocks = [-(-len(k) // page_size) for k in ks]
    total = sum(blocks) + extra_pages
    order = rng.permutation(total)
    max_blocks = max(blocks) + 1
    table = np.full((len(ks), max_blocks), -1, dtype=np.int32)
    k_cache = np.full((total * page_size, nkv, hd), 7.0)  # garbage in unused slots must not matter
    v_cache = np.full((total * page_size, nkv, hd), -7.0)
    at = 0
    for s, (k, v) in enumerate(zip(ks, vs)):
        for b in range(blocks[s]):
            page = int(order[at])
            at += 1
            table[s, b] = page
            lo, hi = b * page_size, min((b + 1) * page_size, len(k))
            k_cache[page * page_size : page * page_size + hi - lo] = np.asarray(k[lo:hi]).reshape(hi - lo, nkv, hd)
            v_cache[page * page_size : page * page_size + hi - lo] = np.asarray(v[lo:hi]).reshape(hi - lo, nkv, hd)
    return dev(k_cache, dtype), dev(v_cache, dtype), dev(table)


def assert_close(got, want, tol, what=""):
    got = np.asarray(got, dtype=np.float64)
    want = np.asarray(want, dtype=np.float64)
    assert got.shape == want.shape, f"{what}: shape {got.shape} vs {want.shape}"
    bound = tol * max(1.0, float(np.abs(want).max()))
    diff = float(np.abs(got - want).max())
    assert diff <= bound, f"{what}: max |diff| {diff:.3e} > {bound:.3e}"
