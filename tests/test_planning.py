"""How the tensor-core product is tiled and its depth split, from sizes alone
(no GPU): the choices must be functions of (tokens, weight shape) only, stay
inside what the kernel takes, and never leave a split empty."""
import itertools

import pytest

from alofa_b200.parts import fast_linear as fl


SIZES = [(896, 896), (1152, 896), (9728 // 2, 896), (896, 4864), (151936, 896),  # the 0.5B shape
         (1536, 1536), (2048, 1536), (8960, 1536), (1536, 8960),  # the 1.5B shape
         (3584, 3584), (4608, 3584), (18944, 3584), (3584, 18944), (152064, 3584),  # the 7B shape
         (379, 96), (131, 512)]
TOKENS = [1, 7, 8, 16, 17, 32, 33, 64, 65, 128, 300, 2048]


def real_splits(depth, splits):
    """What the kernel makes of a wanted split count: slices per split rounded
    up, then no empty split (the arithmetic of alofa_gemm_tc_splits)."""
    total = -(-depth // fl.K_SLICE)
    splits = max(1, min(splits, total))
    per = -(-total // splits)
    return -(-total // per)


@pytest.mark.parametrize("gated", [False, True])
def test_tiles_are_ones_the_kernel_has(gated):
    for (features, depth), tokens in itertools.product(SIZES, TOKENS):
        tile = fl._tile(tokens, features, gated)
        if tile > 0:
            assert tile in (16, 32, 64) and tokens <= 64 and tile >= min(tokens, 64)
        else:
            assert tile in (-128, -256)
            if gated:
                assert tile == -256  # 128 gate rows beside their 128 up rows
        assert fl._tile(tokens, features, gated) == tile  # a function of the sizes alone


def test_few_tokens_keep_the_weights_on_m_except_for_a_very_tall_weight():
    assert fl._tile(8, 896, False) == 16
    assert fl._tile(8, 4864, True) == 16
    assert fl._tile(8, 151936, False) == -256  # an output head: wide tiles stream it faster
    assert fl._tile(64, 896, False) == 64
    assert fl._tile(65, 896, False) == -128  # narrow output: 128-wide tiles keep more SMs busy
    assert fl._tile(2048, 151936, False) == -256


def test_splits_fill_the_gpu_once_and_leave_no_split_empty():
    for (features, depth), tokens, gated in itertools.product(SIZES, TOKENS, (False, True)):
        tile = fl._tile(tokens, features, gated)
        ctas = fl._ctas(tokens, features, tile, gated)
        assert ctas >= 1
        for deferrable in (False, True):
            splits = fl._splits(ctas, depth, deferrable)
            slices = -(-depth // fl.K_SLICE)
            assert 1 <= splits <= max(1, slices)
            real = real_splits(depth, splits)
            assert 1 <= real <= splits
            per = -(-slices // real)
            assert per * (real - 1) < slices  # the last split has at least one slice
            if ctas < fl.SMS // 2 and slices >= 2:
                assert ctas * splits <= fl.SMS  # one wave
            if ctas >= fl.SMS:
                assert splits == 1


def test_a_deep_product_that_underfills_the_gpu_is_halved_only_for_a_consumer_that_adds():
    # down projection of a 2,048-token prompt: 7 x 16 = 112 CTAs, 76 slices deep
    tile = fl._tile(2048, 896, False)
    ctas = fl._ctas(2048, 896, tile, False)
    assert (tile, ctas) == (-128, 112)
    assert fl._splits(ctas, 4864, deferrable=True) == 2
    assert fl._splits(ctas, 4864, deferrable=False) == 1
    assert fl._splits(ctas, 896, deferrable=True) == 1  # shallow: not worth a second pass


def test_decode_attention_splits_keep_a_step_resident_at_once():
    """Keys per CTA of a decode-only step (GQAttention.decode_split_keys), for
    a device of 148 SMs: head size 64 has the eight-warp kernel (148 CTAs at a
    time, splits in multiples of 512), head size 128 the four-warp one only
    (148 CTAs, multiples of 256)."""
    from alofa_b200.parts.attention import GQAttention as A

    def keys(n_tokens, pairs, longest, now, wide=148, slots=444):
        return A.decode_split_keys(n_tokens, pairs, longest, now, wide, slots)

    # 14 heads on 2 (pairs = 2 x requests), contexts of 2,049 in a bucket of 4,096
    assert keys(1, 2, 4096, 2049) == 512
    assert keys(8, 16, 4096, 2049) == 512  # five splits x 16 pairs = 80 CTAs, one per SM
    assert keys(12, 24, 4096, 2049) == 512  # 120 CTAs
    assert keys(16, 32, 4096, 2049) == 1024  # 96 CTAs where 160 would not be resident together
    assert keys(17, 34, 4096, 2049) == 1024
    assert keys(24, 48, 4096, 2049) == 4096  # 0.3 pairs per SM and more, past 16 tokens: one split per pair
    assert keys(64, 128, 4096, 2049) == 4096
    assert keys(8, 16, 256, 200) == 512  # one split reaches to the end of the bucket: nothing to merge
    # few tokens keep at most 16 splits for the output product to merge, up to 16k keys
    assert keys(1, 2, 16384, 16000) == 1024 and -(-16384 // 1024) == 16
    assert keys(1, 2, 32768, 32000) == 512  # beyond that the merge kernel takes them, as many as are resident
    # 28 heads of 128 on 4: no eight-warp kernel, 148 CTAs of four warps at a time
    assert keys(8, 32, 4096, 2049, wide=0, slots=148) == 768  # three splits x 32 pairs
    assert keys(64, 256, 4096, 2049, wide=0, slots=148) == 4096  # more pairs than SMs: one split each
    assert keys(1, 4, 4096, 2049, wide=0, slots=148) == 256
    # the same head size with its six-warp form (splits in multiples of 384 keys, 148 CTAs at a time)
    wide128 = dict(wide_slots=148, slots=148, wide_unit=384)
    assert A.decode_split_keys(8, 32, 4096, 2049, **wide128) == 768  # six blocks of 384 over four resident splits: two each
    assert A.decode_split_keys(64, 256, 4096, 2049, **wide128) == 4224  # one split, the bucket rounded up to 384s
    assert A.decode_split_keys(1, 4, 4096, 2049, **wide128) == 384
    # every answer covers the launch in whole units and never asks for an empty split first
    for n, pairs, longest, now, wide, slots in itertools.product((1, 8, 16, 17, 40, 64), (1, 7, 64, 300), (256, 4096, 65536), (1, 200, 4000), (0, 148), (148, 444)):
        if now > longest:
            continue
        k = A.decode_split_keys(n, pairs, longest, now, wide, slots)
        unit = 512 if wide else 256
        assert k % unit == 0 and k >= unit and k <= unit * -(-longest // unit)
        if n <= 16 and longest <= 16384:
            assert -(-longest // k) <= 16
