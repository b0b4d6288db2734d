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
