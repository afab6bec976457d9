"""Host-side shape policies of the GEMM launcher (no device needed): the tile width of the one-CTA
kernel, the number of K ranges of the fp32-sum GEMMs that feed a LayerNorm, and when the SM-pair
kernel takes over.  The expected values restate the rules in words; the numbers are for 148 SMs."""
import ctypes as C

import pytest

SMS = 148


@pytest.fixture(scope="module")
def policy():
    from bytetransformer_b200 import _abi, build
    build.build_core()  # no-op when the library is up to date
    lib = _abi.load()
    fn = lib.bt_debug_policy
    fn.restype = C.c_int
    fn.argtypes = [C.c_int] * 5
    return fn


@pytest.mark.parametrize("rows,N,want", [
    (64, 2304, 64),      # never 148 tiles: the narrowest width spreads the weights over most SMs
    (4096, 768, 128),    # 32 row tiles x 3 = 96 tiles of 256 columns, 192 of 128: the widest that fills the SMs
    (18944, 3072, 256),
    (2560, 3072, 256),   # 20 x 12 = 240 tiles
    (128, 192, 64),      # 192 % 128 != 0
])
def test_tile_width_is_the_widest_that_gives_every_sm_a_tile(policy, rows, N, want):
    assert policy(0, rows, N, 768, SMS) == want


@pytest.mark.parametrize("rows,K,want", [
    (38, 3072, 8), (256, 3072, 8),        # 12 or 24 tiles of 64 columns: 8 ranges still fit 1.5 x the SMs
    (384, 3072, 4), (512, 3072, 4),
    (640, 3072, 2), (1024, 3072, 2),
    (1280, 3072, 1),                      # 120 tiles: even two ranges would be more than 1.5 x the SMs
    (38, 768, 4),                         # 12 K blocks: 8 does not divide them, 4 leaves three blocks per range
    (512, 768, 4), (640, 768, 2),
    (38, 128, 1),                         # two K blocks: nothing to cut
])
def test_k_is_cut_into_as_many_ranges_as_still_fit_the_machine(policy, rows, K, want):
    assert policy(1, rows, 768, K, SMS) == want


@pytest.mark.parametrize("rows,N,want", [
    (18944, 2304, 1), (4352, 2304, 1),    # 17 x 9 = 153 pair tiles >= 148
    (4096, 2304, 0),                      # 16 x 9 = 144
    (18944, 2240, 0),                     # N % 256 != 0
])
def test_pair_kernel_takes_over_at_two_tiles_per_sm_pair(policy, rows, N, want):
    assert policy(2, rows, N, 768, SMS) == want
