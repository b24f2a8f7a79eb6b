"""Rules that choose a kernel's shape from the problem's sizes (no GPU needed)."""
import pytest

from crucible_b200.ops import tensor_core


@pytest.mark.parametrize("m", [33, 64, 128, 200, 512, 2048])
@pytest.mark.parametrize("n", [96, 768, 1280, 4096, 50304])
@pytest.mark.parametrize("k", [64, 136, 768, 2048, 8192, 14336])
def test_shares_of_k_leave_no_share_empty_and_fit_the_sms(m, n, k):
    for bn in tensor_core.TILE_WIDTHS:
        s = tensor_core.k_splits(m, n, k, bn)
        tiles = -(-m // 128) * -(-n // bn)
        k_blocks = -(-k // 64)
        assert 1 <= s <= 4
        if s > 1:
            assert tiles * s <= tensor_core.N_SMS
            per = -(-k_blocks // s)
            assert (s - 1) * per < k_blocks                      # the last share has work
            assert k_blocks >= 16                                # a short K is never worth a cluster


def test_large_products_are_not_split():
    assert tensor_core.k_splits(2048, 768, 2048, 96) == 1
    assert tensor_core.k_splits(64, 768, 128, 64) == 1
    assert tensor_core.k_splits(64, 768, 768, 64) == 1
    assert tensor_core.k_splits(64, 768, 2048, 64) == 4
    assert tensor_core.k_splits(64, 2048, 8192, 64) == 4
    assert tensor_core.k_splits(512, 768, 2048, 64) == 2


def test_tall_tiles_only_where_they_fill_the_sms():
    assert tensor_core._tall_tiles(2048, 28672, 4096)          # Llama-3-8B gate/up
    assert tensor_core._tall_tiles(2048, 4096, 14336)          # ... down: 128 tiles of 256 x 256
    assert not tensor_core._tall_tiles(2048, 2048, 8192)       # Llama-3.2-1B down: 64 tiles
    assert tensor_core._tall_tiles(2048, 4096, 768)            # the 120M shape's gate/up: 128 tiles
    assert not tensor_core._tall_tiles(2048, 768, 2048)        # ... its down projection: 24 tiles
    assert not tensor_core._tall_tiles(512, 28672, 4096)
