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


@pytest.mark.parametrize("bucket", [256, 512, 1024, 4096, 8192])
@pytest.mark.parametrize("blocks", [1, 4, 32, 48, 96, 128, 160, 256, 1000])
@pytest.mark.parametrize("tcgen05", [True, False])
def test_decode_chunks_divide_the_bucket(blocks, bucket, tcgen05):
    chunk = tensor_core.decode_chunk_keys(blocks, bucket, tcgen05)
    assert 256 <= chunk <= bucket and bucket % chunk == 0
    if tcgen05 and chunk >= 512:
        assert chunk * 2 != bucket                  # never one full chunk and a scrap


def test_decode_chunks_of_the_benchmark_points():
    # 4 KV heads, contexts of 2,048 to 2,304 tokens (bucket 4,096)
    assert tensor_core.decode_chunk_keys(1 * 4, 4096, True) == 256
    assert tensor_core.decode_chunk_keys(8 * 4, 4096, True) == 512
    assert tensor_core.decode_chunk_keys(24 * 4, 4096, True) == 1024
    assert tensor_core.decode_chunk_keys(32 * 4, 4096, True) == 1024
    assert tensor_core.decode_chunk_keys(64 * 4, 4096, True) == 4096
