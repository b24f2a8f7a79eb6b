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


@pytest.mark.parametrize("bucket", [256, 512, 768, 1024, 2304, 4096, 8192, 8448])
@pytest.mark.parametrize("blocks", [1, 4, 32, 48, 96, 128, 160, 256, 1000])
@pytest.mark.parametrize("tcgen05, head_dim", [(True, 64), (True, 128), (False, 64)])
def test_decode_chunks_cover_the_bucket_in_whole_tiles(blocks, bucket, tcgen05, head_dim):
    unit = 128 if tcgen05 else 256
    chunk = tensor_core.decode_chunk_keys(blocks, bucket, tcgen05, head_dim)
    assert unit <= chunk <= -(-bucket // unit) * unit and chunk % unit == 0
    n_chunks = -(-bucket // chunk)
    assert (n_chunks - 1) * chunk < bucket <= n_chunks * chunk     # no chunk is empty
    target = tensor_core.DECODE_TC_TARGET_BLOCKS if tcgen05 else tensor_core.DECODE_MMA_TARGET_BLOCKS
    # never far more blocks than fit at once unless a chunk is already a single tile
    assert blocks * n_chunks <= max(1.5 * target, tensor_core.DECODE_TC_SHORT_BLOCKS, blocks) or chunk == unit


def test_decode_chunks_of_the_benchmark_points():
    # 4 KV heads, contexts of 2,056 to 2,304 tokens (bucket 2,304)
    assert tensor_core.decode_chunk_keys(1 * 4, 2304, True) == 256         # 9 chunks, 36 blocks
    assert tensor_core.decode_chunk_keys(4 * 4, 2304, True) == 256         # 9 chunks, 144 blocks
    assert tensor_core.decode_chunk_keys(8 * 4, 2304, True) == 256         # 9 chunks, 288 blocks, three to an SM
    assert tensor_core.decode_chunk_keys(8 * 4, 768, True) == 128          # short contexts: a tile per block
    assert tensor_core.decode_chunk_keys(8 * 4, 3840, True) == 640         # 480 blocks of two tiles would not fit
    assert tensor_core.decode_chunk_keys(16 * 4, 2304, True) == 768        # 3 chunks, 192 blocks
    assert tensor_core.decode_chunk_keys(32 * 4, 2304, True) == 1152       # 2 chunks, 256 blocks
    assert tensor_core.decode_chunk_keys(64 * 4, 2304, True) == 2304       # a block per request and KV head
    # heads of 128 features, 8 KV heads: one block to an SM, so never more blocks than SMs
    assert tensor_core.decode_chunk_keys(1 * 8, 2304, True, 128) == 256    # 9 chunks, 72 blocks
    assert tensor_core.decode_chunk_keys(2 * 8, 2304, True, 128) == 256    # 9 chunks, 144 blocks
    assert tensor_core.decode_chunk_keys(4 * 8, 2304, True, 128) == 640    # 4 chunks, 128 blocks
    assert tensor_core.decode_chunk_keys(8 * 8, 2304, True, 128) == 1152   # 2 chunks, 128 blocks
    assert tensor_core.decode_chunk_keys(16 * 8, 2304, True, 128) == 2304  # a block per request and KV head


def test_step_shape_key_follows_what_launches_depend_on():
    from crucible_b200.engine.context import HostStep
    decode = HostStep(list("abc"), [1, 1, 1], [2100, 300, 40], [2101, 301, 41], [0, 1, 2])
    assert decode.context_bucket == 2304 and decode.lead_single == 3
    assert decode.shape_key() == (1, 3, 2304, 2304)
    mixed = HostStep(list("abc"), [1, 1, 500], [2100, 300, 4000], [2101, 301, 4500], [0, 1, 2])
    # the portion's own context does not enter the key: the tile kernels walk it from metadata
    assert mixed.shape_key() == (500, 2, 0, 2304)
    assert mixed.lead_context_bucket == 2304 and mixed.context_bucket == 4608
    later = HostStep(list("abc"), [1, 1, 500], [2101, 301, 4500], [2102, 302, 5000], [0, 1, 2])
    assert later.shape_key() == mixed.shape_key()
    prompts = HostStep(list("ab"), [700, 1], [0, 50], [700, 51], [0, 1])
    assert prompts.shape_key() == (700, 0, 0, 0)
