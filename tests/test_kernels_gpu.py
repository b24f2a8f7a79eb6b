"""Each kernel alone against a plain PyTorch fp32 reference of the same
operation, at other sizes than the engine tests use."""
import math
import random
from types import SimpleNamespace

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

DEV = "cuda:0"


def _ops():
    from crucible_b200 import ops
    return ops


def rel(got, ref):
    got, ref = got.double().cpu(), ref.double().cpu()
    return float((got - ref).abs().max()) / max(float(ref.abs().max()), 1e-6)


# ---------------------------------------------------------------------------
# row-wise kernels
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_embed_rows(dtype):
    ops = _ops()
    table = torch.randn(301, 72, device=DEV).to(dtype)
    ids = torch.tensor([0, 300, 17, 17, 5], dtype=torch.int32, device=DEV)
    out = torch.empty(5, 72, device=DEV)
    ops.embed_rows(table, ids, out)
    assert torch.equal(out, table[ids.long()].float())


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("width,eps", [(72, 1e-5), (1000, 1e-6), (4100, 1e-3), (768, 1e-5), (4096, 1e-6)])
@pytest.mark.parametrize("rows", [9, 203])                 # few rows: a block per row; many: a warp per row
def test_rmsnorm(dtype, width, eps, rows):
    ops = _ops()
    x = torch.randn(rows, width, device=DEV) * 3.0
    gain = 1.0 + 0.2 * torch.randn(width, device=DEV)
    out = torch.empty(rows, width, device=DEV, dtype=dtype)
    ops.rmsnorm(x, gain, eps, out)
    ref = x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + eps) * gain.double()
    assert rel(out, ref) < (2e-6 if dtype == torch.float32 else 5e-3)


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
def test_swiglu(dtype):
    ops = _ops()
    gu = (torch.randn(11, 2 * 88, device=DEV) * 2).to(dtype)
    out = torch.empty(11, 88, device=DEV, dtype=dtype)
    ops.swiglu(gu, out)
    g, u = gu[:, :88].double(), gu[:, 88:].double()
    assert rel(out, g / (1 + torch.exp(-g)) * u) < (2e-6 if dtype == torch.float32 else 5e-3)


def test_gather_rows():
    ops = _ops()
    x = torch.randn(20, 40, device=DEV)
    rows = torch.tensor([19, 0, 7], dtype=torch.int32, device=DEV)
    out = torch.empty(3, 40, device=DEV)
    ops.gather_rows(x, rows, out)
    assert torch.equal(out, x[rows.long()])


# ---------------------------------------------------------------------------
# matrix products
# ---------------------------------------------------------------------------

SHAPES = [(1, 64, 64), (7, 509, 96), (130, 192, 320), (300, 1280, 768), (64, 2050, 136),
          (257, 100, 24)]


@pytest.mark.parametrize("m,n,k", SHAPES + [(5, 33, 7), (70, 65, 129)])
def test_linear_plain_fp32(m, n, k):
    ops = _ops()
    # mantissa-dense and single-signed data, so that a dropped or doubled term shows
    a = torch.rand(m, k, device=DEV) + 0.5
    w = torch.rand(n, k, device=DEV) + 0.5
    out = torch.empty(m, n, device=DEV)
    ops.linear_plain(a, w, out)
    ref = a.double() @ w.double().T
    assert rel(out, ref) < 2e-6
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    ops.linear_plain(a, w, acc, accumulate=True)
    assert rel(acc, ref + base.double()) < 2e-6


@pytest.mark.parametrize("tile", [64, 96, 128, 160, 192, 256])
@pytest.mark.parametrize("m,n,k", SHAPES)
def test_linear_tensor_core(m, n, k, tile):
    from crucible_b200.ops import tensor_core
    a = (torch.rand(m, k, device=DEV) + 0.5).bfloat16()
    w = (torch.rand(n, k, device=DEV) * 0.1 + 0.05).bfloat16()
    ref = a.double() @ w.double().T
    out = torch.empty(m, n, device=DEV)
    assert tensor_core.linear(a, w, out, tile=tile)
    assert rel(out, ref) < 1e-5
    out16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.linear(a, w, out16, tile=tile)
    assert rel(out16, ref) < 5e-3
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    assert tensor_core.linear(a, w, acc, accumulate=True, tile=tile)
    assert rel(acc, ref + base.double()) < 1e-5
    tensor_core.check_status(DEV)


@pytest.mark.parametrize("m,n,k", [(300, 1280, 768), (1000, 512, 320), (257, 100, 24), (130, 192, 1096)])
def test_linear_tensor_core_two_accumulators(m, n, k):
    """256 x 256 of output per block: two accumulators in tensor memory, the W tile shared."""
    from crucible_b200.ops import tensor_core
    a = (torch.rand(m, k, device=DEV) + 0.5).bfloat16()
    w = (torch.rand(n, k, device=DEV) * 0.1 + 0.05).bfloat16()
    ref = a.double() @ w.double().T
    out = torch.empty(m, n, device=DEV)
    assert tensor_core.linear(a, w, out, tile=(256, 0))
    assert rel(out, ref) < 1e-5
    out16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.linear(a, w, out16, tile=(256, 0))      # rows of 200 bytes: the 128-row tiles step in
    assert rel(out16, ref) < 5e-3
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    assert tensor_core.linear(a, w, acc, accumulate=True, tile=(256, 0))
    assert rel(acc, ref + base.double()) < 1e-5
    inter = n // 2 // 8 * 8
    h = torch.randn(m, k, device=DEV).bfloat16()
    w2 = (torch.randn(2 * inter, k, device=DEV) * 0.05).bfloat16()
    act = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.linear_swiglu(h, w2, act, tile=(256, 0))
    y = h.double() @ w2.double().T
    g, u = y[:, :inter], y[:, inter:]
    assert rel(act, g / (1 + torch.exp(-g)) * u) < 6e-3
    tensor_core.check_status(DEV)


@pytest.mark.parametrize("tile", [64, 96, 128, 160, 192, 256])
@pytest.mark.parametrize("m,inter,k", [(1, 176, 64), (33, 320, 96), (300, 2048, 768), (130, 88, 40)])
def test_linear_swiglu_tensor_core(m, inter, k, tile):
    from crucible_b200.ops import tensor_core
    h = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(2 * inter, k, device=DEV) * 0.2).bfloat16()
    out = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.linear_swiglu(h, w, out, tile=tile)
    y = h.double() @ w.double().T
    g, u = y[:, :inter], y[:, inter:]
    assert rel(out, g / (1 + torch.exp(-g)) * u) < 6e-3
    tensor_core.check_status(DEV)


@pytest.mark.parametrize("tile", [64, 128, 256])
@pytest.mark.parametrize("splits", [2, 3, 8])
@pytest.mark.parametrize("m,n,k", [(40, 768, 2048), (64, 100, 520), (130, 192, 1000), (300, 96, 4096)])
def test_linear_tensor_core_shares_of_k(m, n, k, splits, tile):
    """A cluster of blocks shares one tile's K and sums over distributed shared memory;
    a number of shares that would leave one empty is refused."""
    from crucible_b200.ops import tensor_core
    a = (torch.rand(m, k, device=DEV) + 0.5).bfloat16()
    w = (torch.rand(n, k, device=DEV) * 0.1 + 0.05).bfloat16()
    k_blocks = -(-k // 64)
    fits = (splits - 1) * -(-k_blocks // splits) < k_blocks
    out = torch.empty(m, n, device=DEV)
    assert tensor_core.linear(a, w, out, tile=(tile, 1, splits)) is fits
    if not fits:
        return
    ref = a.double() @ w.double().T
    assert rel(out, ref) < 1e-5
    again = torch.empty(m, n, device=DEV)
    assert tensor_core.linear(a, w, again, tile=(tile, 1, splits))
    assert torch.equal(out, again)                     # the order of the sum is fixed
    out16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.linear(a, w, out16, tile=(tile, 1, splits))
    assert rel(out16, ref) < 5e-3
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    assert tensor_core.linear(a, w, acc, accumulate=True, tile=(tile, 1, splits))
    assert rel(acc, ref + base.double()) < 1e-5
    inter = n // 2
    h = torch.randn(m, k, device=DEV).bfloat16()
    w2 = (torch.randn(2 * inter, k, device=DEV) * 0.05).bfloat16()
    act = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.linear_swiglu(h, w2, act, tile=(tile, 1, splits))
    y = h.double() @ w2.double().T
    g, u = y[:, :inter], y[:, inter:]
    assert rel(act, g / (1 + torch.exp(-g)) * u) < 6e-3
    tensor_core.check_status(DEV)


def test_linear_tensor_core_takes_shares_of_k_by_itself():
    from crucible_b200.ops import tensor_core
    m, n, k = 64, 768, 2048
    assert tensor_core.k_splits(m, n, k, 64) == 4
    a = (torch.rand(m, k, device=DEV) + 0.5).bfloat16()
    w = (torch.rand(n, k, device=DEV) * 0.1 + 0.05).bfloat16()
    base = torch.randn(m, n, device=DEV)
    acc = base.clone()
    assert tensor_core.linear(a, w, acc, accumulate=True)
    assert rel(acc, a.double() @ w.double().T + base.double()) < 1e-5
    tensor_core.check_status(DEV)


@pytest.mark.parametrize("splits", [1, 2, 5, None])
@pytest.mark.parametrize("m,n,k", [(1, 64, 64), (7, 509, 96), (16, 1280, 768), (33, 768, 2048),
                                   (64, 200, 320), (8, 50304, 768), (3, 100, 1000)])
def test_linear_few_rows_split_along_k(m, n, k, splits):
    """The product for decoded tokens: W on the MMA's M side, K split over blocks,
    the last block to arrive sums the partials in a fixed order."""
    from crucible_b200.ops import tensor_core
    a = (torch.rand(m, k, device=DEV) + 0.5).bfloat16()
    w = (torch.rand(n, k, device=DEV) * 0.1 + 0.05).bfloat16()
    ref = a.double() @ w.double().T
    base = torch.randn(m, n, device=DEV)
    for _ in range(2):                                   # twice: the counters must be back at zero
        out = torch.empty(m, n, device=DEV)
        assert tensor_core._gemm_skinny(a, w, out, n, tensor_core.STORE_F32, splits)
        assert rel(out, ref) < 1e-5
        out16 = torch.empty(m, n, device=DEV, dtype=torch.bfloat16)
        assert tensor_core._gemm_skinny(a, w, out16, n, tensor_core.STORE_BF16, splits)
        assert rel(out16, ref) < 5e-3
        acc = base.clone()
        assert tensor_core._gemm_skinny(a, w, acc, n, tensor_core.ACCUM_F32, splits)
        assert rel(acc, ref + base.double()) < 1e-5
    first = torch.empty(m, n, device=DEV)
    again = torch.empty(m, n, device=DEV)
    tensor_core._gemm_skinny(a, w, first, n, tensor_core.STORE_F32, splits)
    tensor_core._gemm_skinny(a, w, again, n, tensor_core.STORE_F32, splits)
    assert torch.equal(first, again)                      # the order of the sum is fixed
    tensor_core.check_status(DEV)


@pytest.mark.parametrize("splits", [1, 3, None])
@pytest.mark.parametrize("m,inter,k", [(1, 176, 64), (8, 2048, 768), (33, 320, 96), (64, 90, 136)])
def test_linear_swiglu_few_rows(m, inter, k, splits):
    from crucible_b200.ops import tensor_core
    h = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(2 * inter, k, device=DEV) * 0.2).bfloat16()
    y = h.double() @ w.double().T
    g, u = y[:, :inter], y[:, inter:]
    for _ in range(2):
        out = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
        assert tensor_core._gemm_skinny(h, w, out, inter, tensor_core.SWIGLU_BF16, splits)
        assert rel(out, g / (1 + torch.exp(-g)) * u) < 6e-3
    tensor_core.check_status(DEV)


@pytest.mark.parametrize("m", [1, 2, 3, 8, 11, 16])
@pytest.mark.parametrize("n,k", [(768, 768), (100, 2048), (33, 40), (1280, 1032), (64, 4104)])
def test_small_batch_linear_and_swiglu(m, n, k):
    """The fused kernels for a few rows: bf16 input or fp32 rows normalised on the fly."""
    from crucible_b200.ops import small_batch
    w = (torch.randn(n, k, device=DEV) * 0.1).bfloat16()
    a = torch.randn(m, k, device=DEV).bfloat16()
    base = torch.randn(m, n, device=DEV)
    out = base.clone()
    assert small_batch.linear(a, w, out, accumulate=True)
    assert rel(out, base.double() + a.double() @ w.double().T) < 1e-5
    x = torch.randn(m, k, device=DEV) * 2
    gain = 1 + 0.2 * torch.randn(k, device=DEV)
    lazy = small_batch.LazyNorm(x, gain, 1e-5, lambda: None)
    normed = x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-5) * gain.double()
    out = torch.empty(m, n, device=DEV)
    assert small_batch.linear(lazy, w, out)
    assert rel(out, normed @ w.double().T) < 5e-3        # the normalised rows are rounded to bfloat16
    if n % 2 == 0:
        inter = n // 2
        act = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
        assert small_batch.linear_swiglu(lazy, w, act)
        y = normed @ w.double().T
        g, u = y[:, :inter], y[:, inter:]
        assert rel(act, g / (1 + torch.exp(-g)) * u) < 5e-3
    too_many = small_batch.MAX_ROWS + 1
    big = torch.randn(too_many, k, device=DEV).bfloat16()
    assert small_batch.linear(big, w, torch.empty(too_many, n, device=DEV)) is False
    odd = torch.randn(m, 12, device=DEV).bfloat16()
    assert small_batch.linear(odd, torch.randn(n, 12, device=DEV).bfloat16(),
                              torch.empty(m, n, device=DEV)) is False             # K not a multiple of 8


@pytest.mark.parametrize("m", [9, 13, 16, 17, 27, 32])
@pytest.mark.parametrize("n,k", [(768, 768), (100, 2048), (1280, 1032), (64, 4104)])
def test_small_batch_row_groups(m, n, k):
    """9 to 32 rows of bf16 input: two or four groups of 8 rows share each weight fragment."""
    from crucible_b200.ops import small_batch
    w = (torch.randn(n, k, device=DEV) * 0.1).bfloat16()
    a = torch.randn(m, k, device=DEV).bfloat16()
    base = torch.randn(m, n, device=DEV)
    out = base.clone()
    groups = 2 if m <= 16 else 4
    if 8 * groups * (k + 32) * 2 > 200 * 1024:           # the staged rows do not fit: refused
        assert small_batch.linear(a, w, out, accumulate=True) is False
        return
    assert small_batch.linear(a, w, out, accumulate=True)
    assert rel(out, base.double() + a.double() @ w.double().T) < 1e-5
    out2 = torch.empty(m, n, device=DEV)
    assert small_batch.linear(a, w, out2)
    assert rel(out2, a.double() @ w.double().T) < 1e-5
    inter = n // 2
    act = torch.empty(m, inter, device=DEV, dtype=torch.bfloat16)
    assert small_batch.linear_swiglu(a, w, act)
    y = a.double() @ w.double().T
    g, u = y[:, :inter], y[:, inter:]
    assert rel(act, g / (1 + torch.exp(-g)) * u) < 5e-3


def test_small_batch_large_weights_take_other_paths():
    """Beyond a few megabytes the norm is run once instead of in every block; beyond
    tens of megabytes the kernels refuse and the caller's tensor-core kernel streams."""
    from crucible_b200.ops import small_batch
    ops = _ops()
    m, n, k = 5, 2560, 2048                                    # 10.5 MB
    assert n * k * 2 > small_batch.NORM_FUSE_MAX_BYTES
    w = (torch.randn(n, k, device=DEV) * 0.05).bfloat16()
    x = torch.randn(m, k, device=DEV) * 2
    gain = 1 + 0.2 * torch.randn(k, device=DEV)
    ran = []

    def materialize():
        ran.append(1)
        out = torch.empty(m, k, device=DEV, dtype=torch.bfloat16)
        ops.rmsnorm(x, gain, 1e-5, out)
        return out
    lazy = small_batch.LazyNorm(x, gain, 1e-5, materialize)
    out = torch.empty(m, n, device=DEV)
    assert small_batch.linear(lazy, w, out)
    assert ran == [1]
    normed = x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-5) * gain.double()
    assert rel(out, normed @ w.double().T) < 5e-3
    huge = torch.empty(small_batch.MAX_WEIGHT_BYTES // (2 * k) + 8, k, device=DEV, dtype=torch.bfloat16)
    assert small_batch.linear(lazy, huge, torch.empty(m, huge.shape[0], device=DEV)) is False


def _rows_ahead_of_their_norm(rows, width, spread, eps, parts=3):
    """(what the norm hands on, the product's bf16 rows, the normalised rows in float64) for
    rows whose sums of squares lie in `parts` shares, as the product before them left them."""
    from crucible_b200.ops import small_batch
    x = torch.randn(rows, width, device=DEV) * spread
    x *= torch.linspace(0.1, 4.0, rows, device=DEV).unsqueeze(1)          # rows of very different size
    gain = 1.0 + 0.2 * torch.randn(width, device=DEV)
    edges = [round(width * p / parts) for p in range(parts + 1)]
    sumsq = torch.stack([x[:, a:b].pow(2).sum(1) for a, b in zip(edges[:-1], edges[1:])]).contiguous()
    scaled = (x * gain).bfloat16()
    normed = x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + eps) * gain.double()
    return small_batch.LazyNorm(x, gain, eps, None, scaled, sumsq, parts), scaled, normed


@pytest.mark.parametrize("m,n,k,tile", [(300, 768, 2048, 96), (40, 768, 768, 64), (64, 768, 2048, (64, 1, 4)),
                                        (130, 96, 320, 128), (2048, 1024, 512, 128)])
def test_accumulate_product_leaves_the_next_norms_input(m, n, k, tile):
    """x += a W^T with bf16(x * gain) and the tiles' shares of every row's sum of squares
    beside it; then a gate/up product that takes those rows and applies the rows' factors."""
    from crucible_b200.ops import small_batch, tensor_core
    torch.manual_seed(m + n)
    a = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.1).bfloat16()
    x0 = torch.randn(m, n, device=DEV) * torch.linspace(0.2, 5.0, m, device=DEV).unsqueeze(1)
    gain = 1.0 + 0.2 * torch.randn(n, device=DEV)
    x = x0.clone()
    emit = tensor_core.NormEmit(gain, torch.zeros(m, n, device=DEV, dtype=torch.bfloat16),
                                torch.zeros(-(-n // 64), m, device=DEV))
    assert tensor_core.linear(a, w, x, accumulate=True, tile=tile, emit=emit)
    tensor_core.check_status(DEV)
    bn = tile if isinstance(tile, int) else tile[0]
    assert emit.parts == -(-n // bn)
    ref = x0.double() + a.double() @ w.double().T
    assert rel(x, ref) < 2e-5
    assert torch.equal(emit.scaled, (x * gain).bfloat16())                 # of the rows as written
    shares = torch.stack([x[:, i * bn:(i + 1) * bn].double().pow(2).sum(1) for i in range(emit.parts)])
    assert rel(emit.sumsq[:emit.parts], shares) < 1e-5
    # without the request the product is the same to the bit
    y = x0.clone()
    assert tensor_core.linear(a, w, y, accumulate=True, tile=tile)
    assert rel(y, x) < 1e-6
    # the consumer: gate/up over these rows
    eps, inter = 1e-5, 160
    pre = small_batch.LazyNorm(x, gain, eps, None, emit.scaled, emit.sumsq, emit.parts)
    w2 = (torch.randn(2 * inter, n, device=DEV) * 0.1).bfloat16()
    for t2 in (64, 128, 256, (256, 0)):
        act = torch.zeros(m, inter, device=DEV, dtype=torch.bfloat16)
        assert tensor_core.linear_swiglu(emit.scaled, w2, act, tile=t2, pre=pre)
        normed = ref * torch.rsqrt(ref.pow(2).mean(-1, keepdim=True) + eps) * gain.double()
        z = normed @ w2.double().T
        g, u = z[:, :inter], z[:, inter:]
        assert rel(act, g / (1 + torch.exp(-g)) * u) < 6e-3, t2
    # a plain product has no such form: refused, and the norm's own kernel runs for it
    assert not tensor_core.linear(emit.scaled, w2, torch.zeros(m, 2 * inter, device=DEV), pre=pre)
    tensor_core.check_status(DEV)


def test_a_product_that_cannot_leave_the_norms_input_says_so():
    from crucible_b200.ops import tensor_core
    m, n, k = 200, 520, 256                     # 520 columns: the last chunk of 32 is not whole
    a = torch.randn(m, k, device=DEV).bfloat16()
    w = (torch.randn(n, k, device=DEV) * 0.1).bfloat16()
    for n_cols, tile in ((520, 64), (512, 256)):
        x = torch.zeros(m, n_cols, device=DEV)
        emit = tensor_core.NormEmit(torch.ones(n_cols, device=DEV),
                                    torch.zeros(m, n_cols, device=DEV, dtype=torch.bfloat16),
                                    torch.zeros(16, m, device=DEV))
        assert tensor_core.linear(a, w[:n_cols], x, accumulate=True, tile=tile, emit=emit)
        assert emit.parts is None and float(emit.scaled.abs().sum()) == 0
        assert rel(x, a.double() @ w[:n_cols].double().T) < 2e-5


@pytest.mark.parametrize("hd,n_heads,n_kv,rows,d", [(64, 6, 2, 300, 256), (64, 5, 1, 40, 256),
                                                    (128, 3, 1, 150, 256), (64, 6, 2, 60, 1024)])
@pytest.mark.parametrize("write", [True, False])
@pytest.mark.parametrize("tall", [False, True])
@pytest.mark.parametrize("ahead", [False, True])
def test_linear_rope_append_tensor_core(hd, n_heads, n_kv, rows, d, write, tall, ahead):
    """The q/k/v product for many rows with rotation and cache write in its epilogue (the
    last case: few tiles and a long K, so clusters share K); `tall`: 256 x 256 tiles;
    `ahead`: its rows are bf16(x * gain) of rows not yet divided by their root mean square,
    with every row's sum of squares in three shares."""
    from crucible_b200.ops import tensor_core
    page = 16
    torch.manual_seed(rows)
    n_req = 3
    # rows of three requests, each at its own positions; pages shuffled
    per = [rows // 3, rows // 3, rows - 2 * (rows // 3)]
    starts = [7, 0, 33]
    positions, row_request = [], []
    for r in range(n_req):
        positions += list(range(starts[r], starts[r] + per[r]))
        row_request += [r] * per[r]
    pages_per = [-(-(starts[r] + per[r]) // page) for r in range(n_req)]
    ids = list(range(sum(pages_per) + 2))
    random.Random(1).shuffle(ids)
    tables = torch.zeros(n_req, max(pages_per) + 1, dtype=torch.int32)
    for r in range(n_req):
        for i in range(pages_per[r]):
            tables[r, i] = ids.pop()
    tables = tables.to(DEV)
    h = torch.randn(rows, d, device=DEV).bfloat16()
    pre, h_ref = None, h.double()
    if ahead:
        pre, h, h_ref = _rows_ahead_of_their_norm(rows, d, 3.0 + rows / 100, 1e-5)
    w = (torch.randn((n_heads + 2 * n_kv) * hd, d, device=DEV) * 0.2).bfloat16()
    i = torch.arange(hd // 2, dtype=torch.float64)
    ang = torch.outer(torch.arange(max(positions) + 1, dtype=torch.float64), 10000.0 ** (-2 * i / hd))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    n_pages = sum(pages_per) + 2
    kv = torch.zeros(1, 2, n_pages, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)

    class Cache:
        page_tokens = page
        keys = staticmethod(lambda slot: kv[slot, 0])
        values = staticmethod(lambda slot: kv[slot, 1])
    ctx = SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                          row_request=torch.tensor(row_request, dtype=torch.int32, device=DEV),
                          block_table=lambda g: tables)
    qkv = torch.zeros(rows, w.shape[0], device=DEV, dtype=torch.bfloat16)
    try:
        tensor_core.ROPE_TALL = tall
        assert tensor_core.linear_rope_append(h, w, qkv, n_heads, n_kv, hd, cos, sin, hd, ctx, Cache,
                                              SimpleNamespace(group=0, slot=0, write=write), pre=pre)
    finally:
        tensor_core.ROPE_TALL = None
    torch.cuda.synchronize()
    tensor_core.check_status(DEV)
    y = (h_ref @ w.double().T).cpu().view(rows, n_heads + 2 * n_kv, hd)
    pos_t = torch.tensor(positions)
    c, s = ang[pos_t].cos()[:, None, :], ang[pos_t].sin()[:, None, :]

    def rotate(v):
        x1, x2 = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)
    assert rel(qkv[:, :n_heads * hd].view(rows, n_heads, hd), rotate(y[:, :n_heads])) < 6e-3
    page_of = tables.cpu()[torch.tensor(row_request), pos_t // page].long()
    got_k = kv[0, 0].cpu()[page_of, :, pos_t % page]
    got_v = kv[0, 1].cpu()[page_of, :, pos_t % page]
    if write:
        assert rel(got_k, rotate(y[:, n_heads:n_heads + n_kv])) < 6e-3
        assert rel(got_v, y[:, n_heads + n_kv:]) < 6e-3
        written = torch.zeros(n_pages, page, dtype=torch.bool)
        written[page_of, pos_t % page] = True
        assert kv[0, 0].cpu().float().abs().sum(dim=(1, 3))[~written].sum() == 0     # nothing else touched
    else:
        assert kv.abs().sum() == 0


@pytest.mark.parametrize("write", [True, False])
@pytest.mark.parametrize("many", [False, True])
def test_small_batch_qkv_rope_append(write, many):
    """A few rows not yet normalised (the norm runs inside), or up to 32 normalised bf16 rows."""
    from crucible_b200.ops import small_batch
    n_heads, n_kv, hd, page, d = 6, 2, 32, 8, 96
    positions = [5, 17, 0, 40] + ([41, 42, 43, 44, 18, 19, 1, 2, 3, 4, 5, 6, 7, 20, 21, 22, 23, 45] if many else [])
    row_request = [0, 0, 1, 2] + ([2, 2, 2, 2, 0, 0, 1, 1, 1, 1, 1, 1, 1, 0, 0, 0, 0, 2] if many else [])
    tables = torch.tensor([[3, 1, 7, 0, 0, 0], [2, 0, 0, 0, 0, 0], [4, 5, 6, 8, 9, 10]],
                          dtype=torch.int32, device=DEV)
    t = len(positions)
    x = torch.randn(t, d, device=DEV)
    gain = 1 + 0.1 * torch.randn(d, device=DEV)
    w = (torch.randn((n_heads + 2 * n_kv) * hd, d, device=DEV) * 0.2).bfloat16()
    i = torch.arange(hd // 2, dtype=torch.float64)
    ang = torch.outer(torch.arange(64, dtype=torch.float64), 10000.0 ** (-2 * i / hd))
    cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)
    kv = torch.zeros(1, 2, 11, n_kv, page, hd, dtype=torch.bfloat16, device=DEV)

    class Cache:
        page_tokens = page
        keys = staticmethod(lambda slot: kv[slot, 0])
        values = staticmethod(lambda slot: kv[slot, 1])
    ctx = SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                          row_request=torch.tensor(row_request, dtype=torch.int32, device=DEV),
                          block_table=lambda g: tables)
    qkv = torch.zeros(t, w.shape[0], device=DEV, dtype=torch.bfloat16)
    normed = x.double() * torch.rsqrt(x.double().pow(2).mean(-1, keepdim=True) + 1e-6) * gain.double()
    lazy = small_batch.LazyNorm(x, gain, 1e-6, lambda: normed.to(torch.bfloat16))
    assert small_batch.qkv_rope_append(lazy, w, qkv, n_heads, n_kv, hd, cos, sin, hd, ctx, Cache,
                                       SimpleNamespace(group=0, slot=0, write=write))
    y = (normed @ w.double().T).cpu().view(t, n_heads + 2 * n_kv, hd)

    def rotate(v, pos):
        c, s = ang[pos].cos(), ang[pos].sin()
        x1, x2 = v[..., :hd // 2], v[..., hd // 2:]
        return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c], dim=-1)
    for r, pos in enumerate(positions):
        assert rel(qkv[r, :n_heads * hd].view(n_heads, hd), rotate(y[r, :n_heads], pos)) < 8e-3
        page_id = int(tables[row_request[r], pos // page])
        if write:
            assert rel(kv[0, 0, page_id, :, pos % page], rotate(y[r, n_heads:n_heads + n_kv], pos)) < 8e-3
            assert rel(kv[0, 1, page_id, :, pos % page], y[r, n_heads + n_kv:]) < 8e-3
    if not write:
        assert float(kv.abs().max()) == 0.0
    # a partially rotated head is refused
    assert small_batch.qkv_rope_append(lazy, w, qkv, n_heads, n_kv, hd, cos[:, :8].contiguous(),
                                       sin[:, :8].contiguous(), 16, ctx, Cache,
                                       SimpleNamespace(group=0, slot=0, write=True)) is False


def test_linear_refuses_what_tma_cannot_read():
    from crucible_b200.ops import tensor_core
    a = torch.randn(4, 100, device=DEV).bfloat16()      # 200-byte rows: not a multiple of 16
    w = torch.randn(8, 100, device=DEV).bfloat16()
    out = torch.empty(4, 8, device=DEV)
    assert tensor_core.linear(a, w, out) is False
    ops = _ops()
    ops.linear(a, w, out)                                # the CUDA-core product takes over
    assert rel(out, a.double() @ w.double().T) < 1e-5


# ---------------------------------------------------------------------------
# attention over a paged cache
# ---------------------------------------------------------------------------

def _paged_case(dtype, n_heads, n_kv, hd, page_tokens, requests, seed, window=None, peak=True,
                shuffle=True, released="null"):
    """requests: list of (context_before, new_tokens).  Builds random q, k, v for
    whole sequences, scatters k/v of the context into shuffled pages, and returns
    what the kernels need plus the reference output for the new rows.  With a window,
    pages that lie wholly below the window of a request's first new token are taken
    away as the cache manager does: their contents become the loud value and their
    table entries name the null page (`released="null"`: one more page, all zeros, as
    the engine uploads it) or are -1 (`released="minus"`)."""
    g = torch.Generator(device="cpu").manual_seed(seed)
    rng = random.Random(seed)
    total_pages = sum(-(-(c + n) // page_tokens) for c, n in requests) + 3
    order = list(range(total_pages))
    if shuffle:
        rng.shuffle(order)
    else:
        order.reverse()              # pages are handed out in ascending order: runs of pages
    kv = torch.full((1, 2, total_pages + 1, n_kv, page_tokens, hd), float("nan"))   # poison
    null_page = total_pages
    kv[:, :, null_page] = 0.0
    stride = max(-(-(c + n) // page_tokens) for c, n in requests) + 2
    tables = torch.zeros(len(requests), stride, dtype=torch.int32)
    q_rows, refs, positions, row_request, row_start, first_pos = [], [], [], [], [0], []
    n_rep = n_heads // n_kv
    for r, (ctx_len, n_new) in enumerate(requests):
        length = ctx_len + n_new
        q = torch.randn(length, n_heads, hd, generator=g)
        k = torch.randn(length, n_kv, hd, generator=g)
        v = torch.randn(length, n_kv, hd, generator=g)
        if peak and length > 3:
            # one far key stands out for the last query of every head: a kernel that
            # loses it (a page's edge, a chunk's edge) is off by far more than rounding
            far = rng.randrange(0, max(1, length // 3))
            if window is not None:
                far = max(far, length - window)
            for h in range(n_heads):
                k[far, h // n_rep] = q[length - 1, h] * (6.0 / math.sqrt(hd))
        q, k, v = q.to(dtype), k.to(dtype), v.to(dtype)
        pages = [order.pop() for _ in range(-(-length // page_tokens))]
        tables[r, :len(pages)] = torch.tensor(pages, dtype=torch.int32)
        for pos in range(length):
            kv[0, 0, pages[pos // page_tokens], :, pos % page_tokens] = k[pos].float()
            kv[0, 1, pages[pos // page_tokens], :, pos % page_tokens] = v[pos].float()
        if window is not None and released:
            for b in range(max(0, ctx_len - window + 1) // page_tokens):
                kv[0, :, pages[b]] = float("nan")
                tables[r, b] = null_page if released == "null" else -1
        qd, kd, vd = q.double(), k.double(), v.double()
        out = torch.zeros(n_new, n_heads, hd, dtype=torch.float64)
        for i, pos in enumerate(range(ctx_len, length)):
            lo = 0 if window is None else max(0, pos - window + 1)
            for h in range(n_heads):
                s = (kd[lo:pos + 1, h // n_rep] @ qd[pos, h]) / math.sqrt(hd)
                p = torch.softmax(s, dim=0)
                out[i, h] = p @ vd[lo:pos + 1, h // n_rep]
        refs.append(out)
        q_rows.append(q[ctx_len:])
        positions += list(range(ctx_len, length))
        row_request += [r] * n_new
        row_start.append(row_start[-1] + n_new)
        first_pos.append(ctx_len)
    t = len(positions)
    qkv = torch.zeros(t, (n_heads + 2 * n_kv) * hd, dtype=dtype)
    qkv[:, :n_heads * hd] = torch.cat(q_rows).reshape(t, n_heads * hd)
    kv = torch.nan_to_num(kv, nan=1e4).to(dtype).to(DEV)       # unused slots hold a loud value

    class Cache:
        pass
    cache = Cache()
    cache.page_tokens = page_tokens
    cache.keys = lambda slot: kv[slot, 0]
    cache.values = lambda slot: kv[slot, 1]
    dev = lambda x: torch.tensor(x, dtype=torch.int32, device=DEV)
    table_dev = tables.to(DEV)
    scratch = {}

    def get_scratch(name, shape, dt):
        key = (name, tuple(shape), dt)
        if key not in scratch:
            scratch[key] = torch.empty(*shape, dtype=dt, device=DEV)
        return scratch[key]
    from crucible_b200.engine.context import HostStep
    ctx = SimpleNamespace(
        positions=dev(positions), row_request=dev(row_request), req_row_start=dev(row_start),
        req_first_pos=dev(first_pos), n_tokens=t, n_requests=len(requests),
        block_table=lambda group: table_dev, scratch=get_scratch,
        host=HostStep(list(range(len(requests))), [n for _, n in requests],
                      [c for c, _ in requests], [c + n for c, n in requests],
                      [0] * len(requests)))
    binding = SimpleNamespace(group=0, slot=0, write=True)
    return qkv.to(DEV), ctx, cache, binding, torch.cat(refs).reshape(t, n_heads * hd)


ATTN_CASES = [
    # heads, kv heads, head size, page, [(context before, new tokens)], window
    (12, 4, 64, 16, [(0, 130), (300, 1), (17, 40)], None),
    (8, 8, 128, 32, [(0, 70), (511, 1)], None),
    (6, 2, 48, 16, [(5, 33), (257, 2), (0, 1)], None),
    (4, 1, 16, 8, [(1023, 1), (0, 260)], None),
    (4, 2, 32, 16, [(100, 60), (400, 1)], 96),
    (2, 1, 256, 16, [(40, 30)], None),
]


@pytest.mark.parametrize("case", ATTN_CASES)
def test_attention_plain_fp32(case):
    ops = _ops()
    n_heads, n_kv, hd, page, requests, window = case
    qkv, ctx, cache, binding, ref = _paged_case(torch.float32, n_heads, n_kv, hd, page, requests, 3,
                                                window)
    out = torch.zeros(qkv.shape[0], n_heads * hd, device=DEV)
    ops.paged_attention_plain(qkv, out, n_heads, n_kv, hd, 1 / math.sqrt(hd), window, ctx, cache,
                              binding)
    assert rel(out.cpu(), ref) < 1e-5


@pytest.mark.parametrize("case", ATTN_CASES)
def test_attention_tensor_core_tiles_and_split(case):
    from crucible_b200.ops import tensor_core
    n_heads, n_kv, hd, page, requests, window = case
    qkv, ctx, cache, binding, ref = _paged_case(torch.bfloat16, n_heads, n_kv, hd, page, requests,
                                                4, window)
    out = torch.zeros(qkv.shape[0], n_heads * hd, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.paged_attention(qkv, out, n_heads, n_kv, hd, 1 / math.sqrt(hd), window, ctx,
                                       cache, binding)
    assert rel(out.cpu(), ref) < 1.5e-2
    # the split form on the decoded rows alone must agree with the tiled form
    single = [(c + n - 1, 1) for c, n in requests]
    qkv1, ctx1, cache1, binding1, ref1 = _paged_case(torch.bfloat16, n_heads, n_kv, hd, page, single,
                                                     4, window)
    out1 = torch.zeros(qkv1.shape[0], n_heads * hd, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.paged_attention(qkv1, out1, n_heads, n_kv, hd, 1 / math.sqrt(hd), window,
                                       ctx1, cache1, binding1)
    assert rel(out1.cpu(), ref1) < 1.5e-2


@pytest.mark.parametrize("case", [
    (12, 4, 64, 16, [(0, 130), (300, 1), (17, 40)], None),
    (4, 4, 64, 32, [(0, 700)], None),
    (6, 1, 64, 8, [(513, 300), (0, 129)], None),
    (8, 2, 64, 128, [(100, 260)], 200),
    (4, 2, 128, 16, [(0, 600), (40, 70)], None),            # head size 128: two stages, one P buffer
    (2, 1, 128, 64, [(300, 420)], 256),
])
@pytest.mark.parametrize("lean", [0, 1])
def test_attention_tcgen05_matches_reference_and_mma(case, lean):
    """Prompt portions with head size 64 or 128: S and O in tensor memory, K and V by TMA; for
    head size 64 both forms of the kernel (an SM to a block, or two lean blocks to an SM)."""
    from crucible_b200.ops import tensor_core
    n_heads, n_kv, hd, page, requests, window = case
    qkv, ctx, cache, binding, ref = _paged_case(torch.bfloat16, n_heads, n_kv, hd, page, requests,
                                                6, window)
    k_cache = cache.keys(0)
    cache.n_pages = k_cache.shape[0]
    out = torch.zeros(qkv.shape[0], n_heads * hd, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.USE_TCGEN05_ATTENTION
    try:
        tensor_core.ATTENTION_LEAN = lean
        whole = tensor_core._Requests(ctx, ctx.block_table(0), 0, ctx.n_requests,
                                      ctx.host.max_new_tokens, ctx.host.context_bucket, ctx.n_tokens)
        assert tensor_core._attention_tcgen05(qkv, out, k_cache, cache.values(0), whole, n_heads, n_kv,
                                              hd, 1 / math.sqrt(hd), window, cache)
    finally:
        tensor_core.ATTENTION_LEAN = -1
    torch.cuda.synchronize()
    tensor_core.check_status(DEV)
    assert rel(out, ref) < 1.5e-2
    try:
        tensor_core.USE_TCGEN05_ATTENTION = False
        other = torch.zeros_like(out)
        assert tensor_core.paged_attention(qkv, other, n_heads, n_kv, hd, 1 / math.sqrt(hd), window,
                                           ctx, cache, binding)
    finally:
        tensor_core.USE_TCGEN05_ATTENTION = True
    assert rel(out, other.float()) < 1.5e-2


@pytest.mark.parametrize("case", [
    # heads, kv heads, head size, page, [(context before, new tokens)], window
    (12, 4, 64, 16, [(2047, 1), (300, 1), (0, 1), (127, 1), (128, 1)], None),
    (8, 1, 64, 32, [(1500, 2), (40, 1)], None),              # 8 heads on one KV head: 16 packed rows
    (6, 2, 64, 8, [(700, 3), (255, 1), (256, 5)], None),     # a few tokens per request
    (4, 4, 64, 128, [(900, 1), (3000, 1)], 400),             # window: leading chunks take no part
    (12, 4, 64, 16, [(5000, 1), (64, 1)], None),             # several chunks merged
    (8, 2, 128, 16, [(2047, 1), (300, 2), (0, 1)], None),    # head size 128
    (4, 4, 128, 64, [(700, 1), (1500, 1)], 512),
])
@pytest.mark.parametrize("shuffle", [True, False])
def test_attention_decode_tcgen05_matches_reference_and_mma(case, shuffle):
    """Decoded tokens with head size 64: the keys on the tensor-memory lanes.  With
    pages in ascending order a tile's pages come in with one copy."""
    from crucible_b200.ops import tensor_core
    n_heads, n_kv, hd, page, requests, window = case
    qkv, ctx, cache, binding, ref = _paged_case(torch.bfloat16, n_heads, n_kv, hd, page, requests,
                                                8, window, shuffle=shuffle)
    outs = {}
    for use in (True, False):
        try:
            tensor_core.USE_TCGEN05_DECODE = use
            before = tensor_core.build._loaded.get("attention_decode_tcgen05")
            out = torch.zeros(qkv.shape[0], n_heads * hd, device=DEV, dtype=torch.bfloat16)
            assert tensor_core.paged_attention(qkv, out, n_heads, n_kv, hd, 1 / math.sqrt(hd), window,
                                               ctx, cache, binding)
            torch.cuda.synchronize()
            tensor_core.check_status(DEV)
            outs[use] = out
        finally:
            tensor_core.USE_TCGEN05_DECODE = True
    assert "attention_decode_tcgen05" in tensor_core.build._loaded
    assert rel(outs[True].cpu(), ref) < 1.5e-2
    assert rel(outs[True], outs[False].float()) < 1.5e-2
    # twice in a row: the counters were left zero
    again = torch.zeros_like(outs[True])
    assert tensor_core.paged_attention(qkv, again, n_heads, n_kv, hd, 1 / math.sqrt(hd), window, ctx,
                                       cache, binding)
    assert torch.equal(again, outs[True])


@pytest.mark.parametrize("case", [
    # decoded tokens first, then portions: the step is two launches over its requests
    (12, 4, 64, 16, [(300, 1), (2047, 1), (0, 1), (0, 130), (17, 40)], None),
    (8, 2, 128, 16, [(700, 1), (40, 200), (1000, 1)], None),      # a decoded token after a portion: tiles
    (6, 2, 48, 16, [(257, 1), (900, 1), (5, 33)], None),           # heads of 48: both forms of the mma.sync kernel
    (4, 2, 64, 32, [(900, 1), (100, 1), (400, 90)], 300),          # a window, with pages given back
])
@pytest.mark.parametrize("released", ["null", "minus"])
def test_attention_of_a_mixed_step_chooses_the_kernel_per_request(case, released):
    from crucible_b200.ops import tensor_core
    n_heads, n_kv, hd, page, requests, window = case
    qkv, ctx, cache, binding, ref = _paged_case(torch.bfloat16, n_heads, n_kv, hd, page, requests,
                                                11, window, released=released)
    lead = ctx.host.lead_single
    assert 0 < lead < len(requests)
    out = torch.zeros(qkv.shape[0], n_heads * hd, device=DEV, dtype=torch.bfloat16)
    launches = tensor_core_launches()
    assert tensor_core.paged_attention(qkv, out, n_heads, n_kv, hd, 1 / math.sqrt(hd), window, ctx,
                                       cache, binding)
    assert tensor_core_launches() - launches == 2
    torch.cuda.synchronize()
    tensor_core.check_status(DEV)
    assert rel(out.cpu(), ref) < 1.5e-2
    # and once more: the split form left its counters at zero
    again = torch.zeros_like(out)
    assert tensor_core.paged_attention(qkv, again, n_heads, n_kv, hd, 1 / math.sqrt(hd), window, ctx,
                                       cache, binding)
    assert torch.equal(again, out)


def tensor_core_launches():
    from crucible_b200 import ops
    return ops.LAUNCHES[0]


def test_attention_odd_head_size_falls_to_plain_kernel():
    from crucible_b200.ops import tensor_core
    ops = _ops()
    qkv, ctx, cache, binding, ref = _paged_case(torch.bfloat16, 4, 2, 24, 16, [(30, 5)], 5)
    out = torch.zeros(qkv.shape[0], 4 * 24, device=DEV, dtype=torch.bfloat16)
    assert tensor_core.paged_attention(qkv, out, 4, 2, 24, 0.2, None, ctx, cache, binding) is False
    ops.paged_attention(qkv, out, 4, 2, 24, 1 / math.sqrt(24), None, ctx, cache, binding)
    assert rel(out.cpu(), ref) < 1.5e-2


# ---------------------------------------------------------------------------
# rotary encoding + cache write
# ---------------------------------------------------------------------------

@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16])
@pytest.mark.parametrize("hd,rot", [(16, 16), (64, 64), (48, 32), (32, 0)])
def test_rope_kv_append(dtype, hd, rot):
    ops = _ops()
    n_heads, n_kv, page = 3, 1, 8
    positions = [5, 6, 7, 8, 40, 0]
    row_request = [0, 0, 0, 0, 1, 2]
    tables = torch.tensor([[3, 1, 0, 0, 0, 0], [2, 5, 6, 7, 8, 9], [4, 0, 0, 0, 0, 0]],
                          dtype=torch.int32, device=DEV)
    t = len(positions)
    qkv = torch.randn(t, (n_heads + 2 * n_kv) * hd).to(dtype)
    before = qkv.clone()
    kv = torch.zeros(1, 2, 10, n_kv, page, hd, dtype=dtype, device=DEV)
    cos = sin = None
    if rot:
        i = torch.arange(rot // 2, dtype=torch.float64)
        ang = torch.outer(torch.arange(64, dtype=torch.float64), 500.0 ** (-2 * i / rot))
        cos, sin = ang.cos().float().to(DEV), ang.sin().float().to(DEV)

    class Cache:
        page_tokens = page
        keys = staticmethod(lambda slot: kv[slot, 0])
        values = staticmethod(lambda slot: kv[slot, 1])
    ctx = SimpleNamespace(positions=torch.tensor(positions, dtype=torch.int32, device=DEV),
                          row_request=torch.tensor(row_request, dtype=torch.int32, device=DEV),
                          block_table=lambda g: tables)
    dev_qkv = qkv.to(DEV)
    ops.rope_kv_append(dev_qkv, n_heads, n_kv, hd, cos, sin, rot, ctx, Cache,
                       SimpleNamespace(group=0, slot=0, write=True))
    got = dev_qkv.cpu().double()
    x = before.double().view(t, n_heads + 2 * n_kv, hd)

    def rotate(v, pos):
        if not rot:
            return v
        c, s = ang[pos].cos(), ang[pos].sin()
        x1, x2 = v[..., :rot // 2], v[..., rot // 2:rot]
        return torch.cat([x1 * c - x2 * s, x1 * s + x2 * c, v[..., rot:]], dim=-1)
    tol = 1e-6 if dtype == torch.float32 else 8e-3
    for r, pos in enumerate(positions):
        want_q = rotate(x[r, :n_heads], pos)
        assert rel(got[r].view(-1, hd)[:n_heads], want_q) < tol
        page_id = int(tables[row_request[r], pos // page])
        want_k = rotate(x[r, n_heads:n_heads + n_kv], pos)
        assert rel(kv[0, 0, page_id, :, pos % page].cpu(), want_k) < tol
        assert torch.equal(kv[0, 1, page_id, :, pos % page].cpu().double(), x[r, n_heads + n_kv:])


# ---------------------------------------------------------------------------
# token selection
# ---------------------------------------------------------------------------

def test_argmax_ties_nan_and_edges():
    import plain_model as pm
    ops = _ops()
    nan, inf = float("nan"), float("inf")
    rows = [
        [1.0, 3.0, 3.0, 2.0],            # tie -> lowest index
        [nan, 1.0, 0.5, nan],            # a NaN at index 0 is never displaced -> 0
        [1.0, nan, 2.0, nan],            # a NaN elsewhere displaces nothing -> 2
        [-inf, -inf, -inf, -inf],        # all -inf -> 0
        [0.0, -0.0, 0.0, -1.0],          # signed zeros tie -> 0
        [1.0, 2.0, 3.0, inf],            # last position
        [nan, nan, nan, nan],            # all NaN -> 0
        [-inf, nan, -inf, -inf],         # nothing exceeds the first -> 0
    ]
    logits = torch.tensor(rows, device=DEV)
    out = torch.empty(len(rows), dtype=torch.int32, device=DEV)
    ops.argmax_rows(logits, out)
    want = [pm.plain_argmax(r) for r in rows]
    assert want == [1, 0, 2, 0, 0, 3, 0, 0]
    assert out.tolist() == want
    # the same rules through the greedy rows of the sampling kernel
    out2 = torch.empty(len(rows), dtype=torch.int32, device=DEV)
    ops.sample_rows(logits, torch.zeros(len(rows), device=DEV),
                    torch.ones(len(rows), dtype=torch.int32, device=DEV),
                    torch.zeros(len(rows), device=DEV), 1, out2)
    assert out2.tolist() == want
    # wide rows take the two-stage form
    big = torch.randn(5, 50304, device=DEV)
    big[1, 50303] = 100.0
    big[2, 77] = big[2, 40000] = 50.0
    big[3, 0] = nan                       # never displaced
    big[4, 1] = nan                       # displaces nothing
    out = torch.empty(5, dtype=torch.int32, device=DEV)
    ops.argmax_rows(big, out)
    assert out.tolist() == [pm.plain_argmax(r) for r in big.tolist()]
    assert out.tolist()[1:4] == [50303, 77, 0]


@pytest.mark.parametrize("vocab", [509, 50304])
def test_sample_rows_matches_plain_sampler(vocab):
    import plain_model as pm
    ops = _ops()
    torch.manual_seed(1)
    n = 6
    logits = torch.randn(n, vocab, device=DEV) * 3
    logits[2, 10] = logits[2, 20] = logits[2].max() + 1         # a tie among the best
    logits[3, 5] = float("nan")
    temps = [0.8, 0.0, 1.5, 0.3, 100.0, 0.8]
    ks = [40, 40, 5, 1, 128, 1000]
    seeds = [1234, 1, 7, 8, 9, 10]
    from crucible_b200.sampling.rng import Xorshift64Star
    for draw in range(3):
        rngs = [Xorshift64Star(s) for s in seeds]
        plains = [pm.PlainRng(s) for s in seeds]
        for _ in range(draw):
            for r, p_ in zip(rngs, plains):
                r.next_f32(), p_.next_f32()
        us = [r.next_f32() if t > 0 else 0.0 for r, t in zip(rngs, temps)]
        out = torch.empty(n, dtype=torch.int32, device=DEV)
        ops.sample_rows(logits, torch.tensor(temps, device=DEV),
                        torch.tensor([min(k, vocab) for k in ks], dtype=torch.int32, device=DEV),
                        torch.tensor(us, device=DEV), max(min(k, vocab) for k in ks), out)
        want = [pm.plain_sample(logits[i].tolist(), temps[i], ks[i], plains[i]) for i in range(n)]
        assert out.tolist() == want


def test_issue_probes_report_what_the_loops_were_shaped_by():
    """One thread's cost of sending an MMA and a TMA box (`csrc/issue_probe.cu`): the kernels'
    unrolled loops rest on these being tens and hundreds of cycles, whatever the tile or box."""
    from crucible_b200.ops import issue_probe
    narrow = issue_probe.mma_send_cycles(128, 64)
    wide = issue_probe.mma_send_cycles(128, 256)
    plain = issue_probe.mma_send_cycles(128, 64, tight=False)
    assert 30 <= narrow <= 90, narrow                 # 54 measured: the thread, not the 32 of the tensor cores
    assert 110 <= wide <= 170, wide                   # 128: the tensor cores' own time
    assert plain >= narrow                            # descriptors and flags per MMA cost on top
    small = issue_probe.tma_send_cycles(16)
    big = issue_probe.tma_send_cycles(128)
    assert 20 <= small[0] <= 300 and 20 <= big[0] <= 300, (small, big)     # 60 and 97 measured
    assert big[1] >= big[0]
