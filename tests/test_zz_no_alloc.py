"""The argmax entry point that allocates nothing, called through its exported C
symbol the way a host that cannot call cudaMalloc would call it, against the
library's usual argmax.  This file is collected last on purpose."""
import ctypes

import pytest
import torch

pytestmark = pytest.mark.gpu

MAX_ROWS = 256                 # CB_ARGMAX_STATIC_MAX_ROWS in csrc/no_alloc_argmax.h
TOO_LARGE = 100002             # CB_ERR_STATIC_TOO_LARGE


def _static_argmax(lib, logits, out):
    fn = lib.cb_argmax_rows_static
    fn.restype = ctypes.c_int
    fn.argtypes = [ctypes.c_void_p, ctypes.c_int, ctypes.c_int, ctypes.c_void_p, ctypes.c_void_p]
    return fn(logits.data_ptr(), logits.shape[0], logits.shape[1], out.data_ptr(),
              torch.cuda.current_stream().cuda_stream)


def test_static_scratch_argmax_matches_the_usual_one_twice_in_a_row():
    from crucible_b200 import ops
    from crucible_b200.ops import build
    lib = build.load("sampling")
    torch.manual_seed(5)
    dev = "cuda:0"
    first = torch.randn(7, 50304, device=dev)
    first[2, 50303] = 99.0                              # the very last column wins
    first[3, 100] = first[3, 40000] = 50.0              # a tie: the lower index wins
    first[4, 5] = float("nan")                          # NaN never wins
    second = torch.randn(64, 9001, device=dev) * 3      # other rows, other width: the scratch is reused
    # one call first: it also looks up the scratch array's address, once for this device
    warm = torch.empty(7, dtype=torch.int32, device=dev)
    assert _static_argmax(lib, first, warm) == 0
    torch.cuda.synchronize()
    for logits in (first, second):
        want = torch.empty(logits.shape[0], dtype=torch.int32, device=dev)
        ops.argmax_rows(logits, want)
        got = torch.full((logits.shape[0],), -1, dtype=torch.int32, device=dev)
        torch.cuda.synchronize()
        # free bytes as the driver counts them: a cudaMalloc inside the library would show
        # here, which a counter of torch's own allocator would not
        free_before = torch.cuda.mem_get_info(dev)[0]
        assert _static_argmax(lib, logits, got) == 0
        torch.cuda.synchronize()
        assert torch.cuda.mem_get_info(dev)[0] == free_before
        assert torch.equal(got, want)
    ids = torch.empty(7, dtype=torch.int32, device=dev)
    assert _static_argmax(lib, first, ids) == 0
    torch.cuda.synchronize()
    assert ids.tolist()[2:4] == [50303, 100]


def test_static_scratch_argmax_refuses_more_rows_than_it_holds():
    from crucible_b200.ops import build
    lib = build.load("sampling")
    logits = torch.zeros(MAX_ROWS + 1, 8, device="cuda:0")
    out = torch.full((MAX_ROWS + 1,), -7, dtype=torch.int32, device="cuda:0")
    assert _static_argmax(lib, logits, out) == TOO_LARGE
    torch.cuda.synchronize()
    assert int(out.min()) == -7 and int(out.max()) == -7          # nothing ran
    ok = torch.zeros(MAX_ROWS, 4096, device="cuda:0")
    ok[:, 17] = 1.0
    out = torch.empty(MAX_ROWS, dtype=torch.int32, device="cuda:0")
    assert _static_argmax(lib, ok, out) == 0
    torch.cuda.synchronize()
    assert out.tolist() == [17] * MAX_ROWS
