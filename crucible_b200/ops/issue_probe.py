"""What one thread can send per cycle on this GPU: the two probes of `csrc/issue_probe.cu`.

    python -m crucible_b200.ops.issue_probe

prints cycles per `tcgen05.mma` sent by one thread (by tile width, with a loop as tight as the
kernels' and with a straightforward one) and cycles per TMA box sent by one thread (by the
box's height).  The tensor-core kernels' loops are shaped by these figures: for tiles up to
128 columns wide a step of K costs what its MMA thread's own instructions cost.
"""
from __future__ import annotations

import ctypes

import torch

from . import build, tensor_core

build.register_module("issue_probe", ["common.cuh", "tc_common.cuh"])


def _vp(t) -> ctypes.c_void_p:
    return ctypes.c_void_p(t.data_ptr())


def _stream() -> ctypes.c_void_p:
    return ctypes.c_void_p(torch.cuda.current_stream().cuda_stream)


def mma_send_cycles(m: int, n: int, count: int = 1025, tight: bool = True, device="cuda:0") -> float:
    """Cycles per MMA of m x n x 16 when one thread sends `count` of them back to back."""
    lib = build.load("issue_probe")
    out = torch.zeros(1, dtype=torch.int64, device=device)
    status = tensor_core.status_word(device)
    for _ in range(2):                                   # the first launch also loads the code
        code = lib.cb_probe_mma_send(ctypes.c_int(m), ctypes.c_int(n), ctypes.c_int(count),
                                     ctypes.c_int(1 if tight else 0), _vp(out), _vp(status), _stream())
        if code != 0:
            raise RuntimeError(f"the MMA probe was refused or failed to launch (code {code})")
        torch.cuda.synchronize(device)
    tensor_core.check_status(device)
    return out.item() / count


def tma_send_cycles(rows: int, count: int = 32, device="cuda:0"):
    """(cycles per box for the sending loop, cycles per box until all have landed) when one
    thread sends `count` boxes of `rows` x 128 bytes."""
    lib = build.load("issue_probe")
    matrix = torch.zeros((256, 2048), dtype=torch.bfloat16, device=device)
    out = torch.zeros(2, dtype=torch.int64, device=device)
    status = tensor_core.status_word(device)
    for _ in range(2):
        code = lib.cb_probe_tma_send(_vp(matrix), ctypes.c_int(256), ctypes.c_int(2048), ctypes.c_int(rows),
                                     ctypes.c_int(count), _vp(out), _vp(status), _stream())
        if code != 0:
            raise RuntimeError(f"the TMA probe was refused or failed to launch (code {code})")
        torch.cuda.synchronize(device)
    tensor_core.check_status(device)
    sent, landed = out.tolist()
    return sent / count, landed / count


def main() -> None:
    for m, n in ((128, 64), (128, 128), (128, 256), (64, 64)):
        tight, plain = mma_send_cycles(m, n, tight=True), mma_send_cycles(m, n, tight=False)
        print(f"tcgen05.mma {m} x {n} x 16 sent by one thread: {tight:6.1f} cycles each with loop-invariant "
              f"descriptors, {plain:6.1f} with descriptors and flag computed per MMA "
              f"(the tensor cores' own time: {n / 2:.0f})")
    for rows in (16, 64, 128):
        sent, landed = tma_send_cycles(rows)
        print(f"TMA box of {rows:3d} rows x 128 B sent by one thread: {sent:6.1f} cycles each to send, "
              f"{landed:6.1f} until all have landed")


if __name__ == "__main__":
    main()
