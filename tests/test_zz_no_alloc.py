"""srt_bn_stats_static: BatchNorm statistics with the partial sums in the library's built-in array.

Collected last on purpose (file name), so a run that stops at the first failure has already run
every other test. The entry point is for callers that cannot allocate scratch (a trainer in the
middle of handing its memory to the colocated inference server, or a control thread that must not
block in the allocator); it has to give exactly what srt_bn_stats gives with caller scratch, call
after call, although all calls share one array that still holds the previous call's partial sums.
"""
import ctypes as C

import pytest
import torch

pytestmark = pytest.mark.gpu

from sirius_b200 import _lib
from sirius_b200._lib import SRT_BF16, SRT_F32, call

DEV = "cuda:0"


def _both(z, gamma, beta, seed_stats):
    """Runs the regular and the allocation-free entry point on the same input; returns both results."""
    Cc = z.shape[-1]
    rows = z.numel() // Cc
    dt = SRT_F32 if z.dtype == torch.float32 else SRT_BF16
    stream = torch.cuda.current_stream().cuda_stream
    outs = []
    for static in (False, True):
        rm, rv = seed_stats[0].clone(), seed_stats[1].clone()
        o = [torch.empty(Cc, dtype=torch.float32, device=DEV) for _ in range(4)]
        if static:
            call("srt_bn_stats_static", dt, z.data_ptr(), rows, Cc, gamma.data_ptr(), beta.data_ptr(), 1e-5, 0.1,
                 rm.data_ptr(), rv.data_ptr(), *(t.data_ptr() for t in o), stream)
        else:
            n = _lib.lib().srt_bn_scratch_bytes(rows, Cc)
            scratch = torch.empty(n, dtype=torch.uint8, device=DEV)
            call("srt_bn_stats", dt, z.data_ptr(), rows, Cc, gamma.data_ptr(), beta.data_ptr(), 1e-5, 0.1,
                 rm.data_ptr(), rv.data_ptr(), *(t.data_ptr() for t in o), scratch.data_ptr(), n, stream)
        torch.cuda.synchronize()
        outs.append([rm, rv] + o)
    return outs


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_static_scratch_matches_caller_scratch_on_consecutive_calls(dtype):
    g = torch.Generator().manual_seed(11)
    # two calls in a row with different shapes and data: the second finds the first one's partial
    # sums in the shared array and must not be influenced by them
    for shape in ((4, 14, 14, 256), (2, 28, 28, 64)):
        Cc = shape[-1]
        z = (torch.randn(shape, generator=g) * 3 + 1).to(DEV, dtype)
        gamma = (torch.rand(Cc, generator=g) + 0.5).to(DEV)
        beta = torch.randn(Cc, generator=g).to(DEV)
        stats = (torch.randn(Cc, generator=g).to(DEV), (torch.rand(Cc, generator=g) + 0.5).to(DEV))
        ref, got = _both(z, gamma, beta, stats)
        for a, b in zip(ref, got):
            # same kernels, same order of summation: the tolerance of the other BatchNorm tests (1e-5)
            # is met with equality
            assert torch.allclose(a, b, rtol=1e-5, atol=1e-6)
            assert torch.equal(a, b)


def test_calls_after_the_prepared_one_leave_free_device_memory_unchanged():
    """After srt_bn_static_prepare() and one warm call, further calls (here on a non-default stream, back to back,
    which is how a handover would issue them) change the free device memory by not one byte: neither the entry
    point nor anything under it allocates."""
    call("srt_bn_static_prepare")
    g = torch.Generator().manual_seed(5)
    Cc, shape = 128, (8, 28, 28, 128)
    z = (torch.randn(shape, generator=g) * 2).to(DEV, torch.bfloat16)
    rows = z.numel() // Cc
    gamma, beta = torch.ones(Cc, device=DEV), torch.zeros(Cc, device=DEV)
    rm, rv = torch.zeros(Cc, device=DEV), torch.ones(Cc, device=DEV)
    o = [torch.empty(Cc, dtype=torch.float32, device=DEV) for _ in range(4)]
    side = torch.cuda.Stream()
    args = (SRT_BF16, z.data_ptr(), rows, Cc, gamma.data_ptr(), beta.data_ptr(), 1e-5, 0.1, rm.data_ptr(), rv.data_ptr(),
            *(t.data_ptr() for t in o))
    call("srt_bn_stats_static", *args, side.cuda_stream)          # warm call
    torch.cuda.synchronize()
    first = [t.clone() for t in o]
    free_before, _ = torch.cuda.mem_get_info()
    for _ in range(6):                                            # consecutive calls on the same stream: ordered, no race
        call("srt_bn_stats_static", *args, side.cuda_stream)
    torch.cuda.synchronize()
    free_after, _ = torch.cuda.mem_get_info()
    assert free_after == free_before
    for a, b in zip(first, o):                                    # mean / invstd / scale / shift do not depend on the running stats
        assert torch.equal(a, b)


def test_static_scratch_rejects_oversized_problem():
    # the smallest power-of-two row count of a 32768-channel tensor whose slab partials exceed the 4 MiB
    Cc, rows = 32768, 1024
    while _lib.lib().srt_bn_scratch_bytes(rows, Cc) <= (4 << 20) and rows < (1 << 16):
        rows *= 2
    assert _lib.lib().srt_bn_scratch_bytes(rows, Cc) > (4 << 20)
    z = torch.empty(rows, Cc, device=DEV)
    o = [torch.empty(Cc, dtype=torch.float32, device=DEV) for _ in range(4)]
    status = _lib.lib().srt_bn_stats_static(SRT_F32, z.data_ptr(), rows, Cc, None, None, 1e-5, 0.1, None, None,
                                            *(t.data_ptr() for t in o), torch.cuda.current_stream().cuda_stream)
    assert status == 1  # SRT_ERR_INVALID
    msg = _lib.lib().srt_last_error().decode()
    assert "built-in scratch" in msg and "srt_bn_stats" in msg
