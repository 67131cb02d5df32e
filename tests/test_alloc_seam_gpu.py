"""The allocator seam and the shared pool on a GPU.

1. PyTorch with srt_alloc / srt_free as its CUDA allocator (torch.cuda.memory.CUDAPluggableAllocator), in a
   child process because the allocator has to be installed before the first CUDA allocation: tensors come out of
   the pool's training allocator, a block freed while a side stream still uses it is held back until that stream
   has passed the free (srt_record_stream), tagged intermediates are dropped at once, and empty-cache returns
   whole pages to the pool.
2. Two processes on one CUDA-VMM pool: the owner (the inference server's role) creates it, the child (a
   trainer) attaches through the exported page handles; pages the trainer releases are mapped and used by
   the owner's kernels, and come back."""
import ctypes as C
import multiprocessing as mp
import os
import uuid

import pytest
import torch

pytestmark = pytest.mark.gpu


def _torch_on_the_pool(q):
    try:
        os.environ["SIRIUS_PORT"] = f"{30000 + os.getpid() % 20000}"
        os.environ.pop("COLTRAIN_HAS_SHARED_TENSOR_SERVER", None)
        import torch
        from sirius_b200 import _lib, _runtime  # noqa: F401
        from sirius_b200._lib import LIB_PATH, call
        lib = _lib.lib()
        PAGE = 32 << 20
        call("srt_pool_init", 0, 2 << 30, 1)
        alloc = torch.cuda.memory.CUDAPluggableAllocator(str(LIB_PATH), "srt_alloc", "srt_free")
        torch.cuda.memory.change_current_allocator(alloc)
        stat = lambda w: lib.srt_pool_stat_dev(0, w)
        pages0 = stat(4)
        x = torch.randn(4096, 4096, device="cuda")               # 64 MiB from the pool
        y = torch.randn(4096, 4096, device="cuda")
        z = (x @ y).relu_()                                        # cuBLAS workspace and result come from it too
        ref = (x.cpu() @ y.cpu()).relu_()
        assert torch.allclose(z.cpu(), ref, rtol=2e-2, atol=2e-1)
        assert stat(1) >= 3 * 64 << 20 and stat(4) < pages0      # train usage, fewer free pages
        counters = lambda: [v.value for v in _counters(lib)]
        # record_stream: a block freed while a side stream may still read it is not reused until that stream got there
        side = torch.cuda.Stream()
        big = torch.full((16 << 20,), 3.0, device="cuda")         # 64 MiB
        ptr = big.data_ptr()
        with torch.cuda.stream(side):
            warm = big[:1024].sum()                                # loads the reduction kernels now, not inside the window
        torch.cuda.synchronize()
        with torch.cuda.stream(side):
            torch.cuda._sleep(2_000_000_000)                       # ~1 s of side-stream work queued before the use
            s = big.sum()
        call("srt_record_stream", C.c_void_p(ptr), 0, C.c_void_p(side.cuda_stream))
        del big
        c = counters()
        assert c[2] == 1 and c[3] == 1, (c, side.query())         # one deferred free, still pending
        again = torch.empty(16 << 20, device="cuda")
        assert again.data_ptr() != ptr                             # its memory is not handed out yet
        side.synchronize()
        assert float(s) == 3.0 * (16 << 20)
        del again
        tmp = torch.empty(1024, device="cuda")                     # any call processes the finished events
        assert counters()[3] == 0
        # tagged intermediates go in one call while their tensors still exist
        acts = [torch.empty(48 << 20, dtype=torch.uint8, device="cuda") for _ in range(4)]
        for a in acts:
            call("srt_tag_interm", C.c_void_p(a.data_ptr()), 0)
        torch.cuda.synchronize()
        free_before = stat(4)
        rel = C.c_size_t()
        call("srt_release_interm", 0, C.byref(rel))
        assert rel.value >= 4 * PAGE and stat(4) == free_before + rel.value // PAGE
        fresh = torch.ones(40 << 20, dtype=torch.uint8, device="cuda")
        assert fresh.data_ptr() not in [a.data_ptr() for a in acts]
        del acts                                                   # the framework's late frees are harmless
        assert int(fresh.sum()) == 40 << 20
        del fresh, x, y, z, tmp, s, ref, warm
        torch.cuda.synchronize()
        call("srt_empty_cache", 0, C.byref(rel))
        # what stays is what PyTorch keeps for itself (the cuBLAS workspace)
        assert stat(1) <= 64 << 20, stat(1)
        assert stat(4) >= pages0 - 3
        q.put("ok")
    except BaseException as e:  # noqa: BLE001
        import traceback
        q.put("".join(traceback.format_exception(e)))


def _counters(lib):
    from sirius_b200._lib import call
    n = [C.c_int64() for _ in range(5)]
    call("srt_alloc_counters", 0, *[C.byref(v) for v in n])
    return n


@pytest.mark.timeout(300)
def test_pytorch_allocates_from_the_pool_through_the_pluggable_allocator():
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    p = ctx.Process(target=_torch_on_the_pool, args=(q,))
    p.start()
    msg = q.get(timeout=240)
    p.join(60)
    assert msg == "ok", msg
    assert p.exitcode == 0


def _attached_trainer(name, q_in, q_out):
    try:
        import torch
        from sirius_b200.pool import TRAIN, PagePool
        torch.cuda.set_device(0)
        pool = PagePool.attach(name, device=0, timeout_ms=20000)
        page = pool.stat("page_nbytes")
        n = 8
        ptr = pool.alloc(TRAIN, n * page)

        class Buf:
            __cuda_array_interface__ = {"shape": (n * page,), "typestr": "|u1", "data": (ptr, False), "version": 2}
        t = torch.as_tensor(Buf(), device="cuda:0")
        t.fill_(0x5a)
        torch.cuda.synchronize()
        q_out.put(("allocated", pool.stat("train_all"), pool.stat("free_pages")))
        assert q_in.get(timeout=60) == "release"
        del t
        pool.free(TRAIN, ptr)
        released = pool.empty_cache(TRAIN)
        q_out.put(("released", released))
        assert q_in.get(timeout=60) == "regain"
        ptr2 = pool.alloc(TRAIN, n * page)

        class Buf2:
            __cuda_array_interface__ = {"shape": (n * page,), "typestr": "|u1", "data": (ptr2, False), "version": 2}
        t2 = torch.as_tensor(Buf2(), device="cuda:0")
        t2.fill_(1)
        assert int(t2[:: page // 4].sum()) == 4 * n
        q_out.put(("regained", pool.stat("num_reuse")))
        del t2
        pool.free(TRAIN, ptr2)
        pool.close()
        q_out.put(("ok",))
    except BaseException as e:  # noqa: BLE001
        import traceback
        q_out.put(("error", "".join(traceback.format_exception(e))))


@pytest.mark.timeout(300)
def test_two_processes_trade_device_pages_of_one_pool():
    from sirius_b200.pool import INFER, PagePool
    name = f"srt_gpu_pool_{os.getpid()}_{uuid.uuid4().hex[:6]}"
    server = PagePool(0.5, device=0, shared_name=name)            # 16 pages of 32 MiB
    page = server.stat("page_nbytes")
    ctx = mp.get_context("spawn")
    q_in, q_out = ctx.Queue(), ctx.Queue()
    child = ctx.Process(target=_attached_trainer, args=(name, q_in, q_out))
    child.start()
    try:
        msg = q_out.get(timeout=120)
        assert msg[0] == "allocated", msg
        assert msg[1] == 8 * page and server.stat("train_all") == 8 * page and server.stat("free_pages") == 8
        q_in.put("release")
        msg = q_out.get(timeout=60)
        assert msg == ("released", 8 * page), msg
        # the owner maps all 16 pages, 8 of which the other process just gave up, and computes on them
        p = server.alloc(INFER, 16 * page)

        class Buf:
            __cuda_array_interface__ = {"shape": (16 * page // 4,), "typestr": "<f4", "data": (p, False), "version": 2}
        t = torch.as_tensor(Buf(), device="cuda:0")
        t.fill_(2.0)
        assert float(t.sum()) == 2.0 * (16 * page // 4)
        assert server.stat("free_pages") == 0
        del t
        server.free(INFER, p)
        assert server.empty_cache(INFER) == 16 * page
        q_in.put("regain")
        msg = q_out.get(timeout=60)
        assert msg[0] == "regained" and msg[1] >= 8, msg          # kept mappings taken back without driver calls
        assert q_out.get(timeout=60) == ("ok",)
    finally:
        child.join(60)
        if child.is_alive():
            child.terminate()
        server.close()
    assert child.exitcode == 0
