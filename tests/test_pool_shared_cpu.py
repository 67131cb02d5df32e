"""The page pool shared between two processes, on the host backend (a memfd stands in for device pages): the
owner plays the inference server, a child process attaches as the trainer. What the reference's design promises
(common/cuda_allocator.cc:61-99: pool and allocators in shared memory, created by one process, opened by the
others): the trainer's empty-cache makes pages available to the server's allocator in the other process, both see
the same ownership counters, a page really is the same memory in both, and nobody attaches to a dead owner."""
import ctypes as C
import multiprocessing as mp
import os
import uuid

import pytest

from sirius_b200._lib import SrtError
from sirius_b200.pool import INFER, TRAIN, PagePool

PAGE_MB, POOL_MB = 2, 32
PAGE = PAGE_MB << 20


def _trainer(name, q_in, q_out):
    pool = PagePool.attach(name, timeout_ms=5000)
    try:
        assert pool.stat("pool_nbytes") == POOL_MB << 20 and pool.stat("page_nbytes") == PAGE
        blocks = [pool.alloc(TRAIN, 3 * PAGE) for _ in range(4)]          # 12 of 16 pages
        for i, b in enumerate(blocks):
            C.memset(b, 0x40 + i, 3 * PAGE)
        q_out.put(("allocated", pool.stat("train_all"), pool.stat("free_pages")))
        assert q_in.get(timeout=30) == "release"                          # the adjust: hand memory over
        for b in blocks[1:]:
            pool.free(TRAIN, b)
        released = pool.empty_cache(TRAIN)
        q_out.put(("released", released, pool.stat("free_pages"), pool.stat("infer_usage")))
        assert q_in.get(timeout=30) == "regain"                           # inference went idle
        again = pool.alloc(TRAIN, 9 * PAGE)
        first = bytes((C.c_ubyte * 4).from_address(blocks[0]))            # the block that stayed is untouched
        q_out.put(("regained", pool.stat("train_all"), pool.stat("num_reuse"), list(first)))
        pool.free(TRAIN, again)
        pool.free(TRAIN, blocks[0])
        assert q_in.get(timeout=30) == "exit"
    finally:
        pool.close()
    q_out.put(("closed",))


@pytest.mark.timeout(120)
def test_pages_released_by_one_process_are_mapped_by_the_other():
    name = f"srt_pool_test_{os.getpid()}_{uuid.uuid4().hex[:6]}"
    server = PagePool(POOL_MB / 1024, page_mb=PAGE_MB, host_backend=True, shared_name=name)
    ctx = mp.get_context("spawn")
    q_in, q_out = ctx.Queue(), ctx.Queue()
    child = ctx.Process(target=_trainer, args=(name, q_in, q_out))
    child.start()
    try:
        tag, train_all, free_pages = q_out.get(timeout=60)
        assert tag == "allocated" and train_all == 12 * PAGE and free_pages == 4
        # the server sees the trainer's footprint and cannot take more than what is free
        assert server.stat("train_all") == 12 * PAGE and server.stat("free_pages") == 4
        with pytest.raises(SrtError):
            server.alloc(INFER, 6 * PAGE)
        q_in.put("release")
        tag, released, free_pages, _ = q_out.get(timeout=30)
        assert tag == "released" and released == 9 * PAGE and free_pages == 13
        # handover: the pages the trainer released are now backing the server's allocation, in this process
        p = server.alloc(INFER, 12 * PAGE)
        assert server.stat("infer_usage") == 12 * PAGE and server.stat("free_pages") == 1
        C.memset(p, 0x7f, 12 * PAGE)
        assert bytes((C.c_ubyte * 2).from_address(p + 12 * PAGE - 2)) == b"\x7f\x7f"
        server.free(INFER, p)
        assert server.empty_cache(INFER) == 12 * PAGE
        q_in.put("regain")
        tag, train_all, reuse, first = q_out.get(timeout=30)
        assert tag == "regained" and train_all == 12 * PAGE
        assert reuse >= 9            # the trainer's slots took their kept pages back without mapping calls
        assert first == [0x40] * 4
        q_in.put("exit")
        assert q_out.get(timeout=30) == ("closed",)
        # a process that detaches returns what it still held
        assert server.stat("free_pages") == 16 and server.stat("train_all") == 0
    finally:
        child.join(30)
        if child.is_alive():
            child.terminate()
        server.close()
    assert child.exitcode == 0


def test_the_same_page_is_the_same_memory_in_both_processes():
    """One page in the pool: what the owner writes through its mapping, the attached process reads through its
    own mapping after the page changed hands."""
    name = f"srt_pool_one_{os.getpid()}_{uuid.uuid4().hex[:6]}"
    server = PagePool(PAGE_MB / 1024, page_mb=PAGE_MB, host_backend=True, shared_name=name)
    other = PagePool.attach(name)
    try:
        a = server.alloc(INFER, PAGE)
        C.memmove(a, b"handover", 8)
        server.free(INFER, a)
        server.empty_cache(INFER)
        b = other.alloc(TRAIN, PAGE)
        assert a != b or True       # different virtual ranges as a rule; the physical page is the only one there is
        assert bytes((C.c_ubyte * 8).from_address(b)) == b"handover"
        other.free(TRAIN, b)
    finally:
        other.close()
        server.close()


def test_no_attach_without_a_live_owner():
    """A segment whose owner is gone (here: never existed, and: was closed) cannot be attached to; the error is a
    status with a message, not a hang."""
    with pytest.raises(SrtError, match="no live pool"):
        PagePool.attach(f"srt_pool_nobody_{uuid.uuid4().hex[:6]}", timeout_ms=50)
    name = f"srt_pool_gone_{os.getpid()}_{uuid.uuid4().hex[:6]}"
    PagePool(PAGE_MB / 1024, page_mb=PAGE_MB, host_backend=True, shared_name=name).close()
    with pytest.raises(SrtError, match="no live pool"):
        PagePool.attach(name, timeout_ms=50)
    # and a second owner under a live name is refused
    first = PagePool(PAGE_MB / 1024, page_mb=PAGE_MB, host_backend=True, shared_name=name)
    try:
        with pytest.raises(SrtError, match="alive already"):
            PagePool(PAGE_MB / 1024, page_mb=PAGE_MB, host_backend=True, shared_name=name)
    finally:
        first.close()
