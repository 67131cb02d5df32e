"""The PyTorch allocator seam (srt_alloc / srt_free and friends) on the host backend: sizes, alignment, live
accounting, tagging of intermediate blocks, release of all tagged blocks while their pointers are still held
(the hazard: such an address must not be handed out again before its holder frees it), and error statuses
instead of aborts. Stream-ordered deferred frees need CUDA events and are covered by the GPU test."""
import ctypes as C
import os
import uuid

import pytest

from sirius_b200 import _lib, _runtime  # noqa: F401
from sirius_b200._lib import SrtError, call

DEV = 5      # any slot of the per-device table; nothing here touches a GPU
PAGE = 2 << 20


@pytest.fixture()
def seam():
    os.environ["SIRIUS_B200_POOL_HOST_BACKEND"] = "1"
    os.environ["SIRIUS_B200_POOL_PAGE_MB"] = "2"
    os.environ["SIRIUS_PORT"] = str(20000 + os.getpid() % 20000) + uuid.uuid4().hex[:4]
    os.environ.pop("COLTRAIN_HAS_SHARED_TENSOR_SERVER", None)
    call("srt_pool_init", DEV, 32 << 20, 1)
    yield _lib.lib()
    call("srt_pool_shutdown", DEV)
    for k in ("SIRIUS_B200_POOL_HOST_BACKEND", "SIRIUS_B200_POOL_PAGE_MB", "SIRIUS_PORT"):
        os.environ.pop(k, None)


def _stat(lib, which): return lib.srt_pool_stat_dev(DEV, which)


def test_alloc_free_and_accounting(seam):
    lib = seam
    assert lib.srt_alloc(0, DEV, None) is None
    a = lib.srt_alloc(3 * PAGE + 100, DEV, None)
    b = lib.srt_alloc(1000, DEV, None)
    assert a and b and a % 1024 == 0 and b % 1024 == 0
    C.memset(a, 1, 3 * PAGE + 100)
    assert _stat(lib, 1) >= 3 * PAGE + 100 + 1000            # train usage
    n = [C.c_int64() for _ in range(5)]
    call("srt_alloc_counters", DEV, *[C.byref(v) for v in n])
    assert [v.value for v in n] == [2, 0, 0, 0, 2]
    lib.srt_free(a, 3 * PAGE + 100, DEV, None)
    lib.srt_free(b, 1000, DEV, None)
    rel = C.c_size_t()
    call("srt_empty_cache", DEV, C.byref(rel))
    assert rel.value == 4 * PAGE and _stat(lib, 4) == 16    # every page is free again
    # an unknown pointer or an uninitialised device is an error message, not a crash
    lib.srt_free(12345 * 1024, 1, DEV, None)
    assert b"was not allocated" in lib.srt_last_error()
    assert lib.srt_alloc(64, DEV + 1, None) is None and b"srt_pool_init" in lib.srt_last_error()
    with pytest.raises(SrtError):
        call("srt_record_stream", C.c_void_p(999 * 1024), DEV, None)


def test_release_of_tagged_blocks_keeps_their_addresses_reserved(seam):
    lib = seam
    call("srt_tag_model_begin")
    weights = lib.srt_alloc(PAGE, DEV, None)
    call("srt_tag_interm", C.c_void_p(weights), DEV)          # ignored during model set-up
    call("srt_tag_model_end")
    acts = [lib.srt_alloc(3 * PAGE, DEV, None) for _ in range(3)]
    for p in acts:
        call("srt_tag_interm", C.c_void_p(p), DEV)
    keep = lib.srt_alloc(PAGE, DEV, None)                     # an untagged block allocated in between
    free_before = _stat(lib, 4)
    rel = C.c_size_t()
    call("srt_release_interm", DEV, C.byref(rel))
    assert rel.value >= 8 * PAGE and _stat(lib, 4) == free_before + rel.value // PAGE
    # new allocations never land on an address whose old holder has not freed it yet
    fresh = [lib.srt_alloc(3 * PAGE, DEV, None) for _ in range(2)]
    assert all(f and f not in acts for f in fresh)
    C.memset(fresh[0], 7, 3 * PAGE)
    # the framework now drops the dead tensors: no double free, no damage to the fresh blocks
    for p in acts:
        lib.srt_free(p, 3 * PAGE, DEV, None)
    assert bytes((C.c_ubyte * 2).from_address(fresh[0])) == b"\x07\x07"
    for p in fresh + [keep, weights]:
        lib.srt_free(p, 1, DEV, None)
    call("srt_empty_cache", DEV, C.byref(rel))
    assert _stat(lib, 4) == 16 and _stat(lib, 1) == 0
    n = [C.c_int64() for _ in range(5)]
    call("srt_alloc_counters", DEV, *[C.byref(v) for v in n])
    assert n[4].value == 0


def test_out_of_memory_is_null_with_a_message(seam):
    lib = seam
    a = lib.srt_alloc(30 << 20, DEV, None)
    assert a
    assert lib.srt_alloc(8 << 20, DEV, None) is None
    assert b"pool has" in lib.srt_last_error() or b"no contiguous" in lib.srt_last_error()
    lib.srt_free(a, 30 << 20, DEV, None)
