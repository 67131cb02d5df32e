"""The C-ABI library loads without a GPU and exports every function the public headers declare."""
import ctypes as C
import pathlib
import re

ROOT = pathlib.Path(__file__).resolve().parents[1]
DECL = re.compile(r"^\s*(?:const\s+)?[A-Za-z_][\w\s\*]*?\b(srt_\w+)\s*\(", re.M)


def header_functions():
    names = {}
    for h in sorted((ROOT / "include").glob("*.h")):
        text = re.sub(r"/\*.*?\*/", "", h.read_text(), flags=re.S)
        text = re.sub(r"//[^\n]*", "", text)
        text = re.sub(r"^\s*#[^\n]*(?:\\\n[^\n]*)*", "", text, flags=re.M)
        for m in DECL.finditer(text):
            line = text[text.rfind("\n", 0, m.start()) + 1:m.end()]
            if "typedef" in line:
                continue
            names.setdefault(m.group(1), h.name)
    return names


def test_headers_declare_functions():
    names = header_functions()
    assert len(names) > 100, len(names)
    for must in ("srt_conv_fprop", "srt_step_forward_backward", "srt_pool_alloc", "srt_comm_open", "srt_stub_create"):
        assert must in names, must


def test_library_exports_every_declared_function():
    from sirius_b200 import _lib
    lib = _lib.lib()
    missing = [f"{n} ({h})" for n, h in header_functions().items() if not hasattr(lib, n)]
    assert not missing, missing


def test_every_declared_function_has_a_python_signature():
    from sirius_b200 import _lib, _runtime, bert_infer, ddp, gpt2_step, ops, pool, qwen2_step, server, step, swin_step  # noqa: F401  (each registers its signatures)
    bound = set(_lib.declared_symbols())
    unbound = sorted(set(header_functions()) - bound)
    assert not unbound, unbound
    extra = sorted(n for n in bound if n not in header_functions())
    assert not extra, f"bound in Python but not declared in include/: {extra}"


def test_error_string_and_version_calls_need_no_gpu():
    from sirius_b200 import _lib
    lib = _lib.lib()
    lib.srt_last_error.restype = C.c_char_p
    assert isinstance(lib.srt_last_error(), bytes)


def test_conv_bn_stats_sizing_and_support_are_host_side():
    """srt_conv_fprop_bn_stats_bytes / _supported do no device work: one double2 per 128-row tile and output
    channel, and only the bf16 tensor-core path has the statistics epilogue."""
    from sirius_b200 import _lib
    from sirius_b200._lib import IMPL_AUTO, IMPL_SIMT, IMPL_TCGEN05, SRT_BF16, SRT_F32, ConvDesc
    lib = _lib.lib()
    for (N, H, W, Cin, K, R, stride, pad) in ((64, 56, 56, 64, 256, 1, 1, 0), (3, 9, 11, 24, 40, 3, 1, 1), (2, 28, 28, 128, 128, 3, 2, 1)):
        d = ConvDesc.make(N, H, W, Cin, K, R, R, stride, pad)
        rows = N * d.P * d.Q
        assert lib.srt_conv_fprop_bn_stats_bytes(C.byref(d)) == -(-rows // 128) * K * 16
        assert lib.srt_conv_fprop_bn_stats_supported(C.byref(d), SRT_BF16, IMPL_AUTO) == 1
        assert lib.srt_conv_fprop_bn_stats_supported(C.byref(d), SRT_BF16, IMPL_TCGEN05) == 1
        assert lib.srt_conv_fprop_bn_stats_supported(C.byref(d), SRT_BF16, IMPL_SIMT) == 0
        assert lib.srt_conv_fprop_bn_stats_supported(C.byref(d), SRT_F32, IMPL_AUTO) == 0
    assert lib.srt_conv_fprop_bn_stats_bytes(None) == 0


def test_gradient_exchange_entry_points_fail_cleanly_without_a_communicator():
    """The NCCL-backed exchange is resolved at run time: loading the library needs neither NCCL nor a GPU, and
    calls with a missing communicator or arguments return an error status with a message instead of crashing."""
    from sirius_b200 import _lib, ddp
    lib = _lib.lib()
    assert lib.srt_ddp_available() in (0, 1)
    off, cnt = (C.c_int64 * 1)(0), (C.c_int64 * 1)(8)
    assert lib.srt_allreduce_begin(None, None, 1, off, cnt, None, _lib.SRT_F32) != 0
    assert b"allreduce_begin" in lib.srt_last_error()
    assert lib.srt_allreduce_wait(None, None) != 0
    assert lib.srt_ddp_allreduce(None, None, 0, _lib.SRT_F32, None) != 0
    assert lib.srt_ddp_destroy(None) == 0
    assert ddp.WIRE["bf16"] == _lib.SRT_BF16


def test_filter_gradient_pair_switch_does_not_change_the_scratch_a_caller_sized():
    """srt_conv_wgrad_pairs flips which kernel a filter gradient takes, process-wide, at any time (the gradient
    exchange turns the pairs off); the scratch size reported for a problem covers both kernels, so scratch sized
    before the flip is still enough after it. The call returns the previous setting; -1 only reads."""
    import ctypes as C
    from sirius_b200 import _lib
    from sirius_b200._lib import ConvDesc, IMPL_AUTO, SRT_BF16
    lib = _lib.lib()
    lib.srt_conv_wgrad_scratch_bytes.restype = C.c_size_t
    start = lib.srt_conv_wgrad_pairs(-1)
    try:
        for shape in ((64, 14, 14, 256, 256, 3, 3, 1, 1), (64, 14, 14, 1024, 256, 1, 1, 1, 0), (64, 56, 56, 64, 64, 3, 3, 1, 1),
                      (8192, 1, 1, 768, 50304, 1, 1, 1, 0), (64, 7, 7, 512, 2048, 1, 1, 1, 0), (5, 9, 11, 24, 40, 3, 3, 1, 1)):
            d = ConvDesc.make(*shape)
            assert lib.srt_conv_wgrad_pairs(1) in (0, 1)
            on = lib.srt_conv_wgrad_scratch_bytes(C.byref(d), SRT_BF16, IMPL_AUTO)
            assert lib.srt_conv_wgrad_pairs(0) == 1
            off = lib.srt_conv_wgrad_scratch_bytes(C.byref(d), SRT_BF16, IMPL_AUTO)
            assert lib.srt_conv_wgrad_pairs(-1) == 0
            assert on == off, shape
    finally:
        lib.srt_conv_wgrad_pairs(start)
