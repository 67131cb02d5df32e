"""Per-operator parity on the GPU: every kernel family, called through the C ABI, against the
PyTorch CPU fp32 operator the reference's training scripts execute (train/resnet152.py:86-89).

fp32 kernels: tight tolerance. bf16 kernels: inputs are rounded to bf16 first so the only
differences are accumulation order and the final rounding to bf16.
"""
import pytest
import torch
import torch.nn.functional as F

pytestmark = pytest.mark.gpu

from sirius_b200 import ops
from sirius_b200._lib import IMPL_SIMT, IMPL_TCGEN05, IMPL_AUTO, lib

DEV = "cuda:0"

# (name, N, H, W, C, K, R, S, stride, pad)
CONV_CASES = [
    ("1x1_s1_c256_k64", 2, 14, 14, 256, 64, 1, 1, 1, 0),
    ("1x1_s1_c64_k256", 3, 14, 14, 64, 256, 1, 1, 1, 0),
    ("3x3_s1_c64_k64", 2, 14, 14, 64, 64, 3, 3, 1, 1),
    ("3x3_s1_c128_k128", 2, 14, 14, 128, 128, 3, 3, 1, 1),
    ("3x3_s2_c128_k128", 2, 28, 28, 128, 128, 3, 3, 2, 1),
    ("1x1_s2_c256_k512", 2, 28, 28, 256, 512, 1, 1, 2, 0),
    ("7x7_s2_c8_k64_stem", 2, 64, 64, 8, 64, 7, 7, 2, 3),
    ("fc_2048_1000", 64, 1, 1, 2048, 1000, 1, 1, 1, 0),
    ("tail_7x7_c512_k512", 1, 7, 7, 512, 512, 3, 3, 1, 1),
    ("odd_c24_k40", 2, 9, 11, 24, 40, 3, 3, 1, 1),
]
IDS = [c[0] for c in CONV_CASES]


def _mk(case, dtype, seed=0):
    _, N, H, W, C, K, R, S, stride, pad = case
    g = torch.Generator().manual_seed(seed)
    x = torch.randn(N, H, W, C, generator=g)
    w = torch.randn(K, R, S, C, generator=g) * (1.0 / (R * S * C) ** 0.5)
    P = (H + 2 * pad - R) // stride + 1
    Q = (W + 2 * pad - S) // stride + 1
    dy = torch.randn(N, P, Q, K, generator=g)
    if dtype == torch.bfloat16:
        x, w, dy = (t.to(torch.bfloat16).float() for t in (x, w, dy))
    return x, w, dy


def _ref(x, w, dy, stride, pad):
    xn = x.permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    wn = w.permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    y = F.conv2d(xn, wn, stride=stride, padding=pad)
    y.backward(dy.permute(0, 3, 1, 2).contiguous())
    return (y.detach().permute(0, 2, 3, 1).contiguous(),
            xn.grad.permute(0, 2, 3, 1).contiguous(),
            wn.grad.permute(0, 2, 3, 1).contiguous())


def _err(a, b):
    return ((a.float().cpu() - b).abs().max() / (b.abs().max() + 1e-12)).item()


@pytest.mark.parametrize("case", CONV_CASES, ids=IDS)
def test_conv_fp32_simt(case):
    stride, pad = case[8], case[9]
    x, w, dy = _mk(case, torch.float32)
    y_ref, dx_ref, dw_ref = _ref(x, w, dy, stride, pad)
    xd, wd, dyd = x.to(DEV), w.to(DEV), dy.to(DEV)
    y = ops.conv_fprop(xd, wd, stride, pad)
    dx = ops.conv_dgrad(dyd, ops.filter_transpose(wd), x.shape, stride, pad)
    dw = ops.conv_wgrad(dyd, xd, case[6], case[7], stride, pad)
    torch.cuda.synchronize()
    assert _err(y, y_ref) < 2e-5
    assert _err(dx, dx_ref) < 2e-5
    assert _err(dw, dw_ref) < 2e-5


def _run_bf16(case, impl):
    stride, pad = case[8], case[9]
    x, w, dy = _mk(case, torch.bfloat16)
    y_ref, dx_ref, dw_ref = _ref(x, w, dy, stride, pad)
    bf = torch.bfloat16
    xd, wd, dyd = x.to(DEV, bf), w.to(DEV, bf), dy.to(DEV, bf)
    y = ops.conv_fprop(xd, wd, stride, pad, impl=impl)
    dx = ops.conv_dgrad(dyd, ops.filter_transpose(wd), x.shape, stride, pad, impl=impl)
    dw = ops.conv_wgrad(dyd, xd, case[6], case[7], stride, pad, impl=impl)
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    errs = (_err(y, y_ref), _err(dx, dx_ref), _err(dw, dw_ref))
    print(case[0], "impl", impl, "rel-max errors y/dx/dw:", errs)
    assert errs[0] < 1e-2 and errs[1] < 1e-2
    assert errs[2] < 2e-3  # fp32 output


@pytest.mark.parametrize("case", CONV_CASES, ids=IDS)
def test_conv_bf16_simt(case):
    _run_bf16(case, IMPL_SIMT)


# fprop/dgrad kernel plans (gather, tile width, CTA pair): the heuristic, every forced tile width with one CTA
# per 128-row tile, and two CTAs per 256-row tile (tcgen05 cta_group::2) with each of its tile widths
PLANS = {"auto": (0, 0, -1), "single_bn64": (0, 64, 0), "single_bn128": (0, 128, 0), "single_bn256": (0, 256, 0),
         "pair_bn128": (0, 128, 1), "pair_bn256": (0, 256, 1), "gather": (1, 0, -1), "gather_pair": (1, 0, 1)}


def _with_plan(plan, fn):
    lib().srt_conv_plan_override(*plan)
    try:
        return fn()
    finally:
        lib().srt_conv_plan_override(0, 0, -1)


@pytest.mark.parametrize("plan", list(PLANS), ids=list(PLANS))
@pytest.mark.parametrize("case", CONV_CASES, ids=IDS)
def test_conv_bf16_tcgen05(case, plan):
    _with_plan(PLANS[plan], lambda: _run_bf16(case, IMPL_TCGEN05))


def test_conv_tcgen05_many_tiles_per_cta():
    """More tiles than SMs with a short reduction: the persistent kernel's stage ring and the two
    accumulator buffers wrap many times per CTA (and per CTA pair)."""
    case = ("many_tiles", 40, 28, 28, 64, 128, 1, 1, 1, 0)  # M = 31360 -> 245 row tiles (odd: a pair's last half is empty)
    for plan in ((0, 64, 0), (0, 128, 0), (0, 128, 1)):
        _with_plan(plan, lambda: _run_bf16(case, IMPL_TCGEN05))
    case = ("many_tiles_wide", 40, 28, 28, 64, 512, 1, 1, 1, 0)  # two 256-wide tiles per row tile
    for plan in ((0, 256, 0), (0, 256, 1)):
        _with_plan(plan, lambda: _run_bf16(case, IMPL_TCGEN05))
    case = ("many_tiles_3x3", 24, 28, 28, 64, 64, 3, 3, 1, 1)  # gathered A, 147 row tiles
    _run_bf16(case, IMPL_TCGEN05)
    case = ("many_tiles_3x3_pair", 24, 28, 28, 64, 128, 3, 3, 1, 1)  # gathered A through CTA pairs
    _with_plan((0, 128, 1), lambda: _run_bf16(case, IMPL_TCGEN05))


@pytest.mark.parametrize("K", [64, 128, 256])
def test_conv_tcgen05_ten_tiles_per_cta(K):
    """1568 row tiles over 148 SMs: every CTA walks ten or more tiles, so the epilogue groups fall behind the MMA
    warp and catch up again, the accumulator buffers and the per-group barriers wrap many times, and a 64-, 128-
    and 256-column tile deal their slabs to the groups in all three patterns."""
    case = (f"ten_tiles_k{K}", 64, 56, 56, 64, K, 1, 1, 1, 0)
    _run_bf16(case, IMPL_TCGEN05)
    if K > 64:
        _with_plan((0, 0, 1), lambda: _run_bf16(case, IMPL_TCGEN05))
        _with_plan((1, 0, -1), lambda: _run_bf16(case, IMPL_TCGEN05))   # the same through the gather path


def test_conv_pair_equals_single_bitwise():
    """Two CTAs per 256-row tile accumulate every output in the same k order as one CTA per 128-row tile:
    fprop and dgrad of a 1x1 (TMA-fed) and a 3x3 (gathered) problem must agree bit for bit, ragged last tile
    included."""
    bf = torch.bfloat16
    for case in (("p1x1", 9, 14, 14, 256, 320, 1, 1, 1, 0), ("p3x3", 5, 14, 14, 128, 192, 3, 3, 1, 1)):
        x, w, dy = _mk(case, bf)
        xd, wd, dyd = x.to(DEV, bf), w.to(DEV, bf), dy.to(DEV, bf)
        stride, pad = case[8], case[9]
        wt = ops.filter_transpose(wd)
        run = lambda: (ops.conv_fprop(xd, wd, stride, pad, impl=IMPL_TCGEN05),
                       ops.conv_dgrad(dyd, wt, x.shape, stride, pad, impl=IMPL_TCGEN05))
        single = _with_plan((0, 0, 0), run)
        pair = _with_plan((0, 0, 1), run)
        torch.cuda.synchronize()
        assert ops.tc_status() == 0
        assert torch.equal(single[0], pair[0]), case[0]
        assert torch.equal(single[1], pair[1]), case[0]


def test_conv_tcgen05_gather_equals_tma():
    """1x1 stride-1 problems take the TMA path for A; the gather path must agree bit for bit."""
    case = CONV_CASES[0]
    x, w, dy = _mk(case, torch.bfloat16)
    bf = torch.bfloat16
    xd, wd = x.to(DEV, bf), w.to(DEV, bf)
    dyd = dy.to(DEV, bf)
    y_tma = ops.conv_fprop(xd, wd, 1, 0, impl=IMPL_TCGEN05)
    dw_tma = ops.conv_wgrad(dyd, xd, 1, 1, 1, 0, impl=IMPL_TCGEN05)
    y_g, dw_g = _with_plan((1, 0, -1), lambda: (ops.conv_fprop(xd, wd, 1, 0, impl=IMPL_TCGEN05),
                                                 ops.conv_wgrad(dyd, xd, 1, 1, 1, 0, impl=IMPL_TCGEN05)))
    torch.cuda.synchronize()
    assert ops.tc_status() == 0
    assert torch.equal(y_tma, y_g)
    assert torch.equal(dw_tma, dw_g)


IM2COL_CASES = [
    ("i3x3_tail", 5, 14, 14, 128, 192, 3, 3, 1, 1),          # 980 rows: tiles cross image borders, ragged last tile
    ("i3x3_c64_two_taps_per_tile", 3, 28, 28, 64, 64, 3, 3, 1, 1),
    ("i3x3_s2", 3, 28, 28, 128, 128, 3, 3, 2, 1),
    ("i1x1_s2", 3, 28, 28, 256, 512, 1, 1, 2, 0),
    ("i5x5_pad2", 2, 12, 10, 64, 72, 5, 5, 1, 2),
    ("i3x3_pad0", 2, 16, 16, 64, 64, 3, 3, 1, 0),
    ("i3x3_7x7_image", 67, 7, 7, 128, 256, 3, 3, 1, 1),      # 49-pixel images: a tile spans three of them
]


@pytest.mark.parametrize("case", IM2COL_CASES, ids=[c[0] for c in IM2COL_CASES])
def test_conv_im2col_tma_equals_gather_bitwise(case):
    """Filters wider than 1x1 (and strided 1x1 filters) fetch their activation operand with im2col TMA loads when
    the channel count is a multiple of 64; the cp.async gather delivers the same tiles, so fprop, dgrad (stride 1)
    and wgrad agree bit for bit with it, through single CTAs and CTA pairs, and match the fp32 reference."""
    bf = torch.bfloat16
    _, N, H, W, C, K, R, S, stride, pad = case
    x, w, dy = _mk(case, bf)
    xd, wd, dyd = x.to(DEV, bf), w.to(DEV, bf), dy.to(DEV, bf)
    wt = ops.filter_transpose(wd)

    def run():
        y = ops.conv_fprop(xd, wd, stride, pad, impl=IMPL_TCGEN05)
        dx = ops.conv_dgrad(dyd, wt, x.shape, stride, pad, impl=IMPL_TCGEN05)
        dw = ops.conv_wgrad(dyd, xd, R, S, stride, pad, impl=IMPL_TCGEN05)
        return y, dx, dw
    ref = _ref(x, w, dy, stride, pad)
    base = _with_plan((1, 0, 0), run)                     # everything gathered, one CTA per tile
    for plan in ((0, 0, 0), (0, 0, 1), (0, 64, 0)):
        got = _with_plan(plan, run)
        torch.cuda.synchronize()
        assert ops.tc_status() == 0
        for name, a, b in zip(("fprop", "dgrad", "wgrad"), got, base):
            if name == "wgrad" and plan[2] == 1:
                # CTA pairs split the pixel range differently: the same sums in another fp32 order
                assert _err(a, b.float().cpu()) < 1e-5, (case[0], plan, name)
            else:
                assert torch.equal(a, b), (case[0], plan, name)
    for name, a, r in zip(("fprop", "dgrad", "wgrad"), base, ref):
        assert _err(a, r) < 2e-2, (case[0], name)


def test_conv_epilogue_bias_addend():
    case = ("fc", 8, 1, 1, 256, 40, 1, 1, 1, 0)
    for dtype, impl, tol in ((torch.float32, IMPL_AUTO, 2e-5), (torch.bfloat16, IMPL_TCGEN05, 1e-2)):
        x, w, _ = _mk(case, dtype)
        g = torch.Generator().manual_seed(5)
        bias = torch.randn(40, generator=g)
        add = torch.randn(8, 1, 1, 40, generator=g)
        if dtype == torch.bfloat16:
            add = add.to(dtype).float()
        ref = (x.reshape(8, 256) @ w.reshape(40, 256).t() + bias).reshape(8, 1, 1, 40) + add
        y = ops.conv_fprop(x.to(DEV, dtype), w.to(DEV, dtype), 1, 0, bias=bias.to(DEV),
                           addend=add.to(DEV, dtype), impl=impl)
        torch.cuda.synchronize()
        assert _err(y, ref) < tol


STATS_CASES = CONV_CASES + [
    ("1x1_c64_k256_98tiles", 4, 56, 56, 64, 256, 1, 1, 1, 0),
    ("3x3_c64_k64_multi_tile_per_cta", 6, 56, 56, 64, 64, 3, 3, 1, 1),
    ("1x1_c128_k72_ragged_slab", 3, 10, 10, 128, 72, 1, 1, 1, 0),
]


@pytest.mark.parametrize("case", STATS_CASES, ids=[c[0] for c in STATS_CASES])
@pytest.mark.parametrize("with_terms", [False, True], ids=["plain", "bias_addend"])
def test_conv_fprop_bn_stats_matches_separate_passes(case, with_terms):
    """The convolution that takes the BatchNorm sums in its epilogue: same y bit for bit as srt_conv_fprop, and the
    finalized statistics equal those srt_bn_stats computes from that y (both sum the rounded bf16 values; only the
    order of the fp32/fp64 additions differs)."""
    _, N, H, W, Cc, K, R, S, stride, pad = case
    x, w, dy = _mk(case, torch.bfloat16)
    g = torch.Generator().manual_seed(11)
    xd, wd = x.to(DEV, torch.bfloat16), w.to(DEV, torch.bfloat16)
    bias = (torch.randn(K, generator=g) * 3).to(DEV) if with_terms else None
    addend = torch.randn(dy.shape, generator=g).to(DEV, torch.bfloat16) if with_terms else None
    gamma = (torch.rand(K, generator=g) + 0.5).to(DEV)
    beta = torch.randn(K, generator=g).to(DEV)
    rm1, rv1 = torch.zeros(K, device=DEV), torch.ones(K, device=DEV)
    rm2, rv2 = torch.zeros(K, device=DEV), torch.ones(K, device=DEV)
    y_ref = ops.conv_fprop(xd, wd, stride, pad, bias=bias, addend=addend, impl=IMPL_TCGEN05)
    want = ops.bn_stats(y_ref, gamma, beta, rm1, rv1)
    y, *got = ops.conv_fprop_bn_stats(xd, wd, stride, pad, gamma, beta, rm2, rv2, bias=bias, addend=addend,
                                      impl=IMPL_TCGEN05)
    torch.cuda.synchronize()
    assert torch.equal(y, y_ref)
    for name, a, b in zip(("mean", "invstd", "scale", "shift"), got, want):
        assert torch.allclose(a, b, rtol=2e-5, atol=2e-6), (name, (a - b).abs().max().item())
    assert torch.allclose(rm2, rm1, rtol=2e-5, atol=2e-6) and torch.allclose(rv2, rv1, rtol=2e-5, atol=2e-6)
    # and against the definition, in fp64 on the host
    yf = y.double().cpu().reshape(-1, K)
    assert torch.allclose(got[0].cpu().double(), yf.mean(0), rtol=1e-4, atol=1e-5)
    assert torch.allclose(got[1].cpu().double(), 1.0 / torch.sqrt(yf.var(0, unbiased=False) + 1e-5), rtol=1e-4)


def test_conv_fprop_bn_stats_rejects_what_it_cannot_do():
    x = torch.randn(1, 4, 4, 8, device=DEV)
    w = torch.randn(8, 1, 1, 8, device=DEV)
    one = torch.ones(8, device=DEV)
    with pytest.raises(RuntimeError):
        ops.conv_fprop_bn_stats(x, w, 1, 0, one, one, one.clone(), one.clone())  # fp32 has no statistics epilogue


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape", [(2, 14, 14, 64), (3, 7, 7, 2048), (2, 5, 5, 24)], ids=str)
def test_batchnorm_fwd_bwd(dtype, shape):
    g = torch.Generator().manual_seed(1)
    C = shape[-1]
    z = torch.randn(shape, generator=g) * 2 + 0.5
    res = torch.randn(shape, generator=g)
    dy = torch.randn(shape, generator=g)
    gamma = torch.rand(C, generator=g) + 0.5
    beta = torch.randn(C, generator=g)
    if dtype == torch.bfloat16:
        z, res, dy = (t.to(dtype).float() for t in (z, res, dy))
    rm, rv = torch.zeros(C), torch.ones(C)
    zn = z.permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    resn = res.permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    gp, bp = gamma.clone().requires_grad_(True), beta.clone().requires_grad_(True)
    rm_ref, rv_ref = rm.clone(), rv.clone()
    out = F.relu(F.batch_norm(zn, rm_ref, rv_ref, gp, bp, True, 0.1, 1e-5) + resn)
    out.backward(dy.permute(0, 3, 1, 2).contiguous())
    y_ref = out.detach().permute(0, 2, 3, 1)
    dz_ref = zn.grad.permute(0, 2, 3, 1)
    dres_ref = resn.grad.permute(0, 2, 3, 1)

    zd, resd, dyd = z.to(DEV, dtype), res.to(DEV, dtype), dy.to(DEV, dtype)
    gd, bd, rmd, rvd = gamma.to(DEV), beta.to(DEV), rm.to(DEV), rv.to(DEV)
    mean, invstd, scale, shift = ops.bn_stats(zd, gd, bd, rmd, rvd)
    y = ops.bn_apply(zd, scale, shift, residual=resd, relu=True)
    dz, dres, dgamma, dbeta = ops.bn_backward(dyd, y, zd, gd, mean, invstd, relu=True, want_dresidual=True)
    torch.cuda.synchronize()
    tol = 1e-5 if dtype == torch.float32 else 1.5e-2
    assert _err(rmd, rm_ref) < 1e-5 and _err(rvd, rv_ref) < 1e-5
    assert _err(y, y_ref) < tol
    if dtype == torch.float32:
        assert _err(dz, dz_ref) < 1e-4
        assert _err(dres, dres_ref) < 1e-6
        assert _err(dgamma, gp.grad) < 1e-5 and _err(dbeta, bp.grad) < 1e-5
    else:
        # the ReLU mask comes from the bf16-rounded y; elements that round to 0 may flip, so
        # compare the bulk statistics rather than every element
        assert (dz.float().cpu() - dz_ref).abs().mean() / dz_ref.abs().mean() < 2e-2
        assert _err(dgamma, gp.grad) < 2e-2 and _err(dbeta, bp.grad) < 2e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_batchnorm_mask_recomputed_from_z_is_identical(dtype):
    """Units without a residual skip reading y in the backward pass: the ReLU mask recomputed from
    z*scale + shift must give bit-identical results to the mask read from the stored y."""
    g = torch.Generator().manual_seed(7)
    shape = (4, 9, 9, 128)
    z = (torch.randn(shape, generator=g) * 2).to(DEV, dtype)
    dy = torch.randn(shape, generator=g).to(DEV, dtype)
    gamma = (torch.rand(128, generator=g) + 0.5).to(DEV)
    beta = torch.randn(128, generator=g).to(DEV)
    mean, invstd, scale, shift = ops.bn_stats(z, gamma, beta, None, None)
    y = ops.bn_apply(z, scale, shift, relu=True)
    a = ops.bn_backward(dy, y, z, gamma, mean, invstd, relu=True)
    b = ops.bn_backward(dy, None, z, gamma, mean, invstd, relu=True, scale=scale, shift=shift)
    torch.cuda.synchronize()
    assert torch.equal(a[0], b[0]) and torch.equal(a[2], b[2]) and torch.equal(a[3], b[3])


@pytest.mark.parametrize("shape", [(16, 14, 14, 256), (3, 7, 7, 2048), (5, 9, 11, 48), (64, 28, 28, 128)], ids=str)
def test_relu_bit_mask_replaces_the_stored_output_bit_for_bit(shape):
    """A residual unit's ReLU mask as one bit per element: the forward apply pass writes it next to y, both backward
    paths (three kernels, one launch) read it where they would read y and give the same bits, and a data gradient
    that adds dout under the bits equals one that adds the masked copy."""
    bf = torch.bfloat16
    g = torch.Generator().manual_seed(5)
    C = shape[-1]
    z = (torch.randn(shape, generator=g) * 2 + 0.3).to(DEV, bf)
    res = torch.randn(shape, generator=g).to(DEV, bf)
    dy = torch.randn(shape, generator=g).to(DEV, bf)
    gamma, beta = (torch.rand(C, generator=g) + 0.5).to(DEV), torch.randn(C, generator=g).to(DEV)
    mean, invstd, scale, shift = ops.bn_stats(z, gamma, beta, None, None)
    y = ops.bn_apply(z, scale, shift, residual=res, relu=True)
    y2, bits = ops.bn_apply_bits(z, scale, shift, residual=res)
    torch.cuda.synchronize()
    assert torch.equal(y, y2)
    want = ((y.reshape(-1, 8) > 0).to(torch.int32) << torch.arange(8, device=DEV, dtype=torch.int32)).sum(1).to(torch.uint8)
    assert torch.equal(bits, want)
    for one_launch in (False, True):
        for want_dres in (True, False):
            ref = (ops.bn_backward_fused if one_launch else ops.bn_backward)(dy, y, z, gamma, mean, invstd, relu=True,
                                                                             want_dresidual=want_dres)
            got = ops.bn_backward_bits(dy, bits, z, gamma, mean, invstd, want_dresidual=want_dres, one_launch=one_launch)
            torch.cuda.synchronize()
            for name, a, b in zip(("dz", "dres", "dgamma", "dbeta"), got, ref):
                assert (a is None and b is None) or torch.equal(a, b), (name, one_launch, want_dres)
    # dx = dgrad(dz) + dout under the mask, against dx = dgrad(dz) + (masked copy of dout)
    K = 64
    w = (torch.randn(K, 1, 1, C, generator=g) * C ** -0.5).to(DEV, bf)
    dz1 = torch.randn(*shape[:3], K, generator=g).to(DEV, bf)
    wt = ops.filter_transpose(w)
    masked = torch.where(y > 0, dy, torch.zeros_like(dy))
    for impl in (IMPL_TCGEN05, IMPL_SIMT):
        a = ops.conv_dgrad(dz1, wt, shape, 1, 0, addend=masked, impl=impl)
        b = ops.conv_dgrad(dz1, wt, shape, 1, 0, addend=dy, addend_bits=bits, impl=impl)
        torch.cuda.synchronize()
        assert torch.equal(a, b), impl
    assert ops.tc_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
@pytest.mark.parametrize("shape,residual", [((64, 14, 14, 256), False), ((8, 7, 7, 2048), True), ((3, 5, 5, 48), True),
                                            ((2, 3, 3, 1024), False), ((16, 28, 28, 128), True), ((1, 1, 1, 8), False)])
def test_batchnorm_one_launch_path_matches_the_three_kernel_path(dtype, shape, residual):
    """The one-launch kernels (sums, grid barrier, finalize, grid barrier, apply) compute the same BatchNorm as
    statistics + finalize + apply and partial + finalize + apply; only the order of the sums differs. Repeated
    launches on one stream reuse the barrier words and give the same bits every time."""
    g = torch.Generator().manual_seed(11)
    C = shape[-1]
    z = (torch.randn(shape, generator=g) * 2 + 0.5).to(DEV, dtype)
    res = torch.randn(shape, generator=g).to(DEV, dtype) if residual else None
    dy = torch.randn(shape, generator=g).to(DEV, dtype)
    gamma, beta = (torch.rand(C, generator=g) + 0.5).to(DEV), torch.randn(C, generator=g).to(DEV)
    assert ops.bn_fused_fits(z) and ops.bn_fused_fits(z, backward=True)
    rm1, rv1, rm2, rv2 = (torch.zeros(C, device=DEV), torch.ones(C, device=DEV), torch.zeros(C, device=DEV),
                          torch.ones(C, device=DEV))
    mean, invstd, scale, shift = ops.bn_stats(z, gamma, beta, rm1, rv1)
    y = ops.bn_apply(z, scale, shift, residual=res, relu=True)
    y2, mean2, invstd2, scale2, shift2 = ops.bn_forward_fused(z, gamma, beta, rm2, rv2, residual=res, relu=True)
    torch.cuda.synchronize()
    for a, b in ((mean, mean2), (invstd, invstd2), (scale, scale2), (shift, shift2), (rm1, rm2), (rv1, rv2)):
        assert _err(b, a.cpu()) < 2e-6
    assert _err(y2, y.float().cpu()) < (1e-6 if dtype == torch.float32 else 4e-3)
    for _ in range(3):
        again = ops.bn_forward_fused(z, gamma, beta, None, None, residual=res, relu=True)
        assert torch.equal(again[0], y2) and torch.equal(again[1], mean2) and torch.equal(again[2], invstd2)
    # backward from identical saved values, both mask variants
    ref = ops.bn_backward(dy, y if residual else None, z, gamma, mean, invstd, relu=True, want_dresidual=residual,
                          scale=scale, shift=shift)
    got = ops.bn_backward_fused(dy, y if residual else None, z, gamma, mean, invstd, relu=True, want_dresidual=residual,
                                scale=scale, shift=shift)
    torch.cuda.synchronize()
    tol = 2e-5 if dtype == torch.float32 else 4e-3
    assert _err(got[0], ref[0].float().cpu()) < tol
    if residual:
        assert torch.equal(got[1], ref[1])
    assert _err(got[2], ref[2].cpu()) < 1e-5 and _err(got[3], ref[3].cpu()) < 1e-5
    again = ops.bn_backward_fused(dy, y if residual else None, z, gamma, mean, invstd, relu=True, want_dresidual=residual,
                                  scale=scale, shift=shift)
    assert all(torch.equal(p, q) for p, q in zip(again, got) if p is not None)
    # the stored-output mask without a residual gradient (mask taken from y in both phases)
    if not residual:
        via_y = ops.bn_backward_fused(dy, y, z, gamma, mean, invstd, relu=True)
        assert torch.equal(via_y[0], got[0])
    assert ops.tc_status() == 0


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_pools(dtype):
    g = torch.Generator().manual_seed(2)
    x = torch.randn(2, 13, 16, 16, generator=g).clamp_min(0)  # zeros create ties like post-ReLU data
    if dtype == torch.bfloat16:
        x = x.to(dtype).float()
    xn = x.permute(0, 3, 1, 2).contiguous().requires_grad_(True)
    y_ref = F.max_pool2d(xn, 3, 2, 1)
    dy = torch.randn(y_ref.shape, generator=g)
    if dtype == torch.bfloat16:
        dy = dy.to(dtype).float()
    y_ref.backward(dy)
    xd = x.to(DEV, dtype)
    y, arg = ops.maxpool_fwd(xd)
    dx = ops.maxpool_bwd(dy.permute(0, 2, 3, 1).contiguous().to(DEV, dtype), arg, x.shape)
    torch.cuda.synchronize()
    assert torch.equal(y.float().cpu(), y_ref.detach().permute(0, 2, 3, 1))
    tol = 1e-6 if dtype == torch.float32 else 1e-2
    assert _err(dx, xn.grad.permute(0, 2, 3, 1)) < tol

    a = torch.randn(3, 7, 7, 64, generator=g)
    if dtype == torch.bfloat16:
        a = a.to(dtype).float()
    ya = ops.avgpool_fwd(a.to(DEV, dtype))
    da = ops.avgpool_bwd(ya, 49)
    torch.cuda.synchronize()
    assert _err(ya, a.mean(dim=(1, 2))) < (1e-6 if dtype == torch.float32 else 1e-2)
    assert _err(da.reshape(3, 7, 7, 64), (ya.float().cpu() / 49)[:, None, None, :].expand(3, 7, 7, 64)) < 1e-2


@pytest.mark.parametrize("dtype", [torch.float32, torch.bfloat16], ids=["f32", "bf16"])
def test_softmax_ce_and_colsum(dtype):
    g = torch.Generator().manual_seed(3)
    logits = torch.randn(16, 1000, generator=g) * 3
    if dtype == torch.bfloat16:
        logits = logits.to(dtype).float()
    labels = torch.randint(0, 1000, (16,), generator=g)
    lr = logits.clone().requires_grad_(True)
    loss = F.cross_entropy(lr, labels)
    loss.backward()
    row_loss, dlogits = ops.softmax_ce(logits.to(DEV, dtype), labels.to(DEV), 1.0 / 16)
    cs = ops.colsum(dlogits)
    torch.cuda.synchronize()
    assert abs(row_loss.sum().item() - loss.item()) < 1e-5 * max(1, abs(loss.item()))
    assert _err(dlogits, lr.grad) < (1e-6 if dtype == torch.float32 else 1e-2)
    assert _err(cs, dlogits.float().cpu().sum(0)) < 1e-5


def test_optimizers_match_torch():
    g = torch.Generator().manual_seed(4)
    n = 100003
    p0 = torch.randn(n, generator=g)
    grads = [torch.randn(n, generator=g) for _ in range(3)]
    pr = p0.clone().requires_grad_(True)
    opt = torch.optim.SGD([pr], lr=0.1, momentum=0.9, weight_decay=1e-4)
    pd, md = p0.to(DEV), torch.zeros(n, device=DEV)
    pb = torch.empty(n, dtype=torch.bfloat16, device=DEV)
    for i, gr in enumerate(grads):
        pr.grad = gr.clone()
        opt.step()
        ops.sgd_momentum(pd, gr.to(DEV), md, 0.1, 0.9, 1e-4, i == 0, p_bf16=pb)
    torch.cuda.synchronize()
    assert _err(pd, pr.detach()) < 1e-6
    assert torch.equal(pb.cpu(), pd.cpu().to(torch.bfloat16))

    pr = p0.clone().requires_grad_(True)
    opt = torch.optim.AdamW([pr], lr=1e-3)
    pd, md, vd = p0.to(DEV), torch.zeros(n, device=DEV), torch.zeros(n, device=DEV)
    for i, gr in enumerate(grads):
        pr.grad = gr.clone()
        opt.step()
        ops.adamw(pd, gr.to(DEV), md, vd, 1e-3, 0.9, 0.999, 1e-8, 0.01, i + 1)
    torch.cuda.synchronize()
    assert _err(pd, pr.detach()) < 1e-5

    acc, gg = torch.zeros(n, device=DEV), grads[0].to(DEV)
    ops.grad_accumulate(acc, gg)
    torch.cuda.synchronize()
    assert torch.equal(acc.cpu(), grads[0]) and gg.abs().max().item() == 0.0


def test_nchw_to_nhwc():
    g = torch.Generator().manual_seed(6)
    src = torch.randn(2, 3, 9, 7, generator=g)
    out = ops.nchw_to_nhwc(src.to(DEV), torch.float32, 8)
    torch.cuda.synchronize()
    ref = torch.zeros(2, 9, 7, 8)
    ref[..., :3] = src.permute(0, 2, 3, 1)
    assert torch.equal(out.cpu(), ref)
