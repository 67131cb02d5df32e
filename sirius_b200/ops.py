"""Tensor-level wrappers over the C ABI: each takes CUDA torch tensors (used only as device
buffers) and calls one entry point on the current stream. Layouts are NHWC / KRSC."""
from __future__ import annotations

import ctypes as C

import torch

from . import _lib
from ._lib import ConvDesc, ConvEpilogue, IMPL_AUTO, SRT_BF16, SRT_F32, call


def _dt(t: torch.Tensor) -> int:
    if t.dtype == torch.float32:
        return SRT_F32
    if t.dtype == torch.bfloat16:
        return SRT_BF16
    raise TypeError(f"unsupported dtype {t.dtype}")


def _p(t):
    if t is None:
        return None
    assert t.is_cuda and t.is_contiguous(), "device-resident contiguous tensor required"
    return t.data_ptr()


def _stream():
    return torch.cuda.current_stream().cuda_stream


def _ep(bias, addend, addend_bits=None):
    if bias is None and addend is None:
        return None
    return C.byref(ConvEpilogue(_p(bias), _p(addend), _p(addend_bits)))


def conv_fprop(x, w, stride, pad, bias=None, addend=None, impl=IMPL_AUTO, out=None):
    N, H, W, Cin = x.shape
    K, R, S, _ = w.shape
    d = ConvDesc.make(N, H, W, Cin, K, R, S, stride, pad)
    y = out if out is not None else torch.empty((N, d.P, d.Q, K), dtype=x.dtype, device=x.device)
    call("srt_conv_fprop", C.byref(d), _dt(x), impl, _p(x), _p(w), _p(y), _ep(bias, addend), _stream())
    return y


def conv_fprop_bn_stats(x, w, stride, pad, gamma, beta, running_mean, running_var, eps=1e-5, momentum=0.1,
                        bias=None, addend=None, impl=IMPL_AUTO):
    """Convolution whose epilogue takes the BatchNorm sums of its output, then the finalize step:
    returns (y, mean, invstd, scale, shift) like conv_fprop followed by bn_stats."""
    N, H, W, Cin = x.shape
    K, R, S, _ = w.shape
    d = ConvDesc.make(N, H, W, Cin, K, R, S, stride, pad)
    if not _lib.lib().srt_conv_fprop_bn_stats_supported(C.byref(d), _dt(x), impl):
        raise RuntimeError("conv_fprop_bn_stats: this dtype/impl has no statistics epilogue")
    y = torch.empty((N, d.P, d.Q, K), dtype=x.dtype, device=x.device)
    nbytes = _lib.lib().srt_conv_fprop_bn_stats_bytes(C.byref(d))
    partial = torch.empty(nbytes, dtype=torch.uint8, device=x.device)
    slabs = C.c_int(0)
    call("srt_conv_fprop_bn_stats", C.byref(d), _dt(x), impl, _p(x), _p(w), _p(y), _ep(bias, addend), _p(partial),
         nbytes, C.byref(slabs), _stream())
    f = lambda: torch.empty(K, dtype=torch.float32, device=x.device)
    mean, invstd, scale, shift = f(), f(), f(), f()
    call("srt_bn_finalize", _p(partial), slabs.value, K, N * d.P * d.Q, _p(gamma), _p(beta), eps, momentum,
         _p(running_mean), _p(running_var), _p(mean), _p(invstd), _p(scale), _p(shift), _stream())
    return y, mean, invstd, scale, shift


def filter_transpose(w):
    K, R, S, Cin = w.shape
    d = ConvDesc.make(1, R, S, Cin, K, R, S, 1, 0)
    wt = torch.empty((Cin, R, S, K), dtype=w.dtype, device=w.device)
    call("srt_conv_filter_transpose", C.byref(d), _dt(w), _p(w), _p(wt), _stream())
    return wt


def conv_dgrad(dy, wt, x_shape, stride, pad, addend=None, impl=IMPL_AUTO, addend_bits=None):
    N, H, W, Cin = x_shape
    _, R, S, K = wt.shape
    d = ConvDesc.make(N, H, W, Cin, K, R, S, stride, pad)
    dx = torch.empty((N, H, W, Cin), dtype=dy.dtype, device=dy.device)
    call("srt_conv_dgrad", C.byref(d), _dt(dy), impl, _p(dy), _p(wt), _p(dx), _ep(None, addend, addend_bits), _stream())
    return dx


def conv_wgrad(dy, x, R, S, stride, pad, impl=IMPL_AUTO):
    N, H, W, Cin = x.shape
    K = dy.shape[-1]
    d = ConvDesc.make(N, H, W, Cin, K, R, S, stride, pad)
    nbytes = _lib.lib().srt_conv_wgrad_scratch_bytes(C.byref(d), _dt(x), impl)
    scratch = torch.empty(max(nbytes, 16), dtype=torch.uint8, device=x.device)
    dw = torch.empty((K, R, S, Cin), dtype=torch.float32, device=x.device)
    call("srt_conv_wgrad", C.byref(d), _dt(x), impl, _p(dy), _p(x), _p(dw), _p(scratch), nbytes, _stream())
    return dw


def bn_scratch(rows, Cc, device):
    n = _lib.lib().srt_bn_scratch_bytes(rows, Cc)
    return torch.empty(n, dtype=torch.uint8, device=device), n


def bn_stats(z, gamma, beta, running_mean, running_var, eps=1e-5, momentum=0.1):
    Cc = z.shape[-1]
    rows = z.numel() // Cc
    f = lambda: torch.empty(Cc, dtype=torch.float32, device=z.device)
    mean, invstd, scale, shift = f(), f(), f(), f()
    scratch, n = bn_scratch(rows, Cc, z.device)
    call("srt_bn_stats", _dt(z), _p(z), rows, Cc, _p(gamma), _p(beta), eps, momentum, _p(running_mean),
         _p(running_var), _p(mean), _p(invstd), _p(scale), _p(shift), _p(scratch), n, _stream())
    return mean, invstd, scale, shift


def bn_apply(z, scale, shift, residual=None, relu=True):
    Cc = z.shape[-1]
    y = torch.empty_like(z)
    call("srt_bn_apply", _dt(z), _p(z), _p(residual), _p(y), z.numel() // Cc, Cc, _p(scale), _p(shift),
         int(relu), _stream())
    return y


def bn_apply_bits(z, scale, shift, residual=None):
    """bn_apply under a ReLU that also returns the mask as one bit per element (uint8 [numel / 8])."""
    Cc = z.shape[-1]
    y = torch.empty_like(z)
    bits = torch.empty(z.numel() // 8, dtype=torch.uint8, device=z.device)
    call("srt_bn_apply_bits", _dt(z), _p(z), _p(residual), _p(y), z.numel() // Cc, Cc, _p(scale), _p(shift), _p(bits), _stream())
    return y, bits


def bn_backward_bits(dy, bits, z, gamma, mean, invstd, want_dresidual=False, one_launch=False):
    Cc = z.shape[-1]
    rows = z.numel() // Cc
    dz = torch.empty_like(z)
    dres = torch.empty_like(z) if want_dresidual else None
    dgamma = torch.empty(Cc, dtype=torch.float32, device=z.device)
    dbeta = torch.empty_like(dgamma)
    scratch, n = bn_scratch(rows, Cc, z.device)
    call("srt_bn_backward_bits", _dt(z), _p(dy), _p(bits), _p(z), rows, Cc, _p(gamma), _p(mean), _p(invstd), _p(dz), _p(dres),
         _p(dgamma), _p(dbeta), _p(scratch), n, int(one_launch), _stream())
    return dz, dres, dgamma, dbeta


def bn_backward(dy, y, z, gamma, mean, invstd, relu=True, want_dresidual=False, scale=None, shift=None):
    Cc = z.shape[-1]
    rows = z.numel() // Cc
    dz = torch.empty_like(z)
    dres = torch.empty_like(z) if want_dresidual else None
    dgamma = torch.empty(Cc, dtype=torch.float32, device=z.device)
    dbeta = torch.empty_like(dgamma)
    scratch, n = bn_scratch(rows, Cc, z.device)
    call("srt_bn_backward", _dt(z), _p(dy), _p(y), _p(z), rows, Cc, _p(gamma), _p(mean), _p(invstd),
         _p(scale), _p(shift), int(relu), _p(dz), _p(dres), _p(dgamma), _p(dbeta), _p(scratch), n, _stream())
    return dz, dres, dgamma, dbeta


def bn_fused_fits(z, backward=False) -> bool:
    Cc = z.shape[-1]
    return bool(_lib.lib().srt_bn_fused_fits(_dt(z), z.numel() // Cc, Cc, int(backward)))


def bn_forward_fused(z, gamma, beta, running_mean, running_var, residual=None, relu=True, eps=1e-5, momentum=0.1):
    """Statistics + apply in one cooperative launch; returns (y, mean, invstd, scale, shift)."""
    Cc = z.shape[-1]
    f = lambda: torch.empty(Cc, dtype=torch.float32, device=z.device)
    mean, invstd, scale, shift = f(), f(), f(), f()
    y = torch.empty_like(z)
    call("srt_bn_forward_fused", _dt(z), _p(z), _p(residual), _p(y), z.numel() // Cc, Cc, _p(gamma), _p(beta), eps, momentum,
         _p(running_mean), _p(running_var), _p(mean), _p(invstd), _p(scale), _p(shift), int(relu), _stream())
    return y, mean, invstd, scale, shift


def bn_backward_fused(dy, y, z, gamma, mean, invstd, relu=True, want_dresidual=False, scale=None, shift=None):
    Cc = z.shape[-1]
    dz = torch.empty_like(z)
    dres = torch.empty_like(z) if want_dresidual else None
    dgamma = torch.empty(Cc, dtype=torch.float32, device=z.device)
    dbeta = torch.empty_like(dgamma)
    call("srt_bn_backward_fused", _dt(z), _p(dy), _p(y), _p(z), z.numel() // Cc, Cc, _p(gamma), _p(mean), _p(invstd),
         _p(scale), _p(shift), int(relu), _p(dz), _p(dres), _p(dgamma), _p(dbeta), _stream())
    return dz, dres, dgamma, dbeta


def maxpool_fwd(x):
    N, H, W, Cc = x.shape
    P, Q = (H - 1) // 2 + 1, (W - 1) // 2 + 1
    y = torch.empty((N, P, Q, Cc), dtype=x.dtype, device=x.device)
    arg = torch.empty((N, P, Q, Cc), dtype=torch.uint8, device=x.device)
    call("srt_maxpool3x3s2_fwd", _dt(x), _p(x), _p(y), _p(arg), N, H, W, Cc, _stream())
    return y, arg


def maxpool_bwd(dy, arg, x_shape):
    N, H, W, Cc = x_shape
    dx = torch.empty(x_shape, dtype=dy.dtype, device=dy.device)
    call("srt_maxpool3x3s2_bwd", _dt(dy), _p(dy), _p(arg), _p(dx), N, H, W, Cc, _stream())
    return dx


def avgpool_fwd(x):
    N, H, W, Cc = x.shape
    y = torch.empty((N, Cc), dtype=x.dtype, device=x.device)
    call("srt_avgpool_fwd", _dt(x), _p(x), _p(y), N, H * W, Cc, _stream())
    return y


def avgpool_bwd(dy, HW):
    N, Cc = dy.shape
    dx = torch.empty((N, HW, Cc), dtype=dy.dtype, device=dy.device)
    call("srt_avgpool_bwd", _dt(dy), _p(dy), _p(dx), N, HW, Cc, _stream())
    return dx


def softmax_ce(logits, labels, grad_scale):
    B, classes = logits.shape
    row_loss = torch.empty(B, dtype=torch.float32, device=logits.device)
    dlogits = torch.empty_like(logits)
    call("srt_softmax_ce", _dt(logits), _p(logits), _p(labels), B, classes, float(grad_scale),
         _p(row_loss), _p(dlogits), _stream())
    return row_loss, dlogits


def colsum(dy):
    rows, K = dy.shape
    out = torch.empty(K, dtype=torch.float32, device=dy.device)
    call("srt_colsum", _dt(dy), _p(dy), rows, K, _p(out), _stream())
    return out


def sgd_momentum(p, g, m, lr, mu, wd, first_step, p_bf16=None):
    call("srt_sgd_momentum", _p(p), _p(g), _p(m), _p(p_bf16), p.numel(), lr, mu, wd, int(first_step), _stream())


def adamw(p, g, m, v, lr, b1, b2, eps, wd, step, p_bf16=None):
    call("srt_adamw", _p(p), _p(g), _p(m), _p(v), _p(p_bf16), p.numel(), lr, b1, b2, eps, wd, step, _stream())


def grad_accumulate(acc, g):
    call("srt_grad_accumulate", _p(acc), _p(g), acc.numel(), _stream())


def nchw_to_nhwc(src, dtype, Cpad):
    N, Cc, H, W = src.shape
    dst = torch.empty((N, H, W, Cpad), dtype=dtype, device=src.device)
    call("srt_nchw_to_nhwc", SRT_F32 if dtype == torch.float32 else SRT_BF16, _p(src), _p(dst), N, Cc, H, W,
         Cpad, _stream())
    return dst


def tc_status() -> int:
    s = C.c_int(0)
    call("srt_tc_status", C.byref(s))
    return s.value
