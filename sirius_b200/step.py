"""Python handle over the C-ABI training-step executor (srt_resnet_create / srt_step_*)."""
from __future__ import annotations

import ctypes as C
from dataclasses import dataclass, field

import numpy as np

from . import _lib
from . import _runtime  # noqa: F401  (registers the runtime entry points)
from ._lib import IMPL_AUTO, SRT_BF16, SRT_F32, call, register


class ResNetConfigC(C.Structure):
    _fields_ = [("layers", C.c_int * 4), ("num_classes", C.c_int), ("max_batch", C.c_int),
                ("image", C.c_int), ("dtype", C.c_int), ("impl", C.c_int), ("lr", C.c_float),
                ("momentum", C.c_float), ("weight_decay", C.c_float), ("bn_eps", C.c_float),
                ("bn_momentum", C.c_float)]


_vp, _i, _i64 = C.c_void_p, C.c_int, C.c_int64
register({
    "srt_resnet_create": (None, [C.POINTER(ResNetConfigC), C.POINTER(_vp)]),
    "srt_step_destroy": (None, [_vp]),
    "srt_step_num_params": (_i, [_vp]),
    "srt_step_param_info": (None, [_vp, _i, C.c_char_p, _i, C.POINTER(_i64), C.POINTER(_i), C.POINTER(_i)]),
    "srt_step_set_param": (None, [_vp, _i, _vp]),
    "srt_step_get_param": (None, [_vp, _i, _vp, _i]),
    "srt_step_set_state": (None, [_vp, _i, _vp, _i]),
    "srt_step_commit_params": (None, [_vp]),
    "srt_step_stream": (_vp, [_vp]),
    "srt_step_upload_batch": (None, [_vp, _vp, _vp, _i]),
    "srt_step_set_batch_device": (None, [_vp, _vp, _vp, _i]),
    "srt_step_forward_backward": (None, [_vp, _i, _i]),
    "srt_step_forward_only": (None, [_vp, _i]),
    "srt_step_forward_infer": (None, [_vp, _i]),
    "srt_step_accumulate": (None, [_vp]),
    "srt_step_optimizer": (None, [_vp]),
    "srt_step_loss": (None, [_vp, C.POINTER(C.c_float)]),
    "srt_step_logits": (None, [_vp, _vp, _i]),
    "srt_step_synchronize": (None, [_vp]),
    "srt_step_memory_bytes": (_i64, [_vp, _i]),
    "srt_step_grad_buffer": (None, [_vp, _i, C.POINTER(_vp), C.POINTER(_i64)]),
    "srt_step_profile": (None, [_vp, _i]),
    "srt_step_profile_read": (None, [_vp, C.POINTER(C.c_double), C.POINTER(C.c_double), C.POINTER(_i64)]),
    "srt_launch_count": (_i64, []),
})
PROF_CATS = ("conv_fprop_dgrad", "conv_wgrad", "batchnorm", "other", "optimizer")

RESNET_LAYERS = {"resnet50": (3, 4, 6, 3), "resnet101": (3, 4, 23, 3), "resnet152": (3, 8, 36, 3)}
GET_VALUE, GET_GRAD, GET_ACCUM, GET_MOMENTUM = 0, 1, 2, 3


@dataclass
class ParamInfo:
    index: int
    name: str
    shape: tuple
    kind: int


class ResNetStep:
    """One colocated training step object: forward, loss, backward, SGD on the GPU.

    Mirrors what the reference's loop body does with torch modules (train/resnet152.py:84-91);
    `forward_backward(micro_bs, global_bs)` + `accumulate()` + `optimizer_step()` follow
    MicroBatchManager/GradAccumulator (pytorch/torch_col/dynamic_batch.py:112-153)."""

    def __init__(self, arch="resnet152", num_classes=1000, max_batch=16, image=224, dtype="bf16",
                 impl=IMPL_AUTO, lr=0.1, momentum=0.9, weight_decay=1e-4, layers=None, pool=None, pool_kind=0):
        cfg = ResNetConfigC()
        lay = tuple(layers) if layers is not None else RESNET_LAYERS[arch]
        cfg.layers = (C.c_int * 4)(*lay)
        cfg.num_classes, cfg.max_batch, cfg.image = num_classes, max_batch, image
        cfg.dtype = SRT_F32 if dtype in ("f32", "fp32", "float32") else SRT_BF16
        cfg.impl = impl
        cfg.lr, cfg.momentum, cfg.weight_decay = lr, momentum, weight_decay
        cfg.bn_eps, cfg.bn_momentum = 1e-5, 0.1
        self.cfg = cfg
        self.max_batch = max_batch
        self.dtype = "f32" if cfg.dtype == SRT_F32 else "bf16"
        self._h = _vp()
        self.pool = pool
        call("srt_resnet_create_on_allocator", C.byref(cfg), pool if pool else None, int(pool_kind), C.byref(self._h))
        self.params: dict[str, ParamInfo] = {}
        n = _lib.lib().srt_step_num_params(self._h)
        name = C.create_string_buffer(256)
        shape = (_i64 * 4)()
        ndim, kind = _i(), _i()
        for i in range(n):
            call("srt_step_param_info", self._h, i, name, 256, shape, C.byref(ndim), C.byref(kind))
            self.params[name.value.decode()] = ParamInfo(i, name.value.decode(), tuple(shape[:ndim.value]), kind.value)

    def close(self):
        if self._h:
            call("srt_step_destroy", self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    # ---- parameters -------------------------------------------------------------------
    def load_state_dict(self, sd) -> None:
        """sd: mapping name -> array-like (torch tensors or numpy), torchvision names and layouts."""
        for name, info in self.params.items():
            if name not in sd:
                raise KeyError(f"state dict lacks {name}")
            a = np.ascontiguousarray(_to_numpy(sd[name]), dtype=np.float32)
            if tuple(a.shape) != info.shape:
                raise ValueError(f"{name}: shape {a.shape} != {info.shape}")
            call("srt_step_set_param", self._h, info.index, a.ctypes.data)
        call("srt_step_commit_params", self._h)

    def load_momentum(self, momentum: dict) -> None:
        """Momentum buffers of torch.optim.SGD (mapping parameter name -> array, torch layouts), to continue a
        run from a saved optimizer state."""
        for name, v in momentum.items():
            info = self.params[name]
            a = np.ascontiguousarray(_to_numpy(v), dtype=np.float32)
            if tuple(a.shape) != info.shape:
                raise ValueError(f"{name}: shape {a.shape} != {info.shape}")
            call("srt_step_set_state", self._h, info.index, a.ctypes.data, GET_MOMENTUM)

    def get(self, name, which=GET_VALUE) -> np.ndarray:
        info = self.params[name]
        out = np.empty(info.shape, dtype=np.float32)
        call("srt_step_get_param", self._h, info.index, out.ctypes.data, which)
        return out

    def state_dict(self) -> dict:
        return {n: self.get(n) for n in self.params}

    # ---- step -------------------------------------------------------------------------
    @property
    def stream(self) -> int:
        return _lib.lib().srt_step_stream(self._h) or 0

    def upload_batch(self, images, labels) -> int:
        """images: host float32 [B,3,H,W] (numpy or CPU torch, ideally pinned); labels int64 [B]."""
        B = int(images.shape[0])
        images, labels = _host_contig(images, np.float32), _host_contig(labels, np.int64)
        # keep the host buffers of the last two uploads alive: their copies run asynchronously on the copy stream
        self._staged = (getattr(self, '_staged', ()) + ((images, labels),))[-2:]
        call("srt_step_upload_batch", self._h, _host_ptr(images), _host_ptr(labels), B)
        return B

    def set_batch_device(self, images_ptr: int, labels_ptr: int, B: int) -> None:
        call("srt_step_set_batch_device", self._h, images_ptr, labels_ptr, B)

    def forward_backward(self, micro_bs: int, global_bs: int | None = None) -> None:
        call("srt_step_forward_backward", self._h, micro_bs, global_bs or micro_bs)

    def forward_only(self, B: int) -> None:
        call("srt_step_forward_only", self._h, B)

    def forward_infer(self, B: int) -> None:
        call("srt_step_forward_infer", self._h, B)

    def accumulate(self) -> None:
        call("srt_step_accumulate", self._h)

    def optimizer_step(self) -> None:
        call("srt_step_optimizer", self._h)

    def loss(self) -> float:
        v = C.c_float()
        call("srt_step_loss", self._h, C.byref(v))
        return v.value

    def logits(self, B: int) -> np.ndarray:
        out = np.empty((B, self.cfg.num_classes), dtype=np.float32)
        call("srt_step_logits", self._h, out.ctypes.data, B)
        return out

    def synchronize(self) -> None:
        call("srt_step_synchronize", self._h)

    def memory_bytes(self) -> tuple[int, int]:
        l = _lib.lib()
        return l.srt_step_memory_bytes(self._h, 0), l.srt_step_memory_bytes(self._h, 1)

    def grad_buffer(self, accumulated=False) -> tuple[int, int]:
        p, n = _vp(), _i64()
        call("srt_step_grad_buffer", self._h, int(accumulated), C.byref(p), C.byref(n))
        return p.value, n.value

    def profile(self, enable: bool) -> None:
        call("srt_step_profile", self._h, int(enable))

    def profile_read(self) -> dict:
        ms, work, n = (C.c_double * 5)(), (C.c_double * 5)(), (_i64 * 5)()
        call("srt_step_profile_read", self._h, ms, work, n)
        return {c: {"ms": ms[i], "work": work[i], "launches": n[i]} for i, c in enumerate(PROF_CATS)}

    def release_activations(self) -> int:
        """Frees the activation set and returns emptied pages to the pool; bytes handed back."""
        n = C.c_size_t()
        call("srt_step_release_activations", self._h, C.byref(n))
        return n.value

    def shrink_activations(self, B: int) -> int:
        """Keeps an activation set for micro-batches of B samples and hands the other pages back; bytes returned."""
        n = C.c_size_t()
        call("srt_step_shrink_activations", self._h, int(B), C.byref(n))
        return n.value

    def reserve_activations(self, B: int) -> None:
        call("srt_step_reserve_activations", self._h, B)

    def grad_buckets(self) -> list[tuple[int, int]]:
        """(offset, count) in floats of each gradient bucket, in the order backward completes them."""
        out = []
        for i in range(_lib.lib().srt_step_num_grad_buckets(self._h)):
            off, cnt = C.c_int64(), C.c_int64()
            call("srt_step_grad_bucket", self._h, i, C.byref(off), C.byref(cnt))
            out.append((off.value, cnt.value))
        return out

    def wait_grad_bucket(self, i: int, cuda_stream: int) -> None:
        call("srt_step_wait_grad_bucket", self._h, i, C.c_void_p(cuda_stream))

    def wait_event(self, cuda_event: int) -> None:
        call("srt_step_wait_event", self._h, C.c_void_p(cuda_event))

    def overlap_wgrad(self, on: bool = True) -> None:
        call("srt_step_overlap_wgrad", self._h, int(on))

    def follow_sm_mask(self, on: bool = True) -> None:
        """Run on the green-context partition that fits the process-wide allowed-SM mask (checked between units)."""
        call("srt_step_follow_sm_mask", self._h, int(on))

    def follow_infer_tpc(self, comm_handle, device: int = 0, min_train_tpc: int = 5, max_train_tpc: int = 0) -> None:
        """Follow the inference side's required-TPC counter on the information board (None detaches)."""
        call("srt_step_follow_infer_tpc", self._h, comm_handle, device, min_train_tpc, max_train_tpc)

    def current_sms(self) -> int:
        n = C.c_int()
        call("srt_step_current_sms", self._h, C.byref(n))
        return n.value

    def request_abort(self, on: bool = True) -> None:
        call("srt_step_request_abort", self._h, int(on))

    def train_step(self, images, labels) -> float:
        """Whole-batch step through host buffers: H2D, forward, backward, SGD, loss readback."""
        B = self.upload_batch(images, labels)
        self.forward_backward(B, B)
        self.optimizer_step()
        return self.loss()


def _to_numpy(t):
    if hasattr(t, "detach"):
        return t.detach().cpu().numpy()
    return np.asarray(t)


def _host_contig(a, np_dtype):
    if hasattr(a, "data_ptr"):
        assert not a.is_cuda, "host tensor expected"
        return a.contiguous()
    return np.ascontiguousarray(a, dtype=np_dtype)


def _host_ptr(a) -> int:
    return a.data_ptr() if hasattr(a, "data_ptr") else a.ctypes.data
