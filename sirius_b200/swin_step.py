"""Swin transformer training step on the CUDA library (torchvision `swin_b` layout): the loop body of the
reference's `train/swin_b.py:83-95` as calls on one object."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import call, register
from .gpt2_step import GradBucketsMixin

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


class SwinConfigC(C.Structure):
    _fields_ = [("image", _i), ("patch", _i), ("embed", _i), ("depths", _i * 4), ("heads", _i * 4), ("window", _i),
                ("num_classes", _i), ("max_batch", _i), ("lr", _f), ("beta1", _f), ("beta2", _f), ("eps", _f),
                ("weight_decay", _f), ("ln_eps", _f)]


register({
    "srt_swin_create": (None, [C.POINTER(SwinConfigC), C.POINTER(_vp)]),
    "srt_swin_destroy": (None, [_vp]),
    "srt_swin_num_params": (_i, [_vp]),
    "srt_swin_param_info": (None, [_vp, _i, C.c_char_p, _i, C.POINTER(_i64), C.POINTER(_i)]),
    "srt_swin_set_param": (None, [_vp, _i, _vp]),
    "srt_swin_get_param": (None, [_vp, _i, _vp, _i]),
    "srt_swin_commit_params": (None, [_vp]),
    "srt_swin_upload_batch": (None, [_vp, _vp, _vp, _i]),
    "srt_swin_forward_backward": (None, [_vp, _i, _i]),
    "srt_swin_forward_only": (None, [_vp, _i]),
    "srt_swin_optimizer": (None, [_vp]),
    "srt_swin_loss": (None, [_vp, C.POINTER(_f)]),
    "srt_swin_logits": (None, [_vp, _vp, _i]),
    "srt_swin_synchronize": (None, [_vp]),
    "srt_swin_grad_buffer": (None, [_vp, C.POINTER(_vp), C.POINTER(_i64)]),
    "srt_swin_stream": (_vp, [_vp]),
    "srt_swin_memory_bytes": (_i64, [_vp]),
})

GET_VALUE, GET_GRAD, GET_MOMENTUM = 0, 1, 3
SWIN_B = dict(image=224, patch=4, embed=128, depths=(2, 2, 18, 2), heads=(4, 8, 16, 32), window=7, num_classes=1000)


class SwinStep(GradBucketsMixin):
    _buckets_fn = "srt_swin_grad_buckets"

    """`SwinStep(**SWIN_B, max_batch=32)`; parameters use the names and shapes of torchvision's `swin_b().state_dict()`
    (the `relative_position_index` buffers are derived, not parameters)."""

    def __init__(self, image=224, patch=4, embed=128, depths=(2, 2, 18, 2), heads=(4, 8, 16, 32), window=7, num_classes=1000,
                 max_batch=32, lr=1e-3, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, ln_eps=1e-5):
        cfg = SwinConfigC(image, patch, embed, (_i * 4)(*depths), (_i * 4)(*heads), window, num_classes, max_batch, lr, betas[0],
                          betas[1], eps, weight_decay, ln_eps)
        self.cfg, self.image, self.num_classes, self.max_batch = cfg, image, num_classes, max_batch
        self._h = _vp()
        call("srt_swin_create", C.byref(cfg), C.byref(self._h))
        self.params = {}
        name, shape, ndim = C.create_string_buffer(256), (_i64 * 4)(), _i()
        for i in range(_lib.lib().srt_swin_num_params(self._h)):
            call("srt_swin_param_info", self._h, i, name, 256, shape, C.byref(ndim))
            self.params[name.value.decode()] = (i, tuple(shape[:ndim.value]))

    def close(self):
        if self._h:
            call("srt_swin_destroy", self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_state_dict(self, sd) -> None:
        for name, (idx, shape) in self.params.items():
            v = sd[name]
            a = np.ascontiguousarray(np.asarray(v.detach().cpu().numpy() if hasattr(v, "detach") else v, dtype=np.float32))
            assert a.shape == shape, (name, a.shape, shape)
            call("srt_swin_set_param", self._h, idx, a.ctypes.data_as(_vp))
        call("srt_swin_commit_params", self._h)

    def get(self, name, which=GET_VALUE) -> np.ndarray:
        idx, shape = self.params[name]
        out = np.empty(shape, dtype=np.float32)
        call("srt_swin_get_param", self._h, idx, out.ctypes.data_as(_vp), which)
        return out

    def upload_batch(self, images, labels) -> None:
        """images: float32 [B, 3, image, image] (pinned for an asynchronous copy), labels: int64 [B]."""
        self._keep = (images, labels)  # the copy is asynchronous: keep the host buffers alive
        self._B = int(images.shape[0])
        call("srt_swin_upload_batch", self._h, C.c_void_p(images.data_ptr()), C.c_void_p(labels.data_ptr()), self._B)

    def forward_backward(self, global_batch=None) -> None:
        call("srt_swin_forward_backward", self._h, self._B, global_batch or self._B)

    def forward_only(self) -> None:
        call("srt_swin_forward_only", self._h, self._B)

    def optimizer_step(self) -> None:
        call("srt_swin_optimizer", self._h)

    def loss(self) -> float:
        v = _f()
        call("srt_swin_loss", self._h, C.byref(v))
        return float(v.value)

    def logits(self) -> np.ndarray:
        out = np.empty((self._B, self.num_classes), dtype=np.float32)
        call("srt_swin_logits", self._h, out.ctypes.data_as(_vp), self._B)
        return out

    def synchronize(self) -> None:
        call("srt_swin_synchronize", self._h)

    def grad_buffer(self):
        p, n = _vp(), _i64()
        call("srt_swin_grad_buffer", self._h, C.byref(p), C.byref(n))
        return p.value, n.value

    @property
    def stream(self) -> int:
        return _lib.lib().srt_swin_stream(self._h)

    def follow_infer_tpc(self, comm_handle, device: int = 0, min_train_tpc: int = 5, max_train_tpc: int = 0) -> None:
        """Between layers, move to the SM partition that the inference side's required-TPC counter on the
        information board leaves to training (pytorch/torch_col/csrc/init.cc:56-62); None detaches."""
        from . import _runtime  # noqa: F401  (registers the entry points)
        call("srt_swin_follow_infer_tpc", self._h, comm_handle, device, min_train_tpc, max_train_tpc, 0 if comm_handle is None else 1)

    def follow_sm_mask(self, on: bool = True) -> None:
        """Follow the process-wide allowed-SM mask instead of a board."""
        from . import _runtime  # noqa: F401
        call("srt_swin_follow_infer_tpc", self._h, None, 0, 0, 0, int(on))

    def current_sms(self) -> int:
        from . import _runtime  # noqa: F401
        return _lib.lib().srt_swin_current_sms(self._h)

    def memory_bytes(self) -> int:
        return _lib.lib().srt_swin_memory_bytes(self._h)

    def train_step(self, images, labels) -> float:
        self.upload_batch(images, labels)
        self.forward_backward()
        self.optimizer_step()
        return self.loss()
