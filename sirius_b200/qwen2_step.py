"""Qwen2 style decoder training step on the CUDA library: the loop body of the reference's `train/qwen.py:80-91`
(`loss = model(ids, labels=ids).loss; loss.backward(); optimizer.step()`) as calls on one object."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import call, register
from .gpt2_step import GradBucketsMixin

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


class Qwen2ConfigC(C.Structure):
    _fields_ = [("n_layer", _i), ("n_head", _i), ("n_kv_head", _i), ("hidden", _i), ("intermediate", _i), ("vocab", _i),
                ("max_batch", _i), ("seq", _i), ("rope_theta", _f), ("rms_eps", _f), ("lr", _f), ("beta1", _f), ("beta2", _f),
                ("eps", _f), ("weight_decay", _f)]


register({
    "srt_qwen2_create": (None, [C.POINTER(Qwen2ConfigC), C.POINTER(_vp)]),
    "srt_qwen2_create_with_pool": (None, [C.POINTER(Qwen2ConfigC), _vp, C.POINTER(_vp)]),
    "srt_qwen2_accumulate": (None, [_vp]),
    "srt_qwen2_release_activations": (None, [_vp, C.POINTER(C.c_size_t)]),
    "srt_qwen2_shrink_activations": (None, [_vp, _i, C.POINTER(C.c_size_t)]),
    "srt_qwen2_request_abort": (None, [_vp, _i]),
    "srt_qwen2_destroy": (None, [_vp]),
    "srt_qwen2_num_params": (_i, [_vp]),
    "srt_qwen2_param_info": (None, [_vp, _i, C.c_char_p, _i, C.POINTER(_i64), C.POINTER(_i)]),
    "srt_qwen2_set_param": (None, [_vp, _i, _vp]),
    "srt_qwen2_get_param": (None, [_vp, _i, _vp, _i]),
    "srt_qwen2_commit_params": (None, [_vp]),
    "srt_qwen2_upload_tokens": (None, [_vp, _vp, _i]),
    "srt_qwen2_forward_backward": (None, [_vp, _i, _i]),
    "srt_qwen2_forward_only": (None, [_vp, _i]),
    "srt_qwen2_optimizer": (None, [_vp]),
    "srt_qwen2_loss": (None, [_vp, C.POINTER(_f)]),
    "srt_qwen2_logits": (None, [_vp, _vp, _i]),
    "srt_qwen2_synchronize": (None, [_vp]),
    "srt_qwen2_grad_buffer": (None, [_vp, C.POINTER(_vp), C.POINTER(_i64)]),
    "srt_qwen2_stream": (_vp, [_vp]),
    "srt_qwen2_memory_bytes": (_i64, [_vp]),
})

GET_VALUE, GET_GRAD, GET_MOMENTUM = 0, 1, 3
QWEN2_05B = dict(n_layer=24, n_head=14, n_kv_head=2, hidden=896, intermediate=4864, vocab=151936)


class Qwen2Step(GradBucketsMixin):
    _buckets_fn = "srt_qwen2_grad_buckets"

    """`Qwen2Step(**QWEN2_05B, max_batch=4, seq=2048)`; parameters use the names and shapes of
    `transformers.Qwen2ForCausalLM.state_dict()` (`lm_head.weight` is the tied token table and is not listed)."""

    def __init__(self, n_layer=24, n_head=14, n_kv_head=2, hidden=896, intermediate=4864, vocab=151936, max_batch=4, seq=2048,
                 rope_theta=1e6, rms_eps=1e-6, lr=3e-4, betas=(0.9, 0.999), eps=1e-8, weight_decay=0.01, pool=None):
        cfg = Qwen2ConfigC(n_layer, n_head, n_kv_head, hidden, intermediate, vocab, max_batch, seq, rope_theta, rms_eps, lr,
                           betas[0], betas[1], eps, weight_decay)
        self.cfg, self.seq, self.vocab, self.max_batch = cfg, seq, vocab, max_batch
        self._h = _vp()
        self.pool = pool
        call("srt_qwen2_create_with_pool", C.byref(cfg), pool if pool else None, C.byref(self._h))
        self.params = {}
        name, shape, ndim = C.create_string_buffer(256), (_i64 * 2)(), _i()
        for i in range(_lib.lib().srt_qwen2_num_params(self._h)):
            call("srt_qwen2_param_info", self._h, i, name, 256, shape, C.byref(ndim))
            self.params[name.value.decode()] = (i, tuple(shape[:ndim.value]))

    def close(self):
        if self._h:
            call("srt_qwen2_destroy", self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass

    def load_state_dict(self, sd) -> None:
        for name, (idx, shape) in self.params.items():
            a = np.ascontiguousarray(np.asarray(sd[name].detach().cpu().numpy() if hasattr(sd[name], "detach") else sd[name],
                                                dtype=np.float32))
            assert a.shape == shape, (name, a.shape, shape)
            call("srt_qwen2_set_param", self._h, idx, a.ctypes.data_as(_vp))
        call("srt_qwen2_commit_params", self._h)

    def get(self, name, which=GET_VALUE) -> np.ndarray:
        idx, shape = self.params[name]
        out = np.empty(shape, dtype=np.float32)
        call("srt_qwen2_get_param", self._h, idx, out.ctypes.data_as(_vp), which)
        return out

    def state_dict(self) -> dict:
        return {n: self.get(n) for n in self.params}

    def upload_tokens(self, ids) -> None:
        a = np.ascontiguousarray(np.asarray(ids.cpu().numpy() if hasattr(ids, "cpu") else ids, dtype=np.int32))
        assert a.ndim == 2 and a.shape[1] == self.seq and a.shape[0] <= self.max_batch, a.shape
        self._B = a.shape[0]
        call("srt_qwen2_upload_tokens", self._h, a.ctypes.data_as(_vp), self._B)

    def forward_backward(self, global_batch=None) -> None:
        call("srt_qwen2_forward_backward", self._h, self._B, global_batch or self._B)

    def forward_only(self) -> None:
        call("srt_qwen2_forward_only", self._h, self._B)

    def optimizer_step(self) -> None:
        call("srt_qwen2_optimizer", self._h)

    def loss(self) -> float:
        v = _f()
        call("srt_qwen2_loss", self._h, C.byref(v))
        return float(v.value)

    def logits(self) -> np.ndarray:
        out = np.empty((self._B * self.seq, self.vocab), dtype=np.float32)
        call("srt_qwen2_logits", self._h, out.ctypes.data_as(_vp), self._B)
        return out

    def synchronize(self) -> None:
        call("srt_qwen2_synchronize", self._h)

    # ---- colocation hooks (the same surface as ResNetStep and Gpt2Step) ----
    def accumulate(self) -> None:
        call("srt_qwen2_accumulate", self._h)

    def release_activations(self) -> int:
        n = C.c_size_t()
        call("srt_qwen2_release_activations", self._h, C.byref(n))
        return n.value

    def shrink_activations(self, B: int) -> int:
        n = C.c_size_t()
        call("srt_qwen2_shrink_activations", self._h, int(B), C.byref(n))
        return n.value

    def request_abort(self, on: bool = True) -> None:
        call("srt_qwen2_request_abort", self._h, int(on))

    def abort_target(self):
        """(function address, handle) for srt_stub_set_abort_target: the control thread raises the kill flag through it."""
        return C.cast(_lib.lib().srt_qwen2_request_abort, _vp), self._h

    @property
    def stream(self) -> int:
        return _lib.lib().srt_qwen2_stream(self._h)

    def grad_buffer(self):
        p, n = _vp(), _i64()
        call("srt_qwen2_grad_buffer", self._h, C.byref(p), C.byref(n))
        return p.value, n.value

    def follow_infer_tpc(self, comm_handle, device: int = 0, min_train_tpc: int = 5, max_train_tpc: int = 0) -> None:
        """Between layers, move to the SM partition that the inference side's required-TPC counter on the
        information board leaves to training (pytorch/torch_col/csrc/init.cc:56-62); None detaches."""
        from . import _runtime  # noqa: F401  (registers the entry points)
        call("srt_qwen2_follow_infer_tpc", self._h, comm_handle, device, min_train_tpc, max_train_tpc, 0 if comm_handle is None else 1)

    def follow_sm_mask(self, on: bool = True) -> None:
        """Follow the process-wide allowed-SM mask instead of a board."""
        from . import _runtime  # noqa: F401
        call("srt_qwen2_follow_infer_tpc", self._h, None, 0, 0, 0, int(on))

    def current_sms(self) -> int:
        from . import _runtime  # noqa: F401
        return _lib.lib().srt_qwen2_current_sms(self._h)

    def memory_bytes(self) -> int:
        return _lib.lib().srt_qwen2_memory_bytes(self._h)

    def train_step(self, ids) -> float:
        self.upload_tokens(ids)
        self.forward_backward()
        self.optimizer_step()
        return self.loss()
