"""DistilBERT-style encoder forward on the CUDA library: the second model of the stand-in inference worker
(the reference serves `distilbert_base` through TVM, `server/model_store/infer_model.cc:46-58,394-523`)."""
from __future__ import annotations

import ctypes as C

import numpy as np

from . import _lib
from ._lib import call, register

_vp, _i, _i64, _f = C.c_void_p, C.c_int, C.c_int64, C.c_float


class BertConfigC(C.Structure):
    _fields_ = [("n_layer", _i), ("n_head", _i), ("dim", _i), ("hidden_dim", _i), ("vocab", _i), ("max_pos", _i),
                ("max_batch", _i), ("seq", _i), ("ln_eps", _f)]


register({
    "srt_bert_create": (None, [C.POINTER(BertConfigC), _vp, C.POINTER(_vp)]),
    "srt_bert_destroy": (None, [_vp]),
    "srt_bert_num_params": (_i, [_vp]),
    "srt_bert_param_info": (None, [_vp, _i, C.c_char_p, _i, C.POINTER(_i64), C.POINTER(_i)]),
    "srt_bert_set_param": (None, [_vp, _i, _vp]),
    "srt_bert_commit_params": (None, [_vp]),
    "srt_bert_upload_tokens": (None, [_vp, _vp, _i]),
    "srt_bert_forward": (None, [_vp, _i]),
    "srt_bert_output": (None, [_vp, _vp, _i]),
    "srt_bert_synchronize": (None, [_vp]),
    "srt_bert_stream": (None, [_vp, C.POINTER(_vp)]),
    "srt_bert_release_activations": (None, [_vp, C.POINTER(C.c_size_t)]),
    "srt_bert_reserve_activations": (None, [_vp]),
    "srt_bert_memory_bytes": (None, [_vp, C.POINTER(C.c_size_t), C.POINTER(C.c_size_t)]),
})

DISTILBERT_BASE = dict(n_layer=6, n_head=12, dim=768, hidden_dim=3072, vocab=30522, max_pos=512)


class DistilBertInfer:
    """`DistilBertInfer(**DISTILBERT_BASE, max_batch=1, seq=128)`; parameters use the names and shapes of
    `transformers.DistilBertModel.state_dict()`. `pool` is a page-pool handle (`PagePool.handle`): activations then
    come from its inference allocator."""

    def __init__(self, n_layer=6, n_head=12, dim=768, hidden_dim=3072, vocab=30522, max_pos=512, max_batch=1, seq=128,
                 ln_eps=1e-12, pool=None):
        cfg = BertConfigC(n_layer, n_head, dim, hidden_dim, vocab, max_pos, max_batch, seq, ln_eps)
        self.cfg, self.seq, self.dim, self.vocab, self.max_batch = cfg, seq, dim, vocab, max_batch
        self._h = _vp()
        call("srt_bert_create", C.byref(cfg), pool, C.byref(self._h))
        self.params = {}
        name, shape, ndim = C.create_string_buffer(256), (_i64 * 2)(), _i()
        for i in range(_lib.lib().srt_bert_num_params(self._h)):
            call("srt_bert_param_info", self._h, i, name, 256, shape, C.byref(ndim))
            self.params[name.value.decode()] = (i, tuple(shape[:ndim.value]))
        self._B = 0

    def close(self):
        if self._h:
            call("srt_bert_destroy", self._h)
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
            call("srt_bert_set_param", self._h, idx, a.ctypes.data)
        call("srt_bert_commit_params", self._h)

    def upload_tokens(self, ids) -> None:
        a = np.ascontiguousarray(np.asarray(ids, dtype=np.int32))
        assert a.ndim == 2 and a.shape[1] == self.seq and a.shape[0] <= self.max_batch
        call("srt_bert_upload_tokens", self._h, a.ctypes.data, a.shape[0])
        self._B = a.shape[0]

    def forward(self) -> None:
        call("srt_bert_forward", self._h, self._B)

    def output(self) -> np.ndarray:
        out = np.empty((self._B, self.seq, self.dim), dtype=np.float32)
        call("srt_bert_output", self._h, out.ctypes.data, self._B)
        return out

    def synchronize(self) -> None:
        call("srt_bert_synchronize", self._h)

    def stream(self) -> int:
        s = _vp()
        call("srt_bert_stream", self._h, C.byref(s))
        return s.value or 0

    def release_activations(self) -> int:
        n = C.c_size_t()
        call("srt_bert_release_activations", self._h, C.byref(n))
        return n.value

    def reserve_activations(self) -> None:
        call("srt_bert_reserve_activations", self._h)

    def memory_bytes(self):
        w, a = C.c_size_t(), C.c_size_t()
        call("srt_bert_memory_bytes", self._h, C.byref(w), C.byref(a))
        return w.value, a.value
