"""Gradient exchange between data-parallel ranks through the library's own NCCL communicator
(srt_ddp_* / srt_allreduce_*): what the reference's c10d Reducer and ProcessGroupNCCL extension do for DDP
training (pytorch/torch_col/csrc/dist_ext.h:109-243, dist_ext.cc:59-123, 673-784).

    ex = GradExchange(rank, world)            # rank 0's unique id travels through torch.distributed by default
    step.forward_backward(...)                # returns once everything is enqueued
    ex.begin(step)                            # one all-reduce per gradient bucket, each behind its ready event
    ex.wait(step)                             # the step's stream waits for the exchange
    step.optimizer_step()

The all-reduce is a sum: the loss is scaled by micro_batch / global_batch (MicroBatchManager.scale_loss,
pytorch/torch_col/dynamic_batch.py:112-120), so the sum over ranks is the global-batch mean."""
from __future__ import annotations

import contextlib
import ctypes as C
import os
import sys
import weakref
from typing import Callable, Optional

from . import _lib
from ._lib import SRT_BF16, SRT_F32, call, register

_vp, _i, _i64 = C.c_void_p, C.c_int, C.c_int64
ID_BYTES = 128

register({
    "srt_ddp_available": (_i, []),
    "srt_ddp_nccl_version": (None, [C.POINTER(_i)]),
    "srt_ddp_unique_id": (None, [_vp]),
    "srt_ddp_create": (None, [_vp, _i, _i, _i, _i, C.POINTER(_vp)]),
    "srt_ddp_destroy": (None, [_vp]),
    "srt_ddp_abort": (None, [_vp]),
    "srt_ddp_restart": (None, [_vp, _vp]),
    "srt_ddp_stream": (_vp, [_vp]),
    "srt_ddp_stats": (None, [_vp, C.POINTER(_i64), C.POINTER(_i64)]),
    "srt_ddp_allreduce": (None, [_vp, _vp, _i64, _i, _vp]),
    "srt_allreduce_begin": (None, [_vp, _vp, _i, C.POINTER(_i64), C.POINTER(_i64), C.POINTER(_vp), _i]),
    "srt_allreduce_wait": (None, [_vp, _vp]),
    "srt_step_allreduce_begin": (None, [_vp, _vp, _i, _i]),
    "srt_step_allreduce_wait": (None, [_vp, _vp]),
    "srt_gb_allreduce_begin": (None, [_vp, _vp, _vp, _i]),
})

WIRE = {"f32": SRT_F32, "fp32": SRT_F32, "bf16": SRT_BF16}
_LIVE = weakref.WeakSet()     # the exchanges of this process that have not been closed (torch_col.xsched.get_nccl_streams)


def live_streams() -> list:
    """cudaStream_t values of the communication streams NCCL work of this process is enqueued on."""
    return [ex.stream for ex in list(_LIVE) if ex._h]


def available() -> bool:
    return bool(_lib.lib().srt_ddp_available())


def nccl_version() -> int:
    v = _i(0)
    call("srt_ddp_nccl_version", C.byref(v))
    return v.value


def _torch_broadcast(payload: Optional[bytes]) -> bytes:
    """Rank 0's bytes to every rank of the default torch.distributed group (any backend)."""
    import torch.distributed as dist
    box = [payload]
    dist.broadcast_object_list(box, src=0)
    return box[0]


@contextlib.contextmanager
def _stdout_to_stderr():
    """Route file descriptor 1 to stderr for the duration (native libraries write there directly)."""
    sys.stdout.flush()
    saved = os.dup(1)
    try:
        os.dup2(2, 1)
        yield
    finally:
        sys.stdout.flush()
        os.dup2(saved, 1)
        os.close(saved)


class GradExchange:
    """One NCCL communicator + communication stream owned by the library.

    broadcast(payload) hands rank 0's unique id to the other ranks: called with the id on rank 0 and with None
    elsewhere, returns the id everywhere. The default uses torch.distributed's default group.
    wire = "bf16" halves the bytes on NVLink (each bucket is rounded to bf16, summed, widened back);
    "f32" sums the fp32 gradients in place. max_ctas caps the SMs NCCL's kernels occupy."""

    def __init__(self, rank: int, world: int, device: Optional[int] = None, wire: str = "bf16", max_ctas: int = 0,
                 broadcast: Callable[[Optional[bytes]], bytes] = _torch_broadcast):
        if not available():
            raise RuntimeError("NCCL could not be loaded (libnccl.so.2): no gradient exchange without it")
        self.rank, self.world, self.wire = rank, world, WIRE[wire]
        self._broadcast = broadcast
        if device is None:
            import torch
            device = torch.cuda.current_device()
        self.device = device
        self._h = _vp()
        # (srt_ddp_create also switches the CTA-pair filter-gradient kernel off for the process: srt_conv_wgrad_pairs)
        uid = self._new_id()
        with _stdout_to_stderr():   # NCCL announces its version on stdout; callers may own that stream (one JSON line)
            call("srt_ddp_create", uid, rank, world, device, max_ctas, C.byref(self._h))
        _LIVE.add(self)

    def _new_id(self) -> bytes:
        buf = None
        if self.rank == 0:
            raw = C.create_string_buffer(ID_BYTES)
            call("srt_ddp_unique_id", raw)
            buf = raw.raw
        buf = self._broadcast(buf)
        assert len(buf) == ID_BYTES
        return buf

    # ---- exchange ----------------------------------------------------------------------------------
    def begin(self, step, accumulated: bool = False) -> None:
        """Enqueue the exchange of the step's gradients (after forward_backward has returned), or of its
        accumulated-gradient buffer when ranks ran different numbers of micro-batches."""
        if hasattr(step, "_buckets_fn"):     # transformer executors: bucket list + flat buffer
            if accumulated:
                raise ValueError("accumulated exchange is provided for the ResNet executor only")
            ptr, _ = step.grad_buffer()
            call("srt_gb_allreduce_begin", step._gb(), _vp(ptr), self._h, self.wire)
        else:
            call("srt_step_allreduce_begin", step._h, self._h, 1 if accumulated else 0, self.wire)

    def wait(self, step) -> None:
        """The step's stream waits for the exchange begun last (the optimizer kernels queue up behind it)."""
        if hasattr(step, "_buckets_fn"):
            call("srt_allreduce_wait", self._h, _vp(step.stream))
        else:
            call("srt_step_allreduce_wait", step._h, self._h)

    def allreduce(self, step, accumulated: bool = False) -> None:
        self.begin(step, accumulated)
        self.wait(step)

    def allreduce_tensor(self, ptr: int, count: int, dtype: str = "f32", stream: int = 0) -> None:
        call("srt_ddp_allreduce", self._h, _vp(ptr), count, WIRE[dtype], _vp(stream))

    # ---- after a killed batch (ProcessGroupNCCL._set_nccl_comm_abort_flag / _restart_nccl_comm) -------------
    def abort(self) -> None:
        call("srt_ddp_abort", self._h)

    def restart(self) -> None:
        uid = self._new_id()
        with _stdout_to_stderr():
            call("srt_ddp_restart", self._h, uid)

    @property
    def stream(self) -> int:
        return int(_lib.lib().srt_ddp_stream(self._h) or 0)

    def stats(self) -> dict:
        n, b = _i64(0), _i64(0)
        call("srt_ddp_stats", self._h, C.byref(n), C.byref(b))
        return {"exchanges": n.value, "bytes_on_wire": b.value}

    def close(self) -> None:
        if self._h:
            call("srt_ddp_destroy", self._h)
            self._h = _vp()

    def __del__(self):
        try:
            self.close()
        except Exception:
            pass
