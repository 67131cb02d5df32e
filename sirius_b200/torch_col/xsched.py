"""torch_col.xsched (pytorch/torch_col/xsched.py:69-155). The reference intercepts libcuda to keep a
bounded queue of launches it can drop; here every training kernel is launched by the step executor,
which keeps a bounded number of units in flight and stops between units when asked, so these
functions act on the step object registered with torch_col.set_train_step()."""
from __future__ import annotations

from . import _C

_streams = []
_guess_nccl = False


def register_stream(stream, is_train_stream: bool = True): _streams.append(stream)
def unregister_stream(stream):
    if stream in _streams:
        _streams.remove(stream)
def unregister_all_streams(): _streams.clear()


def get_xqueue_size(stream=None) -> int:
    return 0  # launches already handed to CUDA cannot be dropped; the executor never queues more than 8 units


def set_reject_cuda_calls(reject: bool):
    step = _C.get_train_step()
    if step is not None and hasattr(step, 'request_abort'):
        step.request_abort(bool(reject))


def kill_batch(synchronize: bool = True):
    """Stop the in-flight micro-batch: raise the abort flag and wait for the units already launched."""
    step = _C.get_train_step()
    if step is None:
        return 0
    if hasattr(step, 'request_abort'):
        step.request_abort(True)
    if synchronize and hasattr(step, 'synchronize'):
        step.synchronize()
    return 0


def initial_kill_batch(epoch, batch): pass
def guess_nccl_begin():
    global _guess_nccl
    _guess_nccl = True
def guess_nccl_end():
    global _guess_nccl
    _guess_nccl = False
def is_guess_nccl_begined(): return _guess_nccl
def get_nccl_streams():
    """The streams NCCL kernels of this process run on: the communication streams of the library's gradient
    exchanges (the reference guesses them by watching stream creation between guess_nccl_begin/end)."""
    from .. import ddp
    return ddp.live_streams()
