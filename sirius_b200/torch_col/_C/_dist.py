"""torch_col._C._dist: barrier, mailboxes, the dynamic batch distributor and the performance model under the
module path of the reference's second Cython extension (cython/dist.pyx:25-194), plus the two c10d classes whose
extra methods the reference's Trainer calls (csrc/dist_ext.cc:673-784)."""
import sys as _sys

_impl = _sys.modules[__name__.rsplit('.', 1)[0]]
_ns = _impl._DistNamespace

wait_barrier = _ns.wait_barrier
send_msg = _ns.send_msg
recv_msg = _ns.recv_msg
init_dynamic_batch_distributor = _ns.init_dynamic_batch_distributor
init_train_performance_model = _ns.init_train_performance_model
_DynamicBatchDistirbutor = _impl._DynamicBatchDistirbutor
_PerfModel = _impl._PerfModel

_exchange = None


def set_default_exchange(exchange):
    """The sirius_b200.ddp.GradExchange the two classes below act on."""
    global _exchange
    _exchange = exchange


def _need_exchange():
    if _exchange is None:
        raise RuntimeError("not available: no gradient exchange registered (torch_col._C._dist.set_default_exchange)")
    return _exchange


class Reducer:
    """c10d's Reducer with finalize_dropped_batch (csrc/dist_ext.cc:673-700): after a killed batch the buckets
    already reduced are forgotten. The library's exchange keeps no state between exchanges (a bucket's all-reduce
    is enqueued only after the vote has decided that the batch goes through), so there is nothing to undo."""

    @staticmethod
    def finalize_dropped_batch():
        return None


class ProcessGroupNCCL:
    """The three additions of the reference's process group (csrc/dist_ext.cc:700-784), on the library's
    communicator."""

    @staticmethod
    def _set_nccl_comm_abort_flag(devices=None):
        _need_exchange().abort()

    @staticmethod
    def _restart_nccl_comm(devices=None):
        _need_exchange().restart()

    @staticmethod
    def _set_as_default_pg():
        return None
