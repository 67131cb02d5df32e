"""Bindings layer of torch_col: what the reference exposes as torch_col._C._main / _C._dist
(pytorch/torch_col/cython/main.pyx:77-567, dist.pyx:25-194), here over libsirius_b200.so via ctypes.

Configuration comes from the same COLTRAIN_* environment variables the reference's launcher sets
(pytorch/torch_col/csrc/config.cc:49-148)."""
from __future__ import annotations

import ctypes as C
import enum
import os
import time
from typing import List, Optional, Tuple

from ... import _lib
from ..._lib import call
from ..._runtime import CtrlMsg, StubConfig, TrainInfo


# ---- enums --------------------------------------------------------------------------------
class CtrlEvent(enum.IntEnum):  # common/inf_tra_comm/message_queue.h:18-40
    kTrainStart = 0
    kTrainEnd = 1
    kInterruptTrainDone = 2
    kResumeTrainDone = 3
    kColocateAdjustL1Done = 4
    kColocateAdjustL2Done = 5
    kReportBatchSize = 6
    kInterruptTrain = 7
    kResumeTrain = 8
    kColocateAdjustL1 = 9
    kColocateAdjustL2 = 10
    kInferExit = 11
    kInferenceWorkloadDone = 12
    kNumEvent = 13


class TrainMode(enum.Enum):  # cython/main.pyx TrainMode
    NORMAL = 'normal'
    COLOCATE_L1 = 'colocate-l1'
    COLOCATE_L2 = 'colocate-l2'
    TASKSWITCH_L0 = 'taskswitch-l0'
    TASKSWITCH_L1 = 'taskswitch-l1'
    TASKSWITCH_L2 = 'taskswitch-l2'
    TASKSWITCH_L3 = 'taskswitch-l3'

    def is_normal(self): return self == TrainMode.NORMAL
    def is_colocate(self): return self in (TrainMode.COLOCATE_L1, TrainMode.COLOCATE_L2)
    def is_taskswitch(self): return self.value.startswith('taskswitch')
    def is_kill_batch(self): return self in (TrainMode.COLOCATE_L1, TrainMode.TASKSWITCH_L1)


class ColocateCtrlHookMode(enum.Enum):
    NONE = 'none'
    SYNC = 'sync'
    XSCHED_SYNC = 'xsched-sync'
    XSCHED_SYNC2 = 'xsched-sync2'

    def use_xsched(self): return self in (ColocateCtrlHookMode.XSCHED_SYNC, ColocateCtrlHookMode.XSCHED_SYNC2)


# ---- TorchColConfig -------------------------------------------------------------------------
def _env_bool(name, default=False):
    v = os.environ.get(name)
    return default if v is None else v.strip() not in ('', '0', 'false', 'False')


class _Config:
    configured = False
    rank = 0
    world_size = 1
    use_shared_tensor = False
    use_xsched = False
    has_infer_server = False
    has_shared_tensor_server = False
    shared_tensor_pool_gb = 12.0
    dynamic_sm_partition = False
    hook_mode = ColocateCtrlHookMode.NONE
    train_mode = TrainMode.NORMAL
    profile_log_path = ''
    log_dynamic_batch = False
    log_control_stub = False
    release_interm_memory_by_grad_fn = False
    release_interm_memory_by_tagging = True
    use_fbward_hook = True
    comm_name: Optional[str] = None
    dist_name: Optional[str] = None

    @classmethod
    def init(cls):
        cls.use_shared_tensor = _env_bool('COLTRAIN_USE_SHARED_TENSOR')
        cls.use_xsched = _env_bool('COLTRAIN_USE_XSCHED')
        cls.has_infer_server = _env_bool('COLTRAIN_HAS_INFER_SERVER')
        cls.has_shared_tensor_server = _env_bool('COLTRAIN_HAS_SHARED_TENSOR_SERVER')
        cls.shared_tensor_pool_gb = float(os.environ.get('COLTRAIN_SHARED_TENSOR_POOL_GB', '12'))
        cls.dynamic_sm_partition = _env_bool('COLTRAIN_DYNAMIC_SM_PARTITION')
        cls.hook_mode = ColocateCtrlHookMode(os.environ.get('COLTRAIN_HOOK_MODE', 'none'))
        cls.train_mode = TrainMode(os.environ.get('COLTRAIN_MODE', 'normal'))
        cls.profile_log_path = os.environ.get('COLTRAIN_PROFILE_LOG_PATH', '')
        cls.log_dynamic_batch = _env_bool('COLTRAIN_LOG_DYNAMIC_BATCH') or _env_bool('COLTRAIN_LOG_ALL')
        cls.log_control_stub = _env_bool('COLTRAIN_LOG_CONTROL_STUB') or _env_bool('COLTRAIN_LOG_ALL')
        cls.comm_name = os.environ.get('SIRIUS_B200_COMM_NAME')
        cls.dist_name = os.environ.get('SIRIUS_B200_DIST_NAME')
        cls.configured = True

    @classmethod
    def kill_batch_on_recv(cls):  # config.cc:98-102
        return cls.hook_mode == ColocateCtrlHookMode.XSCHED_SYNC2 and cls.use_xsched


_comm = C.c_void_p()   # InfTraCommunicator
_dist_h = C.c_void_p()   # DistTrainSync (+ distributor + perf model)
_step = None           # the training step object kill_batch acts on


def is_configured(): return _Config.configured
def is_enable_shared_tensor(): return _Config.use_shared_tensor
def is_enable_dynamic_sm_partition(): return _Config.dynamic_sm_partition
def is_enable_xsched(): return _Config.use_xsched
def get_colocate_ctrl_hook_mode(): return _Config.hook_mode
def get_colocate_train_mode(): return _Config.train_mode
def is_release_interm_memory_v1(): return _Config.release_interm_memory_by_grad_fn
def is_release_interm_memory_v2(): return _Config.release_interm_memory_by_tagging
def disable_release_interm_memory():
    _Config.release_interm_memory_by_grad_fn = False
    _Config.release_interm_memory_by_tagging = False
def disable_fbward_hook(): _Config.use_fbward_hook = False
def is_enable_fbward_hook(): return _Config.use_fbward_hook
def is_train_master(): return _Config.rank == 0
def get_train_rank(): return _Config.rank
def set_train_rank(rank): _Config.rank = rank
def get_train_world_size(): return _Config.world_size
def set_train_world_size(ws): _Config.world_size = ws
def set_train_rank_world_size(rank, ws): _Config.rank, _Config.world_size = rank, ws
def has_colocated_infer_server(): return _Config.has_infer_server
def get_train_profile_log_path(): return _Config.profile_log_path
def get_unix_timestamp(): return int(time.time() * 1000)
def get_unix_timestamp_us(): return int(time.time() * 1e6)


def torch_col_init(rank: int, world_size: int, dist_timeout_ms: int = 10000):
    """TorchColInit (pytorch/torch_col/csrc/init.cc:17-41): config, the inf_tra_comm channel (opened
    as a trainer when an inference server exists) and the DistTrainSync segment of the job."""
    global _comm, _dist_h
    _Config.init()
    _Config.rank, _Config.world_size = rank, world_size
    if _Config.has_infer_server and not _comm:
        name = _Config.comm_name.encode() if _Config.comm_name else None
        call("srt_comm_open", name, 0, 0, world_size, 10000, C.byref(_comm))
    if not _dist_h:
        name = _Config.dist_name.encode() if _Config.dist_name else None
        call("srt_dist_open", name, rank, world_size, dist_timeout_ms, C.byref(_dist_h))


def torch_col_shutdown():
    global _comm, _dist_h
    if _dist_h:
        call("srt_dist_close", _dist_h)
        _dist_h = C.c_void_p()
    if _comm:
        call("srt_comm_close", _comm)
        _comm = C.c_void_p()
    _Config.configured = False


def comm_handle(): return _comm
def dist_handle(): return _dist_h


def set_train_step(step):
    """The step object (sirius_b200.step.ResNetStep or compatible) that kill_batch / memory release act on."""
    global _step
    _step = step


def get_train_step(): return _step


def init_train_info(init_batch_size: int, current_batch_size: int, model_name: str = ''):
    """cython/main.pyx:485-515: publish pid / batch sizes / model name on the information board."""
    if not _comm:
        return
    ti = TrainInfo(os.getpid(), _Config.rank, _Config.world_size, init_batch_size, current_batch_size,
                   init_batch_size, init_batch_size, model_name.encode()[:255], 0)
    call("srt_comm_set_train_info", _comm, _Config.rank, C.byref(ti))


def update_current_batch_size(batch_size: int):
    if _comm:
        call("srt_comm_update_train_field", _comm, _Config.rank, 4, int(batch_size))


def CallGLOG_INFO(msg, file='torch_col', line=0):
    m = msg.decode() if isinstance(msg, bytes) else str(msg)
    f = file.decode() if isinstance(file, bytes) else str(file)
    print(f'I {time.strftime("%H:%M:%S")} {os.path.basename(f)}:{line}] {m}', flush=True)


def CallGLOG_DINFO(msg, file='torch_col', line=0):
    if _env_bool('COLTRAIN_LOG_ALL'):
        CallGLOG_INFO(msg, file, line)


# ---- memory pool statistics (cython/main.pyx cuda_memory_pool_*) ------------------------------
_pool = C.c_void_p()


def set_memory_pool(pool_handle):
    global _pool
    _pool = pool_handle if isinstance(pool_handle, C.c_void_p) else C.c_void_p(pool_handle)


def memory_pool_handle(): return _pool
def _pool_stat(which): return _lib.lib().srt_pool_stat(_pool, which) if _pool else 0
def cuda_memory_pool_infer_usage(device_id=0): return _pool_stat(0)
def cuda_memory_pool_train_usage(device_id=0): return _pool_stat(1)
def cuda_memory_pool_train_peak_usage(device_id=0): return _pool_stat(2)
def cuda_memory_pool_train_all_usage(device_id=0): return _pool_stat(3)


def cuda_memory_pool_free_train_local(device_id=0):
    if _pool:
        n = C.c_size_t()
        call("srt_pool_empty_cache", _pool, 0, C.byref(n))
        return n.value
    return 0


# ---- PyTorch on the pool (csrc/torch_allocator_plugin.cc: the allocator installed into c10) -----------------
_torch_allocator_device = None


def install_torch_allocator(pool_gb: float = None, device: int = 0, cleanup: bool = True):
    """Make PyTorch's CUDA allocator allocate from the training side of the page pool: creates the default pool
    of `device` (COLTRAIN_SHARED_TENSOR_POOL_GB gigabytes by default, 12 as in the reference's config.cc), or
    attaches to the server's when COLTRAIN_HAS_SHARED_TENSOR_SERVER=1 and cleanup is False, and installs
    srt_alloc / srt_free through torch.cuda.memory.CUDAPluggableAllocator. Call before the first CUDA allocation
    of the process (PyTorch allows the switch only then). Returns the pool handle for the step executors."""
    global _torch_allocator_device
    import torch
    if pool_gb is None:
        pool_gb = float(os.environ.get('COLTRAIN_SHARED_TENSOR_POOL_GB', '12'))
    call("srt_pool_init", device, int(pool_gb * (1 << 30)), 1 if cleanup else 0)
    alloc = torch.cuda.memory.CUDAPluggableAllocator(str(_lib.LIB_PATH), "srt_alloc", "srt_free")
    torch.cuda.memory.change_current_allocator(alloc)
    h = C.c_void_p()
    call("srt_pool_default", device, C.byref(h))
    set_memory_pool(h)
    _torch_allocator_device = device
    return h


def release_interm_memory(keep_batch: int = 0):
    """CUDAColAllocator::ReleaseIntermMemory (torch_allocator_plugin.cc:343-369): drop every tagged
    intermediate tensor. The step object owns its activations, so this releases its activation set.
    With keep_batch > 0 the step keeps a set for that micro-batch size on pages that are already mapped
    and returns only the rest, which is what release + the next iteration's allocations amount to.
    Without a step object but with PyTorch on the pool (install_torch_allocator) the tagged blocks of the
    allocator seam are dropped."""
    if _step is not None and keep_batch > 0 and hasattr(_step, 'shrink_activations'):
        return _step.shrink_activations(min(int(keep_batch), getattr(_step, 'max_batch', int(keep_batch))))
    if _step is not None and hasattr(_step, 'release_activations'):
        return _step.release_activations()
    if _torch_allocator_device is not None:
        n = C.c_size_t()
        call("srt_release_interm", _torch_allocator_device, C.byref(n))
        return n.value
    return 0


# A step object knows its activations; these matter when PyTorch itself allocates from the pool.
def tag_model_start():
    if _torch_allocator_device is not None:
        call("srt_tag_model_begin")


def tag_model_end():
    if _torch_allocator_device is not None:
        call("srt_tag_model_end")


def tag_interm_memory(t):
    if _torch_allocator_device is not None and getattr(t, 'is_cuda', False):
        call("srt_tag_interm", C.c_void_p(t.data_ptr()), _torch_allocator_device)


def untag_interm_memory():
    if _torch_allocator_device is not None:
        call("srt_untag_interm", _torch_allocator_device)


def rearrange_memory(): raise RuntimeError('rearrange_memory is deprecated in the reference (mem_tagging.cc:47-49)')


# ---- stubs ------------------------------------------------------------------------------------
class _StubBase:
    def __init__(self, batch_size: int, kill_batch_on_recv=None, poll_ms=0, task_switch=False):
        cfg = StubConfig(_Config.rank, _Config.world_size,
                         int(_Config.kill_batch_on_recv() if kill_batch_on_recv is None else kill_batch_on_recv),
                         int(_Config.train_mode == TrainMode.COLOCATE_L1), batch_size, poll_ms, int(task_switch))
        self._h = C.c_void_p()
        # the ResNet executor is known to the stub directly; any other step object names its kill entry point
        target = _step.abort_target() if hasattr(_step, 'abort_target') else None
        step_h = None if target else getattr(_step, '_h', None)
        call("srt_stub_create", _comm if _comm else None, step_h, _dist_h if _dist_h else None, C.byref(cfg), C.byref(self._h))
        if target:
            call("srt_stub_set_abort_target", self._h, target[0], target[1])

    @property
    def cmd(self):
        v = _lib.lib().srt_stub_cmd(self._h)
        return CtrlEvent(v) if 0 <= v < CtrlEvent.kNumEvent else None

    @cmd.setter
    def cmd(self, v):
        call("srt_stub_set_cmd", self._h, -1 if v is None else int(v))

    def train_start(self): call("srt_stub_train_start", self._h)
    def train_end(self): call("srt_stub_train_end", self._h)
    def report_batch_size(self, bs): call("srt_stub_report_batch_size", self._h, int(bs))
    def StepsNoInteruptBegin(self): call("srt_stub_steps_no_interrupt_begin", self._h)
    def StepsNoInteruptEnd(self): call("srt_stub_steps_no_interrupt_end", self._h)
    def set_train_first_epoch_done(self): call("srt_stub_set_train_first_epoch_done", self._h)
    def can_exit_after_infer_worklaod_done(self): return bool(_lib.lib().srt_stub_can_exit_after_infer_workload_done(self._h))
    def EnableTorchColEngine(self): pass  # the step executor polls the kill flag itself

    def stop(self):
        if self._h:
            call("srt_stub_stop", self._h)
            self._h = C.c_void_p()


class PyDummyStub(_StubBase):
    def __init__(self):
        super().__init__(0, kill_batch_on_recv=False)


class PyColocateStub(_StubBase):
    def adjust_l1_done(self): call("srt_stub_adjust_l1_done", self._h)
    def adjust_l2_done(self): call("srt_stub_adjust_l2_done", self._h)
    def set_killed_batch_recover(self): call("srt_stub_set_killed_batch_recover", self._h)
    def set_killed_batch_reconfiged(self): call("srt_stub_set_killed_batch_reconfiged", self._h)
    def passed_time_from_set_cmd(self): return _lib.lib().srt_stub_passed_ms_from_set_cmd(self._h)

    def _bs(self, unpub):
        v = C.c_int()
        call("srt_stub_target_batch_size", self._h, int(unpub), C.byref(v))
        return v.value

    @property
    def target_batch_size(self): return self._bs(False)

    @property
    def unpub_target_batch_size(self): return self._bs(True)

    def _stamps(self, done):
        n = _lib.lib().srt_stub_adjust_timestamps(self._h, done, None, 0)
        buf = (C.c_int64 * max(n, 1))()
        n = _lib.lib().srt_stub_adjust_timestamps(self._h, done, buf, n)
        return list(buf[:n])


class PySwitchStub(_StubBase):
    """SwitchStub of the reference (cython/ctrl_stub.pxi, csrc/control_stub.cc:186-400): interrupt / resume of the
    whole training job for the task-switch modes."""

    def __init__(self, batch_size: int = 0, poll_ms: int = 0):
        super().__init__(batch_size, poll_ms=poll_ms, task_switch=True)

    def try_interrupt_train_done(self, barrier: bool = False) -> bool:
        v = C.c_int()
        call("srt_stub_try_interrupt_train_done", self._h, int(barrier), C.byref(v))
        return bool(v.value)

    def prepare_resume(self) -> bool:
        v = C.c_int()
        call("srt_stub_prepare_resume", self._h, C.byref(v))
        return bool(v.value)

    def _flag(self, which, set_, value=0):
        v = C.c_int()
        call("srt_stub_switch_flag", self._h, which, int(set_), int(value), C.byref(v))
        return bool(v.value)

    def get_global_interrupt_flag(self) -> bool: return self._flag(0, False)
    def set_global_interrupt_flag(self, flag: bool): self._flag(0, True, flag)
    def get_global_has_batch_killed(self) -> bool: return self._flag(1, False)
    def set_global_has_batch_killed(self, flag: bool): self._flag(1, True, flag)
    def set_killed_batch_recover(self): call("srt_stub_set_killed_batch_recover", self._h)

    def _stamps(self, done):
        n = _lib.lib().srt_stub_adjust_timestamps(self._h, done, None, 0)
        buf = (C.c_int64 * max(n, 1))()
        n = _lib.lib().srt_stub_adjust_timestamps(self._h, done, buf, n)
        return list(buf[:n])


_last_colocate_stub: Optional[PyColocateStub] = None


def get_adjust_request_time_stamp():
    return _last_colocate_stub._stamps(0) if _last_colocate_stub else []


def get_adjust_done_time_stamp():
    return _last_colocate_stub._stamps(1) if _last_colocate_stub else []


# ---- PyInfTraCommunicator (used by DebugServer and the inference stand-in) ------------------------
class PyCtrlMsgEntry:
    def __init__(self, id: int, event: int, value: int):
        self.id, self.event, self.value = id, CtrlEvent(event), value

    def __repr__(self): return f'CtrlMsgEntry(id={self.id}, event={self.event.name}, value={self.value})'


class PyInfTraCommunicator:
    """Server-side or trainer-side handle on the channel (ctrl::InfTraCommunicator)."""

    def __init__(self, is_server=True, cleanup=True, train_world_size=1, name: Optional[str] = None, timeout_ms=10000):
        self._h = C.c_void_p()
        self.is_server = is_server
        call("srt_comm_open", name.encode() if name else None, int(is_server), int(cleanup), train_world_size,
             timeout_ms, C.byref(self._h))

    def close(self):
        if self._h:
            call("srt_comm_close", self._h)
            self._h = C.c_void_p()

    def put(self, msg: PyCtrlMsgEntry, direction: int, rank: int):
        m = CtrlMsg(msg.id, int(msg.event), msg.value)
        call("srt_comm_put", self._h, C.byref(m), direction, rank)

    def put_inf2tra(self, event, id_, value, rank): self.put(PyCtrlMsgEntry(id_, event, value), 0, rank)
    def put_tra2inf(self, event, id_, value, rank): self.put(PyCtrlMsgEntry(id_, event, value), 1, rank)

    def put_all_inf2tra(self, event, id_, values):
        arr = (CtrlMsg * len(values))(*[CtrlMsg(id_, int(event), v) for v in values])
        call("srt_comm_put_all", self._h, arr, len(values), 0)

    def timed_get(self, timeout_ms, direction, rank) -> Optional[PyCtrlMsgEntry]:
        m, got = CtrlMsg(), C.c_int()
        call("srt_comm_timed_get", self._h, timeout_ms, direction, rank, C.byref(m), C.byref(got))
        return PyCtrlMsgEntry(m.id, m.event, m.value) if got.value else None

    def timed_get_from_any(self, timeout_ms, direction) -> Optional[Tuple[int, PyCtrlMsgEntry]]:
        m, got, rank = CtrlMsg(), C.c_int(), C.c_int()
        call("srt_comm_timed_get_from_any", self._h, timeout_ms, direction, C.byref(rank), C.byref(m), C.byref(got))
        return (rank.value, PyCtrlMsgEntry(m.id, m.event, m.value)) if got.value else None

    def get_train_info(self, rank) -> TrainInfo:
        ti = TrainInfo()
        call("srt_comm_get_train_info", self._h, rank, C.byref(ti))
        return ti

    def set_train_info(self, rank, **kw):
        ti = self.get_train_info(rank)
        for k, v in kw.items():
            setattr(ti, k, v.encode() if k == 'model_name' else v)
        call("srt_comm_set_train_info", self._h, rank, C.byref(ti))

    def update_field(self, rank, field, value): call("srt_comm_update_train_field", self._h, rank, field, value)

    def get_field(self, rank, field):
        v = C.c_int()
        call("srt_comm_get_train_field", self._h, rank, field, C.byref(v))
        return v.value

    def infer_tpc(self, device, op, value=0):
        v = C.c_int()
        call("srt_comm_infer_tpc", self._h, device, op, value, C.byref(v))
        return v.value


# ---- _dist_h: barrier, mailboxes, distributor, perf model (cython/dist.pyx) --------------------------
class _DistNamespace:
    @staticmethod
    def wait_barrier(timeout_ms: int = 60000): call("srt_dist_barrier", _dist_h, timeout_ms)

    @staticmethod
    def send_msg(dst: int, msg: str):
        data = msg.encode()
        # the mailbox holds 16 KiB; longer strings go in pieces, as the reference chunks by 256 bytes
        n = (len(data) + 16000 - 1) // 16000 or 1
        call("srt_dist_send", _dist_h, dst, str(n).encode(), len(str(n)))
        for i in range(n):
            piece = data[i * 16000:(i + 1) * 16000]
            call("srt_dist_send", _dist_h, dst, piece, len(piece))

    @staticmethod
    def recv_msg(src: int, timeout_ms: int = 60000) -> str:
        buf, n = C.create_string_buffer(16384), C.c_int()
        call("srt_dist_recv", _dist_h, src, buf, 16384, timeout_ms, C.byref(n))
        pieces = int(buf.raw[:n.value].decode())
        out = b''
        for _ in range(pieces):
            call("srt_dist_recv", _dist_h, src, buf, 16384, timeout_ms, C.byref(n))
            out += buf.raw[:n.value]
        return out.decode()

    @staticmethod
    def init_dynamic_batch_distributor(dataset_size, input_batch_size, global_batch_size, lazy, policy: str):
        pol = {'fix': 0, 'simple': 1, 'by_performance': 2}[policy.lower()]
        call("srt_dbd_init", _dist_h, dataset_size, input_batch_size, global_batch_size, int(lazy), pol)
        _DynamicBatchDistirbutor._lazy_distributing = bool(lazy)

    @staticmethod
    def init_train_performance_model(): pass  # the table lives in the DistTrainSync segment already


class _DynamicBatchDistirbutor:
    """Static facade over the shared ledger (cython/dist.pyx:84-146)."""
    _lazy_distributing = False

    @staticmethod
    def _ranges(batch_range_vec):
        flat = [v for r in batch_range_vec for v in r]
        return (C.c_int * max(len(flat), 1))(*flat), len(batch_range_vec)

    @staticmethod
    def distribute_batch(check_num_unproced_samples, distribute_to_all, at_global_batch_begin):
        call("srt_dbd_distribute_batch", _dist_h, _comm if _comm else None, int(check_num_unproced_samples),
             int(distribute_to_all), int(at_global_batch_begin))

    @staticmethod
    def get_batch(batch_size) -> Tuple[List[Tuple[int, int]], bool]:
        cap = 1024
        buf, n, last = (C.c_int * (2 * cap))(), C.c_int(), C.c_int()
        call("srt_dbd_get_batch", _dist_h, int(batch_size), buf, cap, C.byref(n), C.byref(last))
        return [(buf[2 * i], buf[2 * i + 1]) for i in range(n.value)], bool(last.value)

    @staticmethod
    def query_next_batch_size(batch_size) -> int:
        v = C.c_int()
        call("srt_dbd_query_next_batch_size", _dist_h, int(batch_size), C.byref(v))
        return v.value

    @staticmethod
    def finish_batch(batch_range_vec, end_of_global_batch):
        arr, n = _DynamicBatchDistirbutor._ranges(batch_range_vec)
        call("srt_dbd_finish_batch", _dist_h, arr, n, int(end_of_global_batch))

    @staticmethod
    def abort_batch(batch_range_vec, end_of_global_batch):
        arr, n = _DynamicBatchDistirbutor._ranges(batch_range_vec)
        call("srt_dbd_abort_batch", _dist_h, arr, n, int(end_of_global_batch))

    @staticmethod
    def vote_finish_last_micro_batch(timeout_ms=60000) -> bool:
        v = C.c_int()
        call("srt_dbd_vote_finish_last_micro_batch", _dist_h, timeout_ms, C.byref(v))
        return bool(v.value)

    @staticmethod
    def vote_abort_last_micro_batch(): call("srt_dbd_vote_abort_last_micro_batch", _dist_h)

    @staticmethod
    def reset_last_micro_batch_finish_vote(): call("srt_dbd_reset_last_micro_batch_finish_vote", _dist_h)

    @staticmethod
    def next_global_batch(timeout_ms=60000): call("srt_dbd_next_global_batch", _dist_h, _comm if _comm else None, timeout_ms)

    @staticmethod
    def next_epoch() -> int:
        v = C.c_int()
        call("srt_dbd_next_epoch", _dist_h, C.byref(v))
        return v.value

    @staticmethod
    def _info(which, rank=0):
        v = C.c_int()
        call("srt_dbd_info", _dist_h, which, rank, C.byref(v))
        return v.value

    @staticmethod
    def get_global_batch_size(): return _DynamicBatchDistirbutor._info(0)

    @staticmethod
    def get_num_global_batch_per_epoch(): return _DynamicBatchDistirbutor._info(1)

    @staticmethod
    def get_num_proced_global_batch(): return _DynamicBatchDistirbutor._info(2)


class _PerfModel:
    @staticmethod
    def record_thpt(batch_size, batch_time_ms):
        if batch_size > 0 and batch_time_ms > 0:
            call("srt_perf_record_thpt", _dist_h, int(batch_size), float(batch_time_ms))

    @staticmethod
    def get_thpt(batch_size) -> float:
        v = C.c_double()
        call("srt_perf_get_thpt", _dist_h, int(batch_size), C.byref(v))
        return v.value


_DistNamespace._DynamicBatchDistirbutor = _DynamicBatchDistirbutor
_DistNamespace._PerfModel = _PerfModel
dist = _DistNamespace


# ---- names of the reference's extension module that scripts and tools import (cython/main.pyx) -----------
def TorchColInit(train_rank: int = 0, train_world_size: int = 1):
    """csrc/init.cc:17-41 under its C++ name."""
    torch_col_init(train_rank, train_world_size)


def TorchDistExtInit():
    """The reference swaps c10d's Reducer / ProcessGroupNCCL for droppable ones here (csrc/dist_ext.cc:673-784).
    This library brings its own gradient exchange (sirius_b200.ddp.GradExchange: communicator, abort, restart), so
    there is nothing to patch inside PyTorch; the call reports whether that exchange can be used."""
    from ... import ddp
    return ddp.available()


def SMPartitionInit(stream: int = 0, device: int = 0):
    """common/sm_partition.cc: prepare the SM partition of `device`. Here: build the ladder of green-context
    partitions (one stream per width) the step executor switches between; returns the widths in SMs.
    `stream` is accepted for signature compatibility (the reference masks that stream; here a kernel is confined
    by the partition stream it is launched on)."""
    cap = 64
    sms, n = (C.c_int * cap)(), C.c_int()
    call("srt_smp_partition_levels", device, sms, cap, C.byref(n))
    return [sms[i] for i in range(n.value)]


def sm_partition_state(device: int = 0, gpu_tpc_num: int = 74, min_train_tpc: int = 5, max_train_tpc: int = 0):
    """(TPCs inference holds, TPCs training may use, mask of the TPCs closed to training) as the pre-launch hook
    computes them (common/sm_partition.cc:78-112) from the board's infer_required_tpc_num."""
    if not _comm:
        raise RuntimeError("not available: no colocated inference server (COLTRAIN_HAS_INFER_SERVER is off)")
    v = C.c_int()
    call("srt_comm_infer_tpc", _comm, device, 3, 0, C.byref(v))   # op 3: read
    mx = max_train_tpc if max_train_tpc > 0 else gpu_tpc_num
    lib = _lib.lib()
    return (v.value, lib.srt_smp_train_avail_tpc_num(v.value, gpu_tpc_num, min_train_tpc, mx),
            lib.srt_smp_train_avail_tpc_mask(v.value, gpu_tpc_num, min_train_tpc, mx))


def monitor_sm_partition(interval: float, iterations: int = None, out=None):
    """cython/main.pyx:323-340: print the partition state every `interval` seconds (forever by default)."""
    import sys
    out = out or sys.stdout
    if not has_colocated_infer_server() or not _comm:
        print("There not exist colocated infer server", file=out)
        return
    i = 0
    while iterations is None or i < iterations:
        infer, train, mask = sm_partition_state()
        print("Infer TPC Num: {}, Train TPC Num: {}, Train Avail TPC Mask: {}".format(infer, train, hex(mask)), file=out)
        i += 1
        if iterations is None or i < iterations:
            time.sleep(interval)


class PyTensorWeakRef:
    """cython/main.pyx:550-567: sizes and address of a tensor without keeping it alive."""

    def __init__(self, tensor):
        import weakref
        self._ref = weakref.ref(tensor)

    def _get(self): return self._ref()

    def nbytes(self):
        t = self._get()
        return 0 if t is None else t.numel() * t.element_size()

    def storage_nbytes(self):
        t = self._get()
        return 0 if t is None else t.untyped_storage().nbytes()

    def data_ptr(self):
        t = self._get()
        return 0 if t is None else t.data_ptr()


def release_underlying_storage(tensor):
    """csrc/mem_tagging.cc ReleaseUnderlyingStorage: give the tensor's memory back to the allocator now; the
    tensor object stays (empty). With PyTorch on the pool (install_torch_allocator) the block returns to the
    training allocator at once."""
    tensor.untyped_storage().resize_(0)


def release_grad_fn_saved_tensor(grad_fn):
    """csrc/mem_tagging.cc ReleaseGradFnSavedTensor: walk the autograd graph below grad_fn and free the storage
    of every tensor the nodes saved for backward (the batch was killed; the graph will never run). Returns the
    number of bytes freed."""
    seen, stack, freed = set(), [grad_fn], 0
    while stack:
        node = stack.pop()
        if node is None or id(node) in seen:
            continue
        seen.add(id(node))
        for name in dir(node):
            if not name.startswith('_saved_'):
                continue
            try:
                v = getattr(node, name)
            except Exception:      # already released by autograd
                continue
            for t in (v if isinstance(v, (list, tuple)) else (v,)):
                if hasattr(t, 'untyped_storage') and getattr(t, 'is_cuda', False):
                    st = t.untyped_storage()
                    freed += st.nbytes()
                    st.resize_(0)
        stack.extend(fn for fn, _ in getattr(node, 'next_functions', ()))
    return freed


def DumpMempoolFreeList(filename):
    raise RuntimeError("not available: removed in the reference as well (csrc/util.cc:38-43 aborts with 'removed, to be re-impl'); "
                       "srt_pool_stat / MemoryPool report the pool's state")


def DumpMempoolBlockList(filename):
    raise RuntimeError("not available: removed in the reference as well (csrc/util.cc:38-43 aborts with 'removed, to be re-impl'); "
                       "srt_pool_stat / MemoryPool report the pool's state")


# The xsched calls under their C++ names (cython/main.pyx:286-301). Every training kernel is launched by the
# step executor, which stops between units when asked and never has more than a few units in flight, so the
# "queue" these act on is the executor's launch-ahead window.
def RegisterStream(stream):
    from .. import xsched
    xsched.register_stream(stream)
    return int(stream) if isinstance(stream, int) else 0


def UnRegisterStream(stream):
    from .. import xsched
    xsched.unregister_stream(stream)


def UnRegisterAllStreams():
    from .. import xsched
    xsched.unregister_all_streams()


def GetXQueueSize(stream=None):
    from .. import xsched
    return xsched.get_xqueue_size(stream)


def GetXQueueSizeAllStreams(): return GetXQueueSize(None)
def GetTotalXQueueSize(): return GetXQueueSize(None)


def AbortStream(stream=None):
    from .. import xsched
    return xsched.kill_batch(synchronize=False)


def AbortAllStreams(): return AbortStream(None)


def SyncStream(stream=None):
    if _step is not None and hasattr(_step, 'synchronize'):
        _step.synchronize()
    return 0


def SyncAllStreams(): return SyncStream(None)


def SetRejectCudaCalls(reject: bool):
    from .. import xsched
    xsched.set_reject_cuda_calls(reject)


def GuessNcclBegin():
    from .. import xsched
    xsched.guess_nccl_begin()


def GuessNcclEnd():
    from .. import xsched
    xsched.guess_nccl_end()


def IsGuessNcclBegined():
    from .. import xsched
    return xsched.is_guess_nccl_begined()


def GetNcclStreams():
    from .. import xsched
    return xsched.get_nccl_streams()


# torch_col._C._dist names at this level too (cython/dist.pyx:25-194)
wait_barrier = _DistNamespace.wait_barrier
send_msg = _DistNamespace.send_msg
recv_msg = _DistNamespace.recv_msg
init_dynamic_batch_distributor = _DistNamespace.init_dynamic_batch_distributor
init_train_performance_model = _DistNamespace.init_train_performance_model

from . import _dist, _main  # noqa: E402,F401  (torch_col._C._main / torch_col._C._dist, as pytorch/setup.py:101-114 builds them)
