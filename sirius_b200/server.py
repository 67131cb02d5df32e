"""Python handles on the server side of the colocation protocol (include/sirius_server.h): Controller,
ResourceManager, ColdModelCache, TrainLauncher, KVCachePool. An inference server (or the stand-in inference
workers of the benchmarks) drives the trainers through these, as the reference's server does through the
classes of the same names (server/control/controller.cc, server/resource_manager.cc,
server/model_store/model_cache.cc, server/train_launcher.cc, server/llm/kv_cache_pool.cc)."""
from __future__ import annotations

import ctypes as C
import enum
from typing import List, Optional, Sequence, Tuple

from . import _lib, _runtime  # noqa: F401
from ._lib import call, register

_vp, _i, _i64, _u64, _d, _sz = C.c_void_p, C.c_int, C.c_int64, C.c_uint64, C.c_double, C.c_size_t
_pi, _pu64, _pd, _psz = C.POINTER(_i), C.POINTER(_u64), C.POINTER(_d), C.POINTER(_sz)


class ServeMode(enum.IntEnum):
    NORMAL = 0
    TASKSWITCH_L1 = 1
    TASKSWITCH_L3 = 2
    COLOCATE_L1 = 3
    COLOCATE_L2 = 4


class TrainStatus(enum.IntEnum):
    IDLE = 0
    RUNNING = 1
    INTERRUPTED = 2


class ControllerConfig(C.Structure):
    _fields_ = [("serve_mode", _i), ("dummy_adjust", _i)]


class ColdCacheConfig(C.Structure):
    _fields_ = [("min_capacity_nbytes", _sz), ("max_capacity_nbytes", _sz), ("ratio", _d)]


class LauncherConfig(C.Structure):
    _fields_ = [("serve_mode", _i), ("use_xsched", _i), ("use_shared_tensor_train", _i), ("cuda_memory_pool_gb", _d),
                ("freelist_policy", C.c_char_p), ("train_profile", C.c_char_p), ("skip_set_mps_thread_percent", _i),
                ("dynamic_sm_partition", _i), ("train_mps_thread_percent", _i), ("enable_train_adjust_balance", _i)]


class KvPoolConfig(C.Structure):
    _fields_ = [("device_id", _i), ("train_memory_over_predict_mb", _d), ("train_over_adjust_nbytes", _sz),
                ("min_adjust_nbytes", _sz), ("reclaim_free_nbytes", _sz), ("reclaim_margin_nbytes", _sz),
                ("adjust_timeout_ms", _i)]


register({
    "srt_controller_create": (None, [_vp, _vp, C.POINTER(ControllerConfig), C.POINTER(_vp)]),
    "srt_controller_destroy": (None, [_vp]),
    "srt_controller_train_status": (None, [_vp, _pi]),
    "srt_controller_cur_batch_size": (None, [_vp, _pi]),
    "srt_controller_set_train_pid": (None, [_vp, _i]),
    "srt_controller_interrupt_train": (None, [_vp, _pu64]),
    "srt_controller_resume_train": (None, [_vp, _pu64]),
    "srt_controller_colocate_adjust": (None, [_vp, _i, _i, _pu64]),
    "srt_controller_infer_require_adjust": (None, [_vp, _i, _pi, _i, _pu64]),
    "srt_controller_infer_release_adjust": (None, [_vp, _pi, _i, _pu64]),
    "srt_controller_dummy_infer_exit": (None, [_vp, _i, _i, _pu64]),
    "srt_controller_inference_workload_done": (None, [_vp]),
    "srt_controller_wait_train_not_running": (None, [_vp, _i]),
    "srt_controller_wait_task_switch_done": (None, [_vp, _u64, _i]),
    "srt_controller_wait_colocate_adjust_done": (None, [_vp, _i, _u64, _i]),
    "srt_controller_set_infer_status": (None, [_vp, _i]),
    "srt_controller_wait_infer_idle": (None, [_vp, _i]),
    "srt_controller_has_flying_colocate_adjust": (None, [_vp, _pi]),
    "srt_resmgr_infer_memory_mb": (_d, [_vp]),
    "srt_resmgr_train_memory_mb": (_d, [_vp]),
    "srt_resmgr_free_memory_mb": (None, [_vp, _vp, _i, _d, _pd]),
    "srt_resmgr_train_avail_memory_mb": (None, [_vp, _d, _pd]),
    "srt_cold_cache_create": (None, [C.POINTER(ColdCacheConfig), C.POINTER(_vp)]),
    "srt_cold_cache_destroy": (None, [_vp]),
    "srt_cold_cache_push": (None, [_vp, C.c_char_p, _d, _psz, _i, _pi, _i, _pi, C.c_char_p, _sz, _pi]),
    "srt_cold_cache_pop": (None, [_vp, C.c_char_p, _i, _pi, _i, _pi, _pi]),
    "srt_cold_cache_take_space": (None, [_vp, _sz, _pi]),
    "srt_cold_cache_set_capacity": (None, [_vp, _sz]),
    "srt_cold_cache_info": (None, [_vp, _psz, _psz]),
    "srt_cold_cache_reserve_mb": (_d, [_vp]),
    "srt_cold_cache_releasable_mb": (_d, [_vp]),
    "srt_cold_cache_buffer_mb": (_d, [_vp, _d]),
    "srt_launcher_env": (None, [C.POINTER(LauncherConfig), C.c_char_p, _sz]),
    "srt_launcher_argv": (None, [C.c_char_p, C.c_char_p, C.c_char_p, _sz, _pi]),
    "srt_launcher_launch": (None, [C.POINTER(LauncherConfig), C.c_char_p, C.c_char_p, C.c_char_p, C.c_char_p, _pi]),
    "srt_launcher_wait": (None, [_i, _i, _pi, _pi]),
    "srt_launcher_kill": (None, [_i]),
    "srt_launcher_supervise": (None, [_vp, _vp, _i, _i, _pi, _pi]),
    "srt_launcher_kill_train": (None, [_vp, _pi]),
    "srt_launcher_dummy_adjust": (None, [_vp, _i, _i, _i, C.c_uint, _i, _i, _pi]),
    "srt_kvpool_create": (None, [_vp, _vp, _vp, C.POINTER(KvPoolConfig), C.POINTER(_vp)]),
    "srt_kvpool_destroy": (None, [_vp]),
    "srt_kvpool_set_block_shape": (None, [_vp, _i64, _i64, _i64, _i64, _sz]),
    "srt_kvpool_num_gpu_blocks": (_i64, [_vp]),
    "srt_kvpool_shape": (None, [_vp, C.POINTER(_i64), C.POINTER(_i64)]),
    "srt_kvpool_layer_block_info": (None, [_vp, C.POINTER(_i64), C.POINTER(_i64)]),
    "srt_kvpool_update_free_layer_blocks": (None, [_vp, _i64]),
    "srt_kvpool_update_free_layer_blocks_by_train_base": (None, [_vp, _sz]),
    "srt_kvpool_alloc_pages": (None, [_vp, _sz, _i, _pu64, _pi]),
    "srt_kvpool_free_pages": (None, [_vp, _pu64, _i, _pi]),
    "srt_kvpool_util": (_d, [_vp]),
    "srt_adjuster_predict_train_mem_usage_mb": (None, [_vp, _i, _pd]),
    "srt_adjuster_llm_require_plan": (None, [_vp, _i, _d, _d, _pd, _pi, _pi]),
    "srt_adjuster_llm_release_plan": (None, [_vp, _pd, _pd, _pi, _pi]),
})


def _h(x):
    """Accept a raw handle or any wrapper that carries one in ._h / .handle."""
    if x is None:
        return None
    for attr in ("_h", "handle"):
        if hasattr(x, attr):
            return getattr(x, attr)
    return x


class Controller:
    """server/control/controller.cc:84-445. comm: the channel opened as server (PyInfTraCommunicator(True, ...))."""

    def __init__(self, comm, adjuster=None, serve_mode: ServeMode = ServeMode.COLOCATE_L1, dummy_adjust: bool = False):
        cfg = ControllerConfig(int(serve_mode), int(dummy_adjust))
        self._h = _vp()
        self._keep = (comm, adjuster)
        call("srt_controller_create", _h(comm), _h(adjuster), C.byref(cfg), C.byref(self._h))

    def _cmd(self, name, *args) -> int:
        cid = _u64(0)
        call(name, self._h, *args, C.byref(cid))
        return cid.value

    def interrupt_train(self) -> int: return self._cmd("srt_controller_interrupt_train")
    def resume_train(self) -> int: return self._cmd("srt_controller_resume_train")
    def colocate_adjust(self, device_id: int, batch_size: int) -> int: return self._cmd("srt_controller_colocate_adjust", device_id, batch_size)

    def colocate_infer_require_adjust(self, device_id: int, plan: Sequence[int]) -> int:
        arr = (_i * len(plan))(*plan)
        return self._cmd("srt_controller_infer_require_adjust", device_id, arr, len(plan))

    def colocate_infer_release_adjust(self, plan: Sequence[int]) -> int:
        arr = (_i * len(plan))(*plan)
        return self._cmd("srt_controller_infer_release_adjust", arr, len(plan))

    def dummy_infer_exit(self, device_id: int, target_batch_size: int) -> int:
        return self._cmd("srt_controller_dummy_infer_exit", device_id, target_batch_size)

    def inference_workload_done(self): call("srt_controller_inference_workload_done", self._h)
    def wait_train_not_running(self, timeout_ms=-1): call("srt_controller_wait_train_not_running", self._h, timeout_ms)
    def wait_task_switch_done(self, cmd_id, timeout_ms=-1): call("srt_controller_wait_task_switch_done", self._h, cmd_id, timeout_ms)

    def wait_colocate_adjust_done(self, device_id, cmd_id, timeout_ms=-1):
        call("srt_controller_wait_colocate_adjust_done", self._h, device_id, cmd_id, timeout_ms)

    def set_infer_status(self, running: bool): call("srt_controller_set_infer_status", self._h, int(running))
    def wait_infer_idle(self, timeout_ms=-1): call("srt_controller_wait_infer_idle", self._h, timeout_ms)
    def set_train_pid(self, pid: int): call("srt_controller_set_train_pid", self._h, pid)

    def train_status(self) -> TrainStatus:
        v = _i()
        call("srt_controller_train_status", self._h, C.byref(v))
        return TrainStatus(v.value)

    def is_train_idle(self) -> bool: return self.train_status() == TrainStatus.IDLE

    def cur_batch_size(self) -> int:
        v = _i()
        call("srt_controller_cur_batch_size", self._h, C.byref(v))
        return v.value

    def has_flying_colocate_adjust(self) -> bool:
        v = _i()
        call("srt_controller_has_flying_colocate_adjust", self._h, C.byref(v))
        return bool(v.value)

    def close(self):
        if self._h:
            call("srt_controller_destroy", self._h)
            self._h = _vp()


class ResourceManager:
    """server/resource_manager.cc:22-104 in shared-tensor mode: every figure comes from the page pool."""

    def __init__(self, pool, adjuster=None, train_memory_over_predict_mb: float = 0.0):
        self.pool, self.adjuster, self.over = pool, adjuster, train_memory_over_predict_mb

    def infer_memory_mb(self) -> float: return _lib.lib().srt_resmgr_infer_memory_mb(_h(self.pool))
    def train_memory_mb(self) -> float: return _lib.lib().srt_resmgr_train_memory_mb(_h(self.pool))

    def free_memory_mb(self, device_id: int = 0) -> float:
        v = _d()
        call("srt_resmgr_free_memory_mb", _h(self.pool), _h(self.adjuster), device_id, self.over, C.byref(v))
        return v.value

    def train_avail_memory_mb(self) -> float:
        v = _d()
        call("srt_resmgr_train_avail_memory_mb", _h(self.pool), self.over, C.byref(v))
        return v.value


class ColdModelCache:
    """server/model_store/model_cache.{h,cc}: which parameter groups of cold models stay in GPU memory."""

    def __init__(self, min_capacity_nbytes: int, max_capacity_nbytes: int, ratio: float = 1.0):
        cfg = ColdCacheConfig(min_capacity_nbytes, max_capacity_nbytes, ratio)
        self._h = _vp()
        call("srt_cold_cache_create", C.byref(cfg), C.byref(self._h))

    def push(self, name: str, groups_nbytes: Sequence[int], hotness: float = 0.0) -> Tuple[List[int], List[str], bool]:
        n = len(groups_nbytes)
        g = (_sz * n)(*groups_nbytes)
        cached, nc, ok = (_i * n)(), _i(), _i()
        ev = C.create_string_buffer(1 << 16)
        call("srt_cold_cache_push", self._h, name.encode(), float(hotness), g, n, cached, n, C.byref(nc), ev, len(ev), C.byref(ok))
        names = ev.value.decode().split("\n") if ev.value else []
        return [cached[i] for i in range(nc.value)], names, bool(ok.value)

    def pop(self, name: str, pop_to_inference: bool) -> Tuple[List[int], bool]:
        cap = 4096
        cached, nc, ok = (_i * cap)(), _i(), _i()
        call("srt_cold_cache_pop", self._h, name.encode(), int(pop_to_inference), cached, cap, C.byref(nc), C.byref(ok))
        return [cached[i] for i in range(min(nc.value, cap))], bool(ok.value)

    def take_space(self, nbytes: int) -> bool:
        ok = _i()
        call("srt_cold_cache_take_space", self._h, nbytes, C.byref(ok))
        return bool(ok.value)

    def set_new_capacity(self, nbytes: int): call("srt_cold_cache_set_capacity", self._h, nbytes)

    def capacity_and_cache(self) -> Tuple[int, int]:
        a, b = _sz(), _sz()
        call("srt_cold_cache_info", self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def reserve_memory_mb(self) -> float: return _lib.lib().srt_cold_cache_reserve_mb(self._h)
    def releasable_memory_mb(self) -> float: return _lib.lib().srt_cold_cache_releasable_mb(self._h)
    def buffer_mb(self, free_memory_mb: float) -> float: return _lib.lib().srt_cold_cache_buffer_mb(self._h, free_memory_mb)

    def close(self):
        if self._h:
            call("srt_cold_cache_destroy", self._h)
            self._h = _vp()


class JobOutcome(enum.IntEnum):
    RUNNING = 0
    FINISHED = 1
    KILLED = 2
    FAILED = 3


class TrainLauncher:
    """server/train_launcher.cc:88-311: the environment and command line a training job is started with."""

    def __init__(self, serve_mode: ServeMode = ServeMode.COLOCATE_L1, use_xsched: bool = True,
                 use_shared_tensor_train: bool = True, cuda_memory_pool_gb: float = 12.0, freelist_policy: str = "best-fit",
                 train_profile: str = "", skip_set_mps_thread_percent: bool = True, dynamic_sm_partition: bool = False,
                 train_mps_thread_percent: int = -1, enable_train_adjust_balance: bool = False):
        self._policy, self._profile = freelist_policy.encode(), train_profile.encode()
        self.cfg = LauncherConfig(int(serve_mode), int(use_xsched), int(use_shared_tensor_train), cuda_memory_pool_gb,
                                  self._policy, self._profile, int(skip_set_mps_thread_percent), int(dynamic_sm_partition),
                                  train_mps_thread_percent, int(enable_train_adjust_balance))
        self.pid = -1
        self.job_batch_size = 0

    def env(self) -> dict:
        buf = C.create_string_buffer(4096)
        call("srt_launcher_env", C.byref(self.cfg), buf, len(buf))
        return dict(line.split("=", 1) for line in buf.value.decode().splitlines())

    def argv(self, script: str, args: str) -> List[str]:
        buf, bs = C.create_string_buffer(1 << 16), _i()
        call("srt_launcher_argv", script.encode(), args.encode(), buf, len(buf), C.byref(bs))
        self.job_batch_size = bs.value
        return buf.value.decode().split("\n")

    def launch(self, script: str, args: str = "", interpreter: Optional[str] = None, log_path: Optional[str] = None) -> int:
        self.argv(script, args)
        pid = _i()
        call("srt_launcher_launch", C.byref(self.cfg), interpreter.encode() if interpreter else None, script.encode(),
             args.encode(), log_path.encode() if log_path else None, C.byref(pid))
        self.pid = pid.value
        return self.pid

    def wait(self, timeout_ms: int = -1) -> Optional[int]:
        """Exit status of the job, or None when it still runs after timeout_ms."""
        done, st = _i(), _i()
        call("srt_launcher_wait", self.pid, timeout_ms, C.byref(done), C.byref(st))
        return st.value if done.value else None

    def kill(self):
        if self.pid > 0:
            call("srt_launcher_kill", self.pid)

    def supervise(self, controller=None, comm=None, timeout_ms: int = -1):
        """(outcome, exit status) of the job: JobOutcome.RUNNING after timeout_ms, FINISHED, KILLED (SIGKILL: launch
        it again, as the reference's Train() loop does). A job that died of another signal raises SrtError after
        every rank on the board has been killed (server/train_launcher.cc:335-381)."""
        out, st = _i(), _i()
        call("srt_launcher_supervise", _h(controller), _h(comm), self.pid, timeout_ms, C.byref(out), C.byref(st))
        if out.value != JobOutcome.RUNNING:
            self.pid = -1
        return JobOutcome(out.value), (st.value if out.value != JobOutcome.RUNNING else None)

    @staticmethod
    def kill_train(comm) -> int:
        """KillTrain: SIGKILL to every rank registered on the board; returns how many were signalled."""
        n = _i()
        call("srt_launcher_kill_train", _h(comm), C.byref(n))
        return n.value

    @staticmethod
    def dummy_adjust(controller, original_target_bs: int, delay_ms: int = -1, duration_ms: int = 0, seed: int = 42,
                     min_gap_ms: int = 0, max_gap_ms: int = 0) -> int:
        """DummyAdjust (blocking; run it on a thread): random shrink-by-one / grow-back rounds while training runs.
        Returns the number of rounds."""
        n = _i()
        call("srt_launcher_dummy_adjust", _h(controller), original_target_bs, delay_ms, duration_ms, seed, min_gap_ms,
             max_gap_ms, C.byref(n))
        return n.value


class KVCachePool:
    """server/llm/kv_cache_pool.cc:232-347: the LLM's KV cache in pages of the pool's inference allocator; asks
    training to shrink when the pool runs short, lets it grow again when pages come back."""

    def __init__(self, pool, controller: Optional[Controller] = None, adjuster=None, device_id: int = 0,
                 train_memory_over_predict_mb: float = 0.0, train_over_adjust_nbytes: int = 0, min_adjust_nbytes: int = 0,
                 reclaim_free_nbytes: int = 0, reclaim_margin_nbytes: int = 0, adjust_timeout_ms: int = 0):
        cfg = KvPoolConfig(device_id, train_memory_over_predict_mb, train_over_adjust_nbytes, min_adjust_nbytes,
                           reclaim_free_nbytes, reclaim_margin_nbytes, adjust_timeout_ms)
        self._h = _vp()
        self._keep = (pool, controller, adjuster)
        call("srt_kvpool_create", _h(pool), _h(controller), _h(adjuster), C.byref(cfg), C.byref(self._h))

    def set_block_shape(self, block_size, num_layers, num_heads, head_size, block_nbytes):
        call("srt_kvpool_set_block_shape", self._h, block_size, num_layers, num_heads, head_size, block_nbytes)

    def num_gpu_blocks(self) -> int: return _lib.lib().srt_kvpool_num_gpu_blocks(self._h)

    def shape_and_stride(self):
        s, t = (_i64 * 3)(), (_i64 * 3)()
        call("srt_kvpool_shape", self._h, s, t)
        return list(s), list(t)

    def layer_block_info(self) -> Tuple[int, int]:
        a, b = _i64(), _i64()
        call("srt_kvpool_layer_block_info", self._h, C.byref(a), C.byref(b))
        return a.value, b.value

    def update_num_free_layer_blocks(self, delta: int): call("srt_kvpool_update_free_layer_blocks", self._h, delta)
    def update_num_free_layer_blocks_by_train_base(self, nbytes: int): call("srt_kvpool_update_free_layer_blocks_by_train_base", self._h, nbytes)

    def alloc_pages(self, page_nbytes: int, n: int) -> Tuple[List[int], bool]:
        out, adj = (_u64 * n)(), _i()
        call("srt_kvpool_alloc_pages", self._h, page_nbytes, n, out, C.byref(adj))
        return list(out), bool(adj.value)

    def free_pages(self, pages: Sequence[int]) -> bool:
        arr, rec = (_u64 * len(pages))(*pages), _i()
        call("srt_kvpool_free_pages", self._h, arr, len(pages), C.byref(rec))
        return bool(rec.value)

    def util(self) -> float: return _lib.lib().srt_kvpool_util(self._h)

    def close(self):
        if self._h:
            call("srt_kvpool_destroy", self._h)
            self._h = _vp()
