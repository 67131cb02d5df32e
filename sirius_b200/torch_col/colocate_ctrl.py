"""Colocate controllers (pytorch/torch_col/colocate_ctrl.py): the object the training loop talks to.

ColocateCtrl wraps the control stub; `steps_no_interrupt()` is the critical section around the
optimizer step, `adjust_l1()` / `adjust_l2()` release memory and reply to the inference server."""
from __future__ import annotations

import abc
import contextlib
import os
import time
from typing import List, Optional, Union

from . import _C, xsched
from ._C import ColocateCtrlHookMode, CtrlEvent, TrainMode
from .util import EventManager, MemoryPool


_saved_tensor_hook_on = False


def register_saved_tensor_hook():
    """colocate_ctrl.py:18-29: every tensor autograd saves for backward is tagged as an intermediate, so that
    release_interm_memory() can give its memory back in one call. Only matters when PyTorch itself allocates from the
    pool (torch_col._C.install_torch_allocator); a step object knows its own activation set."""
    global _saved_tensor_hook_on
    if _saved_tensor_hook_on:
        return
    try:
        import torch
    except ImportError:
        return

    def pack_hook(x):
        _C.tag_interm_memory(x)
        return x

    torch._C._autograd._push_saved_tensors_default_hooks(pack_hook, lambda x: x)
    _saved_tensor_hook_on = True


class ColocateAdjustL1Exception(Exception):
    pass


class EngineColocateAdjustL1Exception(Exception):
    pass


class SwitchL1Exception(Exception):
    pass


class CtrlBase(abc.ABC):
    _colocate_ctrl = None

    def __init__(self, train_mode: TrainMode, hook_mode: ColocateCtrlHookMode, num_epoch: int, batch_size: int):
        if CtrlBase._colocate_ctrl is not None:
            raise RuntimeError("Only one instance of Colocate Ctrl can be created.")
        CtrlBase._colocate_ctrl = self
        self.train_mode = train_mode
        self.hook_mode = hook_mode
        self.input_batch_size = batch_size
        self.num_epoch = num_epoch
        self._stub = None

    @classmethod
    def _reset(cls):
        if cls._colocate_ctrl is not None and cls._colocate_ctrl._stub is not None:
            cls._colocate_ctrl._stub.stop()
        cls._colocate_ctrl = None

    def release_and_reply(self, barrier: Optional[bool] = None):
        if self.train_mode.is_colocate():
            return self.adjust()
        if self.train_mode.is_taskswitch():
            return self.switch(bool(barrier))

    # ---- forward / backward hooks for torch modules (colocate_ctrl.py:101-110, 176-260, 355-400) ------------------
    # A step object polls the kill flag between its units by itself; a torch.nn.Module trained on the allocator seam
    # gets the reference's hooks: every leaf module checks the command after its forward and before its backward.
    _kill_event = None         # the command that ends a micro-batch in this mode
    _kill_exception = None

    @classmethod
    def register_fbward_hook(cls, module, fwd_hook, bwd_hook):
        if not _C.is_enable_fbward_hook():
            return
        children = list(module.children())
        if not children:
            module.register_forward_hook(fwd_hook)
            module.register_full_backward_hook(bwd_hook)
        else:
            for child in children:
                cls.register_fbward_hook(child, fwd_hook, bwd_hook)

    def _make_hook(self, where: str):
        sync_first = self.hook_mode == ColocateCtrlHookMode.SYNC

        def hook(module, _in, _out):
            with EventManager.record_duration_event(where):
                if sync_first:
                    import torch
                    if torch.cuda.is_available():
                        torch.cuda.current_stream().synchronize()
                if self._stub.cmd == self._kill_event:
                    if not sync_first:
                        xsched.kill_batch()
                    raise self._kill_exception(f'[{where}]')
        return hook

    def register_pytorch_hook(self, module_list: List = ()):
        """Hooks on every leaf of the torch modules in module_list (entries that are not torch modules, such as step
        objects, are skipped). xsched-sync2 relies on an autograd-engine hook in the reference's PyTorch fork; on stock
        PyTorch it gets the module-level hooks of xsched-sync."""
        if self._kill_event is None or self.hook_mode == ColocateCtrlHookMode.NONE:
            return
        name = {ColocateCtrlHookMode.SYNC: 'sync'}.get(self.hook_mode, 'xsched_sync')
        n = 0
        for module in module_list:
            if hasattr(module, 'children') and hasattr(module, 'register_forward_hook'):
                CtrlBase.register_fbward_hook(module, self._make_hook(f'{name}_fwd'), self._make_hook(f'{name}_bwd'))
                n += 1
        if n and _C.is_release_interm_memory_v2():
            register_saved_tensor_hook()

    def train_start(self): self._stub.train_start()
    def train_end(self): self._stub.train_end()
    def stop(self): self._stub.stop()
    def can_exit_after_infer_worklaod_done(self): return self._stub.can_exit_after_infer_worklaod_done()
    def set_train_first_epoch_done(self): self._stub.set_train_first_epoch_done()


class ColocateCtrl(CtrlBase):
    def __init__(self, train_mode, hook_mode, num_epoch, batch_size, stub_poll_ms: int = 0):
        assert train_mode in (TrainMode.COLOCATE_L1, TrainMode.COLOCATE_L2)
        super().__init__(train_mode, hook_mode, num_epoch, batch_size)
        self._stub = _C.PyColocateStub(batch_size, poll_ms=stub_poll_ms)
        _C._last_colocate_stub = self._stub
        if train_mode == TrainMode.COLOCATE_L1:
            self._kill_event, self._kill_exception = CtrlEvent.kColocateAdjustL1, ColocateAdjustL1Exception
        # keep an activation set for the announced batch size through an L1 adjust instead of dropping
        # everything and mapping it again at the next iteration (COLTRAIN_KEEP_TARGET_SET=0 restores that)
        self.keep_target_set = os.environ.get('COLTRAIN_KEEP_TARGET_SET', '1') != '0'
        self.adjust_log = []  # (release_ms, empty_cache_ms, reply_ms, released_bytes, start time.time())

    def check_kill(self, where: str):
        """What the reference's forward/backward hooks do (colocate_ctrl.py:360-400)."""
        if self.train_mode == TrainMode.COLOCATE_L1 and self._stub.cmd == CtrlEvent.kColocateAdjustL1:
            xsched.kill_batch()
            raise ColocateAdjustL1Exception(where)

    @contextlib.contextmanager
    def steps_no_interrupt(self):
        if self.train_mode == TrainMode.COLOCATE_L1:
            step = _C.get_train_step()
            if step is not None and hasattr(step, 'synchronize'):
                step.synchronize()  # SyncAllStreams
            if self._stub.cmd == CtrlEvent.kColocateAdjustL1:
                raise ColocateAdjustL1Exception('before_critical_section')
            self._stub.StepsNoInteruptBegin()
            if self._stub.cmd == CtrlEvent.kColocateAdjustL1:
                self._stub.StepsNoInteruptEnd()
                raise ColocateAdjustL1Exception('before_critical_section')
            try:
                yield
                if step is not None and hasattr(step, 'synchronize'):
                    step.synchronize()
            finally:
                self._stub.StepsNoInteruptEnd()
            # an adjust may have arrived during the critical section: nothing is executing now
            if _C.get_train_world_size() == 1 and self._stub.cmd == CtrlEvent.kColocateAdjustL1:
                with EventManager.record_duration_event('adjust_after_step'):
                    self.adjust()
        else:
            self._stub.StepsNoInteruptBegin()
            try:
                yield
            finally:
                self._stub.StepsNoInteruptEnd()

    def adjust(self):
        if self.train_mode == TrainMode.COLOCATE_L1:
            return self.adjust_l1()
        return self.adjust_l2()

    def adjust_l1(self):
        """Release the activation set, return empty pages to the pool, reply (colocate_ctrl.py:413-445)."""
        t0 = time.time()
        with EventManager.record_duration_event('adjust_l1'):
            released = _C.release_interm_memory(self.unpub_target_batch_size if self.keep_target_set else 0)
            t1 = time.time()
            released = max(int(released or 0), int(MemoryPool.empty_cache() or 0))
            t2 = time.time()
            self._stub.adjust_l1_done()
            t3 = time.time()
        self.adjust_log.append(((t1 - t0) * 1e3, (t2 - t1) * 1e3, (t3 - t2) * 1e3, released, t0))
        if _C._Config.log_control_stub:
            print(f'[Rank {_C.get_train_rank()} | PID {os.getpid()}] [Adjust L1 {(t1-t0)*1e3:.1f} | {(t2-t1)*1e3:.1f}'
                  f' | {(t3-t2)*1e3:.1f} ms] target batch_size: {self.target_batch_size}, released {released >> 20} MiB',
                  flush=True)

    def adjust_l2(self):
        t0 = time.time()
        with EventManager.record_duration_event('adjust_l2'):
            released = int(MemoryPool.empty_cache() or 0)
            self._stub.adjust_l2_done()
        self.adjust_log.append((0.0, (time.time() - t0) * 1e3, 0.0, released, t0))

    def report_batch_size(self, batch_size): self._stub.report_batch_size(batch_size)

    @property
    def target_batch_size(self): return self._stub.target_batch_size

    @property
    def unpub_target_batch_size(self): return self._stub.unpub_target_batch_size

    def train_end(self):
        if _C.is_enable_shared_tensor():
            MemoryPool.empty_cache()
        self._stub.train_end()

    def set_killed_batch_recover(self): self._stub.set_killed_batch_recover()
    def set_killed_batch_reconfiged(self): self._stub.set_killed_batch_reconfiged()


class DummyCtrl(CtrlBase):
    def __init__(self, train_mode, hook_mode, num_epoch, batch_size):
        super().__init__(train_mode, hook_mode, num_epoch, batch_size)
        self._stub = _C.PyDummyStub()
        assert hook_mode == ColocateCtrlHookMode.NONE

    @contextlib.contextmanager
    def steps_no_interrupt(self):
        yield

    def check_kill(self, where: str): pass
    def report_batch_size(self, batch_size): pass

    @property
    def target_batch_size(self): return self.input_batch_size

    @property
    def unpub_target_batch_size(self): return self.input_batch_size


class SwitchCtrl(CtrlBase):
    """Task-switch controller (colocate_ctrl.py:117-301): on kInterruptTrain the batch in flight is killed, the
    trainer drops its whole activation set, returns the pages and replies kInterruptTrainDone; it then waits in
    `Trainer` until kResumeTrain arrives (`PySwitchStub.prepare_resume`). taskswitch-l0 never interrupts."""

    def __init__(self, train_mode, hook_mode, num_epoch, batch_size, stub_poll_ms: int = 0):
        assert train_mode in (TrainMode.TASKSWITCH_L1, TrainMode.TASKSWITCH_L0)
        super().__init__(train_mode, hook_mode, num_epoch, batch_size)
        self._stub = _C.PySwitchStub(batch_size, poll_ms=stub_poll_ms)
        if train_mode == TrainMode.TASKSWITCH_L1:
            self._kill_event, self._kill_exception = CtrlEvent.kInterruptTrain, SwitchL1Exception
        self.switch_log = []  # (release_ms, empty_cache_ms, reply_ms, released_bytes, start time.time())

    def check_kill(self, where: str):
        """What the reference's forward/backward hooks do (colocate_ctrl.py:183-245)."""
        if self.train_mode == TrainMode.TASKSWITCH_L1 and self._stub.cmd == CtrlEvent.kInterruptTrain:
            xsched.kill_batch()
            raise SwitchL1Exception(where)

    @contextlib.contextmanager
    def steps_no_interrupt(self):
        if self.train_mode == TrainMode.TASKSWITCH_L0:
            yield
            return
        step = _C.get_train_step()
        if step is not None and hasattr(step, 'synchronize'):
            step.synchronize()  # SyncAllStreams
        if self._stub.cmd == CtrlEvent.kInterruptTrain:
            raise SwitchL1Exception('before_critical_section')
        self._stub.StepsNoInteruptBegin()
        if self._stub.cmd == CtrlEvent.kInterruptTrain:
            self._stub.StepsNoInteruptEnd()
            raise SwitchL1Exception('before_critical_section')
        try:
            yield
            if step is not None and hasattr(step, 'synchronize'):
                step.synchronize()
        finally:
            self._stub.StepsNoInteruptEnd()
        # an interrupt may have arrived during the critical section: nothing is executing now
        if _C.get_train_world_size() == 1 and self._stub.cmd == CtrlEvent.kInterruptTrain:
            self.switch(barrier=False)

    def switch(self, barrier: bool):
        if self.train_mode != TrainMode.TASKSWITCH_L1:
            raise RuntimeError(f"Unsupported train_mode: {self.train_mode.name}")
        return self.switch_l1(barrier)

    def switch_l1(self, barrier: bool):
        t0 = time.time()
        with EventManager.record_duration_event('switch_l1'):
            released = _C.release_interm_memory()
            t1 = time.time()
            released = max(int(released or 0), int(MemoryPool.empty_cache() or 0))
            t2 = time.time()
            succ = self.try_reply_interrupt(barrier)
            t3 = time.time()
        if succ:
            self.switch_log.append(((t1 - t0) * 1e3, (t2 - t1) * 1e3, (t3 - t2) * 1e3, released, t0))
        return succ

    def try_reply_interrupt(self, barrier): return self._stub.try_interrupt_train_done(barrier)

    @property
    def target_batch_size(self): return self.input_batch_size

    @property
    def unpub_target_batch_size(self): return self.input_batch_size

    def report_batch_size(self, batch_size): self._stub.report_batch_size(batch_size)

    def train_end(self):
        if _C.is_enable_shared_tensor():
            MemoryPool.empty_cache()
        self._stub.train_end()

    def set_killed_batch_recover(self): self._stub.set_killed_batch_recover()
    def set_killed_batch_reconfiged(self): pass


def create_colocate_ctrl(train_mode: TrainMode, hook_mode: ColocateCtrlHookMode, num_epoch: int, batch_size: int,
                         **kw) -> Union[DummyCtrl, ColocateCtrl]:
    if train_mode == TrainMode.NORMAL:
        return DummyCtrl(train_mode, hook_mode, num_epoch, batch_size)
    if train_mode.is_colocate():
        return ColocateCtrl(train_mode, hook_mode, num_epoch, batch_size, **kw)
    return SwitchCtrl(train_mode, hook_mode, num_epoch, batch_size, **kw)


def get_colocate_ctrl() -> Union[DummyCtrl, ColocateCtrl]:
    assert CtrlBase._colocate_ctrl is not None
    return CtrlBase._colocate_ctrl
