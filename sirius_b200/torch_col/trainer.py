"""Trainer (pytorch/torch_col/trainer.py:69-250): the epoch loop with the abort protocol around
`iter_train_fn`. A killed micro-batch is rolled back in the ledger, memory is released and the reply is
sent, then the remaining samples of the global batch are redistributed and the loop goes on."""
from __future__ import annotations

import time
from dataclasses import dataclass
from typing import Any, Callable, Optional

from . import _C, xsched
from ._C import _DynamicBatchDistirbutor
from .colocate_ctrl import ColocateAdjustL1Exception, EngineColocateAdjustL1Exception, SwitchL1Exception
from .util import Event, EventManager, MemoryPool


@dataclass
class TrainStat:
    killed_batch: int = 0
    finished_batch: int = 0
    tried_batch: int = 0


@dataclass
class EpochStat:
    killed_batch: int = 0
    finished_batch: int = 0
    tried_batch: int = 0
    finished_sample: int = 0
    num_rollback_batch: int = 0
    killed_time: float = 0.0
    finished_time: float = 0.0


class Trainer:
    _trainer: Optional['Trainer'] = None

    def __init__(self, model, iter_train_fn: Callable[[Any], float], ddp_allreduce: Optional[Callable[[], None]] = None):
        from .dynamic_batch import get_dynamic_dataset, get_micro_batch_manager
        Trainer._trainer = self
        self.rank = _C.get_train_rank()
        self.model = model
        self.dynamic_dataset = get_dynamic_dataset()
        self.batch_manager = get_micro_batch_manager()
        self.iter_train_fn = iter_train_fn
        self.ddp_allreduce = ddp_allreduce
        self.overall_stat = TrainStat()
        self.epoch_stats, self.epoch_events = [], []
        self._cur_epoch_stat = None
        self._last_max_batch_size_from_last_kill = None

    def train_one_epoch(self, epoch_idx: int) -> Optional[float]:
        epoch_event = EventManager.record_event(f'epoch_{epoch_idx:02d}_{self.dynamic_dataset.ds_size}')
        self._cur_epoch_stat = EpochStat()
        running_loss = 0.0
        for batch_idx, batch in enumerate(self.dynamic_dataset):
            self._cur_epoch_stat.tried_batch += 1
            self.overall_stat.tried_batch += 1
            if self._last_max_batch_size_from_last_kill is None:
                self._last_max_batch_size_from_last_kill = len(batch)
            elif len(batch) > self._last_max_batch_size_from_last_kill:
                MemoryPool.empty_cache()
                self._last_max_batch_size_from_last_kill = len(batch)
            self.batch_manager.begin_batch(epoch_idx, batch_idx, batch, batch['range'])
            try:
                loss = self.iter_train_fn(batch)
            except (ColocateAdjustL1Exception, SwitchL1Exception, EngineColocateAdjustL1Exception) as exc:
                # The reference votes "abort" only when the killed micro-batch is the syncing one; a rank
                # already waiting in the finish vote would then never learn that its peer was killed on an
                # earlier micro-batch, so here every kill in a multi-rank job casts the abort vote.
                if self._is_ddp_training():
                    self.batch_manager.vote_abort_last_micro_batch()
                self.handle_abort_batch(epoch_idx, batch_idx, batch, exc)
            else:
                if self._is_ddp_training() and batch.should_update_param():
                    if not self.batch_manager.vote_finish_last_micro_batch():
                        self.handle_abort_batch(epoch_idx, batch_idx, batch,
                                                EngineColocateAdjustL1Exception("vote finish failed"))
                        continue
                self.batch_manager.finish_batch(epoch_idx, batch_idx, batch)
                if epoch_idx == 0 and batch_idx == 0:
                    self._default_first_batch_callback()
                running_loss += float(loss or 0.0)
                self._cur_epoch_stat.finished_batch += 1
                self._cur_epoch_stat.finished_sample += self.dynamic_dataset.get_batch_size(batch)
                self.overall_stat.finished_batch += 1
        EventManager.record_event('', epoch_event)
        self._cur_epoch_stat.num_rollback_batch = self.batch_manager.num_rollback_samples
        self.epoch_stats.append(self._cur_epoch_stat)
        self.epoch_events.append(epoch_event)
        self._cur_epoch_stat = None
        return running_loss / self.dynamic_dataset.ds_size

    def get_overall_stat(self) -> TrainStat: return self.overall_stat
    def get_last_epoch_stat(self) -> Optional[EpochStat]: return self.epoch_stats[-1] if self.epoch_stats else None
    def get_last_epoch_event(self) -> Optional[Event]: return self.epoch_events[-1] if self.epoch_events else None

    def get_last_epoch_duration(self) -> Optional[float]:
        ev = self.get_last_epoch_event()
        return None if ev is None else ev.duration

    def handle_abort_batch(self, epoch_idx, batch_idx, batch, exception):
        if epoch_idx == 0 and batch_idx == 0:
            raise RuntimeError("first micro batch could not be interrupted, please increase the delay time")
        _C.dist.wait_barrier()
        xsched.kill_batch()  # the in-flight units drain; nothing of the batch is executing afterwards
        self.batch_manager.abort_batch(epoch_idx, batch_idx, batch)
        from .colocate_ctrl import SwitchCtrl
        if isinstance(self.dynamic_dataset.col_ctrl, SwitchCtrl):
            if _C.is_train_master():
                self.dynamic_dataset.col_ctrl._stub.set_global_has_batch_killed(True)
            _C.dist.wait_barrier()
        bs = self.dynamic_dataset.get_batch_size(batch)
        with EventManager.record_duration_event(f'batch_exception_{epoch_idx:02d}_{batch_idx:03d}_{bs:02d}'):
            self.dynamic_dataset.col_ctrl.release_and_reply(True)
        self._cur_epoch_stat.killed_batch += 1
        self.overall_stat.killed_batch += 1
        with EventManager.record_duration_event(f'batch_restart_{epoch_idx:02d}_{batch_idx:03d}'):
            if _C.get_train_rank() == 0:
                self.batch_manager.reset_last_micro_batch_finish_vote()
            _C.dist.wait_barrier()
            if _C.get_colocate_train_mode().is_colocate():
                self.dynamic_dataset.col_ctrl.set_killed_batch_recover()
            if _C.get_train_rank() == 0:
                _DynamicBatchDistirbutor.distribute_batch(True, True, False)
                if _C.get_colocate_train_mode().is_colocate():
                    self.dynamic_dataset.col_ctrl.set_killed_batch_reconfiged()
            _C.dist.wait_barrier()
        # task switch: the job stays off the GPU until the server sends kResumeTrain (trainer.py:243-248)
        if _C.get_colocate_train_mode().is_taskswitch():
            with EventManager.record_duration_event(f'wait_resume_{epoch_idx:02d}_{batch_idx:03d}'):
                while not self.dynamic_dataset.col_ctrl._stub.prepare_resume():
                    time.sleep(1e-3)
                _C.dist.wait_barrier()
        self._last_max_batch_size_from_last_kill = None

    def _default_first_batch_callback(self):
        """After the first finished micro-batch (trainer.py:252-266): what has been allocated so far is the model, not
        intermediates; the communication stream of the gradient exchange becomes known to the launch layer."""
        if _C.is_enable_shared_tensor():
            _C.tag_model_end()
        if _C.is_enable_xsched():
            if xsched.is_guess_nccl_begined():
                xsched.guess_nccl_end()
                nccl_streams = xsched.get_nccl_streams()
                assert len(nccl_streams) <= 1, f"nccl streams {nccl_streams}"
                if len(nccl_streams) == 1:
                    xsched.register_stream(nccl_streams[0], False)
            step = _C.get_train_step()
            if step is not None and hasattr(step, 'synchronize'):
                step.synchronize()
            xsched.initial_kill_batch(0, 0)

    def _default_first_epoch_callback(self):
        pass

    def _is_ddp_training(self):
        return _C.get_train_world_size() > 1
