"""Dynamic batching (pytorch/torch_col/dynamic_batch.py): the dataset that yields micro-batches whose
size follows the target batch size set by the inference server, and the MicroBatchManager that
finishes / aborts them in the shared ledger, scales the loss and runs the optimizer stage."""
from __future__ import annotations

import contextlib
import dataclasses
import sys
import time
from enum import Enum, IntEnum
from typing import Iterator, List, Optional, Tuple, Union

import numpy as np
import torch

from . import _C
from ._C import CtrlEvent, TrainMode, _DynamicBatchDistirbutor, _PerfModel
from .colocate_ctrl import ColocateCtrl, CtrlBase, DummyCtrl, get_colocate_ctrl
from .util import EventManager, MemoryPool

_BATCH_FINISH_TAG = 'finish'
_BATCH_CANCEL_TAG = 'cancel'


class BatchDistributePolicy(Enum):
    FIX = 'fix'
    SIMPLE = 'simple'
    BY_PERFORMANCE = 'by_performance'


def _num_sample_of_batch_range_vec(v: List[Tuple[int, int]]) -> int:
    return sum(j - i for i, j in v)


def _num_sample_of_batch_range(r) -> int:
    return _num_sample_of_batch_range_vec(r) if r and isinstance(r[0], (tuple, list)) else r[1] - r[0]


class DatasetType(IntEnum):
    VISION = 0
    TEXT_GEN = 1
    TEXT_CLS = 2
    DYNAMIC_BATCH = 3


class DatasetState(IntEnum):
    INIT = 0
    ITER = 1
    NEXT = 2


@dataclasses.dataclass
class VisionDatasetConfig:
    input_shape: tuple
    num_class: int


@dataclasses.dataclass
class TextDatasetConfig:
    seq_len: int


class Batch(dict):
    def __init__(self, inputs: Optional[dict] = None):
        super().__init__()
        for k, v in (inputs or {}).items():
            self[k] = v

    def should_update_param(self):
        return self.get('do_step', True)

    def get_range(self) -> List[Tuple[int, int]]:
        return self['range']

    def __len__(self) -> int:
        return DynamicBatchDataset._dynamic_batch_dataset.get_batch_size(self)


class MicroBatchManager:
    _micro_batch_manager: Optional['MicroBatchManager'] = None

    def __init__(self, dynamic_dataset, enable_grad_accumulate=False, checkpoint_micro_batch=False):
        assert MicroBatchManager._micro_batch_manager is None
        MicroBatchManager._micro_batch_manager = self
        self._dynamic_dataset = dynamic_dataset
        self._enable_grad_accumulate = enable_grad_accumulate
        self._checkpoint_micro_batch = checkpoint_micro_batch
        self._last_batch = None
        self._batch_event = None
        self._global_batch_event = None
        self._past_micro_batch_range_vecs_in_global_batch = []
        self._last_batch_range_vec = None
        self.num_rollback_samples = 0

    # -- loss scaling: loss /= global_bs / micro_bs, so accumulated gradients are the global mean
    def loss_scale(self, batch: Batch) -> float:
        if not self._enable_grad_accumulate:
            return 1.0
        return self._dynamic_dataset.get_batch_size(batch) / _DynamicBatchDistirbutor.get_global_batch_size()

    def scale_loss(self, batch: Batch, loss):
        if self._enable_grad_accumulate:
            loss /= _DynamicBatchDistirbutor.get_global_batch_size() / self._dynamic_dataset.get_batch_size(batch)
        return loss

    def optimizer_step(self, batch: Batch, optimizer=None, amp_scaler=None, grad_accumulator=None):
        if self._should_checkpoint_micro_batch():
            assert grad_accumulator is not None
            with get_colocate_ctrl().steps_no_interrupt():
                ev = EventManager.record_event('optimizer_step')
                grad_accumulator.accumulate()
                if batch.should_update_param():
                    grad_accumulator.step(optimizer, amp_scaler)
                    ev.tag = 'global'
                else:
                    ev.tag = 'local'
                EventManager.record_event('', ev)
        else:
            def _step():
                if hasattr(optimizer, 'optimizer_step'):   # a sirius_b200 step object
                    optimizer.optimizer_step()
                elif amp_scaler is not None:
                    amp_scaler.step(optimizer)
                    amp_scaler.update()
                    optimizer.zero_grad()
                else:
                    optimizer.step()
                    optimizer.zero_grad()
            if not self._enable_grad_accumulate or batch.should_update_param():
                with get_colocate_ctrl().steps_no_interrupt():
                    ev = EventManager.record_event('optimizer_step')
                    _step()
                    EventManager.record_event('', ev)

    @contextlib.contextmanager
    def ddp_sync_context(self, model, batch: Batch):
        if not self._enable_grad_accumulate or batch.should_update_param() or not hasattr(model, 'no_sync'):
            yield
        else:
            with model.no_sync():
                yield

    def begin_batch(self, epoch_idx, batch_idx, batch: Batch, batch_range_vec):
        self._last_batch_range_vec = batch_range_vec
        self._last_batch = batch
        self._record_batch_event(epoch_idx, batch_idx, len(batch))

    def finish_batch(self, epoch_idx, batch_idx, batch: Batch):
        step = _C.get_train_step()
        if step is not None and hasattr(step, 'synchronize'):
            step.synchronize()
        col_ctrl = get_colocate_ctrl()
        if col_ctrl.train_mode == TrainMode.COLOCATE_L2 and col_ctrl._stub.cmd == CtrlEvent.kColocateAdjustL2:
            if _C.get_train_world_size() == 1:
                col_ctrl.release_and_reply(False)
                if not batch.should_update_param():
                    _DynamicBatchDistirbutor.distribute_batch(True, True, False)
            elif batch.should_update_param():
                _C.dist.wait_barrier()
                col_ctrl.release_and_reply(False)
        self._complete_batch_event(_BATCH_FINISH_TAG, batch)
        self._past_micro_batch_range_vecs_in_global_batch.append(self._last_batch_range_vec)
        if (not self._enable_grad_accumulate or not _C.get_colocate_train_mode().is_kill_batch()
                or self._should_checkpoint_micro_batch()):
            _DynamicBatchDistirbutor.finish_batch(batch.get_range(), batch.should_update_param())
        if batch.should_update_param():
            self._next_global_batch()
        self._last_batch = None
        self._last_batch_range_vec = None
        self._dynamic_dataset._next_batch()

    def abort_batch(self, epoch_idx, batch_idx, batch: Batch):
        self._complete_batch_event(_BATCH_CANCEL_TAG, batch)
        if self._enable_grad_accumulate and not self._checkpoint_micro_batch:
            self._rollback_micro_batch()
        else:
            _DynamicBatchDistirbutor.abort_batch(self._last_batch_range_vec, batch.should_update_param())
        self._last_batch = None
        self._last_batch_range_vec = None

    def vote_finish_last_micro_batch(self) -> bool: return _DynamicBatchDistirbutor.vote_finish_last_micro_batch()
    def vote_abort_last_micro_batch(self): _DynamicBatchDistirbutor.vote_abort_last_micro_batch()
    def reset_last_micro_batch_finish_vote(self): _DynamicBatchDistirbutor.reset_last_micro_batch_finish_vote()

    def _record_batch_event(self, epoch_idx, batch_idx, batch_size):
        self._batch_event = EventManager.record_event(f'batch_{epoch_idx:02d}_{batch_idx:03d}_{batch_size:02d}')
        if self._enable_grad_accumulate and self._global_batch_event is None:
            gbs = _DynamicBatchDistirbutor.get_global_batch_size()
            self._global_batch_event = EventManager.record_event(
                f'global_batch_{epoch_idx:02d}_{batch_idx:03d}_{gbs:02d}')

    def _complete_batch_event(self, tag, batch):
        assert self._batch_event is not None
        self._batch_event.tag = tag
        EventManager.record_event('', self._batch_event)
        if _C.get_train_rank() == 0 and tag == _BATCH_FINISH_TAG:
            _PerfModel.record_thpt(len(batch), self._batch_event.duration)
        self._batch_event = None

    def _complate_global_batch_event(self, tag):
        assert self._global_batch_event is not None
        self._global_batch_event.tag = tag
        EventManager.record_event('', self._global_batch_event)
        self._global_batch_event = None

    def _should_checkpoint_micro_batch(self):
        return self._enable_grad_accumulate and self._checkpoint_micro_batch

    def _rollback_micro_batch(self):
        assert self._enable_grad_accumulate and not self._checkpoint_micro_batch
        self._complate_global_batch_event(_BATCH_CANCEL_TAG)
        for rv in self._past_micro_batch_range_vecs_in_global_batch:
            self.num_rollback_samples += _num_sample_of_batch_range_vec(rv)
            _DynamicBatchDistirbutor.abort_batch(rv, False)
        _DynamicBatchDistirbutor.abort_batch(self._last_batch_range_vec, self._last_batch.should_update_param())
        self.num_rollback_samples += _num_sample_of_batch_range_vec(self._last_batch_range_vec)
        self._past_micro_batch_range_vecs_in_global_batch = []
        self._last_batch_range_vec = None

    def _next_global_batch(self):
        if self._enable_grad_accumulate:
            self._complate_global_batch_event(_BATCH_FINISH_TAG)
        if (self._enable_grad_accumulate and _C.get_colocate_train_mode().is_kill_batch()
                and not self._checkpoint_micro_batch):
            n = len(self._past_micro_batch_range_vecs_in_global_batch)
            for i, rv in enumerate(self._past_micro_batch_range_vecs_in_global_batch):
                _DynamicBatchDistirbutor.finish_batch(rv, i == n - 1)
        self._past_micro_batch_range_vecs_in_global_batch = []
        _DynamicBatchDistirbutor.next_global_batch()


class DynamicBatchDataset(torch.utils.data.IterableDataset):
    """Holds the (pinned) host copy of the data set and yields micro-batches sized by the ledger.
    Batches are host tensors; the step object copies them to the device (srt_step_upload_batch), where
    the reference filled a fresh device tensor slice by slice (dynamic_batch.py:438-459)."""
    _dynamic_batch_dataset: Optional['DynamicBatchDataset'] = None

    def __init__(self, ds_type: DatasetType, ds_size: int, colocate_ctrl, vision_dataset_config=None,
                 text_dataset_config=None, empty_cache_at_larger_batch_size=False, fake_data=True, seed: int = 0,
                 pin_memory: Optional[bool] = None):
        assert DynamicBatchDataset._dynamic_batch_dataset is None
        DynamicBatchDataset._dynamic_batch_dataset = self
        super().__init__()
        self.ds_type, self.ds_size, self.col_ctrl = ds_type, ds_size, colocate_ctrl
        self.vision_dataset_config, self.text_dataset_config = vision_dataset_config, text_dataset_config
        self._empty_cache_at_larger_batch_size = empty_cache_at_larger_batch_size
        self._state = DatasetState.INIT
        self._last_batch = None
        if not fake_data:
            raise RuntimeError("only synthetic data is available (the reference's cifar10 files are not shipped)")
        g = torch.Generator().manual_seed(seed)
        pin = torch.cuda.is_available() if pin_memory is None else pin_memory
        if ds_type == DatasetType.VISION:
            self.all_inputs = {
                'images': torch.randn(ds_size, *vision_dataset_config.input_shape, generator=g),
                'labels': torch.randint(0, vision_dataset_config.num_class, (ds_size,), generator=g)}
        elif ds_type == DatasetType.TEXT_GEN:
            ids = torch.randint(100, 30000, (ds_size, text_dataset_config.seq_len), generator=g)
            self.all_inputs = {'input_ids': ids, 'labels': ids}
        else:
            raise RuntimeError(f"Unsupported dataset type: {ds_type}")
        if pin:
            self.all_inputs = {k: v.pin_memory() for k, v in self.all_inputs.items()}

    def get_target_batch_size(self): return self.col_ctrl.target_batch_size
    def get_next_batch_size(self): return _DynamicBatchDistirbutor.query_next_batch_size(self.get_target_batch_size())

    def get_batch_size(self, batch: Batch):
        key = 'images' if self.ds_type == DatasetType.VISION else 'input_ids'
        return len(batch[key])

    def _next_batch(self):
        assert self._state == DatasetState.ITER
        self._state = DatasetState.NEXT

    def _retrieve_batch(self, batch_range_vec) -> dict:
        batch = {}
        for k, src in self.all_inputs.items():
            parts = []
            for i, j in batch_range_vec:
                if i >= len(src):
                    l = j - i
                    i = i % len(src)
                    j = i + l
                parts.append(src[i:j])
            batch[k] = parts[0] if len(parts) == 1 else torch.cat(parts)  # one range: a view of pinned memory
        return batch

    def _wait_valid_batch_size(self):
        bs = self.get_next_batch_size()
        if self.col_ctrl.train_mode.is_colocate():
            while bs <= 0:
                _C.update_current_batch_size(bs)
                if self.col_ctrl._stub.cmd in (CtrlEvent.kColocateAdjustL1, CtrlEvent.kColocateAdjustL2):
                    self.col_ctrl.release_and_reply()
                time.sleep(1e-3)
                bs = self.get_next_batch_size()
        return bs

    def _get_batch(self) -> Batch:
        with EventManager.record_duration_event('wait_valid_batch'):
            want = self._wait_valid_batch_size()
        rng, last = _DynamicBatchDistirbutor.get_batch(want)
        batch = Batch(self._retrieve_batch(rng))
        got = self.get_batch_size(batch)
        if not _DynamicBatchDistirbutor._lazy_distributing:
            assert got == want, f"batch size mismatch: {got} != {want}"
        else:
            assert 1 <= got <= want
        batch['do_step'] = bool(last)
        batch['range'] = rng
        return batch

    def __iter__(self) -> Iterator[Batch]:
        n_global = _DynamicBatchDistirbutor.get_num_global_batch_per_epoch()
        _DynamicBatchDistirbutor.next_epoch()
        _DynamicBatchDistirbutor.next_global_batch()
        while _DynamicBatchDistirbutor.get_num_proced_global_batch() < n_global:
            batch = self._get_batch()
            bs = self.get_batch_size(batch)
            if (self._state != DatasetState.INIT and _C.is_enable_shared_tensor()
                    and self._empty_cache_at_larger_batch_size and self.get_batch_size(self._last_batch) < bs):
                MemoryPool.empty_cache()
            self._state = DatasetState.ITER
            self._last_batch = batch
            if self.col_ctrl is not None:
                self.col_ctrl.report_batch_size(bs)
                _C.update_current_batch_size(bs)
            yield batch


def init_dynamic_batch(dataset_size: int, dataset_type: DatasetType, dataset_config, batch_size: int,
                       global_batch_size: Optional[int] = None, enable_grad_accumulate: bool = False,
                       checkpoint_micro_batch: bool = False, empty_cache_at_larger_batch_size: bool = False,
                       batch_distribute_policy: BatchDistributePolicy = BatchDistributePolicy.FIX,
                       lazy_batch_distributing: bool = False, fake_data: bool = True, seed: int = 0
                       ) -> Tuple[DynamicBatchDataset, MicroBatchManager]:
    assert _C.is_configured(), "torch_col is not initialized"
    assert CtrlBase._colocate_ctrl is not None, "colocate control must be initialized before dynamic batch dataset."
    assert not (_C.get_colocate_train_mode().is_colocate() and not enable_grad_accumulate), \
        "enable grad accumulate when colocate training."
    assert not (global_batch_size is not None and not enable_grad_accumulate), \
        "enable grad accumulate when global batch size is set."
    if global_batch_size is None:
        global_batch_size = batch_size * _C.get_train_world_size()
    if not enable_grad_accumulate and checkpoint_micro_batch:
        print('torch_col: Warning: checkpoint_micro_batch needs gradient accumulation; disabled.', file=sys.stderr)
        checkpoint_micro_batch = False
    if not _C.get_colocate_train_mode().is_colocate() and batch_distribute_policy != BatchDistributePolicy.FIX:
        batch_distribute_policy = BatchDistributePolicy.FIX
    vis = dataset_config if dataset_type == DatasetType.VISION else None
    txt = dataset_config if dataset_type == DatasetType.TEXT_GEN else None
    ds = DynamicBatchDataset(dataset_type, dataset_size, CtrlBase._colocate_ctrl, vis, txt,
                             empty_cache_at_larger_batch_size, fake_data, seed)
    _C.dist.init_dynamic_batch_distributor(dataset_size, batch_size, global_batch_size, lazy_batch_distributing,
                                           batch_distribute_policy.value)
    mgr = MicroBatchManager(ds, enable_grad_accumulate, checkpoint_micro_batch)
    _C.dist.init_train_performance_model()
    return ds, mgr


def get_dynamic_dataset() -> DynamicBatchDataset:
    assert DynamicBatchDataset._dynamic_batch_dataset is not None
    return DynamicBatchDataset._dynamic_batch_dataset


def get_micro_batch_manager() -> MicroBatchManager:
    assert MicroBatchManager._micro_batch_manager is not None
    return MicroBatchManager._micro_batch_manager


def _reset_singletons():
    DynamicBatchDataset._dynamic_batch_dataset = None
    MicroBatchManager._micro_batch_manager = None
