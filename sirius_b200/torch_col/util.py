"""torch_col.util: logging helpers, MemoryPool statistics, the EventManager trace
(pytorch/torch_col/util.py:18-190). The CSV schema (timestamp, name, loc, duration, tag, rank) and the
event names are the reference's, so its log parsers apply unchanged."""
from __future__ import annotations

import contextlib
import inspect
from dataclasses import dataclass
from typing import Optional

from . import _C
from ._C import TrainMode  # noqa: F401


def _fmt(args):
    return args[0] if len(args) == 1 and isinstance(args[0], str) else ' '.join(f'{a}' for a in args)


def info(*args): _C.CallGLOG_INFO(_fmt(args), 'torch_col', 0)


def info_with_frame(*args):
    c = inspect.getframeinfo(inspect.stack()[1][0])
    _C.CallGLOG_INFO(_fmt(args), c.filename, c.lineno)


def dinfo(*args):
    c = inspect.getframeinfo(inspect.stack()[1][0])
    _C.CallGLOG_DINFO(_fmt(args), c.filename, c.lineno)


class MemoryPool:
    """GB figures of the training side of the page pool (util.py:64-97)."""
    @classmethod
    def get_memory_usage(cls): return _C.cuda_memory_pool_train_all_usage(_C.get_train_rank()) / 2 ** 30

    @classmethod
    def get_memory_peak_usage(cls): return _C.cuda_memory_pool_train_peak_usage(_C.get_train_rank()) / 2 ** 30

    @classmethod
    def get_allocated_memory(cls): return _C.cuda_memory_pool_train_usage(_C.get_train_rank()) / 2 ** 30

    @classmethod
    def empty_cache(cls): return _C.cuda_memory_pool_free_train_local(_C.get_train_rank())


@dataclass
class Event:
    timestamp: int
    name: str
    loc: str
    duration: float
    tag: str

    def __str__(self): return f'{self.timestamp} {self.loc} {self.name} {self.duration} {self.tag}'


class EventManager:
    _event_list: list = []
    _default_event_log_path = 'train-profile.csv'

    @classmethod
    def reset(cls): cls._event_list = []

    @classmethod
    def record_event(cls, name: str, prev_event: Optional[Event] = None, record_loc: bool = False):
        ts = _C.get_unix_timestamp_us()
        loc = 'none'
        if record_loc:
            c = inspect.getframeinfo(inspect.stack()[1][0])
            loc = f'{c.filename}:{c.lineno}'
        if prev_event is not None:
            prev_event.duration = (ts - prev_event.timestamp) / 1000
        if len(name) > 0:
            ev = Event(ts, name, loc, 0, '')
            cls._event_list.append(ev)
            return ev

    @classmethod
    @contextlib.contextmanager
    def record_duration_event(cls, name: str):
        ts = _C.get_unix_timestamp_us()
        ev = Event(ts, name, 'none', 0, '')
        cls._event_list.append(ev)
        yield
        ev.duration = (_C.get_unix_timestamp_us() - ts) / 1000

    @classmethod
    def to_csv(cls, header=True, train_mode: Optional[TrainMode] = None) -> str:
        events = list(cls._event_list)
        if train_mode is not None and train_mode.is_colocate():
            events += [Event(ts, 'recv_adjust', 'none', 0, '') for ts in _C.get_adjust_request_time_stamp()]
            events += [Event(ts, 'adjust_done', 'none', 0, '') for ts in _C.get_adjust_done_time_stamp()]
        lines = ['timestamp,name,loc,duration,tag,rank'] if header else []
        for e in events:
            lines.append(f'{e.timestamp / 1000:.2f},{e.name},{e.loc},{e.duration:.2f},{e.tag},{_C.get_train_rank()}')
        return '\n'.join(lines)

    @classmethod
    def dump(cls, path: Optional[str] = None, train_mode: Optional[TrainMode] = None):
        if path is None:
            path = _C.get_train_profile_log_path() or cls._default_event_log_path
        if _C.get_train_rank() == 0:
            text = cls.to_csv(True, train_mode) + '\n'
            for i in range(1, _C.get_train_world_size()):
                text += _C.dist.recv_msg(i) + '\n'
            with open(path, 'w') as f:
                f.write(text)
        else:
            _C.dist.send_msg(0, cls.to_csv(False, train_mode))
        _C.dist.wait_barrier()


def initialize_sgd_optimizer(model, optimizer):
    """util.py:182-190: pre-allocate gradients and momentum buffers so the first step allocates nothing.
    The step object keeps both in its flat buffers from construction; for torch modules do as the reference."""
    import torch
    if not isinstance(model, torch.nn.Module):
        return
    for p in model.parameters():
        if p.requires_grad:
            p.grad = torch.zeros_like(p)
    for g in optimizer.param_groups:
        for p in g['params']:
            optimizer.state[p]['momentum_buffer'] = torch.zeros_like(p)
