"""DebugServer (pytorch/torch_col/debug_server.py:6-60): plays the inference server's side of the
channel inside a test: creates the shared segment as "server", fills the information board, and
injects colocate_l1 / colocate_l2 / infer_exit commands by hand."""
from __future__ import annotations

import threading
import time
from typing import List, Optional

from ._C import CtrlEvent, PyInfTraCommunicator


class DebugServer:
    def __init__(self, train_world_size: int = 1, name: Optional[str] = None):
        self.world = train_world_size
        self.comm = PyInfTraCommunicator(is_server=True, cleanup=True, train_world_size=train_world_size, name=name)
        self.cmd_id = 1
        self.status: List = []     # (rank, PyCtrlMsgEntry) received on Tra2Inf
        self._stop = False
        self._lock = threading.Lock()
        self._thread = threading.Thread(target=self._monitor, daemon=True)
        self._thread.start()

    def _monitor(self):  # Controller::TrainMonitor (server/control/controller.cc:84-160)
        while not self._stop:
            got = self.comm.timed_get_from_any(50, 1)
            if got is not None:
                with self._lock:
                    self.status.append(got)

    def _send_adjust(self, event, batch_sizes):
        assert len(batch_sizes) == self.world
        for r, bs in enumerate(batch_sizes):
            self.comm.update_field(r, 6, bs)  # target_batch_size_unpublished, as TrainAdjuster does
        cid = self.cmd_id
        self.cmd_id += 1
        self.comm.put_all_inf2tra(event, cid, list(batch_sizes))
        return cid

    def colocate_l1(self, batch_sizes): return self._send_adjust(CtrlEvent.kColocateAdjustL1, batch_sizes)
    def colocate_l2(self, batch_sizes): return self._send_adjust(CtrlEvent.kColocateAdjustL2, batch_sizes)

    def infer_exit(self, batch_sizes):
        for r, bs in enumerate(batch_sizes):
            self.comm.update_field(r, 6, bs)
        self.comm.put_all_inf2tra(CtrlEvent.kInferExit, 0, [0] * self.world)

    def interrupt_train(self) -> int:
        """Controller::InterruptTrain (controller.cc:152-170): kInterruptTrain to every rank."""
        cid = self.cmd_id
        self.cmd_id += 1
        self.comm.put_all_inf2tra(CtrlEvent.kInterruptTrain, cid, [0] * self.world)
        return cid

    def resume_train(self) -> int:
        """Controller::ResumeTrain (controller.cc:190-206): kResumeTrain to rank 0 only."""
        cid = self.cmd_id
        self.cmd_id += 1
        self.comm.put_inf2tra(CtrlEvent.kResumeTrain, cid, 0, 0)
        return cid

    def wait_event(self, event: CtrlEvent, cmd_id: Optional[int] = None, count: int = 1, timeout_s: float = 30.0) -> float:
        """Seconds until `count` status messages of `event` (with this command id, when given) have arrived."""
        t0 = time.time()
        while time.time() - t0 < timeout_s:
            with self._lock:
                n = sum(1 for _, m in self.status if m.event == event and (cmd_id is None or m.id == cmd_id))
            if n >= count:
                return time.time() - t0
            time.sleep(0.0005)
        raise TimeoutError(f"{event.name} (id {cmd_id}) not received {count} time(s)")

    def inference_workload_done(self):
        self.comm.put_all_inf2tra(CtrlEvent.kInferenceWorkloadDone, 0, [0] * self.world)

    def wait_adjust_done(self, cmd_id: int, timeout_s: float = 30.0, ranks=None) -> float:
        """Controller::WaitColocateAdjustDone (controller.cc:377-386): seconds until every rank replied."""
        t0 = time.time()
        need = set(range(self.world) if ranks is None else ranks)
        while time.time() - t0 < timeout_s:
            with self._lock:
                done = {r for r, m in self.status
                        if m.id == cmd_id and m.event in (CtrlEvent.kColocateAdjustL1Done, CtrlEvent.kColocateAdjustL2Done)}
            if need <= done:
                return time.time() - t0
            time.sleep(0.0005)
        raise TimeoutError(f"adjust {cmd_id} not acknowledged by ranks {sorted(need - done)}")

    def events(self, event: CtrlEvent):
        with self._lock:
            return [(r, m) for r, m in self.status if m.event == event]

    def close(self):
        self._stop = True
        self._thread.join()
        self.comm.close()
