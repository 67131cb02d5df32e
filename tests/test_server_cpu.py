"""The server side of the colocation protocol on the CPU: Controller against a trainer that speaks the protocol
by hand over the same shared-memory channel, ResourceManager and KVCachePool on a host-backend page pool, the
ColdModelCache bookkeeping, and the TrainLauncher's environment contract with a real child process.
The reference has no tests for these classes; the expectations are its code's behaviour
(server/control/controller.cc, resource_manager.cc, model_store/model_cache.cc, train_launcher.cc,
llm/kv_cache_pool.cc)."""
import ctypes as C
import os
import sys
import threading
import time
import uuid

import pytest

from sirius_b200._lib import SrtError, call
from sirius_b200._runtime import AdjusterConfig
from sirius_b200.pool import INFER, TRAIN, PagePool
from sirius_b200.server import (ColdModelCache, Controller, JobOutcome, KVCachePool, ResourceManager, ServeMode,
                                TrainLauncher, TrainStatus)
from sirius_b200.torch_col._C import CtrlEvent, PyInfTraCommunicator

MB = 1 << 20


def _name(tag): return f"srt_srv_{tag}_{os.getpid()}_{uuid.uuid4().hex[:6]}"


def _wait(pred, timeout=5.0):
    t0 = time.time()
    while not pred():
        assert time.time() - t0 < timeout, "condition never became true"
        time.sleep(0.002)


def _adjuster(srv, world, base_mb, slope_mb, balance=False):
    cfg = AdjusterConfig(base_mb, slope_mb, 0, int(balance), 1500.0, world, 1)
    h = C.c_void_p()
    call("srt_adjuster_create", srv._h, C.byref(cfg), C.byref(h))
    return h


def _register_trainers(srv, world, bs):
    for r in range(world):
        srv.set_train_info(r, train_pid=os.getpid(), train_rank=r, train_world_size=world, init_batch_size=bs,
                           current_batch_size=bs, target_batch_size=bs, target_batch_size_unpublished=bs,
                           model_name="resnet152")


def test_controller_colocate_protocol_with_two_trainer_ranks():
    nm = _name("ctl")
    srv = PyInfTraCommunicator(True, True, 2, nm)
    tra = PyInfTraCommunicator(False, False, 2, nm)
    _register_trainers(srv, 2, 32)
    adj = _adjuster(srv, 2, 1000.0, 100.0)
    ctl = Controller(srv, adj, ServeMode.COLOCATE_L1)
    try:
        assert ctl.is_train_idle()
        # nothing is sent, and nobody is waited for, while no training runs
        cid = ctl.colocate_infer_require_adjust(0, [8, 8])
        ctl.wait_colocate_adjust_done(0, cid, 100)
        assert tra.timed_get(0, 0, 0) is None
        tra.put_tra2inf(CtrlEvent.kTrainStart, 0, 0, 0)
        _wait(lambda: ctl.train_status() == TrainStatus.RUNNING)
        tra.put_tra2inf(CtrlEvent.kReportBatchSize, 0, 32, 0)
        _wait(lambda: ctl.cur_batch_size() == 32)
        # a require plan: one kColocateAdjustL1 per rank with that rank's batch size and one command id
        cid = ctl.colocate_infer_require_adjust(0, [8, 12])
        got = [tra.timed_get(1000, 0, r) for r in range(2)]
        assert [(m.event, m.id, m.value) for m in got] == [(CtrlEvent.kColocateAdjustL1, cid, 8), (CtrlEvent.kColocateAdjustL1, cid, 12)]
        assert ctl.has_flying_colocate_adjust()
        with pytest.raises(SrtError, match="not acknowledged"):
            ctl.wait_colocate_adjust_done(1, cid, 50)
        threading.Timer(0.05, lambda: [tra.put_tra2inf(CtrlEvent.kColocateAdjustL1Done, cid, 0, r) for r in range(2)]).start()
        ctl.wait_colocate_adjust_done(0, cid, 2000)
        ctl.wait_colocate_adjust_done(1, cid, 2000)
        assert not ctl.has_flying_colocate_adjust()
        # ColocateAdjust skips when no rank's unpublished target lies below its published one, sends otherwise
        assert ctl.colocate_adjust(0, 4) == 0 and tra.timed_get(0, 0, 0) is None
        srv.update_field(0, 6, 20)                       # target_batch_size_unpublished of rank 0: 32 -> 20
        cid2 = ctl.colocate_adjust(0, 4)
        m = tra.timed_get(1000, 0, 1)
        assert cid2 > cid and (m.event, m.id, m.value) == (CtrlEvent.kColocateAdjustL1, cid2, 16)
        tra.timed_get(1000, 0, 0)
        # the release plan travels as kInferExit
        cid3 = ctl.colocate_infer_release_adjust([32, 32])
        m = tra.timed_get(1000, 0, 0)
        assert (m.event, m.id, m.value) == (CtrlEvent.kInferExit, cid3, 32)
        assert tra.timed_get(1000, 0, 1).event == CtrlEvent.kInferExit
        with pytest.raises(SrtError, match="one batch size per training rank"):
            ctl.colocate_infer_require_adjust(0, [8])
        ctl.inference_workload_done()
        assert tra.timed_get(1000, 0, 1).event == CtrlEvent.kInferenceWorkloadDone
        # inference status
        ctl.set_infer_status(True)
        with pytest.raises(SrtError, match="still running"):
            ctl.wait_infer_idle(30)
        ctl.set_infer_status(False)
        ctl.wait_infer_idle(30)
        # TrainEnd: idle again, the queues are cleared, waiters are released
        tra.put_tra2inf(CtrlEvent.kTrainEnd, 0, 0, 0)
        ctl.wait_train_not_running(2000)
        assert ctl.is_train_idle()
        ctl.wait_colocate_adjust_done(0, cid3 + 10, 100)
    finally:
        ctl.close()
        call("srt_adjuster_destroy", adj)
        tra.close()
        srv.close()


def test_controller_task_switch_interrupt_and_resume():
    nm = _name("sw")
    srv = PyInfTraCommunicator(True, True, 2, nm)
    tra = PyInfTraCommunicator(False, False, 2, nm)
    ctl = Controller(srv, None, ServeMode.TASKSWITCH_L1)
    try:
        assert ctl.interrupt_train() == 0                                    # no training: nothing to interrupt
        tra.put_tra2inf(CtrlEvent.kTrainStart, 0, 0, 0)
        _wait(lambda: not ctl.is_train_idle())
        cid = ctl.interrupt_train()
        assert cid > 0 and [tra.timed_get(1000, 0, r).event for r in range(2)] == [CtrlEvent.kInterruptTrain] * 2
        assert ctl.interrupt_train() == 0                                    # not again before a resume
        threading.Timer(0.05, lambda: tra.put_tra2inf(CtrlEvent.kInterruptTrainDone, cid, 0, 0)).start()
        ctl.wait_task_switch_done(cid, 2000)
        assert ctl.train_status() == TrainStatus.INTERRUPTED
        ctl.wait_train_not_running(100)
        rid = ctl.resume_train()
        m = tra.timed_get(1000, 0, 0)                                         # rank 0 only: it releases the others
        assert (m.event, m.id) == (CtrlEvent.kResumeTrain, rid) and tra.timed_get(0, 0, 1) is None
        tra.put_tra2inf(CtrlEvent.kResumeTrainDone, rid, 0, 0)
        _wait(lambda: ctl.train_status() == TrainStatus.RUNNING)
        assert ctl.interrupt_train() > cid
        with pytest.raises(SrtError, match="dummy-adjust"):
            ctl.dummy_infer_exit(0, 8)
    finally:
        ctl.close()
        tra.close()
        srv.close()


def test_controller_task_switch_l3_kills_the_training_process(tmp_path):
    """taskswitch-l3 (server/control/controller.cc:172-182): InterruptTrain sends no message, it kills the training
    process the launcher started (SIGKILL); with no training process it does nothing. The command id is 0 either way."""
    nm = _name("l3")
    srv = PyInfTraCommunicator(True, True, 1, nm)
    ctl = Controller(srv, None, ServeMode.TASKSWITCH_L3)
    tl = TrainLauncher(ServeMode.TASKSWITCH_L3, use_xsched=False, use_shared_tensor_train=False)
    try:
        assert ctl.interrupt_train() == 0                                    # no pid known: nothing happens
        sleeper = tmp_path / "sleep.py"
        sleeper.write_text("import time\ntime.sleep(60)\n")
        pid = tl.launch(str(sleeper), "", interpreter=sys.executable)
        assert tl.wait(50) is None
        ctl.set_train_pid(pid)
        assert ctl.interrupt_train() == 0
        assert tl.wait(5000) == 128 + 9
    finally:
        tl.kill()
        ctl.close()
        srv.close()


def test_resource_manager_figures_follow_the_pool_and_the_memory_model():
    nm = _name("res")
    srv = PyInfTraCommunicator(True, True, 1, nm)
    _register_trainers(srv, 1, 16)
    adj = _adjuster(srv, 1, 8.0, 1.0)                 # 8 MB + 1 MB per sample: 24 MB predicted at batch 16
    call("srt_adjuster_load_train_info", adj)
    pool = PagePool(64 / 1024, page_mb=2, host_backend=True)
    rm = ResourceManager(pool, adj, train_memory_over_predict_mb=2.0)
    try:
        assert rm.free_memory_mb() == 64 - 0 - 24 - 2          # nothing mapped yet: the prediction counts
        a = pool.alloc(INFER, 10 * MB)
        t = pool.alloc(TRAIN, 30 * MB)
        assert rm.infer_memory_mb() == 10 and rm.train_memory_mb() == 30
        assert rm.free_memory_mb() == 64 - 10 - 30 - 2         # training holds more than predicted: its usage counts
        assert rm.train_avail_memory_mb() == 64 - 10 - 2
        pool.free(TRAIN, t)
        pool.free(INFER, a)
    finally:
        pool.close()
        call("srt_adjuster_destroy", adj)
        srv.close()


def test_cold_model_cache_reserves_evicts_and_gives_space_back():
    c = ColdModelCache(min_capacity_nbytes=100 * MB, max_capacity_nbytes=400 * MB, ratio=0.5)
    try:
        assert c.capacity_and_cache() == (100 * MB, 0)
        # half of the model may stay: groups are taken while half of the next one still fits that share
        groups, evicted, ok = c.push("a", [40 * MB, 40 * MB, 40 * MB, 40 * MB], hotness=3.0)
        assert ok and groups == [0, 1] and not evicted        # 40, +40 (60 <= 80), not +40 (100 > 80)
        assert c.capacity_and_cache() == (260 * MB, 80 * MB)   # the whole model is reserved, half of it is cached
        assert c.reserve_memory_mb() == 180 and c.releasable_memory_mb() == 0
        assert c.push("a", [1 * MB], 0.0)[2] is False          # already there
        groups, evicted, ok = c.push("b", [60 * MB, 60 * MB], hotness=1.0)
        assert ok and groups == [0] and not evicted and c.capacity_and_cache() == (380 * MB, 140 * MB)
        # over the maximum, but what is cached lies below the stable point (250 MB): nothing is evicted, the
        # capacity shrinks to what is cached (the first group of a model is always kept)
        groups, evicted, ok = c.push("c", [100 * MB, 20 * MB], hotness=2.0)
        assert ok and groups == [0] and evicted == [] and c.capacity_and_cache() == (240 * MB, 240 * MB)
        groups, evicted, ok = c.push("d", [120 * MB], hotness=5.0)
        assert ok and not evicted and c.capacity_and_cache() == (360 * MB, 360 * MB)
        # now over the maximum with 360 MB cached: the coldest models go until 250 MB are left
        groups, evicted, ok = c.push("e", [100 * MB], hotness=4.0)
        assert ok and evicted == ["b", "c"] and c.capacity_and_cache() == (300 * MB, 300 * MB)
        assert c.releasable_memory_mb() == 200
        assert c.buffer_mb(free_memory_mb=50.0) == 250 and c.buffer_mb(free_memory_mb=500.0) == 300
        # loading a cached model for inference takes its groups out of the cache and out of the capacity
        assert c.pop("d", pop_to_inference=True) == ([0], True) and c.capacity_and_cache() == (180 * MB, 180 * MB)
        assert c.pop("nope", False) == ([], False)
        assert not c.take_space(1)                             # no spare capacity
        c.set_new_capacity(260 * MB)
        assert c.take_space(50 * MB) and c.capacity_and_cache()[0] == 210 * MB
        with pytest.raises(SrtError):
            c.set_new_capacity(10 * MB)                        # below what is cached
    finally:
        c.close()


def test_train_launcher_environment_command_line_and_child(tmp_path):
    tl = TrainLauncher(ServeMode.COLOCATE_L1, use_xsched=True, use_shared_tensor_train=True, cuda_memory_pool_gb=13.5,
                       train_profile="/tmp/p.csv", dynamic_sm_partition=True, enable_train_adjust_balance=True)
    env = tl.env()
    assert env == {"COLTRAIN_USE_XSCHED": "1", "COLTRAIN_HAS_INFER_SERVER": "1", "COLTRAIN_USE_SHARED_TENSOR": "1",
                   "COLTRAIN_HAS_SHARED_TENSOR_SERVER": "1", "COLTRAIN_SHARED_TENSOR_POOL_GB": "13.5",
                   "SHARED_TENSOR_POOL_FREELIST_POLICY": "best-fit", "COLTRAIN_HOOK_MODE": "xsched-sync2",
                   "COLTRAIN_MODE": "colocate-l1", "COLTRAIN_PROFILE_LOG_PATH": "/tmp/p.csv",
                   "COLTRAIN_DYNAMIC_SM_PARTITION": "1", "COLTRAIN_BATCH_DISTRIBUTE_POLICY": "BY_PERFORMANCE"}
    plain = TrainLauncher(ServeMode.TASKSWITCH_L3, use_xsched=False, use_shared_tensor_train=False,
                          skip_set_mps_thread_percent=False, train_mps_thread_percent=40).env()
    assert plain["COLTRAIN_MODE"] == "taskswitch-l3" and plain["COLTRAIN_HOOK_MODE"] == "none"
    assert plain["COLTRAIN_USE_SHARED_TENSOR"] == "0" and plain["CUDA_MPS_ACTIVE_THREAD_PERCENTAGE"] == "40"
    assert plain["COLTRAIN_BATCH_DISTRIBUTE_POLICY"] == "FIX" and "COLTRAIN_SHARED_TENSOR_POOL_GB" not in plain
    assert tl.argv("train/resnet152.py", "batch-size=64, num-epoch=3 global-batch-size=128") == [
        "python", "train/resnet152.py", "--batch-size", "64", "--num-epoch", "3", "--global-batch-size", "128"]
    assert tl.job_batch_size == 128 or tl.job_batch_size == 64    # the last argument whose name contains "batch-size"
    # a real child: it sees the contract's variables and the parsed arguments
    script = tmp_path / "job.py"
    script.write_text("import os, sys\nprint(os.environ['COLTRAIN_MODE'], os.environ['COLTRAIN_HOOK_MODE'], "
                      "os.environ['COLTRAIN_SHARED_TENSOR_POOL_GB'], sys.argv[1:])\nsys.exit(7)\n")
    log = tmp_path / "job.log"
    pid = tl.launch(str(script), "batch-size=8", interpreter=sys.executable, log_path=str(log))
    assert pid > 0 and tl.wait(20000) == 7
    assert log.read_text().strip() == "colocate-l1 xsched-sync2 13.5 ['--batch-size', '8']"
    sleeper = tmp_path / "sleep.py"
    sleeper.write_text("import time\ntime.sleep(60)\n")
    tl.launch(str(sleeper), "", interpreter=sys.executable)
    assert tl.wait(50) is None
    tl.kill()
    assert tl.wait(5000) == 128 + 9


def test_launcher_supervises_the_job_it_started(tmp_path):
    """The tail of LaunchTrain (server/train_launcher.cc:335-381): when the job ends the controller is told that training
    has ended even if the trainer never said so; a normal exit is FINISHED, SIGKILL means "start it again", any other
    signal is a crash: the other ranks on the board are killed and the call fails with what the board knew."""
    nm = _name("sup")
    srv = PyInfTraCommunicator(True, True, 2, nm)
    tra = PyInfTraCommunicator(False, False, 2, nm)
    ctl = Controller(srv, None, ServeMode.TASKSWITCH_L3)
    tl = TrainLauncher(ServeMode.TASKSWITCH_L3, use_xsched=False, use_shared_tensor_train=False)
    sleeper = tmp_path / "sleep.py"
    sleeper.write_text("import time\ntime.sleep(60)\n")
    quick = tmp_path / "quick.py"
    quick.write_text("import sys\nsys.exit(3)\n")
    crash = tmp_path / "crash.py"
    crash.write_text("import os, signal, time\ntime.sleep(0.3)\nos.kill(os.getpid(), signal.SIGTERM)\ntime.sleep(60)\n")
    other = None
    try:
        # 1. a job that exits by itself, having announced its start but not its end
        tl.launch(str(quick), "", interpreter=sys.executable)
        tra.put_tra2inf(CtrlEvent.kTrainStart, 0, 0, 0)
        _wait(lambda: not ctl.is_train_idle())
        assert tl.supervise(ctl, srv, 20000) == (JobOutcome.FINISHED, 3)
        _wait(ctl.is_train_idle)
        # 2. task-switch l3: the interrupt kills the job, supervision says "launch it again"
        pid = tl.launch(str(sleeper), "", interpreter=sys.executable)
        ctl.set_train_pid(pid)
        tra.put_tra2inf(CtrlEvent.kTrainStart, 0, 0, 0)
        _wait(lambda: not ctl.is_train_idle())
        assert tl.supervise(ctl, srv, 50) == (JobOutcome.RUNNING, None)
        ctl.interrupt_train()
        assert tl.supervise(ctl, srv, 20000) == (JobOutcome.KILLED, 128 + 9)
        _wait(ctl.is_train_idle)
        assert ctl.interrupt_train() == 0                      # the pid is forgotten: nothing left to kill
        # 3. a crash (SIGTERM) of rank 0 takes the other rank on the board with it
        other = TrainLauncher(ServeMode.TASKSWITCH_L3, use_xsched=False, use_shared_tensor_train=False)
        other.launch(str(sleeper), "", interpreter=sys.executable)
        pid0 = tl.launch(str(crash), "", interpreter=sys.executable)
        for r, p in enumerate((pid0, other.pid)):
            srv.set_train_info(r, train_pid=p, train_rank=r, train_world_size=2, init_batch_size=64, current_batch_size=48,
                               target_batch_size=48, target_batch_size_unpublished=40, model_name="resnet152")
        with pytest.raises(SrtError, match="signal is Terminated.*current 48, target 48, unpublished 40.*1 other rank"):
            tl.supervise(ctl, srv, 20000)
        assert other.wait(5000) == 128 + 9
        # KillTrain on a board without a job does nothing
        call("srt_comm_invalidate_train_info", srv._h, 0)
        assert TrainLauncher.kill_train(srv) == 0
    finally:
        tl.kill()
        if other is not None:
            other.kill()
        ctl.close()
        tra.close()
        srv.close()


def test_dummy_adjust_injects_shrink_and_grow_rounds_while_training_runs():
    """DummyAdjust (server/train_launcher.cc:383-408): every round is a ColocateAdjust by one sample (sent when a plan
    of the adjuster is still unpublished, skipped otherwise, as Controller::ColocateAdjust decides), a wait for Done and
    a kInferExit with the original batch size; the rounds end when training does."""
    nm = _name("dum")
    srv = PyInfTraCommunicator(True, True, 1, nm)
    tra = PyInfTraCommunicator(False, False, 1, nm)
    _register_trainers(srv, 1, 32)
    call("srt_comm_update_train_field", srv._h, 0, 6, 31)          # an unpublished plan: target 32 -> 31
    ctl = Controller(srv, None, ServeMode.COLOCATE_L1, dummy_adjust=True)
    seen, stop = [], threading.Event()

    def trainer():
        tra.put_tra2inf(CtrlEvent.kTrainStart, 0, 0, 0)
        while not stop.is_set():
            m = tra.timed_get(20, 0, 0)
            if m is None:
                continue
            seen.append((int(m.event), m.value))
            if m.event == CtrlEvent.kColocateAdjustL1:
                tra.put_tra2inf(CtrlEvent.kColocateAdjustL1Done, m.id, 0, 0)
            if len([e for e in seen if e[0] == CtrlEvent.kInferExit]) >= 3:
                tra.put_tra2inf(CtrlEvent.kTrainEnd, 0, 0, 0)
                return

    th = threading.Thread(target=trainer)
    th.start()
    try:
        _wait(lambda: not ctl.is_train_idle())
        rounds = TrainLauncher.dummy_adjust(ctl, 32, delay_ms=0, duration_ms=20000, seed=42, min_gap_ms=5, max_gap_ms=15)
        th.join(10)
        assert rounds >= 3 and ctl.is_train_idle()
        adjusts = [v for e, v in seen if e == CtrlEvent.kColocateAdjustL1]
        exits = [v for e, v in seen if e == CtrlEvent.kInferExit]
        assert adjusts[:3] == [30, 30, 30] and exits[:3] == [32, 32, 32]
        assert [e for e, _ in seen[:4]] == [CtrlEvent.kColocateAdjustL1, CtrlEvent.kInferExit] * 2   # Done awaited in between
        plain = Controller(srv, None, ServeMode.COLOCATE_L1)
        with pytest.raises(SrtError, match="dummy_adjust"):
            TrainLauncher.dummy_adjust(plain, 32, delay_ms=0, duration_ms=10)
        plain.close()
    finally:
        stop.set()
        th.join(5)
        ctl.close()
        tra.close()
        srv.close()


def test_kv_cache_pool_trades_pages_with_a_trainer():
    """A 64 MiB pool, a trainer holding 44 MiB of it at batch 16 (12 MiB + 2 MiB per sample), an LLM server whose
    KV-cache pages are 8 MiB: the first pages fit beside training; the next request does not, so training is asked
    to shrink (LLM require plan -> kColocateAdjustL1 -> Done) before the pages are mapped; when the server frees
    its pages and enough of the pool is free, training is told it may grow again (kInferExit)."""
    nm = _name("kv")
    srv = PyInfTraCommunicator(True, True, 1, nm)
    tra = PyInfTraCommunicator(False, False, 1, nm)
    _register_trainers(srv, 1, 16)
    adj = _adjuster(srv, 1, 12.0, 2.0)
    pool = PagePool(64 / 1024, page_mb=2, host_backend=True)
    ctl = Controller(srv, adj, ServeMode.COLOCATE_L1)
    kv = KVCachePool(pool, ctl, adj, min_adjust_nbytes=8 * MB, reclaim_free_nbytes=32 * MB, reclaim_margin_nbytes=2 * MB,
                     adjust_timeout_ms=5000)
    held = {"blocks": [pool.alloc(TRAIN, 2 * MB) for _ in range(22)]}     # 44 MiB = 12 + 2 * 16
    seen = []

    def trainer():
        while True:
            m = tra.timed_get(50, 0, 0)
            if m is None:
                if stop.is_set():
                    return
                continue
            seen.append((m.event, m.value))
            if m.event == CtrlEvent.kColocateAdjustL1:                     # shrink to the new batch size, then reply
                keep = (12 + 2 * m.value) // 2
                for b in held["blocks"][keep:]:
                    pool.free(TRAIN, b)
                held["blocks"] = held["blocks"][:keep]
                pool.empty_cache(TRAIN)
                srv.update_field(0, 5, m.value)                            # publish the target
                tra.put_tra2inf(CtrlEvent.kColocateAdjustL1Done, m.id, 0, 0)

    stop = threading.Event()
    th = threading.Thread(target=trainer)
    try:
        kv.set_block_shape(block_size=16, num_layers=4, num_heads=2, head_size=64, block_nbytes=1 * MB)
        assert kv.num_gpu_blocks() == 64 and kv.layer_block_info() == (256, 0)
        assert kv.shape_and_stride() == ([2, 256, 2048], [2048, 4096, 1])
        kv.update_num_free_layer_blocks_by_train_base(12 * MB)
        assert kv.layer_block_info() == (52 * 4, 0)
        kv.update_num_free_layer_blocks(-8)
        assert kv.layer_block_info() == (200, 8)
        tra.put_tra2inf(CtrlEvent.kTrainStart, 0, 0, 0)
        _wait(lambda: not ctl.is_train_idle())
        th.start()
        pages, adjusted = kv.alloc_pages(8 * MB, 2)                         # 16 of the 20 free MiB
        assert len(pages) == 2 and not adjusted and pool.stat("infer_usage") == 16 * MB
        C.memset(pages[1], 0x11, 8 * MB)
        assert kv.util() == pytest.approx(8 * 1 * MB / 4 / (16 * MB))
        more, adjusted = kv.alloc_pages(8 * MB, 2)                          # 16 more: only 4 are free
        assert adjusted and len(more) == 2 and pool.stat("infer_usage") == 32 * MB
        ev, new_bs = seen[0]
        assert ev == CtrlEvent.kColocateAdjustL1 and new_bs < 16
        assert pool.stat("train_all") == (12 + 2 * new_bs) * MB
        # give everything back: with 32 MiB or more free training may grow, up to what the free memory allows
        assert kv.free_pages(pages + more) is True and pool.stat("infer_usage") == 0
        _wait(lambda: len(seen) == 2)
        ev, grown = seen[1]
        assert ev == CtrlEvent.kInferExit and new_bs < grown <= 16
        with pytest.raises(SrtError, match="not a KV-cache page"):
            kv.free_pages([12345])
    finally:
        stop.set()
        if th.is_alive():
            th.join(5)
        kv.close()
        ctl.close()
        for b in held["blocks"]:
            pool.free(TRAIN, b)
        pool.close()
        call("srt_adjuster_destroy", adj)
        tra.close()
        srv.close()


def test_the_colocation_trainer_understands_the_command_line_the_launcher_builds():
    """The two-process colocation experiment starts its trainer through TrainLauncher: the "key=value" argument string
    the server side writes must expand (server/train_launcher.cc:213-238: "--key value", a bare key is a flag) into
    what the trainer's own parser accepts, with and without the SM partition."""
    from sirius_b200.colocate_proc import make_parser
    from sirius_b200.server import ServeMode, TrainLauncher
    launcher = TrainLauncher(ServeMode.COLOCATE_L1)
    for extra, flag in (("", False), (" no-sm-partition", True)):
        argv = launcher.argv("/tmp/train.py", "role=trainer batch=64 result=/tmp/r.json max-seconds=150.0" + extra)
        assert argv[:2] == ["python", "/tmp/train.py"]
        a = make_parser().parse_args(argv[2:])
        assert (a.role, a.batch, a.result, a.max_seconds, a.no_sm_partition) == ("trainer", 64, "/tmp/r.json", 150.0, flag)
