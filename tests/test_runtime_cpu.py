"""CPU suite of the host-side runtime: the shared-memory channel, SM-partition arithmetic, ledger,
performance model, train adjuster and page pool, through the C ABI, against the Python restatement
of the reference's logic (oracle/control_oracle.py)."""
import ctypes as C
import multiprocessing as mp
import os
import random
import time
import uuid

import pytest

from oracle import control_oracle as O
from sirius_b200 import _lib, _runtime  # noqa: F401
from sirius_b200._lib import call, SrtError
from sirius_b200._runtime import AdjusterConfig, CtrlMsg, PoolConfig, TrainInfo
from sirius_b200.torch_col import _C as TC
from sirius_b200.torch_col._C import CtrlEvent, PyInfTraCommunicator


def _name(tag):
    return f"srt_test_{tag}_{os.getpid()}_{uuid.uuid4().hex[:8]}"


# ---------------------------------------------------------------- inf_tra_comm
def test_comm_queues_and_info_board():
    nm = _name("comm")
    srv = PyInfTraCommunicator(True, True, 2, nm)
    cli = PyInfTraCommunicator(False, False, 2, nm)
    try:
        assert cli.timed_get(0, 0, 0) is None                       # TryGet on an empty queue
        t0 = time.time()
        assert cli.timed_get(50, 0, 1) is None                      # TimedGet times out
        assert 0.04 < time.time() - t0 < 1.0
        srv.put_all_inf2tra(CtrlEvent.kColocateAdjustL1, 7, [12, 34])  # PutAll, one message per rank
        a, b = cli.timed_get(100, 0, 0), cli.timed_get(100, 0, 1)
        assert (a.id, a.event, a.value) == (7, CtrlEvent.kColocateAdjustL1, 12)
        assert (b.id, b.event, b.value) == (7, CtrlEvent.kColocateAdjustL1, 34)
        for i in range(5):                                          # FIFO per queue
            cli.put_tra2inf(CtrlEvent.kReportBatchSize, 0, i, 1)
        got = [srv.timed_get_from_any(100, 1) for _ in range(5)]
        assert [m.value for r, m in got] == list(range(5)) and all(r == 1 for r, _ in got)
        assert srv.timed_get_from_any(20, 1) is None
        # information board
        cli.set_train_info(0, train_pid=os.getpid(), train_rank=0, train_world_size=2, init_batch_size=64,
                           current_batch_size=64, target_batch_size=64, target_batch_size_unpublished=64,
                           model_name="resnet152")
        ti = srv.get_train_info(0)
        assert ti.model_name == b"resnet152" and ti.init_batch_size == 64
        srv.update_field(0, 6, 40)
        assert cli.get_field(0, 6) == 40 and cli.get_field(0, 5) == 64
        with pytest.raises(SrtError):                               # rank 1 never registered: invalid
            cli.get_field(1, 5)
        # TPC counters shared with the SM partitioner
        assert srv.infer_tpc(0, 1, 27) == 27 and srv.infer_tpc(0, 1, 6) == 33
        assert cli.infer_tpc(0, 2, 27) == 6 and cli.infer_tpc(0, 3) == 6
    finally:
        cli.close()
        srv.close()


def test_comm_open_without_server_fails_quickly():
    with pytest.raises(SrtError):
        PyInfTraCommunicator(False, False, 1, _name("absent"), timeout_ms=100)


def _blocking_getter(nm, q):
    c = PyInfTraCommunicator(False, False, 1, nm)
    m = c.timed_get(5000, 0, 0)
    q.put((m.id, int(m.event), m.value))
    c.close()


def test_comm_wakes_a_blocked_getter_in_another_process():
    nm = _name("comm2")
    srv = PyInfTraCommunicator(True, True, 1, nm)
    q = mp.get_context("spawn").Queue()
    p = mp.get_context("spawn").Process(target=_blocking_getter, args=(nm, q))
    p.start()
    time.sleep(0.3)
    srv.put_inf2tra(CtrlEvent.kInferExit, 3, 9, 0)
    assert q.get(timeout=10) == (3, int(CtrlEvent.kInferExit), 9)
    p.join(10)
    srv.close()


# ---------------------------------------------------------------- SM partition
def test_sm_partition_mask_matches_reference_arithmetic():
    lib = _lib.lib()
    rnd = random.Random(0)
    for _ in range(2000):
        gpu_tpc = rnd.choice([40, 54, 66, 74])
        mn, mx = rnd.randint(1, 8), rnd.choice([gpu_tpc, gpu_tpc - 3, 200])
        req = rnd.randint(0, 100)
        want = O.train_avail_tpc_mask(req, gpu_tpc, mn, mx) & (2 ** 64 - 1)
        if O.train_avail_tpc_mask(req, gpu_tpc, mn, mx) >= 2 ** 64:
            want = 2 ** 64 - 1
        assert lib.srt_smp_train_avail_tpc_mask(req, gpu_tpc, mn, mx) == want
        assert lib.srt_smp_train_avail_tpc_num(req, gpu_tpc, mn, mx) == O.train_avail_tpc_num(req, gpu_tpc, mn, mx)
    # wide mask on a 148-SM part: 27 TPCs requested -> SMs 0..53 leave training, 54..147 stay
    m = (C.c_uint64 * 3)()
    call("srt_smp_allowed_sm_mask", 27, 148, 5, 74, m)
    bits = [(m[i >> 6] >> (i & 63)) & 1 for i in range(192)]
    assert sum(bits) == 148 - 54 and bits[53] == 0 and bits[54] == 1 and bits[147] == 1 and bits[148] == 0


# ---------------------------------------------------------------- ledger, single rank
@pytest.fixture
def dist1():
    TC._Config.has_infer_server = False
    os.environ["SIRIUS_B200_DIST_NAME"] = _name("dist")
    os.environ.pop("COLTRAIN_HAS_INFER_SERVER", None)
    TC.torch_col_init(0, 1)
    yield TC.dist
    TC.torch_col_shutdown()


def test_ledger_single_rank_global_batches(dist1):
    D = TC._DynamicBatchDistirbutor
    dist1.init_dynamic_batch_distributor(100, 16, 40, False, "fix")
    assert D.get_global_batch_size() == 40 and D.get_num_global_batch_per_epoch() == 3
    assert D.next_epoch() == 0
    seen = []
    for gb, size in enumerate([40, 40, 20]):                  # last global batch is the remainder
        D.next_global_batch()
        assert D._info(3) == size and D._info(6, 0) == size
        done = 0
        while True:
            want = D.query_next_batch_size(16)
            rng, last = D.get_batch(want)
            n = sum(j - i for i, j in rng)
            assert n == want == min(16, size - done)
            if gb == 0 and done == 16:                        # abort once: samples go back, come again
                D.abort_batch(rng, last)
                assert D._info(3) == size - done and D._info(4) == 0
                rng2, last2 = D.get_batch(want)
                assert rng2 == rng and last2 == last
            done += n
            seen += rng
            D.finish_batch(rng, last)
            if last:
                break
        assert done == size and D._info(5) == size and D.get_num_proced_global_batch() == gb + 1
    covered = sorted(seen)
    assert covered[0][0] == 0 and covered[-1][1] == 100
    assert all(a[1] == b[0] for a, b in zip(covered, covered[1:]))   # every sample exactly once
    with pytest.raises(SrtError):
        D.finish_batch([(0, 5)], False)                                 # not in the processing set
    assert D.next_epoch() == 1


def test_perf_model_matches_reference_interpolation(dist1):
    P = TC._PerfModel
    ref = O.PerfModel()
    assert P.get_thpt(8) == -1 and P.get_thpt(0) == 0
    rnd = random.Random(1)
    for _ in range(200):
        bs, ms = rnd.choice([4, 8, 16, 24, 32, 64]), rnd.uniform(5, 80)
        P.record_thpt(bs, ms)
        ref.record(bs, ms)
    for bs in range(-2, 100):
        assert P.get_thpt(bs) == pytest.approx(ref.get(bs), rel=1e-12, abs=1e-12)


# ---------------------------------------------------------------- ledger, two ranks
def _ledger_worker(rank, dist_name, policy, q):
    os.environ["SIRIUS_B200_DIST_NAME"] = dist_name
    TC.torch_col_init(rank, 2)
    D = TC._DynamicBatchDistirbutor
    TC.dist.init_dynamic_batch_distributor(64, 8, 32, False, policy)
    if rank == 0 and policy == "by_performance":
        TC._PerfModel.record_thpt(8, 10.0)
    TC.dist.wait_barrier()
    D.next_epoch()
    mine, votes = [], []
    for gb in range(2):
        D.next_global_batch()
        share = D._info(6, rank)
        while True:
            rng, last = D.get_batch(D.query_next_batch_size(8))
            mine += rng
            if last:
                votes.append(D.vote_finish_last_micro_batch())
            D.finish_batch(rng, last)
            if last:
                break
    TC.dist.wait_barrier()
    if rank == 1:
        TC.dist.send_msg(0, "hello from rank 1 " * 2000)          # longer than one mailbox slot
    else:
        assert TC.dist.recv_msg(1) == "hello from rank 1 " * 2000
    q.put((rank, mine, votes, share))
    TC.dist.wait_barrier()
    TC.torch_col_shutdown()


@pytest.mark.parametrize("policy", ["simple", "by_performance"])
def test_ledger_two_ranks_split_every_global_batch(policy):
    ctx = mp.get_context("spawn")
    q, nm = ctx.Queue(), _name("dist2")
    ps = [ctx.Process(target=_ledger_worker, args=(r, nm, policy, q)) for r in range(2)]
    for p in ps:
        p.start()
    out = sorted(q.get(timeout=60) for _ in range(2))
    for p in ps:
        p.join(30)
        assert p.exitcode == 0
    ranges = sorted(out[0][1] + out[1][1])
    assert ranges[0][0] == 0 and ranges[-1][1] == 64
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    assert all(all(v) for _, _, v, _ in out)                          # both ranks voted "finish" each time
    assert out[0][3] + out[1][3] == 32                                # shares of a global batch add up


def _tail_worker(rank, world, dist_name, policy, q):
    os.environ["SIRIUS_B200_DIST_NAME"] = dist_name
    TC.torch_col_init(rank, world)
    D = TC._DynamicBatchDistirbutor
    TC.dist.init_dynamic_batch_distributor(34, 8, 32, False, policy)     # second global batch: 2 samples for 4 ranks
    if rank == 0:
        TC._PerfModel.record_thpt(8, 10.0)
    TC.dist.wait_barrier()
    D.next_epoch()
    mine, shares = [], []
    for gb in range(2):
        D.next_global_batch()
        shares.append(D._info(6, rank))
        while True:
            rng, last = D.get_batch(D.query_next_batch_size(8))
            mine += rng
            if last:
                D.vote_finish_last_micro_batch()
            D.finish_batch(rng, last)
            if last:
                break
    q.put((rank, mine, shares))
    TC.dist.wait_barrier()
    TC.torch_col_shutdown()


@pytest.mark.parametrize("policy", ["simple", "by_performance"])
def test_fewer_samples_than_ranks_at_the_tail_of_an_epoch(policy):
    """34 samples, global batch 32, four ranks: the last global batch has two samples. Two ranks get one each,
    the other two get none, the shares add up to what the ledger holds (throughput-proportional splitting used to
    hand every rank at least one sample and over-commit the ledger), and every sample is trained once."""
    ctx = mp.get_context("spawn")
    q, nm = ctx.Queue(), _name("tail")
    ps = [ctx.Process(target=_tail_worker, args=(r, 4, nm, policy, q)) for r in range(4)]
    for p in ps:
        p.start()
    out = sorted(q.get(timeout=90) for _ in range(4))
    for p in ps:
        p.join(30)
        assert p.exitcode == 0
    assert sum(o[2][0] for o in out) == 32 and sum(o[2][1] for o in out) == 2
    assert sorted(o[2][1] for o in out) == [0, 0, 1, 1]
    ranges = sorted(r for o in out for r in o[1] if r[1] > r[0])
    assert ranges[0][0] == 0 and ranges[-1][1] == 34 and all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))


def _ledger_ranks(world, ds, bs, gbs, lazy, policy):
    """`world` handles on one segment, opened and initialised from one thread per rank (the lazy mode's init and every
    NextGlobalBatch meet at the job's barrier)."""
    import threading
    name = _name("led")
    hs = [C.c_void_p() for _ in range(world)]
    call("srt_dist_open", name.encode(), 0, world, 5000, C.byref(hs[0]))
    for r in range(1, world):
        call("srt_dist_open", name.encode(), r, world, 5000, C.byref(hs[r]))

    def together(fn):
        errs = []

        def run(r):
            try:
                fn(r)
            except BaseException as e:  # noqa: BLE001
                errs.append(repr(e))
        ts = [threading.Thread(target=run, args=(r,)) for r in range(world)]
        for t in ts:
            t.start()
        for t in ts:
            t.join(30)
        assert not errs, errs

    together(lambda r: call("srt_dbd_init", hs[r], ds, bs, gbs, int(lazy), {"fix": 0, "simple": 1, "by_performance": 2}[policy]))
    return hs, together


def _ledger_info(h, which, rank=0):
    v = C.c_int()
    call("srt_dbd_info", h, which, rank, C.byref(v))
    return v.value


@pytest.mark.parametrize("world,lazy,policy", [(1, False, "fix"), (1, True, "simple"), (2, False, "fix"), (2, False, "simple"),
                                               (2, False, "by_performance"), (3, False, "by_performance"), (2, True, "simple")])
def test_ledger_follows_the_restated_reference_on_random_schedules(world, lazy, policy):
    """Random micro-batch sizes, aborts and finishes over several global batches and two epochs, on `world` ranks of one
    job: every range handed out, every last-micro-batch flag and every counter equal those of the restated
    DynamicBatchDistirbutor (oracle/control_oracle.py: Ledger), whose assertions are the reference's CHECKs."""
    ds, bs, gbs = 150, 16, 64                                   # the last global batch of an epoch is a remainder of 22
    hs, together = _ledger_ranks(world, ds, bs, gbs, lazy, policy)
    ref = O.Ledger(world, ds, bs, gbs, lazy, policy)
    rnd = random.Random(int(os.environ.get("SRT_LEDGER_SEED", "0")) + 100 * world + 10 * int(lazy) + len(policy))

    def same_counters():
        assert [_ledger_info(hs[0], w) for w in (3, 4, 5)] == [ref.n_unproc, ref.n_procing, ref.n_proced]
        for r in range(world):
            assert [_ledger_info(hs[0], w, r) for w in (6, 7, 8)] == [ref.unproc_per[r], ref.procing_per[r], ref.proced_per[r]]

    def get(r, want):
        buf, n, last = (C.c_int * 128)(), C.c_int(), C.c_int()
        q = C.c_int()
        call("srt_dbd_query_next_batch_size", hs[r], want, C.byref(q))
        assert q.value == ref.query_next_batch_size(r, want)
        call("srt_dbd_get_batch", hs[r], want, buf, 64, C.byref(n), C.byref(last))
        got = [(buf[2 * i], buf[2 * i + 1]) for i in range(n.value)]
        exp, exp_last = ref.get_batch(r, want)
        assert (got, bool(last.value)) == (exp, bool(exp_last)), (r, want)
        return got, bool(last.value)

    def flat(ranges):
        arr = (C.c_int * (2 * max(len(ranges), 1)))()
        for i, (a, b) in enumerate(ranges):
            arr[2 * i], arr[2 * i + 1] = a, b
        return arr

    try:
        for epoch in range(2):
            for r in range(world):
                e = C.c_int()
                call("srt_dbd_next_epoch", hs[r], C.byref(e))
                assert e.value == ref.next_epoch(r) == epoch
            for gb in range(ref.num_gb_per_epoch):
                together(lambda r: call("srt_dbd_next_global_batch", hs[r], None, 10000))
                ref.next_global_batch()
                same_counters()
                # A rank holds its last micro-batch until every rank has one (the finish vote); a kill anywhere makes
                # every rank that waits in the vote give its last micro-batch back too, then rank 0 hands the
                # remainder out again (Trainer.handle_abort_batch).
                pending, kills = {}, 0

                def abort(r, ranges, last):
                    call("srt_dbd_abort_batch", hs[r], flat(ranges), len(ranges), int(last))
                    ref.abort_batch(r, ranges)

                def kill_all(first=None):
                    if first is not None:
                        abort(*first)
                    for q, rg in pending.items():
                        abort(q, rg, True)
                    pending.clear()
                    call("srt_dbd_distribute_batch", hs[0], None, 1, 1, 0)
                    ref.distribute(True, True, False)
                    same_counters()

                while True:
                    free = [i for i in range(world) if i not in pending]
                    if not free:
                        if kills < 2 and rnd.random() < 0.3:
                            kills += 1
                            kill_all()
                            continue
                        for q, rg in pending.items():
                            call("srt_dbd_finish_batch", hs[q], flat(rg), len(rg), 1)
                            ref.finish_batch(q, rg, True)
                        same_counters()
                        break
                    r = rnd.choice(free)
                    ranges, last = get(r, rnd.choice([1, 3, 7, 16, 40]))
                    same_counters()
                    if kills < 4 and ranges and rnd.random() < 0.2:
                        kills += 1
                        kill_all((r, ranges, last))
                    elif last:
                        pending[r] = ranges
                    else:
                        call("srt_dbd_finish_batch", hs[r], flat(ranges), len(ranges), 0)
                        ref.finish_batch(r, ranges, False)
                        same_counters()
                assert ref.n_unproc == 0 and ref.n_procing == 0
                assert [_ledger_info(hs[r], 2) for r in range(world)] == ref.num_proced_gb
    finally:
        for h in hs:
            call("srt_dist_close", h)


def test_ledger_splits_by_measured_throughput_at_each_ranks_target_batch_size():
    """BY_PERFORMANCE with a colocated server: a rank's share of a global batch is proportional to the throughput the
    performance model holds for that rank's unpublished target batch size (dynamic_batch.cc:254-314,
    perf_model.cc:65-95), here 16 samples at 1.6 samples/ms against 8 at 1.0, and the targets are published."""
    world, ds, gbs = 2, 400, 100
    hs, together = _ledger_ranks(world, ds, 16, gbs, False, "by_performance")
    nm = _name("ledc")
    srv = PyInfTraCommunicator(True, True, world, nm)
    ref = O.Ledger(world, ds, 16, gbs, False, "by_performance")
    try:
        for r, tgt in enumerate((16, 8)):
            srv.set_train_info(r, train_pid=os.getpid(), train_rank=r, train_world_size=world, init_batch_size=16,
                               current_batch_size=16, target_batch_size=16, target_batch_size_unpublished=tgt,
                               model_name="resnet152")
        for bs, ms in ((16, 10.0), (8, 8.0), (16, 10.0)):
            call("srt_perf_record_thpt", hs[0], bs, C.c_double(ms))
            ref.perf.record(bs, ms)
        for r in range(world):
            e = C.c_int()
            call("srt_dbd_next_epoch", hs[r], C.byref(e))
            ref.next_epoch(r)
        together(lambda r: call("srt_dbd_next_global_batch", hs[r], srv._h, 10000))
        ref.next_global_batch([16, 8])
        shares = [_ledger_info(hs[0], 6, r) for r in range(world)]
        assert shares == ref.unproc_per == [62, 38]       # int(61.5) + int(38.5) = 99: the round-off loop gives rank 0 the last one
        assert [srv.get_field(r, 5) for r in range(world)] == [16, 8]     # target := unpublished target
    finally:
        for h in hs:
            call("srt_dist_close", h)
        srv.close()


def test_distribute_batch_matches_reference_for_every_policy():
    rnd = random.Random(2)
    for _ in range(300):
        n = rnd.randint(1, 8)
        unproc = rnd.randint(n, 5000)
        perf = [rnd.choice([0.0, rnd.uniform(0.1, 9.0)]) for _ in range(n)]
        for pol in ("simple", "by_performance"):
            got = O.distribute_batch(pol, unproc, perf, n)
            assert sum(got) == unproc and (pol == "simple" or min(got) >= 1)


# ---------------------------------------------------------------- diagnostic lines
def test_log_switches_of_the_environment_contract(dist1, capfd, monkeypatch):
    """COLTRAIN_LOG_CONTROL_STUB / COLTRAIN_LOG_DYNAMIC_BATCH / COLTRAIN_LOG_ALL = "1" turn on the runtime's
    diagnostic lines on stderr (the reference's LOG_IF(INFO, TorchColConfig::log_*),
    pytorch/torch_col/csrc/config.cc:66-69,91-98); without them the runtime is silent."""
    from sirius_b200._runtime import StubConfig
    nm = _name("log")
    srv = PyInfTraCommunicator(True, True, 1, nm)
    tra = PyInfTraCommunicator(False, False, 1, nm)
    cfg = StubConfig(0, 1, 1, 1, 16, 20, 0)
    stub = C.c_void_p()
    call("srt_stub_create", tra._h, None, None, C.byref(cfg), C.byref(stub))
    D = TC._DynamicBatchDistirbutor
    dist1.init_dynamic_batch_distributor(512, 16, 32, False, "fix")
    D.next_epoch()

    def one_adjust_and_one_batch(cmd_id):
        srv.put_inf2tra(CtrlEvent.kColocateAdjustL1, cmd_id, 8, 0)
        t0 = time.time()
        while _lib.lib().srt_stub_cmd(stub) != CtrlEvent.kColocateAdjustL1:
            assert time.time() - t0 < 5
            time.sleep(0.005)
        call("srt_stub_adjust_l1_done", stub)
        call("srt_stub_set_killed_batch_recover", stub)
        assert srv.timed_get(1000, 1, 0).event == CtrlEvent.kColocateAdjustL1Done
        D.next_global_batch()
        rng, last = D.get_batch(16)
        D.abort_batch(rng, last)
        rng, last = D.get_batch(16)
        D.finish_batch(rng, last)
        rng, last = D.get_batch(16)
        D.finish_batch(rng, last)

    try:
        for v in ("COLTRAIN_LOG_ALL", "COLTRAIN_LOG_CONTROL_STUB", "COLTRAIN_LOG_DYNAMIC_BATCH"):
            monkeypatch.delenv(v, raising=False)
        one_adjust_and_one_batch(1)
        assert "torch_col" not in capfd.readouterr().err
        monkeypatch.setenv("COLTRAIN_LOG_CONTROL_STUB", "1")
        one_adjust_and_one_batch(2)
        err = capfd.readouterr().err
        assert "[torch_col control_stub" in err and "kill batch on adjust L1, cmd_id 2, target batch size 8" in err
        assert f"replies event {int(CtrlEvent.kColocateAdjustL1Done)} for cmd_id 2" in err and "dynamic_batch" not in err
        monkeypatch.delenv("COLTRAIN_LOG_CONTROL_STUB")
        monkeypatch.setenv("COLTRAIN_LOG_DYNAMIC_BATCH", "1")
        one_adjust_and_one_batch(3)
        err = capfd.readouterr().err
        assert "control_stub" not in err
        assert "[DistributeBatch] 32 unprocessed samples -> per rank [32]" in err
        assert "[AbortBatch] rank 0 gives back 16 samples: 32 unprocessed, 0 processing, 0 processed" in err
        assert "[FinishBatch] rank 0 finished 16 samples (end of global batch): 0 unprocessed, 0 processing, 32 processed" in err
        monkeypatch.setenv("COLTRAIN_LOG_DYNAMIC_BATCH", "yes")          # only "1" counts, as in the reference
        one_adjust_and_one_batch(4)
        assert "torch_col" not in capfd.readouterr().err
        monkeypatch.setenv("COLTRAIN_LOG_ALL", "1")
        one_adjust_and_one_batch(5)
        err = capfd.readouterr().err
        assert "control_stub" in err and "dynamic_batch" in err
    finally:
        call("srt_stub_stop", stub)
        tra.close()
        srv.close()


# ---------------------------------------------------------------- train adjuster
def _make_adjuster(world, targets, init_bs, cfg):
    nm = _name("adj")
    srv = PyInfTraCommunicator(True, True, world, nm)
    for r in range(world):
        srv.set_train_info(r, train_pid=1, train_rank=r, train_world_size=world, init_batch_size=init_bs,
                           current_batch_size=targets[r], target_batch_size=targets[r],
                           target_batch_size_unpublished=targets[r], model_name="resnet152")
    h = C.c_void_p()
    call("srt_adjuster_create", srv._h, C.byref(cfg), C.byref(h))
    call("srt_adjuster_load_train_info", h)
    return srv, h


def test_train_adjuster_plans_match_reference_logic():
    rnd = random.Random(3)
    b, s = C.c_double(), C.c_double()
    call("srt_adjuster_model_mem_param", b"gpt2", C.byref(b), C.byref(s))
    assert (b.value, s.value) == O.MODEL_MEM_PARAM["gpt2"]
    for trial in range(60):
        world = rnd.choice([1, 2, 4])
        init_bs = rnd.choice([32, 64, 128])
        targets = [rnd.randint(0, init_bs)] * world if rnd.random() < 0.6 else [rnd.randint(0, init_bs) for _ in range(world)]
        balance = rnd.random() < 0.5
        cfg = AdjusterConfig(1150.0, 85.0, rnd.choice([0, 4]), int(balance), 1500.0, world, 1)
        srv, h = _make_adjuster(world, targets, init_bs, cfg)
        ref = O.TrainAdjuster(1150.0, 85.0, targets, init_bs, cfg.batch_size_limit, balance, 1500.0, world, True)
        try:
            for _ in range(6):
                plan, n = (C.c_int * 8)(), C.c_int()
                if rnd.random() < 0.6:
                    dev, need = rnd.randrange(world), rnd.uniform(-100, 6000)
                    avail = [rnd.uniform(0, 20000) for _ in range(world)]
                    arr = (C.c_double * world)(*avail)
                    call("srt_adjuster_infer_require_plan", h, dev, need, arr, plan, C.byref(n))
                    want = ref.require(dev, need, avail)
                else:
                    av = [rnd.uniform(0, 20000) for _ in range(world)]
                    fr = [rnd.uniform(0, 9000) for _ in range(world)]
                    rs = [rnd.uniform(0, 2000) for _ in range(world)]
                    call("srt_adjuster_infer_release_plan", h, (C.c_double * world)(*av), (C.c_double * world)(*fr),
                         (C.c_double * world)(*rs), plan, C.byref(n))
                    want = ref.release(av, fr, rs)
                assert list(plan[:n.value]) == want, (trial, want, list(plan[:n.value]))
                if want:                                                   # published to the information board
                    assert [srv.get_field(r, 6) for r in range(world)] == want
        finally:
            call("srt_adjuster_destroy", h)
            srv.close()


def test_llm_adjust_plans_match_reference_logic():
    """The KV-cache pool's plans (server/train_adjuster.cc:342-519): on a require the target is the smaller of what the
    memory left for training allows and the current target minus the requirement's worth of samples, never below 0 and
    the same for every rank; on a release the smaller of what fits and the current target plus the freed memory's
    worth, never below the current target; both are published as the unpublished target."""
    rnd = random.Random(11)
    for trial in range(40):
        world, init_bs = rnd.choice([1, 2, 4]), rnd.choice([32, 64])
        t0 = rnd.randint(0, init_bs)
        cfg = AdjusterConfig(1150.0, 85.0, 0, 0, 1500.0, world, 1)
        srv, h = _make_adjuster(world, [t0] * world, init_bs, cfg)
        ref = O.TrainAdjuster(1150.0, 85.0, [t0] * world, init_bs, 0, False, 1500.0, world, True)
        try:
            for _ in range(8):
                plan, n = (C.c_int * 8)(), C.c_int()
                if rnd.random() < 0.5:
                    dev, need, avail = rnd.randrange(world), rnd.uniform(-50, 3000), rnd.uniform(-500, 9000)
                    call("srt_adjuster_llm_require_plan", h, dev, C.c_double(need), C.c_double(avail), None, plan, C.byref(n))
                    want = ref.llm_require(dev, need, avail)
                else:
                    av = [rnd.uniform(-500, 9000) for _ in range(world)]
                    fr = [rnd.uniform(-500, 4000) for _ in range(world)]
                    call("srt_adjuster_llm_release_plan", h, (C.c_double * world)(*av), (C.c_double * world)(*fr), plan,
                         C.byref(n))
                    want = ref.llm_release(av, fr)
                assert list(plan[:n.value]) == want, (trial, want, list(plan[:n.value]))
                if want:
                    assert [srv.get_field(r, 6) for r in range(world)] == want
        finally:
            call("srt_adjuster_destroy", h)
            srv.close()


# ---------------------------------------------------------------- page pool (host backend)
def _pool(pool_mb=64, page_mb=2, unmap_on_release=0):
    cfg = PoolConfig(0, 1, page_mb << 20, pool_mb << 20, 4, 1, unmap_on_release)
    h = C.c_void_p()
    call("srt_pool_create", C.byref(cfg), C.byref(h))
    return h


def _stat(h, which): return _lib.lib().srt_pool_stat(h, which)


@pytest.mark.parametrize("unmap_on_release", [0, 1])
def test_pool_alloc_free_empty_cache_and_handover(unmap_on_release):
    h = _pool(unmap_on_release=unmap_on_release)
    try:
        assert _stat(h, 4) == 32 and _stat(h, 5) == 64 << 20 and _stat(h, 6) == 2 << 20
        ptrs = []
        for nbytes in (3 << 20, 1 << 20, 5 << 20, 700, 2 << 20):
            p = C.c_void_p()
            call("srt_pool_alloc", h, 0, nbytes, C.byref(p))
            C.memset(p.value, 0xAB, nbytes)                 # mapped and writable
            ptrs.append(p)
        used_pages = 32 - _stat(h, 4)
        assert used_pages >= 6 and _stat(h, 3) == used_pages * (2 << 20)
        assert _stat(h, 1) >= (3 + 1 + 5 + 2) << 20
        # free the 5 MiB block: its wholly-free pages go back on empty_cache, partially used ones stay
        call("srt_pool_free", h, 0, ptrs[2])
        rel = C.c_size_t()
        call("srt_pool_empty_cache", h, 0, C.byref(rel))
        assert rel.value >= 2 << 20 and rel.value % (2 << 20) == 0
        free_after = _stat(h, 4)
        assert free_after == 32 - used_pages + rel.value // (2 << 20)
        # the inference allocator can now take everything that is free, and not one page more
        q = C.c_void_p()
        call("srt_pool_alloc", h, 1, free_after * (2 << 20), C.byref(q))
        assert _stat(h, 4) == 0 and _stat(h, 0) == free_after * (2 << 20)
        with pytest.raises(SrtError):
            call("srt_pool_alloc", h, 0, 8 << 20, C.byref(C.c_void_p()))
        with pytest.raises(SrtError):
            call("srt_pool_free", h, 0, ptrs[2])              # double free is an error, not a crash
        call("srt_pool_free", h, 1, q)
        call("srt_pool_empty_cache", h, 1, C.byref(rel))
        assert rel.value == free_after * (2 << 20)
        for i in (0, 1, 3, 4):
            call("srt_pool_free", h, 0, ptrs[i])
        call("srt_pool_empty_cache", h, 0, C.byref(rel))
        assert _stat(h, 4) == 32 and _stat(h, 1) == 0 and _stat(h, 3) == 0
        if unmap_on_release:
            assert _stat(h, 7) == _stat(h, 8) > 0             # every map has its unmap
        else:
            assert _stat(h, 7) > 0 and _stat(h, 8) <= _stat(h, 7)   # mappings are kept until a slot needs another page
    finally:
        call("srt_pool_destroy", h)


def test_pool_keeps_mappings_so_a_repeated_handover_makes_no_driver_calls():
    """Training and inference trade the same pages back and forth: after the first exchange the slots
    take their kept pages back (num_reuse grows) and neither num_map nor num_unmap moves."""
    page = 2 << 20
    h = _pool(pool_mb=32, page_mb=2)                          # 16 pages
    try:
        def alloc(kind, n):
            p = C.c_void_p()
            call("srt_pool_alloc", h, kind, n, C.byref(p))
            C.memset(p.value, kind + 1, n)
            return p
        rel = C.c_size_t()
        big = alloc(0, 16 * page)                             # training owns the whole pool
        counts = []
        for cycle in range(4):
            # handover: training shrinks to 12 pages, inference takes the 4 it gave up
            call("srt_pool_free", h, 0, big)
            small = alloc(0, 12 * page)
            call("srt_pool_empty_cache", h, 0, C.byref(rel))
            assert rel.value == 4 * page and _stat(h, 4) == 4
            inf = alloc(1, 4 * page)
            assert _stat(h, 4) == 0
            # give-back: inference leaves, training grows to the whole pool again
            call("srt_pool_free", h, 1, inf)
            call("srt_pool_empty_cache", h, 1, C.byref(rel))
            assert rel.value == 4 * page
            call("srt_pool_free", h, 0, small)
            big = alloc(0, 16 * page)
            assert _stat(h, 4) == 0
            counts.append((_stat(h, 7), _stat(h, 8), _stat(h, 10)))
        assert counts[0][:2] == (20, 0)                       # 16 training maps + 4 inference maps, nothing unmapped
        assert all(c[:2] == counts[0][:2] for c in counts[1:])
        assert [c[2] for c in counts] == [4, 12, 20, 28]      # later exchanges are served by kept mappings alone
        # a slot whose kept page serves someone else gets another page: that costs one unmap and one map
        call("srt_pool_free", h, 0, big)
        call("srt_pool_empty_cache", h, 0, C.byref(rel))
        inf = alloc(1, 4 * page)                              # inference slots 0..3 take their kept pages (12..15) back
        low = alloc(0, 16 * page - 4 * page)                  # training slots 0..11 take theirs
        assert (_stat(h, 7), _stat(h, 8)) == counts[0][:2]
    finally:
        call("srt_pool_destroy", h)


def test_pool_oom_handler_gets_a_chance_to_release_memory():
    h = _pool(pool_mb=16, page_mb=2)
    held = C.c_void_p()
    call("srt_pool_alloc", h, 0, 12 << 20, C.byref(held))
    calls = []
    FN = C.CFUNCTYPE(None, C.c_void_p, C.c_int, C.c_size_t)

    def on_oom(user, kind, nbytes):   # what the trainer does on an L1 adjust: drop activations, empty the cache
        calls.append((kind, nbytes))
        call("srt_pool_free", h, 0, held)
        call("srt_pool_empty_cache", h, 0, None)

    cb = FN(on_oom)
    call("srt_pool_set_oom_handler", h, C.cast(cb, C.c_void_p), None)
    try:
        p = C.c_void_p()
        call("srt_pool_alloc", h, 1, 10 << 20, C.byref(p))   # inference needs more than is free
        assert calls == [(1, 10 << 20)] and p.value
    finally:
        call("srt_pool_destroy", h)


def test_pool_random_workload_keeps_invariants():
    h = _pool(pool_mb=128, page_mb=2)
    rnd = random.Random(4)
    live = {}
    try:
        for it in range(3000):
            if live and (rnd.random() < 0.45 or len(live) > 60):
                k = rnd.choice(list(live))
                kind, ptr, n, tag = live.pop(k)
                assert C.string_at(ptr.value, 1)[0] == tag and C.string_at(ptr.value + n - 1, 1)[0] == tag
                call("srt_pool_free", h, kind, ptr)
            else:
                kind, n = rnd.randint(0, 1), rnd.choice([512, 4096, 100000, 1 << 20, 3 << 20, 7 << 20])
                p = C.c_void_p()
                try:
                    call("srt_pool_alloc", h, kind, n, C.byref(p))
                except SrtError:
                    call("srt_pool_empty_cache", h, 1 - kind, None)
                    continue
                tag = it % 251
                C.memset(p.value, tag, n)
                live[it] = (kind, p, n, tag)
            if it % 97 == 0:
                call("srt_pool_empty_cache", h, rnd.randint(0, 1), None)
            mapped = (_stat(h, 3) + _stat(h, 0)) // (2 << 20)
            assert mapped + _stat(h, 4) == 64                       # every page is FREE, TRAIN or INFER
            assert _stat(h, 1) <= _stat(h, 3)
        for kind, ptr, n, tag in live.values():
            call("srt_pool_free", h, kind, ptr)
        call("srt_pool_empty_cache", h, 0, None)
        call("srt_pool_empty_cache", h, 1, None)
        assert _stat(h, 4) == 64
    finally:
        call("srt_pool_destroy", h)


def test_pool_and_channel_under_several_threads():
    """Six threads allocate, tag, check and free on both allocators of one pool (with empty_cache calls in between)
    while four putters and three getters share one channel: no allocation overlaps another live one (every block keeps
    its tag), the page accounting closes, every message put is received exactly once. The sanitizer builds
    (`python -m sirius_b200._build --tsan|--asan`) run the same test."""
    import threading
    h = _pool(pool_mb=192, page_mb=2)
    srv = PyInfTraCommunicator(True, True, 4, _name("mt"))
    stop, errors = threading.Event(), []
    put, got = [0] * 4, [0] * 3

    def alloc_worker(i):
        kind, rnd, held = i % 2, random.Random(i), []
        try:
            while not stop.is_set():
                if held and (len(held) > 12 or rnd.random() < 0.45):
                    ptr, n, tag = held.pop(rnd.randrange(len(held)))
                    assert C.string_at(ptr.value, 1)[0] == tag and C.string_at(ptr.value + n - 1, 1)[0] == tag
                    call("srt_pool_free", h, kind, ptr)
                else:
                    n, ptr = rnd.choice([512, 4096, 100000, 1 << 20, 3 << 20]), C.c_void_p()
                    try:
                        call("srt_pool_alloc", h, kind, n, C.byref(ptr))
                    except SrtError:
                        continue                                   # the other side holds the pages right now
                    tag = (i * 37 + len(held)) % 251
                    C.memset(ptr.value, tag, n)
                    held.append((ptr, n, tag))
                if rnd.random() < 0.02:
                    call("srt_pool_empty_cache", h, kind, None)
            for ptr, n, tag in held:
                assert C.string_at(ptr.value, 1)[0] == tag
                call("srt_pool_free", h, kind, ptr)
        except BaseException as e:  # noqa: BLE001
            errors.append(repr(e))

    def putter(i):
        rnd = random.Random(50 + i)
        try:
            while not stop.is_set():
                try:
                    srv.put_tra2inf(CtrlEvent.kReportBatchSize, put[i] + 1, i, rnd.randrange(4))
                    put[i] += 1
                except SrtError:
                    time.sleep(0.0005)                             # that ring is full: let the getters catch up
        except BaseException as e:  # noqa: BLE001
            errors.append(repr(e))

    def getter(i):
        try:
            while not stop.is_set():
                m = srv.timed_get_from_any(5, 1) if i else srv.timed_get(5, 1, 0)
                if m is not None:
                    got[i] += 1
        except BaseException as e:  # noqa: BLE001
            errors.append(repr(e))

    threads = ([threading.Thread(target=alloc_worker, args=(i,)) for i in range(6)]
               + [threading.Thread(target=putter, args=(i,)) for i in range(4)])
    getters = [threading.Thread(target=getter, args=(i,)) for i in range(3)]
    try:
        for t in threads + getters:
            t.start()
        time.sleep(1.5)
        stop.set()
        for t in threads + getters:
            t.join(30)
        assert not errors, errors[:3]
        while srv.timed_get_from_any(0, 1) is not None:           # what the getters left behind when they stopped
            got[0] += 1
        assert sum(put) == sum(got) and sum(put) > 100
        call("srt_pool_empty_cache", h, 0, None)
        call("srt_pool_empty_cache", h, 1, None)
        assert _stat(h, 4) == 96 and _stat(h, 0) == 0 and _stat(h, 1) == 0
    finally:
        stop.set()
        srv.close()
        call("srt_pool_destroy", h)


# ---------------------------------------------------------------- orphaned segments
def _orphan_maker(name):
    """Rank 0 of an earlier job: creates the segment, then dies without cleaning up."""
    h = C.c_void_p()
    call("srt_dist_open", name.encode(), 0, 2, 2000, C.byref(h))
    os._exit(0)


def _late_rank(rank, name, delay, q):
    import time
    time.sleep(delay)
    h = C.c_void_p()
    t0 = time.time()
    call("srt_dist_open", name.encode(), rank, 2, 20000, C.byref(h))
    opened = time.time()
    call("srt_dist_barrier", h, 20000)                       # both ranks are on the SAME segment: the barrier opens
    if rank == 1:
        call("srt_dist_send", h, 0, b"same job", 8)
    else:
        buf, n = C.create_string_buffer(64), C.c_int()
        call("srt_dist_recv", h, 1, buf, 64, 20000, C.byref(n))
        assert buf.raw[:n.value] == b"same job"
    call("srt_dist_barrier", h, 20000)
    q.put((rank, (t0, opened)))
    call("srt_dist_close", h)


def test_a_rank_that_starts_first_does_not_attach_to_the_segment_of_a_dead_job():
    """A ready dist_train_sync segment left in /dev/shm by a killed job, and rank 1 of the next job starting
    before its rank 0: rank 1 must not map the orphan (the two ranks would then wait on different barriers);
    it waits until this job's rank 0 has replaced the segment."""
    ctx = mp.get_context("spawn")
    nm = _name("orphan")
    maker = ctx.Process(target=_orphan_maker, args=(nm,))
    maker.start()
    maker.join(30)
    assert maker.exitcode == 0 and os.path.exists("/dev/shm/" + nm)     # the orphan is there, ready, and ownerless
    q = ctx.Queue()
    ps = [ctx.Process(target=_late_rank, args=(1, nm, 0.0, q)), ctx.Process(target=_late_rank, args=(0, nm, 2.0, q))]
    for p in ps:
        p.start()
    out = dict(q.get(timeout=60) for _ in range(2))
    for p in ps:
        p.join(30)
        assert p.exitcode == 0
    # rank 1 waited for rank 0 instead of taking the orphan at once: its open returned after rank 0 had begun its own
    assert out[1][0] < out[0][0] and out[1][1] >= out[0][0]
    # and with nobody to replace it, opening fails with a message instead of succeeding on the orphan
    maker = ctx.Process(target=_orphan_maker, args=(nm,))
    maker.start()
    maker.join(30)
    h = C.c_void_p()
    with pytest.raises(SrtError, match="no longer runs"):
        call("srt_dist_open", nm.encode(), 1, 2, 300, C.byref(h))
    os.unlink("/dev/shm/" + nm)
