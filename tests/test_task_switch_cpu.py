"""Task-switch mode on CPU ranks (SwitchStub / SwitchCtrl, pytorch/torch_col/csrc/control_stub.cc:186-400 and
pytorch/torch_col/colocate_ctrl.py:117-301): two trainer processes run the torch_col Trainer loop in taskswitch-l1;
this process plays the server with DebugServer. kInterruptTrain kills the micro-batch in flight, the trainers release
their memory and the master replies kInterruptTrainDone with the command id; while interrupted nothing trains and a
second interrupt is answered at once; kResumeTrain (to rank 0 only) releases both ranks, the master replies
kResumeTrainDone, and every sample of every epoch is still trained exactly once."""
import multiprocessing as mp
import os
import time
import uuid

import pytest

from sirius_b200.torch_col._C import CtrlEvent

DS, GLOBAL_BS, BS, EPOCHS = 96, 32, 8, 3


def _trainer(rank, world, comm_name, dist_name, port, q):
    os.environ.update({
        "COLTRAIN_MODE": "taskswitch-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
        "COLTRAIN_HAS_INFER_SERVER": "1", "SIRIUS_B200_COMM_NAME": comm_name, "SIRIUS_B200_DIST_NAME": dist_name,
        "MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port)})
    import torch
    import torch.distributed as tdist
    from sirius_b200 import torch_col as tc
    torch.manual_seed(0)
    torch.set_num_threads(1)
    tc.setup_colocate_training(rank, world, True, True)   # gloo process group on CPU
    model = torch.nn.Sequential(torch.nn.Flatten(), torch.nn.Linear(3 * 8 * 8, 10))
    opt = torch.optim.SGD(model.parameters(), 0.05, momentum=0.9)
    crit = torch.nn.CrossEntropyLoss()
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), EPOCHS, BS,
                                   stub_poll_ms=20)
    assert isinstance(ctrl, tc.SwitchCtrl)
    ds, mgr = tc.init_dynamic_batch(DS, tc.DatasetType.VISION, tc.VisionDatasetConfig((3, 8, 8), 10), BS,
                                    global_batch_size=GLOBAL_BS, enable_grad_accumulate=True,
                                    checkpoint_micro_batch=True, batch_distribute_policy=tc.BatchDistributePolicy.SIMPLE)
    tc.init_train_info(BS, BS, "resnet152")
    tc.util.initialize_sgd_optimizer(model, opt)

    class Acc(tc.GradAccumulator):
        def step(self, optimizer=None, scaler=None, do_zero_grad=True):
            for p in self.param_list:
                tdist.all_reduce(self.param_grads[p]['global'])
            super().step(optimizer, scaler, do_zero_grad)

    acc = Acc(model)
    seen = []

    def iter_train_fn(batch):
        ctrl.check_kill('fwd')
        out = model(batch['images'])
        loss = mgr.scale_loss(batch, crit(out, batch['labels']))
        time.sleep(0.004)
        ctrl.check_kill('bwd')
        loss.backward()
        mgr.optimizer_step(batch, opt, grad_accumulator=acc)
        seen.append((list(batch['range']), len(batch), time.time()))
        return loss.item()

    trainer = tc.Trainer(model, iter_train_fn)
    tc.dist.wait_barrier()
    ctrl.train_start()
    for e in range(EPOCHS):
        trainer.train_one_epoch(e)
    ctrl.train_end()
    stat = trainer.get_overall_stat()
    w = torch.cat([p.detach().flatten() for p in model.parameters()])
    q.put((rank, seen, stat.killed_batch, float(w.double().sum()), ctrl.switch_log,
           tc.EventManager.to_csv(True, tc.get_colocate_train_mode())))
    tc.dist.wait_barrier()
    tc.cleanup_colocate_training(True)


@pytest.mark.timeout(180)
def test_two_rank_task_switch_interrupt_and_resume():
    from sirius_b200.torch_col import DebugServer
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    comm_name, dist_name = f"srt_ts_comm_{tag}", f"srt_ts_dist_{tag}"
    srv = DebugServer(2, comm_name)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 31500 + (os.getpid() % 2000)
    ps = [ctx.Process(target=_trainer, args=(r, 2, comm_name, dist_name, port, q)) for r in range(2)]
    for p in ps:
        p.start()
    try:
        t0 = time.time()
        while not srv.events(CtrlEvent.kTrainStart):
            assert time.time() - t0 < 90, "trainers never started"
            time.sleep(0.01)
        while len(srv.events(CtrlEvent.kReportBatchSize)) < 6:     # let a few micro-batches pass
            time.sleep(0.002)
        cid = srv.interrupt_train()
        wait_s = srv.wait_event(CtrlEvent.kInterruptTrainDone, cid, 1, 60)
        t_int = time.time()
        cid2 = srv.interrupt_train()                                # already interrupted: answered at once
        wait2_s = srv.wait_event(CtrlEvent.kInterruptTrainDone, cid2, 1, 30)
        time.sleep(0.4)                                             # the job is off the processor meanwhile
        t_res = time.time()
        srv.resume_train()
        srv.wait_event(CtrlEvent.kResumeTrainDone, None, 1, 60)
        out = sorted(q.get(timeout=120) for _ in range(2))
    finally:
        for p in ps:
            p.join(60)
        srv.close()
    assert all(p.exitcode == 0 for p in ps)
    ranges = sorted(r for _, seen, *_ in out for rv, _, _ in seen for r in rv)
    assert sum(j - i for i, j in ranges) == DS * EPOCHS            # every sample of every epoch exactly once
    assert ranges[0][0] == 0 and ranges[-1][1] == DS
    assert out[0][3] == pytest.approx(out[1][3], rel=1e-6)         # identical parameters on both ranks
    assert wait_s < 30 and wait2_s < 5
    # only the master replies, with the command ids in order
    assert [(r, m.id) for r, m in srv.events(CtrlEvent.kInterruptTrainDone)] == [(0, cid), (0, cid2)]
    assert [r for r, _ in srv.events(CtrlEvent.kResumeTrainDone)] == [0]
    # no micro-batch finished between the reply and the resume command
    for _, seen, *_ in out:
        assert not [t for _, _, t in seen if t_int + 0.05 < t < t_res]
    assert all(len(o[4]) == 1 for o in out)                        # one switch handled per rank
    for o in out:
        assert "switch_l1" in o[5] and "wait_resume" in o[5]
