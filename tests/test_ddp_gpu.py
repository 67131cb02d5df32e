"""Data-parallel gradient exchange on two GPUs through the library's NCCL communicator (srt_ddp_*,
srt_allreduce_begin / wait): one process per GPU, as in training. Skipped with fewer than two GPUs.

The ranks find each other through a gloo process group (it only carries the communicator's unique id and the
values the test compares); the gradients travel through the library. NVLS is off in the children so that a rank
that fails in a test cannot leave its peer bound to a multicast object."""
import multiprocessing as mp
import os
import time
import uuid

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

needs_two = pytest.mark.skipif(torch.cuda.device_count() < 2, reason="needs two GPUs")

ARCH, B, IMG = "resnet14", 8, 64


def _child_env(rank, port):
    os.environ.update({"MASTER_ADDR": "127.0.0.1", "MASTER_PORT": str(port), "NCCL_NVLS_ENABLE": "0",
                       "RANK": str(rank), "WORLD_SIZE": "2"})


def _exchange_rank(rank, port, q):
    _child_env(rank, port)
    import torch.distributed as dist
    from oracle import resnet_oracle as O
    from sirius_b200 import ddp, ops
    from sirius_b200.step import GET_GRAD, ResNetStep
    torch.cuda.set_device(rank)
    dist.init_process_group("gloo", rank=rank, world_size=2)
    model = O.build_model(ARCH, 0)
    step = ResNetStep(layers=O.LAYERS[ARCH], max_batch=B, image=IMG, dtype="bf16")
    step.load_state_dict(O.state_arrays(model))
    im, lb = O.make_batches(B, 1, IMG, seed=100 + rank)[0]      # every rank its own samples
    ptr, n = step.grad_buffer()

    class Buf:
        __cuda_array_interface__ = {"shape": (n,), "typestr": "<f4", "data": (ptr, False), "version": 2}
    grad = torch.as_tensor(Buf(), device=f"cuda:{rank}")
    out = {}
    for wire in ("f32", "bf16"):
        ex = ddp.GradExchange(rank, 2, device=rank, wire=wire, max_ctas=8)
        step.upload_batch(im, lb)
        step.forward_backward(B, 2 * B)
        step.synchronize()
        mine = grad.clone().cpu()
        both = [torch.empty_like(mine) for _ in range(2)]
        dist.all_gather(both, mine)
        # the same backward again, this time exchanged while it runs
        step.forward_backward(B, 2 * B)
        ex.begin(step)
        ex.wait(step)
        step.synchronize()
        got = grad.clone().cpu()
        if wire == "f32":
            want = both[0] + both[1]
            assert torch.equal(got, want), float((got - want).abs().max())
        else:
            bf = torch.bfloat16
            want = (both[0].to(bf).float() + both[1].to(bf).float())
            err = (got - want).abs().max() / want.abs().max()
            assert float(err) < 2 ** -8, float(err)
        st = ex.stats()
        assert st["exchanges"] == 1 and st["bytes_on_wire"] == n * (4 if wire == "f32" else 2)
        # abort and rejoin under a new id (what the reference does after a killed batch left ranks out of step)
        if wire == "f32":
            ex.abort()
            ex.restart()
            step.forward_backward(B, 2 * B)
            ex.allreduce(step)
            step.synchronize()
            assert torch.equal(grad.cpu(), want)
        step.optimizer_step()
        step.synchronize()
        out[wire] = float(torch.as_tensor(step.get("layer2.0.conv2.weight")).double().sum())
        ex.close()
    assert ops.tc_status() == 0
    q.put((rank, out))
    dist.barrier()
    dist.destroy_process_group()
    step.close()


def _run_two(target, extra=()):
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29600 + (os.getpid() % 2000)
    ps = [ctx.Process(target=target, args=(r, port, q) + tuple(extra)) for r in range(2)]
    for p in ps:
        p.start()
    try:
        out = sorted(q.get(timeout=240) for _ in range(2))
    finally:
        for p in ps:
            p.join(60)
            if p.is_alive():
                p.terminate()
    assert all(p.exitcode == 0 for p in ps), [p.exitcode for p in ps]
    return out


@needs_two
@pytest.mark.timeout(300)
def test_bucketed_exchange_sums_the_ranks_gradients_in_both_wire_formats():
    """fp32 on the wire: every rank ends with exactly g0 + g1 in its gradient buffer (bucket by bucket, each behind
    its ready event while backward still runs). bf16 on the wire: the sum of the bf16-rounded gradients, to bf16
    precision, at half the bytes. After the optimizer step both ranks hold the same parameters."""
    out = _run_two(_exchange_rank)
    assert out[0][1] == out[1][1]


DS, GBS, EPOCHS = 96, 32, 2


def _trainer_rank(rank, port, q, comm_name, dist_name):
    _child_env(rank, port)
    os.environ.update({"COLTRAIN_MODE": "colocate-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
                       "COLTRAIN_HAS_INFER_SERVER": "1", "SIRIUS_B200_COMM_NAME": comm_name,
                       "SIRIUS_B200_DIST_NAME": dist_name})
    from oracle import resnet_oracle as O
    from sirius_b200 import ddp, ops
    from sirius_b200 import torch_col as tc
    from sirius_b200._lib import SrtError
    from sirius_b200.step import ResNetStep
    torch.cuda.set_device(rank)
    tc.setup_colocate_training(rank, 2, True, True)            # gloo group: carries the communicator id
    model = O.build_model(ARCH, 0)
    step = ResNetStep(layers=O.LAYERS[ARCH], max_batch=B, image=IMG, dtype="bf16")
    step.load_state_dict(O.state_arrays(model))
    tc.set_train_step(step)
    ex = ddp.GradExchange(rank, 2, device=rank, wire="f32")
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), EPOCHS, B,
                                   stub_poll_ms=5)
    ds, mgr = tc.init_dynamic_batch(DS, tc.DatasetType.VISION, tc.VisionDatasetConfig((3, IMG, IMG), 1000), B,
                                    global_batch_size=GBS, enable_grad_accumulate=True, checkpoint_micro_batch=True,
                                    batch_distribute_policy=tc.BatchDistributePolicy.SIMPLE)
    tc.init_train_info(B, B, "resnet152")
    acc = tc.GradAccumulator(step, exchange=ex)
    seen = []

    def iter_train_fn(batch):
        step.upload_batch(batch["images"], batch["labels"])
        try:
            step.forward_backward(len(batch), GBS)
        except SrtError as e:
            if "aborted" in str(e):
                raise tc.ColocateAdjustL1Exception("killed in the executor")
            raise
        ctrl.check_kill("after backward")
        loss = step.loss()
        mgr.optimizer_step(batch, step, grad_accumulator=acc)
        seen.append((list(batch["range"]), len(batch)))
        return loss

    trainer = tc.Trainer(step, iter_train_fn)
    tc.dist.wait_barrier()
    ctrl.train_start()
    for e in range(EPOCHS):
        trainer.train_one_epoch(e)
    ctrl.train_end()
    step.synchronize()
    assert ops.tc_status() == 0
    w = step.get("layer3.0.conv2.weight")
    q.put((rank, seen, trainer.get_overall_stat().killed_batch, w.tobytes(), ex.stats()["exchanges"]))
    tc.dist.wait_barrier()
    ex.close()
    step.close()
    tc.cleanup_colocate_training(True)
    tc.set_train_step(None)


@needs_two
@pytest.mark.timeout(400)
def test_trainer_on_two_gpus_exchanges_accumulated_gradients_and_survives_an_adjust():
    """The torch_col Trainer loop on two GPUs, each with a ResNet step object, the accumulated gradients summed over
    the ranks by the library's NCCL exchange right before every update, while a debug server sends an L1 adjust
    (batch 8 -> 4) in mid-run and gives the memory back later: every sample of every epoch is trained exactly
    once over the two ranks, and both ranks end with bit-identical weights."""
    from sirius_b200.torch_col import DebugServer
    from sirius_b200.torch_col._C import CtrlEvent
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    comm_name, dist_name = f"srt_ddp_comm_{tag}", f"srt_ddp_dist_{tag}"
    srv = DebugServer(2, comm_name)
    ctx = mp.get_context("spawn")
    q = ctx.Queue()
    port = 29700 + (os.getpid() % 2000)
    ps = [ctx.Process(target=_trainer_rank, args=(r, port, q, comm_name, dist_name)) for r in range(2)]
    for p in ps:
        p.start()
    try:
        t0 = time.time()
        while not srv.events(CtrlEvent.kTrainStart):
            assert time.time() - t0 < 240, "trainers never started"
            time.sleep(0.01)
        while len(srv.events(CtrlEvent.kReportBatchSize)) < 4:
            assert time.time() - t0 < 300
            time.sleep(0.002)
        cid = srv.colocate_l1([4, 4])
        srv.wait_adjust_done(cid, 60)
        srv.infer_exit([B, B])
        out = sorted(q.get(timeout=240) for _ in range(2))
    finally:
        for p in ps:
            p.join(60)
            if p.is_alive():
                p.terminate()
        srv.close()
    assert all(p.exitcode == 0 for p in ps), [p.exitcode for p in ps]
    ranges = sorted(r for _, seen, *_ in out for rv, _ in seen for r in rv)
    assert sum(j - i for i, j in ranges) == DS * EPOCHS
    assert out[0][3] == out[1][3]                              # identical weights on both ranks
    assert out[0][4] == out[1][4] >= DS * EPOCHS // GBS        # one exchange per global batch, the same count
