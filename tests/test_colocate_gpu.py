"""Colocation on the GPU: a pool-backed ResNet step is killed in mid-batch by an L1 adjust from the
(debug) inference server, releases its activation pages, replies, and carries on; the freed pages are
immediately usable by the inference allocator. Mirrors the reference's kill-vs-no-kill check
(train/train_valiation.py:83-95): a run with a kill must reproduce the losses and weights of a run
without one, because the killed micro-batch is redone from the same samples."""
import os
import time
import uuid

import numpy as np
import pytest
import torch

pytestmark = pytest.mark.gpu

from oracle import resnet_oracle as O
from sirius_b200 import ops
from sirius_b200._lib import SrtError
from sirius_b200.pool import INFER, TRAIN, PagePool
from sirius_b200.step import ResNetStep

ARCH, B, IMG = "resnet50", 16, 64


def _wait_cmd(ctrl, event, limit_s=5.0):
    """Until the trainer's control thread has taken the command in (it raises the kill flag before it publishes the
    command): a fixed sleep would be a guess about the host's load."""
    t0 = time.time()
    while ctrl._stub.cmd != event:
        assert time.time() - t0 < limit_s, f"the control thread never saw {event}"
        time.sleep(0.002)


def _batches(n):
    return O.make_batches(B, n, IMG)


def test_pool_backed_step_matches_cudamalloc_step_and_releases_pages():
    pool = PagePool(2.0)
    model = O.build_model(ARCH, 0)
    ref = ResNetStep(layers=O.LAYERS[ARCH], max_batch=B, image=IMG, dtype="bf16")
    stp = ResNetStep(layers=O.LAYERS[ARCH], max_batch=B, image=IMG, dtype="bf16", pool=pool.handle)
    for s in (ref, stp):
        s.load_state_dict(O.state_arrays(model))
    batches = _batches(3)
    l_ref = [ref.train_step(*b) for b in batches]
    l_stp = [stp.train_step(*b) for b in batches[:2]]
    # handover: everything the step took from the pool for activations comes back as whole pages
    used = pool.stat("train_all")
    assert used > 0 and pool.stat("free_pages") * pool.stat("page_nbytes") + used == pool.stat("pool_nbytes")
    t0 = time.perf_counter()
    released = stp.release_activations()
    dt = time.perf_counter() - t0
    assert released == used and pool.stat("train_all") == 0
    print(f"released {released / 2**20:.0f} MiB in {dt * 1e3:.2f} ms = {dt * 1e3 / (released / 2**30):.2f} ms/GiB")
    # the inference allocator can map all of it at once, and training cannot while it is held
    p = pool.alloc(INFER, pool.stat("pool_nbytes"))
    with pytest.raises(SrtError):
        stp.reserve_activations(B)
    pool.free(INFER, p)
    pool.empty_cache(INFER)
    # regain: the next step re-allocates and continues bit-exactly
    l_stp.append(stp.train_step(*batches[2]))
    assert l_stp == l_ref
    for k in ("conv1.weight", "layer3.2.conv2.weight", "fc.weight"):
        assert np.array_equal(stp.get(k), ref.get(k))
    assert ops.tc_status() == 0
    stp.close(); ref.close(); pool.close()


def test_l1_adjust_kills_batch_releases_memory_and_training_reproduces_undisturbed_run():
    from sirius_b200 import torch_col as tc
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    os.environ.update({"COLTRAIN_MODE": "colocate-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
                       "COLTRAIN_HAS_INFER_SERVER": "1", "COLTRAIN_USE_SHARED_TENSOR": "1",
                       "COLTRAIN_KEEP_TARGET_SET": "0",   # the adjust names the same batch size: release everything
                       "SIRIUS_B200_COMM_NAME": f"srt_gpu_comm_{tag}", "SIRIUS_B200_DIST_NAME": f"srt_gpu_dist_{tag}"})
    model = O.build_model(ARCH, 0)
    DS, GBS, EPOCHS = 96, 32, 2

    def run(inject):
        srv = tc.DebugServer(1, os.environ["SIRIUS_B200_COMM_NAME"])
        pool = PagePool(2.0)
        tc.setup_colocate_training(0, 1, False, False)
        step = ResNetStep(layers=O.LAYERS[ARCH], max_batch=B, image=IMG, dtype="bf16", pool=pool.handle)
        step.load_state_dict(O.state_arrays(model))
        tc.set_train_step(step)
        tc.set_memory_pool(pool.handle)
        ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), EPOCHS, B,
                                       stub_poll_ms=5)
        ds, mgr = tc.init_dynamic_batch(DS, tc.DatasetType.VISION, tc.VisionDatasetConfig((3, IMG, IMG), 1000), B,
                                        global_batch_size=GBS, enable_grad_accumulate=True, checkpoint_micro_batch=True)
        tc.init_train_info(B, B, "resnet152")
        acc = tc.GradAccumulator(step)
        losses, state = [], {"n": 0, "cid": None, "free_before": None}

        def iter_train_fn(batch):
            state["n"] += 1
            step.upload_batch(batch["images"], batch["labels"])
            if inject and state["n"] == 4 and state["cid"] is None:
                state["free_before"] = pool.stat("free_pages")
                state["cid"] = srv.colocate_l1([B])        # same target: the batch is redone as it was
                _wait_cmd(ctrl, tc.CtrlEvent.kColocateAdjustL1)
            try:
                step.forward_backward(len(batch), GBS)
            except SrtError as e:
                if "aborted" in str(e):
                    raise tc.ColocateAdjustL1Exception("killed in the executor")
                raise
            ctrl.check_kill("after backward")
            loss = step.loss()
            mgr.optimizer_step(batch, step, grad_accumulator=acc)
            losses.append(loss)
            return loss

        trainer = tc.Trainer(step, iter_train_fn)
        ctrl.train_start()
        for e in range(EPOCHS):
            trainer.train_one_epoch(e)
        ctrl.train_end()
        step.synchronize()
        out = {"losses": losses, "w": step.get("layer2.1.conv2.weight"), "killed": trainer.get_overall_stat().killed_batch,
               "adjust": list(ctrl.adjust_log), "done": srv.events(tc.CtrlEvent.kColocateAdjustL1Done),
               "cid": state["cid"], "free_before": state["free_before"], "page": pool.stat("page_nbytes")}
        assert ops.tc_status() == 0
        step.close()
        tc.cleanup_colocate_training(False)
        tc.set_train_step(None)
        pool.close()
        srv.close()
        return out

    quiet = run(False)
    noisy = run(True)
    assert quiet["killed"] == 0 and noisy["killed"] == 1
    assert [m.id for _, m in noisy["done"]] == [noisy["cid"]]
    rel_ms, cache_ms, reply_ms, released = noisy["adjust"][0][:4]
    assert released > 0 and released % noisy["page"] == 0
    print(f"L1 adjust: release {rel_ms:.2f} ms, empty cache {cache_ms:.2f} ms, reply {reply_ms:.2f} ms, "
          f"{released / 2**20:.0f} MiB handed over = {(rel_ms + cache_ms + reply_ms) / (released / 2**30):.2f} ms/GiB")
    # the killed micro-batch was redone from the same samples: identical finished-batch losses and weights
    assert noisy["losses"] == quiet["losses"]
    assert np.array_equal(noisy["w"], quiet["w"])


@pytest.mark.parametrize("unmap_on_release", [False, True])
def test_shrink_keeps_a_smaller_set_on_mapped_pages_and_regrow_maps_only_the_difference(unmap_on_release):
    model = O.build_model(ARCH, 0)
    batches = O.make_batches(B, 1, IMG)
    pool = PagePool(2.0, unmap_on_release=unmap_on_release)
    page = pool.stat("page_nbytes")
    step = ResNetStep(layers=O.LAYERS[ARCH], max_batch=B, image=IMG, dtype="bf16", pool=pool.handle)
    step.load_state_dict(O.state_arrays(model))
    im, lb = batches[0]
    step.upload_batch(im, lb); step.forward_backward(B, B); loss_full = step.loss()
    mapped_full, maps0, unmaps0 = pool.stat("train_all"), pool.stat("num_map"), pool.stat("num_unmap")
    released = step.shrink_activations(B // 2)
    assert released > 0 and released % page == 0
    assert pool.stat("num_map") == maps0                       # nothing was mapped to place the smaller set
    assert pool.stat("num_unmap") - unmaps0 == (released // page if unmap_on_release else 0)
    assert pool.stat("train_all") == mapped_full - released and pool.stat("free_pages") * page >= released
    # the inference allocator can use what was handed over while training runs the smaller batch
    q = pool.alloc(INFER, released)
    torch.cuda.synchronize()
    step.upload_batch(im[:B // 2].contiguous(), lb[:B // 2].contiguous())
    step.forward_backward(B // 2, B // 2)
    assert np.isfinite(step.loss()) and pool.stat("num_map") == maps0 + released // page
    pool.free(INFER, q)
    pool.empty_cache(INFER)
    # growing back takes exactly the pages that were returned, and the full batch reproduces its loss
    reuse0 = pool.stat("num_reuse")
    step.upload_batch(im, lb); step.forward_backward(B, B)
    if unmap_on_release:
        assert pool.stat("num_map") - maps0 == 2 * (released // page)
    else:
        assert pool.stat("num_map") - maps0 == released // page and pool.stat("num_reuse") - reuse0 == released // page
    assert pool.stat("train_all") == mapped_full
    assert step.loss() == loss_full
    assert ops.tc_status() == 0
    step.close(); pool.close()


def test_inference_mode_forward_uses_running_statistics():
    model = O.build_model("resnet14", 0)
    (im, lb), = O.make_batches(4, 1, 64)
    with torch.no_grad():
        model.train(); model(im); model(im)        # move the running statistics away from their defaults
        model.eval(); ref = model(im[:1]).numpy()
    step = ResNetStep(layers=O.LAYERS["resnet14"], max_batch=4, image=64, dtype="f32")
    step.load_state_dict(O.state_arrays(model))
    step.upload_batch(im[:1].contiguous(), lb[:1].contiguous())
    step.forward_infer(1)
    got = step.logits(1)
    assert np.abs(got - ref).max() <= 1e-4 * np.abs(ref).max()


def test_gpt2_batch_size_adjustment_on_inference_arrival():
    """The GPT-2 colocation workload's control path on a small GPT-2: the trainer runs the torch_col loop on a pool-backed
    Gpt2Step; an L1 adjust that names a smaller batch kills the micro-batch in flight (the control thread raises
    the executor's flag through srt_stub_set_abort_target), the step keeps an activation set for the new batch size
    and hands the other pages back, and training goes on with gradient accumulation so that every global batch still
    sees all of its samples."""
    from oracle import gpt2_oracle as GO
    from sirius_b200 import torch_col as tc
    from sirius_b200.gpt2_step import Gpt2Step
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    os.environ.update({"COLTRAIN_MODE": "colocate-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
                       "COLTRAIN_HAS_INFER_SERVER": "1", "COLTRAIN_USE_SHARED_TENSOR": "1", "COLTRAIN_KEEP_TARGET_SET": "1",
                       "SIRIUS_B200_COMM_NAME": f"srt_gpt_comm_{tag}", "SIRIUS_B200_DIST_NAME": f"srt_gpt_dist_{tag}"})
    cfg = dict(n_layer=2, n_head=4, d_model=128, vocab=30016, ctx=64)
    BS, SEQ, DS, EPOCHS = 4, 64, 32, 2
    model = GO.build_model(**cfg, seed=0)
    srv = tc.DebugServer(1, os.environ["SIRIUS_B200_COMM_NAME"])
    pool = PagePool(1.0, page_mb=2)
    tc.setup_colocate_training(0, 1, False, False)
    step = Gpt2Step(**cfg, max_batch=BS, seq=SEQ, pool=pool.handle)
    step.load_state_dict(GO.state_arrays(model))
    tc.set_train_step(step)
    tc.set_memory_pool(pool.handle)
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), EPOCHS, BS, stub_poll_ms=5)
    ds, mgr = tc.init_dynamic_batch(DS, tc.DatasetType.TEXT_GEN, tc.TextDatasetConfig(SEQ), BS, global_batch_size=BS,
                                    enable_grad_accumulate=True, checkpoint_micro_batch=True)
    tc.init_train_info(BS, BS, "gpt2")
    acc = tc.GradAccumulator(step)
    state = {"n": 0, "cid": None, "mapped_before": None, "sizes": [], "losses": []}

    def iter_train_fn(batch):
        state["n"] += 1
        n = len(batch)
        step.upload_tokens(batch["input_ids"])
        if state["n"] == 3 and state["cid"] is None:
            state["mapped_before"] = pool.stat("train_all")
            state["cid"] = srv.colocate_l1([2])            # the inference side needs memory: continue at batch 2
            _wait_cmd(ctrl, tc.CtrlEvent.kColocateAdjustL1)
        try:
            step.forward_backward(BS)
        except SrtError as e:
            if "aborted" in str(e):
                raise tc.ColocateAdjustL1Exception("killed in the executor")
            raise
        ctrl.check_kill("after backward")
        loss = step.loss()
        mgr.optimizer_step(batch, step, grad_accumulator=acc)
        state["sizes"].append(n)
        state["losses"].append(loss)
        return loss

    trainer = tc.Trainer(step, iter_train_fn)
    ctrl.train_start()
    for e in range(EPOCHS):
        trainer.train_one_epoch(e)
    ctrl.train_end()
    step.synchronize()
    stat = trainer.get_overall_stat()
    assert stat.killed_batch == 1
    assert [m.id for _, m in srv.events(tc.CtrlEvent.kColocateAdjustL1Done)] == [state["cid"]]
    released = ctrl.adjust_log[0][3]
    assert released > 0 and released % pool.stat("page_nbytes") == 0
    assert pool.stat("train_all") == state["mapped_before"] - released      # the pages stay with the pool
    # before the adjust full batches, afterwards micro-batches of at most 2 that add up to every global batch
    assert state["sizes"][:2] == [BS, BS] and max(state["sizes"][2:]) <= 2
    assert sum(state["sizes"]) == DS * EPOCHS                               # every sample of every epoch trained once
    assert [e.finished_sample for e in trainer.epoch_stats] == [DS] * EPOCHS
    assert all(np.isfinite(state["losses"])) and ops.tc_status() == 0
    step.close()
    tc.cleanup_colocate_training(False)
    tc.set_train_step(None)
    pool.close()
    srv.close()


def test_lm_colocation_experiment_runs_on_small_models():
    """The Qwen2 + DistilBERT colocation experiment (the reference's LLM colocation workload) on small models: requests on
    the gamma trace are served, cold ones trigger a handover that shrinks the training batch, every global batch is
    still trained in full, and training returns to the full batch after the idle give-back."""
    from sirius_b200.colocate_bench_lm import run
    out = run(duration_s=2.0, rate=100.0, cv=4.0, idle_ms=150.0, batch=4, seq=128, infer_seq=32,
              train_cfg=dict(n_layer=2, n_head=4, n_kv_head=2, hidden=128, intermediate=256, vocab=30016),
              infer_cfg=dict(n_layer=2, n_head=4, dim=128, hidden_dim=256, vocab=500, max_pos=64), pool_page_mb=2)
    assert out["requests"] > 20 and out["handovers"] >= 1 and out["final_loss_finite"]
    assert out["train_sequences"] > 0 and out["train_sequences"] % 4 == 0 or out["killed_micro_batches"] > 0
    assert min(out["micro_batch_sizes_seen"]) < 4 <= max(out["micro_batch_sizes_seen"])
    assert out["infer_p99_ms"] < 2000 and out["handover_gib_median"] > 0
    assert ops.tc_status() == 0


def test_gpt2_task_switch_releases_everything_and_resumes():
    """taskswitch-l1 on a pool-backed Gpt2Step: kInterruptTrain kills the micro-batch in flight, the trainer returns
    its whole activation set to the pool and the master replies kInterruptTrainDone; it stays off the GPU until
    kResumeTrain, then maps its pages again and trains every sample of every epoch."""
    import threading
    from oracle import gpt2_oracle as GO
    from sirius_b200 import torch_col as tc
    from sirius_b200.gpt2_step import Gpt2Step
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    os.environ.update({"COLTRAIN_MODE": "taskswitch-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
                       "COLTRAIN_HAS_INFER_SERVER": "1", "COLTRAIN_USE_SHARED_TENSOR": "1",
                       "SIRIUS_B200_COMM_NAME": f"srt_ts_comm_{tag}", "SIRIUS_B200_DIST_NAME": f"srt_ts_dist_{tag}"})
    cfg = dict(n_layer=2, n_head=4, d_model=128, vocab=30016, ctx=64)
    BS, SEQ, DS, EPOCHS = 4, 64, 32, 2
    model = GO.build_model(**cfg, seed=0)
    srv = tc.DebugServer(1, os.environ["SIRIUS_B200_COMM_NAME"])
    pool = PagePool(1.0, page_mb=2)
    tc.setup_colocate_training(0, 1, False, False)
    step = Gpt2Step(**cfg, max_batch=BS, seq=SEQ, pool=pool.handle)
    step.load_state_dict(GO.state_arrays(model))
    tc.set_train_step(step)
    tc.set_memory_pool(pool.handle)
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), EPOCHS, BS, stub_poll_ms=5)
    assert isinstance(ctrl, tc.SwitchCtrl)
    ds, mgr = tc.init_dynamic_batch(DS, tc.DatasetType.TEXT_GEN, tc.TextDatasetConfig(SEQ), BS, global_batch_size=BS,
                                    enable_grad_accumulate=True, checkpoint_micro_batch=True)
    tc.init_train_info(BS, BS, "gpt2")
    acc = tc.GradAccumulator(step)
    state = {"n": 0, "cid": None, "usage_interrupted": None, "sizes": [], "losses": [], "free_before": None}

    def server():                                              # answers the interrupt reply with a resume, later
        srv.wait_event(tc.CtrlEvent.kInterruptTrainDone, None, 1, 60)
        state["usage_interrupted"] = (pool.stat("train_usage"), pool.stat("free_pages"))
        time.sleep(0.2)
        srv.resume_train()

    th = threading.Thread(target=server, daemon=True)
    th.start()

    def iter_train_fn(batch):
        state["n"] += 1
        step.upload_tokens(batch["input_ids"])
        if state["n"] == 3 and state["cid"] is None:
            state["free_before"] = pool.stat("free_pages")
            state["cid"] = srv.interrupt_train()
            _wait_cmd(ctrl, tc.CtrlEvent.kInterruptTrain)
        try:
            step.forward_backward(BS)
        except SrtError as e:
            if "aborted" in str(e):
                raise tc.SwitchL1Exception("killed in the executor")
            raise
        ctrl.check_kill("after backward")
        loss = step.loss()
        mgr.optimizer_step(batch, step, grad_accumulator=acc)
        state["sizes"].append(len(batch))
        state["losses"].append(loss)
        return loss

    trainer = tc.Trainer(step, iter_train_fn)
    ctrl.train_start()
    for e in range(EPOCHS):
        trainer.train_one_epoch(e)
    ctrl.train_end()
    step.synchronize()
    th.join(30)
    assert trainer.get_overall_stat().killed_batch == 1
    assert [m.id for _, m in srv.events(tc.CtrlEvent.kInterruptTrainDone)] == [state["cid"]]
    assert len(srv.events(tc.CtrlEvent.kResumeTrainDone)) == 1
    usage, free_pages = state["usage_interrupted"]
    assert usage == 0 and free_pages > state["free_before"]    # the whole activation set went back to the pool
    assert len(ctrl.switch_log) == 1 and ctrl.switch_log[0][3] > 0
    assert sum(state["sizes"]) == DS * EPOCHS and set(state["sizes"]) == {BS}
    assert all(np.isfinite(state["losses"])) and ops.tc_status() == 0
    step.close()
    tc.cleanup_colocate_training(False)
    tc.set_train_step(None)
    pool.close()
    srv.close()
