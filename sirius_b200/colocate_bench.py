"""Colocation experiment on one GPU: ResNet-152 training (torch_col Trainer, colocate-l1) next to a
stand-in inference worker that serves batch-1 ResNet-152 requests arriving as a seeded Poisson process.

    python -m sirius_b200.colocate_bench [--duration 10] [--rate 50] [--idle-ms 500] [--burst-s 1] [--gap-s 1]

The worker plays the inference server's part of the reference's protocol (server/model_store/
infer_model.cc:394-523,656-686 and server/control/controller.cc:268-386): when a request finds the
inference allocator without memory it asks the TrainAdjuster for a plan, sends kColocateAdjustL1 to the
trainer, waits for kColocateAdjustL1Done, maps the freed pages and runs the forward pass; it raises the
required-TPC counter while a request runs; after `idle-ms` without requests it frees its pages and sends
kInferExit so training grows back. The page pool is sized to the training footprint plus a small slack,
so inference cannot run without a handover. Reports training samples/s over the window, request latency
percentiles, and the handover latency (adjust sent -> done received) per GiB released.

Arrivals stand in for the reference harness's trace generators (eval/runner/hyper_workload.py:350-373):
exponential inter-arrival times from numpy's MT19937 seeded with 0, switched on and off in bursts so that
the idle give-back and the next cold request both occur; no trace file is replayed.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import threading
import time
import uuid

import numpy as np


def run(duration_s=10.0, rate=50.0, idle_ms=500.0, burst_s=1.0, gap_s=1.0, batch=64, image=224, arch="resnet152", seed=0, per_arrival=False, sm_partition=True):
    import torch
    from . import torch_col as tc
    from ._lib import SrtError, call
    from ._runtime import AdjusterConfig
    from .pool import INFER, PagePool
    from .step import RESNET_LAYERS, ResNetStep
    from torchvision.models.resnet import Bottleneck, ResNet

    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    os.environ.update({"COLTRAIN_MODE": "colocate-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
                       "COLTRAIN_HAS_INFER_SERVER": "1", "COLTRAIN_USE_SHARED_TENSOR": "1",
                       "SIRIUS_B200_COMM_NAME": f"srt_col_comm_{tag}", "SIRIUS_B200_DIST_NAME": f"srt_col_dist_{tag}"})
    torch.manual_seed(0)
    sd = {k: v for k, v in ResNet(Bottleneck, list(RESNET_LAYERS[arch]), num_classes=1000).state_dict().items()
          if not k.endswith("num_batches_tracked")}

    # size the pool from a probe run on a roomy pool: the pages the training step maps at `batch`, plus one.
    # The allocator is deterministic, so the same sequence of requests maps the same pages again.
    page = 32 << 20
    probe = ResNetStep(arch=arch, max_batch=batch, image=image, dtype="bf16")
    train_bytes = probe.memory_bytes()[1]
    probe.close()
    probe_pool = PagePool((train_bytes * 3 // 2 + (16 * page)) / 2 ** 30)
    probe = ResNetStep(arch=arch, max_batch=batch, image=image, dtype="bf16", pool=probe_pool.handle)
    total_pages = probe_pool.stat("pool_nbytes") // page
    train_pages = total_pages - probe_pool.stat("free_pages")
    probe.close()
    probe_pool.close()
    pool = PagePool((train_pages + 1) * page / 2 ** 30)
    slope_mb = train_pages * page / batch / 2 ** 20

    srv = tc.DebugServer(1, os.environ["SIRIUS_B200_COMM_NAME"])
    tc.setup_colocate_training(0, 1, False, False)
    # the inference stand-in maps its pages first, measures its need and gives them back
    infer = ResNetStep(arch=arch, max_batch=1, image=image, dtype="bf16", pool=pool.handle, pool_kind=INFER)
    infer.load_state_dict(sd)
    infer_bytes = infer.memory_bytes()[1]
    infer_pages = pool.stat("pool_nbytes") // page - pool.stat("free_pages")
    infer.release_activations()
    step = ResNetStep(arch=arch, max_batch=batch, image=image, dtype="bf16", pool=pool.handle)
    step.load_state_dict(sd)
    if pool.stat("free_pages") >= infer_pages:
        raise RuntimeError("pool sizing: inference fits beside training without a handover")
    # warm-up exchange, as a deployment would do before taking traffic: training shrinks by the plan's
    # batch delta, inference maps the pages it gives up, then both return to their starting state. From
    # here on both sides find their slots still mapped to the pages they trade (no driver call).
    delta = -(-((infer_pages + 1) * page) // (train_pages * page // batch))
    step.shrink_activations(max(batch - delta, 1))
    infer.reserve_activations(1)
    infer.release_activations()
    step.reserve_activations(batch)
    tc.set_train_step(step)
    tc.set_memory_pool(pool.handle)
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), 1, batch, stub_poll_ms=2)
    ds_size = batch * 8
    ds, mgr = tc.init_dynamic_batch(ds_size, tc.DatasetType.VISION, tc.VisionDatasetConfig((3, image, image), 1000), batch,
                                    global_batch_size=batch, enable_grad_accumulate=True, checkpoint_micro_batch=True)
    tc.init_train_info(batch, batch, "resnet152")
    acc = tc.GradAccumulator(step)

    adj_cfg = AdjusterConfig(0.0, slope_mb, 0, 0, 1500.0, 1, 1)
    adj = C.c_void_p()
    call("srt_adjuster_create", srv.comm._h, C.byref(adj_cfg), C.byref(adj))
    call("srt_adjuster_load_train_info", adj)

    stop = threading.Event()
    t_start = [None]
    lat_ms, handover, sent_at, kill_seen = [], [], [], []
    phase = {"reserve": [], "serve": [], "give_back": []}
    gpu_tpc = torch.cuda.get_device_properties(0).multi_processor_count // 2
    infer_tpc = max(1, gpu_tpc * 27 // 40)   # the reference asks for 27 of a V100's 40 TPCs for resnet152

    def inference_worker():
        rng = np.random.RandomState(np.random.MT19937(np.random.SeedSequence(seed)))
        img = torch.randn(1, 3, image, image).pin_memory()
        lab = torch.zeros(1, dtype=torch.int64).pin_memory()
        while t_start[0] is None and not stop.is_set():
            time.sleep(0.001)
        t_next = t_start[0] + 1.0             # let the first training steps pass
        have_mem, last_done, target = False, 0.0, batch
        while not stop.is_set():
            now = time.perf_counter()
            if have_mem and now - last_done > idle_ms / 1e3 and t_next - now > 0:
                t1 = time.perf_counter()
                infer.release_activations()   # frees the blocks and unmaps the inference pages
                phase["give_back"].append((time.perf_counter() - t1) * 1e3)
                plan, n = (C.c_int * 8)(), C.c_int()
                avail = (C.c_double * 1)(pool.stat("pool_nbytes") / 2 ** 20)
                free = (C.c_double * 1)(pool.stat("free_pages") * page / 2 ** 20)
                zero = (C.c_double * 1)(0.0)
                call("srt_adjuster_infer_release_plan", adj, avail, free, zero, plan, C.byref(n))
                srv.infer_exit([min(plan[0], batch)])
                have_mem = False
            if t_next > now:
                time.sleep(min(t_next - now, 0.002))
                continue
            t_arr = t_next
            t_next += rng.exponential(1.0 / rate)
            if burst_s > 0 and (t_next - t_start[0] - 1.0) % (burst_s + gap_s) > burst_s:   # off period: next burst
                t_next = t_start[0] + 1.0 + ((t_next - t_start[0] - 1.0) // (burst_s + gap_s) + 1) * (burst_s + gap_s)
            if not have_mem or per_arrival:
                if not have_mem:
                    plan, n = (C.c_int * 8)(), C.c_int()
                    need_mb = (infer_pages + 1) * page / 2 ** 20
                    call("srt_adjuster_infer_require_plan", adj, 0, need_mb, None, plan, C.byref(n))
                    target = max(plan[0], 1) if n.value else batch
                t0 = time.perf_counter()
                sent_at.append(time.time())
                cid = srv.colocate_l1([target])       # warm request in per-arrival mode: same target again
                srv.wait_adjust_done(cid, 30)
                dt = time.perf_counter() - t0
                handover.append(dt * 1e3)
                if not have_mem:
                    t1 = time.perf_counter()
                    infer.reserve_activations(1)
                    phase["reserve"].append((time.perf_counter() - t1) * 1e3)
                    have_mem = True
            t2 = time.perf_counter()
            srv.comm.infer_tpc(0, 1, infer_tpc)            # AddInferRequiredTpcNum
            infer.upload_batch(img, lab)
            infer.forward_infer(1)
            infer.synchronize()
            srv.comm.infer_tpc(0, 2, infer_tpc)            # DecInferRequiredTpcNum
            last_done = time.perf_counter()
            phase["serve"].append((last_done - t2) * 1e3)
            lat_ms.append((last_done - t_arr) * 1e3)

    losses, finished = [], [0]

    # SM partition: between units the training step reads the inference side's required-TPC counter and
    # moves to the green-context partition that leaves those TPCs alone (the reference's pre-launch hook)
    if sm_partition:
        step.follow_infer_tpc(srv.comm._h, 0, 5, gpu_tpc)
    sms_seen = set()

    def iter_train_fn(b):
        sms_seen.add(step.current_sms())
        step.upload_batch(b["images"], b["labels"])
        try:
            step.forward_backward(len(b), batch)
        except SrtError as e:
            if "aborted" in str(e):
                kill_seen.append(time.time())
                raise tc.ColocateAdjustL1Exception("killed in the executor")
            raise
        ctrl.check_kill("after backward")
        loss = step.loss()
        losses.append(loss)
        mgr.optimizer_step(b, step, grad_accumulator=acc)
        finished[0] += len(b)
        return loss

    trainer = tc.Trainer(step, iter_train_fn)
    th = threading.Thread(target=inference_worker, daemon=True)
    th.start()
    ctrl.train_start()
    trainer.train_one_epoch(0)               # warm-up epoch without inference traffic
    finished[0] = 0
    t_start[0] = time.perf_counter()
    epoch = 1
    while time.perf_counter() - t_start[0] < duration_s + 1.0:
        trainer.train_one_epoch(epoch)
        epoch += 1
    step.synchronize()
    window = time.perf_counter() - t_start[0]
    stop.set()
    th.join(10)
    ctrl.train_end()
    stat = trainer.get_overall_stat()
    lat = np.sort(np.array(lat_ms)) if lat_ms else np.array([float("nan")])
    ho_ms = np.array(handover) if handover else np.array([float("nan")])
    # bytes the trainer handed back at each adjust (its own count of unmapped pages)
    rel = [a[3] / 2 ** 30 for a in ctrl.adjust_log][:len(handover)]
    ho_gib = np.array(rel) if rel and len(rel) == len(handover) else np.full(len(ho_ms), float("nan"))
    pct = lambda v, q: round(float(np.sort(np.array(v))[min(len(v) - 1, int(len(v) * q))]), 3) if v else None
    out = {
        "train_samples_per_s": round(finished[0] / window, 1), "window_s": round(window, 2),
        "requests": len(lat_ms), "request_rate_per_s": rate,
        "infer_p50_ms": round(float(lat[len(lat) // 2]), 3),
        "infer_p99_ms": round(float(lat[min(len(lat) - 1, len(lat) * 99 // 100)]), 3),   # client/src/workload/workload.cc.in:871-885
        "infer_max_ms": round(float(lat[-1]), 3),
        "handovers": len(handover), "killed_micro_batches": stat.killed_batch,
        "handover_ms_median": round(float(np.median(ho_ms)), 3), "handover_ms_max": round(float(np.max(ho_ms)), 3),
        "handover_gib_median": round(float(np.median(ho_gib)), 3),
        "handover_ms_per_gib": (round(float(np.median(ho_ms[ho_gib > 0] / ho_gib[ho_gib > 0])), 3)
                                if np.any(ho_gib > 0) else None),
        "worker_phase_ms": {k: {"p50": pct(v, 0.5), "p99": pct(v, 0.99), "max": pct(v, 1.0)} for k, v in phase.items()},
        "trainer_adjust_ms": [[round(x, 2) for x in a[:3]] for a in ctrl.adjust_log][:8],
        # each kill is paired with the latest adjust sent before it (not every adjust kills a micro-batch)
        "kill_seen_after_ms": [round((k - max(s0 for s0 in sent_at if s0 <= k)) * 1e3, 2)
                               for k in kill_seen if any(s0 <= k for s0 in sent_at)][:8],
        "adjust_start_after_ms": [round((a[4] - s0) * 1e3, 2) for a, s0 in zip(ctrl.adjust_log, sent_at)][:8],
        "pool_gib": round(pool.stat("pool_nbytes") / 2 ** 30, 2), "train_activation_gib": round(train_bytes / 2 ** 30, 2),
        "infer_activation_mib": round(infer_bytes / 2 ** 20, 1), "idle_ms": idle_ms,
        "arrivals": f"Poisson {rate}/s in bursts of {burst_s} s separated by {gap_s} s of silence, MT19937 seed {seed}",
        "adjust": "one L1 adjust per arrival" if per_arrival else "one L1 adjust per cold request",
        "policy": "handover when a request finds no inference memory; pages return to training after idle_ms "
                  "without requests (server/config.cc:75 defaults to 3000 ms, eval/ablation.py:162 uses 500)",
        "sm_partition": ({"infer_required_tpc": infer_tpc, "of_tpc": gpu_tpc, "train_sms_seen": sorted(sms_seen),
                          "how": "green-context partition streams, switched between conv+BN units"}
                         if sm_partition else "off"),
        "final_loss_finite": bool(np.isfinite(losses[-1])) if losses else None,
    }
    call("srt_adjuster_destroy", adj)
    if sm_partition:
        step.follow_infer_tpc(None)
    step.close()
    infer.close()
    tc.cleanup_colocate_training(False)
    tc.set_train_step(None)
    pool.close()
    srv.close()
    return out


def main():
    ap = argparse.ArgumentParser()
    ap.add_argument("--duration", type=float, default=10.0)
    ap.add_argument("--rate", type=float, default=50.0)
    ap.add_argument("--idle-ms", type=float, default=500.0)
    ap.add_argument("--burst-s", type=float, default=1.0)
    ap.add_argument("--gap-s", type=float, default=1.0)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--no-sm-partition", action="store_true")
    ap.add_argument("--per-arrival", action="store_true", help="send an L1 adjust for every request, not only cold ones")
    a = ap.parse_args()
    print(json.dumps(run(a.duration, a.rate, a.idle_ms, a.burst_s, a.gap_s, a.batch, per_arrival=a.per_arrival, sm_partition=not a.no_sm_partition)), flush=True)


if __name__ == "__main__":
    main()
