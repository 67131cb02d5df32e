"""Colocation experiment with the two sides in two PROCESSES, as the reference deploys them: an inference server
process that owns the page pool, the control channel and the Controller, and a training process it launches
with the TrainLauncher's environment, which attaches to the same physical pages.

    python -m sirius_b200.colocate_proc [--duration 30] [--rate 50] [--policy per-request|cold-request]

Server (this process): creates the shared pool (srt_pool_init: pages exported as file descriptors), the
inf_tra_comm channel, TrainAdjuster, Controller and ResourceManager; loads a batch-1 ResNet-152 on the pool's
inference allocator; launches the trainer; then serves requests arriving as a seeded Poisson process. For a
request that finds no inference memory it asks the TrainAdjuster for a require plan, sends it through the
Controller (kColocateAdjustL1), waits for the trainer's Done, maps the pages the trainer gave up, raises the
required-TPC counter (the trainer's SM partition shrinks), runs the forward pass, lowers the counter. Policy
"per-request" gives the pages back right after every request (release plan -> kInferExit), so every request
triggers a handover and an SM-mask shrink; "cold-request" keeps them until the server has been idle for
--idle-ms (the reference server's infer_model_max_idle_ms behaviour).

Trainer (child, --role trainer): torch_col's Trainer in colocate-l1 mode on a ResNet-152 step whose activations
come from the attached pool; follows the SM partition; stops when the server announces the end of the inference
workload, and leaves its counters in a JSON file.

Handover is measured at the protocol level, across the process boundary: from the Controller call that sends
the adjust to the return of the wait for Done, per GiB of pages that became free in between.
"""
from __future__ import annotations

import argparse
import ctypes as C
import json
import os
import sys
import tempfile
import time
import uuid

import numpy as np

if __name__ == "__main__" and __package__ in (None, ""):
    # started by path, as the TrainLauncher starts a training script (python <script> --name value ...)
    sys.path.insert(0, os.path.dirname(os.path.dirname(os.path.abspath(__file__))))
    __package__ = "sirius_b200"

ARCH, IMAGE = "resnet152", 224
_CHILDREN = []   # launchers of training processes this module has started and not yet seen exit


def kill_children():
    """Ends training processes still running (for a caller that has to leave early)."""
    for launcher in list(_CHILDREN):
        try:
            if launcher.wait(0) is None:
                launcher.kill()
        except Exception:  # noqa: BLE001
            pass
        _CHILDREN.remove(launcher)


def _seeded_state(arch):
    import torch
    from torchvision.models.resnet import Bottleneck, ResNet
    from .step import RESNET_LAYERS
    torch.manual_seed(0)
    return {k: v for k, v in ResNet(Bottleneck, list(RESNET_LAYERS[arch]), num_classes=1000).state_dict().items()
            if not k.endswith("num_batches_tracked")}


# ----------------------------------------------------------------------------------------------------- trainer
def trainer_main(a):
    import torch
    from . import torch_col as tc
    from ._lib import SrtError, call
    from .step import ResNetStep
    torch.cuda.set_device(0)
    call("srt_pool_init", 0, 0, 0)                      # COLTRAIN_HAS_SHARED_TENSOR_SERVER=1: attach to the server's pool
    pool = C.c_void_p()
    call("srt_pool_default", 0, C.byref(pool))
    tc.setup_colocate_training(0, 1, False, False)
    step = ResNetStep(arch=ARCH, max_batch=a.batch, image=IMAGE, dtype="bf16", pool=pool)
    step.load_state_dict(_seeded_state(ARCH))
    tc.set_train_step(step)
    tc.set_memory_pool(pool)
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), 1, a.batch, stub_poll_ms=2)
    ds, mgr = tc.init_dynamic_batch(a.batch * 8, tc.DatasetType.VISION, tc.VisionDatasetConfig((3, IMAGE, IMAGE), 1000), a.batch,
                                    global_batch_size=a.batch, enable_grad_accumulate=True, checkpoint_micro_batch=True)
    tc.init_train_info(a.batch, a.batch, "resnet152")
    acc = tc.GradAccumulator(step)
    gpu_tpc = torch.cuda.get_device_properties(0).multi_processor_count // 2
    if not a.no_sm_partition:
        step.follow_infer_tpc(tc._C.comm_handle(), 0, 5, gpu_tpc)
    sms_seen, losses, finished, kills = set(), [], [0], []

    def iter_train_fn(b):
        sms_seen.add(step.current_sms())
        step.upload_batch(b["images"], b["labels"])
        try:
            step.forward_backward(len(b), a.batch)
        except SrtError as e:
            if "aborted" in str(e):
                kills.append(time.time())
                raise tc.ColocateAdjustL1Exception("killed in the executor")
            raise
        ctrl.check_kill("after backward")
        loss = step.loss()
        losses.append(loss)
        mgr.optimizer_step(b, step, grad_accumulator=acc)
        finished[0] += len(b)
        return loss

    trainer = tc.Trainer(step, iter_train_fn)
    ctrl.train_start()
    trainer.train_one_epoch(0)                           # warm-up epoch
    finished[0] = 0
    with open(a.result + ".ready", "w") as f:            # tells the server that the measured window may begin
        f.write("ready")
    t0 = time.time()
    epoch = 1
    marks = []                                           # (time, samples finished): the server cuts its window out of these
    # The reference's trainer keeps going for 30 s after kInferenceWorkloadDone (can_exit_after_infer_worklaod_done);
    # the experiment has nothing left to measure then, so the server also drops a stop file.
    while (not os.path.exists(a.result + ".stop") and not ctrl._stub.can_exit_after_infer_worklaod_done()
           and time.time() - t0 < a.max_seconds):
        trainer.train_one_epoch(epoch)
        epoch += 1
        marks.append((time.time(), finished[0]))
    step.synchronize()
    ctrl.train_end()
    out = {"t_ready": t0, "marks": marks, "killed_micro_batches": trainer.get_overall_stat().killed_batch,
           "adjust_log": [list(x) for x in ctrl.adjust_log], "kill_times": kills, "train_sms_seen": sorted(sms_seen),
           "final_loss_finite": bool(np.isfinite(losses[-1])) if losses else None}
    with open(a.result, "w") as f:
        json.dump(out, f)
    if not a.no_sm_partition:
        step.follow_infer_tpc(None)
    step.close()
    tc.cleanup_colocate_training(False)
    tc.set_train_step(None)
    call("srt_pool_shutdown", 0)


# ------------------------------------------------------------------------------------------------------ server
def run(duration_s=30.0, rate=50.0, policy="per-request", idle_ms=500.0, batch=64, seed=0, sm_partition=True,
        multi_gib=False):
    import torch
    from . import _lib
    from ._lib import call
    from ._runtime import AdjusterConfig
    from .pool import INFER, PagePool
    from .server import Controller, ResourceManager, ServeMode, TrainLauncher
    from .step import ResNetStep
    from .torch_col._C import PyInfTraCommunicator

    torch.cuda.set_device(0)
    port = f"{20000 + os.getpid() % 20000}{uuid.uuid4().hex[:3]}"
    os.environ["SIRIUS_PORT"] = port                    # names the pool, the channel and the trainer's segments
    os.environ.pop("COLTRAIN_HAS_SHARED_TENSOR_SERVER", None)
    page = 32 << 20
    # pool size: the pages the training step maps at `batch`, plus one (probe on a private pool)
    probe = ResNetStep(arch=ARCH, max_batch=batch, image=IMAGE, dtype="bf16")
    train_bytes = probe.memory_bytes()[1]
    probe.close()
    probe_pool = PagePool((train_bytes * 3 // 2 + 16 * page) / 2 ** 30)
    probe = ResNetStep(arch=ARCH, max_batch=batch, image=IMAGE, dtype="bf16", pool=probe_pool.handle)
    train_pages = probe_pool.stat("pool_nbytes") // page - probe_pool.stat("free_pages")
    probe.close()
    probe_pool.close()
    pool_bytes = (train_pages + 1) * page
    call("srt_pool_init", 0, pool_bytes, 1)             # the shared pool; the trainer attaches to it
    pool = C.c_void_p()
    call("srt_pool_default", 0, C.byref(pool))
    stat = lambda w: _lib.lib().srt_pool_stat(pool, w)
    FREE_PAGES = 4

    comm = PyInfTraCommunicator(True, True, 1)          # default name: from SIRIUS_PORT
    slope_mb = train_pages * page / batch / 2 ** 20
    adj_cfg = AdjusterConfig(0.0, slope_mb, 0, 0, 1500.0, 1, 1)
    adj = C.c_void_p()
    call("srt_adjuster_create", comm._h, C.byref(adj_cfg), C.byref(adj))
    ctl = Controller(comm, adj, ServeMode.COLOCATE_L1)
    resmgr = ResourceManager(pool, adj)

    sd = _seeded_state(ARCH)
    infer = ResNetStep(arch=ARCH, max_batch=1, image=IMAGE, dtype="bf16", pool=pool, pool_kind=INFER)
    infer.load_state_dict(sd)
    infer_bytes = infer.memory_bytes()[1]
    infer_pages = stat(5) // page - stat(FREE_PAGES)
    infer.release_activations()

    result = os.path.join(tempfile.gettempdir(), f"srt_colocate_{port}.json")
    launcher = TrainLauncher(ServeMode.COLOCATE_L1, use_xsched=True, use_shared_tensor_train=True,
                             cuda_memory_pool_gb=pool_bytes / 2 ** 30, dynamic_sm_partition=sm_partition)
    args = f"role=trainer batch={batch} result={result} max-seconds={duration_s + 120}" + ("" if sm_partition else " no-sm-partition")
    launcher.launch(os.path.abspath(__file__), args, interpreter=sys.executable,
                    log_path=os.path.join(tempfile.gettempdir(), f"srt_colocate_{port}.log"))
    _CHILDREN.append(launcher)
    ctl.set_train_pid(launcher.pid)
    t0 = time.time()
    while not os.path.exists(result + ".ready"):
        if launcher.wait(0) is not None or time.time() - t0 > 300:
            raise RuntimeError("the training process did not come up: " + open(
                os.path.join(tempfile.gettempdir(), f"srt_colocate_{port}.log")).read()[-2000:])
        time.sleep(0.01)
    if stat(FREE_PAGES) >= infer_pages:
        raise RuntimeError("pool sizing: inference fits beside training without a handover")

    gpu_tpc = torch.cuda.get_device_properties(0).multi_processor_count // 2
    infer_tpc = max(1, gpu_tpc * 27 // 40)              # the reference asks for 27 of a V100's 40 TPCs for resnet152
    rng = np.random.RandomState(np.random.MT19937(np.random.SeedSequence(seed)))
    img = torch.randn(1, 3, IMAGE, IMAGE).pin_memory()
    lab = torch.zeros(1, dtype=torch.int64).pin_memory()
    need_mb = (infer_pages + 1) * page / 2 ** 20
    lat_ms, handover, phase = [], [], {"adjust": [], "reserve": [], "serve": [], "give_back": []}

    def give_back():
        t1 = time.perf_counter()
        infer.release_activations()                      # pages back to FREE (their mappings stay)
        plan, n = (C.c_int * 8)(), C.c_int()
        avail = (C.c_double * 1)(resmgr.train_avail_memory_mb())
        free = (C.c_double * 1)(stat(FREE_PAGES) * page / 2 ** 20)
        zero = (C.c_double * 1)(0.0)
        call("srt_adjuster_infer_release_plan", adj, avail, free, zero, plan, C.byref(n))
        if n.value:
            ctl.colocate_infer_release_adjust([min(plan[0], batch)])
        phase["give_back"].append((time.perf_counter() - t1) * 1e3)

    t_begin = time.time()
    t_next = time.perf_counter() + 0.5
    t_end = t_next + duration_s
    have_mem, last_done = False, 0.0
    while True:
        now = time.perf_counter()
        if policy == "cold-request" and have_mem and now - last_done > idle_ms / 1e3 and t_next > now:
            give_back()
            have_mem = False
        if now >= t_end:
            break
        if t_next > now:
            time.sleep(min(t_next - now, 0.001))
            continue
        t_arr = t_next
        t_next += rng.exponential(1.0 / rate)
        if not have_mem:
            plan, n = (C.c_int * 8)(), C.c_int()
            call("srt_adjuster_infer_require_plan", adj, 0, need_mb, None, plan, C.byref(n))
            free_before = stat(FREE_PAGES)
            t1 = time.perf_counter()
            if n.value:
                cid = ctl.colocate_infer_require_adjust(0, [max(plan[0], 1)])
                ctl.wait_colocate_adjust_done(0, cid, 30000)
            dt = (time.perf_counter() - t1) * 1e3
            freed = (stat(FREE_PAGES) - free_before) * page
            handover.append((dt, freed))
            phase["adjust"].append(dt)
            t1 = time.perf_counter()
            infer.reserve_activations(1)
            phase["reserve"].append((time.perf_counter() - t1) * 1e3)
            have_mem = True
        t2 = time.perf_counter()
        comm.infer_tpc(0, 1, infer_tpc)                  # AddInferRequiredTpcNum: the trainer's partition shrinks
        infer.upload_batch(img, lab)
        infer.forward_infer(1)
        infer.synchronize()
        comm.infer_tpc(0, 2, infer_tpc)
        last_done = time.perf_counter()
        phase["serve"].append((last_done - t2) * 1e3)
        lat_ms.append((last_done - t_arr) * 1e3)
        if policy == "per-request":
            give_back()
            have_mem = False
    t_stop = time.time()
    if have_mem:
        give_back()
    # One multi-GiB handover across the process boundary: ask training to continue at an eighth of its batch (the
    # adjust names the batch size, as every kColocateAdjustL1 does), from the Controller call to the Done reply,
    # per GiB of pages that became free in between; then let it grow back.
    big = None
    try:
        if not multi_gib:
            raise StopIteration
        small = max(1, batch // 8)
        free_before = stat(FREE_PAGES)
        t1 = time.perf_counter()
        cid = ctl.colocate_infer_require_adjust(0, [small])
        ctl.wait_colocate_adjust_done(0, cid, 30000)
        dt = (time.perf_counter() - t1) * 1e3
        freed = (stat(FREE_PAGES) - free_before) * page
        if freed > 0:
            big = {"target_batch": small, "freed_gib": round(freed / 2 ** 30, 3), "ms": round(dt, 3),
                   "ms_per_gib": round(dt / (freed / 2 ** 30), 3)}
        ctl.colocate_infer_release_adjust([batch])
        time.sleep(0.2)                                  # a few training steps at the full batch again
    except StopIteration:
        pass
    except Exception as e:  # noqa: BLE001  (the per-request figures stand without it)
        big = {"error": f"{type(e).__name__}: {e}"[:200]}
    ctl.inference_workload_done()
    with open(result + ".stop", "w") as f:
        f.write("stop")
    status = launcher.wait(120000)
    if status is None:
        launcher.kill()
    if launcher in _CHILDREN:
        _CHILDREN.remove(launcher)
    tr = json.load(open(result)) if os.path.exists(result) else {}
    for f in (result, result + ".ready", result + ".stop"):
        if os.path.exists(f):
            os.unlink(f)
    # training throughput inside the server's window, from the trainer's per-epoch marks
    inside = [(t, s) for t, s in tr.get("marks", []) if t_begin <= t <= t_stop]
    if len(inside) >= 2:
        samples = inside[-1][1] - inside[0][1]
        span = inside[-1][0] - inside[0][0]
    else:
        samples, span = 0, float("nan")
    lat = np.sort(np.array(lat_ms)) if lat_ms else np.array([float("nan")])
    ho = np.array([h for h in handover if h[1] > 0], dtype=np.float64).reshape(-1, 2)
    pct = lambda v, q: round(float(np.sort(np.array(v))[min(len(v) - 1, int(len(v) * q))]), 3) if v else None
    out = {
        "processes": 2, "policy": policy,
        "train_samples_per_s": round(samples / span, 1) if span == span and span > 0 else None,
        "window_s": round(t_stop - t_begin, 2), "requests": len(lat_ms), "request_rate_per_s": rate,
        "infer_p50_ms": round(float(lat[len(lat) // 2]), 3),
        "infer_p99_ms": round(float(lat[min(len(lat) - 1, len(lat) * 99 // 100)]), 3),
        "infer_max_ms": round(float(lat[-1]), 3),
        "handovers": len(handover), "killed_micro_batches": tr.get("killed_micro_batches"),
        "handover_ms_median": round(float(np.median(ho[:, 0])), 3) if len(ho) else None,
        "handover_ms_p99": pct(list(ho[:, 0]), 0.99) if len(ho) else None,
        "handover_gib_median": round(float(np.median(ho[:, 1])) / 2 ** 30, 3) if len(ho) else None,
        "handover_ms_per_gib": round(float(np.median(ho[:, 0] / (ho[:, 1] / 2 ** 30))), 3) if len(ho) else None,
        "handover_multi_gib": big,
        "server_phase_ms": {k: {"p50": pct(v, 0.5), "p99": pct(v, 0.99), "max": pct(v, 1.0)} for k, v in phase.items()},
        "trainer_adjust_ms_first": [[round(x, 2) for x in a[:3]] for a in tr.get("adjust_log", [])][:4],
        "pool_gib": round(pool_bytes / 2 ** 30, 2), "train_activation_gib": round(train_bytes / 2 ** 30, 2),
        "infer_activation_mib": round(infer_bytes / 2 ** 20, 1),
        "arrivals": f"Poisson {rate}/s, continuous, numpy MT19937 seed {seed}",
        "sm_partition": ({"infer_required_tpc": infer_tpc, "of_tpc": gpu_tpc, "train_sms_seen": tr.get("train_sms_seen")}
                         if sm_partition else "off"),
        "trainer_exit_status": status, "final_loss_finite": tr.get("final_loss_finite"),
    }
    if policy == "cold-request":
        out["idle_ms"] = idle_ms
    infer.close()
    ctl.close()
    call("srt_adjuster_destroy", adj)
    comm.close()
    call("srt_pool_shutdown", 0)
    return out


def make_parser():
    ap = argparse.ArgumentParser()
    ap.add_argument("--role", default="server", choices=["server", "trainer"])
    ap.add_argument("--duration", type=float, default=30.0)
    ap.add_argument("--rate", type=float, default=50.0)
    ap.add_argument("--policy", default="per-request", choices=["per-request", "cold-request"])
    ap.add_argument("--idle-ms", type=float, default=500.0)
    ap.add_argument("--batch", type=int, default=64)
    ap.add_argument("--no-sm-partition", action="store_true")
    ap.add_argument("--multi-gib", action="store_true",
                    help="after the window, one adjust to an eighth of the batch: handover of several GiB across the processes")
    ap.add_argument("--result", default="")
    ap.add_argument("--max-seconds", type=float, default=300.0)
    return ap


def main():
    a = make_parser().parse_args()
    if a.role == "trainer":
        trainer_main(a)
    else:
        print(json.dumps(run(a.duration, a.rate, a.policy, a.idle_ms, a.batch, sm_partition=not a.no_sm_partition,
                             multi_gib=a.multi_gib)), flush=True)


if __name__ == "__main__":
    main()
