"""Colocation experiment on one GPU with language models: Qwen2-0.5B-shaped training (torch_col Trainer,
colocate-l1, 4 x 2048 tokens per step) next to a stand-in inference worker that serves batch-1 DistilBERT-base
requests (128 tokens) arriving on a seeded bursty trace.

    python -m sirius_b200.colocate_bench_lm [--duration 10] [--rate 100] [--cv 4] [--idle-ms 500]

Same protocol as `colocate_bench` (the inference server's part of server/model_store/infer_model.cc:394-523,656-686
and server/control/controller.cc:268-386): a request that finds the inference allocator without memory asks the
TrainAdjuster for a plan, sends kColocateAdjustL1 to the trainer, waits for kColocateAdjustL1Done, maps the freed
pages and runs the forward pass; after `idle-ms` without requests the pages go back and kInferExit lets training
grow to its full batch again. The pool holds the training footprint plus one page less than inference needs, so
inference cannot run without a handover.

Arrivals: inter-arrival times drawn from a gamma distribution with the given mean rate and coefficient of
variation (shape 1/cv^2, scale cv^2/rate) from numpy's MT19937 seeded with 0, standing in for the reference
harness's trace generators (eval/runner/hyper_workload.py:350-373); no trace file is replayed. Weights are
seeded random values (normal, std 0.02; norm scales 1): there are no checkpoints on the box.
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


def _random_state(params, seed):
    rng = np.random.default_rng(seed)
    sd = {}
    for name, (_, shape) in params.items():
        if name.endswith("norm.weight") or "LayerNorm.weight" in name or "layer_norm.weight" in name:
            sd[name] = np.ones(shape, dtype=np.float32)
        elif name.endswith(".bias"):
            sd[name] = (rng.standard_normal(shape, dtype=np.float32) * 0.01).astype(np.float32)
        else:
            sd[name] = (rng.standard_normal(shape, dtype=np.float32) * 0.02).astype(np.float32)
    return sd


def run(duration_s=10.0, rate=100.0, cv=4.0, idle_ms=500.0, batch=4, seq=2048, infer_seq=128, seed=0, train_cfg=None,
        infer_cfg=None, pool_page_mb=32):
    from . import torch_col as tc
    from ._lib import SrtError, call
    from ._runtime import AdjusterConfig
    from .bert_infer import DISTILBERT_BASE, DistilBertInfer
    from .pool import PagePool
    from .qwen2_step import QWEN2_05B, Qwen2Step

    train_cfg = dict(train_cfg or QWEN2_05B)
    infer_cfg = dict(infer_cfg or DISTILBERT_BASE)
    tag = f"{os.getpid()}_{uuid.uuid4().hex[:6]}"
    os.environ.update({"COLTRAIN_MODE": "colocate-l1", "COLTRAIN_HOOK_MODE": "xsched-sync2", "COLTRAIN_USE_XSCHED": "1",
                       "COLTRAIN_HAS_INFER_SERVER": "1", "COLTRAIN_USE_SHARED_TENSOR": "1", "COLTRAIN_KEEP_TARGET_SET": "1",
                       "SIRIUS_B200_COMM_NAME": f"srt_lm_comm_{tag}", "SIRIUS_B200_DIST_NAME": f"srt_lm_dist_{tag}"})
    page = pool_page_mb << 20

    # size the pool from a probe on a roomy pool: the pages training maps at `batch`, plus one page less than
    # inference needs, so that a request always finds the inference allocator short of memory
    probe = Qwen2Step(**train_cfg, max_batch=batch, seq=seq)
    total_bytes = probe.memory_bytes()
    probe.close()
    probe_pool = PagePool((total_bytes + 64 * page) / 2 ** 30, page_mb=pool_page_mb)
    pages_used = lambda: probe_pool.stat("pool_nbytes") // page - probe_pool.stat("free_pages")
    probe_i = DistilBertInfer(**infer_cfg, max_batch=1, seq=infer_seq, pool=probe_pool.handle)
    infer_pages = pages_used()
    probe = Qwen2Step(**train_cfg, max_batch=batch, seq=seq, pool=probe_pool.handle)
    train_pages = pages_used() - infer_pages
    probe.close()
    probe_i.close()
    probe_pool.close()
    pool = PagePool((train_pages + infer_pages - 1) * page / 2 ** 30, page_mb=pool_page_mb)
    slope_mb = train_pages * page / batch / 2 ** 20

    srv = tc.DebugServer(1, os.environ["SIRIUS_B200_COMM_NAME"])
    tc.setup_colocate_training(0, 1, False, False)
    infer = DistilBertInfer(**infer_cfg, max_batch=1, seq=infer_seq, pool=pool.handle)
    infer.load_state_dict(_random_state(infer.params, seed + 1))
    infer_bytes = infer.memory_bytes()[1]
    infer.release_activations()
    step = Qwen2Step(**train_cfg, max_batch=batch, seq=seq, pool=pool.handle)
    step.load_state_dict(_random_state(step.params, seed))
    if pool.stat("free_pages") >= infer_pages:
        raise RuntimeError("pool sizing: inference fits beside training without a handover")
    # warm-up exchange: training shrinks by the plan's batch delta, inference maps the pages it gives up, then both
    # return to their starting state; from here on both sides find their slots still mapped to the pages they trade
    delta = max(1, -(-((infer_pages + 1) * page) // (train_pages * page // batch)))
    step.shrink_activations(max(batch - delta, 1))
    infer.reserve_activations()
    infer.release_activations()
    step.shrink_activations(batch)
    tc.set_train_step(step)
    tc.set_memory_pool(pool.handle)
    ctrl = tc.create_colocate_ctrl(tc.get_colocate_train_mode(), tc.get_colocate_ctrl_hook_mode(), 1, batch, stub_poll_ms=2)
    ds_size = batch * 4
    ds, mgr = tc.init_dynamic_batch(ds_size, tc.DatasetType.TEXT_GEN, tc.TextDatasetConfig(seq), batch,
                                    global_batch_size=batch, enable_grad_accumulate=True, checkpoint_micro_batch=True)
    tc.init_train_info(batch, batch, "qwen")
    acc = tc.GradAccumulator(step)
    adj_cfg = AdjusterConfig(0.0, slope_mb, 0, 0, 1500.0, 1, 1)
    adj = C.c_void_p()
    call("srt_adjuster_create", srv.comm._h, C.byref(adj_cfg), C.byref(adj))
    call("srt_adjuster_load_train_info", adj)

    stop = threading.Event()
    t_start = [None]
    lat_ms, handover, sent_at, kill_seen = [], [], [], []
    phase = {"reserve": [], "serve": [], "give_back": []}
    infer_tpc = 33 * 74 // 40   # the reference asks for 33 of a V100's 40 TPCs for distilbert_base

    def inference_worker():
        rng = np.random.RandomState(np.random.MT19937(np.random.SeedSequence(seed)))
        ids = rng.randint(0, infer_cfg["vocab"], size=(1, infer_seq)).astype(np.int32)
        while t_start[0] is None and not stop.is_set():
            time.sleep(0.001)
        t_next = t_start[0] + 1.0             # let the first training steps pass
        have_mem, last_done, target = False, 0.0, batch
        while not stop.is_set():
            now = time.perf_counter()
            if have_mem and now - last_done > idle_ms / 1e3 and t_next - now > 0:
                t1 = time.perf_counter()
                infer.release_activations()
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
            t_next += rng.gamma(1.0 / (cv * cv), cv * cv / rate)
            if not have_mem:
                plan, n = (C.c_int * 8)(), C.c_int()
                need_mb = (infer_pages + 1) * page / 2 ** 20
                call("srt_adjuster_infer_require_plan", adj, 0, need_mb, None, plan, C.byref(n))
                target = max(plan[0], 1) if n.value else batch
                t0 = time.perf_counter()
                sent_at.append(time.time())
                cid = srv.colocate_l1([target])
                srv.wait_adjust_done(cid, 60)
                handover.append((time.perf_counter() - t0) * 1e3)
                t1 = time.perf_counter()
                infer.reserve_activations()
                phase["reserve"].append((time.perf_counter() - t1) * 1e3)
                have_mem = True
            t2 = time.perf_counter()
            srv.comm.infer_tpc(0, 1, infer_tpc)            # AddInferRequiredTpcNum
            infer.upload_tokens(ids)
            infer.forward()
            infer.synchronize()
            srv.comm.infer_tpc(0, 2, infer_tpc)            # DecInferRequiredTpcNum
            last_done = time.perf_counter()
            phase["serve"].append((last_done - t2) * 1e3)
            lat_ms.append((last_done - t_arr) * 1e3)

    losses, finished, sizes = [], [0], []

    def iter_train_fn(b):
        step.upload_tokens(b["input_ids"])
        try:
            step.forward_backward(batch)
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
        sizes.append(len(b))
        return loss

    trainer = tc.Trainer(step, iter_train_fn)
    th = threading.Thread(target=inference_worker, daemon=True)
    th.start()
    ctrl.train_start()
    trainer.train_one_epoch(0)               # warm-up epoch without inference traffic
    finished[0] = 0
    del sizes[:]
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
    rel = [a[3] / 2 ** 30 for a in ctrl.adjust_log][:len(handover)]
    ho_gib = np.array(rel) if rel and len(rel) == len(handover) else np.full(len(ho_ms), float("nan"))
    pct = lambda v, q: round(float(np.sort(np.array(v))[min(len(v) - 1, int(len(v) * q))]), 3) if v else None
    out = {
        "train": "Qwen2-0.5B shape" if train_cfg == dict(QWEN2_05B) else "Qwen2 (custom shape)",
        "infer": "DistilBERT-base" if infer_cfg == dict(DISTILBERT_BASE) else "DistilBERT (custom shape)",
        "train_tokens_per_s": round(finished[0] * seq / window, 1), "train_sequences": finished[0], "window_s": round(window, 2),
        "micro_batch_sizes_seen": sorted(set(sizes)),
        "requests": len(lat_ms), "request_rate_per_s": rate, "arrival_cv": cv,
        "infer_p50_ms": round(float(lat[len(lat) // 2]), 3),
        "infer_p99_ms": round(float(lat[min(len(lat) - 1, len(lat) * 99 // 100)]), 3),
        "infer_max_ms": round(float(lat[-1]), 3),
        "handovers": len(handover), "killed_micro_batches": stat.killed_batch,
        "handover_ms_median": round(float(np.median(ho_ms)), 3), "handover_ms_max": round(float(np.max(ho_ms)), 3),
        "handover_gib_median": round(float(np.median(ho_gib)), 3),
        "handover_ms_per_gib": (round(float(np.median(ho_ms[ho_gib > 0] / ho_gib[ho_gib > 0])), 3)
                                if np.any(ho_gib > 0) else None),
        "worker_phase_ms": {k: {"p50": pct(v, 0.5), "p99": pct(v, 0.99), "max": pct(v, 1.0)} for k, v in phase.items()},
        # each kill is paired with the latest adjust sent before it (not every adjust kills a micro-batch)
        "kill_seen_after_ms": [round((k - max(s0 for s0 in sent_at if s0 <= k)) * 1e3, 2)
                               for k in kill_seen if any(s0 <= k for s0 in sent_at)][:8],
        "pool_gib": round(pool.stat("pool_nbytes") / 2 ** 30, 2), "train_pages": int(train_pages),
        "infer_activation_mib": round(infer_bytes / 2 ** 20, 1), "idle_ms": idle_ms,
        "arrivals": f"gamma inter-arrival times, mean rate {rate}/s, CV {cv}, MT19937 seed {seed}",
        "policy": "handover when a request finds no inference memory; pages return to training after idle_ms without requests",
        "final_loss_finite": bool(np.isfinite(losses[-1])) if losses else None,
    }
    call("srt_adjuster_destroy", adj)
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
    ap.add_argument("--rate", type=float, default=100.0)
    ap.add_argument("--cv", type=float, default=4.0)
    ap.add_argument("--idle-ms", type=float, default=500.0)
    ap.add_argument("--batch", type=int, default=4)
    ap.add_argument("--seq", type=int, default=2048)
    a = ap.parse_args()
    print(json.dumps(run(a.duration, a.rate, a.cv, a.idle_ms, a.batch, a.seq)), flush=True)


if __name__ == "__main__":
    main()
